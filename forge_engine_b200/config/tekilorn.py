"""The Tekilorn configuration: a decoder whose layers are listed one by one, a stretch of
which may run several times in a row.

``config.json`` names the architecture in ``architecture`` and gives ``vocab``, ``width``,
``norm.eps``, ``layers`` and optionally ``loop``.  Per layer: ``type`` (which mixer), the
mixer's sizes and constants (``mixer``) and its feed-forward (``mlp``, or null for none).

Mixers:

* ``attention`` - differential grouped-query attention without rotation: two score maps per
  head (q and k carry two vectors of ``dim`` per head, [map 1, map 2]) over shared values,
  o = a1 - lambda a2 normalised over the head; scores of a query at position p are multiplied
  by 1 + q_temp.coef ln(floor((p + 1) / q_temp.every) + 1) and capped by
  softcap tanh(score / softcap);
* ``attention_2`` - grouped-query attention with rotary positions on the first ``rot.dims``
  elements of a head (neighbouring pairs), a sliding window ``mask.size`` that keeps the first
  ``mask.keep_first`` tokens visible, and a sigmoid gate per head on the output.

Feed-forwards (``mlp.kind``): ``dense`` - a gated unit g' sigmoid(1.702 g') (u' + 1) with
g' = min(g, limit), u' = clamp(u, +-limit); ``moe`` - ``router.experts`` such units of which a
token uses the ``router.top`` with the largest sigmoid scores, each on score * x, plus a
shared unit times sigmoid(sg . x).

``loop`` = {start, stop, times}: layers start .. stop - 1 run ``times`` times in a row with
the same weights, every pass with a cache of its own; row t of ``loop.step`` [times, width]
is added to the residual stream right before pass t.

Tensor names: ``embed``, ``loop.step``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.norm2``,
``l<i>.mlp.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from dataclasses import dataclass

from ..errors import ConfigError
from .specs import (
    AttentionSpec,
    DifferentialSpec,
    GatedMLPSpec,
    LayerSpec,
    ModelSpec,
    NoPositionSpec,
    NormSpec,
    RotarySpec,
    RoutedMLPSpec,
    RunSpec,
)
from .zofadra import MAX_POSITIONS, _int, _number

SWISH_SLOPE = 1.702              # the gated unit's sigmoid is taken of 1.702 g
LOOP_STEP = "loop.step"

_BARE = (("weight", ""),)        # a norm's weight is stored under the norm's own name
_UNIT = (("gate_proj.weight", "gate"), ("up_proj.weight", "up"), ("down_proj.weight", "down"))
_ATTENTION = (("q_proj.weight", "q"), ("k_proj.weight", "k"), ("v_proj.weight", "v"), ("o_proj.weight", "o"),
              ("gate_proj.weight", "g"), ("lambda_q1", "lq1"), ("lambda_k1", "lk1"), ("lambda_q2", "lq2"),
              ("lambda_k2", "lk2"))


@dataclass(frozen=True)
class TekilornLayer:
    type: str
    mixer: dict
    mlp: dict | None


@dataclass(frozen=True)
class TekilornLoop:
    start: int
    stop: int
    times: int


def _unit(raw: dict, where: str) -> None:
    _int(raw, "ff", where)
    if _number(raw, "limit", where) <= 0:
        raise ConfigError(f"{where}.limit must be positive")


@dataclass(frozen=True)
class TekilornConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple
    loop: TekilornLoop | None

    architecture = "Tekilorn"

    @classmethod
    def from_dict(cls, raw: dict) -> "TekilornConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json 'layers' must be a non-empty list")
        eps = _number(raw.get("norm") or {}, "eps", "norm")
        if eps <= 0:
            raise ConfigError("norm.eps must be positive")
        layers = []
        for index, item in enumerate(layers_raw):
            where = f"layers[{index}]"
            kind = item.get("type")
            mixer = item.get("mixer")
            if not isinstance(mixer, dict):
                raise ConfigError(f"{where}.mixer must be an object")
            if kind not in ("attention", "attention_2"):
                raise ConfigError(f"{where}.type={kind!r}; known: attention, attention_2")
            for key in ("heads", "kv_heads", "dim", "vdim"):
                _int(mixer, key, f"{where}.mixer")
            if mixer["heads"] % mixer["kv_heads"]:
                raise ConfigError(f"{where}.mixer.heads must be a multiple of kv_heads")
            _number(mixer, "scale", f"{where}.mixer")
            if kind == "attention":
                _number(mixer, "diff", f"{where}.mixer")
                if mixer.get("softcap") is not None and _number(mixer, "softcap", f"{where}.mixer") <= 0:
                    raise ConfigError(f"{where}.mixer.softcap must be positive")
                temp = mixer.get("q_temp")
                if temp is not None:
                    _number(temp, "coef", f"{where}.mixer.q_temp")
                    _int(temp, "every", f"{where}.mixer.q_temp")
            else:
                rot = mixer.get("rot")
                if rot is not None:
                    dims = _int(rot, "dims", f"{where}.mixer.rot", 2)
                    if dims % 2 or dims > mixer["dim"]:
                        raise ConfigError(f"{where}.mixer.rot.dims must be even and at most dim")
                    if _number(rot, "base", f"{where}.mixer.rot") <= 0:
                        raise ConfigError(f"{where}.mixer.rot.base must be positive")
                mask = mixer.get("mask")
                if mask is not None:
                    if mask.get("size") is not None:
                        _int(mask, "size", f"{where}.mixer.mask")
                    if mask.get("keep_first") is not None:
                        _int(mask, "keep_first", f"{where}.mixer.mask", 0)
            mlp = item.get("mlp")
            if mlp is not None:
                style = mlp.get("kind", "dense")
                if style == "dense":
                    _unit(mlp, f"{where}.mlp")
                elif style == "moe":
                    router = mlp.get("router") or {}
                    experts = _int(router, "experts", f"{where}.mlp.router")
                    top = _int(router, "top", f"{where}.mlp.router")
                    if top > experts:
                        raise ConfigError(f"{where}.mlp.router.top must be at most experts")
                    _unit(mlp.get("expert") or {}, f"{where}.mlp.expert")
                    if mlp.get("shared") is not None:
                        _unit(mlp["shared"], f"{where}.mlp.shared")
                else:
                    raise ConfigError(f"{where}.mlp.kind={style!r}; known: dense, moe")
            layers.append(TekilornLayer(kind, dict(mixer), None if mlp is None else dict(mlp)))
        loop = None
        if raw.get("loop") is not None:
            loop_raw = raw["loop"]
            loop = TekilornLoop(_int(loop_raw, "start", "loop", 0), _int(loop_raw, "stop", "loop", 0),
                                _int(loop_raw, "times", "loop"))
            if not loop.start <= loop.stop <= len(layers):
                raise ConfigError(f"loop: start={loop.start}, stop={loop.stop} do not name a stretch of the {len(layers)} layers")
        return cls(vocab=_int(raw, "vocab", "config"), width=_int(raw, "width", "config"), eps=eps,
                   layers=tuple(layers), loop=loop)

    # ------------------------------------------------------------------------------
    def _mixer_spec(self, layer: TekilornLayer):
        m = layer.mixer
        common = dict(hidden_size=self.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                      qk_norm=False, qk_norm_eps=self.eps, bias=False, scale=float(m["scale"]), v_head_dim=m["vdim"],
                      rename=_ATTENTION)
        if layer.type == "attention":
            temp = m.get("q_temp")
            return AttentionSpec(
                **common, position=NoPositionSpec(), window=None,
                softcap=None if m.get("softcap") is None else float(m["softcap"]),
                query_temperature=None if temp is None else (float(temp["coef"]), int(temp["every"])),
                differential=DifferentialSpec(offset=float(m["diff"]), eps=self.eps),
            )
        rot = m.get("rot")
        mask = m.get("mask") or {}
        position = NoPositionSpec() if rot is None else RotarySpec(m["dim"], float(rot["base"]), int(rot["dims"]), interleaved=True)
        window = mask.get("size")
        return AttentionSpec(**common, position=position, window=window,
                             keep_first=int(mask.get("keep_first") or 0) if window is not None else 0, head_gate=True)

    def _unit_spec(self, raw: dict) -> GatedMLPSpec:
        return GatedMLPSpec(self.width, raw["ff"], "clamped_swish", rename=_UNIT, limit=float(raw["limit"]), slope=SWISH_SLOPE)

    def _ffn_spec(self, mlp: dict):
        if mlp.get("kind", "dense") == "dense":
            return self._unit_spec(mlp)
        shared = mlp.get("shared")
        return RoutedMLPSpec(
            hidden_size=self.width, experts=mlp["router"]["experts"], top=mlp["router"]["top"],
            expert=self._unit_spec(mlp["expert"]), shared=None if shared is None else self._unit_spec(shared),
            score="sigmoid", renormalise=False, weight_on="input", shared_gate=shared is not None,
        )

    def runs(self) -> list:
        """(layer, pass of the loop or None) for every layer run, in order."""
        count = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(count)]
        out = [(i, None) for i in range(self.loop.start)]
        for t in range(self.loop.times):
            out += [(i, t) for i in range(self.loop.start, self.loop.stop)]
        return out + [(i, None) for i in range(self.loop.stop, count)]

    def to_model_spec(self) -> ModelSpec:
        layers = []
        for index, layer in enumerate(self.layers):
            prefix = f"l{index}"
            ffn = None if layer.mlp is None else self._ffn_spec(layer.mlp)
            layers.append(LayerSpec(
                input_norm=NormSpec(self.width, self.eps, rename=_BARE),
                mixer=self._mixer_spec(layer),
                post_norm=None if ffn is None else NormSpec(self.width, self.eps, rename=_BARE),
                ffn=ffn,
                names={"input_norm": f"{prefix}.norm1", "mixer": f"{prefix}.mix", "post_norm": f"{prefix}.norm2",
                       "ffn": f"{prefix}.mlp"},
            ))
        schedule = []
        for index, t in self.runs():
            first = t is not None and index == self.loop.start
            schedule.append(RunSpec(index, shift=(LOOP_STEP, t) if first else None))
        extra = ()
        if self.loop is not None:
            extra = ((LOOP_STEP, (self.loop.times, self.width), "bias"),)
        return ModelSpec(
            vocab_size=self.vocab, hidden_size=self.width, layers=tuple(layers), schedule=tuple(schedule),
            final_norm=NormSpec(self.width, self.eps, rename=_BARE), tie_embeddings=False,
            max_positions=MAX_POSITIONS, eos_token_ids=(), embed_name="embed", final_norm_name="final.norm",
            head_name="head", extra_tensors=extra,
        )
