"""The Zofadra configuration: a decoder whose layers are listed one by one.

``config.json`` names the architecture in ``architecture`` and gives ``vocab``,
``width``, ``norm.eps``, optionally ``embedding.scale``, ``residual_mult`` and ``streams``,
and ``layers``: per layer its ``type`` (which mixer), the mixer's sizes (``mixer``) and its
feed-forward (``mlp``, or null for a layer that has none).  Three mixers exist:

* ``latent_attention`` - queries through a normalised latent, keys and values expanded from
  one cached latent plus one rotated key part shared by all heads; ``kv_from`` reads an
  earlier layer's cache instead of projecting one;
* ``attention`` - grouped-query attention without rotation, q and k normalised over the
  whole projection, a bias on the distance with slopes 2^(-8 (h + 1) / heads), optionally a
  sliding window (``mask.size``);
* ``lightning`` - linear attention with a fixed decay per head and a 32-bit state.

Every layer is pre-norm (layer norm with a weight, no bias); with ``streams`` the residual
stream exists in that many copies mixed by learned weights (tensors ``hc1.*``, ``hc2.*``).
Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.norm2``, ``l<i>.mlp.*``,
``l<i>.hc<q>.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

from ..errors import ConfigError
from .specs import (
    AttentionSpec,
    GatedMLPSpec,
    LatentAttentionSpec,
    LayerNormSpec,
    LayerSpec,
    LinearRecurrenceSpec,
    ModelSpec,
    NoPositionSpec,
    RotarySpec,
    RunSpec,
    StreamMixSpec,
)

DISTANCE_BIAS_BASE = 256.0       # slopes 2^(-8 (h + 1) / heads)
MAX_POSITIONS = 1 << 24          # positions are exact as 32-bit floats up to here

_BARE = (("weight", ""),)        # a norm's weight is stored under the norm's own name


def _int(raw: dict, key: str, where: str, minimum: int = 1) -> int:
    value = raw.get(key)
    if isinstance(value, bool) or not isinstance(value, int) or value < minimum:
        raise ConfigError(f"{where}.{key}={value!r} must be an integer of at least {minimum}")
    return value


def _number(raw: dict, key: str, where: str) -> float:
    value = raw.get(key)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value):
        raise ConfigError(f"{where}.{key}={value!r} must be a finite number")
    return float(value)


@dataclass(frozen=True)
class ZofadraLayer:
    type: str
    mixer: dict
    ff: int | None          # width of the gated feed-forward, None for a layer without one


@dataclass(frozen=True)
class ZofadraConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    residual_mult: float
    streams: int | None     # None: one residual stream and the plain residual sum
    layers: tuple

    architecture = "Zofadra"

    @classmethod
    def from_dict(cls, raw: dict) -> "ZofadraConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json 'layers' must be a non-empty list")
        norm = raw.get("norm") or {}
        eps = _number(norm, "eps", "norm")
        if eps <= 0:
            raise ConfigError("norm.eps must be positive")
        layers = []
        for index, item in enumerate(layers_raw):
            where = f"layers[{index}]"
            kind = item.get("type")
            mixer = item.get("mixer")
            if not isinstance(mixer, dict):
                raise ConfigError(f"{where}.mixer must be an object")
            if kind == "latent_attention":
                for key in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"):
                    _int(mixer, key, f"{where}.mixer")
                _number(mixer, "scale", f"{where}.mixer")
                rot = mixer.get("rot") or {}
                dims = _int(rot, "dims", f"{where}.mixer.rot", 2)
                if dims % 2 or dims > mixer["rot_dim"]:
                    raise ConfigError(f"{where}.mixer.rot.dims must be even and at most rot_dim")
                if _number(rot, "base", f"{where}.mixer.rot") <= 0:
                    raise ConfigError(f"{where}.mixer.rot.base must be positive")
                source = mixer.get("kv_from")
                if source is not None:
                    if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < index:
                        raise ConfigError(f"{where}.mixer.kv_from must name an earlier layer")
                    other = layers[source]
                    if other.type != "latent_attention" or other.mixer.get("kv_from") is not None:
                        raise ConfigError(f"{where}.mixer.kv_from={source}: that layer projects no latent of its own")
                    for key in ("kv_rank", "rot_dim"):
                        if other.mixer[key] != mixer[key]:
                            raise ConfigError(f"{where}.mixer.{key} differs from layer {source}'s")
                    if other.mixer["rot"] != mixer["rot"]:
                        raise ConfigError(f"{where}.mixer.rot differs from layer {source}'s")
            elif kind == "attention":
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    _int(mixer, key, f"{where}.mixer")
                if mixer["heads"] % mixer["kv_heads"]:
                    raise ConfigError(f"{where}.mixer.heads must be a multiple of kv_heads")
                _number(mixer, "scale", f"{where}.mixer")
                mask = mixer.get("mask")
                if mask is not None and mask.get("size") is not None:
                    _int(mask, "size", f"{where}.mixer.mask")
            elif kind == "lightning":
                for key in ("heads", "dim", "vdim"):
                    _int(mixer, key, f"{where}.mixer")
                decay = mixer.get("decay")
                if not isinstance(decay, list) or len(decay) != mixer["heads"]:
                    raise ConfigError(f"{where}.mixer.decay must list one number per head")
                for d in decay:
                    if isinstance(d, bool) or not isinstance(d, (int, float)) or not math.isfinite(d):
                        raise ConfigError(f"{where}.mixer.decay holds {d!r}")
            else:
                raise ConfigError(f"{where}.type={kind!r}; known: attention, latent_attention, lightning")
            mlp = item.get("mlp")
            ff = None
            if mlp is not None:
                if mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"{where}.mlp.kind={mlp.get('kind')!r}; known: dense")
                ff = _int(mlp, "ff", f"{where}.mlp")
            layers.append(ZofadraLayer(kind, dict(mixer), ff))
        streams = raw.get("streams")
        if streams is not None:
            streams = _int(raw, "streams", "config")
        embedding = raw.get("embedding") or {}
        return cls(
            vocab=_int(raw, "vocab", "config"),
            width=_int(raw, "width", "config"),
            eps=eps,
            embedding_scale=_number(embedding, "scale", "embedding") if "scale" in embedding else 1.0,
            residual_mult=_number(raw, "residual_mult", "config") if "residual_mult" in raw else 1.0,
            streams=streams,
            layers=tuple(layers),
        )

    # ------------------------------------------------------------------------------
    def _mixer_spec(self, layer: ZofadraLayer):
        m = layer.mixer
        if layer.type == "latent_attention":
            rot = m["rot"]
            return LatentAttentionSpec(
                hidden_size=self.width, num_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"],
                v_head_dim=m["vdim"], q_rank=m["q_rank"], kv_rank=m["kv_rank"], norm_eps=self.eps,
                scale=float(m["scale"]),
                position=RotarySpec(m["rot_dim"], float(rot["base"]), int(rot["dims"]), interleaved=True),
                kv_from=m.get("kv_from"),
            )
        if layer.type == "attention":
            mask = m.get("mask") or {}
            return AttentionSpec(
                hidden_size=self.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                qk_norm=True, qk_norm_eps=self.eps, bias=False, scale=float(m["scale"]),
                position=NoPositionSpec(), window=mask.get("size"),
                v_head_dim=m["vdim"], qk_norm_scope="whole", distance_bias_base=DISTANCE_BIAS_BASE,
                rename=(("q_proj.weight", "q"), ("k_proj.weight", "k"), ("v_proj.weight", "v"),
                        ("o_proj.weight", "o"), ("q_norm.weight", "q.norm"), ("k_norm.weight", "k.norm")),
            )
        return LinearRecurrenceSpec(
            hidden_size=self.width, num_heads=m["heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
            decay=tuple(float(d) for d in m["decay"]), norm_eps=self.eps, activation="silu",
        )

    def to_model_spec(self) -> ModelSpec:
        layers, schedule = [], []
        options = StreamMixSpec(streams=self.streams or 1, learned=self.streams is not None,
                                update_scale=self.residual_mult)
        for index, layer in enumerate(self.layers):
            prefix = f"l{index}"
            ffn = None
            if layer.ff is not None:
                ffn = GatedMLPSpec(self.width, layer.ff, "gelu_tanh",
                                   rename=(("gate_proj.weight", "gate"), ("up_proj.weight", "up"),
                                           ("down_proj.weight", "down")))
            layers.append(LayerSpec(
                input_norm=LayerNormSpec(self.width, self.eps, rename=_BARE),
                mixer=self._mixer_spec(layer),
                post_norm=None if ffn is None else LayerNormSpec(self.width, self.eps, rename=_BARE),
                ffn=ffn,
                names={"input_norm": f"{prefix}.norm1", "mixer": f"{prefix}.mix", "post_norm": f"{prefix}.norm2",
                       "ffn": f"{prefix}.mlp", "mix1": f"{prefix}.hc1", "mix2": f"{prefix}.hc2"},
                arrangement="stream_mix",
                options=options,
            ))
            schedule.append(RunSpec(index, cache_of=layer.mixer.get("kv_from") if layer.type == "latent_attention" else None))
        return ModelSpec(
            vocab_size=self.vocab,
            hidden_size=self.width,
            layers=tuple(layers),
            schedule=tuple(schedule),
            final_norm=LayerNormSpec(self.width, self.eps, rename=_BARE),
            tie_embeddings=False,
            max_positions=MAX_POSITIONS,
            eos_token_ids=(),
            embed_name="embed",
            final_norm_name="final.norm",
            head_name="head",
            embedding_scale=self.embedding_scale,
            residual_streams=self.streams or 1,
        )
