"""Linear attention with a fixed decay per head ("lightning" attention).

q = act(W_q x), k = act(W_k x) [heads x dim], v = act(W_v x) [heads x vdim]; per head the
state S [dim, vdim] follows S_t = decay_h S_(t-1) + k_t v_t^T and the output is
o_t = S_t^T q_t.  The heads' outputs are RMS-normalised together, multiplied by
sigmoid(W_g x) and projected.  The state is 32-bit, starts at zero and lives in the request's
state slot between steps; q, k, v, g come from one fused projection whose 32-bit sums the
recurrence kernel reads (the activation is taken there, in 32-bit).
"""

from __future__ import annotations

import torch

from ..cache.manager import CacheNeeds, StateSpec
from ..config.specs import local_name
from ..errors import ConfigError
from ..ops import native
from .base import BuildContext, CacheView, Mixer, WeightInfo, register_part
from .linear import Linear, fused_rows

_ACTIVATIONS = {"silu": native.ACT_SILU, "none": -1}


class LinearRecurrence(Mixer):
    graph_safe = True      # the state is indexed on the device, by the batch's slots

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        if spec.activation not in _ACTIVATIONS:
            raise ConfigError(f"activation {spec.activation!r}; known: {', '.join(_ACTIVATIONS)}")
        if len(spec.decay) != spec.num_heads:
            raise ConfigError("one decay per head is needed")
        self.spec, self.ctx = spec, ctx
        self.h, self.dk, self.dv = spec.num_heads, spec.head_dim, spec.v_head_dim
        self.act = _ACTIVATIONS[spec.activation]
        name = lambda canonical: local_name(spec, canonical)  # noqa: E731
        rows = [self.h * self.dk, self.h * self.dk, self.h * self.dv, self.h * self.dv]
        self.proj = Linear(fused_rows(weights, [name("q"), name("k"), name("v"), name("g")], rows), status=ctx.status)
        self.norm = weights[name("norm")].float().contiguous()
        self.o_proj = Linear(weights[name("o")], status=ctx.status)
        self.decay = torch.tensor(spec.decay, dtype=torch.float64).float().to(ctx.device)

    @classmethod
    def weight_shapes(cls, spec) -> dict:
        name = lambda canonical: local_name(spec, canonical)  # noqa: E731
        qk, v, w = spec.num_heads * spec.head_dim, spec.num_heads * spec.v_head_dim, spec.hidden_size
        return {
            name("q"): WeightInfo((qk, w)),
            name("k"): WeightInfo((qk, w)),
            name("v"): WeightInfo((v, w)),
            name("g"): WeightInfo((v, w)),
            name("o"): WeightInfo((w, v)),
            name("norm"): WeightInfo((v,), "norm"),
        }

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(state=StateSpec((self.h, self.dk, self.dv), "float32"))

    def forward(self, x, batch, cache: CacheView):
        n = x.shape[0]
        qk, v = self.h * self.dk, self.h * self.dv
        with self.ctx.section("mixer.projection"):
            proj = self.proj(x, out_dtype=torch.float32)
        mixed = torch.empty((n, v), dtype=torch.float32, device=x.device)
        with self.ctx.section("mixer.recurrence"):
            native.linear_recurrence(proj, 0, qk, 2 * qk, self.act, cache.state, batch.slots, batch.cu_tokens,
                                     self.decay, mixed, batch.n_entries, batch.max_new)
        gated = torch.empty((n, v), dtype=self.ctx.dtype, device=x.device)
        with self.ctx.section("mixer.gate_norm"):
            native.gated_rmsnorm(mixed, proj[:, 2 * qk + v:], self.norm, gated, self.spec.norm_eps)
        with self.ctx.section("mixer.o_proj"):
            return self.o_proj(gated)


register_part("linear_recurrence", LinearRecurrence, replace=True)
