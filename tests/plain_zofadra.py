"""A slow, plain restatement of the Zofadra design in 64-bit on the CPU: one function per
mechanism, whole sequences only (no cache, no state carried between calls).  The engine is
compared with this; nothing here is shared with the package.

Notation: T tokens, positions 0..T-1; weights are a dict name -> tensor, linear weights
[out, in] applied as x @ W.T.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


# -- small pieces -------------------------------------------------------------------------
def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def layer_norm(x, w, eps):
    centred = x - x.mean(-1, keepdim=True)
    return centred / torch.sqrt((centred * centred).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z**3)))


def rotate_pairs(x, positions, base, dims):
    """Rotate the first ``dims`` elements of the last axis of x [T, ..., D]: elements 2i and
    2i + 1 form a pair turned by the angle position * base^(-2i / dims)."""
    out = x.clone()
    for i in range(dims // 2):
        angle = positions.to(F64) * base ** (-2.0 * i / dims)
        shape = [-1] + [1] * (x.dim() - 2)
        c, s = torch.cos(angle).view(shape), torch.sin(angle).view(shape)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def softmax_rows(scores, visible):
    return torch.softmax(scores.masked_fill(~visible, -math.inf), dim=-1)


# -- mixers -------------------------------------------------------------------------------
def latent_kv(h, W, p, m, eps, positions):
    """The cached pair of a latent-attention layer: (latent [T, kv_rank], rotated shared key
    part [T, rot_dim])."""
    rank = m["kv_rank"]
    both = h @ W[p + ".dkv"].T
    latent = rms_norm(both[:, :rank], W[p + ".dkv.norm"], eps)
    shared = rotate_pairs(both[:, rank:], positions, m["rot"]["base"], m["rot"]["dims"])
    return latent, shared


def latent_attention(h, W, p, m, eps, positions, kv):
    """``kv`` is this layer's own ``latent_kv`` or the one of the layer it reads from."""
    T, H, d, r, dv = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    latent, shared = kv
    q = (rms_norm(h @ W[p + ".dq"].T, W[p + ".dq.norm"], eps) @ W[p + ".uq"].T).view(T, H, d + r)
    q_plain = q[:, :, :d]
    q_turned = rotate_pairs(q[:, :, d:], positions, m["rot"]["base"], m["rot"]["dims"])
    keys = (latent @ W[p + ".uk"].T).view(T, H, d)
    values = (latent @ W[p + ".uv"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    visible = positions[:, None] >= positions[None, :]
    for head in range(H):
        scores = (q_plain[:, head] @ keys[:, head].T + q_turned[:, head] @ shared.T) * m["scale"]
        out[:, head] = softmax_rows(scores, visible) @ values[:, head]
    return out.reshape(T, H * dv) @ W[p + ".o"].T


def biased_attention(h, W, p, m, eps, positions):
    T, H, G, d, dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(h @ W[p + ".q"].T, W[p + ".q.norm"], eps).view(T, H, d)
    k = rms_norm(h @ W[p + ".k"].T, W[p + ".k.norm"], eps).view(T, G, d)
    v = (h @ W[p + ".v"].T).view(T, G, dv)
    distance = (positions[:, None] - positions[None, :]).to(F64)
    visible = distance >= 0
    size = (m.get("mask") or {}).get("size")
    if size is not None:
        visible = visible & (distance < size)
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        group = head // (H // G)
        slope = 2.0 ** (-8.0 * (head + 1) / H)
        scores = (q[:, head] @ k[:, group].T) * m["scale"] - slope * distance
        out[:, head] = softmax_rows(scores, visible) @ v[:, group]
    return out.reshape(T, H * dv) @ W[p + ".o"].T


def lightning(h, W, p, m, eps):
    T, H, d, dv = h.shape[0], m["heads"], m["dim"], m["vdim"]
    silu = torch.nn.functional.silu
    q = silu(h @ W[p + ".q"].T).view(T, H, d)
    k = silu(h @ W[p + ".k"].T).view(T, H, d)
    v = silu(h @ W[p + ".v"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        state = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            state = m["decay"][head] * state + torch.outer(k[t, head], v[t, head])
            out[t, head] = state.T @ q[t, head]
    gated = rms_norm(out.reshape(T, H * dv), W[p + ".norm"], eps) * torch.sigmoid(h @ W[p + ".g"].T)
    return gated @ W[p + ".o"].T


def feed_forward(h, W, p):
    return (gelu_tanh(h @ W[p + ".gate"].T) * (h @ W[p + ".up"].T)) @ W[p + ".down"].T


# -- the model ----------------------------------------------------------------------------
def forward_logits(cfg: dict, weights: dict, tokens, residuals: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence; ``residuals`` collects the summed streams
    after every layer."""
    W = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    mult = cfg.get("residual_mult", 1.0)
    S = cfg.get("streams")
    T = len(tokens)
    positions = torch.arange(T)
    x0 = W["embed"][torch.tensor(list(tokens))] * cfg.get("embedding", {}).get("scale", 1.0)
    streams = [x0.clone() for _ in range(S or 1)]
    cached: dict = {}

    def sublayer(streams, layer, which, fn):
        norm_w = W[f"{layer}.norm{which}"]
        if S is None:
            return [streams[0] + mult * fn(layer_norm(streams[0], norm_w, eps))]
        w_in, w_out, w_mix = (W[f"{layer}.hc{which}.{n}"] for n in ("in", "out", "mix"))
        y = fn(layer_norm(sum(w_in[s] * streams[s] for s in range(S)), norm_w, eps))
        return [sum(w_mix[s, t] * streams[s] for s in range(S)) + mult * w_out[t] * y for t in range(S)]

    for index, entry in enumerate(cfg["layers"]):
        layer, m = f"l{index}", entry["mixer"]
        p = layer + ".mix"
        if entry["type"] == "latent_attention":
            def mixer(h, p=p, m=m, index=index):
                source = m.get("kv_from")
                if source is None:
                    cached[index] = latent_kv(h, W, p, m, eps, positions)
                    source = index
                return latent_attention(h, W, p, m, eps, positions, cached[source])
        elif entry["type"] == "attention":
            def mixer(h, p=p, m=m):
                return biased_attention(h, W, p, m, eps, positions)
        else:
            def mixer(h, p=p, m=m):
                return lightning(h, W, p, m, eps)
        streams = sublayer(streams, layer, 1, mixer)
        if entry.get("mlp") is not None:
            streams = sublayer(streams, layer, 2, lambda h, layer=layer: feed_forward(h, W, layer + ".mlp"))
        if residuals is not None:
            residuals.append(sum(streams).clone())
    return layer_norm(sum(streams), W["final.norm"], eps) @ W["head"].T


def greedy_generate(cfg: dict, weights: dict, prompt, new_tokens: int) -> list:
    ids = list(prompt)
    for _ in range(new_tokens):
        ids.append(int(forward_logits(cfg, weights, ids)[-1].argmax()))
    return ids[len(prompt):]


# -- configurations and weights -------------------------------------------------------------
def tensor_shapes(cfg: dict) -> dict:
    W, out = cfg["width"], {}
    out["embed"] = (cfg["vocab"], W)
    S = cfg.get("streams")
    for index, entry in enumerate(cfg["layers"]):
        layer, m = f"l{index}", entry["mixer"]
        p = layer + ".mix"
        out[layer + ".norm1"] = (W,)
        if entry["type"] == "latent_attention":
            H, d, r = m["heads"], m["dim"], m["rot_dim"]
            out[p + ".dq"], out[p + ".dq.norm"] = (m["q_rank"], W), (m["q_rank"],)
            out[p + ".uq"] = (H * (d + r), m["q_rank"])
            if m.get("kv_from") is None:
                out[p + ".dkv"], out[p + ".dkv.norm"] = (m["kv_rank"] + r, W), (m["kv_rank"],)
            out[p + ".uk"], out[p + ".uv"] = (H * d, m["kv_rank"]), (H * m["vdim"], m["kv_rank"])
            out[p + ".o"] = (W, H * m["vdim"])
        elif entry["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out[p + ".q"], out[p + ".k"], out[p + ".v"] = (H * d, W), (G * d, W), (G * dv, W)
            out[p + ".q.norm"], out[p + ".k.norm"], out[p + ".o"] = (H * d,), (G * d,), (W, H * dv)
        else:
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            out[p + ".q"], out[p + ".k"] = (H * d, W), (H * d, W)
            out[p + ".v"], out[p + ".g"] = (H * dv, W), (H * dv, W)
            out[p + ".o"], out[p + ".norm"] = (W, H * dv), (H * dv,)
        subs = [1]
        if entry.get("mlp") is not None:
            ff = entry["mlp"]["ff"]
            out[layer + ".norm2"] = (W,)
            out[layer + ".mlp.gate"], out[layer + ".mlp.up"], out[layer + ".mlp.down"] = (ff, W), (ff, W), (W, ff)
            subs.append(2)
        if S is not None:
            for q in subs:
                out[f"{layer}.hc{q}.in"], out[f"{layer}.hc{q}.out"], out[f"{layer}.hc{q}.mix"] = (S,), (S,), (S, S)
    out["final.norm"] = (W,)
    out["head"] = (cfg["vocab"], W)
    return out


def seeded_weights(cfg: dict, seed: int) -> dict:
    """Random weights whose values are exact in bfloat16 (so both engines hold the same
    model), sized so that activations stay of order one."""
    gen = torch.Generator().manual_seed(seed)
    weights = {}
    for name, shape in tensor_shapes(cfg).items():
        noise = torch.randn(shape, generator=gen)
        if name.endswith(".mix") and len(shape) == 2 and ".hc" in name:
            value = torch.eye(shape[0]) + 0.2 * noise
        elif len(shape) == 1:
            value = 1.0 + 0.2 * noise
        elif name == "embed":
            value = noise
        else:
            value = noise * (1.5 / math.sqrt(shape[1]))
        weights[name] = value.to(torch.bfloat16).float()
    return weights


def latent_layer(heads=4, dim=16, rot_dim=16, vdim=16, q_rank=32, kv_rank=32, rot_dims=None, base=10000.0,
                 kv_from=None, ff=64):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "rot": {"base": base, "dims": rot_dims or rot_dim}, "scale": (dim + rot_dim) ** -0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=16, window=None, ff=64):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def lightning_layer(heads=2, dim=16, vdim=8, decay=None, ff=None):
    decay = decay or [0.5 + 0.45 * i / max(1, heads - 1) for i in range(heads)]
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(layers, width=64, vocab=96, streams=2, residual_mult=0.5, scale=2.0, eps=1e-5) -> dict:
    cfg = {"architecture": "Zofadra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams is not None:
        cfg["streams"] = streams
    if residual_mult is not None:
        cfg["residual_mult"] = residual_mult
    if scale is not None:
        cfg["embedding"] = {"scale": scale}
    return cfg
