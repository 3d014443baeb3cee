"""A plain, slow restatement of the Tekilorn decoder: whole sequences, no cache, no batch.

One function per mechanism, written from the design's equations with dense tensors
(every score of a sequence at once, a Python loop over experts, over heads where that
reads better).  It shares nothing with the package: tests compare the engine with it.
``weights`` maps checkpoint tensor names to tensors; ``config`` is the dict of config.json.
Everything runs in the dtype of ``work`` (64-bit by default).
"""

from __future__ import annotations

import math

import torch

SIGMOID_SLOPE = 1.702          # the gate of the feed-forward is g * sigmoid(1.702 g)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def weighted_norm(x, weight, eps):
    return rms(x, eps) * weight


def visible(length: int, window: int | None = None, keep_first: int = 0) -> torch.Tensor:
    """[query, key] True where query i may look at key j."""
    i = torch.arange(length)[:, None]
    j = torch.arange(length)[None, :]
    mask = j <= i
    if window is not None:
        mask &= (i - j < window) | (j < keep_first)
    return mask


def softmax_attention(q, k, v, mask, scale, softcap=None, row_scale=None):
    """q [T, d], k [T, d], v [T, dv] of one head -> [T, dv]."""
    scores = (q @ k.T) * scale
    if row_scale is not None:
        scores = scores * row_scale[:, None]
    if softcap is not None:
        scores = softcap * torch.tanh(scores / softcap)
    scores = scores.masked_fill(~mask, float("-inf"))
    return torch.softmax(scores, dim=-1) @ v


def query_temperature(length: int, coef: float, every: int, dtype) -> torch.Tensor:
    p = torch.arange(length)
    return 1.0 + coef * torch.log((torch.div(p + 1, every, rounding_mode="floor") + 1).to(dtype))


def rotate_interleaved(x: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: pairs (2i, 2i + 1) of the first ``dims`` elements turn by p * base^(-2i/dims)."""
    length = x.shape[0]
    out = x.clone()
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    angle = torch.arange(length, dtype=x.dtype)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def differential_attention(h, w, prefix, m, eps):
    """The mixer of type "attention": two softmax maps per head over shared values."""
    heads, kv_heads, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    length = h.shape[0]
    q = (h @ w[prefix + "q"].T).view(length, heads, 2, dim)
    k = (h @ w[prefix + "k"].T).view(length, kv_heads, 2, dim)
    v = (h @ w[prefix + "v"].T).view(length, kv_heads, vdim)
    temp = None
    if m.get("q_temp"):
        temp = query_temperature(length, m["q_temp"]["coef"], m["q_temp"]["every"], h.dtype)
    lam = (torch.exp((w[prefix + "lq1"] * w[prefix + "lk1"]).sum())
           - torch.exp((w[prefix + "lq2"] * w[prefix + "lk2"]).sum()) + m["diff"])
    mask = visible(length)
    out = []
    for head in range(heads):
        g = head // (heads // kv_heads)
        maps = [softmax_attention(q[:, head, part], k[:, g, part], v[:, g], mask, m["scale"], m.get("softcap"), temp)
                for part in range(2)]
        o = maps[0] - lam * maps[1]
        out.append(rms(o, eps) * (1.0 - m["diff"]))
    return torch.cat(out, dim=-1) @ w[prefix + "o"].T


def gated_window_attention(h, w, prefix, m):
    """The mixer of type "attention_2": rotary positions, a window that keeps the first
    tokens, and a gate per head on the output."""
    heads, kv_heads, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    length = h.shape[0]
    q = (h @ w[prefix + "q"].T).view(length, heads, dim)
    k = (h @ w[prefix + "k"].T).view(length, kv_heads, dim)
    v = (h @ w[prefix + "v"].T).view(length, kv_heads, vdim)
    rot = m.get("rot")
    if rot:
        q = rotate_interleaved(q, rot["dims"], rot["base"])
        k = rotate_interleaved(k, rot["dims"], rot["base"])
    mask_cfg = m.get("mask") or {}
    mask = visible(length, mask_cfg.get("size"), mask_cfg.get("keep_first", 0))
    gate = torch.sigmoid(h @ w[prefix + "g"].T)            # [T, heads]
    out = []
    for head in range(heads):
        g = head // (heads // kv_heads)
        o = softmax_attention(q[:, head], k[:, g], v[:, g], mask, m["scale"])
        out.append(o * gate[:, head : head + 1])
    return torch.cat(out, dim=-1) @ w[prefix + "o"].T


def clamped_gated_unit(h, w, prefix, limit):
    """down(g sigmoid(1.702 g) (u + 1)) with g capped from above and u clamped to +-limit."""
    g = torch.clamp(h @ w[prefix + "gate"].T, max=limit)
    u = torch.clamp(h @ w[prefix + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(SIGMOID_SLOPE * g) * (u + 1.0)) @ w[prefix + "down"].T


def routed_feed_forward(h, w, prefix, mlp):
    """Sigmoid router; the chosen experts' scores scale the experts' *inputs*."""
    experts, top = mlp["router"]["experts"], mlp["router"]["top"]
    scores = torch.sigmoid(h @ w[prefix + "router"].T)
    chosen = torch.topk(scores, top, dim=-1).indices
    out = torch.zeros_like(h)
    for token in range(h.shape[0]):
        for e in chosen[token].tolist():
            x = (scores[token, e] * h[token])[None, :]
            out[token] += clamped_gated_unit(x, w, f"{prefix}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        shared_gate = torch.sigmoid(h @ w[prefix + "shared.sg"].T)      # [T, 1]
        out = out + shared_gate * clamped_gated_unit(h, w, prefix + "shared.", mlp["shared"]["limit"])
    return out


def feed_forward(h, w, prefix, mlp):
    if mlp["kind"] == "dense":
        return clamped_gated_unit(h, w, prefix, mlp["limit"])
    return routed_feed_forward(h, w, prefix, mlp)


def layer_order(config: dict) -> list:
    """(layer index, number of the pass or None) for every layer run, in order."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(count)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t) for i in range(loop["start"], loop["stop"])]
    runs += [(i, None) for i in range(loop["stop"], count)]
    return runs


def forward(config: dict, weights: dict, tokens, work=torch.float64, layers_out: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; ``layers_out`` collects the residual stream after every layer run."""
    w = {name: (t.to(work) if t.is_floating_point() else t) for name, t in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    loop = config.get("loop")
    for index, t in layer_order(config):
        if t is not None and index == loop["start"]:
            x = x + w["loop.step"][t]
        layer = config["layers"][index]
        prefix = f"l{index}."
        h = weighted_norm(x, w[prefix + "norm1"], eps)
        if layer["type"] == "attention":
            x = x + differential_attention(h, w, prefix + "mix.", layer["mixer"], eps)
        elif layer["type"] == "attention_2":
            x = x + gated_window_attention(h, w, prefix + "mix.", layer["mixer"])
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp"):
            h = weighted_norm(x, w[prefix + "norm2"], eps)
            x = x + feed_forward(h, w, prefix + "mlp.", layer["mlp"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return weighted_norm(x, w["final.norm"], eps) @ w["head"].T


# ---------------------------------------------------------------------------
# small random models for tests
# ---------------------------------------------------------------------------
def tensor_shapes(config: dict) -> dict:
    width = config["width"]
    shapes = {"embed": (config["vocab"], width), "final.norm": (width,), "head": (config["vocab"], width)}
    if config.get("loop"):
        shapes["loop.step"] = (config["loop"]["times"], width)
    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], f"l{i}."
        shapes[p + "norm1"] = (width,)
        parts = 2 if layer["type"] == "attention" else 1
        shapes[p + "mix.q"] = (m["heads"] * parts * m["dim"], width)
        shapes[p + "mix.k"] = (m["kv_heads"] * parts * m["dim"], width)
        shapes[p + "mix.v"] = (m["kv_heads"] * m["vdim"], width)
        shapes[p + "mix.o"] = (width, m["heads"] * m["vdim"])
        if layer["type"] == "attention":
            for name in ("lq1", "lk1", "lq2", "lk2"):
                shapes[p + "mix." + name] = (m["dim"],)
        else:
            shapes[p + "mix.g"] = (m["heads"], width)
        mlp = layer.get("mlp")
        if not mlp:
            continue
        shapes[p + "norm2"] = (width,)

        def unit(prefix, ff):
            shapes[prefix + "gate"] = (ff, width)
            shapes[prefix + "up"] = (ff, width)
            shapes[prefix + "down"] = (width, ff)

        if mlp["kind"] == "dense":
            unit(p + "mlp.", mlp["ff"])
        else:
            for e in range(mlp["router"]["experts"]):
                unit(f"{p}mlp.e{e}.", mlp["expert"]["ff"])
            shapes[p + "mlp.router"] = (mlp["router"]["experts"], width)
            if mlp.get("shared"):
                unit(p + "mlp.shared.", mlp["shared"]["ff"])
                shapes[p + "mlp.shared.sg"] = (1, width)
    return shapes


def random_weights(config: dict, seed: int, dtype=torch.bfloat16) -> dict:
    """Weights large enough that every mechanism matters: matrices with entries of about
    1/sqrt(fan-in) times a gain, norm weights around 1."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2") or name == "final.norm":
            t = 1.0 + 0.1 * torch.randn(shape, generator=gen)
        elif name == "embed":
            t = torch.randn(shape, generator=gen)
        elif name == "loop.step":
            t = 0.5 * torch.randn(shape, generator=gen)
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            t = 0.3 * torch.randn(shape, generator=gen)
        else:
            gain = {"q": 2.0, "k": 2.0, "router": 3.0, "g": 3.0, "sg": 3.0, "gate": 2.0, "up": 2.0}.get(leaf, 1.0)
            t = gain * torch.randn(shape, generator=gen) / math.sqrt(shape[-1])
        out[name] = t.to(dtype)
    return out


# ---------------------------------------------------------------------------
# builders of small configurations
# ---------------------------------------------------------------------------
def dense(ff=48, limit=1.25):
    return {"kind": "dense", "ff": ff, "limit": limit}


def routed(experts=5, top=2, ff=24, limit=1.25, shared_ff=40, shared_limit=2.0):
    mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared_ff is not None:
        mlp["shared"] = {"ff": shared_ff, "limit": shared_limit}
    return mlp


def differential_layer(heads=4, kv_heads=2, dim=16, vdim=32, diff=0.25, softcap=20.0, q_temp=(0.4, 8), scale=None,
                       mlp="dense"):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff,
             "scale": scale if scale is not None else dim ** -0.5}
    if softcap is not None:
        mixer["softcap"] = softcap
    if q_temp is not None:
        mixer["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return {"type": "attention", "mixer": mixer, "mlp": dense() if mlp == "dense" else mlp}


def window_layer(heads=4, kv_heads=2, dim=16, vdim=16, window=9, keep_first=3, rot_dims=8, base=100.0, scale=None,
                 mlp="dense"):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
             "scale": scale if scale is not None else dim ** -0.5}
    if rot_dims:
        mixer["rot"] = {"dims": rot_dims, "base": base}
    if window is not None:
        mixer["mask"] = {"size": window, "keep_first": keep_first}
    return {"type": "attention_2", "mixer": mixer, "mlp": dense() if mlp == "dense" else mlp}


def config(layers, width=64, vocab=97, eps=1e-5, loop=None) -> dict:
    cfg = {"architecture": "Tekilorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": list(layers)}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def greedy_generate(cfg: dict, weights: dict, prompt, count: int) -> list:
    ids = list(prompt)
    for _ in range(count):
        ids.append(int(forward(cfg, weights, ids)[-1].argmax()))
    return ids[len(prompt):]
