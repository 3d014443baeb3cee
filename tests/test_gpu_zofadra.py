"""The Zofadra design in the engine against the plain implementation of ``plain_zofadra.py``:
every mechanism alone, whole prompts against portions and token-by-token decoding, unequal
batches, reused pages and slots, edges of windows and pages, other sizes, generation."""

from __future__ import annotations

import json
import math

import pytest
import torch
from safetensors.torch import save_file

import plain_zofadra as pz

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")


# -- helpers --------------------------------------------------------------------------------
def write_model(folder, cfg: dict, seed: int) -> dict:
    weights = pz.seeded_weights(cfg, seed)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    return weights


def make_runner(folder, dtype: str, page_size=4, num_pages=96, max_requests=4, use_graphs=True):
    from forge_engine_b200.engine import ModelRunner

    return ModelRunner.from_folder(folder, dtype=dtype, page_size=page_size, num_pages=num_pages,
                                   max_requests=max_requests, use_graphs=use_graphs)


def tokens_of(cfg: dict, length: int, seed: int) -> list:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (length,), generator=gen).tolist()


def run_schedule(runner, requests: dict, schedule: list) -> dict:
    """``schedule``: steps, each a list of (request, number of its next tokens); a request
    begins at its first entry and ends with its last token.  Logits of every position."""
    from forge_engine_b200.engine import StepEntry

    at = {key: 0 for key in requests}
    rows = {key: [] for key in requests}
    for step in schedule:
        entries = []
        for key, count in step:
            if at[key] == 0:
                runner.begin(key)
            entries.append(StepEntry(key, requests[key][at[key] : at[key] + count], list(range(count))))
        logits = runner.step(entries).float().cpu()
        runner.check_status()
        begin = 0
        for key, count in step:
            rows[key].append(logits[begin : begin + count])
            begin += count
            at[key] += count
            if at[key] == len(requests[key]):
                runner.end(key)
        runner.cache.check_consistency()
    assert all(at[key] == len(requests[key]) for key in requests)
    return {key: torch.cat(parts) for key, parts in rows.items()}


def assert_close(got: torch.Tensor, want: torch.Tensor, dtype: str, what: str = "") -> None:
    want = want.float()
    assert got.shape == want.shape, what
    assert torch.isfinite(got).all(), what
    scale = float(want.abs().max())
    if dtype == "float32":
        worst = float((got - want).abs().max())
        assert worst <= 2e-4 * max(1.0, scale), f"{what}: {worst} against a scale of {scale}"
    else:
        error = float(((got - want) ** 2).mean().sqrt() / (want**2).mean().sqrt())
        assert error <= 3e-2, f"{what}: relative error {error}"
        worst = float((got - want).abs().max())
        assert worst <= 0.15 * max(1.0, scale), f"{what}: {worst} against a scale of {scale}"


def oracle(cfg, weights, tokens) -> torch.Tensor:
    return pz.forward_logits(cfg, weights, tokens)


MIXED = [pz.latent_layer(), pz.attention_layer(window=6), pz.lightning_layer(),
         pz.latent_layer(kv_from=0, heads=2, dim=8, vdim=24, ff=None), pz.attention_layer(window=None, ff=None)]


# -- every mechanism alone --------------------------------------------------------------------
SINGLE = {
    "latent": [pz.latent_layer()],
    "latent_no_ff": [pz.latent_layer(ff=None)],
    "latent_shared": [pz.latent_layer(), pz.latent_layer(kv_from=0, heads=2, dim=8, vdim=8)],
    "attention_window": [pz.attention_layer(window=7)],
    "attention_full": [pz.attention_layer()],
    "attention_values_differ": [pz.attention_layer(dim=16, vdim=24, window=9)],
    "lightning": [pz.lightning_layer()],
    "lightning_ff": [pz.lightning_layer(heads=3, dim=8, vdim=16, ff=48)],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(SINGLE))
@pytest.mark.parametrize("streams", (None, 1, 3))
def test_each_mechanism_alone(tmp_path, name, streams, dtype):
    if streams == 1 and name not in ("latent", "lightning"):
        pytest.skip("one learned stream is covered with two of the mixers")
    cfg = pz.config(SINGLE[name], streams=streams)
    weights = write_model(tmp_path / "m", cfg, 3)
    tokens = tokens_of(cfg, 37, 5)
    runner = make_runner(tmp_path / "m", dtype)
    got = run_schedule(runner, {"a": tokens}, [[("a", 37)]])["a"]
    assert_close(got, oracle(cfg, weights, tokens), dtype, name)


def test_many_streams(tmp_path):
    """More copies of the residual stream than the 16-byte form of the kernel keeps in registers."""
    cfg = pz.config([pz.attention_layer(window=5), pz.lightning_layer()], streams=9)
    weights = write_model(tmp_path / "m", cfg, 21)
    tokens = tokens_of(cfg, 21, 5)
    runner = make_runner(tmp_path / "m", "float32")
    got = run_schedule(runner, {"a": tokens}, [[("a", 18)], [("a", 3)]])["a"]
    assert_close(got, oracle(cfg, weights, tokens), "float32", "nine streams")


def test_residual_after_every_layer(tmp_path):
    """The residual stream (the sum of its copies) after every layer, in 32-bit."""
    from forge_engine_b200.engine import StepEntry
    from forge_engine_b200.ops import native

    cfg = pz.config(MIXED, streams=2)
    weights = write_model(tmp_path / "m", cfg, 8)
    tokens = tokens_of(cfg, 19, 2)
    want: list = []
    pz.forward_logits(cfg, weights, tokens, want)
    runner = make_runner(tmp_path / "m", "float32", use_graphs=False)
    seen = []
    for block in runner.model.blocks:
        inner = block.forward

        def spy(h, pending, batch, cache, inner=inner):
            out = inner(h, pending, batch, cache)
            copy = h.clone()
            update, mix, coefficients, scale = out
            native.stream_mix_norm(copy, update, scale, mix, coefficients, None, native.NORM_NONE, None, 0.0, None)
            seen.append(copy.sum(1).cpu())
            return out

        block.forward = spy
    runner.begin("a")
    runner.step([StepEntry("a", tokens, [0])])
    assert len(seen) == len(want)
    for index, (got, ref) in enumerate(zip(seen, want)):
        assert_close(got, ref, "float32", f"layer {index}")


# -- whole prompts, portions, single tokens -----------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_prefill_against_token_by_token_decoding(tmp_path, dtype):
    cfg = pz.config(MIXED)
    weights = write_model(tmp_path / "m", cfg, 11)
    tokens = tokens_of(cfg, 45, 7)
    ref = oracle(cfg, weights, tokens)
    runner = make_runner(tmp_path / "m", dtype)
    whole = run_schedule(runner, {"a": tokens}, [[("a", 45)]])["a"]
    single = run_schedule(runner, {"b": tokens}, [[("b", 1)] for _ in range(45)])["b"]
    assert_close(whole, ref, dtype, "whole prompt")
    assert_close(single, ref, dtype, "token by token")
    if dtype == "float32":
        assert float((whole - single).abs().max()) <= 2e-5 * float(ref.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_portions_of_several_sizes(tmp_path, dtype):
    cfg = pz.config(MIXED)
    weights = write_model(tmp_path / "m", cfg, 12)
    tokens = tokens_of(cfg, 101, 9)
    ref = oracle(cfg, weights, tokens)
    runner = make_runner(tmp_path / "m", dtype)
    for sizes in ([2, 3, 5, 2, 17, 16, 1, 1, 33, 4, 2, 15], [2] * 20 + [61], [64, 2, 35], [7] * 14 + [3]):
        assert sum(sizes) == 101
        got = run_schedule(runner, {"a": tokens}, [[("a", n)] for n in sizes])["a"]
        assert_close(got, ref, dtype, f"portions {sizes[:4]}...")


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_requests_in_one_batch_against_each_alone(tmp_path, dtype):
    cfg = pz.config(MIXED, streams=3)
    weights = write_model(tmp_path / "m", cfg, 13)
    requests = {"a": tokens_of(cfg, 5, 1), "b": tokens_of(cfg, 41, 2), "c": tokens_of(cfg, 70, 3)}
    schedule = [
        [("c", 30)],
        [("c", 1), ("b", 17)],
        [("a", 2), ("c", 1), ("b", 2)],
        [("b", 22), ("a", 1), ("c", 9)],
        [("a", 1), ("c", 29)],
        [("a", 1)],
    ]
    runner = make_runner(tmp_path / "m", dtype)
    together = run_schedule(runner, requests, schedule)
    for key, tokens in requests.items():
        assert_close(together[key], oracle(cfg, weights, tokens), dtype, f"request {key} in the batch")
        alone = run_schedule(runner, {key + "'": tokens}, [[(key + "'", len(tokens))]])[key + "'"]
        if dtype == "float32":
            assert float((together[key] - alone).abs().max()) <= 2e-5 * float(alone.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_pages_and_slots_freed_and_used_again(tmp_path, dtype):
    """Two state slots and a pool that holds two requests at most: later requests get the
    slots (whose state must start at zero again) and the pages of earlier ones."""
    cfg = pz.config([pz.lightning_layer(ff=32), pz.latent_layer(), pz.attention_layer(window=5)])
    weights = write_model(tmp_path / "m", cfg, 14)
    requests = {key: tokens_of(cfg, n, i) for i, (key, n) in enumerate((("a", 22), ("b", 31), ("c", 27), ("d", 9)))}
    schedule = [
        [("a", 20), ("b", 3)],
        [("a", 2), ("b", 20)],          # a ends
        [("c", 11), ("b", 1)],          # c takes a's slot and pages
        [("b", 7), ("c", 16)],          # both end
        [("d", 9)],
    ]
    runner = make_runner(tmp_path / "m", dtype, page_size=4, num_pages=16, max_requests=2)
    got = run_schedule(runner, requests, schedule)
    assert runner.cache.slots.leased_count == 0 and all(n == 0 for n in runner.cache.leased_pages())
    for key, tokens in requests.items():
        assert_close(got[key], oracle(cfg, weights, tokens), dtype, f"request {key}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_past_every_window(tmp_path, dtype):
    """A short prompt, then far more single tokens than any window or page holds; the decode
    steps are replayed from captured graphs."""
    cfg = pz.config([pz.attention_layer(window=8), pz.lightning_layer(decay=[0.999, 0.7]), pz.latent_layer(),
                     pz.attention_layer(window=3, ff=None)])
    weights = write_model(tmp_path / "m", cfg, 15)
    tokens = tokens_of(cfg, 90, 4)
    runner = make_runner(tmp_path / "m", dtype, page_size=4, num_pages=40)
    got = run_schedule(runner, {"a": tokens}, [[("a", 5)]] + [[("a", 1)] for _ in range(85)])["a"]
    assert_close(got, oracle(cfg, weights, tokens), dtype, "long decoding")
    if runner.use_graphs:
        assert runner.graphs.captured


@pytest.mark.parametrize("dtype", DTYPES)
def test_other_sizes_and_values_that_are_one_or_equal(tmp_path, dtype):
    """Sizes that are no powers of two, heads = kv heads, one kv head, one head, a window of
    one, fewer rotated dimensions than rot_dim, a decay of one, one learned stream, no
    update scale, no embedding scale, a recurrence with and a latent layer without
    feed-forward, the recurrence first."""
    layers = [
        pz.lightning_layer(heads=1, dim=24, vdim=40, decay=[1.0], ff=40),
        pz.latent_layer(heads=3, dim=12, rot_dim=6, vdim=20, q_rank=24, kv_rank=40, rot_dims=4, base=50.0, ff=None),
        pz.attention_layer(heads=3, kv_heads=3, dim=20, vdim=12, window=1),
        pz.attention_layer(heads=5, kv_heads=1, dim=8, vdim=8, window=12, ff=24),
        pz.latent_layer(heads=1, dim=8, rot_dim=6, vdim=8, q_rank=16, kv_rank=40, rot_dims=4, base=50.0, kv_from=1),
        pz.lightning_layer(heads=5, dim=8, vdim=8),
    ]
    cfg = pz.config(layers, width=72, vocab=50, streams=1, residual_mult=None, scale=None, eps=1e-3)
    weights = write_model(tmp_path / "m", cfg, 16)
    tokens = tokens_of(cfg, 40, 6)
    ref = oracle(cfg, weights, tokens)
    runner = make_runner(tmp_path / "m", dtype, page_size=8, num_pages=24)
    got = run_schedule(runner, {"a": tokens}, [[("a", 13)], [("a", 2)], [("a", 20)]] + [[("a", 1)]] * 5)["a"]
    assert_close(got, ref, dtype, "other sizes")


# -- edges, with inputs made so that a fault shows ------------------------------------------------
def plain_attention(q, k, v, slopes, window, scale):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] of one sequence -> [T, H, dv], in 64-bit."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=torch.float64)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        for h in range(H):
            g = h // (H // G)
            s = (k[lo : i + 1, g].double() @ q[i, h].double()) * scale
            if slopes is not None:
                s = s - slopes[h] * torch.arange(i - lo, -1, -1, dtype=torch.float64)
            out[i, h] = torch.softmax(s, 0) @ v[lo : i + 1, g].double()
    return out


def paged_attention(q, k, v, slopes, window, scale, dtype, new_tokens, page_size=4, splits=1):
    """Run attention_general for the last ``new_tokens`` queries over keys laid out in
    shuffled pages (bfloat16 with sizes in sixteens: the tensor-core kernel, ``splits`` blocks
    sharing the keys)."""
    from forge_engine_b200.ops import native

    device = "cuda"
    T, H, dk = q.shape
    G, dv = k.shape[1], v.shape[2]
    pages = -(-T // page_size)
    order = torch.randperm(pages + 3, generator=torch.Generator().manual_seed(T))[:pages]
    k_cache = torch.zeros(pages + 3, G, page_size, dk, dtype=dtype, device=device)
    v_cache = torch.zeros(pages + 3, G, page_size, dv, dtype=dtype, device=device)
    for t in range(T):
        k_cache[order[t // page_size], :, t % page_size] = k[t].to(dtype).to(device)
        v_cache[order[t // page_size], :, t % page_size] = v[t].to(dtype).to(device)
    table = order.to(torch.int32).view(1, pages).to(device)
    first = T - new_tokens
    positions = torch.arange(first, T, dtype=torch.int32, device=device)
    entry = torch.zeros(new_tokens, dtype=torch.int32, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    qd = q[first:].to(dtype).to(device).contiguous()
    out = torch.empty(new_tokens, H, dv, dtype=dtype, device=device)
    sl = None if slopes is None else torch.tensor(slopes, dtype=torch.float32, device=device)
    cu_tokens = torch.tensor([0, new_tokens], dtype=torch.int32, device=device)
    starts = torch.tensor([first], dtype=torch.int32, device=device)
    native.attention_general(qd, (H * dk, dk), k_cache, dk, v_cache, dv, out, (H * dv, dv), table, positions, entry,
                             H, sl, window, scale, status, entries=(cu_tokens, starts, 1, new_tokens), splits=splits)
    assert int(status.item()) == 0
    return out.float().cpu()


@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16))
@pytest.mark.parametrize("new_tokens", (1, 0))
@pytest.mark.parametrize("window", (5, 8, 33))
def test_keys_just_inside_and_just_outside_a_window(window, new_tokens, dtype):
    """For every query two keys score far above the rest: the oldest one the window still
    holds and the one before it.  One key too many or too few changes the result by the
    size of the values.  In a prompt (all queries at once) and decoding (one query)."""
    gen = torch.Generator().manual_seed(window)
    T, H, G, dk, dv = 70, 4, 2, 16, 32
    q = 0.1 * torch.randn(T, H, dk, generator=gen)
    k = 0.1 * torch.randn(T, G, dk, generator=gen)
    v = torch.randn(T, G, dv, generator=gen)
    for i in range(T):
        # key j carries a mark in element j % dk that query j + window - 1 and j + window look for
        k[i, :, i % dk] = 4.0
    for i in range(T):
        q[i, :, (i - window + 1) % dk] = 6.0
        if window + 1 <= dk:
            q[i, :, (i - window) % dk] = 6.0
    q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))
    slopes = [2.0 ** (-8.0 * (h + 1) / H) for h in range(H)]
    ref = plain_attention(q, k, v, slopes, window, 0.5)
    count = new_tokens or T
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for splits in (1, 2) if new_tokens else (1,):
        got = paged_attention(q, k, v, slopes, window, 0.5, dtype, count, splits=splits)
        assert float((got - ref[T - count :]).abs().max()) <= tol, splits


@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16))
@pytest.mark.parametrize("new_tokens", (1, 0))
def test_a_key_far_back_among_hundreds(new_tokens, dtype):
    """No window: one early key (also one at a page's last place and one at a page's first)
    outscores hundreds of later ones, for queries far away."""
    gen = torch.Generator().manual_seed(1)
    T, H, G, dk, dv = 600, 2, 1, 32, 16
    q = 0.05 * torch.randn(T, H, dk, generator=gen)
    k = 0.05 * torch.randn(T, G, dk, generator=gen)
    v = torch.randn(T, G, dv, generator=gen)
    for mark, key in enumerate((2, 3, 4, 255)):
        k[key, 0, mark] = 5.0
    for i in range(300, T):
        q[i, :, i % 4] = 8.0
    q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))
    ref = plain_attention(q, k, v, None, None, 1.0)
    count = new_tokens or 200
    assert float((ref[-1, 0] - v[[2, 3, 4, 255][(T - 1) % 4], 0].double()).abs().max()) < 0.05   # the mark decides
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for splits in (1, 4, 8) if new_tokens else (1,):
        got = paged_attention(q, k, v, None, None, 1.0, dtype, count, splits=splits)
        assert float((got - ref[T - count :]).abs().max()) <= tol, splits


@pytest.mark.parametrize("dk, dv", ((48, 32), (320, 288)))
def test_tensor_core_attention_with_the_value_inside_the_key(dk, dv):
    """One cached vector that is key and value (its first elements), many heads on one kv head,
    queries and outputs with strides of their own; prompt portion and decoding, with splits.
    With more than 256 value columns two warp groups share a tile's columns."""
    from forge_engine_b200.ops import native

    gen = torch.Generator().manual_seed(9)
    T, H, page = 333, 6, 8
    q = torch.randn(T, H, dk, generator=gen).to(torch.bfloat16).float()
    kv = torch.randn(T, 1, dk, generator=gen).to(torch.bfloat16).float()
    scale = 0.2 * (48 / dk) ** 0.5
    ref = plain_attention(q, kv, kv[:, :, :dv], None, None, scale)
    device = "cuda"
    pages = -(-T // page)
    order = torch.randperm(pages + 2, generator=gen)[:pages]
    cache = torch.zeros(pages + 2, 1, page, dk, dtype=torch.bfloat16, device=device)
    for t in range(T):
        cache[order[t // page], 0, t % page] = kv[t, 0].to(torch.bfloat16).to(device)
    table = order.to(torch.int32).view(1, pages).to(device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    for count, splits in ((T, 1), (100, 1), (1, 1), (1, 4), (3, 2)):
        first = T - count
        positions = torch.arange(first, T, dtype=torch.int32, device=device)
        entry = torch.zeros(count, dtype=torch.int32, device=device)
        wide = torch.zeros(count, H, dk + 16, dtype=torch.bfloat16, device=device)       # rows wider than the query
        wide[:, :, :dk] = q[first:].to(torch.bfloat16).to(device)
        out = torch.zeros(count, H, dv + 8, dtype=torch.bfloat16, device=device)
        native.attention_general(wide, (H * (dk + 16), dk + 16), cache, dk, cache, dv, out, (H * (dv + 8), dv + 8), table,
                                 positions, entry, H, None, None, scale, status,
                                 entries=(torch.tensor([0, count], dtype=torch.int32, device=device),
                                          torch.tensor([first], dtype=torch.int32, device=device), 1, count),
                                 splits=splits)
        assert int(status.item()) == 0
        assert float((out[:, :, :dv].float().cpu() - ref[first:]).abs().max()) <= 2e-2, (count, splits)
        assert float(out[:, :, dv:].abs().max()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_far_token_decides_through_the_latent_cache(tmp_path, dtype):
    """A model of one latent-attention layer whose weights are arranged so that the logits of
    a late position depend on one early token: changing that token must change them as the
    plain implementation says, in a prompt and when decoding."""
    cfg = pz.config([pz.latent_layer(heads=2, dim=8, rot_dim=4, vdim=8, q_rank=16, kv_rank=16, ff=None)], width=32,
                    streams=None, residual_mult=1.0, scale=1.0)
    weights = write_model(tmp_path / "m", cfg, 17)
    base = tokens_of(cfg, 150, 8)
    other = list(base)
    other[2] = (base[2] + 1) % cfg["vocab"]
    runner = make_runner(tmp_path / "m", dtype, page_size=4, num_pages=80)
    for tokens in (base, other):
        ref = oracle(cfg, weights, tokens)
        got = run_schedule(runner, {"a": tokens}, [[("a", 140)]] + [[("a", 1)]] * 10)["a"]
        assert_close(got, ref, dtype, "far token")


def test_recurrence_state_is_carried_in_32_bit(tmp_path):
    """A decay close to one over many steps: what a state rounded to fewer bits would lose
    shows against the plain implementation."""
    from forge_engine_b200.ops import native

    gen = torch.Generator().manual_seed(4)
    T, H, dk, dv = 300, 2, 16, 40
    proj = torch.randn(T, 2 * H * dk + H * dv, generator=gen)
    decay = [0.9995, 0.5]
    act = torch.nn.functional.silu(proj.double())
    want = torch.zeros(T, H, dv, dtype=torch.float64)
    for h in range(H):
        state = torch.zeros(dk, dv, dtype=torch.float64)
        for t in range(T):
            kt = act[t, H * dk + h * dk : H * dk + (h + 1) * dk]
            vt = act[t, 2 * H * dk + h * dv : 2 * H * dk + (h + 1) * dv]
            state = decay[h] * state + torch.outer(kt, vt)
            want[t, h] = state.T @ act[t, h * dk : (h + 1) * dk]
    device = "cuda"
    # portions of up to 16 tokens are walked token by token, longer ones chunk-parallel
    for cuts in ([T], [1] * 40 + [T - 40], [7, 2, 100, 1, 1, 189], [16] * 18 + [12], [65, 64, 63, 108]):
        state = torch.zeros(3, H, dk, dv, dtype=torch.float32, device=device)
        out = torch.empty(T, H * dv, dtype=torch.float32, device=device)
        begin = 0
        for count in cuts:
            piece = proj[begin : begin + count].to(device).contiguous()
            part = torch.empty(count, H * dv, dtype=torch.float32, device=device)
            native.linear_recurrence(piece, 0, H * dk, 2 * H * dk, native.ACT_SILU, state,
                                     torch.tensor([1], dtype=torch.int32, device=device),
                                     torch.tensor([0, count], dtype=torch.int32, device=device),
                                     torch.tensor(decay, dtype=torch.float32, device=device), part, 1, count)
            out[begin : begin + count] = part
            begin += count
        assert float(state[0].abs().max()) == 0 and float(state[2].abs().max()) == 0
        error = float((out.cpu().double().view(T, H, dv) - want).abs().max() / want.abs().max())
        assert error < 2e-5, (cuts[:3], error)      # a state in 16 bits would be off by 1e-3 and more


# -- generation through the engine's own entry points ------------------------------------------------
def test_greedy_generation_through_engine_and_scheduler(tmp_path):
    from forge_engine_b200.config import EngineConfig, SchedulerConfig
    from forge_engine_b200.engine import Engine

    cfg = pz.config(MIXED)
    weights = write_model(tmp_path / "m", cfg, 18)
    prompts = [tokens_of(cfg, n, 20 + n) for n in (3, 26, 11, 1, 17)]
    engine = Engine.from_pretrained(
        tmp_path / "m",
        engine_config=EngineConfig(max_new_tokens=7, dtype="float32"),
        scheduler_config=SchedulerConfig(max_requests=3, max_batch_size=3, token_budget=12, block_size=4,
                                         block_capacity=48, chunk_size=8),
    )
    outputs = engine.generate(prompts)
    engine.runner.cache.check_consistency()
    assert engine.runner.cache.live_requests == 0
    for prompt, output in zip(prompts, outputs):
        assert len(output) == 7
        ids = list(prompt)
        for token in output:
            ref = oracle(cfg, weights, ids)[-1]
            top = torch.topk(ref, 2).values
            assert token == int(ref.argmax()) or float(top[0] - top[1]) < 1e-3
            ids.append(token)


def test_generate_command(tmp_path, capsys):
    from forge_engine_b200.cli import main

    cfg = pz.config([pz.lightning_layer(), pz.attention_layer(window=4), pz.latent_layer()])
    weights = write_model(tmp_path / "m", cfg, 19)
    prompt = tokens_of(cfg, 9, 1)
    code = main(["generate", "--model", str(tmp_path / "m"), "--prompt-ids", ",".join(map(str, prompt)),
                 "--max-new-tokens", "4", "--dtype", "float32", "--block-size", "4", "--block-capacity", "32"])
    assert code == 0
    printed = [int(t) for t in capsys.readouterr().out.strip().splitlines()[-1].split(",")]
    assert printed == pz.greedy_generate(cfg, weights, prompt, 4)


def test_random_weights_model_steps(tmp_path):
    """Seeded random weights for a configuration (what the benchmark uses): the model is
    assembled without a checkpoint and its steps give finite logits that do not depend on
    how the prompt was cut."""
    from forge_engine_b200.engine import ModelRunner

    cfg = pz.config(MIXED)
    runner = ModelRunner.from_random(cfg, 5, dtype="bfloat16", page_size=16, num_pages=16, max_requests=2, std=0.05)
    tokens = tokens_of(cfg, 40, 3)
    whole = run_schedule(runner, {"a": tokens}, [[("a", 40)]])["a"]
    cut = run_schedule(runner, {"b": tokens}, [[("b", 23)], [("b", 16)], [("b", 1)]])["b"]
    assert torch.isfinite(whole).all()
    assert float((whole - cut).abs().max()) <= 0.05 * max(1.0, float(whole.abs().max()))
