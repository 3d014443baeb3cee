"""The Tekilorn design in the engine against the plain implementation of ``plain_tekilorn.py``:
every mechanism alone, whole prompts against portions and token-by-token decoding, unequal
batches, reused pages and slots, edges of windows, kept first tokens and pages, other sizes,
generation."""

from __future__ import annotations

import json
import math

import pytest
import torch
from safetensors.torch import save_file

import plain_tekilorn as pt

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")


# -- helpers --------------------------------------------------------------------------------
def write_model(folder, cfg: dict, seed: int) -> dict:
    weights = pt.random_weights(cfg, seed)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
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
    return pt.forward(cfg, weights, tokens)


def mixed_config(dtype: str = "float32"):
    """All mechanisms in one model.  A router's close call, decided the other way by the
    rounding of a bfloat16 engine, changes a token's logits by half their size and those of
    the tokens after it by a tenth: the bfloat16 engine is compared on a model whose routed
    layers use every expert (each on its own score times the input), so that nothing rests on
    a close call; routers that choose are compared in 32-bit, and in bfloat16 where the
    margins are known (``test_routed_feed_forward_alone``)."""
    tops = (2, 1) if dtype == "float32" else (5, 5)
    return pt.config(
        [pt.differential_layer(), pt.window_layer(window=6, keep_first=2, mlp=pt.routed(top=tops[0], ff=32)),
         pt.window_layer(heads=2, kv_heads=1, dim=16, vdim=32, window=11, keep_first=5, rot_dims=16, mlp=pt.routed(top=tops[1])),
         pt.differential_layer(heads=2, kv_heads=2, dim=16, vdim=16, softcap=None, mlp=None)],
        loop=(1, 3, 2))


# -- every mechanism alone --------------------------------------------------------------------
SINGLE = {
    "differential": [pt.differential_layer()],
    "differential_plain_scores": [pt.differential_layer(softcap=None, q_temp=None)],
    "differential_no_ff": [pt.differential_layer(mlp=None)],
    "differential_capped_hard": [pt.differential_layer(softcap=1.5, scale=1.0)],
    "window_kept": [pt.window_layer()],
    "window_nothing_kept": [pt.window_layer(keep_first=0)],
    "window_none": [pt.window_layer(window=None)],
    "window_no_rotation": [pt.window_layer(rot_dims=0)],
    "window_whole_head_rotated": [pt.window_layer(rot_dims=16, vdim=32)],
    "window_odd_sizes": [pt.window_layer(heads=3, kv_heads=1, dim=12, vdim=20, rot_dims=6)],
    "routed_two_of_five": [pt.window_layer(mlp=pt.routed())],
    "routed_one_no_shared": [pt.window_layer(mlp=pt.routed(top=1, shared_ff=None))],
    "routed_all": [pt.differential_layer(mlp=pt.routed(experts=3, top=3, ff=20))],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone(tmp_path, name, dtype):
    cfg = pt.config(SINGLE[name])
    weights = write_model(tmp_path / "m", cfg, 3)
    tokens = tokens_of(cfg, 37, 5)
    runner = make_runner(tmp_path / "m", dtype)
    got = run_schedule(runner, {"a": tokens}, [[("a", 37)]])["a"]
    assert_close(got, oracle(cfg, weights, tokens), dtype, name)


@pytest.mark.parametrize("loop", ((0, 1, 3), (0, 2, 2), (1, 2, 1), (1, 1, 4), None))
def test_looped_layers(tmp_path, loop):
    """A stretch at the start, the whole model, one pass, an empty stretch, no loop."""
    cfg = pt.config([pt.window_layer(window=5, keep_first=1), pt.differential_layer(mlp=pt.routed(top=1))], loop=loop)
    weights = write_model(tmp_path / "m", cfg, 4)
    tokens = tokens_of(cfg, 29, 6)
    runner = make_runner(tmp_path / "m", "float32")
    got = run_schedule(runner, {"a": tokens}, [[("a", 17)], [("a", 2)]] + [[("a", 1)]] * 10)["a"]
    assert_close(got, oracle(cfg, weights, tokens), "float32", f"loop {loop}")


def test_residual_after_every_layer_run(tmp_path):
    """The residual stream after every layer run (a looped layer counts each time), in 32-bit."""
    from forge_engine_b200.engine import StepEntry

    cfg = mixed_config()
    weights = write_model(tmp_path / "m", cfg, 8)
    tokens = tokens_of(cfg, 19, 2)
    want: list = []
    pt.forward(cfg, weights, tokens, layers_out=want)
    runner = make_runner(tmp_path / "m", "float32", use_graphs=False)
    seen = []
    for block in runner.model.blocks:
        inner = block.forward

        def spy(h, pending, batch, cache, inner=inner, **extra):
            out = inner(h, pending, batch, cache, **extra)
            seen.append((h.clone() if out is None else h + out.float()).cpu())
            return out

        block.forward = spy
    runner.begin("a")
    runner.step([StepEntry("a", tokens, [0])])
    assert len(seen) == len(want) == 6
    for index, (got, ref) in enumerate(zip(seen, want)):
        assert_close(got, ref, "float32", f"layer run {index}")


# -- whole prompts, portions, single tokens -----------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_prefill_against_token_by_token_decoding(tmp_path, dtype):
    cfg = mixed_config(dtype)
    weights = write_model(tmp_path / "m", cfg, 11)
    tokens = tokens_of(cfg, 45, 7)
    ref = oracle(cfg, weights, tokens)
    runner = make_runner(tmp_path / "m", dtype, num_pages=160)
    whole = run_schedule(runner, {"a": tokens}, [[("a", 45)]])["a"]
    single = run_schedule(runner, {"b": tokens}, [[("b", 1)] for _ in range(45)])["b"]
    assert_close(whole, ref, dtype, "whole prompt")
    assert_close(single, ref, dtype, "token by token")
    if dtype == "float32":
        assert float((whole - single).abs().max()) <= 2e-5 * float(ref.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_portions_of_several_sizes(tmp_path, dtype):
    cfg = mixed_config(dtype)
    weights = write_model(tmp_path / "m", cfg, 12)
    tokens = tokens_of(cfg, 101, 9)
    ref = oracle(cfg, weights, tokens)
    runner = make_runner(tmp_path / "m", dtype, num_pages=200)
    for sizes in ([2, 3, 5, 2, 17, 16, 1, 1, 33, 4, 2, 15], [2] * 20 + [61], [64, 2, 35], [7] * 14 + [3]):
        assert sum(sizes) == 101
        got = run_schedule(runner, {"a": tokens}, [[("a", n)] for n in sizes])["a"]
        assert_close(got, ref, dtype, f"portions {sizes[:4]}...")


@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_requests_in_one_batch_against_each_alone(tmp_path, dtype):
    cfg = mixed_config(dtype)
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
    runner = make_runner(tmp_path / "m", dtype, num_pages=200)
    together = run_schedule(runner, requests, schedule)
    for key, tokens in requests.items():
        assert_close(together[key], oracle(cfg, weights, tokens), dtype, f"request {key} in the batch")
        alone = run_schedule(runner, {key + "'": tokens}, [[(key + "'", len(tokens))]])[key + "'"]
        if dtype == "float32":
            assert float((together[key] - alone).abs().max()) <= 2e-5 * float(alone.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_pages_and_slots_freed_and_used_again(tmp_path, dtype):
    """Two slots and a pool that holds two requests at most: later requests get the pages of
    earlier ones, also the pages that held an earlier request's kept first tokens."""
    cfg = pt.config([pt.window_layer(window=5, keep_first=6),
                     pt.differential_layer(mlp=pt.routed(top=2 if dtype == "float32" else 5)),
                     pt.window_layer(window=9, keep_first=1, mlp=None)])
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
    """A short prompt, then far more single tokens than any window or page holds: the pages a
    window has passed go back to the pool, those of the kept first tokens stay.  The decode
    steps are replayed from captured graphs."""
    cfg = pt.config([pt.window_layer(window=8, keep_first=5), pt.differential_layer(q_temp=(0.7, 16)),
                     pt.window_layer(window=3, keep_first=1, mlp=pt.routed(top=2 if dtype == "float32" else 5))],
                    loop=(0, 1, 2))
    weights = write_model(tmp_path / "m", cfg, 15)
    tokens = tokens_of(cfg, 90, 4)
    runner = make_runner(tmp_path / "m", dtype, page_size=4, num_pages=30)
    got = run_schedule(runner, {"a": tokens}, [[("a", 5)]] + [[("a", 1)] for _ in range(85)])["a"]
    assert_close(got, oracle(cfg, weights, tokens), dtype, "long decoding")
    if runner.use_graphs:
        assert runner.graphs.captured


@pytest.mark.parametrize("dtype", DTYPES)
def test_other_sizes_and_values_that_are_one_or_equal(tmp_path, dtype):
    """Sizes that are no powers of two or multiples of sixteen, heads = kv heads, one kv head,
    one head, a window of one, more kept tokens than a window or a page holds, keys as wide as
    values, one expert of one, every expert chosen, a loop of one pass."""
    layers = [
        pt.window_layer(heads=1, kv_heads=1, dim=24, vdim=40, window=1, keep_first=1, rot_dims=24, mlp=pt.dense(40, 0.5)),
        pt.differential_layer(heads=3, kv_heads=3, dim=8, vdim=8, diff=0.6, q_temp=(1.0, 1), mlp=pt.routed(1, 1, 16, 3.0, None)),
        pt.window_layer(heads=5, kv_heads=1, dim=8, vdim=8, window=4, keep_first=11, rot_dims=2, mlp=pt.routed(4, 4, 8, 1.0, 8, 1.0)),
        pt.differential_layer(heads=6, kv_heads=2, dim=16, vdim=48, softcap=5.0, q_temp=None, mlp=None),
        pt.window_layer(heads=2, kv_heads=2, dim=20, vdim=12, window=12, keep_first=0, rot_dims=10, mlp=pt.dense(24, 9.0)),
    ]
    cfg = pt.config(layers, width=72, vocab=50, eps=1e-3, loop=(2, 4, 1))
    weights = write_model(tmp_path / "m", cfg, 16)
    tokens = tokens_of(cfg, 40, 6)
    ref = oracle(cfg, weights, tokens)
    runner = make_runner(tmp_path / "m", dtype, page_size=8, num_pages=48)
    got = run_schedule(runner, {"a": tokens}, [[("a", 13)], [("a", 2)], [("a", 20)]] + [[("a", 1)]] * 5)["a"]
    assert_close(got, ref, dtype, "other sizes")


# -- kernels alone, with inputs made so that a fault shows ------------------------------------------
def plain_scores_attention(q, k, v, scale, window=None, keep_first=0, softcap=None, temp=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] of one sequence -> [T, H, dv], in 64-bit, one
    query at a time."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=torch.float64)
    for i in range(T):
        keys = [j for j in range(i + 1) if window is None or i - j < window or j < keep_first]
        factor = 1.0 if temp is None else 1.0 + temp[0] * math.log((i + 1) // temp[1] + 1)
        for h in range(H):
            g = h // (H // G)
            s = (k[keys, g].double() @ q[i, h].double()) * scale * factor
            if softcap is not None:
                s = softcap * torch.tanh(s / softcap)
            out[i, h] = torch.softmax(s, 0) @ v[keys, g].double()
    return out


def paged_attention(q, k, v, scale, dtype, new_tokens, page_size=4, splits=1, gate=None, parts=1, hole=None, **options):
    """Run attention_general for the last ``new_tokens`` queries over keys laid out in
    shuffled pages (bfloat16 with sizes in sixteens: the tensor-core kernel, ``splits`` blocks
    sharing the keys).  ``parts`` > 1: q [T, H, parts, d], k [T, G, parts, d]; the output holds
    the maps side by side in 32-bit.  ``hole``: logical pages whose table entry is -1."""
    from forge_engine_b200.ops import native

    device = "cuda"
    T, H = q.shape[:2]
    G, dv = k.shape[1], v.shape[2]
    dk = q.shape[-1]
    pages = -(-T // page_size)
    order = torch.randperm(pages + 3, generator=torch.Generator().manual_seed(T))[:pages]
    k_cache = torch.zeros(pages + 3, G, page_size, parts * dk, dtype=dtype, device=device)
    v_cache = torch.zeros(pages + 3, G, page_size, dv, dtype=dtype, device=device)
    for t in range(T):
        k_cache[order[t // page_size], :, t % page_size] = k[t].reshape(G, parts * dk).to(dtype).to(device)
        v_cache[order[t // page_size], :, t % page_size] = v[t].to(dtype).to(device)
    table = order.to(torch.int32).view(1, pages).clone()
    for page in hole or ():
        k_cache[table[0, page]] = float("nan")     # a page that was given back holds anything
        table[0, page] = -1
    table = table.to(device)
    first = T - new_tokens
    positions = torch.arange(first, T, dtype=torch.int32, device=device)
    entry = torch.zeros(new_tokens, dtype=torch.int32, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    qd = q[first:].reshape(new_tokens, H * parts * dk).to(dtype).to(device).contiguous()
    out = torch.empty(new_tokens, H, parts, dv, dtype=dtype if parts == 1 else torch.float32, device=device)
    cu_tokens = torch.tensor([0, new_tokens], dtype=torch.int32, device=device)
    starts = torch.tensor([first], dtype=torch.int32, device=device)
    gates = None if gate is None else gate[first:].float().to(device).contiguous()
    native.attention_general(qd, (H * parts * dk, parts * dk), k_cache, dk, v_cache, dv, out, (H * parts * dv, parts * dv),
                             table, positions, entry, H, None, options.pop("window", None), scale, status,
                             entries=(cu_tokens, starts, 1, new_tokens), splits=splits, gate=gates, parts=parts,
                             part_strides=(dk, dk, dv) if parts > 1 else (0, 0, 0), **options)
    assert int(status.item()) == 0
    out = out.float().cpu()
    return out[:, :, 0] if parts == 1 else out


@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16))
@pytest.mark.parametrize("new_tokens", (1, 0))
@pytest.mark.parametrize("window, keep_first", ((5, 3), (8, 1), (33, 6), (4, 9), (70, 2)))
def test_keys_at_the_edges_of_the_window_and_of_the_kept_tokens(window, keep_first, new_tokens, dtype):
    """For every query four keys score far above the rest: the oldest one the window still
    holds, the one before it, the last kept token and the one after it.  One key too many or
    too few changes the result by the size of the values.  In a prompt (all queries at once) and
    decoding (one query, also with the keys split over blocks); the pages between the kept
    tokens and the window are missing from the table, as after a release."""
    gen = torch.Generator().manual_seed(window)
    T, H, G, dk, dv, page = 70, 4, 2, 16, 32, 4
    q = 0.1 * torch.randn(T, H, dk, generator=gen)
    k = 0.1 * torch.randn(T, G, dk, generator=gen)
    v = torch.randn(T, G, dv, generator=gen)
    for i in range(T):
        k[i, :, i % dk] = 4.0          # key j carries a mark in element j % dk
    for i in range(T):
        for key in (i - window + 1, i - window, keep_first - 1, keep_first):
            q[i, :, key % dk] = 6.0    # (keys with the same mark sixteen places on are as loud, where visible)
    q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))
    ref = plain_scores_attention(q, k, v, 0.5, window, keep_first)
    count = new_tokens or T
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    hole = None
    if new_tokens:      # decoding at the end: pages wholly between the kept tokens and the window are gone
        hole = range(-(-keep_first // page), max(-(-keep_first // page), (T - 1 - window + 1) // page))
    for splits in (1, 2, 4) if new_tokens else (1,):
        got = paged_attention(q, k, v, 0.5, dtype, count, page_size=page, splits=splits, window=window,
                              keep_first=keep_first, hole=hole)
        assert float((got - ref[T - count :]).abs().max()) <= tol, splits


@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16))
@pytest.mark.parametrize("new_tokens", (1, 0))
def test_a_kept_token_far_back_among_hundreds(new_tokens, dtype):
    """A window of 40 over 600 tokens: kept tokens 1 and 2 outscore everything in the window for
    queries hundreds of positions later; token 3, just as loud, is not kept and must not be seen."""
    gen = torch.Generator().manual_seed(1)
    T, H, G, dk, dv = 600, 2, 1, 32, 16
    q = 0.05 * torch.randn(T, H, dk, generator=gen)
    k = 0.05 * torch.randn(T, G, dk, generator=gen)
    v = torch.randn(T, G, dv, generator=gen)
    for mark, key in enumerate((1, 2, 3)):
        k[key, 0, mark] = 5.0
    for i in range(300, T):
        q[i, :, i % 3] = 8.0
    q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))
    ref = plain_scores_attention(q, k, v, 1.0, 40, 3)
    assert float((ref[-2, 0] - v[[1, 2, 3][(T - 2) % 3], 0].double()).abs().max()) < 0.05     # the mark decides
    count = new_tokens or 200
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for splits in (1, 2) if new_tokens else (1,):
        got = paged_attention(q, k, v, 1.0, dtype, count, splits=splits, window=40, keep_first=3)
        assert float((got - ref[T - count :]).abs().max()) <= tol, splits


@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16))
@pytest.mark.parametrize("new_tokens", (1, 0))
def test_capped_scores_and_query_temperature(new_tokens, dtype):
    """Scores far beyond the cap, so that the softmax is decided by the cap alone, and a
    temperature whose steps (every 7 positions) fall inside the prompt and at its end."""
    gen = torch.Generator().manual_seed(2)
    T, H, G, dk, dv = 150, 4, 2, 16, 16
    q = torch.randn(T, H, dk, generator=gen)
    k = torch.randn(T, G, dk, generator=gen)
    v = torch.randn(T, G, dv, generator=gen)
    q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))
    for options in (dict(softcap=2.0), dict(query_temperature=(0.9, 7)), dict(softcap=6.0, query_temperature=(0.5, 50))):
        ref = plain_scores_attention(q, k, v, 0.8, None, 0, options.get("softcap"), options.get("query_temperature"))
        plain = plain_scores_attention(q, k, v, 0.8)
        assert float((ref - plain).abs().max()) > 0.1          # the option matters
        count = new_tokens or T
        tol = 3e-5 if dtype == torch.float32 else 3e-2
        for splits in (1, 2) if new_tokens else (1,):
            got = paged_attention(q, k, v, 0.8, dtype, count, splits=splits, **options)
            assert float((got - ref[T - count :]).abs().max()) <= tol, (options, splits)


@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16))
@pytest.mark.parametrize("new_tokens", (1, 0))
def test_two_maps_per_head_and_gates(new_tokens, dtype):
    """Two score maps per head over shared values, left side by side in 32-bit, and a
    sigmoid gate per (token, head)."""
    gen = torch.Generator().manual_seed(3)
    T, H, G, dk, dv = 90, 4, 2, 16, 32
    q = torch.randn(T, H, 2, dk, generator=gen)
    k = torch.randn(T, G, 2, dk, generator=gen)
    v = torch.randn(T, G, dv, generator=gen)
    gate = 2.0 * torch.randn(T, H, generator=gen)
    q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))
    count = new_tokens or T
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    for splits in (1, 2) if new_tokens else (1,):
        got = paged_attention(q, k, v, 0.3, dtype, count, splits=splits, parts=2)
        for part in range(2):
            ref = plain_scores_attention(q[:, :, part], k[:, :, part], v, 0.3)
            assert float((got[:, :, part] - ref[T - count :]).abs().max()) <= tol, (part, splits)
        gated = paged_attention(q[:, :, 0], k[:, :, 0], v, 0.3, dtype, count, splits=splits, gate=gate)
        ref = plain_scores_attention(q[:, :, 0], k[:, :, 0], v, 0.3) * torch.sigmoid(gate.double())[:, :, None]
        assert float((gated - ref[T - count :]).abs().max()) <= tol, splits


@pytest.mark.parametrize("dim", (64, 128))
@pytest.mark.parametrize("window, keep_first", ((None, 0), (40, 0), (40, 5), (200, 3), (130, 129), (7, 300)))
def test_prompt_portions_on_the_tcgen05_kernel(window, keep_first, dim):
    """Plain softmax layers with heads of 64 or 128 send prompt portions to the tcgen05 prefill
    kernel: window edges, kept first tokens (fewer and more than a key tile of 128 holds, pages
    between them and the window missing from the table), a gate per head; a whole prompt and a
    portion that starts in the middle of a page and of a key tile, beside a second entry."""
    from forge_engine_b200.ops import native

    gen = torch.Generator().manual_seed(dim + (window or 0))
    T, H, G, page = 420, 4, 2, 4
    q = 0.1 * torch.randn(T, H, dim, generator=gen)
    k = 0.1 * torch.randn(T, G, dim, generator=gen)
    v = torch.randn(T, G, dim, generator=gen)
    gate = 2.0 * torch.randn(T, H, generator=gen)
    for i in range(T):
        k[i, :, i % dim] = 4.0
    if window is not None:
        for i in range(T):
            for key in (i - window + 1, i - window, keep_first - 1, keep_first):
                q[i, :, key % dim] = 6.0
    q, k, v = (t.to(torch.bfloat16).float() for t in (q, k, v))
    ref = plain_scores_attention(q, k, v, 0.5, window, keep_first) * torch.sigmoid(gate.double())[:, :, None]
    device = "cuda"
    pages = -(-T // page)
    order = torch.randperm(pages + 5, generator=gen)[:pages]
    k_cache = torch.zeros(pages + 5, G, page, dim, dtype=torch.bfloat16, device=device)
    v_cache = torch.zeros_like(k_cache)
    for t in range(T):
        k_cache[order[t // page], :, t % page] = k[t].to(torch.bfloat16).to(device)
        v_cache[order[t // page], :, t % page] = v[t].to(torch.bfloat16).to(device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    for first in (0, 203):
        count = T - first
        # a second entry of three tokens (too few rows for this kernel) comes first in the batch
        table = torch.full((2, pages), -1, dtype=torch.int32)
        table[1] = order.to(torch.int32)
        if window is not None and first:
            kept = -(-min(keep_first, T) // page)
            table[1, kept : max(kept, (first - window + 1) // page)] = -1      # given back before this step
        table[0, 0] = int(order[0])
        qd = torch.zeros(3 + count, H * dim, dtype=torch.bfloat16, device=device)
        qd[3:] = q[first:].reshape(count, H * dim).to(torch.bfloat16).to(device)
        gates = torch.zeros(3 + count, H + 3, dtype=torch.float32, device=device)[:, :H]     # rows wider than the gates
        gates[3:] = gate[first:].to(device)
        out = torch.zeros(3 + count, H * dim, dtype=torch.bfloat16, device=device)
        native.attention_prefill_tc5(qd, k_cache, v_cache, out, table.to(device),
                                     torch.tensor([0, 3, 3 + count], dtype=torch.int32, device=device),
                                     torch.tensor([0, first], dtype=torch.int32, device=device), 2, count, H, window,
                                     keep_first, 0.5, gates, 16, status)
        assert int(status.item()) == 0
        got = out[3:].float().cpu().view(count, H, dim)
        assert float((got - ref[first:]).abs().max()) <= 3e-2, first
        assert float(out[:3].abs().max()) == 0          # the short entry is left to the other kernel


def test_plain_layers_with_heads_of_64_in_a_model(tmp_path):
    """A model whose window layers have heads of 64: prompt portions run on the tcgen05 kernel,
    short portions and single tokens on the general one, in one step where both occur."""
    cfg = pt.config([pt.window_layer(heads=4, kv_heads=2, dim=64, vdim=64, window=70, keep_first=3, rot_dims=32),
                     pt.window_layer(heads=2, kv_heads=2, dim=64, vdim=64, window=None, rot_dims=64, mlp=None)], width=64)
    weights = write_model(tmp_path / "m", cfg, 23)
    requests = {"a": tokens_of(cfg, 300, 1), "b": tokens_of(cfg, 41, 2), "c": tokens_of(cfg, 170, 3)}
    schedule = [[("a", 200)], [("a", 1), ("b", 30), ("c", 2)], [("a", 60), ("b", 1), ("c", 100)],
                [("a", 39), ("b", 10), ("c", 68)]]
    for dtype in DTYPES:
        runner = make_runner(tmp_path / "m", dtype, page_size=16, num_pages=48)
        block = runner.model.blocks[0]
        assert block.mixer._prefill_tc5(16) == (dtype == "bfloat16")
        got = run_schedule(runner, requests, schedule)
        for key, tokens in requests.items():
            assert_close(got[key], oracle(cfg, weights, tokens), dtype, f"request {key}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixed_steps_replayed_from_graphs(tmp_path, dtype):
    """Steps that bring a prompt portion beside two decoding requests, captured at first sight
    and replayed (filler entries pad them to their bucket): the tcgen05 prefill kernel for the
    portion, the general kernel for the single tokens, a routed layer, looped layers, kept
    pages.  Logits at every entry's last token against the plain implementation."""
    from forge_engine_b200.engine import StepEntry

    top = 2 if dtype == "float32" else 5
    cfg = pt.config([pt.window_layer(heads=4, kv_heads=2, dim=64, vdim=64, window=70, keep_first=3, rot_dims=32,
                                     mlp=pt.routed(top=top, ff=32)),
                     pt.differential_layer(mlp=None),
                     pt.window_layer(heads=2, kv_heads=2, dim=128, vdim=128, window=150, keep_first=20, rot_dims=64)],
                    width=64, loop=(0, 2, 2))
    weights = write_model(tmp_path / "m", cfg, 31)
    requests = {"a": tokens_of(cfg, 64 * 12 + 5, 1), "b": tokens_of(cfg, 22, 2), "c": tokens_of(cfg, 27, 3)}
    schedule = [[("b", 9), ("c", 14)]] + [[("a", 64), ("b", 1), ("c", 1)] for _ in range(12)] + [[("a", 5), ("b", 1), ("c", 1)]]
    runner = make_runner(tmp_path / "m", dtype, page_size=16, num_pages=80)
    runner.graphs.capture_after = 1
    refs = {key: oracle(cfg, weights, tokens).float() for key, tokens in requests.items()}
    at = {key: 0 for key in requests}
    for step in schedule:
        entries = []
        for key, count in step:
            if at[key] == 0:
                runner.begin(key)
            entries.append(StepEntry(key, requests[key][at[key] : at[key] + count], [count - 1]))
        logits = runner.step(entries).float().cpu()
        runner.check_status()
        for row, (key, count) in enumerate(step):
            at[key] += count
            assert_close(logits[row : row + 1], refs[key][at[key] - 1 : at[key]], dtype, f"{key} at {at[key] - 1}")
    assert len(runner.graphs.captured) >= 2


def test_differential_combine():
    from forge_engine_b200.ops import native

    gen = torch.Generator().manual_seed(5)
    rows, dv, lam, eps, offset = 77, 24, 0.61, 1e-3, 0.3
    maps = torch.randn(rows, 2, dv, generator=gen)
    maps[:, 1] = maps[:, 0] / lam + 1e-3 * torch.randn(rows, dv, generator=gen)      # the difference is small
    o = maps[:, 0].double() - lam * maps[:, 1].double()
    want = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * (1.0 - offset)
    for dtype, tol in ((torch.float32, 2e-3), (torch.bfloat16, 2e-2)):
        out = torch.empty(rows, dv, dtype=dtype, device="cuda")
        native.differential_combine(maps.cuda().view(rows, 2 * dv), out, dv, lam, eps, 1.0 - offset)
        assert float((out.float().cpu() - want).abs().max()) <= tol * float(want.abs().max())


@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16))
@pytest.mark.parametrize("experts, top, tokens, ff", ((7, 2, 150, 32), (3, 3, 5, 24), (40, 1, 33, 16), (6, 4, 1, 48),
                                                      (4, 2, 700, 64), (5, 1, 300, 40)))
def test_routed_feed_forward_alone(experts, top, tokens, ff, dtype):
    """The part alone against a loop over tokens and experts: the chosen experts, weights on
    the input, the shared unit with its gate; tokens whose router margin is not clear are left
    out.  Widths in sixteens run the grouped tensor-core products in bfloat16 (few and many rows
    per expert: narrow and wide row tiles), others the plain grouped kernels."""
    from forge_engine_b200.config.specs import GatedMLPSpec, RoutedMLPSpec
    from forge_engine_b200.parts.base import BuildContext, build_part

    gen = torch.Generator().manual_seed(experts)
    width, limit = 40, 1.0
    cfg = pt.config([pt.window_layer(mlp=pt.routed(experts, top, ff, limit, 16, 2.0))], width=width)
    weights = {name[len("l0.mlp."):]: t for name, t in pt.random_weights(cfg, 7).items() if name.startswith("l0.mlp.")}
    x = torch.randn(tokens, width, generator=gen).to(torch.bfloat16)
    # distinct router scores: every expert's row looks for its own mix of the first elements
    weights["router"] = (3.0 * torch.randn(experts, width, generator=gen) / math.sqrt(width)).to(torch.bfloat16)
    want = pt.routed_feed_forward(x.double(), {"l0.mlp." + k: v.double() for k, v in weights.items()}, "l0.mlp.",
                                  cfg["layers"][0]["mlp"])
    scores = torch.sigmoid(x.double() @ weights["router"].double().T).sort(dim=-1, descending=True).values
    clear = (scores[:, top - 1] - scores[:, top]) > 1e-3 if top < experts else torch.ones(tokens, dtype=torch.bool)
    unit = dict(rename=(("gate_proj.weight", "gate"), ("up_proj.weight", "up"), ("down_proj.weight", "down")), slope=1.702)
    spec = RoutedMLPSpec(width, experts, top, GatedMLPSpec(width, ff, "clamped_swish", limit=limit, **unit),
                         shared=GatedMLPSpec(width, 16, "clamped_swish", limit=2.0, **unit), shared_gate=True)
    engine_dtype = dtype
    ctx = BuildContext(dtype=engine_dtype, device=torch.device("cuda"), status=torch.zeros(1, dtype=torch.int32, device="cuda"))
    part = build_part(spec, {k: v.to(engine_dtype).cuda() for k, v in weights.items()}, ctx)
    assert part.fused == (dtype == torch.bfloat16 and ff % 16 == 0)
    got = part.forward(x.to(engine_dtype).cuda()).float().cpu()
    assert int(ctx.status.item()) == 0
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert float((got[clear] - want[clear]).abs().max()) <= tol * max(1.0, float(want.abs().max()))
    assert int(part.counts.abs().sum()) == 0       # left zero for the next call


@pytest.mark.parametrize("dtype", DTYPES)
def test_far_token_decides_through_kept_pages(tmp_path, dtype):
    """A model whose only mixer keeps two first tokens behind a window of two: changing token 1
    must change late logits as the plain implementation says, in a prompt and when decoding,
    long after the window's pages have gone back to the pool."""
    cfg = pt.config([pt.window_layer(heads=2, kv_heads=1, dim=16, vdim=16, window=2, keep_first=2, rot_dims=4, mlp=None)],
                    width=32)
    weights = write_model(tmp_path / "m", cfg, 17)
    base = tokens_of(cfg, 150, 8)
    other = list(base)
    other[1] = (base[1] + 1) % cfg["vocab"]
    runner = make_runner(tmp_path / "m", dtype, page_size=4, num_pages=44)
    refs = []
    for tokens in (base, other):
        ref = oracle(cfg, weights, tokens)
        refs.append(ref)
        got = run_schedule(runner, {"a": tokens}, [[("a", 140)]] + [[("a", 1)]] * 10)["a"]
        assert_close(got, ref, dtype, "far token")
        assert max(runner.cache.leased_pages()) == 0
    late = slice(140, 150)       # the kept token matters to the decoded positions, far beyond any tolerance
    assert float(((refs[0][late] - refs[1][late]) ** 2).mean().sqrt() / (refs[0][late] ** 2).mean().sqrt()) > 0.1


# -- generation through the engine's own entry points ------------------------------------------------
def test_greedy_generation_through_engine_and_scheduler(tmp_path):
    from forge_engine_b200.config import EngineConfig, SchedulerConfig
    from forge_engine_b200.engine import Engine

    cfg = mixed_config()
    weights = write_model(tmp_path / "m", cfg, 18)
    prompts = [tokens_of(cfg, n, 20 + n) for n in (3, 26, 11, 1, 17)]
    engine = Engine.from_pretrained(
        tmp_path / "m",
        engine_config=EngineConfig(max_new_tokens=7, dtype="float32"),
        scheduler_config=SchedulerConfig(max_requests=3, max_batch_size=3, token_budget=12, block_size=4,
                                         block_capacity=96, chunk_size=8),
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

    cfg = pt.config([pt.differential_layer(), pt.window_layer(window=4, keep_first=1, mlp=pt.routed())], loop=(1, 2, 2))
    weights = write_model(tmp_path / "m", cfg, 19)
    prompt = tokens_of(cfg, 9, 1)
    code = main(["generate", "--model", str(tmp_path / "m"), "--prompt-ids", ",".join(map(str, prompt)),
                 "--max-new-tokens", "4", "--dtype", "float32", "--block-size", "4", "--block-capacity", "32"])
    assert code == 0
    printed = [int(t) for t in capsys.readouterr().out.strip().splitlines()[-1].split(",")]
    assert printed == pt.greedy_generate(cfg, weights, prompt, 4)


def test_random_weights_model_steps():
    """Seeded random weights for a configuration (what the benchmark uses): the model is
    assembled without a checkpoint and its steps give finite logits that do not depend on
    how the prompt was cut."""
    from forge_engine_b200.engine import ModelRunner

    cfg = mixed_config()
    runner = ModelRunner.from_random(cfg, 5, dtype="bfloat16", page_size=16, num_pages=32, max_requests=2, std=0.05)
    tokens = tokens_of(cfg, 40, 3)
    whole = run_schedule(runner, {"a": tokens}, [[("a", 40)]])["a"]
    cut = run_schedule(runner, {"b": tokens}, [[("b", 23)], [("b", 16)], [("b", 1)]])["b"]
    assert torch.isfinite(whole).all()
    assert float((whole - cut).abs().max()) <= 0.05 * max(1.0, float(whole.abs().max()))
