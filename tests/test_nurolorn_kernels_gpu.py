"""The kernels of the Nurolorn parts, each against its plain torch statement (tests/plain_ops.py), at odd sizes, and
attention with inputs built so that one key decides the result: a key hundreds of tokens back, keys on both sides of
a page border, keys just inside and just outside the window, in prompt portions and in decoding."""

from __future__ import annotations

from types import SimpleNamespace

import pytest
import torch

import plain_ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from llmserve_triton_kernels_b200 import ops

    return ops


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def close(a, b, dtype, what=""):
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    scale = float(b.float().abs().max().clamp_min(1e-6))
    err = float((a.float() - b.float()).abs().max())
    assert err <= tol * scale, f"{what}: max |diff| {err:.3e} against scale {scale:.3e}"


def make_ctx(query_lens, context_lens, page_size, num_pages, seed=0):
    """A step's arrays for requests that bring ``query_lens`` tokens and hold ``context_lens`` after it, with the
    pages of each request drawn at random from the pool."""
    g = torch.Generator().manual_seed(seed)
    R = len(query_lens)
    cu = [0]
    for n in query_lens:
        cu.append(cu[-1] + n)
    width = max(-(-c // page_size) for c in context_lens)
    perm = torch.randperm(num_pages, generator=g).tolist()
    table = torch.zeros((R, width), dtype=torch.int32)
    slot_map, positions, owner = [], [], []
    for r, (q, c) in enumerate(zip(query_lens, context_lens)):
        pages = [perm.pop() for _ in range(-(-c // page_size))]
        table[r, : len(pages)] = torch.tensor(pages, dtype=torch.int32)
        for p in range(c - q, c):
            slot_map.append(pages[p // page_size] * page_size + p % page_size)
            positions.append(p)
            owner.append(r)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    ctx = SimpleNamespace(
        num_tokens=cu[-1], num_requests=R, token_request=i32(owner), cu_tokens=i32(cu), context_lens=i32(context_lens),
        positions=i32(positions), max_query_len=max(query_lens), max_context_len=max(context_lens), host_cu_tokens=cu,
    )
    return ctx, table.to(DEV), i32(slot_map)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,groups", [(60, 5), (64, 1), (256, 2), (36, 3), (1024, 4)])
def test_grouped_norm_with_scaled_sum(ops, hidden, groups, dtype):
    n = 7
    resid, delta, w = rnd(n, hidden), rnd(n, hidden, dtype=dtype, seed=1), 1 + rnd(hidden, seed=2, scale=0.1)
    a, b = resid.clone(), resid.clone()
    got = ops.group_rmsnorm(a, w, 1e-5, groups, delta=delta, alpha=0.7, out_dtype=dtype)
    want = plain_ops.group_rmsnorm(b, w, 1e-5, groups, delta=delta, alpha=0.7, out_dtype=dtype)
    close(got, want, dtype, "normalised")
    close(a, b, torch.float32, "stream written back")
    rows = torch.tensor([5, 0, 3], dtype=torch.int32, device=DEV)
    kept = a.clone()
    close(ops.group_rmsnorm(a, w, 1e-5, groups, delta=delta, alpha=0.7, rows=rows, out_dtype=dtype),
          plain_ops.group_rmsnorm(b, w, 1e-5, groups, delta=delta, alpha=0.7, rows=rows, out_dtype=dtype), dtype, "chosen rows")
    assert torch.equal(a, kept), "with chosen rows the stream stays as it was"
    close(ops.group_rmsnorm(a, w, 1e-5, groups, out_dtype=dtype), plain_ops.group_rmsnorm(b, w, 1e-5, groups, out_dtype=dtype), dtype, "no sum")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_stream_inject_activations_and_gates(ops, dtype):
    n, hidden, vocab = 9, 52, 30
    resid, delta, table, vec = rnd(n, hidden), rnd(n, hidden, dtype=dtype, seed=1), rnd(vocab, hidden, dtype=dtype, seed=2), rnd(hidden, seed=3)
    ids = torch.randint(0, vocab, (n,), dtype=torch.int32, device=DEV)
    for args in ((delta, 0.6, ids, table, vec), (None, 1.0, None, None, vec), (delta, 0.6, ids, table, None), (delta, 1.0, None, None, None)):
        a, b = resid.clone(), resid.clone()
        ops.stream_inject(a, *args)
        plain_ops.stream_inject(b, *args)
        close(a, b, torch.float32, "stream after injection")
    x = rnd(n, 70, dtype=dtype, seed=4, scale=2.0)
    for kind in ("relu2", "gelu_tanh", "silu", "scale"):
        close(ops.unary(x, kind, 1.7), plain_ops.unary(x, kind, 1.7), dtype, kind)
    view = x[:, 3:61]  # a row pitch
    close(ops.unary(view, "relu2"), plain_ops.unary(view, "relu2"), dtype, "relu2 with a pitch")
    heads, w = 3, 10
    a = rnd(heads, n, w, dtype=dtype, seed=5).transpose(0, 1)  # head by head in memory
    gate = rnd(n, heads * w + 4, dtype=dtype, seed=6)[:, 4:]
    for kind in ("sigmoid", "silu"):
        close(ops.gate_mul(a, gate, kind), plain_ops.gate_mul(a, gate, kind), dtype, f"gate {kind}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_linear(ops, dtype):
    n, heads, k, m = 19, 3, 24, 40
    rows = rnd(n, heads * (k + 8), dtype=dtype, scale=0.5)
    x = rows.as_strided((n, heads, k), (rows.stride(0), k + 8, 1))
    w = rnd(heads, m, k, dtype=dtype, seed=1, scale=0.3)
    close(ops.head_linear(x, w), plain_ops.head_linear(x, w), dtype, "one product per head")


@pytest.mark.parametrize("lens", [[1, 13, 2, 30], [1, 200, 65, 3], [777, 1, 1, 1]])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_mingru_scan_carries_the_state_of_each_slot(ops, out_dtype, lens):
    """Short requests (a thread walks a channel) and long ones (the warps of a CTA share a request's tokens)."""
    width = 45
    ctx, _, _ = make_ctx(lens, lens, 4, 400)
    slots = torch.tensor([2, 0, 5, 3], dtype=torch.int32, device=DEV)
    bz, bu = rnd(width, seed=1), rnd(width, seed=2)
    states = rnd(7, width, seed=3)
    for step in range(2):  # the second step goes on from the states the first one left
        proj = rnd(sum(lens), 3 * width + 2, seed=10 + step, scale=1.5)[:, : 3 * width]
        a, b = states.clone(), states.clone()
        got = ops.mingru_scan(proj, bz, bu, a, slots, ctx.cu_tokens, 4, width, out_dtype, max(lens))
        want = plain_ops.mingru_scan(proj, bz, bu, b, slots, ctx.cu_tokens, 4, width, out_dtype)
        close(got, want, out_dtype, "outputs")
        close(a, b, torch.float32, "states")
        assert torch.equal(a[[1, 4, 6]], states[[1, 4, 6]]), "slots of no request stay untouched"
        states = a


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_prepare_and_unit_norm_writes(ops, dtype):
    page_size, num_pages = 4, 30
    lens = [3, 17, 1]
    ctx, table, slot_map = make_ctx(lens, [40, 17, 9], page_size, num_pages)
    n = sum(lens)
    heads, dim, rot, rank = 3, 10, 6, 14
    proj = rnd(n, heads * (dim + rot) + rank + rot + 5, dtype=dtype, scale=0.8)
    weight = 1 + rnd(rank, seed=1, scale=0.1)
    freq = (50.0 ** (-torch.arange(2, dtype=torch.float64) * 2 / 4)).float().to(DEV)  # four of the six lanes turn
    a = torch.zeros((num_pages, page_size, rank + rot), dtype=dtype, device=DEV)
    b = a.clone()
    close(ops.latent_prepare(proj, ctx.positions, slot_map, a, weight, freq, 1e-5, heads, dim, rot, rank),
          plain_ops.latent_prepare(proj, ctx.positions, slot_map, b, weight, freq, 1e-5, heads, dim, rot, rank), dtype, "rotated query parts")
    close(a, b, dtype, "cached rows")
    H, KV, dk, dv = 4, 2, 10, 6
    for eps in (1e-5, None):
        qkv = rnd(n, (H + KV) * dk + KV * dv, dtype=dtype, seed=3)
        qa, qb = qkv.clone(), qkv.clone()
        pa = torch.zeros((num_pages, 2, KV, page_size, 10), dtype=dtype, device=DEV)
        pb = pa.clone()
        ops.unit_norm_kv_write(qa, slot_map, pa, eps, H, KV, dk, dv)
        plain_ops.unit_norm_kv_write(qb, slot_map, pb, eps, H, KV, dk, dv)
        close(qa, qb, dtype, "queries")
        close(pa, pb, dtype, "keys and values in their pages")


SHAPES = {  # (heads, kv_heads, key lanes, rotated or extra lanes, value lanes)
    "odd": (3, 1, 20, 6, 20),
    "tensor": (4, 1, 32, 16, 32),
    "wide": (2, 1, 128, 32, 128),
}


@pytest.mark.parametrize("generic", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", sorted(SHAPES))
def test_latent_attention_over_pages(ops, shape, dtype, generic, monkeypatch):
    """Prompt portions beside decoded tokens, contexts of unequal length, on the general kernel and the tensor cores."""
    monkeypatch.setattr(ops, "_FORCE_GENERIC_ATTENTION", generic)
    heads, _, rank, rot, _ = SHAPES[shape]
    page_size, num_pages = 8, 120
    ctx, table, _ = make_ctx([1, 70, 5, 1, 130], [300, 70, 64, 1, 233], page_size, num_pages, seed=3)
    n = ctx.num_tokens
    plane = rnd(num_pages, page_size, rank + rot, dtype=dtype, seed=1)
    q_lat = rnd(heads, n, rank, dtype=dtype, seed=2, scale=0.3).transpose(0, 1)
    q_rot = rnd(n, heads, rot, dtype=dtype, seed=3, scale=0.3)
    got = ops.latent_paged_attention(q_lat, q_rot, plane, table, ctx, rank=rank, scale=0.4)
    want = plain_ops.latent_paged_attention(q_lat, q_rot, plane, table, ctx, rank=rank, scale=0.4)
    close(got, want, dtype, "attention over cached latents")


@pytest.mark.parametrize("generic", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,KV,dk,dv,window", [(4, 2, 10, 6, 5), (4, 2, 32, 16, 33), (6, 3, 16, 48, 1), (8, 1, 64, 64, 100)])
def test_biased_window_attention_over_pages(ops, H, KV, dk, dv, window, dtype, generic, monkeypatch):
    monkeypatch.setattr(ops, "_FORCE_GENERIC_ATTENTION", generic)
    page_size, num_pages = 4, 200
    ctx, table, _ = make_ctx([1, 70, 5, 1, 130], [300, 70, 64, 1, 233], page_size, num_pages, seed=5)
    n = ctx.num_tokens
    pool = rnd(num_pages, 2, KV, page_size, max(dk, dv), dtype=dtype, seed=1)
    qkv = rnd(n, (H + KV) * dk + KV * dv, dtype=dtype, seed=2)
    slopes = torch.pow(2.0, -8.0 * torch.arange(1, H + 1) / H).float().to(DEV)
    kw = dict(num_heads=H, num_kv_heads=KV, key_dim=dk, value_dim=dv, scale=0.3, window=window, slopes=slopes)
    close(ops.biased_paged_attention(qkv, pool, table, ctx, **kw), plain_ops.biased_paged_attention(qkv, pool, table, ctx, **kw), dtype, "window attention")
    kw.update(window=None, slopes=None)
    close(ops.biased_paged_attention(qkv, pool, table, ctx, **kw), plain_ops.biased_paged_attention(qkv, pool, table, ctx, **kw), dtype, "no window, no bias")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_keys_cut_over_several_ctas_are_merged(ops, dtype):
    """Two decoding requests with long contexts: the tensor-core kernel cuts their keys over many CTAs."""
    heads, rank, rot = 16, 64, 16
    page_size, num_pages = 16, 300
    ctx, table, _ = make_ctx([1, 1], [2100, 1777], page_size, num_pages, seed=9)
    plane = rnd(num_pages, page_size, rank + rot, dtype=dtype, seed=1)
    q_lat, q_rot = rnd(2, heads, rank, dtype=dtype, seed=2, scale=0.2), rnd(2, heads, rot, dtype=dtype, seed=3, scale=0.2)
    got = ops.latent_paged_attention(q_lat, q_rot, plane, table, ctx, rank=rank, scale=0.5)
    want = plain_ops.latent_paged_attention(q_lat, q_rot, plane, table, ctx, rank=rank, scale=0.5)
    close(got, want, dtype, "split keys")
    if dtype == torch.bfloat16:
        # the same with the merge, a product per head and a sigmoid gate done by one kernel
        parts = ops.latent_paged_attention(q_lat, q_rot, plane, table, ctx, rank=rank, scale=0.5, leave_parts=True)
        assert isinstance(parts, ops.AttentionParts) and parts.splits > 1
        w = rnd(heads, 24, rank, dtype=dtype, seed=4, scale=0.2)
        gate = rnd(2, heads * 24 + 8, dtype=dtype, seed=5)[:, 8:]
        ref = plain_ops.gate_mul(plain_ops.head_linear(want, w), gate, "sigmoid")
        close(ops.merge_project_gate(parts, w, gate), ref, dtype, "merge, product per head and gate in one")
        close(ops.merge_project_gate(parts, w, None), plain_ops.head_linear(want, w).reshape(2, -1), dtype, "without a gate")
        few = rnd(2, heads + 3, dtype=dtype, seed=6)[:, 1 : 1 + heads]  # one gate a head and token
        ref = plain_ops.gate_mul(plain_ops.head_linear(want, w), few, "sigmoid", per_head=True)
        close(ops.merge_project_gate(parts, w, few, per_head=True), ref, dtype, "merge, product per head and a gate a head in one")


def one_hot_case(ops, dtype, generic, monkeypatch, *, form, context, query_len, target_distance, window, page_size=16):
    """Keys and values are small noise except one key, ``target_distance`` tokens before the LAST query, which points
    where the query points with a large length, and whose value is a known vector.  Returns the last query's output
    and the known vector: they agree if and only if that key was seen."""
    monkeypatch.setattr(ops, "_FORCE_GENERIC_ATTENTION", generic)
    heads, dk, dv = 4, 32, 32
    num_pages = -(-context // page_size) + 3
    ctx, table, _ = make_ctx([query_len], [context], page_size, num_pages, seed=context)
    target = context - 1 - target_distance
    marked = torch.zeros(dk)
    marked[5] = 12.0
    known = torch.linspace(-1, 1, dv)
    page, off = int(table[0, target // page_size]), target % page_size
    q = torch.zeros(query_len, heads, dk)
    q[:, :, 5] = 12.0
    if form == "latent":
        rank, rot = 32, 16
        plane = rnd(num_pages, page_size, rank + rot, dtype=torch.float32, seed=1, scale=0.05)
        # the row is key and value at once: mark lane 5 of the rotated part, and make the latent the known vector
        plane[page, off, rank:] = 0
        plane[page, off, rank + 5] = 12.0
        plane[page, off, :rank] = known.to(DEV)
        q_lat = torch.zeros(query_len, heads, rank)
        q_rot = torch.zeros(query_len, heads, rot)
        q_rot[:, :, 5] = 12.0
        out = ops.latent_paged_attention(q_lat.to(dtype).to(DEV), q_rot.to(dtype).to(DEV), plane.to(dtype), table, ctx, rank=rank, scale=1.0, window=window)
        return out[-1].float().cpu(), known
    pool = rnd(num_pages, 2, 1, page_size, dk, dtype=torch.float32, seed=1, scale=0.05)
    pool[page, 0, 0, off] = marked.to(DEV)
    pool[page, 1, 0, off] = known.to(DEV)
    qkv = q.reshape(query_len, heads * dk).to(dtype).to(DEV)
    slopes = torch.full((heads,), 1e-3, device=DEV)
    out = ops.biased_paged_attention(qkv, pool.to(dtype), table, ctx, num_heads=heads, num_kv_heads=1, key_dim=dk, value_dim=dv, scale=1.0,
                                     window=window, slopes=slopes)
    return out[-1].float().cpu().view(heads, dv), known


@pytest.mark.parametrize("generic", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("query_len", [1, 2, 37])
@pytest.mark.parametrize("form", ["latent", "window"])
def test_a_key_far_back_and_at_page_borders_is_seen(ops, form, query_len, dtype, generic, monkeypatch):
    for context, distance in ((700, 650), (700, 699), (129, 64), (129, 65), (48, 15), (48, 16), (48, 17), (40, 0)):
        if distance >= context:
            continue
        out, known = one_hot_case(ops, dtype, generic, monkeypatch, form=form, context=context, query_len=min(query_len, context - distance),
                                  target_distance=distance, window=None)
        assert float((out - known).abs().max()) < 0.05, f"the key {distance} tokens back of {context} was not seen"


@pytest.mark.parametrize("generic", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("query_len", [1, 2, 40])
@pytest.mark.parametrize("form", ["latent", "window"])
def test_keys_just_inside_and_just_outside_the_window(ops, form, query_len, dtype, generic, monkeypatch):
    for window in (1, 7, 16, 33, 96):
        for context in (window + 41, 200):
            inside, _ = one_hot_case(ops, dtype, generic, monkeypatch, form=form, context=context, query_len=query_len,
                                     target_distance=window - 1, window=window)
            known = torch.linspace(-1, 1, 32)
            assert float((inside - known).abs().max()) < 0.05, f"window {window}: the oldest key inside it was not seen"
            outside, _ = one_hot_case(ops, dtype, generic, monkeypatch, form=form, context=context, query_len=query_len,
                                      target_distance=window, window=window)
            assert float((outside - known).abs().max()) > 0.3, f"window {window}: the key just outside it was seen"
