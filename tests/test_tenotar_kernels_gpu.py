"""The kernels that the Tenotar design added or widened against their plain statements (tests/plain_ops.py) at odd sizes:
softmax attention with kept first keys, blocks of positions, capped scores and a distance bias (both attention kernels);
the heads' preparation with neighbouring lanes rotated and values mixed across layers; the short convolution through its
state slots; the latent preparation with queries of their own and the half layout; the row norm with a pitch; the gate a
head; the router with a bias; the gated experts' plain form.  And attention inputs built so that one key decides the
result, just inside and just outside every window, block and run of kept keys."""

from __future__ import annotations

import itertools
from types import SimpleNamespace

import pytest
import torch

import plain_ops
from test_kafepel_kernels_gpu import DEV, _ops, close, paged_batch

pytestmark = pytest.mark.gpu

# heads, kv heads, key lanes, value lanes, rotated lanes, page size
SHAPES = [(8, 2, 24, 40, 24, 16), (3, 1, 10, 6, 4, 8), (6, 2, 48, 48, 0, 16), (4, 4, 128, 128, 64, 4), (1, 1, 2, 1, 2, 1), (5, 5, 7, 3, 0, 3),
          (4, 2, 64, 32, 64, 16), (12, 4, 16, 32, 8, 8)]
MASKS = [
    ("a window that keeps the first keys", dict(window=33, keep_first=7)),
    ("more kept keys than the window is wide", dict(window=5, keep_first=70)),
    ("kept keys that end on a tile's border", dict(window=64, keep_first=64)),
    ("a window of one and one kept key", dict(window=1, keep_first=1)),
    ("blocks", dict(chunk=48)),
    ("blocks of one tile", dict(chunk=64)),
    ("blocks of one key", dict(chunk=1)),
    ("blocks, a cap and a distance bias", dict(chunk=100, softcap=1.5, slopes=True)),
    ("a cap", dict(softcap=0.7)),
    ("a window, a cap and a distance bias", dict(window=40, softcap=3.0, slopes=True)),
]


@pytest.mark.parametrize("general", [False, True])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("H,KV,D,V,rot,page_size", SHAPES)
def test_masks_caps_and_biases_against_plain(H, KV, D, V, rot, page_size, dtype, tol, general, monkeypatch):
    """``general``: the kernel for any sizes also where the tensor-core kernel would run (bfloat16, lanes in sixteens)."""
    ops = _ops()
    if general and dtype == torch.float32:
        pytest.skip("float32 always runs the general kernel")
    monkeypatch.setattr(ops, "_FORCE_GENERIC_ATTENTION", general)
    torch.manual_seed(H * 100 + D + 2)
    ctx, table, slots, pages = paged_batch([37, 1, 200, 530], [5, 1, 200, 2], page_size)
    N = ctx.num_tokens
    pool = (torch.randn(pages, 2, KV, page_size, max(D, V), device=DEV) * 0.7).to(dtype)
    q = torch.randn(N, H * D, device=DEV).to(dtype)
    slopes = 2.0 ** (-8.0 * torch.arange(1, H + 1, device=DEV) / H)
    common = dict(num_heads=H, num_kv_heads=KV, key_dim=D, value_dim=V, scale=0.3)
    rows = [4, 5, 205, 207]
    few = SimpleNamespace(positions=ctx.positions[rows].contiguous(), token_request=ctx.token_request[rows].contiguous(), max_context_len=530,
                          max_query_len=1, num_requests=4, num_tokens=4, context_lens=ctx.context_lens,
                          cu_tokens=torch.arange(5, dtype=torch.int32, device=DEV), host_cu_tokens=[0, 1, 2, 3, 4])
    for what, more in MASKS:
        more = dict(more)
        if more.pop("slopes", False):
            more["slopes"] = slopes
        full = plain_ops.paged_softmax_attention(q, pool, table, ctx, **common, **more)
        close(ops.paged_softmax_attention(q, pool, table, ctx, **common, **more), full, tol, what)
        # the same rows as single tokens of a small step (long contexts may be cut over several CTAs)
        close(ops.paged_softmax_attention(q[rows].contiguous(), pool, table, few, **common, **more), full[rows], tol, what + ", single tokens")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("general", [False, True])
@pytest.mark.parametrize("news", [[600, 1, 1], [1, 1, 1], [64, 2, 1]])
def test_one_key_at_an_edge_decides(news, dtype, general, monkeypatch):
    """Keys are built from the three base-9 digits of their position (a third of a unit vector per digit), so that a query
    66 times key j scores 66 on key j and at most 44 on any other visible key.  A query that asks for a visible key gets
    that key's value row; one that asks for a key just outside gets a mixture in which that row has no weight (its output
    then equals that of the same query under a mask that hides the key by a wide margin).  Asked for: the key just inside
    and just outside a window of 70, the last kept key and the first not kept (10 kept), the first key of the query's
    block of 96 positions and the key in front of it, and the query's own."""
    ops = _ops()
    monkeypatch.setattr(ops, "_FORCE_GENERIC_ATTENTION", general)
    H, KV, D, V, page_size = 4, 2, 32, 16, 8
    lens = [600, 523, 300]
    ctx, table, slots, pages = paged_batch(lens, news, page_size, seed=3)
    pool = torch.zeros(pages, 2, KV, page_size, D, device=DEV, dtype=dtype)
    j = torch.arange(max(lens))
    code = torch.zeros(max(lens), D)
    for digit in range(3):
        code[j, 9 * digit + (j // 9 ** digit) % 9] = 3 ** -0.5
    vals = {r: torch.randn(n, KV, V) for r, n in enumerate(lens)}
    host_table = table.cpu()
    for r, n in enumerate(lens):
        for jj in range(n):
            page, off = int(host_table[r, jj // page_size]), jj % page_size
            pool[page, 0, :, off] = code[jj].to(dtype)
            pool[page, 1, :, off, :V] = vals[r][jj].to(dtype)
    positions, owner = ctx.positions.cpu().tolist(), ctx.token_request.cpu().tolist()
    tol = 2e-4 if dtype == torch.float32 else 4e-2
    common = dict(num_heads=H, num_kv_heads=KV, key_dim=D, value_dim=V, scale=1.0)
    W, K, C = 70, 10, 96
    cases = [
        ("the query's own key", dict(window=W, keep_first=K), lambda p: p, True),
        ("the oldest key of the window", dict(window=W, keep_first=K), lambda p: max(0, p - W + 1), True),
        ("the key in front of the window", dict(window=W, keep_first=K), lambda p: p - W, False),
        ("the last kept key", dict(window=W, keep_first=K), lambda p: min(p, K - 1), True),
        ("the first key behind the kept ones", dict(window=W, keep_first=K), lambda p: K, False),
        ("the first key of the block", dict(chunk=C), lambda p: p - p % C, True),
        ("the key in front of the block", dict(chunk=C), lambda p: p - p % C - 1, False),
    ]
    for what, mask, target_of, inside in cases:
        targets = [target_of(p) for p in positions]
        q = torch.stack([code[max(t, 0)] * 66.0 for t in targets]).repeat(1, H).to(DEV).to(dtype)
        out = ops.paged_softmax_attention(q, pool, table, ctx, **common, **mask).float().cpu()
        reference = plain_ops.paged_softmax_attention(q, pool, table, ctx, **common, **mask).float().cpu()
        for i, (p, t) in enumerate(zip(positions, targets)):
            row = vals[owner[i]][max(t, 0)].repeat_interleave(H // KV, dim=0).reshape(-1).to(dtype).float()
            visible = 0 <= t <= p and ((p - t < mask["window"] or t < mask["keep_first"]) if "window" in mask else t // C == p // C)
            assert visible or not inside, what
            if visible:
                assert float((out[i] - row).abs().max()) <= tol, f"{what}: position {p} does not get key {t}"
            else:  # the asked-for key has no weight: what is left is the other keys' mixture, as the plain statement has it
                assert float((out[i] - reference[i]).abs().max()) <= tol, f"{what}: position {p} differs from the plain statement"
                if t >= 0 and float((reference[i] - row).abs().max()) > 10 * tol:
                    assert float((out[i] - row).abs().max()) > 5 * tol, f"{what}: position {p} sees key {t}"


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("H,KV,D,V,rot,page_size", SHAPES)
def test_head_prepare_with_neighbouring_lanes_and_mixed_values(H, KV, D, V, rot, page_size, dtype, tol):
    ops = _ops()
    torch.manual_seed(H * 100 + D + 3)
    ctx, table, slots, pages = paged_batch([37, 1, 200, 530], [5, 1, 200, 2], page_size)
    N = ctx.num_tokens
    freq = torch.rand(rot // 2, device=DEV) if rot else None
    qw, kw = torch.randn(D, device=DEV), torch.randn(D, device=DEV)
    cols = (H + KV) * D + KV * V
    proj = torch.randn(N, cols + 5, device=DEV)
    bias = torch.randn(cols, device=DEV)
    first = torch.randn(N, KV * V, device=DEV)
    for what, more in (
        ("neighbouring lanes, norms, bias", dict(bias=bias, q_weight=qw, k_weight=kw, eps=1e-5, freq=freq, interleaved=True)),
        ("values kept for later layers", dict(bias=bias, freq=freq, interleaved=True, keep=True)),
        ("values mixed with an earlier layer's", dict(freq=freq, values_first=first, values_lambda=0.3)),
    ):
        more = dict(more)
        keep = more.pop("keep", False)
        pool = (torch.randn(pages, 2, KV, page_size, max(D, V), device=DEV) * 0.5).to(dtype)
        p1, p2 = pool.clone(), pool.clone()
        k1 = torch.zeros(N, KV * V, device=DEV) if keep else None
        k2 = torch.zeros(N, KV * V, device=DEV) if keep else None
        kwargs = dict(heads=H, kv_heads=KV, dim=D, value_dim=V, slot_map=slots, out_dtype=dtype, **more)
        q1 = ops.head_prepare(proj, ctx.positions, pool=p1, values_out=k1, **kwargs)
        q2 = plain_ops.head_prepare(proj, ctx.positions, pool=p2, values_out=k2, **kwargs)
        close(q1, q2, tol, what + ": queries")
        close(p1, p2, tol, what + ": keys and values in their pages")
        if keep:
            close(k1, k2, 1e-6, what + ": the kept values")
            close(k1, proj[:, (H + KV) * D : cols] + bias[(H + KV) * D :], 1e-6, what + ": the kept values are the projected ones with their bias")


@pytest.mark.parametrize("in_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("C,taps", [(7, 4), (130, 2), (300, 1), (64, 16), (33, 3), (64, 4), (132, 3), (8, 2), (520, 1)])
def test_short_convolution_against_plain_and_across_ways_of_cutting(C, taps, in_dtype):
    """Requests of unequal length in one step against the plain statement (rows with a pitch, slots in any order); then the
    same tokens in portions down to one token through the state slots: bit-equal outputs whatever the cut, and slots that
    hold the last rows."""
    ops = _ops()
    torch.manual_seed(C * 10 + taps)
    lens = [70, 1, 19, 33]
    N = sum(lens)
    if C % 4 == 0 and C != 300:  # rows on 16-byte boundaries with a pitch: the kernel of four channels a thread takes them (up to four taps)
        u = torch.randn(N, C + 8, device=DEV).to(in_dtype)[:, 4 : 4 + C]
    else:
        u = torch.randn(N, C + 9, device=DEV).to(in_dtype)[:, 2 : 2 + C + 3]
    w = torch.randn(C, taps, device=DEV)
    slots = torch.tensor([2, 0, 5, 3], dtype=torch.int32, device=DEV)

    def ctx_of(counts):
        cu = torch.tensor([0] + list(itertools.accumulate(counts)), dtype=torch.int32, device=DEV)
        owner = torch.repeat_interleave(torch.arange(len(counts), dtype=torch.int32), torch.tensor(counts)).to(DEV)
        return SimpleNamespace(cu_tokens=cu, token_request=owner, num_requests=len(counts), max_query_len=max(counts))

    s1 = torch.zeros(6, max(taps - 1, 1), C, device=DEV)[:, : taps - 1]
    s1 = s1.contiguous() if taps > 1 else None
    s2 = None if s1 is None else s1.clone()
    whole = ops.short_conv(u, w, s1, slots, ctx_of(lens), channels=C)
    close(whole, plain_ops.short_conv(u, w, s2, slots, ctx_of(lens), channels=C), 1e-6, "whole requests")
    if taps > 1:
        close(s1, s2, 1e-6, "the slots after whole requests")
        last = u[69 - (taps - 2) : 70, :C].float() if taps - 1 <= 70 else None
        assert torch.equal(s1[2], last), "a slot holds the last rows of its request"
        assert torch.equal(s1[0, : taps - 2], torch.zeros(taps - 2, C, device=DEV)) and torch.equal(s1[0, taps - 2], u[70, :C].float())
    # in portions: 70 tokens as 1, 2, 5, 1, 40, 21; the others whole beside the first portions
    s3 = None if s1 is None else torch.zeros_like(s1)
    starts = [0, 70, 71, 90]
    got = torch.empty_like(whole)
    at = 0
    for step, n in enumerate((1, 2, 5, 1, 40, 21)):
        rows = list(range(at, at + n))
        counts, sl = [n], [2]
        if step < 3:
            other = step + 1
            rows += list(range(starts[other], starts[other] + lens[other]))
            counts.append(lens[other])
            sl.append(int(slots[other]))
        part = ops.short_conv(u[rows].contiguous(), w, s3, torch.tensor(sl, dtype=torch.int32, device=DEV), ctx_of(counts), channels=C)
        got[rows] = part
        at += n
    assert torch.equal(got, whole), "the outputs depend on how the tokens were cut"
    if taps > 1:
        assert torch.equal(s3, s1), "the slots depend on how the tokens were cut"


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("H,dim,rot,rank,qr,dims", [(3, 10, 6, 9, 7, 6), (4, 16, 16, 48, 16, 16), (1, 2, 2, 1, 1, 2), (5, 32, 16, 80, 24, 8), (2, 64, 32, 128, 96, 32)])
def test_latent_prepare_with_queries_of_their_own_and_the_half_layout(H, dim, rot, rank, qr, dims, dtype, tol):
    ops = _ops()
    torch.manual_seed(H * 10 + rank)
    ctx, table, slots, pages = paged_batch([37, 1, 200], [5, 1, 200], 8)
    N = ctx.num_tokens
    proj = torch.randn(N, qr + rank + rot + H + 3, device=DEV).to(dtype)
    queries = torch.randn(N, H * (dim + rot) + 8, device=DEV).to(dtype)[:, : H * (dim + rot)]
    weight, freq = torch.randn(rank, device=DEV), torch.rand(dims // 2, device=DEV)
    for halves in (True, False):
        p1 = torch.zeros(pages, 8, rank + rot, device=DEV, dtype=dtype)
        p2 = p1.clone()
        a, rows_a = ops.latent_prepare(proj, ctx.positions, slots, p1, weight, freq, 1e-5, H, dim, rot, rank, fresh=True, queries=queries, kv_col=qr, halves=halves)
        b, rows_b = plain_ops.latent_prepare(proj, ctx.positions, slots, p2, weight, freq, 1e-5, H, dim, rot, rank, fresh=True, queries=queries, kv_col=qr, halves=halves)
        close(a, b, tol, "the queries' rotated parts")
        close(p1, p2, tol, "the cached rows")
        close(rows_a, rows_b, tol, "the rows token by token")
    # the half layout with the queries in the stacked rows, as a design without a query latent has them
    stacked = torch.randn(N, H * (dim + rot) + rank + rot + 2, device=DEV).to(dtype)
    p1 = torch.zeros(pages, 8, rank + rot, device=DEV, dtype=dtype)
    p2 = p1.clone()
    close(ops.latent_prepare(stacked, ctx.positions, slots, p1, weight, freq, 1e-5, H, dim, rot, rank, halves=True),
          plain_ops.latent_prepare(stacked, ctx.positions, slots, p2, weight, freq, 1e-5, H, dim, rot, rank, halves=True), tol, "stacked rows, half layout")
    close(p1, p2, tol, "stacked rows, half layout: the cached rows")


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
def test_row_norm_with_a_pitch_and_a_gate_a_head(dtype, tol):
    ops = _ops()
    torch.manual_seed(5)
    for n, c in ((1, 1), (7, 88), (130, 33), (5, 700)):
        x = (torch.randn(n, c + 11, device=DEV) * 3).to(dtype)[:, 4 : 4 + c]
        w = torch.randn(c, device=DEV)
        for out_dtype in (dtype, torch.float32):
            close(ops.row_rmsnorm(x, w, 1e-5, out_dtype), plain_ops.row_rmsnorm(x, w, 1e-5, out_dtype), tol, f"row norm {n} x {c}")
    for n, inter in ((1, 1), (5, 36), (130, 7)):  # the feed-forward's biases join in the activation's kernel
        gate_up, bias = torch.randn(n, 2 * inter, device=DEV).to(dtype), torch.randn(2 * inter, device=DEV).to(dtype)
        close(ops.swiglu(gate_up, bias), plain_ops.swiglu(gate_up, bias), tol * 2, f"gated activation with biases {n} x {inter}")
    for n, heads, width in ((1, 1, 1), (9, 5, 40), (40, 3, 10)):
        a = torch.randn(n, heads + 1, width + 3, device=DEV).to(dtype)[:, :heads, :width]
        b = torch.randn(n, heads + 5, device=DEV).to(dtype)[:, 2 : 2 + heads]
        close(ops.gate_mul(a, b, "sigmoid", per_head=True), plain_ops.gate_mul(a, b, "sigmoid", per_head=True), tol, "a gate a head")


@pytest.mark.parametrize("x_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("N,K,E,top", [(1, 40, 5, 2), (33, 160, 10, 2), (70, 96, 37, 4), (4, 64, 1, 1), (9, 64, 3, 3)])
def test_router_with_a_bias_and_gated_experts_against_plain(N, K, E, top, x_dtype):
    ops = _ops()
    torch.manual_seed(N + E)
    x = torch.randn(N, K, device=DEV).to(x_dtype)
    w, b = torch.randn(E, K, device=DEV) * 0.3, torch.randn(E, device=DEV) * 2.0
    for shared_one in (False, True):
        got = ops.route(x, w, None, E, top, 1.0, True, False, bias=b, shared_one=shared_one)
        ref = plain_ops.route(x, w, None, E, top, 1.0, True, False, bias=b, shared_one=shared_one)
        close(got, ref, 2e-5, "router weights")
        assert torch.equal(got != 0, ref != 0), "the router chooses other experts than the plain statement"
        assert got.shape == (N, E + int(shared_one)) and (not shared_one or bool((got[:, E] == 1).all()))
        assert torch.allclose(got[:, :E].sum(-1), torch.ones(N, device=DEV), atol=1e-5)  # the chosen logits' softmax sums to one
    # the bias decides: without it the choice differs somewhere (for more than one expert to choose from)
    if E > top and N >= 9:
        assert not torch.equal(ops.route(x, w, None, E, top, 1.0, True, False) != 0, ops.route(x, w, None, E, top, 1.0, True, False, bias=b) != 0)
    for ff, fs in ((8, 16), (9, 0), (16, 24)):
        for dtype, tol in ((torch.float32, 2e-6), (torch.bfloat16, 1e-2)):
            wide = torch.randn(N, 2 * (E * ff + fs) + 8, device=DEV).to(dtype)
            weights = ops.route(x, w, None, E, top, 1.0, True, False, bias=b, shared_one=fs > 0)
            got = ops.expert_gated_act(wide, E, ff, fs, float("inf"), float("inf"), 1.0, weights=weights, up_shift=0.0)
            ref = plain_ops.expert_gated_act(wide, E, ff, fs, float("inf"), float("inf"), 1.0, weights=weights, up_shift=0.0)
            close(got, ref, tol, "gated experts")
            g, u = wide[:, :ff].float(), wide[:, ff : 2 * ff].float()
            close(got[:, :ff], g * torch.sigmoid(g) * u * weights[:, :1], tol, "the first expert is silu(gate) * up * weight")
