"""The kernels of softmax attention with sinks and gates, of the heads' preparation, of gated linear attention, of
table-routed experts and of a stream kept in copies against their plain statements (tests/plain_ops.py) at odd sizes, and
attention inputs built so that one key, or the sink, decides the result."""

from __future__ import annotations

from types import SimpleNamespace

import pytest
import torch

import plain_ops
from test_kafepel_kernels_gpu import DEV, _ops, close, paged_batch

pytestmark = pytest.mark.gpu

# heads, kv heads, key lanes, value lanes, rotated lanes, page size
SHAPES = [(8, 2, 24, 40, 24, 16), (3, 1, 10, 6, 4, 8), (6, 2, 48, 48, 0, 16), (4, 4, 128, 128, 64, 4), (1, 1, 2, 1, 2, 1), (5, 5, 7, 3, 0, 3),
          (4, 2, 64, 64, 16, 16), (12, 4, 16, 32, 8, 8)]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("H,KV,D,V,rot,page_size", SHAPES)
def test_head_prepare_against_plain(H, KV, D, V, rot, page_size, dtype, tol):
    ops = _ops()
    torch.manual_seed(H * 100 + D)
    ctx, table, slots, pages = paged_batch([37, 1, 200, 530], [5, 1, 200, 2], page_size)
    N = ctx.num_tokens
    freq = torch.rand(rot // 2, device=DEV) if rot else None
    qw, kw = torch.randn(D, device=DEV), torch.randn(D, device=DEV)
    for what, more in (
        ("bias, norms, rotation, values that are the keys", dict(value_dim=D, bias=True, q_weight=qw, k_weight=kw, eps=1e-5, freq=freq, values_are_keys=True)),
        ("bias and the queries' factor", dict(value_dim=V, bias=True, warm=(0.7, 3))),
        ("bare", dict(value_dim=V)),
        ("queries only", dict(value_dim=V, bias=True, warm=(1.3, 64), q_weight=qw, eps=1e-6, freq=freq, no_keys=True)),
    ):
        more = dict(more)
        kv = 0 if more.pop("no_keys", False) else KV
        vak = more.get("values_are_keys", False)
        cols = (H + kv) * D + (0 if vak else kv * more["value_dim"])
        proj = torch.randn(N, cols + 5, device=DEV)
        if more.get("bias"):
            more["bias"] = torch.randn(cols, device=DEV)
        else:
            more.pop("bias", None)
        pool = (torch.randn(pages, 2, KV, page_size, max(D, V), device=DEV) * 0.5).to(dtype)
        p1, p2 = pool.clone(), pool.clone()
        kwargs = dict(heads=H, kv_heads=kv, dim=D, slot_map=slots, out_dtype=dtype, **more)
        q1 = ops.head_prepare(proj, ctx.positions, pool=p1, **kwargs)
        q2 = plain_ops.head_prepare(proj, ctx.positions, pool=p2, **kwargs)
        close(q1, q2, tol, what + ": queries")
        close(p1, p2, tol, what + ": keys and values in their pages")
        if kv == 0:
            assert torch.equal(p1, pool), "a layer without keys of its own wrote into the pages"


@pytest.mark.parametrize("general", [False, True])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("H,KV,D,V,rot,page_size", SHAPES)
def test_softmax_attention_with_sinks_and_gates_against_plain(H, KV, D, V, rot, page_size, dtype, tol, general, monkeypatch):
    """``general``: the kernel for any sizes also where the tensor-core kernel would run (bfloat16, lanes in sixteens)."""
    ops = _ops()
    if general and dtype == torch.float32:
        pytest.skip("float32 always runs the general kernel")
    monkeypatch.setattr(ops, "_FORCE_GENERIC_ATTENTION", general)
    torch.manual_seed(H * 100 + D + 1)
    ctx, table, slots, pages = paged_batch([37, 1, 200, 530], [5, 1, 200, 2], page_size)
    N = ctx.num_tokens
    pool = (torch.randn(pages, 2, KV, page_size, max(D, V), device=DEV) * 0.7).to(dtype)
    q = torch.randn(N, H * D, device=DEV).to(dtype)
    sinks = torch.randn(H, device=DEV) * 2.0
    gate = torch.randn(N, H * V + 9, device=DEV)[:, 3 : 3 + H * V + 2]  # rows with a pitch
    common = dict(num_heads=H, num_kv_heads=KV, key_dim=D, value_dim=V, scale=0.3)
    for what, more in (("sinks and gate", dict(sinks=sinks, gate=gate)), ("sinks", dict(sinks=sinks)), ("gate", dict(gate=gate)), ("bare", {}),
                       ("window and sinks", dict(window=33, sinks=sinks))):
        close(ops.paged_softmax_attention(q, pool, table, ctx, **common, **more), plain_ops.paged_softmax_attention(q, pool, table, ctx, **common, **more), tol, what)
    # the same rows as single tokens of a small step: long contexts are cut over several CTAs, and the sink still counts once
    rows = [4, 5, 205, 207]
    few = SimpleNamespace(positions=ctx.positions[rows].contiguous(), token_request=ctx.token_request[rows].contiguous(), max_context_len=530,
                          max_query_len=1, num_requests=4, num_tokens=4, context_lens=ctx.context_lens,
                          cu_tokens=torch.arange(5, dtype=torch.int32, device=DEV), host_cu_tokens=[0, 1, 2, 3, 4])
    full = plain_ops.paged_softmax_attention(q, pool, table, ctx, **common, sinks=sinks, gate=gate)
    a = ops.paged_softmax_attention(q[rows].contiguous(), pool, table, few, **common, sinks=sinks, gate=gate[rows])
    close(a, full[rows], tol, "keys cut over CTAs")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("general", [False, True])
@pytest.mark.parametrize("news", [[600, 1, 1], [1, 1, 1], [64, 2, 1]])
def test_one_key_or_the_sink_decides(news, dtype, general, monkeypatch):
    """Keys are built from the three base-9 digits of their position (a third of a unit vector per digit), so that a query
    66 times key j scores 66 on key j and at most 44 on any other: only key j is left with a weight.  The chosen key: the
    one at position 0, one 1 / 7 / 8 back (page borders), 63 / 64 / 255 / 256 / 257 back (the borders of key tiles and of
    the shares of several CTAs), and the query's own.  The output must be that key's value row.  With a sink of 66 beside
    it the output is half of that row; with a sink of 90 it is nothing; with a sink of 30 it is the row."""
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
    for back in (None, 0, 1, 7, 8, 63, 64, 255, 256, 257):
        targets = [0 if back is None else max(0, p - back) for p in positions]
        q = torch.stack([code[t] * 66.0 for t in targets]).repeat(1, H).to(DEV).to(dtype)
        want = torch.stack([vals[owner[i]][targets[i]].repeat_interleave(H // KV, dim=0).reshape(-1) for i in range(len(targets))])
        # the score of the chosen key as the rounded operands give it (66 in 32-bit, within a half of it in bfloat16)
        score = (q[:, :D].float().cpu() * torch.stack([code[t] for t in targets]).to(dtype).float()).sum(-1, keepdim=True)
        for sink in (None, 30.0, 66.0, 90.0):
            sinks = None if sink is None else torch.full((H,), sink, device=DEV)
            share = 1.0 if sink is None else torch.sigmoid(score - sink)
            out = ops.paged_softmax_attention(q, pool, table, ctx, num_heads=H, num_kv_heads=KV, key_dim=D, value_dim=V, scale=1.0, sinks=sinks)
            err = float((out.float().cpu() - share * want.to(dtype).float()).abs().max())
            assert err <= (2e-4 if dtype == torch.float32 else 4e-2), f"key {back} back, sink {sink}: off by {err:.3e}"


@pytest.mark.parametrize("v_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,V", [(2, 6, 10), (1, 1, 1), (3, 48, 64), (2, 40, 70), (1, 130, 20), (4, 64, 128), (2, 256, 33)])
def test_gated_scan_against_plain_and_across_ways_of_cutting(H, D, V, v_dtype):
    """Requests of unequal length in one step against the plain statement; then the same tokens in portions down to one
    token through the state slots: the outputs are the same to the last bit, whatever the cut."""
    ops = _ops()
    torch.manual_seed(D * 10 + V)
    lens = [70, 1, 19, 33]
    N = sum(lens)
    cu = torch.tensor([0, 70, 71, 90, 123], dtype=torch.int32, device=DEV)
    slots = torch.tensor([2, 0, 5, 3], dtype=torch.int32, device=DEV)
    wide = torch.randn(N, 3 * H * D + H * V + 5, device=DEV)  # one row pitch for all, as a stacked projection leaves them
    q, k, z = wide[:, : H * D], wide[:, H * D : 2 * H * D], wide[:, 2 * H * D : 3 * H * D] * 3.0
    v = torch.randn(N, H * V, device=DEV).to(v_dtype)
    zb = torch.randn(H * D, device=DEV) * 2.0 + 2.0  # decays from nearly 0 to nearly 1
    states0 = torch.randn(6, H, D, V, device=DEV) * 0.3
    args = (zb, 1.0 / 5.0, D ** -0.5)
    s1, s2 = states0.clone(), states0.clone()
    o1 = ops.gated_scan(q, k, v, z, *args, s1, slots, cu, 4, H, D, V, max_query_len=70)
    o2 = plain_ops.gated_scan(q, k, v, z, *args, s2, slots, cu, 4, H, D, V)
    close(o1, o2, 3e-5, "outputs")
    close(s1, s2, 3e-5, "states")
    # in portions: request 0 in 30 + 39 + 1, request 3 in 16 + 16 + 1, each call with its own offsets
    s3 = states0.clone()
    o3 = torch.empty_like(o1)
    for parts in ([(0, 0, 30), (3, 90, 106)], [(0, 30, 69), (3, 106, 122), (2, 71, 90)], [(0, 69, 70), (3, 122, 123), (1, 70, 71)]):
        idx = torch.cat([torch.arange(a, b) for _, a, b in parts]).to(DEV)
        sizes = [b - a for _, a, b in parts]
        cu_p = torch.tensor([0] + list(torch.tensor(sizes).cumsum(0)), dtype=torch.int32, device=DEV)
        sl = torch.tensor([int(slots[r]) for r, _, _ in parts], dtype=torch.int32, device=DEV)
        o3[idx] = ops.gated_scan(q[idx].contiguous(), k[idx].contiguous(), v[idx].contiguous(), z[idx].contiguous(), *args, s3, sl, cu_p, len(parts), H, D, V,
                                 max_query_len=max(sizes))
    assert torch.equal(o3, o1) and torch.equal(s3, s1), "the recurrence depends on how the tokens were cut"


@pytest.mark.parametrize("H,D,V", [(2, 56, 64), (1, 20, 24), (2, 128, 40), (1, 256, 16), (16, 64, 128)])
def test_gated_scan_of_long_requests_shared_out_in_stretches(H, D, V):
    """Requests long enough that the kernel cuts them into stretches for several CTAs (each walked from a zero state, the
    start states found from the end states and the stretches' products of decays, the missing term added afterwards),
    beside a short one, against the plain statement.  Some channels hardly forget and some forget at once."""
    ops = _ops()
    torch.manual_seed(D + V)
    lens = [900, 3, 517, 130]
    N = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    slots = torch.tensor([1, 4, 0, 2], dtype=torch.int32, device=DEV)
    wide = torch.randn(N, 3 * H * D + H * V + 4, device=DEV)
    q, k, z = wide[:, : H * D], wide[:, H * D : 2 * H * D], wide[:, 2 * H * D : 3 * H * D] * 2.0
    v = wide[:, 3 * H * D : 3 * H * D + H * V]
    zb = torch.randn(H * D, device=DEV) * 3.0 + 4.0
    states0 = torch.randn(5, H, D, V, device=DEV)
    args = (zb, 1.0 / 12.0, D ** -0.5)
    s1, s2 = states0.clone(), states0.clone()
    o1 = ops.gated_scan(q, k, v, z, *args, s1, slots, cu, 4, H, D, V, max_query_len=max(lens))
    o2 = plain_ops.gated_scan(q, k, v, z, *args, s2, slots, cu, 4, H, D, V)
    close(o1, o2, 1e-4, "outputs")
    close(s1, s2, 1e-4, "states")
    assert torch.equal(s1[3], states0[3]), "a slot that no request names was written"


@pytest.mark.parametrize("out_dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("S,W,results", [(1, 40, 1), (2, 192, 2), (3, 33, 1), (4, 1024, 2), (8, 2048, 4), (5, 7, 3)])
def test_hyper_mix_norm_against_plain(S, W, results, out_dtype, tol):
    ops = _ops()
    torch.manual_seed(S * 7 + W)
    N = 19
    X = torch.randn(S, N, W, device=DEV)
    update = ops.StreamUpdate(ops.WeightedSum([torch.randn(N, W, device=DEV) for _ in range(results)], [0.6, -0.5, 1.7, 0.2][:results]),
                              torch.randn(S, S, device=DEV), torch.randn(S, device=DEV))
    read_in, weight = torch.randn(S, device=DEV), torch.randn(W, device=DEV)
    rows = torch.tensor([18, 0, 7], dtype=torch.int32, device=DEV)
    for what, upd, rin, rw in (("update, read in, norm", update, read_in, None), ("read in only", None, read_in, None), ("update and plain sum on chosen rows", update, None, rows),
                               ("plain sum", None, None, None)):
        x1, x2 = X.clone(), X.clone()
        a = ops.hyper_mix_norm(x1, upd, rin, weight, 1e-5, rows=rw, out_dtype=out_dtype)
        b = plain_ops.hyper_mix_norm(x2, upd, rin, weight, 1e-5, rows=rw, out_dtype=out_dtype)
        close(a, b, tol, what)
        close(x1, x2, 1e-5, what + ": the copies")
        if rw is not None or upd is None:
            assert torch.equal(x1, X), what + ": the copies were to stay as they were"
    table = torch.randn(50, W, device=DEV).to(torch.bfloat16)
    ids = torch.randint(0, 50, (N,), device=DEV, dtype=torch.int32)
    assert torch.equal(ops.embed(ids, table, copies=S), plain_ops.embed(ids, table, copies=S))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("E,top,ff,fs", [(5, 2, 12, 20), (16, 2, 48, 80), (1, 1, 32, 0), (37, 4, 6, 10), (3, 3, 7, 5), (8, 1, 8, 8)])
def test_expert_activation_with_a_table_against_plain(E, top, ff, fs, dtype, tol):
    ops = _ops()
    torch.manual_seed(E * 10 + ff)
    N, vocab = 23, 41
    x = (torch.randn(N, 2 * (E * ff + fs) + 8, device=DEV) * 2.0).to(dtype)[:, : 2 * (E * ff + fs)]
    table = torch.rand(vocab, E, device=DEV).argsort(dim=1)[:, :top].to(torch.int32).contiguous()
    ids = torch.randint(0, vocab, (N,), device=DEV, dtype=torch.int32)
    args = (E, ff, fs, 0.8, 1.9, 1.702)
    close(ops.expert_gated_act(x, *args, ids=ids, table=table), plain_ops.expert_gated_act(x, *args, ids=ids, table=table), tol, "by the table")
    w = torch.rand(N, E + 1, device=DEV) * (torch.rand(N, E + 1, device=DEV) > 0.5)
    close(ops.expert_gated_act(x, *args, weights=w), plain_ops.expert_gated_act(x, *args, weights=w), tol, "by given weights")
    # columns of experts that a token does not use are not read: poison them
    poisoned = x.clone().float()
    chosen = torch.zeros(N, E + 1, dtype=torch.bool, device=DEV)
    chosen.scatter_(1, table[ids.long()].long(), True)
    chosen[:, E] = True
    for e in range(E):
        poisoned[~chosen[:, e], e * 2 * ff : (e + 1) * 2 * ff] = float("nan")
    out = ops.expert_gated_act(poisoned.to(dtype), *args, ids=ids, table=table)
    assert torch.isfinite(out.float()).all(), "an unused expert's columns were read"


def test_head_norm_with_a_weight_and_the_32_bit_product_over_stored_weights():
    ops = _ops()
    torch.manual_seed(5)
    o, gate, w = torch.randn(29, 3, 70, device=DEV), torch.randn(29, 3 * 70 + 4, device=DEV)[:, 2 : 2 + 210], torch.randn(70, device=DEV)
    for out_dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
        close(ops.head_norm_gate(o, gate, 1e-5, "silu", out_dtype, weight=w), plain_ops.head_norm_gate(o, gate, 1e-5, "silu", out_dtype, weight=w), tol, "norm, weight, gate")
    x = torch.randn(37, 50, device=DEV)[:, 3:20]
    for wd in (torch.float32, torch.bfloat16):
        wt = torch.randn(45, 17, device=DEV).to(wd)
        close(ops.linear32(x, wt), x.double() @ wt.double().t(), 2e-6, f"linear32 over {wd} weights")
