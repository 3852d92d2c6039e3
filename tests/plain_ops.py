"""A plain torch statement of every device operation, with the signature of the engine's
``ops`` functions.  Two uses: the oracle of each kernel's own test on the GPU, and — patched
over ``ops`` by the ``plain_ops_engine`` fixture — a way to run the engine's host logic (batch
building, cache manager, step function, scheduler) on the CPU, where no kernel can run.
Everything is computed in float32 (float64 where noted) and rounded to the output type once.
"""

from __future__ import annotations

import torch

import plain_llama


def embed(ids, table, copies=None):
    rows = table[ids.long()].float()
    return rows if copies is None else rows[None].repeat(int(copies), 1, 1)


def rmsnorm(resid, weight, eps, delta=None, rows=None, out_dtype=torch.float32):
    if rows is not None:
        v = resid[rows.long()]
        if delta is not None:
            v = v + delta[rows.long()].float()
    else:
        if delta is not None:
            resid.add_(delta.float())
        v = resid
    y = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * weight
    return y.to(out_dtype)


def linear(x, w, out_dtype=None):
    out_dtype = out_dtype or x.dtype
    return (x.float() @ w.float().t()).to(out_dtype)


def _rotate(x, positions, table):
    """x [N, heads, D] float32, table [positions, D] = cos | sin halves."""
    half = x.shape[-1] // 2
    cs = table[positions.long()]
    cos, sin = cs[:, None, :half], cs[:, None, half:]
    a, b = x[..., :half], x[..., half:]
    return torch.cat((a * cos - b * sin, b * cos + a * sin), dim=-1)


def rope_kv_write(qkv, positions, table, slot_map, pool, num_heads, num_kv_heads, head_dim, write_kv=True):
    H, KV, D = num_heads, num_kv_heads, head_dim
    n = qkv.shape[0]
    q = qkv[:, : H * D].float().view(n, H, D)
    if table is not None:
        q = _rotate(q, positions, table)
    qkv[:, : H * D] = q.reshape(n, H * D).to(qkv.dtype)
    if not write_kv:
        return
    k = qkv[:, H * D : (H + KV) * D].float().view(n, KV, D)
    if table is not None:
        k = _rotate(k, positions, table)
    v = qkv[:, (H + KV) * D : (H + 2 * KV) * D].view(n, KV, D)
    page_size = pool.shape[3]
    page = (slot_map // page_size).long()
    off = (slot_map % page_size).long()
    pool[page, 0, :, off, :] = k.to(pool.dtype)
    pool[page, 1, :, off, :] = v.to(pool.dtype)


def rope_inplace(x, positions, table):
    x.copy_(_rotate(x.float(), positions, table).to(x.dtype))


def paged_attention(qkv, pool, page_table, ctx, *, num_heads, num_kv_heads, head_dim, scale, window=None):
    H, KV, D = num_heads, num_kv_heads, head_dim
    page_size = pool.shape[3]
    out = torch.empty((qkv.shape[0], H * D), dtype=qkv.dtype, device=qkv.device)
    cu = ctx.cu_tokens.tolist()
    lens = ctx.context_lens.tolist()
    for r in range(len(lens)):
        t0, t1, n = cu[r], cu[r + 1], lens[r]
        pages = page_table[r, : -(-n // page_size)].long()
        k = pool[pages, 0].float().permute(1, 0, 2, 3).reshape(KV, -1, D)[:, :n]
        v = pool[pages, 1].float().permute(1, 0, 2, 3).reshape(KV, -1, D)[:, :n]
        q = qkv[t0:t1, : H * D].float().view(t1 - t0, H, D).transpose(0, 1)
        k = k.repeat_interleave(H // KV, dim=0)
        v = v.repeat_interleave(H // KV, dim=0)
        s = torch.einsum("htd,hsd->hts", q, k) * scale
        pos = torch.arange(n - (t1 - t0), n, device=qkv.device)[:, None]
        j = torch.arange(n, device=qkv.device)[None, :]
        visible = j <= pos
        if window:
            visible = visible & (j > pos - window)
        s = s.masked_fill(~visible[None], float("-inf"))
        o = torch.einsum("hts,hsd->htd", torch.softmax(s, dim=-1), v)
        out[t0:t1] = o.transpose(0, 1).reshape(t1 - t0, H * D).to(out.dtype)
    return out


def swiglu(gate_up, bias=None):
    inter = gate_up.shape[1] // 2
    row = gate_up.float() if bias is None else gate_up.float() + bias.float()
    g, u = row[:, :inter], row[:, inter:]
    return (g * torch.sigmoid(g) * u).to(gate_up.dtype)


def add_bias(x, bias):
    x.copy_((x.float() + bias.float()).to(x.dtype))
    return x


def linear_swiglu(x, w_gate_up):
    return swiglu(linear(x, w_gate_up))


def linear_qkv_rope(*args, **kwargs):
    return None  # "not taken": the caller runs the product, the rotation and the write one by one


def argmax(logits):
    return torch.argmax(logits, dim=-1).to(torch.int32)


def sample(logits, temperature, top_k, top_p, seeds, counters):
    out = []
    for r in range(logits.shape[0]):
        u = plain_llama.uniform_from(int(seeds[r]) & ((1 << 64) - 1), int(counters[r]))
        out.append(
            plain_llama.sample_token(logits[r].cpu(), float(temperature[r]), int(top_k[r]), float(top_p[r]), u)
        )
    return torch.tensor(out, dtype=torch.int32, device=logits.device)


# ---------------------------------------------------------------------------------------------
# operations of layers that normalise in groups, scale their contributions, gate, recur or attend over a latent
def group_rmsnorm(resid, weight, eps, groups, delta=None, alpha=1.0, rows=None, out_dtype=torch.float32):
    if rows is not None:
        v = resid[rows.long()]
        if delta is not None:
            v = v + alpha * delta[rows.long()].float()
    else:
        if delta is not None:
            resid.add_(delta.float(), alpha=alpha)
        v = resid
    n, d = v.shape
    parts = v.view(n, groups, d // groups)
    y = (parts / torch.sqrt(parts.pow(2).mean(-1, keepdim=True) + eps)).reshape(n, d) * weight
    return y.to(out_dtype)


def stream_inject(resid, delta=None, alpha=1.0, ids=None, table=None, vector=None):
    if delta is not None:
        resid.add_(delta.float(), alpha=alpha)
    if table is not None:
        resid.add_(table[ids.long()].float())
    if vector is not None:
        resid.add_(vector)


def unary(x, kind, alpha=1.0, inplace=False):
    v = x.float()
    if kind == "relu2":
        y = torch.relu(v).pow(2)
    elif kind == "gelu_tanh":
        y = 0.5 * v * (1 + torch.tanh(0.7978845608028654 * (v + 0.044715 * v.pow(3))))
    elif kind == "scale":
        y = alpha * v
    elif kind == "silu":
        y = v * torch.sigmoid(v)
    else:
        raise ValueError(kind)
    if inplace:
        x.copy_(y.to(x.dtype))
        return x
    return y.to(x.dtype)


def linear_act(x, w, activation):
    return unary(linear(x, w), activation, inplace=True)


def gate_mul(a, b, kind="sigmoid", per_head=False):
    if per_head:
        b = b.repeat_interleave(a.shape[2], dim=1)
    return _gate_mul(a, b, kind)


def _gate_mul(a, b, kind="sigmoid"):
    n, heads, w = a.shape
    g = b.float()
    g = torch.sigmoid(g) if kind == "sigmoid" else g * torch.sigmoid(g)
    return (a.float().reshape(n, heads * w) * g).to(a.dtype)


def mingru_scan(proj, bias_z, bias_u, states, state_slots, cu_tokens, num_requests, width, out_dtype, max_query_len=None):
    out = torch.empty((proj.shape[0], width), dtype=out_dtype, device=proj.device)
    p = proj.float()
    cu = cu_tokens.tolist()
    for r in range(num_requests):
        slot = int(state_slots[r])
        s = states[slot].clone()
        for t in range(cu[r], cu[r + 1]):
            z = torch.sigmoid(p[t, :width] + (bias_z if bias_z is not None else 0))
            u = p[t, width : 2 * width] + (bias_u if bias_u is not None else 0)
            c = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
            s = (1 - z) * s + z * c
            g = p[t, 2 * width : 3 * width]
            out[t] = (s * g * torch.sigmoid(g)).to(out_dtype)
        states[slot] = s
    return out


def _rotate_interleaved(x, positions, freq):
    """x [N, ..., lanes] float32; the first 2 * len(freq) lanes turn in pairs (2i, 2i + 1)."""
    dims = 2 * freq.numel()
    angle = positions.float()[:, None] * freq
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = angle.cos().view(shape), angle.sin().view(shape)
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def _rotate_halves(x, positions, freq):
    """x [N, heads, rot]: lanes (i, i + pairs) of the first 2 * len(freq) lanes turn by position * freq[i] (float32 angles)."""
    pairs = freq.numel()
    if pairs == 0:
        return x
    angle = positions.float()[:, None] * freq.float()[None, :]
    c, s = angle.cos()[:, None, :], angle.sin()[:, None, :]
    u, v = x[..., :pairs], x[..., pairs : 2 * pairs]
    return torch.cat((u * c - v * s, v * c + u * s, x[..., 2 * pairs :]), dim=-1)


def latent_prepare(proj, positions, slot_map, plane, weight, freq, eps, heads, dim, rot, rank, fresh=False, queries=None, kv_col=0, halves=False):
    if queries is not None or halves:
        n = proj.shape[0]
        turn = _rotate_halves if halves else _rotate_interleaved
        q_src = proj if queries is None else queries
        col = heads * (dim + rot) if queries is None else kv_col
        q_rot = turn(q_src[:, : heads * (dim + rot)].float().view(n, heads, dim + rot)[..., dim:], positions, freq)
        latent = proj[:, col : col + rank].float()
        latent = latent / torch.sqrt(latent.pow(2).mean(-1, keepdim=True) + eps) * weight
        k_rot = turn(proj[:, col + rank : col + rank + rot].float()[:, None, :], positions, freq)[:, 0]
        rows = torch.cat((latent, k_rot), dim=-1).to(proj.dtype)
        plane.view(-1, rank + rot)[slot_map.long()] = rows
        return (q_rot.to(proj.dtype), rows) if fresh else q_rot.to(proj.dtype)
    return _latent_prepare(proj, positions, slot_map, plane, weight, freq, eps, heads, dim, rot, rank, fresh)


def _latent_prepare(proj, positions, slot_map, plane, weight, freq, eps, heads, dim, rot, rank, fresh=False):
    n = proj.shape[0]
    q = proj[:, : heads * (dim + rot)].float().view(n, heads, dim + rot)
    q_rot = _rotate_interleaved(q[..., dim:], positions, freq).to(proj.dtype)
    base = heads * (dim + rot)
    latent = proj[:, base : base + rank].float()
    latent = latent / torch.sqrt(latent.pow(2).mean(-1, keepdim=True) + eps) * weight
    k_rot = _rotate_interleaved(proj[:, base + rank : base + rank + rot].float(), positions, freq)
    page_size = plane.shape[1]
    page, off = (slot_map // page_size).long(), (slot_map % page_size).long()
    plane[page, off] = torch.cat((latent, k_rot), dim=-1).to(plane.dtype)
    return (q_rot, plane[page, off].clone()) if fresh else q_rot


def latent_two_parts(ctx, dtype, *lanes):
    return False  # the plain operations know one way only


def unit_norm_kv_write(qkv, slot_map, pool, eps, heads, kv_heads, key_dim, value_dim):
    n = qkv.shape[0]
    qk = qkv[:, : (heads + kv_heads) * key_dim].float().view(n, heads + kv_heads, key_dim)
    if eps is not None:
        qk = qk / torch.sqrt(qk.pow(2).mean(-1, keepdim=True) + eps)
    qkv[:, : heads * key_dim] = qk[:, :heads].reshape(n, -1).to(qkv.dtype)
    v = qkv[:, (heads + kv_heads) * key_dim : (heads + kv_heads) * key_dim + kv_heads * value_dim].view(n, kv_heads, value_dim)
    page_size = pool.shape[3]
    page, off = (slot_map // page_size).long(), (slot_map % page_size).long()
    pool[page, 0, :, off, :key_dim] = qk[:, heads:].to(pool.dtype)
    pool[page, 1, :, off, :value_dim] = v.to(pool.dtype)


def head_linear(x, w):
    return torch.einsum("nhk,hmk->nhm", x.float(), w.float()).to(x.dtype)


def _attend(q, k, v, first_pos, scale, window, slopes, sinks=None, keep_first=None, chunk=None, softcap=None):
    """q [T, H, dk], k [n, H, dk], v [n, H, dv] float32; query t stands at position first_pos + t.  ``sinks [H]``: a score
    per head that stands in every row's softmax without a value."""
    n = k.shape[0]
    s = torch.einsum("thd,jhd->htj", q, k) * scale
    pos = torch.arange(first_pos, first_pos + q.shape[0], device=q.device)[:, None]
    j = torch.arange(n, device=q.device)[None, :]
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    if slopes is not None:
        s = s - slopes.float()[:, None, None] * (pos - j).float()
    visible = j <= pos
    if window:
        inside = j > pos - window
        visible = visible & ((inside | (j < keep_first)) if keep_first else inside)
    if chunk:
        visible = visible & (torch.div(j, chunk, rounding_mode="floor") == torch.div(pos, chunk, rounding_mode="floor"))
    s = s.masked_fill(~visible[None], float("-inf"))
    if sinks is not None:
        s = torch.cat((s, sinks.float()[:, None, None].expand(-1, s.shape[1], 1)), dim=-1)
        return torch.einsum("htj,jhd->thd", torch.softmax(s, dim=-1)[..., :-1], v)
    return torch.einsum("htj,jhd->thd", torch.softmax(s, dim=-1), v)


def latent_paged_attention(q_lat, q_rot, plane, page_table, ctx, *, rank, scale, window=None, leave_parts=False):
    page_size = plane.shape[1]
    n_tok, heads = q_lat.shape[0], q_lat.shape[1]
    out = torch.empty((n_tok, heads, rank), dtype=q_lat.dtype, device=q_lat.device)
    cu, lens = ctx.cu_tokens.tolist(), ctx.context_lens.tolist()
    q = torch.cat((q_lat.float(), q_rot.float()), dim=-1)
    for r in range(len(lens)):
        t0, t1, n = cu[r], cu[r + 1], lens[r]
        rows = plane[page_table[r, : -(-n // page_size)].long()].float().reshape(-1, plane.shape[2])[:n]
        k = rows[:, None, :].expand(n, heads, rows.shape[1])
        out[t0:t1] = _attend(q[t0:t1], k, k[..., :rank], n - (t1 - t0), scale, window, None).to(out.dtype)
    return out


def biased_paged_attention(qkv, pool, page_table, ctx, *, num_heads, num_kv_heads, key_dim, value_dim, scale, window=None, slopes=None):
    H, KV = num_heads, num_kv_heads
    page_size = pool.shape[3]
    out = torch.empty((qkv.shape[0], H * value_dim), dtype=qkv.dtype, device=qkv.device)
    cu, lens = ctx.cu_tokens.tolist(), ctx.context_lens.tolist()
    for r in range(len(lens)):
        t0, t1, n = cu[r], cu[r + 1], lens[r]
        pages = page_table[r, : -(-n // page_size)].long()
        k = pool[pages, 0].float().permute(0, 2, 1, 3).reshape(-1, KV, pool.shape[4])[:n, :, :key_dim]
        v = pool[pages, 1].float().permute(0, 2, 1, 3).reshape(-1, KV, pool.shape[4])[:n, :, :value_dim]
        q = qkv[t0:t1, : H * key_dim].float().view(t1 - t0, H, key_dim)
        k, v = k.repeat_interleave(H // KV, dim=1), v.repeat_interleave(H // KV, dim=1)
        out[t0:t1] = _attend(q, k, v, n - (t1 - t0), scale, window, slopes).reshape(t1 - t0, -1).to(out.dtype)
    return out


def paged_softmax_attention(q, pool, page_table, ctx, *, num_heads, num_kv_heads, key_dim, value_dim, scale, window=None, sinks=None, gate=None,
                            keep_first=None, chunk=None, softcap=None, slopes=None):
    H, KV = num_heads, num_kv_heads
    page_size = pool.shape[3]
    out = torch.empty((q.shape[0], H * value_dim), dtype=q.dtype, device=q.device)
    cu, lens = ctx.cu_tokens.tolist(), ctx.context_lens.tolist()
    for r in range(len(lens)):
        t0, t1, n = cu[r], cu[r + 1], lens[r]
        pages = page_table[r, : -(-n // page_size)].long()
        k = pool[pages, 0].float().permute(0, 2, 1, 3).reshape(-1, KV, pool.shape[4])[:n, :, :key_dim]
        v = pool[pages, 1].float().permute(0, 2, 1, 3).reshape(-1, KV, pool.shape[4])[:n, :, :value_dim]
        k, v = k.repeat_interleave(H // KV, dim=1), v.repeat_interleave(H // KV, dim=1)
        o = _attend(q[t0:t1].float().view(t1 - t0, H, key_dim), k, v, n - (t1 - t0), scale, window, slopes, sinks, keep_first, chunk, softcap).reshape(t1 - t0, -1)
        if gate is not None:
            o = o * torch.sigmoid(gate[t0:t1, : H * value_dim].float())
        out[t0:t1] = o.to(out.dtype)
    return out


def head_prepare(proj, positions, *, heads, kv_heads, dim, value_dim=0, bias=None, q_weight=None, k_weight=None, eps=0.0, freq=None,
                 warm=None, values_are_keys=False, pool=None, slot_map=None, out_dtype=None, interleaved=False, values_out=None,
                 values_first=None, values_lambda=0.0):
    n = proj.shape[0]
    cols = (heads + kv_heads) * dim + (0 if values_are_keys else kv_heads * value_dim)
    row = proj[:, :cols].float()
    if bias is not None:
        row = row + bias.float()
    q = row[:, : heads * dim].view(n, heads, dim)
    k = row[:, heads * dim : (heads + kv_heads) * dim].view(n, kv_heads, dim)
    v = k if values_are_keys else row[:, (heads + kv_heads) * dim :].view(n, kv_heads, value_dim)
    if q_weight is not None:
        q = q / torch.sqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_weight.float()
        if kv_heads:
            k = k / torch.sqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_weight.float()
    if freq is not None:
        half = freq.numel()
        angle = positions.float()[:, None] * freq.float()[None, :]
        c, s_ = angle.cos()[:, None, :], angle.sin()[:, None, :]

        def turn(x):
            if interleaved:
                a, b = x[..., 0 : 2 * half : 2], x[..., 1 : 2 * half : 2]
                return torch.cat((torch.stack((a * c - b * s_, b * c + a * s_), dim=-1).flatten(-2), x[..., 2 * half :]), dim=-1)
            a, b = x[..., :half], x[..., half : 2 * half]
            return torch.cat((a * c - b * s_, b * c + a * s_, x[..., 2 * half :]), dim=-1)

        q, k = turn(q), (turn(k) if kv_heads else k)
    if warm:
        coef, every = warm
        q = q * (1.0 + coef * torch.log(torch.div(positions + 1, every, rounding_mode="floor").float() + 1.0))[:, None, None]
    if values_out is not None:
        values_out.copy_(v.reshape(n, -1))
    if values_first is not None:
        v = (1.0 - values_lambda) * v + values_lambda * values_first.view(n, kv_heads, value_dim)
    if kv_heads:
        out_dtype = pool.dtype
        page_size = pool.shape[3]
        page, off = (slot_map // page_size).long(), (slot_map % page_size).long()
        pool[page, 0, :, off, :dim] = k.to(pool.dtype)
        pool[page, 1, :, off, : v.shape[-1]] = v.to(pool.dtype)
    return q.reshape(n, heads * dim).to(out_dtype or proj.dtype)


def hyper_mix_norm(streams, update, read_in, weight, eps, rows=None, out_dtype=torch.float32):
    S = streams.shape[0]
    x = streams if rows is None else streams[:, rows.long()]
    if update is not None:
        tensors, factors = update.results()
        y = sum(f * (t if rows is None else t[rows.long()]).float() for t, f in zip(tensors, factors))
        x = torch.einsum("st,snw->tnw", update.mix.view(S, S).float(), x) + update.take.float().view(S, 1, 1) * y[None]
        if rows is None:
            streams.copy_(x)
    u = x.sum(0) if read_in is None else torch.einsum("s,snw->nw", read_in.float(), x)
    return (u * torch.rsqrt(u.pow(2).mean(-1, keepdim=True) + eps) * weight).to(out_dtype)


def linear32(x, w):
    return x.float() @ w.float().t()


def gated_scan(q, k, v, z, z_bias, inv_tau, q_scale, states, state_slots, cu_tokens, num_requests, heads, dim, value_dim, max_query_len=0):
    out = torch.empty((q.shape[0], heads, value_dim), dtype=torch.float32, device=q.device)
    cu, slots = cu_tokens.tolist(), state_slots.tolist()
    logits = z.float() + (z_bias.float() if z_bias is not None else 0.0)
    alpha = torch.exp(inv_tau * torch.nn.functional.logsigmoid(logits)).view(-1, heads, dim)
    for r in range(num_requests):
        S = states[slots[r]].float()
        for t in range(cu[r], cu[r + 1]):
            S = alpha[t][:, :, None] * S + k[t].float().view(heads, dim)[:, :, None] * v[t].float().view(heads, value_dim)[:, None, :]
            out[t] = torch.einsum("hdv,hd->hv", S, q[t].float().view(heads, dim) * q_scale)
        states[slots[r]] = S
    return out


def expert_gated_act(x, experts, ff, shared_ff, limit, shared_limit, slope, *, weights=None, ids=None, table=None, up_shift=1.0):
    n = x.shape[0]
    xf = x.float()
    if weights is None:
        top = table.shape[1]
        weights = torch.zeros((n, experts + 1), dtype=torch.float32, device=x.device)
        weights.scatter_(1, table[ids.long()].long(), 1.0 / top)
        weights[:, experts] = 1.0
    out = torch.zeros((n, experts * ff + shared_ff), dtype=torch.float32, device=x.device)
    for e in range(experts + int(shared_ff > 0)):
        width, lim = (ff, limit) if e < experts else (shared_ff, shared_limit)
        base = e * 2 * ff
        g = xf[:, base : base + width].clamp(max=lim)
        u = xf[:, base + width : base + 2 * width].clamp(min=-lim, max=lim)
        out[:, e * ff : e * ff + width] = g * torch.sigmoid(slope * g) * (u + up_shift) * weights[:, e : e + 1]
    return out.to(x.dtype)


def qk_prepare(proj, positions, *, heads, kv_heads, dim, value_dim=0, freq=None, q_weight=None, k_weight=None, eps=0.0, k_scale=1.0,
               pool=None, slot_map=None, out_dtype=None):
    n = proj.shape[0]
    q = proj[:, : heads * dim].float()
    k = proj[:, heads * dim : (heads + kv_heads) * dim].float()
    if q_weight is not None:
        q = q / torch.sqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_weight
        k = k / torch.sqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_weight

    def turn(x, count):
        x = x.view(n, count, dim)
        if freq is None or freq.numel() == 0:
            return x
        half = freq.numel()
        angle = positions.float()[:, None] * freq[None, :]
        c, s = angle.cos()[:, None, :], angle.sin()[:, None, :]
        u, v = x[..., :half], x[..., half : 2 * half]
        return torch.cat((u * c - v * s, v * c + u * s, x[..., 2 * half :]), dim=-1)

    q, k = turn(q, heads).reshape(n, -1), turn(k, kv_heads) * k_scale
    if pool is None:
        out_dtype = out_dtype or proj.dtype
        return q.to(out_dtype), k.reshape(n, -1).to(out_dtype)
    v = proj[:, (heads + kv_heads) * dim : (heads + kv_heads) * dim + kv_heads * value_dim].view(n, kv_heads, value_dim)
    page_size = pool.shape[3]
    page, off = (slot_map // page_size).long(), (slot_map % page_size).long()
    pool[page, 0, :, off, :dim] = k.to(pool.dtype)
    pool[page, 1, :, off, :value_dim] = v.to(pool.dtype)
    return q.to(pool.dtype)


def sigmoid_attention(q, pool, page_table, ctx, *, num_heads, num_kv_heads, key_dim, value_dim, scale, softcap=None, head_bias=None,
                      head_mix=None, window=None):
    H, KV = num_heads, num_kv_heads
    page_size = pool.shape[3]
    out = torch.empty((q.shape[0], H * value_dim), dtype=q.dtype, device=q.device)
    cu, lens = ctx.cu_tokens.tolist(), ctx.context_lens.tolist()
    for r in range(len(lens)):
        t0, t1, n = cu[r], cu[r + 1], lens[r]
        pages = page_table[r, : -(-n // page_size)].long()
        k = pool[pages, 0].float().permute(0, 2, 1, 3).reshape(-1, KV, pool.shape[4])[:n, :, :key_dim]
        v = pool[pages, 1].float().permute(0, 2, 1, 3).reshape(-1, KV, pool.shape[4])[:n, :, :value_dim]
        k, v = k.repeat_interleave(H // KV, dim=1), v.repeat_interleave(H // KV, dim=1)
        qq = q[t0:t1].float().view(t1 - t0, H, key_dim)
        s = torch.einsum("thd,jhd->htj", qq, k) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        if head_bias is not None:
            s = s + head_bias.float()[:, None, None]
        pos = torch.arange(n - (t1 - t0), n, device=q.device)[:, None]
        j = torch.arange(n, device=q.device)[None, :]
        visible = j <= pos
        if window:
            visible = visible & (j > pos - window)
        p = torch.sigmoid(s) * visible[None]
        if head_mix is not None:
            p = torch.einsum("hg,gtj->htj", head_mix.float().view(H, H), p)
        out[t0:t1] = torch.einsum("htj,jhd->thd", p, v).reshape(t1 - t0, -1).to(out.dtype)
    return out


def retention_scan(q, k, v, decay, states, state_slots, cu_tokens, num_requests, heads, dim, value_dim, max_query_len=0):
    n = q.shape[0]
    out = torch.empty((n, heads, value_dim), dtype=torch.float32, device=q.device)
    cu, slots = cu_tokens.tolist(), state_slots.tolist()
    g = decay.float()[:, None, None]
    for r in range(num_requests):
        S = states[slots[r]].clone()
        for t in range(cu[r], cu[r + 1]):
            kt, vt = k[t].float().view(heads, dim), v[t].float().view(heads, value_dim)
            S = g * S + kt[:, :, None] * vt[:, None, :]
            out[t] = torch.einsum("hdv,hd->hv", S, q[t].float().view(heads, dim))
        states[slots[r]] = S
    return out


def head_norm_gate(o, gate, eps, kind="silu", out_dtype=torch.float32, weight=None):
    y = o.float()
    if eps is not None:
        y = y / torch.sqrt(y.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    y = y.reshape(o.shape[0], -1)
    if gate is not None:
        z = gate.float()
        y = y * (torch.sigmoid(z) if kind == "sigmoid" else z * torch.sigmoid(z))
    return y.to(out_dtype)


def route_topk(z, correction, experts, top, scale=1.0, renormalize=False, shared_gate=False):
    s = torch.softmax(z[:, :experts].float(), dim=-1)
    choice = s if correction is None else s + correction.float()
    chosen = torch.zeros_like(s, dtype=torch.bool)
    work = choice.clone()
    for _ in range(top):  # the lowest index among equals, as the kernel
        arg = work.argmax(dim=-1, keepdim=True)
        chosen.scatter_(1, arg, True)
        work.scatter_(1, arg, float("-inf"))
    w = s * chosen * scale
    if renormalize:
        w = w / (s * chosen).sum(-1, keepdim=True)
    if shared_gate:
        w = torch.cat((w, torch.sigmoid(z[:, experts : experts + 1].float())), dim=1)
    return w


def route(x, w_router, correction, experts, top, scale=1.0, renormalize=False, shared_gate=False, bias=None, shared_one=False):
    z = x.float() @ w_router.float().t()
    if bias is not None:
        z = torch.cat((z[:, :experts] + bias.float(), z[:, experts:]), dim=1)
    w = route_topk(z, correction, experts, top, scale, renormalize, shared_gate)
    return torch.cat((w, torch.ones_like(w[:, :1])), dim=1) if shared_one else w


def short_conv(u, weight, states, state_slots, ctx, channels=None):
    c = int(channels) if channels is not None else weight.shape[0]
    taps = weight.shape[1]
    out = torch.empty((u.shape[0], c), dtype=torch.float32, device=u.device)
    cu, slots = ctx.cu_tokens.tolist(), state_slots.tolist()
    for r in range(len(cu) - 1):
        t0, t1 = cu[r], cu[r + 1]
        rows = u[t0:t1, :c].float()
        if taps > 1:
            rows = torch.cat((states[slots[r]], rows), dim=0)
            states[slots[r]] = rows[rows.shape[0] - (taps - 1) :]
        out[t0:t1] = sum(weight[:, j].float()[None, :] * rows[j : j + (t1 - t0)] for j in range(taps))
    return out


def row_rmsnorm(x, weight, eps, out_dtype=None):
    v = x.float()
    return (v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps) * weight).to(out_dtype or x.dtype)


def expert_act_scale(x, weights, experts, ff, activation):
    y = unary(x.float(), activation)
    cols = torch.arange(x.shape[1], device=x.device)
    block = torch.where(cols < experts * ff, cols // ff, torch.full_like(cols, experts))
    return (y * weights[:, block]).to(x.dtype)


def branch_norm_sum(branches, weights, eps, factor):
    total = 0
    for x, w in zip(branches, weights):
        total = total + x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w
    return total * factor


def branch_sum_rmsnorm(pending, resid, weight, eps, out_dtype):
    resid.add_(branch_norm_sum(pending.branches, pending.weights, pending.eps, pending.factor))
    return (resid * torch.rsqrt(resid.pow(2).mean(-1, keepdim=True) + eps) * weight).to(out_dtype)


ALL = (
    "short_conv",
    "row_rmsnorm",
    "paged_softmax_attention",
    "head_prepare",
    "hyper_mix_norm",
    "linear32",
    "gated_scan",
    "expert_gated_act",
    "branch_sum_rmsnorm",
    "qk_prepare",
    "sigmoid_attention",
    "retention_scan",
    "head_norm_gate",
    "route_topk",
    "route",
    "expert_act_scale",
    "branch_norm_sum",
    "group_rmsnorm",
    "stream_inject",
    "unary",
    "linear_act",
    "gate_mul",
    "mingru_scan",
    "latent_prepare",
    "latent_two_parts",
    "unit_norm_kv_write",
    "head_linear",
    "latent_paged_attention",
    "biased_paged_attention",
    "embed",
    "rmsnorm",
    "linear",
    "rope_kv_write",
    "rope_inplace",
    "paged_attention",
    "swiglu",
    "add_bias",
    "linear_swiglu",
    "linear_qkv_rope",
    "argmax",
    "sample",
)
