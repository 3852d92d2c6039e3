// Attention in its general form on the tensor cores (bfloat16, mma.sync m16n8k16, 32-bit accumulation): queries in one or
// two runs of lanes, keys of dk lanes and values of dv lanes addressed by strides (the values may be the head of the key
// rows: a cached latent that is key and value at once then crosses shared memory once), an optional distance bias per
// head, a window.  Prompt portions and decoded tokens take the same kernel.
//
// One CTA of four warps owns 64 rows of one (request, key/value head): a row is a (token, group member) pair, so the
// heads that share keys sit side by side in a tile (with one key/value head for all query heads, a decoded token alone
// fills heads-many rows).  Each warp keeps 16 rows: scores of a tile of keys in registers, the online softmax in 32-bit,
// the probabilities straight from the score registers as the next product's left operand, the output in registers.
// Key tiles (64 keys, or 32 where rows are long) arrive by cp.async into a ring of two; keys past the request's length
// are filled with zeros.  The keys of a row tile may be cut over `splits` CTAs, whose partial results (unnormalised
// output, running maximum, sum) a second kernel merges.
#include "attention_rows.cuh"

namespace {

using bf16 = __nv_bfloat16;
constexpr int PAD = 8;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const bf16* p) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const bf16* p) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(bf16* dst, const bf16* src, bool valid) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros and the source is not read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(addr), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ unsigned pack2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}

// BM rows a CTA (64 or 128: sixteen a warp).  The larger tile halves the trips of keys and values from L2 per row, which
// is what bounds requests that bring many rows per key/value head.
template <int DV_MAX, int BN, int BM>
__global__ void __launch_bounds__(BM * 2, (DV_MAX <= 64 ? 4 : (DV_MAX <= 128 ? 3 : 2)) * 64 / BM)
attention_rows_mma_kernel(const RowsArgs<bf16> a, int splits, float* __restrict__ part_o, float* __restrict__ part_ml) {
    constexpr int THREADS = BM * 2;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int dk = a.d0 + a.d1, dv = a.dv, kp = dk + PAD, vp = dv + PAD;
    const bool alias = a.key_part != 2 && a.values == a.keys && a.v_page == a.k_page && a.v_head == a.k_head && a.v_token == a.k_token;
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);  // [BM][kp]
    bf16* Ks = Qs + BM * kp;                       // [2][BN][kp]
    bf16* Vs = alias ? Ks : Ks + 2 * BN * kp;      // [2][BN][vp] unless the values are the head of the key rows
    const int v_pitch = alias ? kp : vp, v_stage = alias ? BN * kp : BN * vp;

    const int r = blockIdx.z, kvh = blockIdx.y;
    // the last row tiles of a request see the most keys: they are handed out first, so that no long CTA starts last
    const int slot = blockIdx.x / splits, split = blockIdx.x - slot * splits;
    const int tile = (int)(gridDim.x / splits) - 1 - slot;
    const int group = a.H / a.KV;
    const int q_begin = a.cu_tokens[r], q_len = a.cu_tokens[r + 1] - q_begin, ctx_len = a.ctx_lens[r];
    const int rows_total = q_len * group, row0 = tile * BM;
    if (row0 >= rows_total) return;
    const int first_pos = ctx_len - q_len;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // the keys this tile's rows see, and this split's share of their tiles
    const int pos_min = first_pos + row0 / group, pos_max = first_pos + min(rows_total - 1, row0 + BM - 1) / group;
    int key_lo = a.window > 0 ? max(0, pos_min - a.window + 1) : 0, key_hi = pos_max;
    if (a.chunk > 0) key_lo = max(key_lo, pos_min - pos_min % a.chunk);  // the oldest row's block of positions starts first
    if (a.key_part == 1) key_hi = min(key_hi, first_pos - 1);  // only what was cached before this step
    if (a.key_part == 2) key_lo = max(key_lo, first_pos);     // only the step's own tokens
    // with a window the keys below keep_first stay visible: their tiles come first, then the window's (one run from key 0
    // where the two meet)
    const int kf = (a.window > 0 && a.key_part == 0) ? a.keep_first : 0;
    int j_first = (key_lo / BN) * BN;
    int kept_tiles = (min(kf, key_lo) + BN - 1) / BN;
    if (kept_tiles * BN >= j_first) { j_first = 0; kept_tiles = 0; }
    const int n_tiles = (key_hi >= j_first ? (key_hi - j_first) / BN + 1 : 0) + kept_tiles;
    auto tile_start = [&](int t) { return t < kept_tiles ? t * BN : j_first + (t - kept_tiles) * BN; };
    const int per = (n_tiles + splits - 1) / splits;
    const int t_begin = split * per, t_end = min(n_tiles, t_begin + per);

    if (n_tiles == 0 && splits == 1 && a.stats) {  // a part without keys for these rows: statistics that say so, and
        for (int i = tid; i < BM; i += THREADS) {     // an output that the merge does not read
            const int R = row0 + i;
            if (R >= rows_total) break;
            const int t = q_begin + R / group, h = kvh * group + R % group;
            a.stats[((size_t)t * a.H + h) * 2] = -INFINITY;
            a.stats[((size_t)t * a.H + h) * 2 + 1] = 0.f;
        }
        return;
    }
    const int* table = a.page_table + (size_t)r * a.table_width;
    const int k_chunks = dk >> 3, v_chunks = dv >> 3;
    pdl_trigger();
    pdl_wait();  // the queries and the newest cached rows are the work of the kernels in front
    // eight lanes a key (128 bytes of its row a pass), sixteen keys a pass of the CTA: a key's page is looked up once
    auto load_tile = [&](int t, int stage) {
        const int j0 = tile_start(t), sub = tid & 7;
        bf16* kd = Ks + stage * BN * kp;
        bf16* vd = Vs + stage * BN * vp;
        for (int key = tid >> 3; key < BN; key += THREADS / 8) {
            const int j = j0 + key;
            if (a.key_part == 2) {  // the step's own tokens, token by token
                const bool valid = j >= first_pos && j < ctx_len;
                const long long i = valid ? q_begin + (j - first_pos) : 0;
                const bf16* k0 = a.keys + i * a.k_token + (long long)kvh * a.k_head;
                const bf16* k1 = a.keys1 ? a.keys1 + i * a.k1_token : k0;
                const int c0 = a.keys1 ? a.fresh_d0 >> 3 : k_chunks;
                for (int c = sub; c < k_chunks; c += 8) cp_async16(kd + key * kp + c * 8, c < c0 ? k0 + c * 8 : k1 + (c - c0) * 8, valid);
                const bf16* v0 = a.values + i * a.v_token + (long long)kvh * a.v_head;
                for (int c = sub; c < v_chunks; c += 8) cp_async16(vd + key * vp + c * 8, v0 + c * 8, valid);
                continue;
            }
            const bool valid = j < ctx_len;
            long long k_off = 0, v_off = 0;
            if (valid) {
                const int page = table[j / a.page_size], off = j % a.page_size;
                k_off = (long long)page * a.k_page + (long long)kvh * a.k_head + (long long)off * a.k_token;
                v_off = (long long)page * a.v_page + (long long)kvh * a.v_head + (long long)off * a.v_token;
            }
            for (int c = sub; c < k_chunks; c += 8) cp_async16(kd + key * kp + c * 8, a.keys + k_off + c * 8, valid);
            if (!alias)
                for (int c = sub; c < v_chunks; c += 8) cp_async16(vd + key * vp + c * 8, a.values + v_off + c * 8, valid);
        }
    };

    // queries of the tile's rows into shared memory (rows past the request's last are zeros)
    for (int i = tid; i < BM * k_chunks; i += THREADS) {
        const int row = i / k_chunks, c = (i - row * k_chunks) * 8, R = row0 + row;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (R < rows_total) {
            const int t = q_begin + R / group, h = kvh * group + R % group;
            const bf16* src = c < a.d0 ? a.q0 + (long long)t * a.q0_token + (long long)h * a.q0_head + c
                                       : a.q1 + (long long)t * a.q1_token + (long long)h * a.q1_head + (c - a.d0);
            v = *reinterpret_cast<const uint4*>(src);
        }
        *reinterpret_cast<uint4*>(Qs + row * kp + c) = v;
    }
    if (t_begin < t_end) load_tile(t_begin, 0);
    cp_async_commit();

    // the two rows of this thread: (lane / 4) and (lane / 4 + 8) of the warp's sixteen
    int pos[2], lo[2], hi[2];
    float slope[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int R = min(row0 + warp * 16 + (lane >> 2) + 8 * e, rows_total - 1);
        pos[e] = first_pos + R / group;
        lo[e] = a.window > 0 ? max(0, pos[e] - a.window + 1) : 0;
        if (a.chunk > 0) lo[e] = max(lo[e], pos[e] - pos[e] % a.chunk);
        if (a.key_part == 2) lo[e] = max(lo[e], first_pos);
        hi[e] = a.key_part == 1 ? min(pos[e], first_pos - 1) : pos[e];
        slope[e] = a.slopes ? a.slopes[kvh * group + R % group] * LOG2E : 0.f;
    }
    const float scale2 = a.scale * LOG2E, cap2 = a.softcap * LOG2E, cap_in2 = a.softcap > 0.f ? 2.f * LOG2E * a.scale / a.softcap : 0.f;
    // the keys that every row of this warp sees: from the newest row's window start to the oldest row's position
    int warp_lo, warp_hi;
    {
        const int R0 = min(row0 + warp * 16, rows_total - 1), R1 = min(row0 + warp * 16 + 15, rows_total - 1);
        const int p0 = first_pos + R0 / group, p1 = first_pos + R1 / group;
        warp_lo = a.window > 0 ? max(0, p1 - a.window + 1) : 0;
        if (a.chunk > 0) warp_lo = max(warp_lo, p1 - p1 % a.chunk);
        if (a.key_part == 2) warp_lo = max(warp_lo, first_pos);
        warp_hi = a.key_part == 1 ? min(p0, first_pos - 1) : p0;
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    if (a.sinks && split == 0) {
        // a sink stands for a key of score sinks[h] (not scaled) without a value; the first split counts it, once a row
        // (a row's sum is kept in four lanes' shares until the end: the share of the first takes it)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int R = min(row0 + warp * 16 + (lane >> 2) + 8 * e, rows_total - 1);
            m[e] = a.sinks[kvh * group + R % group] * LOG2E;
            l[e] = (lane & 3) == 0 ? 1.f : 0.f;
        }
    }
    float o[DV_MAX / 8][4];
#pragma unroll
    for (int i = 0; i < DV_MAX / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    for (int t = t_begin; t < t_end; ++t) {
        const int stage = (t - t_begin) & 1;
        if (t + 1 < t_end) load_tile(t + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const bf16* kt = Ks + stage * BN * kp;
        const bf16* vt = Vs + stage * v_stage;
        const int j0 = tile_start(t);

        float s[BN / 8][4];
#pragma unroll
        for (int i = 0; i < BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll 2
        for (int ks = 0; ks < dk; ks += 16) {
            unsigned qa[4];
            ldmatrix_x4(qa, Qs + (warp * 16 + (lane & 15)) * kp + ks + (lane >> 4) * 8);
#pragma unroll
            for (int nb = 0; nb < BN / 8; nb += 2) {
                unsigned kb[4];
                ldmatrix_x4(kb, kt + (nb * 8 + (lane >> 4) * 8 + (lane & 7)) * kp + ks + ((lane >> 3) & 1) * 8);
                mma_bf16(s[nb], qa, kb[0], kb[1]);
                mma_bf16(s[nb + 1], qa, kb[2], kb[3]);
            }
        }
        // scale, bias, mask (scores in units of log 2 from here on); the tile's maximum per row
        // (maxima and sums are kept in two halves per row, joined at the end: half as long a chain of dependent operations)
        float part_max[2][2] = {{-INFINITY, -INFINITY}, {-INFINITY, -INFINITY}};
        // every row of the warp sees every key of the tile: inside all windows, or among the kept first keys
        const bool whole = (j0 >= warp_lo || j0 + BN <= kf) && j0 + BN - 1 <= warp_hi;
        const bool biased = a.slopes != nullptr, capped = a.softcap > 0.f;
#pragma unroll
        for (int nb = 0; nb < BN / 8; ++nb)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int e = c >> 1, j = j0 + nb * 8 + (lane & 3) * 2 + (c & 1);
                // the cap: tanh(t) = 1 - 2 / (e^(2t) + 1), through exp2 and a reciprocal (absolute error near 1e-7, which the cap
                // multiplies: far below what the bfloat16 operands leave; both ends saturate to +-1)
                float v = capped ? cap2 * (1.f - __fdividef(2.f, exp2f(s[nb][c] * cap_in2) + 1.f)) : s[nb][c] * scale2;
                if (biased) v -= slope[e] * (float)(pos[e] - j);
                if (!whole) v = ((j >= lo[e] || j < kf) && j <= hi[e]) ? v : -INFINITY;
                s[nb][c] = v;
                part_max[e][nb & 1] = fmaxf(part_max[e][nb & 1], v);
            }
        float tile_max[2] = {fmaxf(part_max[0][0], part_max[0][1]), fmaxf(part_max[1][0], part_max[1][1])};
        float rescale[2], m_use[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            tile_max[e] = fmaxf(tile_max[e], __shfl_xor_sync(0xffffffffu, tile_max[e], 1));
            tile_max[e] = fmaxf(tile_max[e], __shfl_xor_sync(0xffffffffu, tile_max[e], 2));
            const float m_new = fmaxf(m[e], tile_max[e]);
            m_use[e] = m_new == -INFINITY ? 0.f : m_new;  // a row that has seen no key yet
            rescale[e] = exp2f(m[e] - m_use[e]);
            m[e] = m_new;
            l[e] *= rescale[e];
        }
#pragma unroll
        for (int i = 0; i < DV_MAX / 8; ++i)
            if (i * 8 < dv) {
                o[i][0] *= rescale[0]; o[i][1] *= rescale[0];
                o[i][2] *= rescale[1]; o[i][3] *= rescale[1];
            }
        float part_sum[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
        for (int nb = 0; nb < BN / 8; ++nb)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float p = exp2f(s[nb][c] - m_use[c >> 1]);
                s[nb][c] = p;
                part_sum[c >> 1][nb & 1] += p;
            }
        l[0] += part_sum[0][0] + part_sum[0][1];
        l[1] += part_sum[1][0] + part_sum[1][1];
        // O += P V
#pragma unroll
        for (int kb = 0; kb < BN / 16; ++kb) {
            unsigned pa[4];
            pa[0] = pack2(s[2 * kb][0], s[2 * kb][1]);
            pa[1] = pack2(s[2 * kb][2], s[2 * kb][3]);
            pa[2] = pack2(s[2 * kb + 1][0], s[2 * kb + 1][1]);
            pa[3] = pack2(s[2 * kb + 1][2], s[2 * kb + 1][3]);
#pragma unroll
            for (int nb = 0; nb < DV_MAX / 8; nb += 2)
                if (nb * 8 < dv) {
                    unsigned vb[4];
                    ldmatrix_x4_trans(vb, vt + (kb * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * v_pitch + nb * 8 + (lane >> 4) * 8);
                    mma_bf16(o[nb], pa, vb[0], vb[1]);
                    mma_bf16(o[nb + 1], pa, vb[2], vb[3]);
                }
        }
        __syncthreads();  // the stage is free for the tile after next
    }
    cp_async_wait<0>();

#pragma unroll
    for (int e = 0; e < 2; ++e) {
        l[e] += __shfl_xor_sync(0xffffffffu, l[e], 1);
        l[e] += __shfl_xor_sync(0xffffffffu, l[e], 2);
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int R = row0 + warp * 16 + (lane >> 2) + 8 * e;
        if (R >= rows_total) continue;
        const int t = q_begin + R / group, h = kvh * group + R % group;
        if (splits == 1) {
            const float inv = l[e] > 0.f ? 1.f / l[e] : 0.f;  // no key seen (a part without keys for this row): zeros
            if (a.stats && (lane & 3) == 0) {
                a.stats[((size_t)t * a.H + h) * 2] = m[e];  // in units of log 2, as the merge expects
                a.stats[((size_t)t * a.H + h) * 2 + 1] = l[e];
            }
            bf16* op = a.out + (long long)t * a.out_token + (long long)h * a.out_head;
            const float* gp = a.gate ? a.gate + (long long)t * a.gate_token + (long long)h * dv : nullptr;
#pragma unroll
            for (int i = 0; i < DV_MAX / 8; ++i)
                if (i * 8 < dv) {
                    const int col = i * 8 + (lane & 3) * 2;
                    float y0 = o[i][2 * e] * inv, y1 = o[i][2 * e + 1] * inv;
                    if (gp) {
                        y0 *= 1.f / (1.f + __expf(-gp[col]));
                        y1 *= 1.f / (1.f + __expf(-gp[col + 1]));
                    }
                    *reinterpret_cast<__nv_bfloat162*>(op + col) = __floats2bfloat162_rn(y0, y1);
                }
        } else {
            const size_t slot = ((size_t)t * a.H + h) * splits + split;
            float* po = part_o + slot * dv;
#pragma unroll
            for (int i = 0; i < DV_MAX / 8; ++i)
                if (i * 8 < dv) {
                    const int col = i * 8 + (lane & 3) * 2;
                    *reinterpret_cast<float2*>(po + col) = make_float2(o[i][2 * e], o[i][2 * e + 1]);
                }
            if ((lane & 3) == 0) {
                part_ml[slot * 2] = m[e];
                part_ml[slot * 2 + 1] = l[e];
            }
        }
    }
}

// out[t, h] = sum_s exp(m_s - M) o_s / sum_s exp(m_s - M) l_s over the splits' partial results; one warp per (token, head)
__global__ void __launch_bounds__(128)
attention_rows_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out,
                            long long out_token, long long out_head, int n_tokens, int H, int dv, int splits,
                            const float* __restrict__ gate, long long gate_token) {
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    pdl_trigger();
    pdl_wait();
    if (item >= (long long)n_tokens * H) return;
    const int t = (int)(item / H), h = (int)(item - (long long)t * H);
    const float* ml = part_ml + (size_t)item * splits * 2;
    // lane s holds the weight of split s (at most 32 splits): exp(m_s - M), and the sum of all of them times their sums
    const float ms = lane < splits ? ml[2 * lane] : -INFINITY, ls = lane < splits ? ml[2 * lane + 1] : 0.f;
    const float M = warp_max(ms);
    const float ws = ms == -INFINITY ? 0.f : exp2f(ms - M);  // the kernel's maxima are in units of log 2
    const float inv = 1.f / warp_sum(ws * ls);
    bf16* op = out + (long long)t * out_token + (long long)h * out_head;
    const float* po = part_o + (size_t)item * splits * dv;
    for (int d0 = 0; d0 < dv; d0 += 256) {  // eight independent sums a lane, so that a split's loads are in flight together
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < splits; ++s) {
            const float w = __shfl_sync(0xffffffffu, ws, s);
            if (w == 0.f) continue;  // uniform across the warp
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int d = d0 + lane + 32 * i;
                if (d < dv) acc[i] = fmaf(w, po[(size_t)s * dv + d], acc[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int d = d0 + lane + 32 * i;
            if (d < dv) {
                float y = acc[i] * inv;
                if (gate) y *= 1.f / (1.f + __expf(-gate[(long long)t * gate_token + (long long)h * dv + d]));
                op[d] = __float2bfloat16_rn(y);
            }
        }
    }
}

// out[t, h] = (w1 o1 + w2 o2) / (w1 + w2) with w = sum * 2^(maximum - M): two parts of one softmax, each normalised by
// itself, joined.  o1, o2 [n, H, dv] with token and head strides; one warp per (token, head).
__global__ void __launch_bounds__(128)
merge_two_parts_kernel(const bf16* __restrict__ o1, long long o1_token, long long o1_head, const float* __restrict__ stats1,
                       const bf16* __restrict__ o2, long long o2_token, long long o2_head, const float* __restrict__ stats2,
                       bf16* __restrict__ out, long long out_token, long long out_head, int n_tokens, int H, int dv) {
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    pdl_trigger();
    pdl_wait();
    if (item >= (long long)n_tokens * H) return;
    const int t = (int)(item / H), h = (int)(item - (long long)t * H);
    const float m1 = stats1[item * 2], l1 = stats1[item * 2 + 1], m2 = stats2[item * 2], l2 = stats2[item * 2 + 1];
    const float M = fmaxf(m1, m2);
    const float w1 = l1 > 0.f ? l1 * exp2f(m1 - M) : 0.f, w2 = l2 > 0.f ? l2 * exp2f(m2 - M) : 0.f;  // maxima in units of log 2
    const float inv = 1.f / (w1 + w2);
    const bf16* a = o1 + (long long)t * o1_token + (long long)h * o1_head;
    const bf16* b = o2 + (long long)t * o2_token + (long long)h * o2_head;
    bf16* o = out + (long long)t * out_token + (long long)h * out_head;
    // a part without keys has weight 0 and an output that was never written: it is not read
    for (int d = lane; d < dv; d += 32) {
        const float av = w1 > 0.f ? __bfloat162float(a[d]) : 0.f, bv = w2 > 0.f ? __bfloat162float(b[d]) : 0.f;
        o[d] = __float2bfloat16_rn((w1 * av + w2 * bv) * inv);
    }
}

// For steps of few rows whose keys were cut over `splits` CTAs: the merge of the partial results, the product with a
// per-head matrix w [H, n_out, dv] (the value up-projection of latent attention) and an optional sigmoid gate, in one
// kernel; one CTA per (token, head).  out[t, h * n_out + e] = gate(g[t, h * n_out + e]) * sum_r w[h, e, r] merged[r].
__global__ void __launch_bounds__(128)
merge_project_gate_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int splits,
                          const bf16* __restrict__ w, const bf16* __restrict__ gate, int ldg, bf16* __restrict__ out, int H,
                          int dv, int n_out, int gate_per_head) {
    extern __shared__ float merged[];  // dv floats, then the splits' weights
    float* weights = merged + dv;
    const int item = blockIdx.x, t = item / H, h = item - t * H, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_trigger();
    pdl_wait();
    const float* ml = part_ml + (size_t)item * splits * 2;
    if (warp == 0) {
        const float ms = lane < splits ? ml[2 * lane] : -INFINITY, ls = lane < splits ? ml[2 * lane + 1] : 0.f;
        const float M = warp_max(ms);
        const float ws = ms == -INFINITY ? 0.f : exp2f(ms - M);
        const float inv = 1.f / warp_sum(ws * ls);
        if (lane < splits) weights[lane] = ws * inv;
    }
    __syncthreads();
    const float* po = part_o + (size_t)item * splits * dv;
    for (int r = threadIdx.x; r < dv; r += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float ws = weights[s];
            if (ws != 0.f) acc = fmaf(ws, po[(size_t)s * dv + r], acc);
        }
        merged[r] = acc;
    }
    __syncthreads();
    const bf16* wh = w + (size_t)h * n_out * dv;
    for (int e = warp; e < n_out; e += 4) {
        const bf16* row = wh + (size_t)e * dv;
        float acc = 0.f;
        for (int r = lane * 2; r < dv; r += 64) {
            const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(row + r);
            acc = fmaf(__low2float(v), merged[r], acc);
            acc = fmaf(__high2float(v), merged[r + 1], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            const size_t col = (size_t)h * n_out + e;
            if (gate) acc *= 1.f / (1.f + expf(-__bfloat162float(gate[(size_t)t * ldg + (gate_per_head ? (size_t)h : col)])));
            out[(size_t)t * H * n_out + col] = __float2bfloat16_rn(acc);
        }
    }
}

template <int DV_MAX, int BN, int BM = 64>
int launch(const RowsArgs<bf16>& a, int requests, int max_query_len, int splits, float* part_o, float* part_ml, size_t smem,
           cudaStream_t stream) {
    constexpr int THREADS = BM * 2;
    auto kernel = attention_rows_mma_kernel<DV_MAX, BN, BM>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int group = a.H / a.KV;
    const long long tiles = ((long long)max_query_len * group + BM - 1) / BM;
    if (tiles * splits > 0x7fffffffLL || a.KV > 65535 || requests > 65535) return LLM_ERR_UNSUPPORTED;
    return launch_pdl(kernel, dim3((unsigned)(tiles * splits), a.KV, requests), dim3(THREADS), smem, stream, a, splits, part_o, part_ml);
}

}  // namespace

// As llm_attention_rows, for bfloat16 with every run of lanes a multiple of 16 and 16-byte aligned rows; dv <= 256.
// `max_query_len`: the most tokens a request brings (it sizes the grid).  `splits` > 1 cuts every row tile's keys over
// that many CTAs; part_o [n_tokens * H * splits * dv] and part_ml [n_tokens * H * splits * 2] (float32) then hold the
// partial results until the merge that follows.  Returns LLM_ERR_UNSUPPORTED for shapes it does not take.
LLM_EXPORT int llm_attention_rows_mma(const void* q0, long long q0_token, long long q0_head, int d0, const void* q1,
                                      long long q1_token, long long q1_head, int d1, void* out, long long out_token,
                                      long long out_head, const void* keys, long long k_page, long long k_head,
                                      long long k_token, const void* values, long long v_page, long long v_head,
                                      long long v_token, int dv, const int* page_table, int table_width,
                                      const int* token_request, const int* cu_tokens, const int* ctx_lens, const float* slopes,
                                      int n_tokens, int requests, int max_query_len, int H, int KV, int page_size, int window,
                                      float scale, int splits, float* part_o, float* part_ml, int key_part, const void* keys1,
                                      long long k1_token, int fresh_d0, float* stats, const float* sinks, const float* gate,
                                      long long gate_token, int keep_first, int chunk, float softcap, cudaStream_t stream) {
    if (n_tokens <= 0 || requests <= 0) return 0;
    if (d0 <= 0 || d1 < 0 || dv <= 0 || H <= 0 || KV <= 0 || H % KV || page_size <= 0 || table_width <= 0 || splits < 1 ||
        max_query_len < 1 || (d1 > 0 && q1 == nullptr) || (splits > 1 && (part_o == nullptr || part_ml == nullptr)))
        return LLM_ERR_BAD_ARGUMENT;
    const int dk = d0 + d1;
    auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    if ((d0 & 15) || (d1 & 15) || (dv & 15) || dv > 256 || dk > 640) return LLM_ERR_UNSUPPORTED;
    if (key_part < 0 || key_part > 2 || (stats && splits != 1)) return LLM_ERR_BAD_ARGUMENT;
    if (keep_first < 0 || chunk < 0 || (keep_first > 0 && key_part != 0)) return LLM_ERR_BAD_ARGUMENT;  // kept keys belong to a whole softmax
    if ((sinks || gate) && (key_part != 0 || stats)) return LLM_ERR_BAD_ARGUMENT;  // a sink belongs to a whole softmax, not to a part of one
    if (gate && (splits > 1 && out == nullptr)) return LLM_ERR_BAD_ARGUMENT;
    if (key_part == 2 && keys1 && ((fresh_d0 & 15) || fresh_d0 <= 0 || fresh_d0 >= dk || (k1_token & 7) || ((uintptr_t)keys1 & 15)))
        return LLM_ERR_UNSUPPORTED;
    if ((q0_token & 7) || (q0_head & 7) || (q1_token & 7) || (q1_head & 7) || (k_page & 7) || (k_head & 7) || (k_token & 7) ||
        (v_page & 7) || (v_head & 7) || (v_token & 7) || (out_token & 1) || (out_head & 1))
        return LLM_ERR_UNSUPPORTED;
    if (!aligned(q0) || (d1 > 0 && !aligned(q1)) || !aligned(keys) || !aligned(values) || ((uintptr_t)out & 3)) return LLM_ERR_UNSUPPORTED;
    RowsArgs<bf16> a;
    a.q0 = (const bf16*)q0; a.q1 = (const bf16*)q1;
    a.q0_token = q0_token; a.q0_head = q0_head; a.q1_token = q1_token; a.q1_head = q1_head;
    a.d0 = d0; a.d1 = d1;
    a.out = (bf16*)out; a.out_token = out_token; a.out_head = out_head;
    a.keys = (const bf16*)keys; a.values = (const bf16*)values;
    a.k_page = k_page; a.k_head = k_head; a.k_token = k_token; a.v_page = v_page; a.v_head = v_head; a.v_token = v_token;
    a.dv = dv;
    a.page_table = page_table; a.token_request = token_request; a.cu_tokens = cu_tokens; a.ctx_lens = ctx_lens;
    a.slopes = slopes;
    a.table_width = table_width; a.n_tokens = n_tokens; a.H = H; a.KV = KV; a.page_size = page_size; a.window = window;
    a.scale = scale; a.keep_first = keep_first; a.chunk = chunk; a.softcap = softcap;
    a.key_part = key_part; a.keys1 = key_part == 2 ? (const bf16*)keys1 : nullptr; a.k1_token = k1_token; a.fresh_d0 = fresh_d0;
    a.stats = stats;
    a.sinks = sinks; a.gate = gate; a.gate_token = gate_token;
    const bool alias = key_part != 2 && values == keys && v_page == k_page && v_head == k_head && v_token == k_token;
    auto smem_for = [&](int bn, int bm = 64) { return (size_t)(bm + 2 * bn) * (dk + PAD) * 2 + (alias ? 0 : (size_t)2 * bn * (dv + PAD) * 2); };
    const bool wide = smem_for(64) <= 160 * 1024;
    size_t smem = smem_for(wide ? 64 : 32);
    if (smem > 220 * 1024) return LLM_ERR_UNSUPPORTED;
    int code;
    // many rows per key/value head (long prompt portions), values of at most 128 lanes: 128 rows a CTA
    const bool tall = wide && dv <= 128 && (long long)max_query_len * (H / KV) >= 512 && smem_for(64, 128) <= 100 * 1024;
    if (tall) {
        smem = smem_for(64, 128);
        code = dv <= 64 ? launch<64, 64, 128>(a, requests, max_query_len, splits, part_o, part_ml, smem, stream)
                        : launch<128, 64, 128>(a, requests, max_query_len, splits, part_o, part_ml, smem, stream);
    } else if (dv <= 64)
        code = wide ? launch<64, 64>(a, requests, max_query_len, splits, part_o, part_ml, smem, stream)
                    : launch<64, 32>(a, requests, max_query_len, splits, part_o, part_ml, smem, stream);
    else if (dv <= 128)
        code = wide ? launch<128, 64>(a, requests, max_query_len, splits, part_o, part_ml, smem, stream)
                    : launch<128, 32>(a, requests, max_query_len, splits, part_o, part_ml, smem, stream);
    else
        code = wide ? launch<256, 64>(a, requests, max_query_len, splits, part_o, part_ml, smem, stream)
                    : launch<256, 32>(a, requests, max_query_len, splits, part_o, part_ml, smem, stream);
    if (code != 0 || splits == 1 || out == nullptr) return code;  // no out: the partial results are what the caller wants
    const long long items = (long long)n_tokens * H;
    return launch_pdl(attention_rows_merge_kernel, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, (const float*)part_o,
                      (const float*)part_ml, (bf16*)out, out_token, out_head, n_tokens, H, dv, splits, gate, gate_token);
}

// The partial results of llm_attention_rows_mma with splits > 1 and no out (part_o, part_ml), merged, multiplied per head
// by w [H, n_out, dv] and by sigmoid(gate [n, H * n_out], row pitch ldg; null: no gate; gate_per_head: one number a head,
// gate [n, H]) -> out [n, H * n_out].  dv even.
LLM_EXPORT int llm_merge_project_gate(const float* part_o, const float* part_ml, int splits, const void* w, const void* gate,
                                      int ldg, void* out, int n_tokens, int H, int dv, int n_out, int gate_per_head, cudaStream_t stream) {
    if (n_tokens <= 0 || H <= 0) return 0;
    if (splits < 1 || splits > 32 || dv <= 0 || (dv & 1) || n_out <= 0 || ((uintptr_t)w & 3)) return LLM_ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)(dv + 32) * sizeof(float);
    return launch_pdl(merge_project_gate_kernel, dim3((unsigned)(n_tokens * H)), dim3(128), smem, stream, part_o, part_ml, splits,
                      (const bf16*)w, (const bf16*)gate, ldg, (bf16*)out, H, dv, n_out, gate_per_head);
}

// Two parts of one softmax, each normalised by itself (o [n, H, dv] bfloat16 with token and head strides, stats [n, H, 2] =
// maximum and sum), joined into out.
LLM_EXPORT int llm_merge_two_parts(const void* o1, long long o1_token, long long o1_head, const float* stats1, const void* o2,
                                   long long o2_token, long long o2_head, const float* stats2, void* out, long long out_token,
                                   long long out_head, int n_tokens, int H, int dv, cudaStream_t stream) {
    if (n_tokens <= 0 || H <= 0 || dv <= 0) return 0;
    const long long items = (long long)n_tokens * H;
    return launch_pdl(merge_two_parts_kernel, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, (const bf16*)o1, o1_token,
                      o1_head, stats1, (const bf16*)o2, o2_token, o2_head, stats2, (bf16*)out, out_token, out_head, n_tokens, H, dv);
}
