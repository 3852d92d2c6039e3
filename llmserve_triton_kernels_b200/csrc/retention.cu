// Retention: linear attention with one fixed decay per head and a matrix of state per (request, head).
//
//   S_t = decay_h S_(t-1) + k_t v_t^T        o_t = S_t^T q_t            S: [D, V] float32, zero when a request starts
//
// Queries, keys, values, the state and the sums are 32-bit.  Column v of S is all that o_t[v] needs, so the columns
// are shared out: a CTA owns 64 (32, 16 for longer keys) columns of one (request, head) in 16 groups, eight threads a
// group, each with D / 8 rows of the group's 4 (2, 1) columns in registers: what a thread reads of a token's q and k serves all
// of its columns (with one column a thread the shared-memory reads, not the arithmetic, set the pace).  The request's new tokens are walked in order and the slot is left with the state after the last.
//
// GATED: the same walk for linear attention whose state decays row by row, each row by a factor that the token chooses:
//
//   S_t = diag(alpha_t) S_(t-1) + k_t v_t^T        o_t = q_scale * S_t^T q_t
//   alpha_t[d] = sigmoid(z_t[d] + zbias[d]) ^ inv_tau = exp(inv_tau * log sigmoid(z_t[d] + zbias[d]))
//
// The logits z come through shared memory like q and k and are turned into decays there, once a CTA, 32-bit.
//
// Also here: the step behind it, each head's o divided by its root mean square and multiplied by a gate.
#include "common.cuh"

namespace {

constexpr int GROUPS = 16;  // groups of threads a CTA: each owns some neighbouring columns of the state
constexpr int TPC = 8;      // threads a group: each holds D / 8 rows of the group's columns

__device__ __forceinline__ void attn_cp16(float* smem, const float* gmem) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(gmem));
}

__device__ __forceinline__ float decay_of(float z, float inv_tau) {
    const float log_sigmoid = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
    return expf(inv_tau * log_sigmoid);
}

// q, k: [N, H, D] float32 (row pitches ldq, ldk); v: [N, H, V] (pitch ldv, any type); states: [slots, H, D, V]
// out: [N, H, V] float32
// The tokens come through shared memory in blocks of TB (queries and keys of the head, the CTA's 16 lanes of the
// values), the next block on its way (cp.async) while one is walked; thread (column, part) holds rows
// part * DPT .. part * DPT + DPT - 1 of its column.  Only S is carried from token to token: the sums o_t of
// neighbouring tokens overlap.
//
// Long requests are shared out over NS CTAs, each a stretch of the request's tokens (see stretch_of).  The recurrence is
// linear in S, so a stretch can be walked from a zero state: its outputs then lack decay^(t - b + 1) S_b^T q_t, where S_b is
// the state at the stretch's start b, and its end state lacks decay^(length) S_b.  Three launches: this kernel over all
// stretches (the first from the slot's state, the others from zero; end states to `ends`), retention_starts_kernel
// (the start state of every stretch, and the slot's new state), and this kernel once more with CORRECT (S = the start
// state, held still; the missing term is added to the outputs).  NS == 1: one launch, as described above.
// GATED: in place of decay^n stands, row by row, the product of the decays of the tokens passed: the CORRECT launch
// carries it along from the stretch's start, and the first launch leaves every stretch's whole product in `spans`
// [requests * NS, H, D] for retention_starts_kernel.
__device__ __forceinline__ void stretch_of(int begin, int end, int s, int NS, int& b, int& e) {
    const int length = ((end - begin + NS - 1) / NS + 7) & ~7;  // whole turns of eight tokens
    b = min(end, begin + s * length);
    e = min(end, b + length);
}

template <typename TV, int DPT, int TB, int CPT, bool CORRECT, bool GATED>
__global__ void __launch_bounds__(GROUPS * TPC)
retention_scan_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk, const TV* __restrict__ v, int ldv,
                      const float* __restrict__ decay, float* __restrict__ states, const int* __restrict__ state_slots,
                      const int* __restrict__ cu_tokens, float* __restrict__ out, int H, int D, int V, int NS,
                      float* __restrict__ ends, const float* __restrict__ starts, const float* __restrict__ z, int ldz,
                      const float* __restrict__ zbias, float inv_tau, float q_scale, float* __restrict__ spans) {
    constexpr int COLS = GROUPS * CPT;  // columns of the state a CTA owns: 16 groups of threads, CPT neighbouring columns a thread
    constexpr int DS = DPT * TPC;   // rows of the state that the CTA's registers have room for (>= D)
    constexpr int SEG = DPT + 4;    // a part's lanes of a token's q or k, then 4 floats of room: the parts' 16-byte reads fall
    constexpr int RP = SEG * TPC;   // into different banks; RP: the pitch of a token's row
    extern __shared__ __align__(16) float shared[];
    float* tile = shared;                       // [DS][COLS + 1], the state on its way in and out
    float* sq = tile + DS * (COLS + 1) + (4 - (DS * (COLS + 1)) % 4) % 4;  // [2][TB][RP], on a 16-byte boundary
    float* sk = sq + 2 * TB * RP;               // [2][TB][RP]
    float* sv = sk + 2 * TB * RP;               // [2][TB][COLS]
    float* sa = sv + 2 * TB * COLS;             // [2][TB][RP] (GATED): the decays' logits, then the decays
    pdl_trigger();
    const int r = blockIdx.z / NS, stretch = blockIdx.z % NS, h = blockIdx.y, v0 = blockIdx.x * COLS;
    const int sub = threadIdx.x % TPC, c0 = (threadIdx.x / TPC) * CPT;  // the thread's first column within the CTA's
    if (CORRECT && stretch == 0) return;  // the first stretch started from the true state
    int begin, end;
    stretch_of(cu_tokens[r], cu_tokens[r + 1], stretch, NS, begin, end);
    const int slot = state_slots[r];
    const float gamma = GATED ? 1.f : decay[h];
    const float log2_gamma = GATED ? 0.f : log2f(gamma);
    // where the state comes from and goes to
    const size_t per_head = (size_t)D * V;
    const float* state_in = CORRECT ? starts + ((size_t)(r * NS + stretch) * H + h) * per_head
                                    : (stretch == 0 ? states + ((size_t)slot * H + h) * per_head : nullptr);
    float* state_out = CORRECT ? nullptr : (NS > 1 ? ends + ((size_t)(r * NS + stretch) * H + h) * per_head : states + ((size_t)slot * H + h) * per_head);
    if (CORRECT && begin >= end) return;
    const bool vec = (D % 4 == 0) && (ldq % 4 == 0) && (ldk % 4 == 0) && ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k)) % 16 == 0) &&
                     (!GATED || (ldz % 4 == 0 && reinterpret_cast<uintptr_t>(z) % 16 == 0));  // rows of q and k (and z) may be copied 16 bytes at a time
    pdl_wait();

    const bool vec_v = sizeof(TV) == 4 && V % 4 == 0 && ldv % 4 == 0 && reinterpret_cast<uintptr_t>(v) % 16 == 0 && v0 + COLS <= V;
    auto fetch = [&](int t0, int buf) {
        const int count = min(TB, end - t0);
        if (vec) {
            const int chunks = D / 4;
            for (int i = threadIdx.x; i < count * chunks; i += blockDim.x) {
                const int tt = i / chunks, d = (i % chunks) * 4;
                const int at = (d / DPT) * SEG + d % DPT;
                attn_cp16(sq + ((size_t)buf * TB + tt) * RP + at, q + (size_t)(t0 + tt) * ldq + (size_t)h * D + d);
                if (!CORRECT) attn_cp16(sk + ((size_t)buf * TB + tt) * RP + at, k + (size_t)(t0 + tt) * ldk + (size_t)h * D + d);
                if (GATED) attn_cp16(sa + ((size_t)buf * TB + tt) * RP + at, z + (size_t)(t0 + tt) * ldz + (size_t)h * D + d);
            }
        } else {
            for (int i = threadIdx.x; i < count * D; i += blockDim.x) {
                const int tt = i / D, d = i % D;
                const int at = (d / DPT) * SEG + d % DPT;
                sq[((size_t)buf * TB + tt) * RP + at] = q[(size_t)(t0 + tt) * ldq + (size_t)h * D + d];
                if (!CORRECT) sk[((size_t)buf * TB + tt) * RP + at] = k[(size_t)(t0 + tt) * ldk + (size_t)h * D + d];
                if (GATED) sa[((size_t)buf * TB + tt) * RP + at] = z[(size_t)(t0 + tt) * ldz + (size_t)h * D + d];
            }
        }
        if (CORRECT) {
        } else if (vec_v) {  // the CTA's lanes of a token's values in copies of 16 bytes, in flight with the rest
            for (int i = threadIdx.x; i < count * (COLS / 4); i += blockDim.x) {
                const int tt = i / (COLS / 4), c = (i % (COLS / 4)) * 4;
                attn_cp16(sv + ((size_t)buf * TB + tt) * COLS + c, reinterpret_cast<const float*>(v) + (size_t)(t0 + tt) * ldv + (size_t)h * V + v0 + c);
            }
        } else {
            for (int i = threadIdx.x; i < count * COLS; i += blockDim.x) {
                const int tt = i / COLS, c = i % COLS;
                sv[((size_t)buf * TB + tt) * COLS + c] = v0 + c < V ? to_float(v[(size_t)(t0 + tt) * ldv + (size_t)h * V + v0 + c]) : 0.f;
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };

    if (begin < end) fetch(begin, 0);
    // lanes of q and k beyond D (the registers' room is a multiple of 8 * DPT) are zeros in both buffers
    for (int i = threadIdx.x; i < 2 * TB * (DS - D); i += blockDim.x) {
        const int row = i / (DS - D), d = D + i % (DS - D);
        const int at = (d / DPT) * SEG + d % DPT;
        sq[(size_t)row * RP + at] = 0.f;
        sk[(size_t)row * RP + at] = 0.f;
        if (GATED) sa[(size_t)row * RP + at] = 0.f;
    }
    for (int i = threadIdx.x; i < D * COLS; i += blockDim.x) {
        const int d = i / COLS, c = i % COLS;
        tile[d * (COLS + 1) + c] = (state_in && v0 + c < V) ? state_in[(size_t)d * V + v0 + c] : 0.f;
    }
    __syncthreads();
    float S[CPT][DPT];
#pragma unroll
    for (int c = 0; c < CPT; ++c)
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = sub * DPT + i;
            S[c][i] = d < D ? tile[d * (COLS + 1) + c0 + c] : 0.f;
        }
    // the thread's columns that exist, and whether its outputs of a token may be stored 16 bytes at a time
    const int live = max(0, min(CPT, V - (v0 + c0)));
    const bool wide_out = CPT == 4 && live == 4 && V % 4 == 0;
    // one token: the state moves on (not when CORRECT) and acc[c] takes this thread's share of o_t[column c]
    // GATED: the product of the decays since the stretch's start, for this thread's rows.  The CORRECT launch weighs the
    // start state by it; in the first launch the threads of the first group of a head's first CTA keep it for `spans`.
    float cum[GATED ? DPT : 1];
#pragma unroll
    for (int i = 0; i < (GATED ? DPT : 1); ++i) cum[i] = 1.f;
    const bool keeps_span = GATED && !CORRECT && NS > 1 && blockIdx.x == 0 && threadIdx.x < TPC;
    auto token = [&](const float* bq, const float* bk, const float* bv, const float* ba, float (&acc)[CPT]) {
        float vt[CPT];
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            vt[c] = CORRECT ? 0.f : bv[c];
            acc[c] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < DPT; i += 4) {
            const float4 q4 = *reinterpret_cast<const float4*>(bq + i);
            float qv[4] = {q4.x, q4.y, q4.z, q4.w};
            float kv[4] = {0.f, 0.f, 0.f, 0.f};
            float av[4] = {gamma, gamma, gamma, gamma};
            if (!CORRECT) {
                const float4 k4 = *reinterpret_cast<const float4*>(bk + i);
                kv[0] = k4.x; kv[1] = k4.y; kv[2] = k4.z; kv[3] = k4.w;
            }
            if constexpr (GATED) {
                const float4 a4 = *reinterpret_cast<const float4*>(ba + i);
                av[0] = a4.x; av[1] = a4.y; av[2] = a4.z; av[3] = a4.w;
                if (CORRECT || keeps_span) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) cum[i + j] *= av[j];
                }
                if (CORRECT) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) qv[j] *= cum[i + j];
                }
            }
#pragma unroll
            for (int c = 0; c < CPT; ++c)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (!CORRECT) S[c][i + j] = fmaf(av[j], S[c][i + j], kv[j] * vt[c]);
                    acc[c] = fmaf(S[c][i + j], qv[j], acc[c]);
                }
        }
    };
    auto store = [&](int t, const float (&total)[CPT]) {
        float* at = out + ((size_t)t * H + h) * V + v0 + c0;
        const float f = GATED ? q_scale : CORRECT ? exp2f((float)(t - begin + 1) * log2_gamma) : 0.f;
        if (wide_out) {
            float4 o = make_float4(total[0], total[1], total[2], total[3]);
            if (GATED && !CORRECT) o = make_float4(o.x * f, o.y * f, o.z * f, o.w * f);
            if (CORRECT) {
                const float4 b4 = *reinterpret_cast<const float4*>(at);
                o = make_float4(fmaf(o.x, f, b4.x), fmaf(o.y, f, b4.y), fmaf(o.z, f, b4.z), fmaf(o.w, f, b4.w));
            }
            *reinterpret_cast<float4*>(at) = o;
        } else {
#pragma unroll
            for (int c = 0; c < CPT; ++c)
                if (c < live) at[c] = CORRECT ? fmaf(total[c], f, at[c]) : GATED ? total[c] * f : total[c];
        }
    };
    int buf = 0;
    for (int t0 = begin; t0 < end; t0 += TB, buf ^= 1) {
        asm volatile("cp.async.wait_group 0;\n" ::);
        __syncthreads();  // this block has landed, and everybody has left the other buffer
        if (t0 + TB < end) fetch(t0 + TB, buf ^ 1);
        const int count = min(TB, end - t0);
        if (GATED) {  // the block's logits become its decays
            for (int i = threadIdx.x; i < count * D; i += blockDim.x) {
                const int tt = i / D, d = i % D;
                float* at = sa + ((size_t)buf * TB + tt) * RP + (d / DPT) * SEG + d % DPT;
                *at = decay_of(*at + (zbias ? zbias[h * D + d] : 0.f), inv_tau);
            }
            __syncthreads();
        }
        const float* bq = sq + (size_t)buf * TB * RP + sub * SEG;
        const float* bk = sk + (size_t)buf * TB * RP + sub * SEG;
        const float* bv = sv + (size_t)buf * TB * COLS + c0;
        const float* ba = sa + (size_t)buf * TB * RP + sub * SEG;
        int tt = 0;
        // eight tokens at a time: their partial sums are independent chains, and the eight lanes of a column then
        // trade halves (4, 2, 1 values) so that lane `sub` ends with the whole sums of token tt + sub: 7 shuffles a
        // column for 8 tokens, and every lane stores one token's columns
        for (; tt + 8 <= count; tt += 8) {
            float o[8][CPT];
#pragma unroll
            for (int u = 0; u < 8; ++u) token(bq + (size_t)(tt + u) * RP, bk + (size_t)(tt + u) * RP, bv + (size_t)(tt + u) * COLS, ba + (size_t)(tt + u) * RP, o[u]);
            const bool h4 = sub & 4, h2 = sub & 2, h1 = sub & 1;
            float total[CPT];
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                float a[4], b[2];
#pragma unroll
                for (int u = 0; u < 4; ++u) a[u] = (h4 ? o[u + 4][c] : o[u][c]) + __shfl_xor_sync(0xffffffffu, h4 ? o[u][c] : o[u + 4][c], 4);
#pragma unroll
                for (int u = 0; u < 2; ++u) b[u] = (h2 ? a[u + 2] : a[u]) + __shfl_xor_sync(0xffffffffu, h2 ? a[u] : a[u + 2], 2);
                total[c] = (h1 ? b[1] : b[0]) + __shfl_xor_sync(0xffffffffu, h1 ? b[0] : b[1], 1);
            }
            store(t0 + tt + sub, total);
        }
        for (; tt < count; ++tt) {
            float acc[CPT];
            token(bq + (size_t)tt * RP, bk + (size_t)tt * RP, bv + (size_t)tt * COLS, ba + (size_t)tt * RP, acc);
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 4);  // the order of the turns of eight: a token's sum has the same
                acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 2);  // bits wherever a step's cut puts it
                acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 1);
            }
            if (sub == 0) store(t0 + tt, acc);
        }
    }
    if (CORRECT) return;
    if constexpr (GATED) if (keeps_span) {
#pragma unroll
        for (int i = 0; i < DPT; ++i)
            if (sub * DPT + i < D) spans[((size_t)(r * NS + stretch) * H + h) * D + sub * DPT + i] = cum[i];
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < CPT; ++c)
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = sub * DPT + i;
            if (d < D) tile[d * (COLS + 1) + c0 + c] = S[c][i];
        }
    __syncthreads();
    for (int i = threadIdx.x; i < D * COLS; i += blockDim.x) {
        const int d = i / COLS, c = i % COLS;
        if (v0 + c < V) state_out[(size_t)d * V + v0 + c] = tile[d * (COLS + 1) + c];
    }
}

// From the stretches' end states (the first from the true state, the others from zero) to the state at every stretch's
// start and the slot's new state:  start_1 = end_0;  start_(s+1) = decay^(length_s) start_s + end_s.  One thread an element.
// `spans` [requests * NS, H, D] (or null): row by row, what stands in place of decay^(length_s) where every token chose its decays.
__global__ void __launch_bounds__(256)
retention_starts_kernel(const float* __restrict__ ends, float* __restrict__ starts, float* __restrict__ states,
                        const float* __restrict__ decay, const int* __restrict__ state_slots, const int* __restrict__ cu_tokens, int H,
                        int per_head, int NS, const float* __restrict__ spans, int V) {
    pdl_trigger();
    const int r = blockIdx.z, h = blockIdx.y, i = blockIdx.x * blockDim.x + threadIdx.x;
    const float log2_gamma = spans ? 0.f : log2f(decay[h]);
    const int t_begin = cu_tokens[r], t_end = cu_tokens[r + 1], slot = state_slots[r];
    pdl_wait();
    if (i >= per_head) return;
    float S = ends[((size_t)(r * NS) * H + h) * per_head + i];
    for (int s = 1; s < NS; ++s) {
        starts[((size_t)(r * NS + s) * H + h) * per_head + i] = S;
        int b, e;
        stretch_of(t_begin, t_end, s, NS, b, e);
        const float over = spans ? spans[((size_t)(r * NS + s) * H + h) * (per_head / V) + i / V] : e > b ? exp2f((float)(e - b) * log2_gamma) : 1.f;
        S = fmaf(over, S, ends[((size_t)(r * NS + s) * H + h) * per_head + i]);
    }
    states[((size_t)slot * H + h) * per_head + i] = S;
}

// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * gate(g[t, h, :]), one warp per (token, head).
// gate_kind: 0 sigmoid(g), 1 silu(g), -1 none.  eps < 0: no norm.  weight [V] (or null): the normed lanes times it, the
// same for every head.
template <typename TG, typename TO>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, const TG* __restrict__ g, int ldg, TO* __restrict__ out, int rows, int heads,
                      int V, float eps, int gate_kind, const float* __restrict__ weight) {
    pdl_trigger();
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    pdl_wait();
    if (row >= rows) return;
    const int t = row / heads, h = row % heads;
    const float* src = o + (size_t)row * V;
    float ss = 0.f;
    for (int i = lane; i < V; i += 32) ss = fmaf(src[i], src[i], ss);
    ss = warp_sum(ss);
    const float scale = eps >= 0.f ? 1.f / sqrtf(ss / (float)V + eps) : 1.f;
    for (int i = lane; i < V; i += 32) {
        float y = src[i] * scale;
        if (weight) y *= weight[i];
        if (gate_kind >= 0) {
            const float z = to_float(g[(size_t)t * ldg + (size_t)h * V + i]);
            const float s = 1.f / (1.f + expf(-z));
            y *= gate_kind == 1 ? z * s : s;
        }
        out[(size_t)row * V + i] = from_float<TO>(y);
    }
}

}  // namespace

namespace {

// Both scans: `decay` [H] and no `z` (one fixed decay a head), or `z` [N, H * D] with `zbias`, `inv_tau`, `q_scale` (GATED).
// `scratch` (stretches > 1): requests * stretches * H * (2 * D * V + D) floats: end states, start states, the stretches' products.
int scan_launch(bool gated, const float* q, int ldq, const float* k, int ldk, const void* v, int v_dtype, int ldv, const float* decay,
                const float* z, int ldz, const float* zbias, float inv_tau, float q_scale, float* states, const int* state_slots,
                const int* cu_tokens, float* out, int requests, int H, int D, int V, int stretches, float* scratch, int few_tokens,
                cudaStream_t stream) {
    if (requests <= 0) return 0;
    if (H <= 0 || D <= 0 || V <= 0 || D > 256 || H > 65535 || stretches < 1 || (stretches > 1 && !scratch) || (long long)requests * stretches > 65535)
        return LLM_ERR_BAD_ARGUMENT;
    if (v_dtype != LLM_F32 && v_dtype != LLM_BF16) return LLM_ERR_BAD_ARGUMENT;
    const int NS = stretches;
    // steps of few tokens a request (decode steps) move the state more than they compute: 16 columns a CTA, more CTAs
    const int cpt = few_tokens ? 1 : D <= 64 ? 4 : D <= 128 ? 2 : 1, cols = GROUPS * cpt;
    const dim3 grid((V + cols - 1) / cols, H, requests * NS), block(GROUPS * TPC);
    float* ends = scratch;
    float* starts = scratch ? scratch + (size_t)requests * NS * H * D * V : nullptr;
    float* spans = scratch && gated ? starts + (size_t)requests * NS * H * D * V : nullptr;
    using bf = __nv_bfloat16;
    auto go = [&](auto kernel, auto* vp, int dpt, int tb) -> int {
        const int ds = dpt * TPC;
        const size_t smem = ((size_t)ds * (cols + 1) + 4 + (size_t)(gated ? 6 : 4) * tb * (dpt + 4) * TPC + (size_t)2 * tb * cols) * sizeof(float);
        if (smem > 48 * 1024) {
            const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        return launch_pdl(kernel, grid, block, smem, stream, q, ldq, k, ldk, vp, ldv, decay, states, state_slots, cu_tokens, out, H, D, V, NS, ends,
                          (const float*)starts, z, ldz, zbias, inv_tau, q_scale, spans);
    };
#define LLM_RET2(DPT, TB, CPT, C, G) \
    (v_dtype == LLM_F32 ? go(retention_scan_kernel<float, DPT, TB, CPT, C, G>, (const float*)v, DPT, TB) : go(retention_scan_kernel<bf, DPT, TB, CPT, C, G>, (const bf*)v, DPT, TB))
#define LLM_RET(C, G, TBS)                                                                                                                  \
    (few_tokens ? (D <= 32 ? LLM_RET2(4, TBS, 1, C, G) : D <= 64 ? LLM_RET2(8, TBS, 1, C, G) : D <= 128 ? LLM_RET2(16, 16, 1, C, G) : LLM_RET2(32, 8, 1, C, G)) \
                : (D <= 32 ? LLM_RET2(4, TBS, 4, C, G) : D <= 64 ? LLM_RET2(8, TBS, 4, C, G) : D <= 128 ? LLM_RET2(16, 16, 2, C, G) : LLM_RET2(32, 8, 1, C, G)))
    int code = gated ? LLM_RET(false, true, 16) : LLM_RET(false, false, 32);
    if (code != 0 || NS == 1) return code;
    const int per_head = D * V;
    code = launch_pdl(retention_starts_kernel, dim3((per_head + 255) / 256, H, requests), dim3(256), 0, stream, (const float*)ends, starts, states, decay,
                      state_slots, cu_tokens, H, per_head, NS, (const float*)spans, V);
    if (code != 0) return code;
    return gated ? LLM_RET(true, true, 16) : LLM_RET(true, false, 32);
#undef LLM_RET
#undef LLM_RET2
}

}  // namespace

// `few_tokens`: no request brings more than a few tokens.  `stretches` > 1: long requests shared out over that many CTAs each; `scratch` then holds 2 * requests * stretches * H * D * V floats.
LLM_EXPORT int llm_retention_scan(const float* q, int ldq, const float* k, int ldk, const void* v, int v_dtype, int ldv,
                                  const float* decay, float* states, const int* state_slots, const int* cu_tokens, float* out,
                                  int requests, int H, int D, int V, int stretches, float* scratch, int few_tokens, cudaStream_t stream) {
    return scan_launch(false, q, ldq, k, ldk, v, v_dtype, ldv, decay, nullptr, 0, nullptr, 0.f, 1.f, states, state_slots, cu_tokens, out, requests,
                       H, D, V, stretches, scratch, few_tokens, stream);
}

// The scan whose decays every token chooses: z [N, H * D] float32 (pitch ldz), zbias [H * D] float32 or null; out = q_scale * S^T q.
// `scratch` (stretches > 1) holds requests * stretches * H * (2 * D * V + D) floats.
LLM_EXPORT int llm_gated_scan(const float* q, int ldq, const float* k, int ldk, const void* v, int v_dtype, int ldv, const float* z,
                              int ldz, const float* zbias, float inv_tau, float q_scale, float* states, const int* state_slots,
                              const int* cu_tokens, float* out, int requests, int H, int D, int V, int stretches, float* scratch,
                              int few_tokens, cudaStream_t stream) {
    if (!z) return LLM_ERR_BAD_ARGUMENT;
    return scan_launch(true, q, ldq, k, ldk, v, v_dtype, ldv, nullptr, z, ldz, zbias, inv_tau, q_scale, states, state_slots, cu_tokens, out, requests,
                       H, D, V, stretches, scratch, few_tokens, stream);
}

LLM_EXPORT int llm_head_norm_gate(const float* o, const void* g, int g_dtype, int ldg, void* out, int out_dtype, int N, int heads,
                                  int V, float eps, int gate_kind, const float* weight, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (heads <= 0 || V <= 0 || (gate_kind >= 0 && !g)) return LLM_ERR_BAD_ARGUMENT;
    const int rows = N * heads;
    const dim3 grid((rows + 3) / 4), block(128);
    using bf = __nv_bfloat16;
    auto go = [&](auto kernel, auto* gp, auto* op) { return launch_pdl(kernel, grid, block, 0, stream, o, gp, ldg, op, rows, heads, V, eps, gate_kind, weight); };
    if (g_dtype == LLM_F32 && out_dtype == LLM_F32) return go(head_norm_gate_kernel<float, float>, (const float*)g, (float*)out);
    if (g_dtype == LLM_F32 && out_dtype == LLM_BF16) return go(head_norm_gate_kernel<float, bf>, (const float*)g, (bf*)out);
    if (g_dtype == LLM_BF16 && out_dtype == LLM_BF16) return go(head_norm_gate_kernel<bf, bf>, (const bf*)g, (bf*)out);
    return LLM_ERR_UNSUPPORTED;
}
