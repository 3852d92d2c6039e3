// What a token's stacked projections become before softmax attention reads them as queries, keys and values.
//
// proj row: [Hq x D queries | Hk x D keys | Hk x V values]  (Hk = 0: a layer that reads another layer's keys and values;
// values_are_keys: no value columns, a key head's value is that head as projected, bias included, before norm and
// rotation).  In this order, each step optional:
//   bias:      the stacked bias (float32, laid out like the row) is added
//   norm:      every query head and every key head is divided by sqrt(mean(x^2) + eps) over its D lanes and multiplied
//              by qw / kw [D], the same for every head
//   rotate:    lanes i and i + rot/2 (i < rot/2) of every head turn by position * freq[i]; lanes >= rot pass
//              (interleaved: lanes 2i and 2i + 1 instead)
//   values:    v_keep [N, Hk * V] (float32) takes the values as projected, bias included; or, with v_first [N, Hk * V],
//              the values become (1 - v_lambda) v + v_lambda v_first (those of the same token in an earlier layer)
//   warm:      queries times 1 + coef * ln(floor((position + 1) / every) + 1)
// Queries go to q_out [N, Hq * D]; keys and values into the token's slot of pool [pages, 2, Hk, page_size, Dp].
// Everything is computed in 32-bit.  One CTA per token, one warp per head at a time.
#include <type_traits>

#include "common.cuh"

namespace {

constexpr int WARPS = 8;

template <typename TI, typename TQ, typename TK>
__global__ void __launch_bounds__(WARPS * 32)
head_prepare_kernel(const TI* __restrict__ proj, int ldp, const float* __restrict__ bias, TQ* __restrict__ q_out, int ldq,
                    TK* __restrict__ pool, const int* __restrict__ slot_map, int page_size, int Dp, const float* __restrict__ qw,
                    const float* __restrict__ kw, float eps, int normed, const float* __restrict__ freq, int rot,
                    const int* __restrict__ positions, float warm_coef, int warm_every, int Hq, int Hk, int D, int V,
                    int values_are_keys, int interleaved, float* __restrict__ v_keep, const float* __restrict__ v_first,
                    float v_lambda) {
    extern __shared__ float smem[];  // [WARPS][D] a head as projected, then rot/2 (cos, sin) pairs
    float2* turn = reinterpret_cast<float2*>(smem + WARPS * D + ((WARPS * D) & 1));
    pdl_trigger();
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = rot >> 1;
    const int position = (half > 0 || warm_every > 0) ? positions[t] : 0;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)position * freq[i], &s, &c);
        turn[i] = make_float2(c, s);
    }
    const float warm = warm_every > 0 ? 1.f + warm_coef * logf((float)((position + 1) / warm_every) + 1.f) : 1.f;
    const int slot = Hk > 0 ? slot_map[t] : 0;
    const int page = slot / page_size, off = slot % page_size;
    __syncthreads();
    pdl_wait();
    const TI* row = proj + (size_t)t * ldp;
    float* buf = smem + warp * D;
    const int per_head = D - half;  // work items a head: `half` pairs, then the lanes that pass
    for (int head = warp; head < Hq + Hk; head += WARPS) {
        const bool is_q = head < Hq;
        const int base = head * D;  // keys follow the queries in the row and in the bias
        TK* vdst = (!is_q && values_are_keys) ? pool + ((((size_t)page * 2 + 1) * Hk + (head - Hq)) * page_size + off) * Dp : nullptr;
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) {
            float v = to_float(row[base + d]);
            if (bias) v += bias[base + d];
            buf[d] = v;
            ss = fmaf(v, v, ss);
            if (vdst) vdst[d] = from_float<TK>(v);
        }
        ss = warp_sum(ss);
        const float ns = normed ? 1.f / sqrtf(ss / (float)D + eps) : 1.f;
        const float* w = normed ? (is_q ? qw : kw) : nullptr;
        const float post = is_q ? warm : 1.f;
        __syncwarp();
        for (int i = lane; i < per_head; i += 32) {
            float a, b = 0.f;
            int da, db = -1;
            if (i < half) {
                da = interleaved ? 2 * i : i; db = interleaved ? 2 * i + 1 : i + half;
                float u = buf[da] * ns, v = buf[db] * ns;
                if (w) { u *= w[da]; v *= w[db]; }
                const float c = turn[i].x, s = turn[i].y;
                a = (u * c - v * s) * post;
                b = (v * c + u * s) * post;
            } else {
                da = i + half;
                float u = buf[da] * ns;
                if (w) u *= w[da];
                a = u * post;
            }
            if (is_q) {
                TQ* dst = q_out + (size_t)t * ldq + base;
                dst[da] = from_float<TQ>(a);
                if (db >= 0) dst[db] = from_float<TQ>(b);
            } else {
                TK* dst = pool + (((size_t)page * 2 * Hk + (head - Hq)) * page_size + off) * Dp;
                dst[da] = from_float<TK>(a);
                if (db >= 0) dst[db] = from_float<TK>(b);
            }
        }
        __syncwarp();
    }
    if (Hk > 0 && !values_are_keys) {
        const int vbase = (Hq + Hk) * D;
        for (int i = threadIdx.x; i < Hk * V; i += blockDim.x) {
            const int kh = i / V, d = i % V;
            float v = to_float(row[vbase + i]);
            if (bias) v += bias[vbase + i];
            if (v_keep) v_keep[(size_t)t * Hk * V + i] = v;
            if (v_first) v = (1.f - v_lambda) * v + v_lambda * v_first[(size_t)t * Hk * V + i];
            pool[((((size_t)page * 2 + 1) * Hk + kh) * page_size + off) * Dp + d] = from_float<TK>(v);
        }
    }
}

}  // namespace

// in_dtype: the projections' type; out_dtype: the type of the queries on their way out and of the pool.
LLM_EXPORT int llm_head_prepare(const void* proj, int in_dtype, int ldp, const float* bias, void* q_out, int ldq, void* pool,
                                int out_dtype, const int* slot_map, int page_size, int Dp, const float* qw, const float* kw, float eps,
                                int normed, const float* freq, int rot, const int* positions, float warm_coef, int warm_every, int N,
                                int Hq, int Hk, int D, int V, int values_are_keys, int interleaved, float* v_keep,
                                const float* v_first, float v_lambda, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (rot < 0 || rot % 2 || rot > D || Hq < 0 || Hk < 0 || D <= 0 || D > 1024 || (Hk > 0 && (!pool || !slot_map || Dp < D || page_size <= 0)) ||
        (Hk > 0 && !values_are_keys && (V <= 0 || Dp < V)) || ((rot > 0 || warm_every > 0) && !positions) || (rot > 0 && !freq) ||
        (normed && (!qw || (Hk > 0 && !kw))) || (Hq > 0 && !q_out) || ((v_keep || v_first) && (values_are_keys || Hk <= 0)))
        return LLM_ERR_BAD_ARGUMENT;
    using bf = __nv_bfloat16;
    const size_t smem = ((size_t)WARPS * D + 1) * sizeof(float) + (size_t)(rot / 2 + 1) * sizeof(float2);
    auto go = [&](auto kernel, auto* in, auto* qo) {
        using TK = std::remove_pointer_t<decltype(qo)>;
        return launch_pdl(kernel, dim3(N), dim3(WARPS * 32), smem, stream, in, ldp, bias, qo, ldq, (TK*)pool, slot_map, page_size, Dp, qw, kw,
                          eps, normed, freq, rot, positions, warm_coef, warm_every, Hq, Hk, D, V, values_are_keys, interleaved, v_keep, v_first, v_lambda);
    };
    if (in_dtype == LLM_F32 && out_dtype == LLM_F32) return go(head_prepare_kernel<float, float, float>, (const float*)proj, (float*)q_out);
    if (in_dtype == LLM_F32 && out_dtype == LLM_BF16) return go(head_prepare_kernel<float, bf, bf>, (const float*)proj, (bf*)q_out);
    if (in_dtype == LLM_BF16 && out_dtype == LLM_BF16) return go(head_prepare_kernel<bf, bf, bf>, (const bf*)proj, (bf*)q_out);
    return LLM_ERR_UNSUPPORTED;
}
