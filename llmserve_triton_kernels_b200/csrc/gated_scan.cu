// Linear attention whose state decays row by row, each row by a factor that the token chooses:
//
//     S_t = diag(alpha_t) S_(t-1) + k_t v_t^T        o_t = S_t^T (q_scale * q_t)        per head, S [D, V]
//     alpha_t[d] = sigmoid(z_t[d] + zbias[d]) ^ inv_tau = exp(inv_tau * log sigmoid(z_t[d] + zbias[d]))
//
// S is float32 in the request's slot of `states` [slots, H, D, V]; it is read at the start of the request's new tokens
// and written back behind them.  Decays, their logarithms, the state and the sums are 32-bit.  The recurrence is walked
// token by token, so the result does not depend on how a request's tokens were cut into steps.
//
// A CTA owns 16 * CPT columns of one (request, head): 16 groups of 8 threads; the 8 threads of a group share the D rows
// (thread g holds rows g, g + 8, ...) of CPT neighbouring columns in registers and sum their shares of o_t by shuffles.
// Tokens come through shared memory in blocks (the decays are worked out as a block is staged).
#include "common.cuh"

namespace {

constexpr int GROUPS = 16, TPC = 8;  // column groups a CTA, threads a group

__device__ __forceinline__ float decay_of(float z, float inv_tau) {
    const float log_sigmoid = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
    return expf(inv_tau * log_sigmoid);
}

template <typename TV, int DPT, int CPT>
__global__ void __launch_bounds__(GROUPS * TPC)
gated_scan_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk, const TV* __restrict__ v, int ldv,
                  const float* __restrict__ z, int ldz, const float* __restrict__ zbias, float inv_tau, float q_scale,
                  float* __restrict__ states, const int* __restrict__ state_slots, const int* __restrict__ cu_tokens,
                  float* __restrict__ out, int H, int D, int V, int TB) {
    constexpr int COLS = GROUPS * CPT;
    extern __shared__ float smem[];
    float* qs = smem;             // [TB][D]
    float* ks = qs + TB * D;      // [TB][D]
    float* as = ks + TB * D;      // [TB][D]
    float* vs = as + TB * D;      // [TB][COLS]
    pdl_trigger();
    const int r = blockIdx.z, h = blockIdx.y, col0 = blockIdx.x * COLS;
    const int grp = threadIdx.x / TPC, g = threadIdx.x % TPC;
    const int begin = cu_tokens[r], end = cu_tokens[r + 1];
    const int slot = state_slots[r];
    pdl_wait();
    float S[DPT][CPT];
    float* sp = states + ((size_t)slot * H + h) * D * V;
#pragma unroll
    for (int j = 0; j < DPT; ++j)
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            const int d = g + TPC * j, col = col0 + grp * CPT + c;
            S[j][c] = (d < D && col < V) ? sp[(size_t)d * V + col] : 0.f;
        }
    for (int t0 = begin; t0 < end; t0 += TB) {
        const int nt = min(TB, end - t0);
        __syncthreads();  // the block before has been read
        for (int i = threadIdx.x; i < nt * D; i += blockDim.x) {
            const int tt = i / D, d = i - tt * D;
            const size_t t = (size_t)(t0 + tt);
            qs[i] = q[t * ldq + h * D + d] * q_scale;
            ks[i] = k[t * ldk + h * D + d];
            as[i] = decay_of(z[t * ldz + h * D + d] + (zbias ? zbias[h * D + d] : 0.f), inv_tau);
        }
        for (int i = threadIdx.x; i < nt * COLS; i += blockDim.x) {
            const int tt = i / COLS, c = i - tt * COLS;
            vs[i] = col0 + c < V ? to_float(v[(size_t)(t0 + tt) * ldv + h * V + col0 + c]) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            float vc[CPT], acc[CPT];
#pragma unroll
            for (int c = 0; c < CPT; ++c) { vc[c] = vs[tt * COLS + grp * CPT + c]; acc[c] = 0.f; }
#pragma unroll
            for (int j = 0; j < DPT; ++j) {
                const int d = g + TPC * j;
                if (d < D) {
                    const float a = as[tt * D + d], kk = ks[tt * D + d], qq = qs[tt * D + d];
#pragma unroll
                    for (int c = 0; c < CPT; ++c) {
                        S[j][c] = fmaf(a, S[j][c], kk * vc[c]);
                        acc[c] = fmaf(S[j][c], qq, acc[c]);
                    }
                }
            }
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 1);
                acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 2);
                acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 4);
                const int col = col0 + grp * CPT + c;
                if (g == 0 && col < V) out[((size_t)(t0 + tt) * H + h) * V + col] = acc[c];
            }
        }
    }
#pragma unroll
    for (int j = 0; j < DPT; ++j)
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            const int d = g + TPC * j, col = col0 + grp * CPT + c;
            if (d < D && col < V) sp[(size_t)d * V + col] = S[j][c];
        }
}

}  // namespace

// q, k, z [N, H * D] float32 (row pitches ldq, ldk, ldz); v [N, H * V] of v_dtype (pitch ldv); zbias [H * D] float32 or null;
// out [N, H, V] float32.  `few_tokens`: no request brings more than a few tokens (a decode step): narrow CTAs, more of them.
LLM_EXPORT int llm_gated_scan(const float* q, int ldq, const float* k, int ldk, const void* v, int v_dtype, int ldv, const float* z,
                              int ldz, const float* zbias, float inv_tau, float q_scale, float* states, const int* state_slots,
                              const int* cu_tokens, float* out, int requests, int H, int D, int V, int few_tokens, cudaStream_t stream) {
    if (requests <= 0) return 0;
    if (H <= 0 || D <= 0 || V <= 0 || D > 256 || H > 65535 || requests > 65535) return LLM_ERR_BAD_ARGUMENT;
    const int cpt = few_tokens ? 1 : D <= 128 ? 4 : 2, cols = GROUPS * cpt;
    const int tb = few_tokens ? 4 : D <= 128 ? 16 : 8;
    const dim3 grid((V + cols - 1) / cols, H, requests), block(GROUPS * TPC);
    const size_t smem = (size_t)tb * (3 * D + cols) * sizeof(float);
    using bf = __nv_bfloat16;
    auto go = [&](auto kernel, auto* vp) -> int {
        if (smem > 48 * 1024) {
            const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        return launch_pdl(kernel, grid, block, smem, stream, q, ldq, k, ldk, vp, ldv, z, ldz, zbias, inv_tau, q_scale, states, state_slots,
                          cu_tokens, out, H, D, V, tb);
    };
#define LLM_GS2(DPT, CPT) \
    (v_dtype == LLM_F32 ? go(gated_scan_kernel<float, DPT, CPT>, (const float*)v) : go(gated_scan_kernel<bf, DPT, CPT>, (const bf*)v))
#define LLM_GS(CPT) (D <= 32 ? LLM_GS2(4, CPT) : D <= 64 ? LLM_GS2(8, CPT) : D <= 128 ? LLM_GS2(16, CPT) : LLM_GS2(32, CPT))
    if (v_dtype != LLM_F32 && v_dtype != LLM_BF16) return LLM_ERR_BAD_ARGUMENT;
    if (cpt == 1) return LLM_GS(1);
    if (cpt == 2) return LLM_GS(2);
    return D <= 32 ? LLM_GS2(4, 4) : D <= 64 ? LLM_GS2(8, 4) : LLM_GS2(16, 4);
#undef LLM_GS
#undef LLM_GS2
}
