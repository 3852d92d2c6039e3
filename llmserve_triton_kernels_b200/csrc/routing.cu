// A router that picks a few of many small feed-forward layers per token, the step that applies its weights, and
// the meeting of mixers that run side by side.
//
// The router's scores, the choice and the weights are 32-bit.
#include "common.cuh"

#include <float.h>

namespace {

// One warp per token.  z: [N, ldz] float32 router logits (the first E of a row; column E, if there is a shared gate,
// holds its logit).
//   s = softmax(z[0:E]);   chosen = the `top` experts with the largest s + correction (lowest index among equals)
//   w[t, e] = scale * s[e] (divided by the chosen scores' sum if renorm) for chosen experts, 0 for the others
//   w[t, E] = sigmoid(z[t, E]) if shared_gate
// w: [N, E + shared_gate] float32
// One warp: from a token's logits zr[0 : E (+ 1)] to its row of weights wr; s, c: E floats of scratch each.
// bias (or null): added to the logits of the E experts first.  shared_gate 2: w[t, E] = 1 (a shared expert without a gate; z has no column E).
__device__ __forceinline__ void route_row(const float* zr, const float* __restrict__ correction, float* wr, float* s, float* c, int E, int top,
                                          float scale, int renorm, int shared_gate, int lane, const float* __restrict__ bias = nullptr) {
    float m = -FLT_MAX;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, zr[e] + (bias ? bias[e] : 0.f));
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
        const float x = expf(zr[e] + (bias ? bias[e] : 0.f) - m);
        s[e] = x;
        sum += x;
    }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
    for (int e = lane; e < E; e += 32) {
        s[e] *= inv;
        c[e] = s[e] + (correction ? correction[e] : 0.f);
        wr[e] = 0.f;
    }
    __syncwarp();
    float chosen_sum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -FLT_MAX;
        int arg = 0x7fffffff;
        for (int e = lane; e < E; e += 32)
            if (c[e] > best) { best = c[e]; arg = e; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg < E) {
            if (lane == 0) {
                c[arg] = -FLT_MAX;
                wr[arg] = -1.f;  // marked; its weight follows
            }
            chosen_sum += s[arg];
        }
        __syncwarp();
    }
    const float f = renorm ? scale / chosen_sum : scale;
    for (int e = lane; e < E; e += 32)
        if (wr[e] < 0.f) wr[e] = s[e] * f;
    if (shared_gate && lane == 0) wr[E] = shared_gate == 2 ? 1.f : 1.f / (1.f + expf(-zr[E]));
}

__global__ void __launch_bounds__(128)
route_topk_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ correction, float* __restrict__ w, int N, int E,
                  int top, float scale, int renorm, int shared_gate) {
    extern __shared__ float sm[];  // per warp: s[E], choice[E]
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    float* s = sm + (size_t)warp * 2 * E;
    pdl_wait();
    if (t >= N) return;
    route_row(z + (size_t)t * ldz, correction, w + (size_t)t * (E + shared_gate), s, s + E, E, top, scale, renorm, shared_gate, lane);
}

// The router's product and the choice in one kernel.  x: [N, K] (any type, read as 32-bit); wr: [E (+ 1), K] float32 (the last
// row, if there is a shared gate, is the gate's); a CTA takes TT tokens (1 or 2): a warp sums up the logits of four rows at a time for all of
// them (a lane its share of the elements, then the lanes' sums: the same order whatever else is in the step), then a warp per token
// chooses.
template <typename TX, int TT>
__global__ void __launch_bounds__(512)
router_kernel(const TX* __restrict__ x, int ldx, const float* __restrict__ wr, const float* __restrict__ correction, float* __restrict__ out,
              int N, int K, int E, int top, float scale, int renorm, int shared_gate, const float* __restrict__ bias) {
    constexpr int RPW = 4;  // rows of the router matrix a warp sums up at once: what it reads of the tokens serves all four
    extern __shared__ float sm[];  // z[TT][rows], then per token s[E], c[E]
    pdl_trigger();
    const int rows = E + (shared_gate == 1), out_w = E + (shared_gate != 0), t0 = blockIdx.x * TT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    float* z = sm;
    pdl_wait();
    // four elements a lane and turn where rows allow 16-byte (weights) and 4-element (x) loads; the lanes' order of sums is fixed
    const bool wide = K % 4 == 0 && ldx % 4 == 0 && reinterpret_cast<uintptr_t>(wr) % 16 == 0 && reinterpret_cast<uintptr_t>(x) % (4 * sizeof(TX)) == 0;
    for (int e0 = warp * RPW; e0 < rows; e0 += warps * RPW) {
        float acc[RPW][TT];
#pragma unroll
        for (int r = 0; r < RPW; ++r)
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) acc[r][tt] = 0.f;
        const float* w[RPW];
        const TX* xr[TT];
#pragma unroll
        for (int r = 0; r < RPW; ++r) w[r] = wr + (size_t)min(e0 + r, rows - 1) * K;  // rows beyond the last read the last one's; not stored
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) xr[tt] = x + (size_t)min(t0 + tt, N - 1) * ldx;
        if (wide) {
#pragma unroll(TT == 1 ? 4 : 2)
            for (int k = lane * 4; k < K; k += 128) {
                float4 wv[RPW];
                float xv[TT][4];
#pragma unroll
                for (int r = 0; r < RPW; ++r) wv[r] = *reinterpret_cast<const float4*>(w[r] + k);
#pragma unroll
                for (int tt = 0; tt < TT; ++tt) load4(xr[tt] + k, xv[tt]);
#pragma unroll
                for (int r = 0; r < RPW; ++r)
#pragma unroll
                    for (int tt = 0; tt < TT; ++tt) {
                        acc[r][tt] = fmaf(wv[r].x, xv[tt][0], acc[r][tt]);
                        acc[r][tt] = fmaf(wv[r].y, xv[tt][1], acc[r][tt]);
                        acc[r][tt] = fmaf(wv[r].z, xv[tt][2], acc[r][tt]);
                        acc[r][tt] = fmaf(wv[r].w, xv[tt][3], acc[r][tt]);
                    }
            }
        } else {
#pragma unroll 2
            for (int k = lane; k < K; k += 32) {
                float wv[RPW], xv[TT];
#pragma unroll
                for (int r = 0; r < RPW; ++r) wv[r] = w[r][k];
#pragma unroll
                for (int tt = 0; tt < TT; ++tt) xv[tt] = to_float(xr[tt][k]);
#pragma unroll
                for (int r = 0; r < RPW; ++r)
#pragma unroll
                    for (int tt = 0; tt < TT; ++tt) acc[r][tt] = fmaf(wv[r], xv[tt], acc[r][tt]);
            }
        }
#pragma unroll
        for (int r = 0; r < RPW; ++r)
#pragma unroll
            for (int tt = 0; tt < TT; ++tt) {
                const float v = warp_sum(acc[r][tt]);
                if (lane == 0 && e0 + r < rows) z[tt * rows + e0 + r] = v;
            }
    }
    __syncthreads();
    if (warp < TT && t0 + warp < N) {
        float* s = sm + (size_t)TT * rows + (size_t)warp * 2 * E;
        route_row(z + warp * rows, correction, out + (size_t)(t0 + warp) * out_w, s, s + E, E, top, scale, renorm, shared_gate, lane, bias);
    }
}

__device__ __forceinline__ float activate(float v, int kind) {
    if (kind == 0) { const float r = fmaxf(v, 0.f); return r * r; }                                                // relu^2
    if (kind == 1) return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));              // gelu (tanh)
    if (kind == 3) return v / (1.f + expf(-v));                                                                    // silu
    return v;
}

// y[t, j] = act(x[t, j]) * w[t, block(j)]: block(j) = j / ff for j < E * ff, and E for the columns behind them (a
// shared expert's).  x, y: [N, C].  In two forms: 16 bytes a thread, where every run of 16 bytes lies within one expert's
// block (ff a multiple of the run) and rows start on 16-byte boundaries; element by element elsewhere.
template <typename T>
__global__ void __launch_bounds__(256)
expert_act_scale_wide_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ w, int ldw, T* __restrict__ y, int ldy, int N, int C,
                             int E, int ff, int kind) {
    constexpr int RUN = 16 / sizeof(T);
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y;
    for (int j = (blockIdx.x * blockDim.x + threadIdx.x) * RUN; j < C; j += gridDim.x * blockDim.x * RUN) {
        const int b = j < E * ff ? j / ff : E;
        const float wt = w[(size_t)t * ldw + b];
        uint4 raw = make_uint4(0, 0, 0, 0);
        T* v = reinterpret_cast<T*>(&raw);
        if (wt != 0.f) {
            raw = *reinterpret_cast<const uint4*>(x + (size_t)t * ldx + j);
#pragma unroll
            for (int e = 0; e < RUN; ++e) v[e] = from_float<T>(activate(to_float(v[e]), kind) * wt);
        }
        *reinterpret_cast<uint4*>(y + (size_t)t * ldy + j) = raw;
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
expert_act_scale_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ w, int ldw, T* __restrict__ y, int ldy, int N, int C,
                        int E, int ff, int kind) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.y;
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < C; j += gridDim.x * blockDim.x) {
        const int b = j < E * ff ? j / ff : E;
        const float wt = w[(size_t)t * ldw + b];
        y[(size_t)t * ldy + j] = from_float<T>(wt == 0.f ? 0.f : activate(to_float(x[(size_t)t * ldx + j]), kind) * wt);
    }
}

// Experts of the gated form whose gate and up products are bounded:
//     g = min(gate, limit)      u = clamp(up, -limit, limit)      y = g * sigmoid(slope * g) * (u + 1) * weight
// x [N, ...]: for every expert e its gate columns [e * 2 ff, e * 2 ff + ff) and its up columns behind them, then a shared
// expert's gate and up columns (fs each, limit_s; fs = 0: none).  y [N, E * ff + fs].  The weight of expert e for token t
// is w[t, e] (float32, the shared expert's at w[t, E]) or, without w, 1 / top where e is one of the `top` entries of
// table[ids[t]] and 0 elsewhere (the shared expert 1).  Where the weight is 0 nothing is read.  RUN consecutive columns a
// thread (16 bytes where sizes and addresses allow, else one).
template <typename T, int RUN>
__global__ void __launch_bounds__(256)
expert_gated_act_kernel(const T* __restrict__ x, int ldx, T* __restrict__ y, int ldy, const float* __restrict__ w, int ldw,
                        const int* __restrict__ ids, const int* __restrict__ table, int top, int vocab, int E, int ff, int fs,
                        float limit, float limit_s, float slope, float up_shift) {
    pdl_trigger();
    const int t = blockIdx.y;
    const int C = E * ff + fs;
    const float share = top > 0 ? 1.f / (float)top : 0.f;
    const int* mine = nullptr;
    if (!w) {
        int id = ids[t];
        if (id < 0 || id >= vocab) id = 0;
        mine = table + (size_t)id * top;
    }
    pdl_wait();
    for (int j = (blockIdx.x * blockDim.x + threadIdx.x) * RUN; j < C; j += gridDim.x * blockDim.x * RUN) {
        const bool shared = j >= E * ff;
        const int e = shared ? E : j / ff, i = shared ? j - E * ff : j - e * ff;
        float wt;
        if (w) wt = w[(size_t)t * ldw + e];
        else if (shared) wt = 1.f;
        else {
            wt = 0.f;
            for (int c = 0; c < top; ++c) wt = mine[c] == e ? share : wt;
        }
        float out[RUN];
#pragma unroll
        for (int c = 0; c < RUN; ++c) out[c] = 0.f;
        if (wt != 0.f) {
            const int width = shared ? fs : ff;
            const float lim = shared ? limit_s : limit;
            const T* gp = x + (size_t)t * ldx + (size_t)E * 2 * ff * (shared ? 1 : 0) + (shared ? 0 : (size_t)e * 2 * ff) + i;
            float g[RUN], u[RUN];
            if constexpr (RUN == 4) { load4(gp, g); load4(gp + width, u); }
            else if constexpr (RUN == 8) {
                float a[4], b[4];
                load4(gp, a); load4(gp + 4, b);
#pragma unroll
                for (int c = 0; c < 4; ++c) { g[c] = a[c]; g[c + 4] = b[c]; }
                load4(gp + width, a); load4(gp + width + 4, b);
#pragma unroll
                for (int c = 0; c < 4; ++c) { u[c] = a[c]; u[c + 4] = b[c]; }
            } else { g[0] = to_float(gp[0]); u[0] = to_float(gp[width]); }
#pragma unroll
            for (int c = 0; c < RUN; ++c) {
                const float gc = fminf(g[c], lim), uc = fminf(fmaxf(u[c], -lim), lim);
                out[c] = gc / (1.f + expf(-slope * gc)) * (uc + up_shift) * wt;
            }
        }
        T* dst = y + (size_t)t * ldy + j;
        if constexpr (RUN == 4) store4(dst, out);
        else if constexpr (RUN == 8) {
            float a[4] = {out[0], out[1], out[2], out[3]}, b[4] = {out[4], out[5], out[6], out[7]};
            store4(dst, a); store4(dst + 4, b);
        } else dst[0] = from_float<T>(out[0]);
    }
}

// out[t, :] = factor * sum_b  x_b[t, :] / sqrt(mean(x_b[t, :]^2) + eps) * w_b        (b < count <= 4), one CTA per row
struct Branches {
    const float* x[4];
    const float* w[4];
};

__global__ void __launch_bounds__(256)
branch_norm_sum_kernel(Branches br, int count, float* __restrict__ out, int C, float eps, float factor, int cached) {
    extern __shared__ float rowbuf[];  // [count][C] when the rows fit (`cached`): every row is read from memory once
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const size_t row = (size_t)blockIdx.x * C;
    float scale[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        if (b >= count) break;
        float ss = 0.f;
        for (int i = threadIdx.x; i < C; i += blockDim.x) {
            const float v = br.x[b][row + i];
            if (cached) rowbuf[b * C + i] = v;
            ss = fmaf(v, v, ss);
        }
        ss = block_sum(ss, scratch);
        scale[b] = 1.f / sqrtf(ss / (float)C + eps);
    }
    for (int i = threadIdx.x; i < C; i += blockDim.x) {
        float s = 0.f;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            if (b >= count) break;
            s += (cached ? rowbuf[b * C + i] : br.x[b][row + i]) * scale[b] * br.w[b][i];
        }
        out[row + i] = s * factor;
    }
}

// The same, straight into the residual stream and through the norm behind it:
//   resid[t, :] += factor * sum_b rmsnorm(x_b[t, :]) * w_b;   out[t, :] = resid[t, :] / sqrt(mean(resid[t, :]^2) + eps_n) * wn
// One CTA a row; the branches' rows and the stream's new row wait in shared memory between the passes.
template <typename TO>
__global__ void __launch_bounds__(256)
branch_sum_norm_kernel(Branches br, int count, float* __restrict__ resid, const float* __restrict__ wn, TO* __restrict__ out, int C, float eps,
                       float factor, float eps_n) {
    extern __shared__ float rowbuf[];  // [count + 1][C]
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const size_t row = (size_t)blockIdx.x * C;
    float scale[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        if (b >= count) break;
        float ss = 0.f;
        for (int i = threadIdx.x; i < C; i += blockDim.x) {
            const float v = br.x[b][row + i];
            rowbuf[b * C + i] = v;
            ss = fmaf(v, v, ss);
        }
        ss = block_sum(ss, scratch);
        scale[b] = 1.f / sqrtf(ss / (float)C + eps);
    }
    float* fresh = rowbuf + (size_t)count * C;
    float ss = 0.f;
    for (int i = threadIdx.x; i < C; i += blockDim.x) {
        float s = 0.f;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            if (b >= count) break;
            s += rowbuf[b * C + i] * scale[b] * br.w[b][i];
        }
        const float v = resid[row + i] + s * factor;
        resid[row + i] = v;
        fresh[i] = v;
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float sn = 1.f / sqrtf(ss / (float)C + eps_n);
    for (int i = threadIdx.x; i < C; i += blockDim.x) out[row + i] = from_float<TO>(fresh[i] * sn * wn[i]);
}

}  // namespace

LLM_EXPORT int llm_branch_sum_norm(const float* x0, const float* w0, const float* x1, const float* w1, const float* x2, const float* w2,
                                   const float* x3, const float* w3, int count, float* resid, const float* wn, void* out, int out_dtype, int N,
                                   int C, float eps, float factor, float eps_n, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (count < 1 || count > 4 || C <= 0) return LLM_ERR_BAD_ARGUMENT;
    const size_t need = (size_t)(count + 1) * C * sizeof(float);
    if (need > 160 * 1024) return LLM_ERR_UNSUPPORTED;
    Branches br = {{x0, x1, x2, x3}, {w0, w1, w2, w3}};
    auto go = [&](auto kernel, auto* op) -> int {
        if (need > 48 * 1024) {
            const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need);
            if (e != cudaSuccess) return (int)e;
        }
        return launch_pdl(kernel, dim3(N), dim3(256), need, stream, br, count, resid, wn, op, C, eps, factor, eps_n);
    };
    if (out_dtype == LLM_F32) return go(branch_sum_norm_kernel<float>, (float*)out);
    return go(branch_sum_norm_kernel<__nv_bfloat16>, (__nv_bfloat16*)out);
}

LLM_EXPORT int llm_route_topk(const float* z, int ldz, const float* correction, float* w, int N, int E, int top, float scale,
                              int renorm, int shared_gate, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (E <= 0 || top < 1 || top > E || E > 4096 || ldz < E + (shared_gate ? 1 : 0)) return LLM_ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)4 * 2 * E * sizeof(float);
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(route_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return launch_pdl(route_topk_kernel, dim3((N + 3) / 4), dim3(128), smem, stream, z, ldz, correction, w, N, E, top, scale, renorm,
                      shared_gate ? 1 : 0);
}

LLM_EXPORT int llm_router(const void* x, int x_dtype, int ldx, const float* wr, const float* correction, float* out, int N, int K, int E,
                          int top, float scale, int renorm, int shared_gate, const float* bias, cudaStream_t stream) {
    if (N <= 0) return 0;
    if (E <= 0 || top < 1 || top > E || E > 2048 || K <= 0 || shared_gate < 0 || shared_gate > 2) return LLM_ERR_BAD_ARGUMENT;
    // tokens a CTA: one for steps of few tokens (more CTAs, more loads in flight a warp), two otherwise (three CTAs an SM)
    const int TT = N <= 32 ? 1 : 2;
    const int rows_all = E + (shared_gate == 1 ? 1 : 0);  // rows of the router's matrix (2: the last column of out is the constant 1)
    const size_t smem = ((size_t)TT * rows_all + (size_t)TT * 2 * E) * sizeof(float);
    const int groups = (rows_all + 3) / 4;  // of four rows: a warp each, as far as 16 warps go
    const dim3 grid((N + TT - 1) / TT), block(32 * (groups < 4 ? 4 : groups > 16 ? 16 : groups));
    auto go = [&](auto kernel, auto* xp) -> int {
        if (smem > 48 * 1024) {
            const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        return launch_pdl(kernel, grid, block, smem, stream, xp, ldx, wr, correction, out, N, K, E, top, scale, renorm, shared_gate, bias);
    };
    using bf = __nv_bfloat16;
    if (x_dtype == LLM_F32) return TT == 1 ? go(router_kernel<float, 1>, (const float*)x) : go(router_kernel<float, 2>, (const float*)x);
    return TT == 1 ? go(router_kernel<bf, 1>, (const bf*)x) : go(router_kernel<bf, 2>, (const bf*)x);
}

LLM_EXPORT int llm_expert_act_scale(const void* x, int ldx, const float* w, int ldw, void* y, int ldy, int dtype, int N, int C, int E,
                                    int ff, int kind, cudaStream_t stream) {
    if (N <= 0 || C <= 0) return 0;
    if (E < 0 || ff <= 0 || (size_t)E * ff > (size_t)C || N > 65535) return LLM_ERR_BAD_ARGUMENT;
    const int run = dtype == LLM_F32 ? 4 : 8;
    if (ff % run == 0 && C % run == 0 && ldx % run == 0 && ldy % run == 0 && ((uintptr_t)x | (uintptr_t)y) % 16 == 0) {
        const int per = 256 * run, blocks = (C + per - 1) / per;
        const dim3 grid(blocks < 64 ? blocks : 64, N), block(256);
        if (dtype == LLM_F32)
            return launch_pdl(expert_act_scale_wide_kernel<float>, grid, block, 0, stream, (const float*)x, ldx, w, ldw, (float*)y, ldy, N, C, E, ff, kind);
        return launch_pdl(expert_act_scale_wide_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)x, ldx, w, ldw,
                          (__nv_bfloat16*)y, ldy, N, C, E, ff, kind);
    }
    const dim3 grid((C + 255) / 256 < 64 ? (C + 255) / 256 : 64, N), block(256);
    if (dtype == LLM_F32)
        return launch_pdl(expert_act_scale_kernel<float>, grid, block, 0, stream, (const float*)x, ldx, w, ldw, (float*)y, ldy, N, C, E, ff, kind);
    return launch_pdl(expert_act_scale_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)x, ldx, w, ldw,
                      (__nv_bfloat16*)y, ldy, N, C, E, ff, kind);
}

LLM_EXPORT int llm_expert_gated_act(const void* x, int ldx, void* y, int ldy, int dtype, const float* w, int ldw, const int* ids,
                                    const int* table, int top, int vocab, int N, int E, int ff, int fs, float limit, float limit_s,
                                    float slope, float up_shift, cudaStream_t stream) {
    const int C = E * ff + fs;
    if (N <= 0 || C <= 0) return 0;
    if (E < 0 || ff < 0 || fs < 0 || N > 65535 || (!w && (!ids || !table || top < 0 || vocab <= 0))) return LLM_ERR_BAD_ARGUMENT;
    const int run = dtype == LLM_F32 ? 4 : 8;
    const bool wide = ff % run == 0 && fs % run == 0 && ldx % run == 0 && ldy % run == 0 && ((uintptr_t)x | (uintptr_t)y) % 16 == 0;
    const int per = 256 * (wide ? run : 1), blocks = (C + per - 1) / per;
    const dim3 grid(blocks < 64 ? blocks : 64, N), block(256);
    using bf = __nv_bfloat16;
    auto go = [&](auto kernel, auto* xp, auto* yp) {
        return launch_pdl(kernel, grid, block, 0, stream, xp, ldx, yp, ldy, w, ldw, ids, table, top, vocab, E, ff, fs, limit, limit_s, slope, up_shift);
    };
    if (dtype == LLM_F32)
        return wide ? go(expert_gated_act_kernel<float, 4>, (const float*)x, (float*)y) : go(expert_gated_act_kernel<float, 1>, (const float*)x, (float*)y);
    if (dtype == LLM_BF16)
        return wide ? go(expert_gated_act_kernel<bf, 8>, (const bf*)x, (bf*)y) : go(expert_gated_act_kernel<bf, 1>, (const bf*)x, (bf*)y);
    return LLM_ERR_BAD_ARGUMENT;
}

LLM_EXPORT int llm_branch_norm_sum(const float* x0, const float* w0, const float* x1, const float* w1, const float* x2, const float* w2,
                                   const float* x3, const float* w3, int count, float* out, int N, int C, float eps, float factor,
                                   cudaStream_t stream) {
    if (N <= 0) return 0;
    if (count < 1 || count > 4 || C <= 0) return LLM_ERR_BAD_ARGUMENT;
    Branches br = {{x0, x1, x2, x3}, {w0, w1, w2, w3}};
    const size_t need = (size_t)count * C * sizeof(float);
    const int cached = need <= 96 * 1024;
    if (cached && need > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(branch_norm_sum_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need);
        if (e != cudaSuccess) return (int)e;
    }
    return launch_pdl(branch_norm_sum_kernel, dim3(N), dim3(256), cached ? need : 0, stream, br, count, out, C, eps, factor, cached);
}
