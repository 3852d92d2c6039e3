// Row-wise kernels around the residual stream for layers that scale their contributions, normalise in groups or
// run a stretch of layers several times: the grouped RMS norm fused with a scaled residual sum, the sum of the
// stream with the token embeddings and a per-pass vector, one-input activations, and output gates.
//
// Statistics, sums and activations are 32-bit whatever the element type; results are rounded once.
#include "common.cuh"

namespace {

constexpr int NORM_WARPS = 4;

__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }

// ---------------------------------------------------------------------------------------------
// v = resid[row] + alpha * delta[row]; resid[row] = v (when all rows are produced); every one of `groups` equal
// consecutive parts of v is divided by sqrt(mean(part^2) + eps); out = that * weight.  One warp per (row, group):
// the order of a part's additions depends on its length alone.
// ---------------------------------------------------------------------------------------------
template <typename TD, typename TO>
__global__ void __launch_bounds__(NORM_WARPS * 32)
group_rmsnorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta, float alpha, const float* __restrict__ weight,
                     float eps, int groups, const int* __restrict__ rows, TO* __restrict__ out, int n_out, int hidden) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * NORM_WARPS + warp;
    if (item >= (long long)n_out * groups) return;
    const int o = (int)(item / groups), g = (int)(item - (long long)o * groups);
    const int r = rows ? rows[o] : o;
    const int len = hidden / groups;
    float* x = resid + (size_t)r * hidden + (size_t)g * len;
    const TD* d = delta ? delta + (size_t)r * hidden + (size_t)g * len : nullptr;
    const float* w = weight + (size_t)g * len;
    TO* y = out + (size_t)o * hidden + (size_t)g * len;
    const bool write_back = d && !rows;
    float ss = 0.f;
    if ((len & 3) == 0 && (hidden & 3) == 0) {
        for (int i = lane * 4; i < len; i += 128) {
            float v[4];
            load4(x + i, v);
            if (d) {
                float dv[4];
                load4(d + i, dv);
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] = fmaf(alpha, dv[e], v[e]);
                if (write_back) store4(x + i, v);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) ss = fmaf(v[e], v[e], ss);
        }
        ss = warp_sum(ss);
        const float scale = 1.f / sqrtf(ss / (float)len + eps);
        for (int i = lane * 4; i < len; i += 128) {
            float v[4], wv[4];
            load4(x + i, v);
            if (d && !write_back) {
                float dv[4];
                load4(d + i, dv);
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] = fmaf(alpha, dv[e], v[e]);
            }
            load4(w + i, wv);
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = v[e] * scale * wv[e];
            store4(y + i, v);
        }
        return;
    }
    for (int i = lane; i < len; i += 32) {
        float v = x[i];
        if (d) {
            v = fmaf(alpha, to_float(d[i]), v);
            if (write_back) x[i] = v;
        }
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float scale = 1.f / sqrtf(ss / (float)len + eps);
    for (int i = lane; i < len; i += 32) {
        float v = x[i];
        if (d && !write_back) v = fmaf(alpha, to_float(d[i]), v);
        y[i] = from_float<TO>(v * scale * w[i]);
    }
}

// The same with a CTA of 128 threads per (row, group) and the part in registers, for steps of few rows (a warp per part
// would walk a part of a thousand elements in 8 dependent trips to memory): parts of at most 4,096 elements, a
// multiple of 4 long.
template <typename TD, typename TO>
__global__ void __launch_bounds__(128)
group_rmsnorm_wide_kernel(float* __restrict__ resid, const TD* __restrict__ delta, float alpha, const float* __restrict__ weight,
                          float eps, int groups, const int* __restrict__ rows, TO* __restrict__ out, int hidden) {
    __shared__ float scratch[33];
    constexpr int NV = 8;
    pdl_trigger();
    const int o = blockIdx.x / groups, g = blockIdx.x - o * groups, len = hidden / groups, t4 = threadIdx.x * 4;
    const float* w = weight + (size_t)g * len;
    float wv[NV][4];
#pragma unroll
    for (int j = 0; j < NV; ++j)  // the weights do not depend on the kernel in front
        if (t4 + j * 512 < len) load4(w + t4 + j * 512, wv[j]);
    pdl_wait();
    const int r = rows ? rows[o] : o;
    float* x = resid + (size_t)r * hidden + (size_t)g * len;
    const TD* d = delta ? delta + (size_t)r * hidden + (size_t)g * len : nullptr;
    float v[NV][4], dv[NV][4];
#pragma unroll
    for (int j = 0; j < NV; ++j)
        if (t4 + j * 512 < len) {
            load4(x + t4 + j * 512, v[j]);
            if (d) load4(d + t4 + j * 512, dv[j]);
        }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j)
        if (t4 + j * 512 < len) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (d) v[j][e] = fmaf(alpha, dv[j][e], v[j][e]);
                ss = fmaf(v[j][e], v[j][e], ss);
            }
        }
    ss = block_sum(ss, scratch);
    const float scale = 1.f / sqrtf(ss / (float)len + eps);
    TO* y = out + (size_t)o * hidden + (size_t)g * len;
    const bool write_back = d && !rows;
#pragma unroll
    for (int j = 0; j < NV; ++j)
        if (t4 + j * 512 < len) {
            if (write_back) store4(x + t4 + j * 512, v[j]);
            float n[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) n[e] = v[j][e] * scale * wv[j][e];
            store4(y + t4 + j * 512, n);
        }
}

template <typename TD, typename TO>
int group_rmsnorm_launch(float* resid, const void* delta, float alpha, const float* weight, float eps, int groups,
                         const int* rows, void* out, int n_out, int hidden, cudaStream_t stream) {
    const long long items = (long long)n_out * groups;
    const int len = hidden / groups;
    if (items <= 1024 && (len & 3) == 0 && (hidden & 3) == 0 && len <= 4096 && len >= 256)
        return launch_pdl(group_rmsnorm_wide_kernel<TD, TO>, dim3((unsigned)items), dim3(128), 0, stream, resid, (const TD*)delta,
                          alpha, weight, eps, groups, rows, (TO*)out, hidden);
    const long long blocks = (items + NORM_WARPS - 1) / NORM_WARPS;
    if (blocks > 0x7fffffffLL) return LLM_ERR_UNSUPPORTED;
    return launch_pdl(group_rmsnorm_kernel<TD, TO>, dim3((unsigned)blocks), dim3(NORM_WARPS * 32), 0, stream, resid,
                      (const TD*)delta, alpha, weight, eps, groups, rows, (TO*)out, n_out, hidden);
}

// ---------------------------------------------------------------------------------------------
// resid[t] = ((resid[t] + alpha * delta[t]) + float(table[ids[t]])) + vector, each addend optional
// ---------------------------------------------------------------------------------------------
template <typename TD, typename TT>
__global__ void stream_inject_kernel(float* __restrict__ resid, const TD* __restrict__ delta, float alpha,
                                     const int* __restrict__ ids, const TT* __restrict__ table, int vocab,
                                     const float* __restrict__ vector, int hidden) {
    pdl_trigger();
    const int t = blockIdx.x;
    int id = table ? ids[t] : 0;
    if (id < 0 || id >= vocab) id = 0;  // launch-side checks reject such ids; never read out of range
    pdl_wait();
    float* x = resid + (size_t)t * hidden;
    const TD* d = delta ? delta + (size_t)t * hidden : nullptr;
    const TT* e = table ? table + (size_t)id * hidden : nullptr;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = x[i];
        if (d) v = fmaf(alpha, to_float(d[i]), v);
        if (e) v += to_float(e[i]);
        if (vector) v += vector[i];
        x[i] = v;
    }
}

// ---------------------------------------------------------------------------------------------
// one-input functions of a matrix with a row pitch: 0 relu(v)^2, 1 gelu (tanh form), 2 alpha * v, 3 silu
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float unary_of(float v, int kind, float alpha) {
    switch (kind) {
        case 0: v = fmaxf(v, 0.f); return v * v;
        case 1: return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
        case 2: return alpha * v;
        default: return v * sigmoid_f(v);
    }
}

template <typename T>
__global__ void unary_kernel(const T* __restrict__ x, int ldx, T* __restrict__ out, int ldo, int cols, size_t total,
                             int kind, float alpha, bool wide) {
    pdl_trigger();
    pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    if (wide) {  // four elements a thread: rows a multiple of four long and apart, bases aligned
        for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < total; i += stride * 4) {
            const size_t t = i / cols;
            const int j = (int)(i - t * cols);
            float v[4];
            load4(x + t * ldx + j, v);
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = unary_of(v[e], kind, alpha);
            store4(out + t * ldo + j, v);
        }
        return;
    }
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t t = i / cols;
        const int j = (int)(i - t * cols);
        out[t * ldo + j] = from_float<T>(unary_of(to_float(x[t * ldx + j]), kind, alpha));
    }
}

// ---------------------------------------------------------------------------------------------
// out[t, h * head_width + j] = a[t, h, j] * gate(b[t, h * head_width + j]); a is addressed by a token stride and a
// head stride (it may lie head by head), gate: 0 sigmoid, 1 silu
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void gate_mul_kernel(const T* __restrict__ a, long long a_token_stride, long long a_head_stride, int head_width,
                                const T* __restrict__ b, int ldb, T* __restrict__ out, int ldo, int cols, size_t total,
                                int kind) {
    pdl_trigger();
    pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t t = i / cols;
        const int c = (int)(i - t * cols);
        const int h = c / head_width, j = c - h * head_width;
        const float av = to_float(a[(long long)t * a_token_stride + (long long)h * a_head_stride + j]);
        const float bv = to_float(b[t * ldb + ((kind & 2) ? h : c)]);  // kind & 2: one gate a head, b [N, heads]
        const float gate = (kind & 1) == 0 ? sigmoid_f(bv) : bv * sigmoid_f(bv);
        out[t * ldo + c] = from_float<T>(av * gate);
    }
}

// out[t, :] = x[t, :cols] / sqrt(mean(x[t, :cols]^2) + eps) * weight: the RMS norm of a run of columns of rows that have
// a pitch (a part of a stacked projection), statistics in 32-bit; a warp a row.
template <typename TI, typename TO>
__global__ void __launch_bounds__(128)
row_rmsnorm_kernel(const TI* __restrict__ x, int ldx, const float* __restrict__ weight, float eps, TO* __restrict__ out, int ldo,
                   int rows, int cols) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const TI* src = x + (size_t)row * ldx;
    float ss = 0.f;
    for (int i = lane; i < cols; i += 32) {
        const float v = to_float(src[i]);
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float scale = 1.f / sqrtf(ss / (float)cols + eps);
    TO* dst = out + (size_t)row * ldo;
    for (int i = lane; i < cols; i += 32) dst[i] = from_float<TO>(to_float(src[i]) * scale * weight[i]);
}

int flat_blocks(size_t total, int threads) {
    const size_t want = (total + threads - 1) / threads, most = 148 * 16;
    return (int)(want < most ? (want ? want : 1) : most);
}

}  // namespace

LLM_EXPORT int llm_group_rmsnorm(float* resid, const void* delta, int delta_dtype, float alpha, const float* weight,
                                 float eps, int groups, const int* rows, void* out, int out_dtype, int n_out, int hidden,
                                 cudaStream_t stream) {
    if (n_out <= 0) return 0;
    if (groups <= 0 || hidden <= 0 || hidden % groups) return LLM_ERR_BAD_ARGUMENT;
    using bf = __nv_bfloat16;
    if (out_dtype == LLM_F32 && (delta == nullptr || delta_dtype == LLM_F32))
        return group_rmsnorm_launch<float, float>(resid, delta, alpha, weight, eps, groups, rows, out, n_out, hidden, stream);
    if (out_dtype == LLM_BF16 && (delta == nullptr || delta_dtype == LLM_F32))
        return group_rmsnorm_launch<float, bf>(resid, delta, alpha, weight, eps, groups, rows, out, n_out, hidden, stream);
    if (out_dtype == LLM_BF16 && delta_dtype == LLM_BF16)
        return group_rmsnorm_launch<bf, bf>(resid, delta, alpha, weight, eps, groups, rows, out, n_out, hidden, stream);
    if (out_dtype == LLM_F32 && delta_dtype == LLM_BF16)
        return group_rmsnorm_launch<bf, float>(resid, delta, alpha, weight, eps, groups, rows, out, n_out, hidden, stream);
    return LLM_ERR_BAD_ARGUMENT;
}

LLM_EXPORT int llm_stream_inject(float* resid, const void* delta, int delta_dtype, float alpha, const int* ids,
                                 const void* table, int table_dtype, int vocab, const float* vector, int n, int hidden,
                                 cudaStream_t stream) {
    if (n <= 0) return 0;
    if (table != nullptr && ids == nullptr) return LLM_ERR_BAD_ARGUMENT;
    using bf = __nv_bfloat16;
    const int threads = hidden >= 1024 ? 256 : 128;
    const bool d32 = delta == nullptr || delta_dtype == LLM_F32, t32 = table == nullptr || table_dtype == LLM_F32;
    if (delta != nullptr && delta_dtype != LLM_F32 && delta_dtype != LLM_BF16) return LLM_ERR_BAD_ARGUMENT;
    if (table != nullptr && table_dtype != LLM_F32 && table_dtype != LLM_BF16) return LLM_ERR_BAD_ARGUMENT;
    auto go = [&](auto kernel, auto* dp, auto* tp) {
        return launch_pdl(kernel, dim3(n), dim3(threads), 0, stream, resid, dp, alpha, ids, tp, vocab, vector, hidden);
    };
    if (d32 && t32) return go(stream_inject_kernel<float, float>, (const float*)delta, (const float*)table);
    if (d32) return go(stream_inject_kernel<float, bf>, (const float*)delta, (const bf*)table);
    if (t32) return go(stream_inject_kernel<bf, float>, (const bf*)delta, (const float*)table);
    return go(stream_inject_kernel<bf, bf>, (const bf*)delta, (const bf*)table);
}

LLM_EXPORT int llm_unary(const void* x, int ldx, void* out, int ldo, int dtype, int rows, int cols, int kind, float alpha,
                         cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if (ldx < cols || ldo < cols || kind < 0 || kind > 3) return LLM_ERR_BAD_ARGUMENT;
    const size_t total = (size_t)rows * cols;
    const bool wide = ((cols | ldx | ldo) & 3) == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0;
    const int threads = 256, blocks = flat_blocks(wide ? (total + 3) / 4 : total, threads);
    if (dtype == LLM_F32)
        return launch_pdl(unary_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float*)x, ldx, (float*)out, ldo,
                          cols, total, kind, alpha, wide);
    if (dtype == LLM_BF16)
        return launch_pdl(unary_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (const __nv_bfloat16*)x, ldx,
                          (__nv_bfloat16*)out, ldo, cols, total, kind, alpha, wide);
    return LLM_ERR_BAD_ARGUMENT;
}

LLM_EXPORT int llm_gate_mul(const void* a, long long a_token_stride, long long a_head_stride, int head_width, const void* b,
                            int ldb, void* out, int ldo, int dtype, int rows, int cols, int kind, cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return 0;
    if (head_width <= 0 || cols % head_width || ldb < ((kind & 2) ? cols / head_width : cols) || ldo < cols || kind < 0 || kind > 3)
        return LLM_ERR_BAD_ARGUMENT;
    const size_t total = (size_t)rows * cols;
    const int threads = 256, blocks = flat_blocks(total, threads);
    if (dtype == LLM_F32)
        return launch_pdl(gate_mul_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float*)a, a_token_stride,
                          a_head_stride, head_width, (const float*)b, ldb, (float*)out, ldo, cols, total, kind);
    if (dtype == LLM_BF16)
        return launch_pdl(gate_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (const __nv_bfloat16*)a,
                          a_token_stride, a_head_stride, head_width, (const __nv_bfloat16*)b, ldb, (__nv_bfloat16*)out, ldo,
                          cols, total, kind);
    return LLM_ERR_BAD_ARGUMENT;
}

// x [rows, >= cols] with row pitch ldx (float32 or bfloat16) -> out [rows, cols] with pitch ldo, of type out_dtype.
LLM_EXPORT int llm_row_rmsnorm(const void* x, int x_dtype, int ldx, const float* weight, float eps, void* out, int out_dtype, int ldo,
                               int rows, int cols, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (cols <= 0 || ldx < cols || ldo < cols || !weight) return LLM_ERR_BAD_ARGUMENT;
    using bf = __nv_bfloat16;
    const dim3 grid((rows + 3) / 4), block(128);
    if (x_dtype == LLM_F32 && out_dtype == LLM_F32)
        return launch_pdl(row_rmsnorm_kernel<float, float>, grid, block, 0, stream, (const float*)x, ldx, weight, eps, (float*)out, ldo, rows, cols);
    if (x_dtype == LLM_F32 && out_dtype == LLM_BF16)
        return launch_pdl(row_rmsnorm_kernel<float, bf>, grid, block, 0, stream, (const float*)x, ldx, weight, eps, (bf*)out, ldo, rows, cols);
    if (x_dtype == LLM_BF16 && out_dtype == LLM_BF16)
        return launch_pdl(row_rmsnorm_kernel<bf, bf>, grid, block, 0, stream, (const bf*)x, ldx, weight, eps, (bf*)out, ldo, rows, cols);
    if (x_dtype == LLM_BF16 && out_dtype == LLM_F32)
        return launch_pdl(row_rmsnorm_kernel<bf, float>, grid, block, 0, stream, (const bf*)x, ldx, weight, eps, (float*)out, ldo, rows, cols);
    return LLM_ERR_BAD_ARGUMENT;
}
