// A residual stream kept in several copies (hyper-connections).
//
// Instead of one row x per token there are S rows x_1 .. x_S, all equal to the token's embedding at the start.  A part
// of a layer reads u = sum_s in[s] x_s, and what it returns (y) is taken up by all copies at once from the old ones:
//     x_t <- sum_s mix[s, t] x_s + out[t] * y                     (mix is indexed [from, to])
// Everything here is 32-bit.  Between two parts the update with the first part's (mix, out), the read-in with the second
// part's `in` and the RMS norm in front of the second part are one pass over the S rows: hyper_mix_norm_kernel.
#include "common.cuh"

namespace {

constexpr int MAX_S = 8;  // most copies of the stream
constexpr int MAX_Y = 4;  // most tensors whose weighted sum is the part's result

// out[c, t, :] = float(table[ids[t], :]) for every copy c < copies.
template <typename T>
__global__ void embed_copies_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out, int hidden,
                                    int vocab, int copies, int n) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= vocab) id = 0;  // launch-side checks reject such ids; never read out of range
    const T* src = table + (size_t)id * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = to_float(src[i]);
        for (int c = 0; c < copies; ++c) out[((size_t)c * n + t) * hidden + i] = v;
    }
}

struct Results {
    const float* y[MAX_Y];  // [N, W] each (null beyond count)
    float factor[MAX_Y];
    int count;  // 0: nothing is taken up, the copies are only read
};

// One CTA per produced row.  `rows` (or null): which token rows are produced; with it the copies are left as they are
// (only the normed read-in of the updated copies is wanted, for the rows whose logits are asked for).
// read_in null: u is the plain sum of the copies.
template <typename TO>
__global__ void __launch_bounds__(256)
hyper_mix_norm_kernel(float* __restrict__ X, const Results res, const float* __restrict__ mix, const float* __restrict__ take,
                      const float* __restrict__ read_in, const float* __restrict__ weight, float eps, const int* __restrict__ rows,
                      TO* __restrict__ out, int S, int N, int W) {
    extern __shared__ float u_row[];  // W floats
    __shared__ float scratch[33];
    __shared__ float mix_s[MAX_S * MAX_S], take_s[MAX_S], in_s[MAX_S];
    pdl_trigger();
    const bool update = res.count > 0;
    for (int i = threadIdx.x; i < S * S; i += blockDim.x) mix_s[i] = update ? mix[i] : 0.f;
    for (int i = threadIdx.x; i < S; i += blockDim.x) {
        take_s[i] = update ? take[i] : 0.f;
        in_s[i] = read_in ? read_in[i] : 1.f;
    }
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;
    __syncthreads();
    pdl_wait();
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float x[MAX_S];
#pragma unroll
        for (int s = 0; s < MAX_S; ++s) x[s] = s < S ? X[((size_t)s * N + r) * W + c] : 0.f;
        float u = 0.f;
        if (update) {
            float y = 0.f;
#pragma unroll
            for (int b = 0; b < MAX_Y; ++b)
                if (b < res.count) y = fmaf(res.factor[b], res.y[b][(size_t)r * W + c], y);
#pragma unroll
            for (int t = 0; t < MAX_S; ++t)
                if (t < S) {
                    float v = take_s[t] * y;
#pragma unroll
                    for (int s = 0; s < MAX_S; ++s)
                        if (s < S) v = fmaf(mix_s[s * S + t], x[s], v);
                    if (!rows) X[((size_t)t * N + r) * W + c] = v;
                    u = fmaf(in_s[t], v, u);
                }
        } else {
#pragma unroll
            for (int s = 0; s < MAX_S; ++s)
                if (s < S) u = fmaf(in_s[s], x[s], u);
        }
        u_row[c] = u;
        ss = fmaf(u, u, ss);
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.f / sqrtf(ss / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) out[(size_t)o * W + c] = from_float<TO>(u_row[c] * scale * weight[c]);
}

}  // namespace

LLM_EXPORT int llm_embed_copies(const int* ids, const void* table, int table_dtype, float* out, int n, int hidden, int vocab,
                                int copies, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (copies < 1 || hidden <= 0) return LLM_ERR_BAD_ARGUMENT;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == LLM_F32)
        return launch_pdl(embed_copies_kernel<float>, dim3(n), dim3(threads), 0, stream, ids, (const float*)table, out, hidden, vocab, copies, n);
    if (table_dtype == LLM_BF16)
        return launch_pdl(embed_copies_kernel<__nv_bfloat16>, dim3(n), dim3(threads), 0, stream, ids, (const __nv_bfloat16*)table, out,
                          hidden, vocab, copies, n);
    return LLM_ERR_BAD_ARGUMENT;
}

// X [S, N, W] float32, in place.  y0..y3 / f0..f3: the part's result as a weighted sum of up to four [N, W] float32
// tensors (count 0: no update); mix [S, S], take [S] of the part that returned it; read_in [S] (null: ones) of the part that
// comes next; weight [W], eps of the norm in front of that part.  out [n_out, W] of out_dtype.
LLM_EXPORT int llm_hyper_mix_norm(float* X, const float* y0, const float* y1, const float* y2, const float* y3, float f0, float f1,
                                  float f2, float f3, int count, const float* mix, const float* take, const float* read_in,
                                  const float* weight, float eps, const int* rows, void* out, int out_dtype, int n_out, int S, int N,
                                  int W, cudaStream_t stream) {
    if (n_out <= 0) return 0;
    if (S < 1 || S > MAX_S || count < 0 || count > MAX_Y || W <= 0 || N <= 0 || (count > 0 && (!mix || !take)) || !weight)
        return LLM_ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)W * sizeof(float);
    if (smem > 200 * 1024) return LLM_ERR_UNSUPPORTED;
    Results res;
    const float* ys[MAX_Y] = {y0, y1, y2, y3};
    const float fs[MAX_Y] = {f0, f1, f2, f3};
    for (int b = 0; b < MAX_Y; ++b) {
        res.y[b] = b < count ? ys[b] : nullptr;
        res.factor[b] = fs[b];
        if (b < count && !ys[b]) return LLM_ERR_BAD_ARGUMENT;
    }
    res.count = count;
    const int threads = W >= 1024 ? 256 : 128;
    auto go = [&](auto kernel, auto* op) -> int {
        if (smem > 48 * 1024) {
            const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        return launch_pdl(kernel, dim3(n_out), dim3(threads), smem, stream, X, res, mix, take, read_in, weight, eps, rows, op, S, N, W);
    };
    if (out_dtype == LLM_F32) return go(hyper_mix_norm_kernel<float>, (float*)out);
    if (out_dtype == LLM_BF16) return go(hyper_mix_norm_kernel<__nv_bfloat16>, (__nv_bfloat16*)out);
    return LLM_ERR_BAD_ARGUMENT;
}
