// A short causal convolution over time on every channel of a token's projections, across the steps of a request.
//
//   y[t, c] = sum_j w[c, j] * u[t - (taps - 1) + j, c]        j = 0 .. taps - 1,  zeros before the request's first token
//
// u are the rows of a flat batch (request r owns rows cu[r] .. cu[r + 1] - 1); what lies before a request's first row of
// this step comes from its slot of `state` [slots, taps - 1, C] (float32): the last taps - 1 rows of u that earlier steps
// brought, oldest first (zeros where the request has had fewer).  A second kernel, which starts when every read of the
// first has been made, moves the slot on to the last taps - 1 rows after this step.  Sums are 32-bit, in the order of j.
#include "common.cuh"

namespace {

constexpr int MAX_TAPS = 16;

// grid (channel blocks, token tiles); a thread a channel, TOKENS rows a CTA
template <typename TI, int TOKENS>
__global__ void __launch_bounds__(128)
short_conv_kernel(const TI* __restrict__ u, int ldu, const float* __restrict__ w, const float* __restrict__ state,
                  const int* __restrict__ state_slots, const int* __restrict__ token_request, const int* __restrict__ cu_tokens,
                  float* __restrict__ y, int ldy, int N, int C, int taps) {
    pdl_trigger();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    float wt[MAX_TAPS];
    if (c < C)
#pragma unroll
        for (int j = 0; j < MAX_TAPS; ++j) wt[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
    pdl_wait();
    if (c >= C) return;
    const int t0 = blockIdx.y * TOKENS, back = taps - 1;
    for (int t = t0; t < min(N, t0 + TOKENS); ++t) {
        const int r = token_request[t], begin = cu_tokens[r];
        const float* old = state + (size_t)state_slots[r] * back * C;
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < MAX_TAPS; ++j) {
            if (j >= taps) break;
            const int src = t - back + j;  // a row of this step, or (before the request's first) of its slot
            const float v = src >= begin ? to_float(u[(size_t)src * ldu + c]) : old[(size_t)(src - begin + back) * C + c];
            acc = fmaf(wt[j], v, acc);
        }
        y[(size_t)t * ldy + c] = acc;
    }
}

// Up to four taps, four neighbouring channels a thread (16-byte loads), `span` tokens a CTA: the rows behind the newest stay in
// registers from token to token, so that a row is read once (and the taps - 1 rows in front of a CTA's first once more).
// Taps stand at the end of arrays of four, zeros in front, as in the walk below: the sums have the same order in every kernel.
template <typename TI>
__global__ void __launch_bounds__(128)
short_conv4_kernel(const TI* __restrict__ u, int ldu, const float* __restrict__ w, const float* __restrict__ state,
                   const int* __restrict__ state_slots, const int* __restrict__ token_request, const int* __restrict__ cu_tokens,
                   float* __restrict__ y, int ldy, int N, int C, int taps, int span) {
    constexpr int W = 4;
    pdl_trigger();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    const int first = W - taps, back = taps - 1;
    float wt[W][4];
    if (c < C)
#pragma unroll
        for (int k = 0; k < W; ++k)
#pragma unroll
            for (int e = 0; e < 4; ++e) wt[k][e] = k >= first ? w[(size_t)(c + e) * taps + (k - first)] : 0.f;
    const int t0 = blockIdx.y * span, t1 = min(N, t0 + span);
    int r = token_request[t0], begin = cu_tokens[r], end = cu_tokens[r + 1];
    pdl_wait();
    if (c >= C) return;
    float hist[W][4];
    // the rows behind token t: place k holds the row W - 1 - k places behind it, from this step or from the request's slot
    auto fill = [&](int t) {
#pragma unroll
        for (int k = 0; k < W - 1; ++k) {
            const int src = t - (W - 1 - k);
            if (k < first) hist[k][0] = hist[k][1] = hist[k][2] = hist[k][3] = 0.f;
            else if (src >= begin) load4(u + (size_t)src * ldu + c, hist[k]);
            else load4(state + ((size_t)state_slots[r] * back + (src - begin + back)) * C + c, hist[k]);
        }
    };
    fill(t0);
    float next[4];
    load4(u + (size_t)t0 * ldu + c, next);
    for (int t = t0; t < t1; ++t) {
        if (t == end) {  // the next request's rows begin: what stands behind them is its own slot
            ++r;
            begin = end;
            end = cu_tokens[r + 1];
            fill(t);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) hist[W - 1][e] = next[e];
        if (t + 1 < t1) load4(u + (size_t)(t + 1) * ldu + c, next);  // on its way while this row is summed
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int k = 0; k < W; ++k)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[e] = fmaf(wt[k][e], hist[k][e], acc[e]);
        store4(y + (size_t)t * ldy + c, acc);
#pragma unroll
        for (int k = 0; k < W - 1; ++k)
#pragma unroll
            for (int e = 0; e < 4; ++e) hist[k][e] = k >= first ? hist[k + 1][e] : 0.f;
    }
}

// grid (channel blocks, requests): the slot's rows after this step are the last taps - 1 of (old rows, this step's rows)
template <typename TI>
__global__ void __launch_bounds__(128)
short_conv_state_kernel(const TI* __restrict__ u, int ldu, float* __restrict__ state, const int* __restrict__ state_slots,
                        const int* __restrict__ cu_tokens, int C, int taps) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
    if (c >= C) return;
    const int begin = cu_tokens[r], count = cu_tokens[r + 1] - begin, back = taps - 1;
    float* slot = state + (size_t)state_slots[r] * back * C;
    float next[MAX_TAPS];
#pragma unroll
    for (int s = 0; s < MAX_TAPS; ++s) {
        if (s >= back) break;
        const int src = count + s - back;  // counted from the request's first row of this step
        next[s] = src >= 0 ? to_float(u[(size_t)(begin + src) * ldu + c]) : slot[(size_t)(count + s) * C + c];
    }
#pragma unroll
    for (int s = 0; s < MAX_TAPS; ++s) {
        if (s >= back) break;
        slot[(size_t)s * C + c] = next[s];
    }
}

// Steps in which no request brings more than a few tokens (decode steps): one launch.  grid (channel blocks, requests); a
// thread walks its request's rows for its channel with the last taps - 1 rows in registers, and leaves them in the slot.
template <typename TI>
__global__ void __launch_bounds__(128)
short_conv_walk_kernel(const TI* __restrict__ u, int ldu, const float* __restrict__ w, float* __restrict__ state,
                       const int* __restrict__ state_slots, const int* __restrict__ cu_tokens, float* __restrict__ y, int ldy, int C, int taps) {
    pdl_trigger();
    const int c = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y, back = taps - 1;
    // taps and rows stand at the END of two arrays of MAX_TAPS (tap j at MAX_TAPS - taps + j, zeros in front), so that every
    // index is known when the kernel is compiled; a product with a zero tap leaves a sum as it is, bit for bit
    float wt[MAX_TAPS], hist[MAX_TAPS];
    const int first = MAX_TAPS - taps;
    if (c < C)
#pragma unroll
        for (int k = 0; k < MAX_TAPS; ++k) wt[k] = k >= first ? w[(size_t)c * taps + (k - first)] : 0.f;
    const int begin = cu_tokens[r], end = cu_tokens[r + 1];
    float* slot = state ? state + (size_t)state_slots[r] * back * C : nullptr;
    pdl_wait();
    if (c >= C) return;
#pragma unroll
    for (int k = 0; k < MAX_TAPS; ++k) hist[k] = k > first ? slot[(size_t)(k - first - 1) * C + c] : 0.f;  // the slot's rows end at the last place
    for (int t = begin; t < end; ++t) {
#pragma unroll
        for (int k = 0; k < MAX_TAPS - 1; ++k) hist[k] = k >= first ? hist[k + 1] : 0.f;  // the oldest row leaves
        hist[MAX_TAPS - 1] = to_float(u[(size_t)t * ldu + c]);
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < MAX_TAPS; ++k) acc = fmaf(wt[k], hist[k], acc);  // the oldest row first, as in the other kernel
        y[(size_t)t * ldy + c] = acc;
    }
#pragma unroll
    for (int k = 0; k < MAX_TAPS; ++k)
        if (k > first) slot[(size_t)(k - first - 1) * C + c] = hist[k];
}

}  // namespace

// u [N, >= C] (float32 or bfloat16, row pitch ldu), w [C, taps] float32, state [slots, taps - 1, C] float32,
// y [N, C] float32 (row pitch ldy).  taps from 1 to 16 (1: a weight a channel, no state).
LLM_EXPORT int llm_short_conv(const void* u, int dtype, int ldu, const float* w, float* state, const int* state_slots,
                              const int* token_request, const int* cu_tokens, float* y, int ldy, int N, int requests, int C,
                              int taps, int max_query_len, cudaStream_t stream) {
    if (N <= 0 || requests <= 0) return 0;
    if (C <= 0 || taps < 1 || taps > MAX_TAPS || ldu < C || ldy < C || (taps > 1 && !state) || requests > 65535) return LLM_ERR_BAD_ARGUMENT;
    constexpr int TOKENS = 8;
    if (max_query_len > 0 && max_query_len <= 16) {  // few tokens a request: the walk, whose sums have the same order
        const dim3 wgrid((C + 127) / 128, requests);
        if (dtype == LLM_F32)
            return launch_pdl(short_conv_walk_kernel<float>, wgrid, dim3(128), 0, stream, (const float*)u, ldu, w, state, state_slots, cu_tokens, y, ldy, C, taps);
        if (dtype == LLM_BF16)
            return launch_pdl(short_conv_walk_kernel<__nv_bfloat16>, wgrid, dim3(128), 0, stream, (const __nv_bfloat16*)u, ldu, w, state, state_slots,
                              cu_tokens, y, ldy, C, taps);
        return LLM_ERR_BAD_ARGUMENT;
    }
    const dim3 block(128), grid((C + 127) / 128, (N + TOKENS - 1) / TOKENS);
    int code;
    const size_t in_align = dtype == LLM_F32 ? 16 : 8;
    const bool wide = taps <= 4 && C % 4 == 0 && ldu % 4 == 0 && ldy % 4 == 0 && (uintptr_t)u % in_align == 0 && (uintptr_t)y % 16 == 0 &&
                      (taps == 1 || (uintptr_t)state % 16 == 0);
    if (wide) {
        const int span = N >= 4096 ? 32 : 16;
        const dim3 g4((C / 4 + 127) / 128, (N + span - 1) / span);
        if (g4.y > 65535) return LLM_ERR_UNSUPPORTED;
        if (dtype == LLM_F32)
            code = launch_pdl(short_conv4_kernel<float>, g4, block, 0, stream, (const float*)u, ldu, w, (const float*)state, state_slots, token_request,
                              cu_tokens, y, ldy, N, C, taps, span);
        else if (dtype == LLM_BF16)
            code = launch_pdl(short_conv4_kernel<__nv_bfloat16>, g4, block, 0, stream, (const __nv_bfloat16*)u, ldu, w, (const float*)state, state_slots,
                              token_request, cu_tokens, y, ldy, N, C, taps, span);
        else
            return LLM_ERR_BAD_ARGUMENT;
    } else if (grid.y > 65535)
        return LLM_ERR_UNSUPPORTED;
    else if (dtype == LLM_F32)
        code = launch_pdl(short_conv_kernel<float, TOKENS>, grid, block, 0, stream, (const float*)u, ldu, w, (const float*)state, state_slots,
                          token_request, cu_tokens, y, ldy, N, C, taps);
    else if (dtype == LLM_BF16)
        code = launch_pdl(short_conv_kernel<__nv_bfloat16, TOKENS>, grid, block, 0, stream, (const __nv_bfloat16*)u, ldu, w,
                          (const float*)state, state_slots, token_request, cu_tokens, y, ldy, N, C, taps);
    else
        return LLM_ERR_BAD_ARGUMENT;
    if (code != 0 || taps == 1) return code;
    const dim3 sgrid((C + 127) / 128, requests);
    if (dtype == LLM_F32)
        return launch_pdl(short_conv_state_kernel<float>, sgrid, block, 0, stream, (const float*)u, ldu, state, state_slots, cu_tokens, C, taps);
    return launch_pdl(short_conv_state_kernel<__nv_bfloat16>, sgrid, block, 0, stream, (const __nv_bfloat16*)u, ldu, state, state_slots,
                      cu_tokens, C, taps);
}
