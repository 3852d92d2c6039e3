// What a token's projections go through between the stacked product and attention, together with the write of what
// the cache keeps: for latent attention the rotation of the query's rotated parts, the RMS norm of the latent and the
// rotation of the shared key part; for attention with unit-RMS queries and keys the two norms.
//
// Angles are 32-bit (float(position) * frequency, then sincosf), statistics are 32-bit, results are rounded once.
#include "common.cuh"

namespace {

// Interleaved rotary layout: lanes (2i, 2i + 1) of the first `rot_dims` lanes turn by position * freq[i]; the lanes
// behind them pass unchanged.
// `turn` holds (cos, sin) of every pair's angle, worked out once per token.
template <typename T>
__device__ __forceinline__ void rotate_pairs(const T* __restrict__ src, T* __restrict__ dst, int lanes, int rot_dims,
                                             const float2* __restrict__ turn, int first, int step) {
    const int pairs = rot_dims >> 1;
    for (int i = first; i < pairs; i += step) {
        const float c = turn[i].x, s = turn[i].y;
        const float u = to_float(src[2 * i]), v = to_float(src[2 * i + 1]);
        dst[2 * i] = from_float<T>(u * c - v * s);
        dst[2 * i + 1] = from_float<T>(v * c + u * s);
    }
    for (int i = rot_dims + first; i < lanes; i += step) dst[i] = src[i];
}

// Half layout: lanes (i, i + rot_dims / 2) of the first `rot_dims` lanes turn by position * freq[i].
template <typename T>
__device__ __forceinline__ void rotate_halves(const T* __restrict__ src, T* __restrict__ dst, int lanes, int rot_dims,
                                              const float2* __restrict__ turn, int first, int step) {
    const int pairs = rot_dims >> 1;
    for (int i = first; i < pairs; i += step) {
        const float c = turn[i].x, s = turn[i].y;
        const float u = to_float(src[i]), v = to_float(src[i + pairs]);
        dst[i] = from_float<T>(u * c - v * s);
        dst[i + pairs] = from_float<T>(v * c + u * s);
    }
    for (int i = rot_dims + first; i < lanes; i += step) dst[i] = src[i];
}

constexpr int MAX_TURNS = 320;  // pairs of a rotated part of at most 640 lanes

// Latent attention.  proj row: [H x (dim | rot) queries][rank latent | rot shared key part][...]; or the queries in rows
// of their own (`queries`, row pitch ldq) and the latent part at column `kv_col` of proj.  `halves`: the rotated lanes
// pair as (i, i + rot_dims / 2) instead of (2i, 2i + 1).
//   q_rot[t, h, :]   = rotate(proj query h's last rot lanes)
//   cache[slot, :]   = [ latent / sqrt(mean(latent^2) + eps) * weight | rotate(shared key part) ]
//   fresh[t, :]      = the same row (optional)
// One block per token.
template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const T* __restrict__ proj, int ldp, T* __restrict__ q_rot, T* __restrict__ fresh,
                      const int* __restrict__ positions, const int* __restrict__ slot_map, T* __restrict__ cache,
                      const float* __restrict__ weight,
                      const float* __restrict__ freq, float eps, int H, int dim, int rot, int rank, int rot_dims,
                      const T* __restrict__ queries, int ldq, int kv_col, int halves) {
    __shared__ float scratch[33];
    __shared__ float2 turn[MAX_TURNS];
    pdl_trigger();
    const int t = blockIdx.x;
    const float position = (float)positions[t];
    const size_t slot = (size_t)slot_map[t];
    // the angles depend on the token alone: every head and the shared key part turn by the same ones
    for (int i = threadIdx.x; i < (rot_dims >> 1); i += blockDim.x) {
        float s, c;
        sincosf(position * freq[i], &s, &c);
        turn[i] = make_float2(c, s);
    }
    __syncthreads();
    pdl_wait();
    const T* row = proj + (size_t)t * ldp;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const T* qrow = queries ? queries + (size_t)t * ldq : row;
    for (int h = warp; h < H; h += warps) {
        if (halves) rotate_halves(qrow + (size_t)h * (dim + rot) + dim, q_rot + ((size_t)t * H + h) * rot, rot, rot_dims, turn, lane, 32);
        else rotate_pairs(qrow + (size_t)h * (dim + rot) + dim, q_rot + ((size_t)t * H + h) * rot, rot, rot_dims, turn, lane, 32);
    }
    const T* latent = row + (queries ? (size_t)kv_col : (size_t)H * (dim + rot));
    T* kept = cache + slot * (size_t)(rank + rot);
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = to_float(latent[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.f / sqrtf(ss / (float)rank + eps);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) kept[i] = from_float<T>(to_float(latent[i]) * scale * weight[i]);
    if (halves) rotate_halves(latent + rank, kept + rank, rot, rot_dims, turn, (int)threadIdx.x, (int)blockDim.x);
    else rotate_pairs(latent + rank, kept + rank, rot, rot_dims, turn, (int)threadIdx.x, (int)blockDim.x);
    if (fresh) {  // the same row once more, token by token, for whoever wants the step's own rows side by side
        __syncthreads();
        T* copy = fresh + (size_t)t * (rank + rot);
        for (int i = threadIdx.x; i < rank + rot; i += blockDim.x) copy[i] = kept[i];
    }
}

// Attention with unit-RMS queries and keys.  qkv row: [H x dk queries | KV x dk keys | KV x dv values].
//   queries: divided by sqrt(mean(q^2) + eps) per head, in place
//   keys:    the same, written to the key plane of the token's slot;  values: copied to the value plane
// pool plane: [pages, 2, KV, page_size, D] with D >= max(dk, dv).  One warp per head, one block per token.
template <typename T>
__global__ void __launch_bounds__(128)
unit_norm_kv_write_kernel(T* __restrict__ qkv, int ld, const int* __restrict__ slot_map, T* __restrict__ pool, float eps,
                          int normed, int H, int KV, int dk, int dv, int D, int page_size) {
    pdl_trigger();
    const int t = blockIdx.x;
    const int slot = slot_map[t];
    const int page = slot / page_size, off = slot - page * page_size;
    pdl_wait();
    T* row = qkv + (size_t)t * ld;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const size_t head_stride = (size_t)page_size * D;
    for (int item = warp; item < H + 2 * KV; item += warps) {
        if (item < H + KV) {
            const T* src = row + (size_t)item * dk;
            T* dst = item < H ? row + (size_t)item * dk
                              : pool + ((size_t)(page * 2 + 0) * KV + (item - H)) * head_stride + (size_t)off * D;
            float scale = 1.f;
            if (normed) {
                float ss = 0.f;
                for (int i = lane; i < dk; i += 32) {
                    const float v = to_float(src[i]);
                    ss = fmaf(v, v, ss);
                }
                ss = warp_sum(ss);
                scale = 1.f / sqrtf(ss / (float)dk + eps);
            }
            for (int i = lane; i < dk; i += 32) dst[i] = from_float<T>(to_float(src[i]) * scale);
        } else {
            const int h = item - H - KV;
            const T* src = row + (size_t)(H + KV) * dk + (size_t)h * dv;
            T* dst = pool + ((size_t)(page * 2 + 1) * KV + h) * head_stride + (size_t)off * D;
            for (int i = lane; i < dv; i += 32) dst[i] = src[i];
        }
    }
}

}  // namespace

LLM_EXPORT int llm_latent_prepare(const void* proj, int dtype, int ldp, void* q_rot, void* fresh, const int* positions,
                                  const int* slot_map, void* cache, const float* weight, const float* freq, float eps, int n,
                                  int H, int dim, int rot, int rank, int rot_dims, const void* queries, int ldq, int kv_col,
                                  int halves, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (H <= 0 || dim < 0 || rot < 0 || rank <= 0 || rot_dims < 0 || rot_dims > rot || (rot_dims & 1) || rot_dims > 2 * MAX_TURNS ||
        (queries ? (ldq < H * (dim + rot) || kv_col < 0 || ldp < kv_col + rank + rot) : ldp < H * (dim + rot) + rank + rot))
        return LLM_ERR_BAD_ARGUMENT;
    if (dtype == LLM_F32)
        return launch_pdl(latent_prepare_kernel<float>, dim3(n), dim3(128), 0, stream, (const float*)proj, ldp, (float*)q_rot,
                          (float*)fresh, positions, slot_map, (float*)cache, weight, freq, eps, H, dim, rot, rank, rot_dims,
                          (const float*)queries, ldq, kv_col, halves);
    if (dtype == LLM_BF16)
        return launch_pdl(latent_prepare_kernel<__nv_bfloat16>, dim3(n), dim3(128), 0, stream, (const __nv_bfloat16*)proj, ldp,
                          (__nv_bfloat16*)q_rot, (__nv_bfloat16*)fresh, positions, slot_map, (__nv_bfloat16*)cache, weight, freq, eps, H, dim, rot,
                          rank, rot_dims, (const __nv_bfloat16*)queries, ldq, kv_col, halves);
    return LLM_ERR_BAD_ARGUMENT;
}

LLM_EXPORT int llm_unit_norm_kv_write(void* qkv, int dtype, int ld, const int* slot_map, void* pool, float eps, int normed,
                                      int n, int H, int KV, int dk, int dv, int D, int page_size, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (H <= 0 || KV <= 0 || dk <= 0 || dv <= 0 || D < dk || D < dv || page_size <= 0 || ld < (H + KV) * dk + KV * dv)
        return LLM_ERR_BAD_ARGUMENT;
    if (dtype == LLM_F32)
        return launch_pdl(unit_norm_kv_write_kernel<float>, dim3(n), dim3(128), 0, stream, (float*)qkv, ld, slot_map,
                          (float*)pool, eps, normed, H, KV, dk, dv, D, page_size);
    if (dtype == LLM_BF16)
        return launch_pdl(unit_norm_kv_write_kernel<__nv_bfloat16>, dim3(n), dim3(128), 0, stream, (__nv_bfloat16*)qkv, ld,
                          slot_map, (__nv_bfloat16*)pool, eps, normed, H, KV, dk, dv, D, page_size);
    return LLM_ERR_BAD_ARGUMENT;
}
