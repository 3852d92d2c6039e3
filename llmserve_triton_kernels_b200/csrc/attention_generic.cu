// Paged attention for any mix of query lengths, any key size up to 640 lanes, any value size up to 512 and any
// group size: one warp per (token, query head).
//
// This is the attention of the true 32-bit path and the fallback of the bfloat16 path for
// shapes its faster kernels refuse.  Scores, the running maximum, the exponentials and the
// weighted sum are 32-bit.  Keys are visited in chunks of 32 that start at multiples of 32 of
// the absolute key position, so the order of every addition depends only on the query's
// position (and the window), never on how the tokens were cut into steps or batched.
//
// A query at position p of request r sees keys max(0, p - window + 1) .. p (window <= 0: from 0), with a window also the
// keys below keep_first; with chunk > 0 only those from the start of its own block of chunk positions on.
#include <type_traits>

#include "attention_rows.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_DK = 640;  // most lanes of a query and a key
constexpr int MAX_DV = 512;  // most lanes of a value

template <typename T>
__global__ void __launch_bounds__(WARPS * 32) attention_rows_kernel(const RowsArgs<T> a) {
    __shared__ float q_s[WARPS][MAX_DK];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)a.n_tokens * a.H) return;
    const int t = (int)(item / a.H), h = (int)(item - (long long)t * a.H);
    const int r = a.token_request[t];
    const int q_begin = a.cu_tokens[r], q_len = a.cu_tokens[r + 1] - q_begin;
    const int pos = a.ctx_lens[r] - q_len + (t - q_begin);
    const int kvh = h / (a.H / a.KV);
    int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    if (a.chunk > 0) lo = max(lo, pos - pos % a.chunk);
    const int kept = a.window > 0 ? min(a.keep_first, lo) : 0;  // keys [0, kept) are seen besides [lo, pos]
    const int dk = a.d0 + a.d1, dv = a.dv;
    const float slope = a.slopes ? a.slopes[h] : 0.f;

    const T* qp = a.q0 + (long long)t * a.q0_token + (long long)h * a.q0_head;
    for (int d = lane; d < a.d0; d += 32) q_s[warp][d] = to_float(qp[d]);
    if (a.d1 > 0) {
        const T* qr = a.q1 + (long long)t * a.q1_token + (long long)h * a.q1_head;
        for (int d = lane; d < a.d1; d += 32) q_s[warp][a.d0 + d] = to_float(qr[d]);
    }
    __syncwarp();

    const int* table = a.page_table + (size_t)r * a.table_width;
    constexpr int ACC = MAX_DV / 32;
    float acc[ACC];
#pragma unroll
    for (int i = 0; i < ACC; ++i) acc[i] = 0.f;
    // a sink stands for a key of score sinks[h] and no value: the running maximum and sum start from it
    float m = a.sinks ? a.sinks[h] : -INFINITY, l = a.sinks ? 1.f : 0.f;

    const int c_lo = (lo / 32) * 32, c_kept = ((kept + 31) / 32) * 32;  // the chunks of the kept keys end before c_kept
    for (int c = kept > 0 ? 0 : c_lo; c <= pos; c += 32) {
        if (c >= c_kept && c < c_lo) c = c_lo;  // nothing is seen between the kept keys and the window
        const int j = c + lane;
        const bool visible = (j >= lo && j <= pos) || j < kept;
        float s = -INFINITY;
        if (visible) {
            const int page = table[j / a.page_size], off = j % a.page_size;
            const T* kp = a.keys + (long long)page * a.k_page + (long long)kvh * a.k_head + (long long)off * a.k_token;
            float dot = 0.f;
            for (int d = 0; d < dk; ++d) dot = fmaf(q_s[warp][d], to_float(kp[d]), dot);
            s = dot * a.scale;
            if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
            s -= slope * (float)(pos - j);
        }
        const float m_new = fmaxf(m, warp_max(s));  // finite: the chunk holds at least one visible key
        const float p = visible ? expf(s - m_new) : 0.f;
        const float rescale = expf(m - m_new);  // 0 on the first chunk (m = -inf)
        l = l * rescale + warp_sum(p);
#pragma unroll
        for (int i = 0; i < ACC; ++i) acc[i] *= rescale;
        m = m_new;
        const int count = min(32, pos - c + 1);
        for (int jj = 0; jj < count; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            if (pj == 0.f) continue;  // uniform across the warp
            const int key = c + jj;
            const int page = table[key / a.page_size], off = key % a.page_size;
            const T* vp = a.values + (long long)page * a.v_page + (long long)kvh * a.v_head + (long long)off * a.v_token;
#pragma unroll
            for (int i = 0; i < ACC; ++i) {
                const int d = lane + 32 * i;
                if (d < dv) acc[i] = fmaf(pj, to_float(vp[d]), acc[i]);
            }
        }
    }
    const float inv = 1.f / l;
    T* op = a.out + (long long)t * a.out_token + (long long)h * a.out_head;
    const float* gp = a.gate ? a.gate + (long long)t * a.gate_token + (long long)h * dv : nullptr;
#pragma unroll
    for (int i = 0; i < ACC; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) {
            float y = acc[i] * inv;
            if (gp) y *= 1.f / (1.f + expf(-gp[d]));
            op[d] = from_float<T>(y);
        }
    }
}

template <typename T>
int launch_rows(const RowsArgs<T>& a, cudaStream_t stream) {
    const long long items = (long long)a.n_tokens * a.H;
    const long long blocks = (items + WARPS - 1) / WARPS;
    if (blocks > 0x7fffffffLL) return LLM_ERR_UNSUPPORTED;
    attention_rows_kernel<T><<<(unsigned)blocks, WARPS * 32, 0, stream>>>(a);
    return launch_status();
}

}  // namespace

// Queries in two runs of lanes, keys and values by strides, an optional distance bias per head: the form that
// attention with other key than value sizes, and attention over a latent that is key and value at once, come in.
LLM_EXPORT int llm_attention_rows(const void* q0, long long q0_token, long long q0_head, int d0, const void* q1,
                                  long long q1_token, long long q1_head, int d1, void* out, long long out_token,
                                  long long out_head, const void* keys, long long k_page, long long k_head, long long k_token,
                                  const void* values, long long v_page, long long v_head, long long v_token, int dv, int dtype,
                                  const int* page_table, int table_width, const int* token_request, const int* cu_tokens,
                                  const int* ctx_lens, const float* slopes, int n_tokens, int H, int KV, int page_size,
                                  int window, float scale, const float* sinks, const float* gate, long long gate_token,
                                  int keep_first, int chunk, float softcap, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (keep_first < 0 || chunk < 0 || d0 <= 0 || d1 < 0 || d0 + d1 > MAX_DK || dv <= 0 || dv > MAX_DV || H <= 0 || KV <= 0 || H % KV || page_size <= 0 ||
        table_width <= 0 || (d1 > 0 && q1 == nullptr))
        return LLM_ERR_BAD_ARGUMENT;
    auto fill = [&](auto& a, auto* tag) {
        using T = std::remove_pointer_t<decltype(tag)>;
        a.q0 = (const T*)q0; a.q1 = (const T*)q1;
        a.q0_token = q0_token; a.q0_head = q0_head; a.q1_token = q1_token; a.q1_head = q1_head;
        a.d0 = d0; a.d1 = d1;
        a.out = (T*)out; a.out_token = out_token; a.out_head = out_head;
        a.keys = (const T*)keys; a.values = (const T*)values;
        a.k_page = k_page; a.k_head = k_head; a.k_token = k_token; a.v_page = v_page; a.v_head = v_head; a.v_token = v_token;
        a.dv = dv;
        a.page_table = page_table; a.token_request = token_request; a.cu_tokens = cu_tokens; a.ctx_lens = ctx_lens;
        a.slopes = slopes;
        a.table_width = table_width; a.n_tokens = n_tokens; a.H = H; a.KV = KV; a.page_size = page_size; a.window = window;
        a.scale = scale; a.keep_first = keep_first; a.chunk = chunk; a.softcap = softcap;
        a.key_part = 0; a.keys1 = nullptr; a.k1_token = 0; a.fresh_d0 = 0; a.stats = nullptr;
        a.sinks = sinks; a.gate = gate; a.gate_token = gate_token;
    };
    if (dtype == LLM_F32) {
        RowsArgs<float> a;
        fill(a, (float*)nullptr);
        return launch_rows(a, stream);
    }
    if (dtype == LLM_BF16) {
        RowsArgs<__nv_bfloat16> a;
        fill(a, (__nv_bfloat16*)nullptr);
        return launch_rows(a, stream);
    }
    return LLM_ERR_BAD_ARGUMENT;
}

// Queries of one run at the head of their rows, keys and values of one size D in a pool plane [pages, 2, KV, page_size, D].
LLM_EXPORT int llm_attention_generic(const void* q, int q_stride, void* out, int out_stride, const void* pool,
                                     int dtype, const int* page_table, int table_width, const int* token_request,
                                     const int* cu_tokens, const int* ctx_lens, int n_tokens, int H, int KV, int D,
                                     int page_size, int window, float scale, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (D <= 0 || D > 256 || H <= 0 || KV <= 0 || H % KV || page_size <= 0 || table_width <= 0)
        return LLM_ERR_BAD_ARGUMENT;
    const long long head = (long long)page_size * D, page = 2LL * KV * head;
    const size_t element = dtype == LLM_F32 ? 4 : 2;
    const void* values = (const char*)pool + (size_t)KV * head * element;
    return llm_attention_rows(q, q_stride, D, D, nullptr, 0, 0, 0, out, out_stride, D, pool, page, head, D, values, page, head,
                              D, D, dtype, page_table, table_width, token_request, cu_tokens, ctx_lens, nullptr, n_tokens, H,
                              KV, page_size, window, scale, nullptr, nullptr, 0, 0, 0, 0.f, stream);
}
