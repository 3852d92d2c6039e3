// The arguments of attention in its general form, shared by the kernels that take it.
#pragma once

#include "common.cuh"

// Where queries, keys and values lie.  A query is one or two runs of lanes (the second may be absent): run 0 holds
// lanes [0, d0), run 1 lanes [d0, d0 + d1); each run is addressed by a token stride and a head stride.  Keys and
// values are addressed by page, key/value head and place in the page; values may be the first dv lanes of the keys
// (the same pointer and strides).
template <typename T>
struct RowsArgs {
    const T *q0, *q1;
    long long q0_token, q0_head, q1_token, q1_head;
    int d0, d1;
    T* out;
    long long out_token, out_head;
    const T *keys, *values;
    long long k_page, k_head, k_token, v_page, v_head, v_token;
    int dv;
    const int *page_table, *token_request, *cu_tokens, *ctx_lens;
    const float* slopes;  // per query head: the score of key j for the query at position i loses slope * (i - j); null: none
    int table_width, n_tokens, H, KV, page_size, window;
    // With a window, keys at positions below keep_first stay visible to every later query (0: none).  chunk > 0: a query
    // sees only keys of its own block of `chunk` positions, counted from position 0.
    int keep_first, chunk;
    float scale;
    // > 0: a score s (scaled) becomes softcap * tanh(s / softcap) before the distance bias is taken off
    float softcap;
    // Which keys: 0 all that a row sees; 1 only those cached before this step (positions before the request's first new
    // token); 2 only the step's own tokens, whose keys and values then lie token by token, not in pages: token i of the
    // flat batch at keys + i * k_token + head * k_head (lanes [0, fresh_d0)) and at keys1 + i * k1_token (the lanes
    // behind them, shared by all heads; null: all lanes at keys), its value at values + i * v_token + head * v_head.
    int key_part;
    const T* keys1;
    long long k1_token;
    int fresh_d0;
    // [n_tokens, H, 2] (or null): the row's maximum score (times log2 e) and the sum of its exponentials, for a merge of two parts; a
    // row that saw no key says (-inf, 0) and its output is not to be read
    float* stats;
    // per query head (or null): one more term exp(sinks[h]) in the softmax's denominator, with no key and no value; it is
    // not scaled and counts once
    const float* sinks;
    // [n_tokens, gate_token] float32 (or null): the output of head h, lane d is multiplied by sigmoid(gate[t, h * dv + d])
    const float* gate;
    long long gate_token;
};

