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
    float scale;
};

