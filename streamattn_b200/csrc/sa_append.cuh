// KV-cache update step (rotary embedding + append of the current token's K/V row, optional
// query rotation): launch descriptor shared by the entry points and the kernel.
#pragma once

#include "sa_common.cuh"

namespace sa {

struct AppendParams {
    // current token: [batch, kv_heads, D] rows
    const void *k_new;
    const void *v_new;
    int64_t new_sb, new_sh;
    // destination cache
    void *k_cache;
    void *v_cache;
    int paged;                      // 0: contiguous (kv_* strides), 1: paged (page table + pg_* strides)
    int64_t kv_sb, kv_sn, kv_sh;    // contiguous cache addressing (elements)
    int64_t capacity;               // tokens a row can hold
    const void *page_table;
    int table_i64;
    int max_pages;
    int page_size;
    int64_t num_pages;
    int64_t pg_sp, pg_st, pg_sh;    // page*sp + slot*st + head*sh
    // where to write
    const void *positions;
    int pos_i64;
    int pos_shared;                 // 1: positions[0] serves every row
    void *lens_out;                 // optional: position + 1 per row (same integer type)
    // rotary embedding (optional)
    const void *cos;
    const void *sin;
    int64_t rope_sb;                // 0: one row shared by the batch
    // query rotation (optional)
    const void *q_in;
    void *q_out;
    int q_heads;
    int64_t qi_sb, qi_sh, qo_sb, qo_sh;
    int batch, kv_heads, head_dim;
    int dtype;
    int *status;
};

cudaError_t launch_append(const AppendParams &p, cudaStream_t stream);

}  // namespace sa
