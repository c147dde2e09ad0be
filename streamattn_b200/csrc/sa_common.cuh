// Shared definitions of the decode-attention kernels: the launch descriptor that
// every C-ABI entry point fills, the virtual-sequence addressing shared by the
// contiguous / paged / seed-block modes, and small device helpers.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/streamattn_b200.h"

namespace sa {

constexpr int kStatusWords = 64;        // int32 status area at the head of the workspace
constexpr int kMaxAutoCtas = 256;       // bound used for workspace sizing
constexpr int kMaxCtas = 4096;
constexpr int kMaxGenericSplits = 64;
constexpr int kMaxSeedBlocks = SA_MAX_SEED_BLOCKS;
constexpr float kLog2e = 1.4426950408889634f;

enum SeqMode : int { kContig = 0, kPaged = 1, kBlocks = 2 };

// A "virtual sequence" per batch row: the tokens a row attends to, in order.
//   kContig : virtual token t is cache token t                    (len from seq_lens/kv_len)
//   kPaged  : virtual token t is slot t%page of page_table[b][t/page]
//   kBlocks : virtual token t is cache token blocks[t/bs]*bs+t%bs (seed-only decode)
struct SeqDesc {
    int mode;
    // contiguous cache addressing (elements)
    int64_t kv_sb, kv_sn, kv_sh;
    int64_t kv_len;
    // optional per-row lengths
    const void *seq_lens;
    int lens_i64;
    // optional row subset: only the batch rows listed here are computed and written
    // (entries outside [0, batch) are ignored, duplicates are harmless); num_rows < 0 = every row
    const void *rows;
    int rows_i64;
    int num_rows;
    // paged addressing (elements): page*sp + slot*st + head*sh
    const void *page_table;
    int table_i64;
    int max_pages;
    int page_size;
    int64_t num_pages;
    int64_t pg_sp, pg_st, pg_sh;
    // seed blocks (ascending, unique): one list for the whole call (`blocks`), or - when
    // blocks_dev is set - one device-resident list of num_blocks entries per (row, kv head) pair,
    // pair = row * blocks_kv_heads + kv head
    int block_size;
    int num_blocks;
    int64_t blocks_vlen;  // number of valid virtual tokens of the block list
    const int32_t *blocks_dev;
    int blocks_kv_heads;
    int32_t blocks[kMaxSeedBlocks];
};

__host__ __device__ inline int64_t load_index(const void *p, int is_i64, int64_t i)
{
    return is_i64 ? static_cast<const int64_t *>(p)[i]
                  : static_cast<int64_t>(static_cast<const int32_t *>(p)[i]);
}

// Whether batch row b is computed by this call (linear scan of the row list: for the kernels
// that handle one row per CTA; the streaming kernel builds a table in shared memory instead).
__device__ inline bool row_selected(const SeqDesc &s, int b)
{
    if (s.num_rows < 0) return true;
    for (int i = 0; i < s.num_rows; ++i)
        if (load_index(s.rows, s.rows_i64, i) == b) return true;
    return false;
}

// Valid virtual length of row b.
__device__ inline int64_t row_vlen(const SeqDesc &s, int b)
{
    if (s.mode == kBlocks) return s.blocks_vlen;
    int64_t cap = s.mode == kPaged ? static_cast<int64_t>(s.max_pages) * s.page_size : s.kv_len;
    int64_t n = s.seq_lens ? load_index(s.seq_lens, s.lens_i64, b) : cap;
    if (n < 0) n = 0;
    return n < cap ? n : cap;
}

struct Workspace {
    int *status;
    int *counters;
    float *partials;
    size_t partial_floats;
};

// Everything a launch needs; filled by the entry points in sa_api.cu.
struct Problem {
    const void *q;
    const void *k;
    const void *v;
    void *out;
    int dtype;
    int out_mode;
    int batch, q_heads, kv_heads, head_dim;
    int64_t q_sb, q_sh;
    SeqDesc seq;
    Workspace ws;
    int32_t *trace;
    int num_ctas;  // requested (0 = auto)
    int sm_count;
    unsigned long long wait_ns;  // limit of every bounded device-side wait of the launch
};

constexpr unsigned long long kDefaultWaitNs = 2000000000ull;  // 2 s

template <typename T> struct Elem;
template <> struct Elem<float> {
    __device__ static float to_float(float x) { return x; }
    __device__ static float from_float(float x) { return x; }
};
template <> struct Elem<__nv_bfloat16> {
    __device__ static float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
    __device__ static __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
};
template <> struct Elem<__half> {
    __device__ static float to_float(__half x) { return __half2float(x); }
    __device__ static __half from_float(float x) { return __float2half_rn(x); }
};

__device__ inline float warp_max(float x)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}

__device__ inline float warp_sum(float x)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// 2^(a-b) with the convention 2^(-inf - anything) = 0 even when b is -inf.
__device__ inline float exp2_diff(float a, float b)
{
    return a == -INFINITY ? 0.0f : exp2f(a - b);
}

// Host-side launchers (one per kernel family); return a cudaError_t.
cudaError_t launch_generic(const Problem &p, int splits, cudaStream_t stream);
int generic_splits(const Problem &p, int64_t max_vlen);
size_t generic_partial_floats(int batch, int q_heads, int head_dim, int splits);

cudaError_t launch_merge_states(const float *states, int parts, int64_t rows, int dim, void *out,
                                int out_dtype, cudaStream_t stream);

size_t exchange_bytes(int world, int64_t rows, int dim);
size_t exchange_status_offset(int world, int64_t rows, int dim);
cudaError_t launch_exchange_merge(const float *local_state, const uint64_t *bases_host, int world, int rank,
                                  uint32_t step, int64_t rows, int dim, void *out, int out_dtype,
                                  unsigned long long wait_ns, cudaStream_t stream);

cudaError_t launch_block_scores(const void *q, const void *k, float *scores, const void *seq_lens, int lens_i64,
                                int batch, int q_heads, int kv_heads, int head_dim, int64_t kv_len, int64_t q_sb,
                                int64_t q_sh, int64_t kv_sb, int64_t kv_sn, int64_t kv_sh, int dtype, int block_size,
                                int selector, cudaStream_t stream);
cudaError_t launch_select_blocks(const float *scores, int32_t *blocks_out, int batch, int q_heads, int kv_heads,
                                 int num_blocks, int sink_blocks, int recent_blocks, int middle_blocks,
                                 int block_order, int list_len, cudaStream_t stream);

cudaError_t launch_o_proj(const void *x, const void *w, const void *bias, void *out, int batch, int in_features,
                          int out_features, int64_t x_stride, int dtype, int prefetch_weights, cudaStream_t stream);

struct StreamGeometry;  // defined in sa_stream.cuh

}  // namespace sa
