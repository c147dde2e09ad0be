// Run-time seed selection for seed-only decode: score every block of the K cache against the
// current query, then pick each (row, KV head) pair's middle seed blocks by score - on the
// device, so the block list never visits the host and the decode that consumes it can be
// enqueued right behind.
//
//   block_scores_kernel   scores[b, q head, block] = max_t q.k_t   (qk_block_max)
//                                                  or mean_t q.k_t (block_mean_proxy: the dot with
//                                                  the block's mean key), t over the block's
//                                                  valid tokens; -inf for blocks without tokens.
//                         One warp per block, one lane per token: the lane walks its key row in
//                         16-byte pieces and keeps one dot product per query head of the KV
//                         group (queries sit in shared memory, read as broadcasts), then the
//                         warp reduces over the tokens.  HBM traffic: the K cache, once.
//   select_blocks_kernel  per (row, KV head): score of a block = max over the group's query
//                         heads; base blocks (sink + recent) are always kept; the `middle`
//                         best-scoring other blocks join them (ties: lower index first, as the
//                         reference's sort key (-score, index) orders them); if fewer than
//                         `middle` blocks have a finite score the policy's fixed middle blocks
//                         fill up.  Output: the pair's block list in ascending order.
#include "sa_common.cuh"

namespace sa {

namespace {

constexpr int kScoreWarps = 8;
constexpr int kScoreMaxGroup = 16;
constexpr int kSelectThreads = 256;

struct ScoreParams {
    const void *q;
    const void *k;
    float *scores;           // [batch, q_heads, num_blocks]
    const void *seq_lens;    // optional per-row valid lengths
    int lens_i64;
    int batch, q_heads, kv_heads, head_dim;
    int64_t q_sb, q_sh;
    int64_t kv_sb, kv_sn, kv_sh;
    int64_t kv_len;
    int block_size, num_blocks;
    int selector;            // SA_SELECT_*
};

template <typename T>
__global__ void __launch_bounds__(kScoreWarps * 32)
block_scores_kernel(const __grid_constant__ ScoreParams p)
{
    extern __shared__ __align__(16) float q_sm[];  // [group][head_dim]
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int group = p.q_heads / p.kv_heads;
    const int pair = blockIdx.y;  // row * kv_heads + kv head
    const int b = pair / p.kv_heads;
    const int kvh = pair - b * p.kv_heads;
    const int D = p.head_dim;
    for (int i = threadIdx.x; i < group * D; i += kScoreWarps * 32) {
        const int h = i / D, d = i - h * D;
        q_sm[i] = Elem<T>::to_float(static_cast<const T *>(p.q)[b * p.q_sb + (static_cast<int64_t>(kvh) * group + h) * p.q_sh + d]);
    }
    __syncthreads();
    int64_t n = p.seq_lens ? load_index(p.seq_lens, p.lens_i64, b) : p.kv_len;
    n = n < 0 ? 0 : (n > p.kv_len ? p.kv_len : n);
    const T *k_pair = static_cast<const T *>(p.k) + b * p.kv_sb + kvh * p.kv_sh;
    for (int blk = blockIdx.x * kScoreWarps + warp; blk < p.num_blocks; blk += gridDim.x * kScoreWarps) {
        float best[kScoreMaxGroup], total[kScoreMaxGroup];
#pragma unroll
        for (int h = 0; h < kScoreMaxGroup; ++h) {
            best[h] = -INFINITY;
            total[h] = 0.0f;
        }
        const int64_t t0 = static_cast<int64_t>(blk) * p.block_size;
        int count = 0;
        for (int off = lane; off < p.block_size; off += 32) {  // one token per lane and round
            const int64_t t = t0 + off;
            if (t >= n) continue;
            ++count;
            const T *row = k_pair + t * p.kv_sn;
            float dot[kScoreMaxGroup];
#pragma unroll
            for (int h = 0; h < kScoreMaxGroup; ++h) dot[h] = 0.0f;
            for (int d = 0; d < D; d += 8) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(row + d);  // 8 elements
                const T *e = reinterpret_cast<const T *>(&raw);
                float kf[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) kf[j] = Elem<T>::to_float(e[j]);
#pragma unroll
                for (int h = 0; h < kScoreMaxGroup; ++h) {
                    if (h < group) {
                        const float4 qa = *reinterpret_cast<const float4 *>(q_sm + h * D + d);
                        const float4 qb = *reinterpret_cast<const float4 *>(q_sm + h * D + d + 4);
                        dot[h] += kf[0] * qa.x + kf[1] * qa.y + kf[2] * qa.z + kf[3] * qa.w + kf[4] * qb.x +
                                  kf[5] * qb.y + kf[6] * qb.z + kf[7] * qb.w;
                    }
                }
            }
#pragma unroll
            for (int h = 0; h < kScoreMaxGroup; ++h) {
                best[h] = fmaxf(best[h], dot[h]);
                total[h] += dot[h];
            }
        }
        count = static_cast<int>(warp_sum(static_cast<float>(count)));
#pragma unroll
        for (int h = 0; h < kScoreMaxGroup; ++h) {
            if (h < group) {
                const float mx = warp_max(best[h]);
                const float sum = warp_sum(total[h]);
                if (lane == 0) {
                    float s = -INFINITY;
                    if (count > 0) s = p.selector == SA_SELECT_BLOCK_MEAN ? sum / static_cast<float>(count) : mx;
                    p.scores[(static_cast<int64_t>(b) * p.q_heads + kvh * group + h) * p.num_blocks + blk] = s;
                }
            }
        }
    }
}

struct SelectParams {
    const float *scores;     // [batch, q_heads, num_blocks]
    int32_t *blocks_out;     // [batch * kv_heads, list_len], ascending
    int batch, q_heads, kv_heads;
    int num_blocks;
    int sink_blocks, recent_blocks, middle_blocks, block_order;
    int list_len;            // sink + recent + middle after de-duplication (host-computed)
};

// Whether block `blk` belongs to the base set (sink or recent blocks).
__device__ __forceinline__ bool is_base_block(const SelectParams &p, int blk)
{
    return blk < p.sink_blocks || blk >= p.num_blocks - p.recent_blocks;
}

__global__ void __launch_bounds__(kSelectThreads)
select_blocks_kernel(const __grid_constant__ SelectParams p)
{
    extern __shared__ __align__(16) float pair_scores[];  // [num_blocks]: max over the group's heads, -inf once taken/base
    __shared__ float red_score[kSelectThreads / 32];
    __shared__ int red_index[kSelectThreads / 32];
    __shared__ int chosen[SA_MAX_SEED_BLOCKS];
    __shared__ int n_chosen;
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int pair = blockIdx.x;
    const int b = pair / p.kv_heads, kvh = pair - b * p.kv_heads;
    const int group = p.q_heads / p.kv_heads;
    for (int blk = tid; blk < p.num_blocks; blk += kSelectThreads) {
        float s = -INFINITY;
        if (!is_base_block(p, blk)) {
            for (int h = 0; h < group; ++h) {
                const float v = p.scores[(static_cast<int64_t>(b) * p.q_heads + kvh * group + h) * p.num_blocks + blk];
                if (isfinite(v)) s = fmaxf(s, v);  // non-finite scores never select a block
            }
        }
        pair_scores[blk] = s;
    }
    if (tid == 0) {
        int n = 0;  // base blocks first: sink, then recent (de-duplicated)
        for (int blk = 0; blk < p.sink_blocks && blk < p.num_blocks; ++blk) chosen[n++] = blk;
        for (int blk = max(p.num_blocks - p.recent_blocks, 0); blk < p.num_blocks; ++blk)
            if (blk >= p.sink_blocks) chosen[n++] = blk;
        n_chosen = n;
    }
    __syncthreads();
    // `middle` rounds of arg-max over the remaining blocks: larger score first, lower index on ties.
    for (int round = 0; round < p.middle_blocks && n_chosen < p.list_len; ++round) {
        float s = -INFINITY;
        int idx = 0x7fffffff;
        for (int blk = tid; blk < p.num_blocks; blk += kSelectThreads) {
            const float v = pair_scores[blk];
            if (v > s || (v == s && v > -INFINITY && blk < idx)) {
                s = v;
                idx = blk;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float os = __shfl_xor_sync(0xffffffffu, s, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (os > s || (os == s && oi < idx)) {
                s = os;
                idx = oi;
            }
        }
        if (lane == 0) {
            red_score[warp] = s;
            red_index[warp] = idx;
        }
        __syncthreads();
        if (tid == 0) {
            float bs = -INFINITY;
            int bi = 0x7fffffff;
            for (int w = 0; w < kSelectThreads / 32; ++w)
                if (red_score[w] > bs || (red_score[w] == bs && red_index[w] < bi)) {
                    bs = red_score[w];
                    bi = red_index[w];
                }
            if (bs > -INFINITY) {
                chosen[n_chosen++] = bi;
                pair_scores[bi] = -INFINITY;
            } else {
                n_chosen = -n_chosen - 1;  // no scored block is left: stop the rounds
            }
        }
        __syncthreads();
        if (n_chosen < 0) break;
    }
    if (tid == 0) {
        int n = n_chosen < 0 ? -n_chosen - 1 : n_chosen;
        // Fewer scored blocks than asked for: the policy's fixed middle blocks fill up.
        const int recent_start = p.num_blocks - p.recent_blocks;
        for (int i = 0; i < p.middle_blocks && n < p.list_len; ++i) {
            const int blk = p.block_order == SA_ORDER_SEQUENTIAL ? p.sink_blocks + i : recent_start - 1 - i;
            if (blk < 0 || blk >= p.num_blocks || is_base_block(p, blk)) continue;
            bool seen = false;
            for (int j = 0; j < n; ++j) seen |= chosen[j] == blk;
            if (!seen) chosen[n++] = blk;
        }
        // Still short (a cache with fewer blocks than the list): repeat nothing, pad with the
        // last block so the list stays ascending; the host sizes list_len so this cannot happen
        // when there are at least list_len blocks.
        n_chosen = n;
    }
    __syncthreads();
    // Ascending order by rank (lists are short), padding with the largest entry.
    const int n = n_chosen;
    for (int i = tid; i < n; i += kSelectThreads) {
        const int mine = chosen[i];
        int rank = 0;
        for (int j = 0; j < n; ++j) rank += chosen[j] < mine;
        p.blocks_out[static_cast<int64_t>(pair) * p.list_len + rank] = mine;
    }
    if (n < p.list_len && n > 0) {
        int largest = 0;
        for (int j = 0; j < n; ++j) largest = max(largest, chosen[j]);
        for (int i = n + tid; i < p.list_len; i += kSelectThreads)
            p.blocks_out[static_cast<int64_t>(pair) * p.list_len + i] = largest;
    }
}

}  // namespace

cudaError_t launch_block_scores(const void *q, const void *k, float *scores, const void *seq_lens, int lens_i64,
                                int batch, int q_heads, int kv_heads, int head_dim, int64_t kv_len, int64_t q_sb,
                                int64_t q_sh, int64_t kv_sb, int64_t kv_sn, int64_t kv_sh, int dtype, int block_size,
                                int selector, cudaStream_t stream)
{
    ScoreParams p;
    p.q = q; p.k = k; p.scores = scores;
    p.seq_lens = seq_lens; p.lens_i64 = lens_i64;
    p.batch = batch; p.q_heads = q_heads; p.kv_heads = kv_heads; p.head_dim = head_dim;
    p.q_sb = q_sb; p.q_sh = q_sh;
    p.kv_sb = kv_sb; p.kv_sn = kv_sn; p.kv_sh = kv_sh;
    p.kv_len = kv_len;
    p.block_size = block_size;
    p.num_blocks = static_cast<int>((kv_len + block_size - 1) / block_size);
    p.selector = selector;
    const int group = q_heads / kv_heads;
    const unsigned per_pair = static_cast<unsigned>((p.num_blocks + kScoreWarps - 1) / kScoreWarps);
    dim3 grid(per_pair < 1024u ? per_pair : 1024u, static_cast<unsigned>(batch * kv_heads));
    const size_t smem = static_cast<size_t>(group) * head_dim * sizeof(float);
    if (dtype == SA_DTYPE_BF16)
        block_scores_kernel<__nv_bfloat16><<<grid, kScoreWarps * 32, smem, stream>>>(p);
    else
        block_scores_kernel<__half><<<grid, kScoreWarps * 32, smem, stream>>>(p);
    return cudaGetLastError();
}

cudaError_t launch_select_blocks(const float *scores, int32_t *blocks_out, int batch, int q_heads, int kv_heads,
                                 int num_blocks, int sink_blocks, int recent_blocks, int middle_blocks,
                                 int block_order, int list_len, cudaStream_t stream)
{
    SelectParams p;
    p.scores = scores;
    p.blocks_out = blocks_out;
    p.batch = batch; p.q_heads = q_heads; p.kv_heads = kv_heads;
    p.num_blocks = num_blocks;
    p.sink_blocks = sink_blocks; p.recent_blocks = recent_blocks; p.middle_blocks = middle_blocks;
    p.block_order = block_order;
    p.list_len = list_len;
    const size_t smem = static_cast<size_t>(num_blocks) * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(select_blocks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(smem));
        if (err != cudaSuccess) return err;
    }
    select_blocks_kernel<<<batch * kv_heads, kSelectThreads, smem, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace sa
