// Generic CUDA-core decode kernel: any float dtype, any head_dim <= 256, any
// strides / page size / layout.  It covers what the TMA + tensor-core streaming
// kernel (sa_stream.cu) does not: fp32 caches, small or odd head sizes, tiny
// pages, misaligned views.  One CTA handles one (row, query head, split); a
// second launch merges the split states exactly.  Also hosts the state-merge
// kernel used after the cross-GPU gather of context-parallel decode.
#include "sa_common.cuh"

namespace sa {

namespace {

constexpr int kGenericWarps = 4;
constexpr int kGenericThreads = kGenericWarps * 32;
constexpr int kMaxDim = 256;

struct GenericParams {
    const void *q;
    const void *k;
    const void *v;
    void *out;
    int out_mode;
    int batch, q_heads, kv_heads, head_dim;
    int64_t q_sb, q_sh;
    SeqDesc seq;
    int *status;
    float *partials;
    int32_t *trace;
    int splits;
    float scale_log2;
};

// Element offset of virtual token t of (row b, kv head h); -1 when the page
// entry is out of range (the token is then skipped, never dereferenced).
__device__ inline int64_t token_offset(const SeqDesc &s, int b, int kvh, int64_t t, int64_t *page_out)
{
    if (s.mode == kContig) return b * s.kv_sb + t * s.kv_sn + kvh * s.kv_sh;
    if (s.mode == kBlocks) {
        const int64_t bi = t / s.block_size;
        const int64_t blk = s.blocks_dev != nullptr
                                ? s.blocks_dev[(static_cast<int64_t>(b) * s.blocks_kv_heads + kvh) * s.num_blocks + bi]
                                : s.blocks[bi];
        const int64_t tok = blk * s.block_size + t % s.block_size;
        *page_out = blk;
        if (blk < 0 || tok >= s.kv_len) return -1;  // device lists are not host-checked: skip and report
        return b * s.kv_sb + tok * s.kv_sn + kvh * s.kv_sh;
    }
    int64_t lp = t / s.page_size;
    int64_t page = load_index(s.page_table, s.table_i64, static_cast<int64_t>(b) * s.max_pages + lp);
    *page_out = page;
    if (page < 0 || page >= s.num_pages) return -1;
    return page * s.pg_sp + (t % s.page_size) * s.pg_st + kvh * s.pg_sh;
}

template <typename T>
__global__ void __launch_bounds__(kGenericThreads)
generic_partial_kernel(const __grid_constant__ GenericParams p)
{
    __shared__ float sm_q[kMaxDim];
    __shared__ float sm_m[kGenericWarps];
    __shared__ float sm_l[kGenericWarps];
    __shared__ float sm_o[kGenericWarps][kMaxDim];

    const int pair = blockIdx.y;
    const int split = blockIdx.x;
    const int b = pair / p.q_heads;
    const int h = pair % p.q_heads;
    const int group = p.q_heads / p.kv_heads;
    const int kvh = h / group;
    const int dim = p.head_dim;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    if (!row_selected(p.seq, b)) return;  // row subset: this row is neither computed nor written
    const T *q = static_cast<const T *>(p.q) + b * p.q_sb + h * p.q_sh;
    const T *kbase = static_cast<const T *>(p.k);
    const T *vbase = static_cast<const T *>(p.v);

    for (int d = threadIdx.x; d < dim; d += kGenericThreads)
        sm_q[d] = Elem<T>::to_float(q[d]) * p.scale_log2;
    __syncthreads();

    const int64_t vlen = row_vlen(p.seq, b);
    int64_t chunk = (vlen + p.splits - 1) / p.splits;
    chunk = (chunk + 31) / 32 * 32;
    const int64_t t_begin = static_cast<int64_t>(split) * chunk;
    const int64_t t_end = t_begin + chunk < vlen ? t_begin + chunk : vlen;

    float m = -INFINITY, l = 0.0f;
    float o[kMaxDim / 32];
#pragma unroll
    for (int i = 0; i < kMaxDim / 32; ++i) o[i] = 0.0f;

    for (int64_t blk = t_begin + warp * 32; blk < t_end; blk += kGenericWarps * 32) {
        const int64_t t = blk + lane;
        bool valid = t < t_end;
        int64_t off = -1;
        if (valid) {
            int64_t page = -1;
            off = token_offset(p.seq, b, kvh, t, &page);
            if (off < 0) {
                valid = false;
                atomicOr(p.status, SA_DEV_BAD_PAGE);
            } else if (p.trace != nullptr && p.seq.mode == kPaged && h == 0 && t % p.seq.page_size == 0) {
                p.trace[static_cast<int64_t>(b) * p.seq.max_pages + t / p.seq.page_size] =
                    static_cast<int32_t>(page);
            }
        }
        float s = -INFINITY;
        if (valid) {
            const T *kr = kbase + off;
            float acc = 0.0f;
            for (int d = 0; d < dim; ++d) acc = fmaf(sm_q[d], Elem<T>::to_float(kr[d]), acc);
            s = acc;
        }
        const float blk_max = warp_max(s);
        if (blk_max == -INFINITY) continue;  // every token of the block was skipped
        const float m_new = fmaxf(m, blk_max);
        const float alpha = exp2_diff(m, m_new);
        const float pr = valid ? exp2f(s - m_new) : 0.0f;
        l = l * alpha + warp_sum(pr);
#pragma unroll
        for (int i = 0; i < kMaxDim / 32; ++i) o[i] *= alpha;
        for (int j = 0; j < 32; ++j) {
            const float pj = __shfl_sync(0xffffffffu, pr, j);
            const int64_t offj = __shfl_sync(0xffffffffu, off, j);
            if (pj == 0.0f || offj < 0) continue;  // warp-uniform
            const T *vr = vbase + offj;
#pragma unroll
            for (int i = 0; i < kMaxDim / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < dim) o[i] = fmaf(pj, Elem<T>::to_float(vr[d]), o[i]);
            }
        }
        m = m_new;
    }

    if (lane == 0) {
        sm_m[warp] = m;
        sm_l[warp] = l;
    }
#pragma unroll
    for (int i = 0; i < kMaxDim / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < dim) sm_o[warp][d] = o[i];
    }
    __syncthreads();

    float big = -INFINITY;
#pragma unroll
    for (int w = 0; w < kGenericWarps; ++w) big = fmaxf(big, sm_m[w]);
    float wgt[kGenericWarps];
    float total_l = 0.0f;
#pragma unroll
    for (int w = 0; w < kGenericWarps; ++w) {
        wgt[w] = exp2_diff(sm_m[w], big);
        total_l += wgt[w] * sm_l[w];
    }
    const bool direct = p.splits == 1;
    for (int d = threadIdx.x; d < dim; d += kGenericThreads) {
        float acc = 0.0f;
#pragma unroll
        for (int w = 0; w < kGenericWarps; ++w) acc += wgt[w] * sm_o[w][d];
        if (direct && p.out_mode == SA_OUT_FINAL) {
            static_cast<T *>(p.out)[static_cast<int64_t>(pair) * dim + d] =
                Elem<T>::from_float(total_l > 0.0f ? acc / total_l : 0.0f);
        } else if (direct) {
            static_cast<float *>(p.out)[static_cast<int64_t>(pair) * (dim + 2) + d] = acc;
        } else {
            p.partials[(static_cast<int64_t>(pair) * p.splits + split) * (dim + 2) + d] = acc;
        }
    }
    if (threadIdx.x == 0 && !(direct && p.out_mode == SA_OUT_FINAL)) {
        float *dst = direct ? static_cast<float *>(p.out) + static_cast<int64_t>(pair) * (dim + 2)
                            : p.partials + (static_cast<int64_t>(pair) * p.splits + split) * (dim + 2);
        dst[dim] = big;
        dst[dim + 1] = total_l;
    }
}

// Exact merge of the `parts` states of one row:  m = max m_i, l = sum l_i 2^(m_i-m),
// o = sum o_i 2^(m_i-m).  State i of row r starts at states + i*part_stride + r*row_stride.
// `scrub` (or null) is the same memory as a writable pointer: the workspace's split states are
// left zero-filled for the next launch, so they are cleared here after use.
template <typename OutT>
__device__ void merge_row(const float *states, int parts, int64_t part_stride, int64_t row_stride, int dim,
                          void *out, int out_mode, float *scrub, int64_t row)
{
    const float *base = states + row * row_stride;
    float big = -INFINITY;
    for (int i = 0; i < parts; ++i) {
        const float *s = base + i * part_stride;
        if (s[dim + 1] > 0.0f) big = fmaxf(big, s[dim]);
    }
    float total_l = 0.0f;
    for (int i = 0; i < parts; ++i) {
        const float *s = base + i * part_stride;
        if (s[dim + 1] > 0.0f) total_l += exp2_diff(s[dim], big) * s[dim + 1];
    }
    for (int d = threadIdx.x; d < dim; d += blockDim.x) {
        float acc = 0.0f;
        for (int i = 0; i < parts; ++i) {
            const float *s = base + i * part_stride;
            if (s[dim + 1] > 0.0f) acc += exp2_diff(s[dim], big) * s[d];
        }
        if (out_mode == SA_OUT_FINAL)
            static_cast<OutT *>(out)[row * dim + d] = Elem<OutT>::from_float(total_l > 0.0f ? acc / total_l : 0.0f);
        else
            static_cast<float *>(out)[row * (dim + 2) + d] = acc;
    }
    if (out_mode != SA_OUT_FINAL && threadIdx.x == 0) {
        static_cast<float *>(out)[row * (dim + 2) + dim] = big;
        static_cast<float *>(out)[row * (dim + 2) + dim + 1] = total_l;
    }
    if (scrub != nullptr) {
        __syncthreads();  // every thread of the row has read what it needs
        float *mine = scrub + row * row_stride;
        for (int i = 0; i < parts; ++i)
            for (int d = threadIdx.x; d < dim + 2; d += blockDim.x) mine[i * part_stride + d] = 0.0f;
    }
}

// Merge of caller-provided states (sa_merge_states): one CTA per row.
template <typename OutT>
__global__ void __launch_bounds__(128)
merge_states_kernel(const float *__restrict__ states, int parts, int64_t part_stride, int64_t row_stride, int dim,
                    void *out, int out_mode)
{
    merge_row<OutT>(states, parts, part_stride, row_stride, dim, out, out_mode, nullptr, blockIdx.x);
}

// Merge of the generic kernel's own split states (cleared after use; honours the row subset).
template <typename T>
__global__ void __launch_bounds__(128)
merge_states_rows_kernel(const __grid_constant__ GenericParams p, int parts, int64_t part_stride, int64_t row_stride)
{
    const int64_t row = blockIdx.x;
    if (!row_selected(p.seq, static_cast<int>(row / p.q_heads))) return;
    merge_row<T>(p.partials, parts, part_stride, row_stride, p.head_dim, p.out, p.out_mode, p.partials, row);
}

template <typename T>
cudaError_t launch_generic_typed(const Problem &p, int splits, cudaStream_t stream)
{
    GenericParams gp;
    gp.q = p.q;
    gp.k = p.k;
    gp.v = p.v;
    gp.out = p.out;
    gp.out_mode = p.out_mode;
    gp.batch = p.batch;
    gp.q_heads = p.q_heads;
    gp.kv_heads = p.kv_heads;
    gp.head_dim = p.head_dim;
    gp.q_sb = p.q_sb;
    gp.q_sh = p.q_sh;
    gp.seq = p.seq;
    gp.status = p.ws.status;
    gp.partials = p.ws.partials;
    gp.trace = p.trace;
    gp.splits = splits;
    gp.scale_log2 = kLog2e / sqrtf(static_cast<float>(p.head_dim));
    const int pairs = p.batch * p.q_heads;
    dim3 grid(splits, pairs);
    generic_partial_kernel<T><<<grid, kGenericThreads, 0, stream>>>(gp);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess || splits == 1) return err;
    const int64_t stride = p.head_dim + 2;
    // The row subset travels by value in the kernel's parameter block (a pointer to host memory
    // would not do): reuse the descriptor inside the launch parameters of the first kernel.
    merge_states_rows_kernel<T><<<pairs, 128, 0, stream>>>(gp, splits, stride, stride * splits);
    return cudaGetLastError();
}

}  // namespace

int generic_splits(const Problem &p, int64_t max_vlen)
{
    const int64_t pairs = static_cast<int64_t>(p.batch) * p.q_heads;
    const int sm = p.sm_count > 0 ? p.sm_count : 148;
    int64_t want = p.num_ctas > 0 ? (p.num_ctas + pairs - 1) / pairs : (4LL * sm + pairs - 1) / pairs;
    const int64_t by_len = (max_vlen + 127) / 128;  // keep >= 128 tokens per split
    if (want > by_len) want = by_len;
    if (want > kMaxGenericSplits) want = kMaxGenericSplits;
    if (want < 1) want = 1;
    return static_cast<int>(want);
}

size_t generic_partial_floats(int batch, int q_heads, int head_dim, int splits)
{
    return static_cast<size_t>(batch) * q_heads * splits * (head_dim + 2);
}

cudaError_t launch_generic(const Problem &p, int splits, cudaStream_t stream)
{
    switch (p.dtype) {
        case SA_DTYPE_BF16: return launch_generic_typed<__nv_bfloat16>(p, splits, stream);
        case SA_DTYPE_F16: return launch_generic_typed<__half>(p, splits, stream);
        default: return launch_generic_typed<float>(p, splits, stream);
    }
}

cudaError_t launch_merge_states(const float *states, int parts, int64_t rows, int dim, void *out,
                                int out_dtype, cudaStream_t stream)
{
    const int64_t part_stride = rows * (dim + 2);
    const int64_t row_stride = dim + 2;
    const unsigned grid = static_cast<unsigned>(rows);
    switch (out_dtype) {
        case SA_DTYPE_BF16:
            merge_states_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(states, parts, part_stride, row_stride,
                                                                         dim, out, SA_OUT_FINAL);
            break;
        case SA_DTYPE_F16:
            merge_states_kernel<__half><<<grid, 128, 0, stream>>>(states, parts, part_stride, row_stride, dim,
                                                                  out, SA_OUT_FINAL);
            break;
        default:
            merge_states_kernel<float><<<grid, 128, 0, stream>>>(states, parts, part_stride, row_stride, dim,
                                                                 out, SA_OUT_FINAL);
            break;
    }
    return cudaGetLastError();
}

}  // namespace sa
