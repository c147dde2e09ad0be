// KV-cache update kernel: per batch row, rotate the current K (and optionally the query) with
// the rotary embedding and write the K/V rows into the contiguous or paged cache at the row's
// position.  A few KB per call - latency-bound - so the whole row is one CTA and the launch
// overlaps its neighbours in the stream (programmatic dependent launch, wait before the first
// global access).
//
// Arithmetic: x' = x * cos + rotate_half(x) * sin in the cache dtype, each product and the sum
// rounded to that dtype (fp32 math on the converted operands, round-to-nearest-even back), which
// gives the bits of the same expression evaluated on torch tensors.
#include "sa_append.cuh"

namespace sa {
namespace {

template <typename T> struct Round;
template <> struct Round<float> {
    __device__ static float mul(float a, float b) { return __fmul_rn(a, b); }
    __device__ static float add(float a, float b) { return __fadd_rn(a, b); }
};
template <> struct Round<__nv_bfloat16> {
    __device__ static float mul(float a, float b) { return __bfloat162float(__float2bfloat16_rn(__fmul_rn(a, b))); }
    __device__ static float add(float a, float b) { return __bfloat162float(__float2bfloat16_rn(__fadd_rn(a, b))); }
};
template <> struct Round<__half> {
    __device__ static float mul(float a, float b) { return __half2float(__float2half_rn(__fmul_rn(a, b))); }
    __device__ static float add(float a, float b) { return __half2float(__float2half_rn(__fadd_rn(a, b))); }
};

// One element of the rotated row: x and its partner (index (d + D/2) % D) are read from `row`.
template <typename T>
__device__ __forceinline__ T rotate(const T *row, const T *cos_row, const T *sin_row, int d, int dim)
{
    const int half = dim >> 1;
    const float x = Elem<T>::to_float(row[d]);
    const float partner = Elem<T>::to_float(row[d < half ? d + half : d - half]);
    const float rotated = d < half ? -partner : partner;
    const float a = Round<T>::mul(x, Elem<T>::to_float(cos_row[d]));
    const float b = Round<T>::mul(rotated, Elem<T>::to_float(sin_row[d]));
    return Elem<T>::from_float(Round<T>::add(a, b));
}

constexpr int kAppendThreads = 512;
constexpr int kAppendBatch = 4;  // elements per thread whose loads are all in flight before any store

template <typename T>
__global__ void __launch_bounds__(kAppendThreads) append_kv_kernel(const __grid_constant__ AppendParams p)
{
    // Let the next kernel of the stream (normally the decode) be scheduled early, and wait for
    // everything launched before this kernel - the producer of k_new / v_new / q - to complete.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int b = blockIdx.x;
    const int tid = threadIdx.x;
    const int dim = p.head_dim;
    const int64_t pos = load_index(p.positions, p.pos_i64, p.pos_shared ? 0 : b);
    bool valid = pos >= 0 && pos < p.capacity;
    int bad = valid ? 0 : SA_DEV_BAD_POSITION;
    T *k_dst = nullptr, *v_dst = nullptr;
    int64_t head_stride = 0;
    if (valid) {
        if (p.paged) {
            const int64_t slot = pos % p.page_size;
            const int64_t page = load_index(p.page_table, p.table_i64, static_cast<int64_t>(b) * p.max_pages + pos / p.page_size);
            if (page < 0 || page >= p.num_pages) {
                valid = false;
                bad = SA_DEV_BAD_PAGE;
            } else {
                const int64_t off = page * p.pg_sp + slot * p.pg_st;
                k_dst = static_cast<T *>(p.k_cache) + off;
                v_dst = static_cast<T *>(p.v_cache) + off;
                head_stride = p.pg_sh;
            }
        } else {
            const int64_t off = b * p.kv_sb + pos * p.kv_sn;
            k_dst = static_cast<T *>(p.k_cache) + off;
            v_dst = static_cast<T *>(p.v_cache) + off;
            head_stride = p.kv_sh;
        }
    }
    if (bad != 0 && tid == 0 && p.status != nullptr) atomicOr(p.status, bad);

    const bool rope = p.cos != nullptr;
    const T *cos_row = rope ? static_cast<const T *>(p.cos) + b * p.rope_sb : nullptr;
    const T *sin_row = rope ? static_cast<const T *>(p.sin) + b * p.rope_sb : nullptr;
    const int kv_items = p.kv_heads * dim;
    const int q_items = p.q_in != nullptr ? p.q_heads * dim : 0;
    const int total = 2 * kv_items + q_items;
    // The call is latency-bound (a few KB per row): every thread first requests all it needs for
    // up to kAppendBatch elements, then stores them, so a row costs one round trip per pass.
    for (int base = 0; base < total; base += kAppendThreads * kAppendBatch) {
        T value[kAppendBatch];
        T *dst[kAppendBatch];
#pragma unroll
        for (int e = 0; e < kAppendBatch; ++e) {
            const int i = base + e * kAppendThreads + tid;
            dst[e] = nullptr;
            value[e] = Elem<T>::from_float(0.0f);
            if (i >= total) continue;
            if (i < kv_items) {  // K row of head h
                const int h = i / dim, d = i - h * dim;
                const T *src = static_cast<const T *>(p.k_new) + b * p.new_sb + h * p.new_sh;
                if (valid) {
                    value[e] = rope ? rotate<T>(src, cos_row, sin_row, d, dim) : src[d];
                    dst[e] = k_dst + h * head_stride + d;
                }
            } else if (i < 2 * kv_items) {  // V row of head h
                const int j = i - kv_items;
                const int h = j / dim, d = j - h * dim;
                if (valid) {
                    value[e] = static_cast<const T *>(p.v_new)[b * p.new_sb + h * p.new_sh + d];
                    dst[e] = v_dst + h * head_stride + d;
                }
            } else {  // query row of head h
                const int j = i - 2 * kv_items;
                const int h = j / dim, d = j - h * dim;
                const T *src = static_cast<const T *>(p.q_in) + b * p.qi_sb + h * p.qi_sh;
                value[e] = rope ? rotate<T>(src, cos_row, sin_row, d, dim) : src[d];
                dst[e] = static_cast<T *>(p.q_out) + b * p.qo_sb + h * p.qo_sh + d;
            }
        }
#pragma unroll
        for (int e = 0; e < kAppendBatch; ++e)
            if (dst[e] != nullptr) *dst[e] = value[e];
    }
    if (p.lens_out != nullptr && valid) {
        // lens_out may be the positions array itself: every thread has read its position above.
        __syncthreads();
        if (tid == 0) {
            if (p.pos_i64) static_cast<int64_t *>(p.lens_out)[b] = pos + 1;
            else static_cast<int32_t *>(p.lens_out)[b] = static_cast<int32_t>(pos + 1);
        }
    }
}

template <typename T> cudaError_t launch_typed(const AppendParams &p, cudaStream_t stream)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(p.batch));
    cfg.blockDim = dim3(kAppendThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, append_kv_kernel<T>, p);
}

}  // namespace

cudaError_t launch_append(const AppendParams &p, cudaStream_t stream)
{
    if (p.dtype == SA_DTYPE_BF16) return launch_typed<__nv_bfloat16>(p, stream);
    if (p.dtype == SA_DTYPE_F16) return launch_typed<__half>(p, stream);
    return launch_typed<float>(p, stream);
}

}  // namespace sa
