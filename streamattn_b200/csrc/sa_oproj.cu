// Output projection of a decode step: out[b, n] = sum_k x[b, k] * W[n, k] (+ bias[n]) for a
// handful of rows b - the skinny GEMM that follows attention.  The weight matrix is read once
// and dominates the traffic (8 MB for 2048 x 2048 bf16 against 32 KB of activations), so the
// kernel is a weight stream: a CTA owns 8 output features, its 8 warps split K between them
// in interleaved 32-column chunks, every lane fetches 16 contiguous bytes of a weight row per
// chunk and all of a warp's fetches are in flight at once.  The products run on the tensor
// cores (m16n8k16, batch rows on M, fp32 accumulation); because a dot product does not care
// about the order of its terms, the 16 bytes a lane loaded are used as they are, as the B
// fragments of two MMAs over a permuted K order, and the activations are fetched with the same
// permutation - no shuffle, no shared-memory staging of the weights.
//
// Launched with programmatic stream serialization.  The weights do not depend on the kernels
// that precede the projection in a decode step, so (unless the caller says otherwise) a CTA
// requests its weight chunks BEFORE it waits for the preceding kernel: the weight stream
// overlaps the tail of the attention kernel, and only the 32 KB of activations are read after.
#include "sa_common.cuh"

namespace sa {

namespace {

constexpr int kProjWarps = 8;
constexpr int kProjFeatures = 8;     // output features per CTA (the N of m16n8k16)
constexpr int kProjRows = 16;        // batch rows per CTA (the M)
constexpr int kProjChunk = 32;       // K columns per lane load round (4 lanes x 8 elements per row)
constexpr int kProjDepth = 8;        // chunks a warp has in flight

struct ProjParams {
    const void *x;
    const void *w;
    const void *bias;
    void *out;
    int batch, in_features, out_features;
    int64_t x_stride;  // elements between consecutive rows of x
    int prefetch_weights;
};

template <typename T> struct ProjMma;
template <> struct ProjMma<__nv_bfloat16> {
    __device__ __forceinline__ static void run(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1)
    {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
            "{%0, %1, %2, %3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
};
template <> struct ProjMma<__half> {
    __device__ __forceinline__ static void run(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1)
    {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
            "{%0, %1, %2, %3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
};

__device__ __forceinline__ uint4 load_weights_16(const void *ptr)
{
    uint4 v;  // read-only, streamed once: no allocation in L1
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(ptr));
    return v;
}

template <typename T>
__global__ void __launch_bounds__(kProjWarps * 32)
o_proj_kernel(const __grid_constant__ ProjParams p)
{
    __shared__ float partial[kProjWarps][kProjRows][kProjFeatures];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int g = lane >> 2;   // weight row (feature) of the lane's loads; batch row of its results
    const int t4 = lane & 3;   // which 8 of the chunk's 32 columns
    const int n0 = blockIdx.x * kProjFeatures;
    const int b0 = blockIdx.y * kProjRows;
    const int K = p.in_features;
    const int chunks = (K + kProjChunk - 1) / kProjChunk;
    const T *w_row = static_cast<const T *>(p.w) + static_cast<int64_t>(n0 + g) * K;
    const bool row_ok = n0 + g < p.out_features;

    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    uint4 wv[kProjDepth];
    // Column of the lane's 8 elements in the warp's i-th chunk of a round starting at `first`.
    auto column = [&](int first, int i) { return (first + warp + i * kProjWarps) * kProjChunk + 8 * t4; };
    auto fetch_weights = [&](int first) {
#pragma unroll
        for (int i = 0; i < kProjDepth; ++i) {
            const int k = column(first, i);
            wv[i] = (row_ok && k + 8 <= K) ? load_weights_16(w_row + k) : make_uint4(0u, 0u, 0u, 0u);
        }
    };

    if (p.prefetch_weights) fetch_weights(0);
    // Let the next kernel of the stream be scheduled, then wait until everything launched before
    // this kernel - the attention output it consumes - is complete and visible.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (!p.prefetch_weights) fetch_weights(0);

    const T *x_lo = static_cast<const T *>(p.x) + static_cast<int64_t>(b0 + g) * p.x_stride;
    const T *x_hi = x_lo + 8 * p.x_stride;
    const bool lo_ok = b0 + g < p.batch, hi_ok = b0 + g + 8 < p.batch;
    for (int first = 0; first < chunks; first += kProjDepth * kProjWarps) {
        if (first > 0) fetch_weights(first);
        uint4 xa[kProjDepth], xb[kProjDepth];
#pragma unroll
        for (int i = 0; i < kProjDepth; ++i) {
            const int k = column(first, i);
            const bool ok = k + 8 <= K;
            xa[i] = (lo_ok && ok) ? *reinterpret_cast<const uint4 *>(x_lo + k) : make_uint4(0u, 0u, 0u, 0u);
            xb[i] = (hi_ok && ok) ? *reinterpret_cast<const uint4 *>(x_hi + k) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int i = 0; i < kProjDepth; ++i) {
            // The lane's 8 columns are two K-steps: (0,1 | 2,3) and (4,5 | 6,7), for A and B alike.
            ProjMma<T>::run(acc, xa[i].x, xb[i].x, xa[i].y, xb[i].y, wv[i].x, wv[i].y);
            ProjMma<T>::run(acc, xa[i].z, xb[i].z, xa[i].w, xb[i].w, wv[i].z, wv[i].w);
        }
    }

    // acc = out[row g | g + 8][feature 2*t4 | 2*t4 + 1] over this warp's share of K.
    partial[warp][g][2 * t4] = acc[0];
    partial[warp][g][2 * t4 + 1] = acc[1];
    partial[warp][g + 8][2 * t4] = acc[2];
    partial[warp][g + 8][2 * t4 + 1] = acc[3];
    __syncthreads();
    if (tid < kProjRows * kProjFeatures) {
        const int m = tid / kProjFeatures, n = tid - m * kProjFeatures;
        float sum = 0.0f;
#pragma unroll
        for (int w = 0; w < kProjWarps; ++w) sum += partial[w][m][n];
        if (b0 + m < p.batch && n0 + n < p.out_features) {
            if (p.bias != nullptr) sum += Elem<T>::to_float(static_cast<const T *>(p.bias)[n0 + n]);
            static_cast<T *>(p.out)[static_cast<int64_t>(b0 + m) * p.out_features + n0 + n] = Elem<T>::from_float(sum);
        }
    }
}

template <typename T>
cudaError_t launch_typed(const ProjParams &p, cudaStream_t stream)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>((p.out_features + kProjFeatures - 1) / kProjFeatures),
                       static_cast<unsigned>((p.batch + kProjRows - 1) / kProjRows));
    cfg.blockDim = dim3(kProjWarps * 32);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, o_proj_kernel<T>, p);
}

}  // namespace

cudaError_t launch_o_proj(const void *x, const void *w, const void *bias, void *out, int batch, int in_features,
                          int out_features, int64_t x_stride, int dtype, int prefetch_weights, cudaStream_t stream)
{
    ProjParams p;
    p.x = x;
    p.w = w;
    p.bias = bias;
    p.out = out;
    p.batch = batch;
    p.in_features = in_features;
    p.out_features = out_features;
    p.x_stride = x_stride;
    p.prefetch_weights = prefetch_weights;
    return dtype == SA_DTYPE_BF16 ? launch_typed<__nv_bfloat16>(p, stream) : launch_typed<__half>(p, stream);
}

}  // namespace sa
