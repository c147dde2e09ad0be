// Context-parallel state exchange fused with the merge: one kernel per decode step that
// (1) stores this GPU's split state into every peer's gather buffer with plain peer stores
// over NVLink, (2) raises a per-rank flag on every peer, (3) waits - bounded - until the
// flags of all ranks have arrived locally and (4) merges the states exactly.  It replaces
// "all-gather, then merge kernel" (a collective launch plus a kernel) by a single launch.
// No multicast, no cluster launch; every wait has a time limit and reports through the
// status word instead of hanging.
//
// Symmetric buffer of every rank (same layout on all ranks, see exchange_layout()):
//   gather[2][world][rows][D+2] float   double-buffered by step parity
//   flags[2][world]             uint32  flags[parity][r] == step once rank r's state landed
//   arrivals                    uint32  CTA ticket of the local kernel (returns to 0)
//   status                      uint32  SA_DEV_* bits
#include "sa_common.cuh"

namespace sa {

namespace {

constexpr int kExchangeMaxWorld = 16;
constexpr int kExchangeThreads = 128;
constexpr int kExchangeMaxCtas = 64;  // small enough to be co-resident: waiting CTAs cannot starve senders

struct ExchangeLayout {
    size_t gather_floats_per_parity;
    size_t flags_offset;     // bytes
    size_t arrivals_offset;  // bytes
    size_t status_offset;    // bytes
    size_t total_bytes;
};

ExchangeLayout exchange_layout(int world, int64_t rows, int dim)
{
    ExchangeLayout l;
    l.gather_floats_per_parity = static_cast<size_t>(world) * rows * (dim + 2);
    const size_t gather_bytes = (2 * l.gather_floats_per_parity * 4 + 127) / 128 * 128;
    l.flags_offset = gather_bytes;
    l.arrivals_offset = l.flags_offset + 2 * kExchangeMaxWorld * 4;
    l.status_offset = l.arrivals_offset + 64;
    l.total_bytes = l.status_offset + 64;
    return l;
}

struct ExchangeParams {
    const float *local_state;  // [rows][D+2]
    uint64_t bases[kExchangeMaxWorld];  // symmetric buffer of every rank, as seen from this GPU
    int world, rank;
    uint32_t step;             // > 0, increases by one per call on every rank
    int64_t rows;
    int dim;
    size_t gather_floats_per_parity, flags_offset, arrivals_offset, status_offset;
    unsigned long long wait_ns;  // limit of the wait for the ranks' flags
    void *out;
};

__device__ __forceinline__ unsigned long long timer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

template <typename OutT>
__global__ void __launch_bounds__(kExchangeThreads)
exchange_merge_kernel(const __grid_constant__ ExchangeParams p)
{
    __shared__ int s_flag;
    const int tid = threadIdx.x;
    const int width = p.dim + 2;
    const uint32_t parity = p.step & 1u;
    char *my_base = reinterpret_cast<char *>(p.bases[p.rank]);

    // (1) my state -> slot [parity][rank] of every rank's gather buffer (own copy included).
    for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const float *src = p.local_state + row * width;
        for (int dst_rank = 0; dst_rank < p.world; ++dst_rank) {
            float *dst = reinterpret_cast<float *>(p.bases[dst_rank]) + parity * p.gather_floats_per_parity +
                         (static_cast<size_t>(p.rank) * p.rows + row) * width;
            for (int i = tid; i < width; i += kExchangeThreads) dst[i] = src[i];
        }
    }
    // (2) once every CTA's stores are out, the last CTA raises my flag on every rank.
    __threadfence_system();
    __syncthreads();
    if (tid == 0) {
        unsigned *arrivals = reinterpret_cast<unsigned *>(my_base + p.arrivals_offset);
        s_flag = atomicAdd(arrivals, 1u) == gridDim.x - 1;
        if (s_flag) *arrivals = 0u;  // ready for the next step (the next launch is stream-ordered)
    }
    __syncthreads();
    if (s_flag && tid < p.world) {
        __threadfence_system();
        unsigned *flag = reinterpret_cast<unsigned *>(reinterpret_cast<char *>(p.bases[tid]) + p.flags_offset) +
                         parity * kExchangeMaxWorld + p.rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(p.step) : "memory");
    }

    // (3) wait until every rank's state for this step is here; give up after a time limit.
    if (tid < p.world) {
        const unsigned *flag =
            reinterpret_cast<const unsigned *>(my_base + p.flags_offset) + parity * kExchangeMaxWorld + tid;
        const unsigned long long t0 = timer_ns();
        unsigned seen;
        while (true) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
            if (seen == p.step) break;
            if (timer_ns() - t0 > p.wait_ns) {
                atomicOr(reinterpret_cast<int *>(my_base + p.status_offset), SA_DEV_PIPELINE_TIMEOUT);
                break;
            }
            __nanosleep(64);
        }
    }
    __syncthreads();

    // (4) exact merge of the world states of each row.  The states were written by peers, so
    // they are read from L2 (ld.cg); every load of a row is issued before the first one is
    // needed - a chain of dependent L2 round trips per rank would cost more than the exchange.
    __shared__ float s_m[kExchangeMaxWorld], s_l[kExchangeMaxWorld], s_w[kExchangeMaxWorld];
    const float *gather = reinterpret_cast<const float *>(my_base) + parity * p.gather_floats_per_parity;
    const size_t rank_stride = static_cast<size_t>(p.rows) * width;
    for (int64_t row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const float *row0 = gather + row * width;
        if (tid < kExchangeMaxWorld) {
            float m = -INFINITY, l = 0.0f;
            if (tid < p.world) {
                const float2 ml = __ldcg(reinterpret_cast<const float2 *>(row0 + tid * rank_stride + p.dim));
                m = ml.x;
                l = ml.y;
            }
            s_m[tid] = l > 0.0f ? m : -INFINITY;
            s_l[tid] = l;
        }
        __syncthreads();
        float big = -INFINITY;
#pragma unroll
        for (int r = 0; r < kExchangeMaxWorld; ++r) big = fmaxf(big, s_m[r]);
        if (tid < kExchangeMaxWorld) s_w[tid] = exp2_diff(s_m[tid], big);
        __syncthreads();
        float total_l = 0.0f;
#pragma unroll
        for (int r = 0; r < kExchangeMaxWorld; ++r) total_l += s_w[r] * s_l[r];
        const float inv = total_l > 0.0f ? 1.0f / total_l : 0.0f;
        for (int d = tid; d < p.dim; d += kExchangeThreads) {
            float o[kExchangeMaxWorld];
#pragma unroll
            for (int r = 0; r < kExchangeMaxWorld; ++r) o[r] = r < p.world ? __ldcg(row0 + r * rank_stride + d) : 0.0f;
            float acc = 0.0f;
#pragma unroll
            for (int r = 0; r < kExchangeMaxWorld; ++r) acc += s_w[r] * o[r];
            static_cast<OutT *>(p.out)[row * p.dim + d] = Elem<OutT>::from_float(acc * inv);
        }
        __syncthreads();  // s_m / s_l / s_w are reused by the next row
    }
}

}  // namespace

size_t exchange_bytes(int world, int64_t rows, int dim) { return exchange_layout(world, rows, dim).total_bytes; }

size_t exchange_status_offset(int world, int64_t rows, int dim) { return exchange_layout(world, rows, dim).status_offset; }

cudaError_t launch_exchange_merge(const float *local_state, const uint64_t *bases_host, int world, int rank,
                                  uint32_t step, int64_t rows, int dim, void *out, int out_dtype,
                                  unsigned long long wait_ns, cudaStream_t stream)
{
    const ExchangeLayout l = exchange_layout(world, rows, dim);
    ExchangeParams p;
    p.local_state = local_state;
    for (int i = 0; i < kExchangeMaxWorld; ++i) p.bases[i] = i < world ? bases_host[i] : 0;
    p.world = world;
    p.rank = rank;
    p.step = step;
    p.rows = rows;
    p.dim = dim;
    p.gather_floats_per_parity = l.gather_floats_per_parity;
    p.flags_offset = l.flags_offset;
    p.arrivals_offset = l.arrivals_offset;
    p.status_offset = l.status_offset;
    p.wait_ns = wait_ns;
    p.out = out;
    const unsigned grid = static_cast<unsigned>(rows < kExchangeMaxCtas ? rows : kExchangeMaxCtas);
    switch (out_dtype) {
        case SA_DTYPE_BF16: exchange_merge_kernel<__nv_bfloat16><<<grid, kExchangeThreads, 0, stream>>>(p); break;
        case SA_DTYPE_F16: exchange_merge_kernel<__half><<<grid, kExchangeThreads, 0, stream>>>(p); break;
        default: exchange_merge_kernel<float><<<grid, kExchangeThreads, 0, stream>>>(p); break;
    }
    return cudaGetLastError();
}

}  // namespace sa
