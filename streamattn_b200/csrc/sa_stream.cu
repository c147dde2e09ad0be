// Streaming decode kernel for sm_100a: K/V tiles move HBM -> shared memory with
// TMA tensor copies (cp.async.bulk.tensor, 128-byte swizzle, mbarrier completion,
// no cluster multicast); every warp owns a private ring of 16 KB K+V tiles so the
// main loop has no cross-warp synchronisation.  QK^T and PV run on the tensor
// cores (m16n8k16, query heads of one KV group on the M rows, fp32 accumulation)
// with a single-pass online softmax in the base-2 domain.
//
// Work is a flat list of tiles over all (row, kv head) pairs, split over the CTAs in
// contiguous slices (balanced by tokens, so ragged rows cost what they hold); a pair
// is usually covered by several CTAs.  Each covering CTA publishes an (m, l, o)
// state; the last one to arrive on the pair (a relaxed atomic ticket, nobody waits
// for another CTA's progress) merges the states exactly and writes the output, so
// one launch does producer and merge.
//
// The same kernel serves contiguous caches, paged caches (page-table lookup per
// fragment) and seed-only decode (a short list of cache blocks).
#include <cstdlib>
#include <mutex>

#include "sa_stream.cuh"

namespace sa {

#ifdef SA_TIMELINE
extern unsigned long long *g_timeline;
#endif

namespace {

#ifndef SA_STREAM_TILE_BYTES
#define SA_STREAM_TILE_BYTES 8192
#endif
constexpr int kTileBytes = SA_STREAM_TILE_BYTES;  // one K or one V tile
constexpr int kStageBytes = 2 * kTileBytes;  // K + V

struct StreamParams {
    const void *q;
    int64_t q_sb, q_sh;
    void *out;
    int out_mode;
    float *partials;
    int *counters;
    int *pool;           // per-pair claim counters of the dynamic schedule (zero between launches)
    int *status;
    int32_t *trace;
    int batch, q_heads, kv_heads, group;
    float scale_log2;
    int frag_tokens;     // rows of one TMA box
    int frags_per_tile;  // TILE_N / frag_tokens
    int frags_per_unit;  // fragments per page / seed block (>= 1)
    int frag_shift;      // log2(frag_tokens)
    int fpt_shift;       // log2(frags_per_tile)
    int fpu_shift;       // log2(frags_per_unit)
    int tok_dim;         // TMA coordinate (1 or 2) that carries the token index
    int uniform_tiles;   // tiles per row when every row has the same length, else -1
    int schedule;        // kScheduleBlocked / kScheduleCyclic / kScheduleClaims
    int kv_split;        // virtual KV heads per physical KV head (kv_heads and group above are virtual)
    unsigned long long wait_ns;  // limit of every bounded wait
    int first_merges;    // the pair's first CTA merges its split states (no ticket): grids of at most one CTA per SM
    SeqDesc seq;
    CpFuse cp;           // context-parallel exchange fused into this launch (cp.world == 0: off)
#ifdef SA_TIMELINE
    unsigned long long *timeline;  // instrumented builds only: 16 words (globaltimer stamps, SM id) per CTA
#endif
};

// Instrumented builds (-DSA_TIMELINE) record %globaltimer per CTA at a few points of the kernel.
#ifdef SA_TIMELINE
#define SA_STAMP_VALUE(i, v) do { if (p.timeline != nullptr && tid == 0) p.timeline[blockIdx.x * 16 + (i)] = (v); } while (0)
#else
#define SA_STAMP_VALUE(i, v) do { } while (0)
#endif
#define SA_STAMP(i) SA_STAMP_VALUE(i, global_timer_ns())

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}

#ifdef SA_TIMELINE
__device__ __forceinline__ unsigned sm_id()
{
    unsigned id;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(id));
    return id;
}
#endif

__device__ __forceinline__ unsigned long long global_timer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait: gives up after `limit_ns` so a lost copy cannot hang the GPU.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned long long limit_ns)
{
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer_ns();
    while (!mbar_try_wait(bar, parity)) {
        if (global_timer_ns() - t0 > limit_ns) return false;
    }
    return true;
}

__device__ __forceinline__ void fence_proxy_async()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ uint64_t make_evict_first_policy()
{
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1,
                                            int c2, int c3, uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%2, %3, %4, %5}], [%6], %7;" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar), "l"(policy)
        : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2,
                                                  uint32_t &r3)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

// Split states travel between the CTAs of one launch as 32-bit words with all bits inverted.
// The workspace is zero between launches, and no float the kernel can produce has the bit
// pattern 0xffffffff (arithmetic results that are NaN carry the canonical pattern 0x7fffffff),
// so a stored word is never zero: "word != 0" means "published", and a reader needs no flag,
// fence or ordering beyond the single-copy atomicity of an aligned 32-bit access.  The merging
// CTA writes zeros back after it has read a state.
__device__ __forceinline__ uint4 state_load4(const float *src)
{
    uint4 v;
    asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(src)
                 : "memory");
    return v;
}

__device__ __forceinline__ uint2 state_load2(const float *src)
{
    uint2 v;
    asm volatile("ld.relaxed.gpu.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(src) : "memory");
    return v;
}

__device__ __forceinline__ void state_store4(float *dst, uint32_t a, uint32_t b, uint32_t c, uint32_t d)
{
    asm volatile("st.relaxed.gpu.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(a), "r"(b), "r"(c), "r"(d)
                 : "memory");
}

__device__ __forceinline__ void state_store2(float *dst, uint32_t a, uint32_t b)
{
    asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(a), "r"(b) : "memory");
}

__device__ __forceinline__ uint32_t inv_bits(float x) { return ~__float_as_uint(x); }
__device__ __forceinline__ float inv_float(uint32_t w) { return __uint_as_float(~w); }

// Context-parallel exchange words: (step << 32 | float bits), written and read as one 64-bit
// scalar (or a vector of two such scalars), which the memory model makes single-copy atomic:
// a reader that sees the step number also has the value.
__device__ __forceinline__ uint64_t cp_word(float value, uint32_t step)
{
    return (static_cast<uint64_t>(step) << 32) | __float_as_uint(value);
}

__device__ __forceinline__ ulonglong2 cp_load2(const uint64_t *src)
{
    ulonglong2 v;
    asm volatile("ld.relaxed.sys.global.v2.b64 {%0, %1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(src) : "memory");
    return v;
}

__device__ __forceinline__ void cp_store2(uint64_t *dst, ulonglong2 v)
{
    asm volatile("st.relaxed.sys.global.v2.b64 [%0], {%1, %2};" ::"l"(dst), "l"(v.x), "l"(v.y) : "memory");
}

template <typename T> struct Mma;
template <> struct Mma<__nv_bfloat16> {
    __device__ __forceinline__ static void run(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
    {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
            "{%0, %1, %2, %3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    __device__ __forceinline__ static uint32_t pack(float lo, float hi)
    {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&v);
    }
};
template <> struct Mma<__half> {
    __device__ __forceinline__ static void run(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
    {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
            "{%0, %1, %2, %3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    __device__ __forceinline__ static uint32_t pack(float lo, float hi)
    {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&v);
    }
};

// Send the tagged words of one pair's state rows - staged in shared memory by the finishing
// CTA - to word offset `start` of every rank's buffer (own rank included).  Consecutive lanes
// move consecutive 16-byte pieces (two words), so one warp store covers 512 contiguous bytes:
// small scattered stores are what NVLink handles worst.  Every word carries its own step tag,
// so the copy needs no ordering beyond the atomicity of an aligned 64-bit access.
template <int NTHREADS>
__device__ __noinline__ void cp_broadcast_pair(const CpFuse &cp, const uint64_t *stage, size_t start, int words,
                                               int tid)
{
    const ulonglong2 *src = reinterpret_cast<const ulonglong2 *>(stage);
    for (int i = tid; i < words / 2; i += NTHREADS) {  // `start` and `words` are even: 16-byte pieces
        const ulonglong2 v = src[i];
        for (int k = 0; k < cp.world; ++k) {
            // Every rank starts with its right-hand neighbour, so the ranks - which finish a step
            // at about the same time - do not all write to the same destination at once.
            const int r = cp.rank + 1 + k < cp.world ? cp.rank + 1 + k : cp.rank + 1 + k - cp.world;
            cp_store2(reinterpret_cast<uint64_t *>(cp.bases[r]) + start + 2 * i, v);
        }
    }
}

// Context-parallel finish of one (row, kv head) pair, run by the CTA that completed the pair on
// this rank after it sent the pair's state rows to every rank: wait (bounded) for the same rows
// from all ranks - each word carries the step number, so the data is its own flag - then merge
// them exactly and write the final output rows.  A work item is 4 columns of one head row;
// NTHREADS / items threads share an item and each polls every (NTHREADS / items)-th rank, four
// ranks' (o[4], m, l) words at a time, so the wait costs one round of loads after the data
// landed; the threads of an item meet through shared memory (`sm`, 6 floats per thread).  Kept
// out of line so its registers do not weigh on the streaming loop.
template <typename T, int D, int NTHREADS>
__device__ __noinline__ void cp_finish_pair(const CpFuse &cp, int *status, unsigned long long wait_ns,
                                            size_t total_rows, int64_t out_row0, int items, float *sm, int tid)
{
    constexpr int STATE_STRIDE = D + 2;
    constexpr int RB = 4;  // ranks polled together by one thread
    const uint64_t *gather = reinterpret_cast<const uint64_t *>(cp.bases[cp.rank]) + (cp.step & 1u) * cp.gather_words_per_parity;
    const size_t rank_stride = total_rows * STATE_STRIDE;
    const int parts = items <= NTHREADS ? NTHREADS / items : 1;
    const unsigned long long t0 = global_timer_ns();
    unsigned polls = 0;
    for (int first = 0; first < items; first += NTHREADS) {  // a single pass unless items > NTHREADS
        const int part = parts > 1 ? tid / items : 0;
        const int item = parts > 1 ? tid - part * items : first + tid;
        const bool active = part < parts && item < items;
        const int row = item / (D / 4);
        const int d4 = (item - row * (D / 4)) * 4;
        float big = -INFINITY, total_l = 0.0f;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (active) {
            const uint64_t *row0 = gather + (out_row0 + row) * STATE_STRIDE;
            for (int r0 = part; r0 < cp.world; r0 += parts * RB) {
                ulonglong2 w[RB][3];  // (o0, o1), (o2, o3), (m, l)
                bool waiting = true;
                while (waiting) {
                    // Unconditional loads (ranks past the last one are clamped to it and given weight
                    // zero below): one straight line of independent requests.
#pragma unroll
                    for (int u = 0; u < RB; ++u) {
                        const int r = r0 + u * parts < cp.world ? r0 + u * parts : cp.world - 1;
                        const uint64_t *st = row0 + r * rank_stride;
                        w[u][0] = cp_load2(st + d4);
                        w[u][1] = cp_load2(st + d4 + 2);
                        w[u][2] = cp_load2(st + D);
                    }
                    uint32_t landed = 1u;
#pragma unroll
                    for (int u = 0; u < RB; ++u)
#pragma unroll
                        for (int j = 0; j < 3; ++j)
                            landed &= static_cast<uint32_t>(static_cast<uint32_t>(w[u][j].x >> 32) == cp.step) &
                                      static_cast<uint32_t>(static_cast<uint32_t>(w[u][j].y >> 32) == cp.step);
                    waiting = landed == 0u;
                    // The clock is slow to read: look at it every 16th round of loads.
                    if (waiting && (++polls & 15u) == 0u && global_timer_ns() - t0 > wait_ns) {
                        atomicOr(status, SA_DEV_PIPELINE_TIMEOUT);
                        break;
                    }
                }
                auto val = [](uint64_t word) { return __uint_as_float(static_cast<uint32_t>(word)); };
                float mr[RB];
                float nb = big;
#pragma unroll
                for (int u = 0; u < RB; ++u) {
                    mr[u] = r0 + u * parts < cp.world ? val(w[u][2].x) : -INFINITY;
                    nb = fmaxf(nb, mr[u]);
                }
                const float keep = exp2_diff(big, nb);
                acc.x *= keep; acc.y *= keep; acc.z *= keep; acc.w *= keep;
                total_l *= keep;
                big = nb;
#pragma unroll
                for (int u = 0; u < RB; ++u) {
                    const float wgt = exp2_diff(mr[u], big);  // 0 for the clamped duplicates
                    acc.x += wgt * val(w[u][0].x);
                    acc.y += wgt * val(w[u][0].y);
                    acc.z += wgt * val(w[u][1].x);
                    acc.w += wgt * val(w[u][1].y);
                    total_l += wgt * val(w[u][2].y);
                }
            }
        }
        if (parts > 1) {
            if (active && part > 0) {
                float *mine = sm + ((part - 1) * items + item) * 6;
                *reinterpret_cast<float2 *>(mine) = make_float2(acc.x, acc.y);
                *reinterpret_cast<float2 *>(mine + 2) = make_float2(acc.z, acc.w);
                *reinterpret_cast<float2 *>(mine + 4) = make_float2(big, total_l);
            }
            __syncthreads();
            if (active && part == 0) {
                for (int q = 1; q < parts; ++q) {
                    const float *other = sm + ((q - 1) * items + item) * 6;
                    const float ob = other[4];
                    const float nb = fmaxf(big, ob);
                    const float keep = exp2_diff(big, nb), wgt = exp2_diff(ob, nb);
                    acc.x = acc.x * keep + wgt * other[0];
                    acc.y = acc.y * keep + wgt * other[1];
                    acc.z = acc.z * keep + wgt * other[2];
                    acc.w = acc.w * keep + wgt * other[3];
                    total_l = total_l * keep + wgt * other[5];
                    big = nb;
                }
            }
        }
        if (active && part == 0) {
            const float inv = total_l > 0.0f ? 1.0f / total_l : 0.0f;
            T *dst = static_cast<T *>(cp.final_out) + (out_row0 + row) * D + d4;
            *reinterpret_cast<uint2 *>(dst) =
                make_uint2(Mma<T>::pack(acc.x * inv, acc.y * inv), Mma<T>::pack(acc.z * inv, acc.w * inv));
        }
    }
}

// Row length read as a hint before the launch's dependency wait: a gpu-scope load, served by
// the L2 (an L1 line allocated now could be stale after the wait).  Same clamping as row_vlen().
__device__ __forceinline__ int64_t row_vlen_hint(const SeqDesc &s, int b)
{
    if (s.mode == kBlocks) return s.blocks_vlen;
    const int64_t cap = s.mode == kPaged ? static_cast<int64_t>(s.max_pages) * s.page_size : s.kv_len;
    int64_t n = cap;
    if (s.seq_lens != nullptr) {
        if (s.lens_i64) {
            asm volatile("ld.relaxed.gpu.global.s64 %0, [%1];"
                         : "=l"(n)
                         : "l"(static_cast<const int64_t *>(s.seq_lens) + b)
                         : "memory");
        } else {
            int v;
            asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];"
                         : "=r"(v)
                         : "l"(static_cast<const int32_t *>(s.seq_lens) + b)
                         : "memory");
            n = v;
        }
    }
    if (n < 0) n = 0;
    return n < cap ? n : cap;
}

// Exact merge of the `nseg` split states of one (row, kv head) pair by all threads of the
// last CTA to arrive on it (items <= NTHREADS).  A work item is 4 columns of one head row;
// NTHREADS / items threads share an item and each takes every (NTHREADS / items)-th state,
// requesting its o rows together with their (m, l) in one batch, so the whole merge costs one
// round trip to L2 (loads with gpu-scope semantics are costly to issue: BATCH, the states one
// thread requests per pass, is chosen to fit the pair).  The CTA's own state (index `self`) does
// not make that trip: it is taken from shared memory (`own`: o[4], m, l per item) and enters the
// sum at its index position, so the order of the additions - and with it every bit of the result
// - does not depend on which CTA happens to arrive last.
// The other states are published with inverted bits (see state_load4): a word that still reads
// zero has not landed yet and the batch is requested again, for at most `wait_ns`.  The merging
// CTA is the pair's first one when the whole grid can be resident at once: it may then be looking
// for microseconds, until the slowest CTA of the pair has stored its state.  In a larger grid it
// is the last CTA to take the pair's ticket: every other CTA has then left its streaming loop,
// and the wait is for a few hundred nanoseconds of work of CTAs that are already running, never
// for a CTA that still has to be scheduled.  The per-thread results meet in shared
// memory; on return sm[item * 6 ..] = (o[4] unnormalised, m, l) and all nseg states are zero
// again.  Out of line so that the rows in flight do not weigh on the streaming loop's registers.
template <int D, int NTHREADS, int BATCH>
__device__ __noinline__ void merge_pair_states(float *first_slot, int64_t slot_stride, int nseg, int self,
                                              const float *own, int items, float *sm, int tid,
                                              unsigned long long wait_ns, int *status)
{
    constexpr int PART_STRIDE = D + 4;
    // Small non-negative integers: floor(a / b) = floor((a + 0.5) * (1 / b)) without the long
    // integer-division sequence (the half keeps the product clear of the next integer).
    const float inv_items = __frcp_rn(static_cast<float>(items));
    const int parts = static_cast<int>((static_cast<float>(NTHREADS) + 0.5f) * inv_items);
    const int part = static_cast<int>((static_cast<float>(tid) + 0.5f) * inv_items);
    const int item = tid - part * items;
    const bool active = part < parts;
    const int row = item / (D / 4);
    const int d4 = (item - row * (D / 4)) * 4;
    float *src = first_slot + row * PART_STRIDE;
    const int other = self == 0 ? 1 : 0;  // some state that is not the CTA's own (nseg >= 2)
    float big = -INFINITY, total_l = 0.0f;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    unsigned long long t0 = 0;
    unsigned polls = 0;
    for (int i0 = part; active && i0 < nseg; i0 += parts * BATCH) {  // one pass up to BATCH * parts states
        // Every load of the batch is issued before the first result is looked at: the loads are
        // unconditional (indices past the last state and the CTA's own index are redirected to
        // another state and given weight zero below), so they form one straight line of
        // independent requests - a branch per state would make each load wait for the one before.
        uint4 o[BATCH];
        uint2 ml[BATCH];
        bool waiting = true;
        while (waiting) {
#pragma unroll
            for (int u = 0; u < BATCH; ++u) {
                int i = i0 + u * parts;
                i = (i >= nseg || i == self) ? other : i;
                o[u] = state_load4(src + i * slot_stride + d4);
                ml[u] = state_load2(src + i * slot_stride + D);
            }
            uint32_t landed = 1u;
#pragma unroll
            for (int u = 0; u < BATCH; ++u)
                landed &= static_cast<uint32_t>(o[u].x != 0u) & static_cast<uint32_t>(o[u].y != 0u) &
                          static_cast<uint32_t>(o[u].z != 0u) & static_cast<uint32_t>(o[u].w != 0u) &
                          static_cast<uint32_t>(ml[u].x != 0u) & static_cast<uint32_t>(ml[u].y != 0u);
            waiting = landed == 0u;
            if (waiting && (++polls & 15) == 0) {  // the clock is slow to read: look at it now and then
                const unsigned long long now = global_timer_ns();
                if (t0 == 0) t0 = now;
                if (now - t0 > wait_ns) {
                    atomicOr(status, SA_DEV_PIPELINE_TIMEOUT);
                    break;
                }
            }
        }
        {   // the CTA's own state takes its place in the sequence (stored like the others)
            const float *mine = own + item * 6;
#pragma unroll
            for (int u = 0; u < BATCH; ++u) {
                if (i0 + u * parts == self) {
                    o[u] = make_uint4(inv_bits(mine[0]), inv_bits(mine[1]), inv_bits(mine[2]), inv_bits(mine[3]));
                    ml[u] = make_uint2(inv_bits(mine[4]), inv_bits(mine[5]));
                }
            }
        }
        float mi[BATCH];
        float nb = big;
#pragma unroll
        for (int u = 0; u < BATCH; ++u) {
            mi[u] = i0 + u * parts < nseg ? inv_float(ml[u].x) : -INFINITY;
            nb = fmaxf(nb, mi[u]);
        }
        const float keep = exp2_diff(big, nb);
        acc.x *= keep; acc.y *= keep; acc.z *= keep; acc.w *= keep;
        total_l *= keep;
        big = nb;
#pragma unroll
        for (int u = 0; u < BATCH; ++u) {
            const float wgt = exp2_diff(mi[u], big);  // 0 for the redirected loads
            acc.x += wgt * inv_float(o[u].x);
            acc.y += wgt * inv_float(o[u].y);
            acc.z += wgt * inv_float(o[u].z);
            acc.w += wgt * inv_float(o[u].w);
            total_l += wgt * inv_float(ml[u].y);
        }
    }
    if (active) {
        float *mine = sm + (part * items + item) * 6;
        *reinterpret_cast<float2 *>(mine) = make_float2(acc.x, acc.y);
        *reinterpret_cast<float2 *>(mine + 2) = make_float2(acc.z, acc.w);
        *reinterpret_cast<float2 *>(mine + 4) = make_float2(big, total_l);
    }
    __syncthreads();  // every thread has read its states: they can be cleared
    if (active) {
        for (int i = part; i < nseg; i += parts) {
            // Plain stores: the next reader is a later launch, which the launch boundary orders.
            *reinterpret_cast<float4 *>(src + i * slot_stride + d4) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (d4 == 0) *reinterpret_cast<float2 *>(src + i * slot_stride + D) = make_float2(0.0f, 0.0f);
        }
    }
    if (part == 0 && parts > 1) {
        for (int q = 1; q < parts; ++q) {
            const float *other_part = sm + (q * items + item) * 6;
            const float ob = other_part[4];
            const float nb = fmaxf(big, ob);
            const float keep = exp2_diff(big, nb), wgt = exp2_diff(ob, nb);
            acc.x = acc.x * keep + wgt * other_part[0];
            acc.y = acc.y * keep + wgt * other_part[1];
            acc.z = acc.z * keep + wgt * other_part[2];
            acc.w = acc.w * keep + wgt * other_part[3];
            total_l = total_l * keep + wgt * other_part[5];
            big = nb;
        }
        float *mine = sm + item * 6;
        *reinterpret_cast<float2 *>(mine) = make_float2(acc.x, acc.y);
        *reinterpret_cast<float2 *>(mine + 2) = make_float2(acc.z, acc.w);
        *reinterpret_cast<float2 *>(mine + 4) = make_float2(big, total_l);
    }
    __syncthreads();
}

// One fragment (TMA box) of a tile as seen by the issuing lane.
struct Frag {
    int x;              // global tile index, -1: no tile (warp-uniform)
    int state;          // 0: nothing to load, 1: load, 2: page id out of range (skip + report)
    int tok;            // token coordinate of the box
    int outer;          // outermost coordinate: batch row or physical page
    int kvh;            // kv head coordinate
    int64_t trace_idx;  // slot of the page-walk trace to record, or -1
};

template <typename T, int D, int WARPS, int STAGES, bool ROWS16>
__global__ void __launch_bounds__(WARPS * 32, 1)
stream_decode_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                     const __grid_constant__ StreamParams p)
{
    constexpr int TILE_N = kTileBytes / (D * 2);  // tokens per tile
    constexpr int HALVES = D / 64;                // 128-byte column groups per row
    constexpr int HALF_BYTES = TILE_N * 128;
    constexpr int NT_S = TILE_N / 8;   // score n-tiles (8 tokens each)
    constexpr int KS_QK = D / 16;      // k-steps of q.k
    constexpr int NT_O = D / 8;        // output n-tiles (8 columns each)
    constexpr int KS_PV = TILE_N / 16; // k-steps of p.v
    constexpr int ROWS = ROWS16 ? 16 : 8;
    constexpr int STATE_STRIDE = D + 2;  // (o[D], m, l): shared-memory states and the SA_OUT_STATE output
    constexpr int PART_STRIDE = D + 4;   // split states in the workspace: padded to 16-byte rows
    constexpr int STATE_FLOATS = ROWS * STATE_STRIDE;  // one warp's (o, m, l) rows
    constexpr int NTHREADS = WARPS * 32;
    constexpr int BAR_BYTES = (WARPS * STAGES * 8 + 15) / 16 * 16;
    constexpr int MERGE_ROWS = NTHREADS / (D / 4);  // head rows one merge pass covers
    constexpr int OWN = (ROWS * (D / 4) + NTHREADS - 1) / NTHREADS;  // work items per thread

    extern __shared__ uint8_t smem_raw[];
    uint8_t *ring = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(ring + WARPS * STAGES * kStageBytes);
    float *states = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(bars) + BAR_BYTES);
    uint64_t *cp_stage = reinterpret_cast<uint64_t *>(states + WARPS * STATE_FLOATS);  // context-parallel: rows to send
    float *scratch = reinterpret_cast<float *>(cp_stage + STATE_FLOATS);  // merges: 6 floats per thread
    int *prefix = reinterpret_cast<int *>(scratch + NTHREADS * 6);         // ragged rows: tiles before row b
    int *vlens = prefix + p.batch + 1;                                     // ragged rows: length of row b (-1: not selected)
    __shared__ int s_last;

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int g = lane >> 2;
    const int t4 = lane & 3;
    const int C = gridDim.x;
    const int c = blockIdx.x;
    const int group = p.group;
    const int Hkv = p.kv_heads;
    const bool ragged = p.uniform_tiles < 0;

    const uint32_t ring_u32 = smem_u32(ring) + warp * STAGES * kStageBytes;
    const uint32_t bar_u32 = smem_u32(bars) + warp * STAGES * 8;
    uint8_t *warp_ring = ring + warp * STAGES * kStageBytes;

    SA_STAMP(0);
    SA_STAMP_VALUE(2, sm_id());  // which SM ran this CTA
    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tm_k)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tm_v)) : "memory");
    }
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; ++s) mbar_init(bar_u32 + s * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Programmatic dependent launch: let the next kernel of the stream be scheduled as this
    // grid's CTAs retire, and hold this grid - before its first global-memory access - until
    // everything launched earlier in the stream has completed and is visible.  Stream order is
    // unchanged; only launch latency and whatever runs before the wait overlap the previous
    // tail.  What runs before it here is the partition of the tile list, about 1.5 us of
    // dependent integer arithmetic:
    //  - rows of one length need nothing from memory for it, so their wait comes after the
    //    partition (below, in front of the first table look-ups and copies);
    //  - ragged rows take their lengths as a HINT before the wait (gpu-scope loads that bypass L1:
    //    an earlier kernel may still be writing them), cut the tile list with it, wait, read the
    //    lengths again and keep the partition if no row's tile count changed - which is the
    //    case in all but one of TILE_N decode steps per row, since a row grows by one token per
    //    step; otherwise the partition is simply made again.  Nothing is copied, written or
    //    dereferenced on the strength of a hint.  Row subsets read their row list too and do
    //    not speculate.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint64_t policy = make_evict_first_policy();
    // Tile indices fit in 32 bits (the host checks the total); only products with the CTA
    // count need 64 bits.  32-bit divisions keep the per-tile bookkeeping cheap.
    auto tiles_before = [&](int b) -> int { return ragged ? prefix[b] : b * p.uniform_tiles; };
    // Row lengths were read once for the prefix sum; uniform rows need no load at all.
    auto vlen_of = [&](int b) -> int64_t { return ragged ? static_cast<int64_t>(vlens[b]) : row_vlen(p.seq, b); };
    int total_tiles = 0;  // set by the partition pass below, like q_t and r_t
    // CTA c owns tiles [c*q + min(c, r), (c+1)*q + min(c+1, r)) with q = T / C, r = T % C:
    // the first r CTAs take one extra tile.  owner(x) is the CTA that owns tile x.
    unsigned q_t = 0, r_t = 0;
    auto range_lo = [&](unsigned cc) -> int { return static_cast<int>(cc * q_t + (cc < r_t ? cc : r_t)); };
    auto owner = [&](int x) -> int {
        const unsigned ux = static_cast<unsigned>(x);
        const unsigned wide = r_t * (q_t + 1);  // tiles held by the CTAs that take q+1
        return static_cast<int>(ux < wide ? ux / (q_t + 1) : r_t + (ux - wide) / q_t);
    };
    // Global tile x -> (row, kv head, first global tile of the pair, tiles per row).
    auto locate = [&](int x, int &b, int &kvh, int &row_tiles, int &pair_start) {
        if (ragged) {
            int lo_b = 0, hi_b = p.batch;  // largest b with Hkv*prefix[b] <= x
            while (hi_b - lo_b > 1) {
                const int mid = (lo_b + hi_b) >> 1;
                if (Hkv * prefix[mid] <= x) lo_b = mid; else hi_b = mid;
            }
            b = lo_b;
        } else {
            b = static_cast<int>(static_cast<unsigned>(x) / static_cast<unsigned>(Hkv * p.uniform_tiles));
        }
        row_tiles = tiles_before(b + 1) - tiles_before(b);
        const int row_start = Hkv * tiles_before(b);
        kvh = static_cast<int>(static_cast<unsigned>(x - row_start) / static_cast<unsigned>(row_tiles));
        pair_start = row_start + kvh * row_tiles;
    };


    // Partition of the tile list over the CTAs.  A segment boundary inside a CTA stalls its four
    // warps for the flush/combine, so when there are at least four CTAs per (row, kv head) pair
    // the slice boundaries are snapped to pair boundaries ("aligned"): pair p gets the CTAs
    // [cs(p), cs(p+1)) with cs(p) = round(C * tiles_before_pair(p) / T), and splits its tiles
    // evenly among them; every CTA then has exactly one segment.  Otherwise the flat rule is used.
    const int num_pairs = p.batch * Hkv;
    int lo = 0, hi = 0;
    int al_first = 0, al_nseg = 0;
    bool aligned = false;
    int al_pair = -1, al_start = 0, al_end = 0;  // aligned mode: this CTA's pair and its tile range
    bool dyn = false;                            // the pair's warps share its tiles (cyclic or claims)
    bool dyn_claims = false;                     // ... through the claim counter
    int dyn_chunk = 1;                           // tiles per claim
    int dyn_nw = 0, dyn_gw = 0;                  // warps working on the pair, this warp's index among them
    auto cut_tile_list = [&]() {
        total_tiles = Hkv * tiles_before(p.batch);
        q_t = static_cast<unsigned>(total_tiles) / static_cast<unsigned>(C);
        r_t = static_cast<unsigned>(total_tiles) - q_t * C;
        lo = hi = 0;
        al_first = al_nseg = 0;
        al_pair = -1;
        al_start = al_end = 0;
        dyn = dyn_claims = false;
        dyn_chunk = 1;
        dyn_nw = dyn_gw = 0;
        aligned = total_tiles > 0 && 4 * num_pairs <= C &&
                  static_cast<uint64_t>(C) * static_cast<uint64_t>(total_tiles) < (1ull << 32);
        if (aligned) {
            // One pair per lane: lane pp computes cs(pp); cs(pp+1) comes from the neighbour lane.
            const unsigned half = static_cast<unsigned>(total_tiles) / 2;
            bool ok = true;
            int s0 = 0, s1 = 0;
            unsigned t0 = 0, t1 = 0;
            for (int base = 0; base < num_pairs && al_pair < 0; base += 31) {
                const int pp = base + lane;  // lanes 0..30 own a pair, lane 31 only supplies cs(pp) to lane 30
                unsigned before = static_cast<unsigned>(total_tiles);
                if (pp < num_pairs) {
                    const int bb = pp / Hkv;
                    const int tb = tiles_before(bb);
                    before = static_cast<unsigned>(Hkv * tb + (pp - bb * Hkv) * (tiles_before(bb + 1) - tb));
                }
                const int start = static_cast<int>((static_cast<unsigned>(C) * before + half) /
                                                   static_cast<unsigned>(total_tiles));
                const int next_start = __shfl_down_sync(0xffffffffu, start, 1);
                const unsigned next_before = __shfl_down_sync(0xffffffffu, before, 1);
                const bool owns = lane < 31 && pp < num_pairs;
                if (owns && next_before > before && next_start <= start) ok = false;
                const bool hit = owns && c >= start && c < next_start;
                const unsigned m = __ballot_sync(0xffffffffu, hit);
                if (m != 0u) {
                    const int src = __ffs(m) - 1;
                    al_pair = base + src;
                    s0 = __shfl_sync(0xffffffffu, start, src);
                    s1 = __shfl_sync(0xffffffffu, next_start, src);
                    t0 = __shfl_sync(0xffffffffu, before, src);
                    t1 = __shfl_sync(0xffffffffu, next_before, src);
                }
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            // The "every pair with tiles gets a CTA" test must cover all pairs even after the hit.
            if (ok && num_pairs > 31) {
                for (int base = 0; base < num_pairs; base += 32) {
                    const int pp = base + lane;
                    if (pp < num_pairs) {
                        auto before_of = [&](int q) -> unsigned {
                            if (q >= num_pairs) return static_cast<unsigned>(total_tiles);
                            const int bb = q / Hkv;
                            const int tb = tiles_before(bb);
                            return static_cast<unsigned>(Hkv * tb + (q - bb * Hkv) * (tiles_before(bb + 1) - tb));
                        };
                        const unsigned b0 = before_of(pp), b1 = before_of(pp + 1);
                        const unsigned c0 = (static_cast<unsigned>(C) * b0 + half) / static_cast<unsigned>(total_tiles);
                        const unsigned c1 = (static_cast<unsigned>(C) * b1 + half) / static_cast<unsigned>(total_tiles);
                        if (b1 > b0 && c1 <= c0) ok = false;
                    }
                }
                ok = __all_sync(0xffffffffu, ok);
            }
            aligned = ok && al_pair >= 0;
            if (aligned) {
                const unsigned tiles_p = t1 - t0;
                const unsigned n_p = static_cast<unsigned>(s1 - s0);
                const unsigned n_eff = n_p < tiles_p ? n_p : tiles_p;  // never more CTAs than tiles
                const unsigned k = static_cast<unsigned>(c - s0);
                al_first = s0;
                al_nseg = static_cast<int>(n_eff);
                al_start = static_cast<int>(t0);
                al_end = static_cast<int>(t1);
                const bool claims = p.schedule == kScheduleClaims;
                if ((claims || p.schedule == kScheduleCyclic) && n_eff == n_p && tiles_p >= n_p * WARPS * (STAGES + 1)) {
                    // Shared schedules: the pair's warps take tiles round-robin by position - all of
                    // them (cyclic), or only their first STAGES + 1, after which every tile is claimed
                    // from the pair's counter, so a CTA that the memory system serves slowly simply
                    // ends up with fewer tiles.
                    dyn = true;
                    dyn_claims = claims;
                    // One counter serves about 30 claims per microsecond: with many CTAs on a pair a
                    // claim covers several consecutive tiles.
                    dyn_chunk = (static_cast<int>(n_p) + 15) / 16;
                    dyn_nw = static_cast<int>(n_p) * WARPS;
                    dyn_gw = static_cast<int>(k) * WARPS + warp;
                    lo = al_start;
                    hi = al_end;
                } else if (k < n_eff) {
                    if (tiles_p < (1u << 20)) {  // products fit 32 bits (n_eff <= C <= 4096)
                        lo = static_cast<int>(t0 + tiles_p * k / n_eff);
                        hi = static_cast<int>(t0 + tiles_p * (k + 1) / n_eff);
                    } else {
                        lo = static_cast<int>(t0 + static_cast<unsigned>(static_cast<uint64_t>(tiles_p) * k / n_eff));
                        hi = static_cast<int>(t0 + static_cast<unsigned>(static_cast<uint64_t>(tiles_p) * (k + 1) / n_eff));
                    }
                }
            }
        }
        if (!aligned) {
            lo = range_lo(c);
            hi = range_lo(c + 1);
        }
    };
    const bool speculate = ragged && p.seq.num_rows < 0;
    bool waited = false;
    if (!ragged) {  // rows of one length: one pass, nothing to read
        __syncwarp();  // this warp's barriers are initialised; nothing else is shared yet
        fence_proxy_async();
        cut_tile_list();
    }
#pragma unroll 1
    for (int pass = 0; ragged && pass < 2; ++pass) {
        const bool hint = speculate && pass == 0;
        if (!hint && !waited) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            waited = true;
        }
        {
            // Tiles per row depend on lengths that live on the device: prefix-sum them once per CTA.
            const bool subset = p.seq.num_rows >= 0;
            if (subset) {
                // Row subset: rows that are not listed keep length -1 (no tiles, output untouched).
                for (int b = tid; b < p.batch; b += NTHREADS) vlens[b] = -1;
                __syncthreads();
                for (int i = tid; i < p.seq.num_rows; i += NTHREADS) {
                    const int64_t r = load_index(p.seq.rows, p.seq.rows_i64, i);
                    if (r >= 0 && r < p.batch) vlens[r] = static_cast<int>(row_vlen(p.seq, static_cast<int>(r)));
                }
                __syncthreads();
            }
            if (warp == 0) {
                int running = 0;
                for (int base = 0; base < p.batch; base += 32) {
                    const int b = base + lane;
                    int x = 0;
                    if (b < p.batch) {
                        int n;
                        if (subset) {
                            n = vlens[b];
                        } else {
                            // < 2^31: the host bounds the capacity
                            n = static_cast<int>(hint ? row_vlen_hint(p.seq, b) : row_vlen(p.seq, b));
                            vlens[b] = n;
                        }
                        x = n > 0 ? (n + TILE_N - 1) / TILE_N : 0;
                    }
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        const int y = __shfl_up_sync(0xffffffffu, x, o);
                        if (lane >= o) x += y;
                    }
                    if (b < p.batch) prefix[b + 1] = running + x;
                    running += __shfl_sync(0xffffffffu, x, 31);
                }
                if (lane == 0) prefix[0] = 0;
            }
            __syncthreads();
        }
        if (pass == 0) fence_proxy_async();

        cut_tile_list();
        if (!hint) break;
        // The partition above rests on a hint: wait, read the lengths for good, compare.
        asm volatile("griddepcontrol.wait;" ::: "memory");
        waited = true;
        bool same = true;
        int fresh = 0;
        if (tid < p.batch) {  // one row per thread; larger batches do not use the hint (below)
            fresh = static_cast<int>(row_vlen(p.seq, tid));
            const int tiles = fresh > 0 ? (fresh + TILE_N - 1) / TILE_N : 0;
            same = tiles == prefix[tid + 1] - prefix[tid];
        }
        if (p.batch > NTHREADS) same = false;
        same = __syncthreads_and(same);  // also: every warp is done reading the hinted lengths
        if (same) {
            if (tid < p.batch) vlens[tid] = fresh;  // the lengths proper (masks of the rows' last tiles)
            __syncthreads();
            break;
        }
    }
    // Static schedule: this warp's tiles are lo + warp + i*WARPS for i in [0, n_w), across all
    // segments of the CTA, so its copy pipeline keeps running through segment boundaries.
    // Dynamic schedule: tiles al_start + i*dyn_nw + dyn_gw for i <= STAGES, then one claim per tile.
    const int n_w = hi - lo > warp ? (hi - lo - warp + WARPS - 1) / WARPS : 0;
    int seq_i = 0;            // tiles of this warp's sequence produced so far
    int claim = 0;            // lane 0: the claim in flight (dynamic schedule)
    bool claiming = dyn_claims;  // false once a claim came back past the end of the pair
    int chunk_x = 0, chunk_left = 0;  // rest of the claimed run of tiles
    const int dyn_base = al_start + (STAGES + 1) * dyn_nw;
    auto start_claim = [&]() {
        if (lane == 0) claim = atomicAdd(p.pool + al_pair, 1);
    };
    // Next tile of this warp's sequence (-1: none).  A claim is consumed one call after it was
    // issued, so the counter's round trip overlaps a whole tile of work.
    auto next_tile = [&]() -> int {
        int x = -1;
        if (!dyn) {
            if (seq_i < n_w) x = lo + warp + seq_i * WARPS;
        } else if (seq_i <= STAGES || !dyn_claims) {
            x = al_start + seq_i * dyn_nw + dyn_gw;
            if (x >= al_end) x = -1;
            if (dyn_claims && seq_i == STAGES) start_claim();
        } else if (chunk_left > 0) {
            --chunk_left;
            x = chunk_x++;
            if (x >= al_end) {
                x = -1;
                chunk_left = 0;
            }
        } else if (claiming) {
            x = dyn_base + __shfl_sync(0xffffffffu, claim, 0) * dyn_chunk;
            if (x < al_end) {
                chunk_x = x + 1;
                chunk_left = dyn_chunk - 1;
                start_claim();
            } else {
                x = -1;
                claiming = false;
            }
        }
        ++seq_i;
        return x;
    };

    // What this lane has to copy for tile x (page-table lookups happen here, one
    // tile before the copies are issued, so their latency stays off the critical path).  The
    // producer keeps its own (row, kv head) cursor: tiles are visited in ascending order, so
    // the cursor only moves when a tile crosses into the next pair.
    int pc_b = -1, pc_kvh = 0, pc_start = 0, pc_end = 0;
    int64_t pc_vlen = 0;
    if (aligned && hi > lo) {  // all of this CTA's tiles belong to one pair: no search needed
        pc_b = al_pair / Hkv;
        pc_kvh = al_pair - pc_b * Hkv;
        pc_start = al_start;
        pc_end = al_end;
        pc_vlen = vlen_of(pc_b);
    }
    auto lookup = [&](int x) -> Frag {
        Frag f;
        f.x = x; f.state = 0; f.tok = 0; f.outer = 0; f.kvh = 0; f.trace_idx = -1;
        if (x < 0) return f;
        if (x >= pc_end) {
            int b, row_tiles;
            locate(x, b, pc_kvh, row_tiles, pc_start);
            pc_end = pc_start + row_tiles;
            if (b != pc_b) pc_vlen = vlen_of(b);
            pc_b = b;
        }
        f.kvh = p.kv_split > 1 ? pc_kvh / p.kv_split : pc_kvh;  // the cache's own head index
        if (lane >= p.frags_per_tile) return f;
        const unsigned vfrag = (static_cast<unsigned>(x - pc_start) << p.fpt_shift) + lane;
        const int64_t vtok0 = static_cast<int64_t>(vfrag) << p.frag_shift;
        if (vtok0 >= pc_vlen) return f;
        if (p.seq.mode == kContig) {
            f.tok = static_cast<int>(vtok0);
            f.outer = pc_b;
            f.state = 1;
        } else if (p.seq.mode == kPaged) {
            const unsigned lp = vfrag >> p.fpu_shift;
            const int sub = static_cast<int>(vfrag - (lp << p.fpu_shift));
            const int64_t slot = static_cast<int64_t>(pc_b) * p.seq.max_pages + lp;
            const int64_t page = load_index(p.seq.page_table, p.seq.table_i64, slot);
            f.tok = sub << p.frag_shift;
            f.outer = static_cast<int>(page);
            f.state = (page >= 0 && page < p.seq.num_pages) ? 1 : 2;
            if (pc_kvh == 0 && sub == 0) f.trace_idx = slot;
        } else {
            const unsigned bi = vfrag >> p.fpu_shift;
            const int sub = static_cast<int>(vfrag - (bi << p.fpu_shift));
            int blk;
            if (p.seq.blocks_dev != nullptr) {  // the pair's own list, written by a kernel before this one
                const int64_t pair = static_cast<int64_t>(pc_b) * p.seq.blocks_kv_heads + f.kvh;
                blk = p.seq.blocks_dev[pair * p.seq.num_blocks + bi];
            } else {
                blk = p.seq.blocks[bi];
            }
            f.tok = blk * p.seq.block_size + (sub << p.frag_shift);
            f.outer = pc_b;
            // A device list cannot be checked by the host: blocks outside the cache are skipped and reported.
            f.state = (blk >= 0 && static_cast<int64_t>(f.tok) < p.seq.kv_len) ? 1 : 2;
        }
        return f;
    };

    // Issue the TMA copies of the warp's j-th tile into ring slot j % STAGES.
    auto issue = [&](int j, const Frag &f) {
        const uint32_t slot = static_cast<uint32_t>(j) % STAGES;
        const uint32_t stage = ring_u32 + slot * kStageBytes;
        const uint32_t bar = bar_u32 + slot * 8;
        const bool ok = f.state == 1;
        if (f.state == 2) atomicOr(p.status, SA_DEV_BAD_PAGE);
        if (ok && p.trace != nullptr && f.trace_idx >= 0) p.trace[f.trace_idx] = static_cast<int32_t>(f.outer);
        const unsigned mask = __ballot_sync(0xffffffffu, ok);
        if (lane == 0)
            mbar_arrive_expect_tx(bar, static_cast<uint32_t>(__popc(mask)) * p.frag_tokens * 128 * HALVES * 2);
        __syncwarp();
        if (ok) {
            const uint32_t dst = stage + lane * p.frag_tokens * 128;
            const int c1 = p.tok_dim == 1 ? f.tok : f.kvh;
            const int c2 = p.tok_dim == 1 ? f.kvh : f.tok;
#pragma unroll
            for (int hf = 0; hf < HALVES; ++hf) {
                tma_load_4d(dst + hf * HALF_BYTES, &tm_k, bar, hf * 64, c1, c2, f.outer, policy);
                tma_load_4d(dst + kTileBytes + hf * HALF_BYTES, &tm_v, bar, hf * 64, c1, c2, f.outer, policy);
            }
        }
    };

    // Rows of one length: the dependency wait (see the note at launch_dependents) comes here, or
    // - when working out the first tiles' coordinates reads no memory either (no device-resident
    // block lists, no claim counter) - after that as well.
    const bool lookups_first = !ragged && p.seq.blocks_dev == nullptr && !dyn_claims;
    if (!ragged && !lookups_first) asm volatile("griddepcontrol.wait;" ::: "memory");
    // Fill the ring before anything else so HBM is busy while the rest of the prologue runs.
    Frag first[STAGES + 1];
#pragma unroll
    for (int s = 0; s <= STAGES; ++s) first[s] = lookup(next_tile());  // all table loads in flight together
    if (lookups_first) asm volatile("griddepcontrol.wait;" ::: "memory");
    int xq[STAGES];  // tiles in the ring, oldest first
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
        xq[s] = first[s].x;
        if (xq[s] >= 0) issue(s, first[s]);
    }
    Frag pending = first[STAGES];
    SA_STAMP(1);

    // Rows with no tokens are not part of the tile list: write their (empty) result here.
    // Rows left out by a row subset (length -1) are not written at all.
    for (int b = c; b < p.batch; b += C) {
        if (tiles_before(b + 1) != tiles_before(b)) continue;
        if (ragged && vlens[b] < 0) continue;
        for (int i = tid; i < p.q_heads * D; i += NTHREADS) {
            const int h = i / D, d = i % D;
            if (p.out_mode == SA_OUT_FINAL)
                static_cast<T *>(p.out)[(static_cast<int64_t>(b) * p.q_heads + h) * D + d] = Elem<T>::from_float(0.0f);
            else
                static_cast<float *>(p.out)[(static_cast<int64_t>(b) * p.q_heads + h) * STATE_STRIDE + d] = 0.0f;
        }
        if (p.out_mode != SA_OUT_FINAL) {
            for (int h = tid; h < p.q_heads; h += NTHREADS) {
                float *st = static_cast<float *>(p.out) + (static_cast<int64_t>(b) * p.q_heads + h) * STATE_STRIDE;
                st[D] = -INFINITY;
                st[D + 1] = 0.0f;
            }
        }
    }

    int cur = lo;
    int j = 0;          // next tile of this warp to consume
    bool dead = false;  // a bounded wait gave up: stop computing, keep the CTA barriers

    while (cur < hi) {
        // The segment: tiles [cur, seg_end) of one (row, kv head) pair.
        int b, kvh, row_tiles, pair_start;
        if (aligned) {
            b = al_pair / Hkv;
            kvh = al_pair - b * Hkv;
            pair_start = al_start;
            row_tiles = al_end - al_start;
        } else {
            locate(cur, b, kvh, row_tiles, pair_start);
        }
        const int pair_end = pair_start + row_tiles;
        const int seg_end = hi < pair_end ? hi : pair_end;
        const int pair = b * Hkv + kvh;
        const int64_t vlen = vlen_of(b);

        // Query fragments of this KV group (A operand of q.k), rows >= group are zero.
        uint32_t qa[KS_QK][4];
        {
            const T *qrow0 = static_cast<const T *>(p.q) + b * p.q_sb + (static_cast<int64_t>(kvh) * group + g) * p.q_sh;
            const T *qrow1 = qrow0 + 8 * p.q_sh;
            const bool ok0 = g < group;
            const bool ok1 = ROWS16 && (g + 8 < group);
#pragma unroll
            for (int ks = 0; ks < KS_QK; ++ks) {
                const int col = ks * 16 + 2 * t4;
                qa[ks][0] = ok0 ? *reinterpret_cast<const uint32_t *>(qrow0 + col) : 0u;
                qa[ks][1] = ok1 ? *reinterpret_cast<const uint32_t *>(qrow1 + col) : 0u;
                qa[ks][2] = ok0 ? *reinterpret_cast<const uint32_t *>(qrow0 + col + 8) : 0u;
                qa[ks][3] = ok1 ? *reinterpret_cast<const uint32_t *>(qrow1 + col + 8) : 0u;
            }
        }

        float m_run[2] = {-INFINITY, -INFINITY};
        float l_run[2] = {0.0f, 0.0f};
        float o_acc[NT_O][4];
#pragma unroll
        for (int i = 0; i < NT_O; ++i) {
            o_acc[i][0] = 0.0f;
            o_acc[i][1] = 0.0f;
            o_acc[i][2] = 0.0f;
            o_acc[i][3] = 0.0f;
        }

        for (;; ++j) {
            const int x = xq[0];
            if (x < 0 || x >= seg_end) break;
            const int lt = x - pair_start;
            const uint32_t slot = static_cast<uint32_t>(j) % STAGES;
            const uint32_t parity = (static_cast<uint32_t>(j) / STAGES) & 1u;
            const uint32_t kb = ring_u32 + slot * kStageBytes;
            const uint32_t vb = kb + kTileBytes;
            if (!dead && !mbar_wait(bar_u32 + slot * 8, parity, p.wait_ns)) {
                dead = true;
                atomicOr(p.status, SA_DEV_PIPELINE_TIMEOUT);
            }
            dead = __any_sync(0xffffffffu, dead);
            if (dead) {  // drop everything that is left; the status word tells the caller
#pragma unroll
                for (int s = 0; s < STAGES; ++s) xq[s] = -1;
                pending.x = -1;
                claiming = false;
                chunk_left = 0;
                seq_i = n_w;
                break;
            }

            const int64_t tile_tok0 = static_cast<int64_t>(lt) * TILE_N;
            const int n_valid = vlen - tile_tok0 < TILE_N ? static_cast<int>(vlen - tile_tok0) : TILE_N;
            const bool tail = n_valid < TILE_N;

            // scores: S[16 rows = heads, TILE_N tokens] = Q K^T
            float s_acc[NT_S][4];
#pragma unroll
            for (int nt = 0; nt < NT_S; ++nt) {
                s_acc[nt][0] = 0.0f;
                s_acc[nt][1] = 0.0f;
                s_acc[nt][2] = 0.0f;
                s_acc[nt][3] = 0.0f;
#pragma unroll
                for (int kk = 0; kk < KS_QK / 2; ++kk) {
                    const int chunk = kk * 4 + (lane >> 3);
                    const int row = nt * 8 + (lane & 7);
                    const uint32_t addr =
                        kb + (chunk >> 3) * HALF_BYTES + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
                    uint32_t r0, r1, r2, r3;
                    ldmatrix_x4(addr, r0, r1, r2, r3);
                    Mma<T>::run(s_acc[nt], qa[2 * kk], r0, r1);
                    Mma<T>::run(s_acc[nt], qa[2 * kk + 1], r2, r3);
                }
            }

            if (tail) {
                // Mask tokens past the row length and clear their V rows so that stale or
                // never-written shared memory cannot reach the accumulators.
#pragma unroll
                for (int nt = 0; nt < NT_S; ++nt) {
                    const int col = nt * 8 + 2 * t4;
                    if (col >= n_valid) {
                        s_acc[nt][0] = -INFINITY;
                        s_acc[nt][2] = -INFINITY;
                    }
                    if (col + 1 >= n_valid) {
                        s_acc[nt][1] = -INFINITY;
                        s_acc[nt][3] = -INFINITY;
                    }
                }
                uint8_t *vtile = warp_ring + slot * kStageBytes + kTileBytes;
                const int chunks = (TILE_N - n_valid) * 8;
                for (int hf = 0; hf < HALVES; ++hf)
                    for (int i = lane; i < chunks; i += 32)
                        *reinterpret_cast<uint4 *>(vtile + hf * HALF_BYTES + n_valid * 128 + i * 16) =
                            make_uint4(0u, 0u, 0u, 0u);
                __syncwarp();
            }

            // online softmax (base-2 domain), rows g and (ROWS16) g+8
            uint32_t pa[KS_PV][4];
            {
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int nt = 0; nt < NT_S; ++nt) {
                    mx0 = fmaxf(mx0, fmaxf(s_acc[nt][0], s_acc[nt][1]));
                    if (ROWS16) mx1 = fmaxf(mx1, fmaxf(s_acc[nt][2], s_acc[nt][3]));
                }
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                if (ROWS16) {
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                }
                const float m_new0 = fmaxf(m_run[0], mx0 * p.scale_log2);
                const float alpha0 = exp2_diff(m_run[0], m_new0);
                const float neg_m0 = m_new0 == -INFINITY ? 0.0f : -m_new0;
                float m_new1 = -INFINITY, alpha1 = 0.0f, neg_m1 = 0.0f;
                if (ROWS16) {
                    m_new1 = fmaxf(m_run[1], mx1 * p.scale_log2);
                    alpha1 = exp2_diff(m_run[1], m_new1);
                    neg_m1 = m_new1 == -INFINITY ? 0.0f : -m_new1;
                }
                float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
                for (int nt = 0; nt < NT_S; ++nt) {
                    const float p0 = exp2f(fmaf(s_acc[nt][0], p.scale_log2, neg_m0));
                    const float p1 = exp2f(fmaf(s_acc[nt][1], p.scale_log2, neg_m0));
                    sum0 += p0 + p1;
                    float p2 = 0.0f, p3 = 0.0f;
                    if (ROWS16) {
                        p2 = exp2f(fmaf(s_acc[nt][2], p.scale_log2, neg_m1));
                        p3 = exp2f(fmaf(s_acc[nt][3], p.scale_log2, neg_m1));
                        sum1 += p2 + p3;
                    }
                    const int kt = nt >> 1;
                    const int hi_half = (nt & 1) * 2;
                    pa[kt][hi_half] = Mma<T>::pack(p0, p1);
                    pa[kt][hi_half + 1] = ROWS16 ? Mma<T>::pack(p2, p3) : 0u;
                }
                l_run[0] = l_run[0] * alpha0 + sum0;
                m_run[0] = m_new0;
                if (ROWS16) {
                    l_run[1] = l_run[1] * alpha1 + sum1;
                    m_run[1] = m_new1;
                }
#pragma unroll
                for (int i = 0; i < NT_O; ++i) {
                    o_acc[i][0] *= alpha0;
                    o_acc[i][1] *= alpha0;
                    if (ROWS16) {
                        o_acc[i][2] *= alpha1;
                        o_acc[i][3] *= alpha1;
                    }
                }
            }

            // O[16 rows, D] += P V
#pragma unroll
            for (int kt = 0; kt < KS_PV; ++kt) {
#pragma unroll
                for (int dp = 0; dp < NT_O / 2; ++dp) {
                    const int row = kt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    const int chunk = dp * 2 + (lane >> 4);
                    const uint32_t addr =
                        vb + (chunk >> 3) * HALF_BYTES + row * 128 + (((chunk & 7) ^ (row & 7)) << 4);
                    uint32_t r0, r1, r2, r3;
                    ldmatrix_x4_trans(addr, r0, r1, r2, r3);
                    Mma<T>::run(o_acc[2 * dp], pa[kt], r0, r1);
                    Mma<T>::run(o_acc[2 * dp + 1], pa[kt], r2, r3);
                }
            }

            // Order this warp's shared-memory accesses before the async-proxy writes of the refill.
            fence_proxy_async();
            __syncwarp();
            if (pending.x >= 0) issue(j + STAGES, pending);
#pragma unroll
            for (int s = 0; s + 1 < STAGES; ++s) xq[s] = xq[s + 1];
            xq[STAGES - 1] = pending.x;
            pending = lookup(next_tile());
        }

        SA_STAMP(3);
        // Warp state -> the warp's state area: [ROWS][D+2] floats = (o, m, l).
        {
            l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1);
            l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
            if (ROWS16) {
                l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 1);
                l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 2);
            }
            float *area = states + warp * STATE_FLOATS;
#pragma unroll
            for (int i = 0; i < NT_O; ++i) {
                const int d = i * 8 + 2 * t4;
                *reinterpret_cast<float2 *>(area + g * STATE_STRIDE + d) = make_float2(o_acc[i][0], o_acc[i][1]);
                if (ROWS16)
                    *reinterpret_cast<float2 *>(area + (g + 8) * STATE_STRIDE + d) =
                        make_float2(o_acc[i][2], o_acc[i][3]);
            }
            if (t4 == 0) {
                area[g * STATE_STRIDE + D] = m_run[0];
                area[g * STATE_STRIDE + D + 1] = l_run[0];
                if (ROWS16) {
                    area[(g + 8) * STATE_STRIDE + D] = m_run[1];
                    area[(g + 8) * STATE_STRIDE + D + 1] = l_run[1];
                }
            }
        }
        __syncthreads();
        SA_STAMP(4);

        // Combine the warps of this CTA, then either finish the pair or publish a state.
        // Work items are 4 consecutive columns of one head row.
        const int first_cta = aligned ? al_first : owner(pair_start);
        const int nseg = aligned ? al_nseg : owner(pair_end - 1) - first_cta + 1;
        const int64_t slot_stride = static_cast<int64_t>(group) * PART_STRIDE;
        float *my_slot = p.partials + (static_cast<int64_t>(c) + pair) * slot_stride;
        const int64_t out_row0 = static_cast<int64_t>(b) * p.q_heads + static_cast<int64_t>(kvh) * group;
        const bool cp_on = p.cp.world > 0;
        auto store_result = [&](int row, int d4, const float4 &acc, float big, float total_l) {
            if (p.out_mode == SA_OUT_FINAL) {
                const float inv = total_l > 0.0f ? 1.0f / total_l : 0.0f;
                T *dst = static_cast<T *>(p.out) + (out_row0 + row) * D + d4;
                *reinterpret_cast<uint2 *>(dst) =
                    make_uint2(Mma<T>::pack(acc.x * inv, acc.y * inv), Mma<T>::pack(acc.z * inv, acc.w * inv));
            } else if (cp_on) {
                // Context-parallel: the pair's state rows are staged in shared memory as tagged
                // words; cp_broadcast_pair() then sends them to every rank's gather buffer with
                // wide, lane-contiguous stores.
                uint64_t *dst = cp_stage + row * STATE_STRIDE;
                dst[d4] = cp_word(acc.x, p.cp.step);
                dst[d4 + 1] = cp_word(acc.y, p.cp.step);
                dst[d4 + 2] = cp_word(acc.z, p.cp.step);
                dst[d4 + 3] = cp_word(acc.w, p.cp.step);
                if (d4 == 0) {
                    dst[D] = cp_word(big, p.cp.step);
                    dst[D + 1] = cp_word(total_l, p.cp.step);
                }
            } else {
                float *dst = static_cast<float *>(p.out) + (out_row0 + row) * STATE_STRIDE;
                *reinterpret_cast<float2 *>(dst + d4) = make_float2(acc.x, acc.y);
                *reinterpret_cast<float2 *>(dst + d4 + 2) = make_float2(acc.z, acc.w);
                if (d4 == 0) *reinterpret_cast<float2 *>(dst + D) = make_float2(big, total_l);
            }
        };
        const int items = group * (D / 4);
        // The pair's ticket is taken now, before this CTA's state is even combined: it counts the
        // CTAs that have finished streaming and elects the last of them as the merger.  The
        // merger recognises a state that has landed by its contents, so the ticket orders
        // nothing, and its round trip overlaps the combine below.  (Asking for it earlier still -
        // when the last tile of warp 0 lands, or right after the tile loop - measured slower: the
        // merger then looks before the last states have landed and pays a second round trip.)
        // That is the form for grids larger than the GPU.  When every CTA can be resident at once
        // (p.first_merges) there is no ticket at all: the pair's first CTA merges, whenever it is
        // done itself, and simply looks until the others' states have landed - the last CTA to
        // finish only has to store its state.
        int old_count = 0;
        if (nseg > 1 && tid == 0 && !p.first_merges)
            asm volatile("atom.add.relaxed.gpu.global.s32 %0, [%1], 1;"
                         : "=r"(old_count)
                         : "l"(p.counters + pair)
                         : "memory");
        // The thread keeps the items it combined (OWN of them at most) and parks them in shared
        // memory once the warps' areas are free: if this CTA turns out to be the one that merges
        // the pair, its own state never has to come back from global memory.
        float own[OWN][6];
#pragma unroll
        for (int k = 0; k < OWN; ++k) {
#pragma unroll
            for (int e = 0; e < 6; ++e) own[k][e] = 0.0f;
            const int item = tid + k * NTHREADS;
            if (item >= items) continue;
            const int row = item / (D / 4);
            const int d4 = (item - row * (D / 4)) * 4;
            float big = -INFINITY;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) big = fmaxf(big, states[w * STATE_FLOATS + row * STATE_STRIDE + D]);
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            float total_l = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                const float *area = states + w * STATE_FLOATS + row * STATE_STRIDE;
                const float wgt = exp2_diff(area[D], big);
                const float2 lo2 = *reinterpret_cast<const float2 *>(area + d4);
                const float2 hi2 = *reinterpret_cast<const float2 *>(area + d4 + 2);
                acc.x += wgt * lo2.x;
                acc.y += wgt * lo2.y;
                acc.z += wgt * hi2.x;
                acc.w += wgt * hi2.y;
                total_l += wgt * area[D + 1];
            }
            if (nseg == 1) {
                store_result(row, d4, acc, big, total_l);
            } else {
                // Publish with inverted bits: a word that reads non-zero has landed (state_load4).
                float *dst = my_slot + row * PART_STRIDE;
                state_store4(dst + d4, inv_bits(acc.x), inv_bits(acc.y), inv_bits(acc.z), inv_bits(acc.w));
                if (d4 == 0) state_store2(dst + D, inv_bits(big), inv_bits(total_l));
                own[k][0] = acc.x; own[k][1] = acc.y; own[k][2] = acc.z; own[k][3] = acc.w;
                own[k][4] = big; own[k][5] = total_l;
            }
        }

        if (nseg == 1 && tid == 0) {
            s_last = 0;
            if (dyn_claims) p.pool[pair] = 0;  // every warp of the only CTA has made its last claim
        }
        if (nseg > 1) {
            __syncthreads();  // the warps' state areas have been read by everybody
#pragma unroll
            for (int k = 0; k < OWN; ++k) {
                const int item = tid + k * NTHREADS;
                if (item < items) {
                    float *dst = states + item * 6;
                    *reinterpret_cast<float2 *>(dst) = make_float2(own[k][0], own[k][1]);
                    *reinterpret_cast<float2 *>(dst + 2) = make_float2(own[k][2], own[k][3]);
                    *reinterpret_cast<float2 *>(dst + 4) = make_float2(own[k][4], own[k][5]);
                }
            }
            if (tid == 0) s_last = p.first_merges ? c == first_cta : old_count == nseg - 1;
            __syncthreads();
            SA_STAMP(5);
            if (s_last) {
                // Last CTA to arrive on this pair: exact merge of its nseg split states.
                float *first_slot = p.partials + (static_cast<int64_t>(first_cta) + pair) * slot_stride;
#pragma unroll
                for (int k = 0; k < OWN; ++k) {
                    const int r0 = k * MERGE_ROWS;
                    if (r0 >= group) continue;
                    const int n_rows = group - r0 < MERGE_ROWS ? group - r0 : MERGE_ROWS;
                    const int sub_items = n_rows * (D / 4);
                    // States each thread has to fetch: the batch size that covers them in one pass.
                    const int sharers = static_cast<int>(
                        (static_cast<float>(MERGE_ROWS) + 0.5f) * __frcp_rn(static_cast<float>(n_rows)));  // threads per item
                    const int per_thread = static_cast<int>(
                        (static_cast<float>(nseg + sharers - 1) + 0.5f) * __frcp_rn(static_cast<float>(sharers)));
                    float *slots = first_slot + r0 * PART_STRIDE;
                    const float *mine = states + k * NTHREADS * 6;
                    if (per_thread <= 3)
                        merge_pair_states<D, NTHREADS, 3>(slots, slot_stride, nseg, c - first_cta, mine,
                                                                  sub_items, scratch, tid, p.wait_ns, p.status);
                    else if (per_thread <= 6)
                        merge_pair_states<D, NTHREADS, 6>(slots, slot_stride, nseg, c - first_cta, mine,
                                                                  sub_items, scratch, tid, p.wait_ns, p.status);
                    else
                        merge_pair_states<D, NTHREADS, 10>(slots, slot_stride, nseg, c - first_cta, mine,
                                                                   sub_items, scratch, tid, p.wait_ns, p.status);
                    if (tid < sub_items) {
                        const int row = tid / (D / 4);
                        const float *r = scratch + tid * 6;
                        store_result(r0 + row, (tid - row * (D / 4)) * 4, make_float4(r[0], r[1], r[2], r[3]), r[4],
                                     r[5]);
                    }
                    __syncthreads();  // the scratch is reused by the next rows
                }
                if (tid == 0) {  // ready for the next launch: every CTA of the pair has arrived
                    if (!p.first_merges) p.counters[pair] = 0;
                    if (dyn_claims) p.pool[pair] = 0;
                }
            }
        }
        if (cp_on && (nseg == 1 || s_last)) {
            __syncthreads();  // the pair's rows are complete in the staging area
            cp_broadcast_pair<NTHREADS>(
                p.cp, cp_stage,
                (p.cp.step & 1u) * p.cp.gather_words_per_parity +
                    (static_cast<size_t>(p.cp.rank) * p.batch * p.q_heads + out_row0) * STATE_STRIDE,
                group * STATE_STRIDE, tid);
            cp_finish_pair<T, D, NTHREADS>(p.cp, p.status, p.wait_ns, static_cast<size_t>(p.batch) * p.q_heads,
                                           out_row0, items, scratch, tid);
        }
        __syncthreads();  // the state areas, the scratch and s_last are reused by the next segment
        SA_STAMP(6);
        cur = seg_end;
    }
}

template <typename T, int D, int WARPS, int STAGES, bool ROWS16>
cudaError_t launch_instance(const CUtensorMap &mk, const CUtensorMap &mv, const StreamParams &sp, int ctas,
                            int batch, cudaStream_t stream)
{
    auto kernel = stream_decode_kernel<T, D, WARPS, STAGES, ROWS16>;
    const size_t smem = stream_smem_bytes(D, ROWS16, STAGES, batch);
    // Opt in to the dynamic shared memory this launch needs (grows only; per device).
    static std::mutex mu;
    static size_t configured[64] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (configured[dev] < smem) {
            err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
            if (err != cudaSuccess) return err;
            configured[dev] = smem;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(ctas));
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    // STREAMATTN_B200_NO_PDL=1 launches with plain stream serialization (for A/B timing).
    static const int overlap_launch = std::getenv("STREAMATTN_B200_NO_PDL") ? 0 : 1;
    attr[0].val.programmaticStreamSerializationAllowed = overlap_launch;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, mk, mv, sp);
}

template <typename T, int D>
cudaError_t launch_dim(const CUtensorMap &mk, const CUtensorMap &mv, const StreamParams &sp, int ctas, int batch,
                       bool rows16, cudaStream_t stream)
{
    if (rows16) {
        // 16 head rows at D128 need 33 KB of state areas: two ring stages instead of three.
        constexpr int kStages16 = (D == 128 && kStreamStages > 2) ? 2 : kStreamStages;
        return launch_instance<T, D, kStreamWarps, kStages16, true>(mk, mv, sp, ctas, batch, stream);
    }
    return launch_instance<T, D, kStreamWarps, kStreamStages, false>(mk, mv, sp, ctas, batch, stream);
}

}  // namespace

#ifdef SA_TIMELINE
// Instrumented builds only: where the kernels write their per-CTA time stamps (16 words per CTA).
unsigned long long *g_timeline = nullptr;
extern "C" __attribute__((visibility("default"))) void sa_debug_timeline(void *ptr)
{
    g_timeline = static_cast<unsigned long long *>(ptr);
}
#endif

int stream_kv_split(int group)
{
    for (int s = 1; s <= group; ++s)
        if (group % s == 0 && group / s <= 16) return s;
    return 0;
}

int stream_tile_tokens(int head_dim) { return kTileBytes / (head_dim * 2); }

int stream_stages(int head_dim, bool rows16)
{
    return (head_dim == 128 && rows16 && kStreamStages > 2) ? 2 : kStreamStages;
}

size_t stream_smem_bytes(int head_dim, bool rows16, int stages, int batch)
{
    const size_t bars = (static_cast<size_t>(kStreamWarps) * stages * 8 + 15) / 16 * 16;
    // Per-warp (o, m, l) areas plus the context-parallel staging rows (8-byte words).
    const size_t states = (static_cast<size_t>(kStreamWarps) + 2) * (rows16 ? 16 : 8) * (head_dim + 2) * 4;
    const size_t scratch = static_cast<size_t>(kStreamWarps) * 32 * 6 * 4;  // merges: 6 floats per thread
    return 1024 + static_cast<size_t>(kStreamWarps) * stages * kStageBytes + bars + states + scratch +
           (2 * static_cast<size_t>(batch) + 1) * 4 + 16;
}

cudaError_t launch_stream(const Problem &p, const StreamGeometry &geo, const CpFuse &cp, cudaStream_t stream)
{
    StreamParams sp;
    sp.q = p.q;
    sp.q_sb = p.q_sb;
    sp.q_sh = p.q_sh;
    sp.out = p.out;
    sp.out_mode = p.out_mode;
    sp.partials = p.ws.partials;
    sp.counters = p.ws.counters;
    sp.pool = p.ws.counters + static_cast<size_t>(p.batch) * p.q_heads;
    sp.status = p.ws.status;
    sp.trace = p.trace;
    sp.batch = p.batch;
    sp.q_heads = p.q_heads;
    sp.kv_heads = p.kv_heads * geo.kv_split;
    sp.group = p.q_heads / sp.kv_heads;
    sp.kv_split = geo.kv_split;
    sp.scale_log2 = kLog2e / sqrtf(static_cast<float>(p.head_dim));
    sp.frag_tokens = geo.frag_tokens;
    sp.frags_per_tile = geo.frags_per_tile;
    sp.frags_per_unit = geo.frags_per_unit;
    auto log2i = [](int x) { int s = 0; while ((1 << s) < x) ++s; return s; };
    sp.frag_shift = log2i(geo.frag_tokens);
    sp.fpt_shift = log2i(geo.frags_per_tile);
    sp.fpu_shift = log2i(geo.frags_per_unit);
    sp.tok_dim = geo.tok_dim;
    // A row subset makes the rows' tile counts differ (rows left out have none).
    sp.uniform_tiles = p.seq.num_rows >= 0 ? -1 : geo.uniform_tiles;
    sp.schedule = geo.schedule;
    sp.wait_ns = p.wait_ns;
    sp.first_merges = geo.first_merges;
    sp.seq = p.seq;
    sp.cp = cp;
#ifdef SA_TIMELINE
    sp.timeline = g_timeline;
#endif
    const bool rows16 = sp.group > 8;
    if (p.dtype == SA_DTYPE_BF16) {
        if (p.head_dim == 64)
            return launch_dim<__nv_bfloat16, 64>(geo.map_k, geo.map_v, sp, geo.num_ctas, p.batch, rows16, stream);
        return launch_dim<__nv_bfloat16, 128>(geo.map_k, geo.map_v, sp, geo.num_ctas, p.batch, rows16, stream);
    }
    if (p.head_dim == 64)
        return launch_dim<__half, 64>(geo.map_k, geo.map_v, sp, geo.num_ctas, p.batch, rows16, stream);
    return launch_dim<__half, 128>(geo.map_k, geo.map_v, sp, geo.num_ctas, p.batch, rows16, stream);
}

}  // namespace sa
