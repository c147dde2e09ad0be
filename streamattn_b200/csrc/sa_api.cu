// C-ABI entry points: argument validation, workspace layout, kernel selection,
// TMA tensor-map construction and bound plans.  No torch types cross this file.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "sa_append.cuh"
#include "sa_stream.cuh"

namespace sa {
namespace {

thread_local char g_error[512] = "";
thread_local bool g_workspace_too_small = false;  // why the last finish_plan() on this thread failed
std::atomic<unsigned long long> g_default_wait_ns{kDefaultWaitNs};

int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

int fail_cuda(cudaError_t err, const char *what)
{
    return fail(SA_ERR_CUDA, "%s: %s", what, cudaGetErrorString(err));
}

size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

int generic_splits_bound(int64_t pairs, int num_ctas)
{
    int64_t want = num_ctas > 0 ? num_ctas : 4LL * kMaxAutoCtas;
    int64_t s = (want + pairs - 1) / pairs;
    s = std::min<int64_t>(std::max<int64_t>(s, 1), kMaxGenericSplits);
    return static_cast<int>(s);
}

// Arrival counters [batch*q_heads] followed by the dynamic schedule's claim counters [batch*q_heads].
size_t counters_bytes(int batch, int q_heads) { return round_up(static_cast<size_t>(batch) * q_heads * 8, 256); }

size_t stream_partial_floats(int batch, int q_heads, int kv_heads, int head_dim, int ctas)
{
    const size_t group = static_cast<size_t>(q_heads / kv_heads);
    return (static_cast<size_t>(ctas) + static_cast<size_t>(batch) * kv_heads) * group * (head_dim + 4);
}

size_t workspace_bytes_impl(int batch, int q_heads, int kv_heads, int head_dim, int num_ctas)
{
    const int ctas = num_ctas > 0 ? std::min(num_ctas, kMaxCtas) : kMaxAutoCtas;
    const int64_t pairs = static_cast<int64_t>(batch) * q_heads;
    const int split = std::max(1, stream_kv_split(q_heads / kv_heads));
    const size_t a = stream_partial_floats(batch, q_heads, kv_heads * split, head_dim, ctas);
    const size_t b = generic_partial_floats(batch, q_heads, head_dim, generic_splits_bound(pairs, num_ctas));
    return kStatusWords * 4 + counters_bytes(batch, q_heads) + round_up(std::max(a, b) * 4, 256);
}

int device_sm_count()
{
    static std::mutex mu;
    static int cache[64];
    static bool have[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    std::lock_guard<std::mutex> lock(mu);
    if (!have[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        cache[dev] = n;
        have[dev] = true;
    }
    return cache[dev];
}

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn()
{
    static std::once_flag once;
    static EncodeTiledFn fn = nullptr;
    std::call_once(once, [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

// 4-D map (column, x1, x2, outer) over a bf16/f16 cache with 128-byte swizzled boxes
// of 64 columns x `box_tokens` tokens; tok_dim says which of x1/x2 is the token axis.
bool encode_map(CUtensorMap *map, int dtype, const void *base, const uint64_t dims[4], const uint64_t strides[3],
                int tok_dim, int box_tokens)
{
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return false;
    if (reinterpret_cast<uintptr_t>(base) % 16) return false;
    cuuint64_t gdim[4] = {dims[0], dims[1], dims[2], dims[3]};
    cuuint64_t gstr[3] = {strides[0] * 2, strides[1] * 2, strides[2] * 2};
    for (int i = 0; i < 4; ++i)
        if (gdim[i] == 0 || gdim[i] > (1ull << 32)) return false;
    for (int i = 0; i < 3; ++i)
        if (gstr[i] == 0 || gstr[i] % 16 || gstr[i] >= (1ull << 40)) return false;
    cuuint32_t box[4] = {64, 1, 1, 1};
    box[tok_dim] = static_cast<cuuint32_t>(box_tokens);
    cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUtensorMapDataType dt =
        dtype == SA_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult rc = fn(map, dt, 4, const_cast<void *>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS;
}

bool is_pow2(int64_t x) { return x > 0 && (x & (x - 1)) == 0; }

}  // namespace
}  // namespace sa

struct sa_plan {
    sa::Problem problem;
    int device;  // device that was current when the plan was made
    mutable sa::CpFuse cp;  // cp.world == 0 unless made by sa_cp_fused_plan_create; cp.step counts runs
    bool use_stream;
    sa::StreamGeometry geo;
    int generic_splits;
    int64_t max_vlen;
};

namespace sa {
namespace {

// Decide whether the streaming kernel covers the problem and, if so, build its geometry.
bool build_stream_geometry(const Problem &p, int64_t max_vlen, StreamGeometry *geo, const char **why)
{
    *why = "";
    if (p.dtype != SA_DTYPE_BF16 && p.dtype != SA_DTYPE_F16) { *why = "dtype is not bf16/fp16"; return false; }
    if (p.head_dim != 64 && p.head_dim != 128) { *why = "head_dim is not 64 or 128"; return false; }
    geo->kv_split = stream_kv_split(p.q_heads / p.kv_heads);
    if (geo->kv_split == 0) { *why = "query heads per KV head cannot be split into groups of at most 16"; return false; }
    const int group = p.q_heads / p.kv_heads / geo->kv_split;  // per virtual KV head
    if (p.batch > 8192) { *why = "batch larger than 8192"; return false; }
    if (stream_smem_bytes(p.head_dim, group > 8, stream_stages(p.head_dim, group > 8), p.batch) > kStreamSmemLimit) {
        *why = "batch too large for the shared-memory schedule table";
        return false;
    }
    if (reinterpret_cast<uintptr_t>(p.q) % 4 || p.q_sb % 2 || p.q_sh % 2) { *why = "query not 4-byte aligned"; return false; }
    if (reinterpret_cast<uintptr_t>(p.out) % 16) { *why = "output not 16-byte aligned"; return false; }
    if (max_vlen <= 0 || max_vlen >= (1ll << 31)) { *why = "sequence length out of range"; return false; }
    const int tile = stream_tile_tokens(p.head_dim);
    const SeqDesc &s = p.seq;
    const uint64_t D = static_cast<uint64_t>(p.head_dim);
    uint64_t dims[4];
    uint64_t strides[3];
    int unit = tile;
    if (s.mode == kPaged) {
        unit = s.page_size;
        if (!is_pow2(unit) || unit < 8) { *why = "page_size is not a power of two >= 8"; return false; }
        if (s.pg_st <= s.pg_sh) {  // HND: [page][head][slot][D]
            dims[0] = D; dims[1] = unit; dims[2] = p.kv_heads; dims[3] = s.num_pages;
            strides[0] = s.pg_st; strides[1] = s.pg_sh; strides[2] = s.pg_sp;
            geo->tok_dim = 1;
        } else {                   // NHD: [page][slot][head][D]
            dims[0] = D; dims[1] = p.kv_heads; dims[2] = unit; dims[3] = s.num_pages;
            strides[0] = s.pg_sh; strides[1] = s.pg_st; strides[2] = s.pg_sp;
            geo->tok_dim = 2;
        }
    } else {
        if (s.mode == kBlocks) {
            unit = s.block_size;
            if (!is_pow2(unit) || unit < 8) { *why = "block_size is not a power of two >= 8"; return false; }
        }
        if (s.kv_len >= (1ll << 31)) { *why = "kv_len too large"; return false; }
        int64_t sn = s.kv_sn, sh = s.kv_sh, sb = s.kv_sb;
        if (sn <= 0 || sh < 0 || sb < 0) { *why = "non-positive KV stride"; return false; }
        // Size-1 axes may carry arbitrary strides; give them a harmless ascending one.
        if (p.kv_heads == 1) sh = sn * s.kv_len;
        if (sn <= sh) {
            if (p.batch == 1) sb = sh * p.kv_heads;
            dims[0] = D; dims[1] = s.kv_len; dims[2] = p.kv_heads; dims[3] = p.batch;
            strides[0] = sn; strides[1] = sh; strides[2] = sb;
            geo->tok_dim = 1;
        } else {
            if (p.batch == 1) sb = sn * s.kv_len;
            dims[0] = D; dims[1] = p.kv_heads; dims[2] = s.kv_len; dims[3] = p.batch;
            strides[0] = sh; strides[1] = sn; strides[2] = sb;
            geo->tok_dim = 2;
        }
    }
    geo->frag_tokens = std::min(unit, tile);
    geo->frags_per_tile = tile / geo->frag_tokens;
    geo->frags_per_unit = s.mode == kContig ? 1 : std::max(1, unit / geo->frag_tokens);
    const bool uniform = s.mode == kBlocks || (s.mode == kContig && s.seq_lens == nullptr);
    geo->uniform_tiles = uniform ? static_cast<int>((max_vlen + tile - 1) / tile) : -1;
    if (!encode_map(&geo->map_k, p.dtype, p.k, dims, strides, geo->tok_dim, geo->frag_tokens) ||
        !encode_map(&geo->map_v, p.dtype, p.v, dims, strides, geo->tok_dim, geo->frag_tokens)) {
        *why = "cache pointers/strides do not satisfy the TMA alignment rules";
        return false;
    }
    const int64_t tiles = static_cast<int64_t>(p.batch) * p.kv_heads * geo->kv_split * ((max_vlen + tile - 1) / tile);
    if (tiles >= (1ll << 30)) { *why = "more than 2^30 tiles"; return false; }
    int64_t ctas;
    if (p.num_ctas > 0) {
        ctas = std::min<int64_t>(p.num_ctas, kMaxCtas);
    } else {
        const int sm = p.sm_count > 0 ? std::min(p.sm_count, kMaxAutoCtas) : 148;
        // Small problems are latency-bound: spread them over many CTAs (four tiles each, so
        // half of a CTA's warps may stay idle) rather than filling every warp of a few CTAs.
        constexpr int kMinTilesPerCta = 4;
        ctas = std::min<int64_t>(sm, (tiles + kMinTilesPerCta - 1) / kMinTilesPerCta);
    }
    ctas = std::max<int64_t>(1, std::min<int64_t>(ctas, tiles));
    geo->num_ctas = static_cast<int>(ctas);
    // Token-major caches ([.., token, head, D]: BNHD, paged NHD) interleave the heads' rows in
    // memory: there the CTAs of a pair take tiles round-robin, so all heads of a row sweep the
    // same addresses together; head-major caches give every CTA one contiguous slice.
    geo->schedule = geo->tok_dim == 2 ? kScheduleCyclic : kScheduleBlocked;
    // Who merges the split states of a pair: its first CTA, which looks until the states of the
    // others have landed - no arrival ticket, whose round trip would sit between the last CTA's
    // last tile and the merge (measured: paged config 3 31.9 -> 31.1 us, config 2 42.5 -> 42.1).
    // The first CTA may be waiting for CTAs that are still to be scheduled, so every CTA of the
    // grid must be able to be resident at once (one per SM); a larger grid, which only an
    // explicit CTA count can ask for, elects the last arriver by ticket instead.
    const char *force = std::getenv("STREAMATTN_B200_MERGER");  // "ticket": the other form, for A/B timing
    geo->first_merges = ctas <= (p.sm_count > 0 ? p.sm_count : 148);
    if (force != nullptr && std::strcmp(force, "ticket") == 0) geo->first_merges = 0;
    return true;
}

int check_common(const void *q, const void *k, const void *v, const void *out, const void *ws, int batch,
                 int q_heads, int kv_heads, int head_dim, int dtype, int out_mode, int num_ctas, int kernel_choice)
{
    if (!q || !k || !v || !out || !ws) return fail(SA_ERR_INVALID, "null tensor or workspace pointer");
    if (batch <= 0 || q_heads <= 0 || kv_heads <= 0) return fail(SA_ERR_INVALID, "batch/heads must be positive");
    if (q_heads % kv_heads) return fail(SA_ERR_INVALID, "query heads must be a multiple of KV heads");
    if (head_dim <= 0 || head_dim > 256) return fail(SA_ERR_INVALID, "head_dim must be in [1, 256]");
    if (dtype < SA_DTYPE_BF16 || dtype > SA_DTYPE_F32) return fail(SA_ERR_INVALID, "unknown dtype");
    if (out_mode != SA_OUT_FINAL && out_mode != SA_OUT_STATE) return fail(SA_ERR_INVALID, "unknown out_mode");
    if (num_ctas < 0) return fail(SA_ERR_INVALID, "num_ctas must be >= 0");
    const int base_choice = kernel_choice & ~SA_KERNEL_FLAG_DYNAMIC;
    if (base_choice < SA_KERNEL_AUTO || base_choice > SA_KERNEL_GENERIC)
        return fail(SA_ERR_INVALID, "unknown kernel_choice");
    if (static_cast<int64_t>(batch) * q_heads > 1 << 24) return fail(SA_ERR_UNSUPPORTED, "too many (row, head) pairs");
    return SA_OK;
}

// Finish a plan from a filled Problem: split the workspace, pick the kernel.
int finish_plan(sa_plan *plan, void *workspace, size_t workspace_bytes, int64_t max_vlen, int kernel_choice)
{
    Problem &p = plan->problem;
    g_workspace_too_small = false;
    p.wait_ns = g_default_wait_ns.load();
    p.sm_count = device_sm_count();
    if (p.sm_count <= 0 || cudaGetDevice(&plan->device) != cudaSuccess)
        return fail(SA_ERR_DEVICE, "no CUDA device is current");
    if (reinterpret_cast<uintptr_t>(workspace) % 16) return fail(SA_ERR_INVALID, "workspace must be 16-byte aligned");
    const size_t head = kStatusWords * 4 + counters_bytes(p.batch, p.q_heads);
    if (workspace_bytes < head) {
        g_workspace_too_small = true;
        return fail(SA_ERR_INVALID, "workspace too small");
    }
    p.ws.status = static_cast<int *>(workspace);
    p.ws.counters = p.ws.status + kStatusWords;
    p.ws.partials = reinterpret_cast<float *>(static_cast<char *>(workspace) + head);
    p.ws.partial_floats = (workspace_bytes - head) / 4;
    plan->max_vlen = max_vlen;

    const char *why = "";
    plan->use_stream = false;
    const bool dynamic = (kernel_choice & SA_KERNEL_FLAG_DYNAMIC) != 0;
    kernel_choice &= ~SA_KERNEL_FLAG_DYNAMIC;
    if (kernel_choice != SA_KERNEL_GENERIC) {
        plan->use_stream = build_stream_geometry(p, max_vlen, &plan->geo, &why);
        if (!plan->use_stream && kernel_choice == SA_KERNEL_STREAM)
            return fail(SA_ERR_UNSUPPORTED, "streaming kernel does not cover this call: %s", why);
        if (plan->use_stream && dynamic) plan->geo.schedule = kScheduleClaims;
    }
    size_t need;
    if (plan->use_stream) {
        need = stream_partial_floats(p.batch, p.q_heads, p.kv_heads * plan->geo.kv_split, p.head_dim, plan->geo.num_ctas);
    } else {
        plan->generic_splits = generic_splits(p, max_vlen);
        need = plan->generic_splits > 1
                   ? generic_partial_floats(p.batch, p.q_heads, p.head_dim, plan->generic_splits)
                   : 0;
    }
    if (need > p.ws.partial_floats) {
        g_workspace_too_small = true;
        return fail(SA_ERR_INVALID, "workspace too small: need %zu bytes, got %zu", head + need * 4, workspace_bytes);
    }
    return SA_OK;
}

int run_plan(const sa_plan *plan, cudaStream_t stream)
{
    if (plan->cp.world > 0) {
        // The step number travels as a launch argument: a captured launch would replay one step
        // number for ever, and ranks would take each other's old words for new ones.
        cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &capturing) == cudaSuccess && capturing != cudaStreamCaptureStatusNone)
            return fail(SA_ERR_UNSUPPORTED, "a fused context-parallel plan cannot be captured into a CUDA graph");
        plan->cp.step += 1;  // every rank advances in lock step, one per run
    }
    cudaError_t err = plan->use_stream ? launch_stream(plan->problem, plan->geo, plan->cp, stream)
                                       : launch_generic(plan->problem, plan->generic_splits, stream);
    if (err != cudaSuccess) return fail_cuda(err, "kernel launch failed");
    return SA_OK;
}

int fill_exact(sa_plan *plan, const void *q, const void *k, const void *v, void *out, void *workspace,
               size_t workspace_bytes, const void *seq_lens, int lens_dtype, int batch, int q_heads, int kv_heads,
               int head_dim, int64_t kv_len, int64_t q_sb, int64_t q_sh, int64_t kv_sb, int64_t kv_sn,
               int64_t kv_sh, int dtype, int out_mode, int num_ctas, int kernel_choice)
{
    int rc = check_common(q, k, v, out, workspace, batch, q_heads, kv_heads, head_dim, dtype, out_mode, num_ctas,
                          kernel_choice);
    if (rc) return rc;
    if (kv_len <= 0) return fail(SA_ERR_INVALID, "kv_len must be positive");
    if (lens_dtype != SA_INDEX_I32 && lens_dtype != SA_INDEX_I64) return fail(SA_ERR_INVALID, "unknown lens_dtype");
    std::memset(plan, 0, sizeof(*plan));
    Problem &p = plan->problem;
    p.q = q; p.k = k; p.v = v; p.out = out;
    p.dtype = dtype; p.out_mode = out_mode;
    p.batch = batch; p.q_heads = q_heads; p.kv_heads = kv_heads; p.head_dim = head_dim;
    p.q_sb = q_sb; p.q_sh = q_sh;
    p.seq.mode = kContig;
    p.seq.num_rows = -1;
    p.seq.kv_sb = kv_sb; p.seq.kv_sn = kv_sn; p.seq.kv_sh = kv_sh;
    p.seq.kv_len = kv_len;
    p.seq.seq_lens = seq_lens;
    p.seq.lens_i64 = lens_dtype == SA_INDEX_I64;
    p.num_ctas = num_ctas;
    return finish_plan(plan, workspace, workspace_bytes, kv_len, kernel_choice);
}

int fill_paged(sa_plan *plan, const void *q, const void *k_pages, const void *v_pages, const void *page_table,
               const void *seq_lens, void *out, void *workspace, size_t workspace_bytes, int32_t *trace, int batch,
               int q_heads, int kv_heads, int head_dim, int page_size, int max_pages, int64_t num_pages, int layout,
               int dtype, int table_dtype, int lens_dtype, int out_mode, int num_ctas, int kernel_choice)
{
    int rc = check_common(q, k_pages, v_pages, out, workspace, batch, q_heads, kv_heads, head_dim, dtype, out_mode,
                          num_ctas, kernel_choice);
    if (rc) return rc;
    if (!page_table || !seq_lens) return fail(SA_ERR_INVALID, "page_table and seq_lens are required");
    if (page_size <= 0 || max_pages <= 0 || num_pages <= 0)
        return fail(SA_ERR_INVALID, "paged cache dimensions must be positive");
    if (layout != SA_LAYOUT_NHD && layout != SA_LAYOUT_HND) return fail(SA_ERR_INVALID, "paged KV layout must be NHD or HND");
    if ((table_dtype != SA_INDEX_I32 && table_dtype != SA_INDEX_I64) ||
        (lens_dtype != SA_INDEX_I32 && lens_dtype != SA_INDEX_I64))
        return fail(SA_ERR_INVALID, "page_table / seq_lens must be int32 or int64");
    std::memset(plan, 0, sizeof(*plan));
    Problem &p = plan->problem;
    p.q = q; p.k = k_pages; p.v = v_pages; p.out = out;
    p.dtype = dtype; p.out_mode = out_mode;
    p.batch = batch; p.q_heads = q_heads; p.kv_heads = kv_heads; p.head_dim = head_dim;
    p.q_sb = static_cast<int64_t>(q_heads) * head_dim; p.q_sh = head_dim;
    p.seq.mode = kPaged;
    p.seq.num_rows = -1;
    p.seq.seq_lens = seq_lens;
    p.seq.lens_i64 = lens_dtype == SA_INDEX_I64;
    p.seq.page_table = page_table;
    p.seq.table_i64 = table_dtype == SA_INDEX_I64;
    p.seq.max_pages = max_pages;
    p.seq.page_size = page_size;
    p.seq.num_pages = num_pages;
    const int64_t D = head_dim;
    p.seq.pg_sp = static_cast<int64_t>(page_size) * kv_heads * D;
    if (layout == SA_LAYOUT_NHD) { p.seq.pg_st = kv_heads * D; p.seq.pg_sh = D; }
    else                         { p.seq.pg_st = D; p.seq.pg_sh = static_cast<int64_t>(page_size) * D; }
    p.trace = trace;
    p.num_ctas = num_ctas;
    return finish_plan(plan, workspace, workspace_bytes, static_cast<int64_t>(max_pages) * page_size, kernel_choice);
}

int fill_seed(sa_plan *plan, const void *q, const void *k, const void *v, void *out, void *workspace,
              size_t workspace_bytes, int batch, int q_heads, int kv_heads, int head_dim, int64_t kv_len,
              int64_t q_sb, int64_t q_sh, int64_t kv_sb, int64_t kv_sn, int64_t kv_sh, int dtype, int block_size,
              const int32_t *blocks_host, int num_blocks, int num_ctas, int kernel_choice)
{
    int rc = check_common(q, k, v, out, workspace, batch, q_heads, kv_heads, head_dim, dtype, SA_OUT_FINAL, num_ctas,
                          kernel_choice);
    if (rc) return rc;
    if (kv_len <= 0 || block_size <= 0) return fail(SA_ERR_INVALID, "kv_len and block_size must be positive");
    if (num_blocks < 0 || (num_blocks > 0 && !blocks_host)) return fail(SA_ERR_INVALID, "bad seed block list");
    std::vector<int32_t> blocks;
    for (int i = 0; i < num_blocks; ++i) {
        const int64_t blk = blocks_host[i];
        if (blk < 0 || blk * block_size >= kv_len) continue;  // out of range: dropped like the reference
        blocks.push_back(static_cast<int32_t>(blk));
    }
    std::sort(blocks.begin(), blocks.end());
    blocks.erase(std::unique(blocks.begin(), blocks.end()), blocks.end());
    if (blocks.empty()) return fail(SA_ERR_INVALID, "seed block list selects no token");
    if (blocks.size() > static_cast<size_t>(kMaxSeedBlocks))
        return fail(SA_ERR_UNSUPPORTED, "more than %d seed blocks", kMaxSeedBlocks);
    std::memset(plan, 0, sizeof(*plan));
    Problem &p = plan->problem;
    p.q = q; p.k = k; p.v = v; p.out = out;
    p.dtype = dtype; p.out_mode = SA_OUT_FINAL;
    p.batch = batch; p.q_heads = q_heads; p.kv_heads = kv_heads; p.head_dim = head_dim;
    p.q_sb = q_sb; p.q_sh = q_sh;
    p.seq.mode = kBlocks;
    p.seq.num_rows = -1;
    p.seq.kv_sb = kv_sb; p.seq.kv_sn = kv_sn; p.seq.kv_sh = kv_sh;
    p.seq.kv_len = kv_len;
    p.seq.block_size = block_size;
    p.seq.num_blocks = static_cast<int>(blocks.size());
    int64_t vlen = 0;
    for (size_t i = 0; i < blocks.size(); ++i) {
        p.seq.blocks[i] = blocks[i];
        vlen += std::min<int64_t>(block_size, kv_len - static_cast<int64_t>(blocks[i]) * block_size);
    }
    // Only the last (largest) block can be clipped by kv_len, so the valid tokens
    // are exactly the first `vlen` virtual tokens.
    p.seq.blocks_vlen = vlen;
    p.num_ctas = num_ctas;
    return finish_plan(plan, workspace, workspace_bytes, vlen, kernel_choice);
}


int fill_seed_device(sa_plan *plan, const void *q, const void *k, const void *v, void *out, void *workspace,
                     size_t workspace_bytes, int batch, int q_heads, int kv_heads, int head_dim, int64_t kv_len,
                     int64_t q_sb, int64_t q_sh, int64_t kv_sb, int64_t kv_sn, int64_t kv_sh, int dtype, int block_size,
                     const int32_t *blocks_dev, int blocks_per_pair, int includes_last_block, int num_ctas,
                     int kernel_choice)
{
    int rc = check_common(q, k, v, out, workspace, batch, q_heads, kv_heads, head_dim, dtype, SA_OUT_FINAL, num_ctas,
                          kernel_choice);
    if (rc) return rc;
    if (kv_len <= 0 || block_size <= 0) return fail(SA_ERR_INVALID, "kv_len and block_size must be positive");
    if (!blocks_dev || blocks_per_pair <= 0) return fail(SA_ERR_INVALID, "a device block list with at least one block per pair is required");
    const int64_t cache_blocks = (kv_len + block_size - 1) / block_size;
    if (blocks_per_pair > cache_blocks) return fail(SA_ERR_INVALID, "more seed blocks per pair than the cache has blocks");
    std::memset(plan, 0, sizeof(*plan));
    Problem &p = plan->problem;
    p.q = q; p.k = k; p.v = v; p.out = out;
    p.dtype = dtype; p.out_mode = SA_OUT_FINAL;
    p.batch = batch; p.q_heads = q_heads; p.kv_heads = kv_heads; p.head_dim = head_dim;
    p.q_sb = q_sb; p.q_sh = q_sh;
    p.seq.mode = kBlocks;
    p.seq.num_rows = -1;
    p.seq.kv_sb = kv_sb; p.seq.kv_sn = kv_sn; p.seq.kv_sh = kv_sh;
    p.seq.kv_len = kv_len;
    p.seq.block_size = block_size;
    p.seq.num_blocks = blocks_per_pair;
    p.seq.blocks_dev = blocks_dev;
    p.seq.blocks_kv_heads = kv_heads;
    // Lists are ascending, so only a pair's last entry can be the cache's (possibly short) last block.
    const int64_t clip = includes_last_block && kv_len % block_size ? block_size - kv_len % block_size : 0;
    p.seq.blocks_vlen = static_cast<int64_t>(blocks_per_pair) * block_size - clip;
    p.num_ctas = num_ctas;
    return finish_plan(plan, workspace, workspace_bytes, p.seq.blocks_vlen, kernel_choice);
}

}  // namespace
}  // namespace sa

using namespace sa;

namespace sa {
namespace {

// Checks shared by the two KV-append entry points; fills the parts of `a` that do not depend
// on the cache kind.
int fill_append(AppendParams *a, const void *k_new, const void *v_new, void *k_cache, void *v_cache,
                const void *positions, int pos_dtype, int num_positions, void *lens_out, const void *cos,
                const void *sin, int64_t rope_stride_b, const void *q_in, void *q_out, int q_heads,
                int64_t q_in_stride_b, int64_t q_in_stride_h, int64_t q_out_stride_b, int64_t q_out_stride_h,
                int batch, int kv_heads, int head_dim, int64_t new_stride_b, int64_t new_stride_h, int dtype,
                int *status)
{
    if (!k_new || !v_new || !k_cache || !v_cache || !positions)
        return fail(SA_ERR_INVALID, "null tensor pointer");
    if (batch <= 0 || kv_heads <= 0) return fail(SA_ERR_INVALID, "batch/heads must be positive");
    if (head_dim <= 0 || head_dim > 256) return fail(SA_ERR_INVALID, "head_dim must be in [1, 256]");
    if (dtype < SA_DTYPE_BF16 || dtype > SA_DTYPE_F32) return fail(SA_ERR_INVALID, "unknown dtype");
    if (pos_dtype != SA_INDEX_I32 && pos_dtype != SA_INDEX_I64) return fail(SA_ERR_INVALID, "positions must be int32 or int64");
    if (num_positions != 1 && num_positions != batch)
        return fail(SA_ERR_INVALID, "positions must hold one entry or one per batch row");
    if (lens_out == positions && num_positions == 1 && batch > 1)
        return fail(SA_ERR_INVALID, "lens_out may alias positions only when there is one position per row");
    if ((cos == nullptr) != (sin == nullptr)) return fail(SA_ERR_INVALID, "cos and sin must be given together");
    if (cos != nullptr && head_dim % 2) return fail(SA_ERR_INVALID, "rotary embedding needs an even head_dim");
    if ((q_in == nullptr) != (q_out == nullptr)) return fail(SA_ERR_INVALID, "q_in and q_out must be given together");
    if (q_in != nullptr && (q_heads <= 0 || q_heads % kv_heads))
        return fail(SA_ERR_INVALID, "query heads must be a positive multiple of KV heads");
    if (q_in != nullptr && q_in == q_out) return fail(SA_ERR_INVALID, "q_out must not alias q_in");
    std::memset(a, 0, sizeof(*a));
    a->k_new = k_new; a->v_new = v_new;
    a->new_sb = new_stride_b; a->new_sh = new_stride_h;
    a->k_cache = k_cache; a->v_cache = v_cache;
    a->positions = positions;
    a->pos_i64 = pos_dtype == SA_INDEX_I64;
    a->pos_shared = num_positions == 1;
    a->lens_out = lens_out;
    a->cos = cos; a->sin = sin; a->rope_sb = rope_stride_b;
    a->q_in = q_in; a->q_out = q_out; a->q_heads = q_heads;
    a->qi_sb = q_in_stride_b; a->qi_sh = q_in_stride_h; a->qo_sb = q_out_stride_b; a->qo_sh = q_out_stride_h;
    a->batch = batch; a->kv_heads = kv_heads; a->head_dim = head_dim;
    a->dtype = dtype;
    a->status = status;
    return SA_OK;
}

}  // namespace
}  // namespace sa

using namespace sa;

extern "C" {

int sa_version(void) { return 100; }

const char *sa_last_error(void) { return g_error; }

int sa_device_supported(int device)
{
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return major == 10 ? 1 : 0;
}

int sa_device_sm_count(int device)
{
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

size_t sa_workspace_bytes(int batch, int q_heads, int kv_heads, int head_dim, int num_ctas)
{
    if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0 || q_heads % kv_heads || num_ctas < 0) {
        fail(SA_ERR_INVALID, "sa_workspace_bytes: bad shape");
        return 0;
    }
    return workspace_bytes_impl(batch, q_heads, kv_heads, head_dim, num_ctas);
}

int sa_workspace_status(void *workspace, sa_stream_t stream)
{
    if (!workspace) return -SA_ERR_INVALID;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int word = 0;
    cudaError_t err = cudaMemcpyAsync(&word, workspace, sizeof(int), cudaMemcpyDeviceToHost, s);
    if (err == cudaSuccess) err = cudaStreamSynchronize(s);
    if (err == cudaSuccess && word != 0) err = cudaMemsetAsync(workspace, 0, sizeof(int), s);
    if (err != cudaSuccess) {
        fail_cuda(err, "sa_workspace_status");
        return -SA_ERR_CUDA;
    }
    return word;
}

int sa_exact_decode(const void *q, const void *k, const void *v, void *out, void *workspace, size_t workspace_bytes,
                    const void *seq_lens, int lens_dtype, int batch, int q_heads, int kv_heads, int head_dim,
                    int64_t kv_len, int64_t q_stride_b, int64_t q_stride_h, int64_t kv_stride_b,
                    int64_t kv_stride_n, int64_t kv_stride_h, int dtype, int out_mode, int num_ctas,
                    int kernel_choice, sa_stream_t stream)
{
    sa_plan plan;
    int rc = fill_exact(&plan, q, k, v, out, workspace, workspace_bytes, seq_lens, lens_dtype, batch, q_heads,
                        kv_heads, head_dim, kv_len, q_stride_b, q_stride_h, kv_stride_b, kv_stride_n, kv_stride_h,
                        dtype, out_mode, num_ctas, kernel_choice);
    if (rc) return rc;
    return run_plan(&plan, static_cast<cudaStream_t>(stream));
}

int sa_paged_decode(const void *q, const void *k_pages, const void *v_pages, const void *page_table,
                    const void *seq_lens, void *out, void *workspace, size_t workspace_bytes, int32_t *trace,
                    int batch, int q_heads, int kv_heads, int head_dim, int page_size, int max_pages_per_request,
                    int64_t num_pages, int layout, int dtype, int table_dtype, int lens_dtype, int out_mode,
                    int num_ctas, int kernel_choice, sa_stream_t stream)
{
    sa_plan plan;
    int rc = fill_paged(&plan, q, k_pages, v_pages, page_table, seq_lens, out, workspace, workspace_bytes, trace,
                        batch, q_heads, kv_heads, head_dim, page_size, max_pages_per_request, num_pages, layout,
                        dtype, table_dtype, lens_dtype, out_mode, num_ctas, kernel_choice);
    if (rc) return rc;
    return run_plan(&plan, static_cast<cudaStream_t>(stream));
}

int sa_seed_blocks(int64_t kv_len, int block_size, int sink_blocks, int recent_blocks, int middle_seed_blocks,
                   int block_order, int32_t *blocks_out, int capacity)
{
    if (kv_len <= 0 || block_size <= 0 || sink_blocks < 0 || recent_blocks < 0 || middle_seed_blocks < 0 ||
        block_order < SA_ORDER_SEQUENTIAL || block_order > SA_ORDER_SINK_RECENT_FIRST || !blocks_out) {
        fail(SA_ERR_INVALID, "sa_seed_blocks: bad argument");
        return -1;
    }
    const int64_t num_blocks = (kv_len + block_size - 1) / block_size;
    const int64_t recent_start = num_blocks - recent_blocks;
    int count = 0;
    auto push = [&](int64_t blk) -> bool {
        if (blk < 0 || blk >= num_blocks) return true;
        for (int i = 0; i < count; ++i)
            if (blocks_out[i] == blk) return true;
        if (count >= capacity) return false;
        blocks_out[count++] = static_cast<int32_t>(blk);
        return true;
    };
    bool ok = true;
    for (int64_t i = 0; ok && i < sink_blocks; ++i) ok = push(i);
    for (int64_t blk = recent_start; ok && blk < num_blocks; ++blk) ok = push(blk);
    for (int64_t i = 0; ok && i < middle_seed_blocks; ++i)
        ok = push(block_order == SA_ORDER_SEQUENTIAL ? sink_blocks + i : recent_start - 1 - i);
    if (!ok) {
        fail(SA_ERR_INVALID, "sa_seed_blocks: capacity too small");
        return -1;
    }
    return count;
}

int64_t sa_seed_token_indices(int64_t kv_len, int block_size, const int32_t *blocks, int num_blocks,
                              int64_t *tokens_out, int64_t capacity)
{
    if (kv_len <= 0 || block_size <= 0 || num_blocks < 0 || (num_blocks > 0 && !blocks) || !tokens_out) {
        fail(SA_ERR_INVALID, "sa_seed_token_indices: bad argument");
        return -1;
    }
    std::vector<int64_t> starts;
    for (int i = 0; i < num_blocks; ++i) {
        const int64_t start = static_cast<int64_t>(blocks[i]) * block_size;
        if (blocks[i] < 0 || start >= kv_len) continue;
        starts.push_back(start);
    }
    std::sort(starts.begin(), starts.end());
    starts.erase(std::unique(starts.begin(), starts.end()), starts.end());
    int64_t n = 0;
    for (int64_t start : starts) {
        const int64_t end = std::min<int64_t>(kv_len, start + block_size);
        for (int64_t t = start; t < end; ++t) {
            if (n >= capacity) {
                fail(SA_ERR_INVALID, "sa_seed_token_indices: capacity too small");
                return -1;
            }
            tokens_out[n++] = t;
        }
    }
    return n;
}

int sa_seed_decode_blocks(const void *q, const void *k, const void *v, void *out, void *workspace,
                          size_t workspace_bytes, int batch, int q_heads, int kv_heads, int head_dim, int64_t kv_len,
                          int64_t q_stride_b, int64_t q_stride_h, int64_t kv_stride_b, int64_t kv_stride_n,
                          int64_t kv_stride_h, int dtype, int block_size, const int32_t *blocks_host, int num_blocks,
                          int num_ctas, int kernel_choice, sa_stream_t stream)
{
    sa_plan plan;
    int rc = fill_seed(&plan, q, k, v, out, workspace, workspace_bytes, batch, q_heads, kv_heads, head_dim, kv_len,
                       q_stride_b, q_stride_h, kv_stride_b, kv_stride_n, kv_stride_h, dtype, block_size, blocks_host,
                       num_blocks, num_ctas, kernel_choice);
    if (rc) return rc;
    return run_plan(&plan, static_cast<cudaStream_t>(stream));
}

int sa_seed_decode(const void *q, const void *k, const void *v, void *out, void *workspace, size_t workspace_bytes,
                   int batch, int q_heads, int kv_heads, int head_dim, int64_t kv_len, int64_t q_stride_b,
                   int64_t q_stride_h, int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h, int dtype,
                   int block_size, int sink_blocks, int recent_blocks, int middle_seed_blocks, int block_order,
                   int num_ctas, int kernel_choice, sa_stream_t stream)
{
    int32_t blocks[SA_MAX_SEED_BLOCKS];
    const int n = sa_seed_blocks(kv_len, block_size, sink_blocks, recent_blocks, middle_seed_blocks, block_order,
                                 blocks, SA_MAX_SEED_BLOCKS);
    if (n < 0) return SA_ERR_INVALID;
    return sa_seed_decode_blocks(q, k, v, out, workspace, workspace_bytes, batch, q_heads, kv_heads, head_dim, kv_len,
                                 q_stride_b, q_stride_h, kv_stride_b, kv_stride_n, kv_stride_h, dtype, block_size,
                                 blocks, n, num_ctas, kernel_choice, stream);
}

sa_plan_t *sa_seed_plan_create_device(const void *q, const void *k, const void *v, void *out, void *workspace,
                                      size_t workspace_bytes, int batch, int q_heads, int kv_heads, int head_dim,
                                      int64_t kv_len, int64_t q_stride_b, int64_t q_stride_h, int64_t kv_stride_b,
                                      int64_t kv_stride_n, int64_t kv_stride_h, int dtype, int block_size,
                                      const int32_t *blocks_dev, int blocks_per_pair, int includes_last_block,
                                      int num_ctas, int kernel_choice)
{
    sa_plan *plan = new (std::nothrow) sa_plan;
    if (!plan) return nullptr;
    if (fill_seed_device(plan, q, k, v, out, workspace, workspace_bytes, batch, q_heads, kv_heads, head_dim, kv_len,
                         q_stride_b, q_stride_h, kv_stride_b, kv_stride_n, kv_stride_h, dtype, block_size, blocks_dev,
                         blocks_per_pair, includes_last_block, num_ctas, kernel_choice)) {
        delete plan;
        return nullptr;
    }
    return plan;
}

int sa_block_scores(const void *q, const void *k, float *scores, const void *seq_lens, int lens_dtype, int batch,
                    int q_heads, int kv_heads, int head_dim, int64_t kv_len, int64_t q_stride_b, int64_t q_stride_h,
                    int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h, int dtype, int block_size,
                    int selector, sa_stream_t stream)
{
    if (!q || !k || !scores) return fail(SA_ERR_INVALID, "sa_block_scores: null tensor pointer");
    if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads)
        return fail(SA_ERR_INVALID, "sa_block_scores: bad batch / head counts");
    if (kv_len <= 0 || block_size <= 0) return fail(SA_ERR_INVALID, "sa_block_scores: kv_len and block_size must be positive");
    if (dtype != SA_DTYPE_BF16 && dtype != SA_DTYPE_F16) return fail(SA_ERR_UNSUPPORTED, "sa_block_scores: dtype must be bf16 or fp16");
    if (selector != SA_SELECT_QK_BLOCK_MAX && selector != SA_SELECT_BLOCK_MEAN)
        return fail(SA_ERR_INVALID, "sa_block_scores: unknown selector");
    if (q_heads / kv_heads > 16) return fail(SA_ERR_UNSUPPORTED, "sa_block_scores: more than 16 query heads per KV head");
    if (head_dim <= 0 || head_dim > 256 || head_dim % 8 || kv_stride_n % 8 || kv_stride_h % 8 || kv_stride_b % 8 ||
        reinterpret_cast<uintptr_t>(k) % 16)
        return fail(SA_ERR_UNSUPPORTED, "sa_block_scores: head_dim and the KV strides must be multiples of 8 (16-byte rows)");
    if (lens_dtype != SA_INDEX_I32 && lens_dtype != SA_INDEX_I64) return fail(SA_ERR_INVALID, "unknown lens_dtype");
    if ((kv_len + block_size - 1) / block_size > (1 << 24)) return fail(SA_ERR_UNSUPPORTED, "sa_block_scores: too many blocks");
    const cudaError_t err = launch_block_scores(q, k, scores, seq_lens, lens_dtype == SA_INDEX_I64, batch, q_heads,
                                                kv_heads, head_dim, kv_len, q_stride_b, q_stride_h, kv_stride_b,
                                                kv_stride_n, kv_stride_h, dtype, block_size, selector,
                                                static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) return fail_cuda(err, "sa_block_scores");
    return SA_OK;
}

int sa_seed_list_length(int64_t kv_len, int block_size, int sink_blocks, int recent_blocks, int middle_seed_blocks)
{
    if (kv_len <= 0 || block_size <= 0 || sink_blocks < 0 || recent_blocks < 0 || middle_seed_blocks < 0) {
        fail(SA_ERR_INVALID, "sa_seed_list_length: bad argument");
        return -1;
    }
    const int64_t nb = (kv_len + block_size - 1) / block_size;
    const int64_t base = std::min<int64_t>(nb, std::min<int64_t>(sink_blocks, nb) + std::min<int64_t>(recent_blocks, nb));
    return static_cast<int>(std::min<int64_t>(nb, base + middle_seed_blocks));
}

int sa_select_seed_blocks(const float *scores, int32_t *blocks_out, int batch, int q_heads, int kv_heads,
                          int64_t kv_len, int block_size, int sink_blocks, int recent_blocks, int middle_seed_blocks,
                          int block_order, sa_stream_t stream)
{
    if (!scores || !blocks_out) return fail(SA_ERR_INVALID, "sa_select_seed_blocks: null tensor pointer");
    if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads)
        return fail(SA_ERR_INVALID, "sa_select_seed_blocks: bad batch / head counts");
    if (block_order < SA_ORDER_SEQUENTIAL || block_order > SA_ORDER_SINK_RECENT_FIRST)
        return fail(SA_ERR_INVALID, "sa_select_seed_blocks: unknown block_order");
    const int list_len = sa_seed_list_length(kv_len, block_size, sink_blocks, recent_blocks, middle_seed_blocks);
    if (list_len <= 0) return fail(SA_ERR_INVALID, "sa_select_seed_blocks: the policy selects no block");
    if (list_len > SA_MAX_SEED_BLOCKS) return fail(SA_ERR_UNSUPPORTED, "more than %d seed blocks", SA_MAX_SEED_BLOCKS);
    const int64_t nb = (kv_len + block_size - 1) / block_size;
    if (nb * 4 > 200 * 1024) return fail(SA_ERR_UNSUPPORTED, "sa_select_seed_blocks: more than 51200 blocks per row");
    const cudaError_t err = launch_select_blocks(scores, blocks_out, batch, q_heads, kv_heads, static_cast<int>(nb),
                                                 sink_blocks, recent_blocks, middle_seed_blocks, block_order, list_len,
                                                 static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) return fail_cuda(err, "sa_select_seed_blocks");
    return SA_OK;
}

int sa_merge_states(const float *states, int num_parts, int64_t rows, int head_dim, void *out, int out_dtype,
                    sa_stream_t stream)
{
    if (!states || !out || num_parts <= 0 || rows <= 0 || head_dim <= 0 || rows > (1ll << 31) - 1)
        return fail(SA_ERR_INVALID, "sa_merge_states: bad argument");
    if (out_dtype < SA_DTYPE_BF16 || out_dtype > SA_DTYPE_F32) return fail(SA_ERR_INVALID, "unknown out_dtype");
    cudaError_t err = launch_merge_states(states, num_parts, rows, head_dim, out, out_dtype,
                                          static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) return fail_cuda(err, "sa_merge_states");
    return SA_OK;
}

namespace {

struct FusedLayout {
    size_t gather_words_per_parity, total_bytes;
};

FusedLayout fused_layout(int world, int batch, int q_heads, int kv_heads, int head_dim)
{
    // gather[2][world][rows][D+2] of 64-bit (step << 32 | value) words; the data is its own flag.
    (void)kv_heads;
    FusedLayout l;
    l.gather_words_per_parity = static_cast<size_t>(world) * batch * q_heads * (head_dim + 2);
    l.total_bytes = (2 * l.gather_words_per_parity * 8 + 127) / 128 * 128 + 128;
    return l;
}

}  // namespace

size_t sa_cp_fused_bytes(int world_size, int batch, int q_heads, int kv_heads, int head_dim)
{
    if (world_size <= 0 || world_size > kCpFuseWorld || batch <= 0 || q_heads <= 0 || kv_heads <= 0 ||
        head_dim <= 0) {
        fail(SA_ERR_INVALID, "sa_cp_fused_bytes: bad argument (world_size must be in [1, %d])", kCpFuseWorld);
        return 0;
    }
    return fused_layout(world_size, batch, q_heads, kv_heads, head_dim).total_bytes;
}

sa_plan_t *sa_cp_fused_plan_create(const void *q, const void *k, const void *v, void *out, void *workspace,
                                   size_t workspace_bytes, int batch, int q_heads, int kv_heads, int head_dim,
                                   int64_t kv_len, int64_t q_stride_b, int64_t q_stride_h, int64_t kv_stride_b,
                                   int64_t kv_stride_n, int64_t kv_stride_h, int dtype, int num_ctas,
                                   const uint64_t *peer_buffers, int world_size, int rank)
{
    if (!peer_buffers || world_size <= 0 || world_size > kCpFuseWorld || rank < 0 || rank >= world_size) {
        fail(SA_ERR_INVALID, "sa_cp_fused_plan_create: world_size must be in [1, %d] and rank inside it", kCpFuseWorld);
        return nullptr;
    }
    for (int i = 0; i < world_size; ++i)
        if (peer_buffers[i] == 0 || peer_buffers[i] % 128) {
            fail(SA_ERR_INVALID, "sa_cp_fused_plan_create: peer buffer %d is null or not 128-byte aligned", i);
            return nullptr;
        }
    sa_plan *plan = new (std::nothrow) sa_plan;
    if (!plan) return nullptr;
    // The shard kernel runs in state mode; its state rows go to the ranks' buffers, not to `out`.
    if (fill_exact(plan, q, k, v, out, workspace, workspace_bytes, nullptr, SA_INDEX_I32, batch, q_heads, kv_heads,
                   head_dim, kv_len, q_stride_b, q_stride_h, kv_stride_b, kv_stride_n, kv_stride_h, dtype,
                   SA_OUT_STATE, num_ctas, SA_KERNEL_STREAM)) {
        delete plan;
        return nullptr;
    }
    if (reinterpret_cast<uintptr_t>(out) % 16) {
        fail(SA_ERR_INVALID, "sa_cp_fused_plan_create: output must be 16-byte aligned");
        delete plan;
        return nullptr;
    }
    const FusedLayout l = fused_layout(world_size, batch, q_heads, kv_heads, head_dim);
    plan->cp.world = world_size;
    plan->cp.rank = rank;
    plan->cp.step = 0;
    for (int i = 0; i < kCpMaxWorld; ++i) plan->cp.bases[i] = i < world_size ? peer_buffers[i] : 0;
    plan->cp.gather_words_per_parity = l.gather_words_per_parity;
    plan->cp.final_out = out;
    return plan;
}

size_t sa_cp_exchange_bytes(int world_size, int64_t rows, int head_dim)
{
    if (world_size <= 0 || world_size > SA_CP_MAX_WORLD || rows <= 0 || head_dim <= 0) {
        fail(SA_ERR_INVALID, "sa_cp_exchange_bytes: bad argument");
        return 0;
    }
    return exchange_bytes(world_size, rows, head_dim);
}

int sa_cp_exchange_merge(const float *local_state, const uint64_t *peer_buffers, int world_size, int rank,
                         uint32_t step, int64_t rows, int head_dim, void *out, int out_dtype, sa_stream_t stream)
{
    if (!local_state || !peer_buffers || !out || rows <= 0 || head_dim <= 0)
        return fail(SA_ERR_INVALID, "sa_cp_exchange_merge: bad argument");
    if (world_size <= 0 || world_size > SA_CP_MAX_WORLD || rank < 0 || rank >= world_size)
        return fail(SA_ERR_INVALID, "sa_cp_exchange_merge: world_size must be in [1, %d] and rank inside it",
                    SA_CP_MAX_WORLD);
    if (step == 0) return fail(SA_ERR_INVALID, "sa_cp_exchange_merge: step counts from 1");
    if (out_dtype < SA_DTYPE_BF16 || out_dtype > SA_DTYPE_F32) return fail(SA_ERR_INVALID, "unknown out_dtype");
    for (int i = 0; i < world_size; ++i)
        if (peer_buffers[i] == 0 || peer_buffers[i] % 128)
            return fail(SA_ERR_INVALID, "sa_cp_exchange_merge: peer buffer %d is null or not 128-byte aligned", i);
    cudaError_t err = launch_exchange_merge(local_state, peer_buffers, world_size, rank, step, rows, head_dim, out,
                                            out_dtype, g_default_wait_ns.load(), static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) return fail_cuda(err, "sa_cp_exchange_merge");
    return SA_OK;
}

int sa_cp_exchange_status(void *exchange_buffer, int world_size, int64_t rows, int head_dim, sa_stream_t stream)
{
    if (!exchange_buffer || world_size <= 0 || world_size > SA_CP_MAX_WORLD || rows <= 0 || head_dim <= 0)
        return -SA_ERR_INVALID;
    return sa_workspace_status(static_cast<char *>(exchange_buffer) + exchange_status_offset(world_size, rows, head_dim),
                               stream);
}

// ---------------------------------------------------------------------------
// Exact decode without any allocation: the scratch lives in this module's image.
// ---------------------------------------------------------------------------

// Split states + arrival counters + status word of sa_exact_decode_static.  A
// file-scope device array: every GPU that loads the library holds these bytes
// until the process exits.  In host code this name is only a stand-in for the
// symbol, never a device address; the address comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[SA_STATIC_SCRATCH_BYTES];

namespace {

// Device address of g_static_scratch on the current device, looked up once per
// device (with that device current) and remembered.
int static_scratch_address(void **out)
{
    static std::mutex mu;
    static void *address[64] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return fail_cuda(err, "sa_exact_decode_static: cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(SA_ERR_DEVICE, "sa_exact_decode_static: device index out of range");
    std::lock_guard<std::mutex> lock(mu);
    if (address[dev] == nullptr) {
        void *ptr = nullptr;
        err = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (err != cudaSuccess || ptr == nullptr)
            return fail_cuda(err, "sa_exact_decode_static: cudaGetSymbolAddress");
        address[dev] = ptr;
    }
    *out = address[dev];
    return SA_OK;
}

}  // namespace

int sa_exact_decode_static(const void *q, const void *k, const void *v, void *out, const void *seq_lens,
                           int lens_dtype, int batch, int q_heads, int kv_heads, int head_dim, int64_t kv_len,
                           int64_t q_stride_b, int64_t q_stride_h, int64_t kv_stride_b, int64_t kv_stride_n,
                           int64_t kv_stride_h, int dtype, int out_mode, int num_ctas, int kernel_choice,
                           sa_stream_t stream)
{
    void *scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if (rc) return rc;
    sa_plan plan;
    rc = fill_exact(&plan, q, k, v, out, scratch, SA_STATIC_SCRATCH_BYTES, seq_lens, lens_dtype, batch, q_heads,
                    kv_heads, head_dim, kv_len, q_stride_b, q_stride_h, kv_stride_b, kv_stride_n, kv_stride_h, dtype,
                    out_mode, num_ctas, kernel_choice);
    if (rc && g_workspace_too_small)
        return fail(SA_ERR_UNSUPPORTED,
                    "sa_exact_decode_static: this shape needs more than the %d bytes of built-in scratch; "
                    "use sa_exact_decode with a caller-provided workspace", SA_STATIC_SCRATCH_BYTES);
    if (rc) return rc;
    // The array keeps whatever the previous call left.  The arrival counters must start at
    // zero, so clear them on the caller's stream (one small stream operation the workspace
    // entry points do not need).  The status word in front of them is left alone: it collects
    // the bits of every call until sa_static_status() reads and clears it.
    cudaError_t err = cudaMemsetAsync(static_cast<char *>(scratch) + kStatusWords * 4, 0,
                                      counters_bytes(batch, q_heads), static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) return fail_cuda(err, "sa_exact_decode_static: clearing the arrival counters");
    return run_plan(&plan, static_cast<cudaStream_t>(stream));
}

int sa_static_status(sa_stream_t stream)
{
    void *scratch = nullptr;
    if (static_scratch_address(&scratch)) return -SA_ERR_DEVICE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int word = 0;
    cudaError_t err = cudaMemcpyAsync(&word, scratch, sizeof(int), cudaMemcpyDeviceToHost, s);
    if (err == cudaSuccess) err = cudaStreamSynchronize(s);
    // A call that gave up a wait may have left split states behind: bring the whole array back
    // to the all-zero state the kernels expect between calls.
    if (err == cudaSuccess && word != 0) err = cudaMemsetAsync(scratch, 0, SA_STATIC_SCRATCH_BYTES, s);
    if (err != cudaSuccess) {
        fail_cuda(err, "sa_static_status");
        return -SA_ERR_CUDA;
    }
    return word;
}

sa_plan_t *sa_exact_plan_create(const void *q, const void *k, const void *v, void *out, void *workspace,
                                size_t workspace_bytes, const void *seq_lens, int lens_dtype, int batch, int q_heads,
                                int kv_heads, int head_dim, int64_t kv_len, int64_t q_stride_b, int64_t q_stride_h,
                                int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h, int dtype,
                                int out_mode, int num_ctas, int kernel_choice)
{
    sa_plan *plan = new (std::nothrow) sa_plan;
    if (!plan) return nullptr;
    if (fill_exact(plan, q, k, v, out, workspace, workspace_bytes, seq_lens, lens_dtype, batch, q_heads, kv_heads,
                   head_dim, kv_len, q_stride_b, q_stride_h, kv_stride_b, kv_stride_n, kv_stride_h, dtype, out_mode,
                   num_ctas, kernel_choice)) {
        delete plan;
        return nullptr;
    }
    return plan;
}

sa_plan_t *sa_paged_plan_create(const void *q, const void *k_pages, const void *v_pages, const void *page_table,
                                const void *seq_lens, void *out, void *workspace, size_t workspace_bytes,
                                int32_t *trace, int batch, int q_heads, int kv_heads, int head_dim, int page_size,
                                int max_pages_per_request, int64_t num_pages, int layout, int dtype, int table_dtype,
                                int lens_dtype, int out_mode, int num_ctas, int kernel_choice)
{
    sa_plan *plan = new (std::nothrow) sa_plan;
    if (!plan) return nullptr;
    if (fill_paged(plan, q, k_pages, v_pages, page_table, seq_lens, out, workspace, workspace_bytes, trace, batch,
                   q_heads, kv_heads, head_dim, page_size, max_pages_per_request, num_pages, layout, dtype,
                   table_dtype, lens_dtype, out_mode, num_ctas, kernel_choice)) {
        delete plan;
        return nullptr;
    }
    return plan;
}

sa_plan_t *sa_seed_plan_create(const void *q, const void *k, const void *v, void *out, void *workspace,
                               size_t workspace_bytes, int batch, int q_heads, int kv_heads, int head_dim,
                               int64_t kv_len, int64_t q_stride_b, int64_t q_stride_h, int64_t kv_stride_b,
                               int64_t kv_stride_n, int64_t kv_stride_h, int dtype, int block_size,
                               const int32_t *blocks_host, int num_blocks, int num_ctas, int kernel_choice)
{
    sa_plan *plan = new (std::nothrow) sa_plan;
    if (!plan) return nullptr;
    if (fill_seed(plan, q, k, v, out, workspace, workspace_bytes, batch, q_heads, kv_heads, head_dim, kv_len,
                  q_stride_b, q_stride_h, kv_stride_b, kv_stride_n, kv_stride_h, dtype, block_size, blocks_host,
                  num_blocks, num_ctas, kernel_choice)) {
        delete plan;
        return nullptr;
    }
    return plan;
}

int sa_plan_run(const sa_plan_t *plan, sa_stream_t stream)
{
    if (!plan) return fail(SA_ERR_INVALID, "null plan");
    int current = -1;
    if (cudaGetDevice(&current) != cudaSuccess) return fail(SA_ERR_DEVICE, "no CUDA device is current");
    if (current == plan->device) return run_plan(plan, static_cast<cudaStream_t>(stream));
    // The plan's buffers live on another device than the caller's current one: switch for the launch.
    if (cudaSetDevice(plan->device) != cudaSuccess) return fail(SA_ERR_DEVICE, "cannot select the plan's device");
    const int rc = run_plan(plan, static_cast<cudaStream_t>(stream));
    cudaSetDevice(current);
    return rc;
}

int sa_plan_kernel(const sa_plan_t *plan) { return plan ? (plan->use_stream ? SA_KERNEL_STREAM : SA_KERNEL_GENERIC) : 0; }

int sa_plan_num_ctas(const sa_plan_t *plan)
{
    if (!plan) return 0;
    if (plan->use_stream) return plan->geo.num_ctas;
    return plan->generic_splits * plan->problem.batch * plan->problem.q_heads;
}

int sa_plan_launches(const sa_plan_t *plan)
{
    if (!plan) return 0;
    return plan->use_stream ? 1 : (plan->generic_splits > 1 ? 2 : 1);
}

void sa_plan_destroy(sa_plan_t *plan) { delete plan; }

int sa_set_wait_limit_ns(uint64_t limit_ns)
{
    if (limit_ns == 0) return fail(SA_ERR_INVALID, "sa_set_wait_limit_ns: the limit must be positive");
    g_default_wait_ns.store(limit_ns);
    return SA_OK;
}

int sa_plan_set_wait_limit_ns(sa_plan_t *plan, uint64_t limit_ns)
{
    if (!plan || limit_ns == 0) return fail(SA_ERR_INVALID, "sa_plan_set_wait_limit_ns: null plan or zero limit");
    plan->problem.wait_ns = limit_ns;
    return SA_OK;
}

int sa_plan_set_rows(sa_plan_t *plan, const void *rows, int index_dtype, int num_rows)
{
    if (!plan) return fail(SA_ERR_INVALID, "sa_plan_set_rows: null plan");
    if (plan->cp.world > 0)
        return fail(SA_ERR_UNSUPPORTED, "sa_plan_set_rows: a fused context-parallel plan computes every row");
    if (rows == nullptr) {  // back to every row
        plan->problem.seq.rows = nullptr;
        plan->problem.seq.num_rows = -1;
        return SA_OK;
    }
    if (num_rows < 0 || (index_dtype != SA_INDEX_I32 && index_dtype != SA_INDEX_I64))
        return fail(SA_ERR_INVALID, "sa_plan_set_rows: num_rows must be >= 0 and the indices int32 or int64");
    plan->problem.seq.rows = rows;
    plan->problem.seq.rows_i64 = index_dtype == SA_INDEX_I64;
    plan->problem.seq.num_rows = num_rows;
    return SA_OK;
}

int sa_o_proj(const void *x, const void *weight, const void *bias, void *out, int batch, int in_features,
              int out_features, int64_t x_stride_b, int dtype, int prefetch_weights, sa_stream_t stream)
{
    if (!x || !weight || !out) return fail(SA_ERR_INVALID, "sa_o_proj: null tensor pointer");
    if (batch <= 0 || in_features <= 0 || out_features <= 0)
        return fail(SA_ERR_INVALID, "sa_o_proj: batch and feature counts must be positive");
    if (dtype != SA_DTYPE_BF16 && dtype != SA_DTYPE_F16) return fail(SA_ERR_INVALID, "sa_o_proj: dtype must be bf16 or fp16");
    if (x_stride_b < in_features) return fail(SA_ERR_INVALID, "sa_o_proj: x_stride_b smaller than in_features");
    if (in_features % 8 || x_stride_b % 8 || reinterpret_cast<uintptr_t>(x) % 16 ||
        reinterpret_cast<uintptr_t>(weight) % 16)
        return fail(SA_ERR_UNSUPPORTED,
                    "sa_o_proj: in_features and x_stride_b must be multiples of 8 and x / weight 16-byte aligned");
    if (batch > 65535 * 16) return fail(SA_ERR_UNSUPPORTED, "sa_o_proj: batch too large");
    const cudaError_t err = launch_o_proj(x, weight, bias, out, batch, in_features, out_features, x_stride_b, dtype,
                                          prefetch_weights != 0, static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) return fail_cuda(err, "sa_o_proj");
    return SA_OK;
}

int sa_append_kv(const void *k_new, const void *v_new, void *k_cache, void *v_cache, const void *positions,
                 int pos_dtype, int num_positions, void *lens_out, const void *cos, const void *sin,
                 int64_t rope_stride_b, const void *q_in, void *q_out, int q_heads, int64_t q_in_stride_b,
                 int64_t q_in_stride_h, int64_t q_out_stride_b, int64_t q_out_stride_h, int batch, int kv_heads,
                 int head_dim, int64_t kv_len, int64_t new_stride_b, int64_t new_stride_h, int64_t kv_stride_b,
                 int64_t kv_stride_n, int64_t kv_stride_h, int dtype, int *status, sa_stream_t stream)
{
    AppendParams a;
    const int rc = fill_append(&a, k_new, v_new, k_cache, v_cache, positions, pos_dtype, num_positions, lens_out, cos,
                               sin, rope_stride_b, q_in, q_out, q_heads, q_in_stride_b, q_in_stride_h,
                               q_out_stride_b, q_out_stride_h, batch, kv_heads, head_dim, new_stride_b,
                               new_stride_h, dtype, status);
    if (rc) return rc;
    if (kv_len <= 0) return fail(SA_ERR_INVALID, "kv_len must be positive");
    if (kv_stride_n <= 0 || kv_stride_h < 0 || kv_stride_b < 0) return fail(SA_ERR_INVALID, "non-positive KV stride");
    a.paged = 0;
    a.kv_sb = kv_stride_b; a.kv_sn = kv_stride_n; a.kv_sh = kv_stride_h;
    a.capacity = kv_len;
    const cudaError_t err = launch_append(a, static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) return fail_cuda(err, "kernel launch failed");
    return SA_OK;
}

int sa_paged_append_kv(const void *k_new, const void *v_new, void *k_pages, void *v_pages, const void *page_table,
                       int table_dtype, const void *positions, int pos_dtype, int num_positions, void *lens_out,
                       const void *cos, const void *sin, int64_t rope_stride_b, const void *q_in, void *q_out,
                       int q_heads, int64_t q_in_stride_b, int64_t q_in_stride_h, int64_t q_out_stride_b,
                       int64_t q_out_stride_h, int batch, int kv_heads, int head_dim, int page_size, int max_pages,
                       int64_t num_pages, int layout, int64_t new_stride_b, int64_t new_stride_h, int dtype,
                       int *status, sa_stream_t stream)
{
    AppendParams a;
    const int rc = fill_append(&a, k_new, v_new, k_pages, v_pages, positions, pos_dtype, num_positions, lens_out, cos,
                               sin, rope_stride_b, q_in, q_out, q_heads, q_in_stride_b, q_in_stride_h,
                               q_out_stride_b, q_out_stride_h, batch, kv_heads, head_dim, new_stride_b,
                               new_stride_h, dtype, status);
    if (rc) return rc;
    if (!page_table) return fail(SA_ERR_INVALID, "page_table is required");
    if (table_dtype != SA_INDEX_I32 && table_dtype != SA_INDEX_I64)
        return fail(SA_ERR_INVALID, "page_table must be int32 or int64");
    if (page_size <= 0 || max_pages <= 0 || num_pages <= 0)
        return fail(SA_ERR_INVALID, "paged cache dimensions must be positive");
    if (layout != SA_LAYOUT_NHD && layout != SA_LAYOUT_HND) return fail(SA_ERR_INVALID, "paged KV layout must be NHD or HND");
    a.paged = 1;
    a.page_table = page_table;
    a.table_i64 = table_dtype == SA_INDEX_I64;
    a.max_pages = max_pages;
    a.page_size = page_size;
    a.num_pages = num_pages;
    a.capacity = static_cast<int64_t>(max_pages) * page_size;
    a.pg_sp = static_cast<int64_t>(page_size) * kv_heads * head_dim;
    if (layout == SA_LAYOUT_NHD) {
        a.pg_st = static_cast<int64_t>(kv_heads) * head_dim;
        a.pg_sh = head_dim;
    } else {
        a.pg_sh = static_cast<int64_t>(page_size) * head_dim;
        a.pg_st = head_dim;
    }
    const cudaError_t err = launch_append(a, static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) return fail_cuda(err, "kernel launch failed");
    return SA_OK;
}

}  // extern "C"
