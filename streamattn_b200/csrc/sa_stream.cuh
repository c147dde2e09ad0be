// Host-side description of one launch of the streaming (TMA + tensor core) kernel.
#pragma once

#include "sa_common.cuh"

namespace sa {

#ifndef SA_STREAM_WARPS
#define SA_STREAM_WARPS 8
#endif
constexpr int kStreamWarps = SA_STREAM_WARPS;    // each with its own ring of tiles
#ifndef SA_STREAM_STAGES
#define SA_STREAM_STAGES 1
#endif
constexpr int kStreamStages = SA_STREAM_STAGES;  // 16 KB K+V tiles in flight per warp

constexpr int kCpMaxWorld = SA_CP_MAX_WORLD;
constexpr int kCpFuseWorld = 8;  // ranks the fused decode+exchange launch supports (one NVSwitch box)

// How the CTAs that share one (row, kv head) pair divide its tiles (pairs with at least four
// CTAs each; otherwise the tile list is cut into equal slices regardless of pair boundaries).
enum StreamSchedule : int {
    kScheduleBlocked = 0,  // one contiguous slice per CTA
    kScheduleCyclic = 1,   // tiles dealt round-robin to the pair's warps
    kScheduleClaims = 2,   // first tiles round-robin, then one claim per tile from a device counter
};

// Context-parallel exchange fused into the decode launch: where the ranks' gather buffers are.
//   gather[2][world][rows][D+2] of 64-bit words (step << 32 | float bits); gather_words_per_parity counts words.
struct CpFuse {
    int world;  // 0 = not a context-parallel launch
    int rank;
    uint32_t step;
    uint64_t bases[kCpMaxWorld];
    unsigned long long gather_words_per_parity;
    void *final_out;  // [batch, q_heads, D] in the query dtype
};

struct StreamGeometry {
    CUtensorMap map_k;
    CUtensorMap map_v;
    int frag_tokens;     // rows of one TMA box
    int frags_per_tile;  // boxes per 8 KB tile
    int frags_per_unit;  // boxes per page / seed block
    int tok_dim;         // TMA coordinate carrying the token index (1 or 2)
    int uniform_tiles;   // tiles per row if all rows are equally long, else -1
    int num_ctas;
    int kv_split;        // groups of more than 16 query heads: virtual KV heads per physical one (else 1)
    int schedule;        // how the CTAs of one (row, kv head) pair share its tiles (kSchedule*)
    int first_merges;    // a pair's first CTA merges its split states (grids of at most one CTA per SM); else a ticket elects the last arriver
};

// Smallest s with group % s == 0 and group / s <= 16 (0 if there is none): a KV head with more
// than 16 query heads is served as s virtual KV heads that read the same K/V rows.
int stream_kv_split(int group);
int stream_tile_tokens(int head_dim);
int stream_stages(int head_dim, bool rows16);
size_t stream_smem_bytes(int head_dim, bool rows16, int stages, int batch);
constexpr size_t kStreamSmemLimit = 227 * 1024 - 64;
cudaError_t launch_stream(const Problem &p, const StreamGeometry &geo, const CpFuse &cp, cudaStream_t stream);

}  // namespace sa
