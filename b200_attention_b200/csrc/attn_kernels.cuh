// Internal interface between the C-ABI layer and the sm_100a attention kernels.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>

namespace b200attn {

constexpr int kHeadDim = 128;      // only head_dim the kernels are written for
constexpr int kBlockM = 128;       // query rows per Q tile (= TMEM lanes)
constexpr int kBlockN = 128;       // keys per K/V tile
constexpr int kQTilesPerItem = 2;  // a work item is two Q tiles that share every K/V tile
constexpr int kItemRows = kBlockM * kQTilesPerItem;

// Device-side watchdog record, 8 ints, written only when something went wrong.
//   [0] code (0 = clean), [1] site id, [2] blockIdx.x, [3] warp, [4] barrier parity,
//   [5] work item, [6] K/V tile, [7] reserved
constexpr int kStatusInts = 8;

enum DeviceCode : int32_t {
  kDevOk = 0,
  kDevWaitTimeout = 1,    // a bounded mbarrier wait ran out
  kDevSmemMisaligned = 2  // dynamic shared memory base was not 1024-byte aligned
};

// Chaining calls over successive K/V shards (the sequence-parallel ring): every call
// but the last leaves a *partial* result, a normalised fp32 O plus its natural-log LSE,
// in caller-provided scratch; every call but the first merges the partial it finds
// there with its own result in the epilogue, in registers:
//   lse' = log(exp(lse_a) + exp(lse_b)),  O' = O_a * exp(lse_a - lse') + O_b * exp(lse_b - lse')
struct PartialState {
  float* o;        // [batch, heads, len_q, 128] fp32 contiguous, or nullptr
  float* lse;      // [batch, heads, len_q]      fp32 contiguous, or nullptr
  int32_t merge;   // 1: combine with the partial already stored in (o, lse)
  int32_t emit;    // 1: store the (merged) partial to (o, lse) instead of the bf16 output
};

constexpr int kSplitMaxRuns = 160;  // runs of a tile-stream split (one per CTA): B200 has 148 SMs

struct FwdParams {
  __nv_bfloat16* o;
  float* lse;  // [batch, heads, len_q] fp32 natural-log LSE, may be null
  int64_t o_stride_b, o_stride_h, o_stride_l;  // in elements; innermost stride is 1
  int32_t batch, heads, len_q, len_kv;
  int32_t m_blocks;     // ceil(len_q / kItemRows)
  int32_t kv_tiles;     // ceil(len_kv / kBlockN)
  int32_t total_items;  // batch * heads * m_blocks
  int32_t kv_group;     // query heads per K/V head (1 unless grouped-query attention)
  int32_t causal;       // 1: key j is visible to row i iff j <= i + causal_off
  int32_t causal_off;   // len_kv - len_q (>= 0): the mask is aligned to the bottom-right corner
  float scale_log2;     // softmax_scale * log2(e)
  int32_t* status;      // kStatusInts ints the kernel can write (device or mapped host memory)
  uint32_t wait_limit_ms;
  PartialState partial;
  // Tile-stream split (dense calls without a caller-side partial chain): when non-null, the
  // launch cuts the sequence of all (work item, K/V tile) pairs into one contiguous run per CTA
  // instead of dealing whole items round-robin; items cut by a run boundary leave fp32 partials
  // in `split_scratch` and the CTA whose piece finishes last merges them (see PieceWalk).
  float* split_scratch;    // 2 slots of kSplitSlotFloats per CTA
  int32_t* split_tickets;  // kSplitTicketsPerCta counters per CTA, zero between launches
  int32_t split_runs;      // how many CTAs (the first ones) share the last round's items
  // first unit of each of those CTAs' runs and, at [split_runs], the number of units; units number
  // the (item, K/V tile) pairs of the last round's items, item-major (see split_fill_cuts)
  int32_t split_cut[kSplitMaxRuns + 1];
  long long* trace;  // clock64 samples for timeline studies; used only by B200ATTN_TRACE builds
};

// Workspace of the tile-stream split, per CTA: two partial slots (a CTA has at most two cut
// pieces, its first and its last), each holding a normalised fp32 O [256 rows][128] and its LSE
// [256], and one arrival counter per (Q tile, epilogue warp).
constexpr int kSplitSlotFloats = kItemRows * (kHeadDim + 1);
constexpr int kSplitTicketsPerCta = kQTilesPerItem * 4;
constexpr int kSplitMinPieceTiles = 4;  // no piece of a cut item is shorter than this
constexpr size_t split_workspace_bytes(int ctas) {
  return size_t(ctas) * (2 * size_t(kSplitSlotFloats) * sizeof(float) + kSplitTicketsPerCta * sizeof(int32_t));
}

// Launchers. Both return cudaGetLastError() of the launch.
cudaError_t launch_fwd_ws(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                          const FwdParams& p, int sm_count, cudaStream_t stream);
// Grid and number of runs of a tile-stream split launch of `p` on `sm_count` SMs; grid == 0 if
// splitting does not apply to `p` or would not shorten the launch.
struct SplitPlan {
  int grid, runs;
};
SplitPlan split_plan(const FwdParams& p, int sm_count);
// Writes p.split_runs and p.split_cut for a plan with grid > 0.
void split_fill_cuts(FwdParams& p, int sm_count, const SplitPlan& plan);
cudaError_t launch_fwd_serial(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                              const FwdParams& p, cudaStream_t stream);

// One-time per-device function attribute set-up (max dynamic shared memory).
cudaError_t prepare_kernels();

}  // namespace b200attn
