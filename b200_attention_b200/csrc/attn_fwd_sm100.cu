// Dense forward attention for sm_100a: O = softmax(Q K^T * scale) V, bf16 in, bf16 out, fp32
// accumulation, optional fp32 LSE, head_dim 128; optionally with a causal mask and with grouped
// K/V heads.
//
// Two kernels share the operand layout, descriptors and epilogue (attn_fwd_ws_short_kernel is the
// first one's body again, launched for items of few K/V tiles):
//
//   attn_fwd_ws_kernel      the production kernel (a template on the causal mask and on how
//                           work is dealt: whole 256-row work items round-robin, or with the
//                           last, partly filled round cut into equal runs of K/V tiles whose cut
//                           items are merged through a caller-provided workspace). Persistent
//                           CTAs (one per SM), 16 warps:
//                             warps 0-3   softmax for Q tile 0 (one query row per thread); also
//                                         the rare rebase of the O accumulator when a row's
//                                         reference maximum has to move
//                             warps 4-7   softmax for Q tile 1
//                             warps 8-11  epilogue: normalise, merge with a previous partial,
//                                         store O / LSE; partial stores, tickets and merges of
//                                         cut work items
//                             warp 12     issues every tcgen05.mma
//                             warp 13     issues every TMA load
//                             warps 14-15 only give their registers away
//                           Q tiles, and a ring of (V, K) tile pairs, sit in 128-byte-swizzled
//                           shared memory; S = Q K^T, the bf16 P that overwrites it, and both O
//                           accumulators live in TMEM (4 x 128 columns).
//
//   attn_fwd_serial_kernel  bring-up / cross-check kernel: one CTA per 128 query rows, every
//                           step serialised, exact rescale on every tile, all exponentials on
//                           the MUFU unit. Used by the tests as an independent second opinion.
//
// Operand layout in shared memory (identical for Q, K and V): a 128 x 128 bf16 tile is two TMA
// boxes of 64 columns x 128 rows, each row 128 bytes, 16-byte chunks XOR-swizzled by (row % 8).
//   Q, K as K-major operands:  row = M/N index, 8-row groups 1024 bytes apart (SBO); a K step
//                              of 16 elements is +32 bytes inside the row, steps 4..7 are in
//                              the second box (+16 KiB).
//   V as MN-major B operand:   row = K index (key), 8-key groups 1024 bytes apart (SBO), the
//                              two 64-wide halves of head_dim 16 KiB apart (LBO); a K step of
//                              16 keys is +2048 bytes.

#include "attn_kernels.cuh"
#include "ptx_sm100.cuh"

#include <cfloat>
#include <cmath>

namespace b200attn {

namespace {

using namespace ptx;

constexpr int kTileBytes = kBlockM * kHeadDim * 2;  // 32 KiB: one Q, K or V tile
constexpr int kBoxBytes = kTileBytes / 2;           // one 64-column TMA box
constexpr int kSwizzleGroupBytes = 1024;            // 8 rows x 128 bytes
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kNegInf = -INFINITY;

constexpr uint32_t kIdescQK = umma_idesc_bf16(kBlockM, kBlockN, /*b_mn_major=*/false);
constexpr uint32_t kIdescPV = umma_idesc_bf16(kBlockM, kHeadDim, /*b_mn_major=*/true);

// Timeline instrumentation, compiled in only for B200ATTN_TRACE builds: block 0 records clock64 at
// fixed points of its first work item, for tiles [kTraceTile0, kTraceTile0 + kTraceTiles).
// Layout: trace[((role * kTraceTiles + tile) * 2 + q) * 8 + event].
#ifdef B200ATTN_TRACE
#ifndef B200ATTN_TRACE_WARP
#define B200ATTN_TRACE_WARP 0
#endif
constexpr int kTraceTile0 = 8, kTraceTiles = 16;
#define B200ATTN_TRACE_EVENT(p, role, item, tile, q, ev)                                          \
  do {                                                                                            \
    if ((p).trace != nullptr && blockIdx.x == 0 && (item) == 0 && (tile) >= kTraceTile0 &&        \
        (tile) < kTraceTile0 + kTraceTiles)                                                       \
      (p).trace[(((role) * kTraceTiles + ((tile) - kTraceTile0)) * 2 + (q)) * 8 + (ev)] = clock64(); \
  } while (0)
// Same, but the clock is read only after `dep` (a float) has been computed.
#define B200ATTN_TRACE_EVENT_AFTER(p, role, item, tile, q, ev, dep)                               \
  do {                                                                                            \
    if ((p).trace != nullptr && blockIdx.x == 0 && (item) == 0 && (tile) >= kTraceTile0 &&        \
        (tile) < kTraceTile0 + kTraceTiles) {                                                     \
      long long t_;                                                                               \
      asm volatile("mov.u64 %0, %%clock64;" : "=l"(t_) : "f"(dep));                               \
      (p).trace[(((role) * kTraceTiles + ((tile) - kTraceTile0)) * 2 + (q)) * 8 + (ev)] = t_;     \
    }                                                                                             \
  } while (0)
#else
#define B200ATTN_TRACE_EVENT(p, role, item, tile, q, ev) do { } while (0)
#define B200ATTN_TRACE_EVENT_AFTER(p, role, item, tile, q, ev, dep) do { } while (0)
#endif

// Time budget instrumentation, compiled in only for B200ATTN_PROFILE builds: a role accumulates
// clock64 deltas per category in registers and block 0 writes the totals once at the end, so the
// measurement itself costs a clock read per boundary and nothing else.
#ifdef B200ATTN_PROFILE
#define PROF_DECL(n) uint32_t prof_acc[n] = {}; uint32_t prof_t = uint32_t(clock())
#define PROF_LAP(slot) do { const uint32_t now_ = uint32_t(clock()); prof_acc[slot] += now_ - prof_t; prof_t = now_; } while (0)
#define PROF_FLUSH(p, base, n) do { if ((p).trace != nullptr && blockIdx.x == 0) { for (int i_ = 0; i_ < (n); ++i_) (p).trace[(base) + i_] = prof_acc[i_]; } } while (0)
#else
#define PROF_DECL(n) do { } while (0)
#define PROF_LAP(slot) do { } while (0)
#define PROF_FLUSH(p, base, n) do { } while (0)
#endif

// ------------------------------------------------------------------------------------------
// Bounded waits
// ------------------------------------------------------------------------------------------
// Suspend-time hint of the polls in the slow path of a wait (see mbarrier.try_wait).
#ifndef B200ATTN_WAIT_HINT_NS
#define B200ATTN_WAIT_HINT_NS 1000
#endif

struct WaitCtx {
  uint32_t abort_addr;  // shared-memory word: non-zero once any thread of the CTA gave up
  int32_t* status;
  uint64_t limit_ns;
  int32_t item;
  int32_t tile;

  __device__ __forceinline__ bool aborted() const {
    uint32_t v;
    asm volatile("ld.volatile.shared::cta.u32 %0, [%1];\n" : "=r"(v) : "r"(abort_addr));
    return v != 0;
  }

  __device__ __forceinline__ void raise(int code, int site, uint32_t parity) const {
    asm volatile("st.volatile.shared::cta.u32 [%0], %1;\n" ::"r"(abort_addr), "r"(1u) : "memory");
    if (status != nullptr && atomicCAS(status, 0, code) == 0) {
      status[1] = site;
      status[2] = static_cast<int32_t>(blockIdx.x);
      status[3] = static_cast<int32_t>(threadIdx.x >> 5);
      status[4] = static_cast<int32_t>(parity);
      status[5] = item;
      status[6] = tile;
      __threadfence_system();
    }
  }

  __device__ __forceinline__ bool wait_slow(uint32_t bar, uint32_t parity, int site) const {
    const uint64_t t0 = global_timer_ns();
    for (uint32_t n = 1;; ++n) {
      if (mbar_try_wait(bar, parity, B200ATTN_WAIT_HINT_NS)) return true;
      if ((n & 7u) == 0) {
        if (aborted()) return false;
        if (global_timer_ns() - t0 > limit_ns) {
          raise(kDevWaitTimeout, site, parity);
          return false;
        }
      }
    }
  }

  // For roles run by a single thread.
  __device__ __forceinline__ bool wait(uint32_t bar, uint32_t parity, int site) const {
    if (mbar_try_wait(bar, parity, 0)) return true;
    return wait_slow(bar, parity, site);
  }

  // For the MMA and TMA roles, which whole warps run with uniform control flow.
  __device__ __forceinline__ bool wait_issue(uint32_t bar, uint32_t parity, int site) const {
    return wait_warp(bar, parity, site);
  }

  // For roles run by whole warps: every lane returns the same answer, so the warp stays
  // converged for the .sync.aligned TMEM instructions that follow.
  __device__ __forceinline__ bool wait_warp(uint32_t bar, uint32_t parity, int site) const {
    bool ok = mbar_try_wait(bar, parity, 0);
    if (__all_sync(0xffffffffu, ok)) return true;
    if (!ok) ok = wait_slow(bar, parity, site);
    return __all_sync(0xffffffffu, ok);
  }
};

// ------------------------------------------------------------------------------------------
// MMA issue helpers (called by one thread)
// ------------------------------------------------------------------------------------------
// (No warp-level synchronisation in these helpers: the serial kernel calls them from one thread.)
// S[128 x 128] = Q_tile * K_tile^T, eight K=16 steps over head_dim. Called by a whole warp with
// uniform operands (so descriptors live in uniform registers); the lane with lead != 0 issues the
// eight MMAs inside one branch. Measured at B4 H16 L8192: whole-warp roles 1311 TFLOPS, the
// same roles run by a single lane 1080.
__device__ __forceinline__ void issue_qk(uint32_t lead, uint32_t s_tmem, uint32_t q_smem,
                                         uint32_t k_smem) {
  constexpr uint32_t hi = umma_desc_hi_sw128(kSwizzleGroupBytes);
  const uint32_t a0 = umma_desc_lo(q_smem, 0);
  const uint32_t b0 = umma_desc_lo(k_smem, 0);
  if (lead) {
#pragma unroll
    for (int kk = 0; kk < kHeadDim / 16; ++kk) {
      const uint32_t off = uint32_t(((kk >> 2) * kBoxBytes + (kk & 3) * 32) >> 4);
      umma_ss(s_tmem, a0 + off, hi, b0 + off, hi, kIdescQK, kk > 0 ? 1u : 0u);
    }
  }
}
// O[128 x 128] (+)= P[128 x 128 keys] * V_tile, eight K = 16 steps over the keys. P is bf16
// pairs in TMEM, 8 columns per K step starting at p_tmem.
__device__ __forceinline__ void issue_pv(uint32_t lead, uint32_t o_tmem, uint32_t p_tmem,
                                         uint32_t v_smem, bool accumulate) {
  constexpr uint32_t hi = umma_desc_hi_sw128(kSwizzleGroupBytes);
  const uint32_t b0 = umma_desc_lo(v_smem, kBoxBytes);
  if (lead) {
#pragma unroll
    for (int kk = 0; kk < kBlockN / 16; ++kk) {
      const uint32_t off = uint32_t((kk * 16 * 128) >> 4);
      umma_ts(o_tmem, p_tmem + kk * 8, b0 + off, hi, kIdescPV, (kk > 0 || accumulate) ? 1u : 0u);
    }
  }
}

// ------------------------------------------------------------------------------------------
// Epilogue shared by both kernels: the calling thread owns one query row whose un-normalised
// accumulator sits in TMEM lane `lane_of_row`, columns o_tmem .. o_tmem+127.
// `after_last_ld` runs once, right after the final TMEM read has landed in registers.
// ------------------------------------------------------------------------------------------
struct RowOut {
  bool valid;            // row < len_q
  __nv_bfloat16* o_row;  // bf16 destination row (128 contiguous elements)
  float* part_row;       // fp32 partial row, or nullptr
  float w_cur;           // weight on this call's accumulator (includes 1 / rowsum)
  float w_prev;          // weight on the stored partial (0 if none)
  bool emit_partial;
};

__device__ __forceinline__ RowOut make_row_out(const FwdParams& p, int b, int h, int row, float m,
                                               float l) {
  RowOut r;
  r.valid = row < p.len_q;
  r.emit_partial = p.partial.emit != 0;
  const int64_t flat = (int64_t(b) * p.heads + h) * p.len_q + row;
  r.o_row = p.o + int64_t(b) * p.o_stride_b + int64_t(h) * p.o_stride_h +
            int64_t(row) * p.o_stride_l;
  r.part_row = (p.partial.o != nullptr) ? p.partial.o + flat * kHeadDim : nullptr;
  const float inv_l = 1.0f / l;
  float lse = (m + log2f(l)) * kLn2;
  r.w_cur = inv_l;
  r.w_prev = 0.0f;
  if (r.valid) {
    if (p.partial.merge != 0) {
      const float lse_prev = p.partial.lse[flat];
      const float top = fmaxf(lse_prev, lse);
      const float lse_new = top + logf(expf(lse_prev - top) + expf(lse - top));
      r.w_prev = expf(lse_prev - lse_new);
      r.w_cur = expf(lse - lse_new) * inv_l;
      lse = lse_new;
    }
    if (r.emit_partial) {
      p.partial.lse[flat] = lse;
    } else if (p.lse != nullptr) {
      p.lse[flat] = lse;
    }
  }
  return r;
}

template <class AfterLastLd>
__device__ __forceinline__ void store_row(const RowOut& r, uint32_t o_tmem_row,
                                          AfterLastLd after_last_ld) {
  constexpr int kChunk = 16;  // columns per TMEM read: keeps the epilogue inside 64 registers
#pragma unroll 1
  for (int c = 0; c < kHeadDim / kChunk; ++c) {
    uint32_t acc[kChunk];
    tmem_ld16(o_tmem_row + c * kChunk, acc);
    tmem_wait_ld();
    if (c == kHeadDim / kChunk - 1) after_last_ld();
    if (!r.valid) continue;
    float v[kChunk];
#pragma unroll
    for (int j = 0; j < kChunk; ++j) v[j] = __uint_as_float(acc[j]) * r.w_cur;
    if (r.w_prev != 0.0f) {
      const float4* prev = reinterpret_cast<const float4*>(r.part_row + c * kChunk);
#pragma unroll
      for (int j = 0; j < kChunk / 4; ++j) {
        const float4 t = prev[j];
        v[4 * j + 0] = fmaf(t.x, r.w_prev, v[4 * j + 0]);
        v[4 * j + 1] = fmaf(t.y, r.w_prev, v[4 * j + 1]);
        v[4 * j + 2] = fmaf(t.z, r.w_prev, v[4 * j + 2]);
        v[4 * j + 3] = fmaf(t.w, r.w_prev, v[4 * j + 3]);
      }
    }
    if (r.emit_partial) {
      float4* dst = reinterpret_cast<float4*>(r.part_row + c * kChunk);
#pragma unroll
      for (int j = 0; j < kChunk / 4; ++j)
        dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
      uint4* dst = reinterpret_cast<uint4*>(r.o_row + c * kChunk);
#pragma unroll
      for (int j = 0; j < kChunk / 8; ++j) {
        uint4 w;
        w.x = pack_bf16x2(v[8 * j + 0], v[8 * j + 1]);
        w.y = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
        w.z = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]);
        w.w = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
        dst[j] = w;
      }
    }
  }
}

// Keys at or beyond `valid` (0 < valid < 128) do not exist: push their scores to -inf.
__device__ __forceinline__ void mask_tail(uint32_t (&s)[4][32], int valid) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (c * 32 + j >= valid) s[c][j] = __float_as_uint(kNegInf);
    }
  }
}

__device__ __forceinline__ float row_max(const uint32_t (&s)[4][32]) {
  float m0 = kNegInf, m1 = kNegInf, m2 = kNegInf, m3 = kNegInf;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      m0 = max3(m0, __uint_as_float(s[c][j + 0]), __uint_as_float(s[c][j + 1]));
      m1 = max3(m1, __uint_as_float(s[c][j + 2]), __uint_as_float(s[c][j + 3]));
      m2 = max3(m2, __uint_as_float(s[c][j + 4]), __uint_as_float(s[c][j + 5]));
      m3 = max3(m3, __uint_as_float(s[c][j + 6]), __uint_as_float(s[c][j + 7]));
    }
  }
  return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// ==========================================================================================
// Warp-specialised persistent kernel
// ==========================================================================================
// A row keeps its reference maximum m until some score exceeds m by this many log2 units.
// With bf16 probabilities and fp32 sums nothing overflows or loses relative precision until the
// excess nears 2^100, so the bound can be generous; 32 makes a rebase a once-in-a-blue-moon event
// on real data while leaving 2^(127-32-20) of headroom for row sums over a million keys.
#ifndef B200ATTN_REBASE_LOG2
#define B200ATTN_REBASE_LOG2 32.0f
#endif

constexpr int kPairSlots = 2;                 // ring of (V, K) pairs
constexpr int kPairBytes = 2 * kTileBytes;    // V tile, then K tile
constexpr int kWsThreads = 512;
constexpr int kRegsSoftmax = 192;
constexpr int kRegsEpilogue = 64;
constexpr int kRegsOther = 64;

enum WsBarrier : int {
  kBarQFull = 0,    // +q   TMA -> MMA       Q tile q landed
  kBarQEmpty = 2,   // +q   MMA -> TMA       last QK of the item that reads Q tile q finished
  kBarSFull = 4,    // +q   MMA -> softmax   S_q holds the scores of the next tile
  kBarPReady = 6,   // +q   softmax (4 warps) -> MMA: P_q stored (and O_q rebased if needed)
  kBarSpare = 8,    // +q   (unused)
  kBarPvDone = 10,  // +q   MMA -> epilogue: final PV of the item finished
  kBarFin = 12,     // +q   softmax (4 warps) -> epilogue: final (max, sum) published
  kBarFinFree = 14, // +q   epilogue (4 warps) -> softmax: final (max, sum) consumed
  kBarOFree = 16,   // +q   epilogue (4 warps) -> MMA: O_q read out, the next item may overwrite it
  kBarDrain = 18,   //      MMA -> MMA       used only when leaving early
  kBarPairFull = 20,   // +slot  TMA -> MMA   the pair's V and K tiles landed
  kBarPairEmpty = 22,  // +slot  MMA -> TMA   PV and QK that read the pair finished
  kNumWsBarriers = 24
};

struct Piece {
  int item, t0, t1;  // K/V tiles [t0, t1) of work item `item`
};
constexpr int kMaxRunPieces = 4;  // a run is shorter than one item plus a snap: two pieces, four slots

struct alignas(16) WsAux {
  uint64_t bar[kNumWsBarriers];
  float row_max[kQTilesPerItem][kBlockM];
  float row_sum[kQTilesPerItem][kBlockM];
  uint32_t tmem_base;
  uint32_t abort_flag;
  // tile-stream split: this CTA's pieces of the last round, worked out once by thread 0
  int32_t run_pieces;
  int32_t whole_items;  // items [0, whole_items) are dealt round-robin as whole items
  Piece run_piece[kMaxRunPieces];
};

constexpr int kWsSmemBytes = kQTilesPerItem * kTileBytes + kPairSlots * kPairBytes + int(sizeof(WsAux));

struct ItemCoord {
  int b, h, row0;
};

// Work items are numbered (batch, head)-major, so consecutive items share K/V in L2. With a causal
// mask items differ in length (2 .. 2 * m_blocks tiles). Their numbers then mean something else:
// heads are taken in groups (the K/V of a group fit in L2, or enough CTAs work on each head at a
// time to share its tiles there), and inside a group the items are numbered by falling length,
// query block index slowest and head fastest. CausalWalk deals these numbers to the CTAs.
// K/V heads per group: as many as keep the group's K and V within 64 MiB, but at least 16 (with
// 148 CTAs on 16 heads, nine CTAs stream each head's tiles at about the same time and share them
// in L2 even where the group as a whole does not fit).
#ifndef B200ATTN_CAUSAL_GROUP
#define B200ATTN_CAUSAL_GROUP 16
#endif
__device__ __forceinline__ int causal_group_heads(const FwdParams& p) {
  const int fit = (64 << 20) / (2 * kHeadDim * 2) / p.len_kv;  // K and V rows of 256 bytes each
  // whole sets of query heads that share a K/V head
  return max(B200ATTN_CAUSAL_GROUP, fit) * p.kv_group;
}
template <bool kCausal>
__device__ __forceinline__ ItemCoord decode_item(const FwdParams& p, int item) {
  ItemCoord c;
  int bh, mb;
  if (kCausal) {
    const int group_heads = causal_group_heads(p);
    const int per_group = group_heads * p.m_blocks;
    const int group = item / per_group;
    const int idx = item - group * per_group;
    const int heads_here = min(group_heads, p.batch * p.heads - group * group_heads);
    const int mb_rev = idx / heads_here;
    bh = group * group_heads + (idx - mb_rev * heads_here);
    mb = p.m_blocks - 1 - mb_rev;
  } else {
    bh = item / p.m_blocks;
    mb = item - bh * p.m_blocks;
  }
  c.row0 = mb * kItemRows;
  c.b = bh / p.heads;
  c.h = bh - c.b * p.heads;
  return c;
}

// K/V tiles an item visits: all of them, or with a causal mask (key j is visible to row i iff
// j <= i + causal_off, causal_off = len_kv - len_q >= 0) those up to its last row's diagonal.
// Per Q tile q of the item: its last row decides (a Q tile past len_q counts as one row, it
// computes rows nobody stores). The second Q tile visits as many tiles as the first or one more.
template <bool kCausal>
__device__ __forceinline__ int q_tile_tiles(const FwdParams& p, int row0, int q) {
  if (!kCausal) return p.kv_tiles;
  const int first_row = row0 + q * kBlockM;
  const int last_row = min(first_row + kBlockM - 1, max(p.len_q - 1, first_row));
  return min(p.kv_tiles, (last_row + p.causal_off) / kBlockN + 1);
}
// The K/V stream of the item: what its second (longer) Q tile visits.
template <bool kCausal>
__device__ __forceinline__ int item_tiles(const FwdParams& p, int row0) {
  return q_tile_tiles<kCausal>(p, row0, kQTilesPerItem - 1);
}

// ---- work distribution ----------------------------------------------------------------------
// A piece is K/V tiles [t0, t1) of one work item. Without splitting (kSplit == false) a piece is a
// whole item and CTA c takes items c, c + grid, c + 2 * grid, ... With splitting, the full rounds
// are dealt the same way (all CTAs then stream the K/V of the same few heads at the same time,
// which is what keeps K/V in L2), and only the items of the last, partly filled round are treated
// differently (and taken first, see PieceWalk::take): the sequence of their (item, tile) pairs,
// item-major, is cut into one contiguous run per CTA of near-equal length, so every CTA gets the
// same amount of tensor work whatever items % grid is. A CTA's run is a (possibly cut) first item,
// whole items, and a (possibly cut) last item. The host chooses the cuts (split_fill_cuts) such
// that no piece is shorter than kSplitMinPieceTiles and hands them over in the parameters. Every
// role of a CTA walks the same pieces in the same order.
__device__ __forceinline__ int split_first_item(const FwdParams& p, int grid) {
  return (p.total_items / grid) * grid;  // items before this one belong to full rounds
}
// First unit of CTA c's run; CTAs past the last run get the number of units (an empty run).
__device__ __forceinline__ int split_cut(const FwdParams& p, int c) {
  return p.split_cut[c < p.split_runs ? c : p.split_runs];
}
// The CTA whose run holds unit u (runs that lie inside an item are never empty).
__device__ __forceinline__ int split_owner(const FwdParams& p, int u) {
  const int runs = p.split_runs;
  int c = int(static_cast<long long>(u) * runs / p.split_cut[runs]);
  while (c + 1 < runs && p.split_cut[c + 1] <= u) ++c;
  while (c > 0 && p.split_cut[c] > u) --c;
  return c;
}

// Hands out a CTA's pieces one by one. Without splitting that is the plain round-robin walk over
// whole items, with nothing but the item number live between two pieces.
template <bool kSplit>
struct PieceWalk;

template <>
struct PieceWalk<false> {
  int item;
  __device__ __forceinline__ PieceWalk(const FwdParams&, const WsAux*) : item(int(blockIdx.x)) {}
  __device__ __forceinline__ bool take(const FwdParams& p, Piece& out) {
    if (item >= p.total_items) return false;
    out.item = item;
    out.t0 = 0;
    out.t1 = p.kv_tiles;
    item += int(gridDim.x);
    return true;
  }
};

// With splitting: the CTA's run through the last round's items comes first (its pieces were put
// into shared memory at start-up) and the whole items of the full rounds after it: the merge of a
// cut item (done by the epilogue warps of whichever CTA finishes its piece last) then overlaps
// that CTA's remaining whole items instead of standing at the end of the launch. Between two
// pieces only a counter is live, which matters to the warps that run on 64 registers.
template <>
struct PieceWalk<true> {
  const WsAux* aux;
  int k;
  __device__ __forceinline__ PieceWalk(const FwdParams&, const WsAux* a) : aux(a), k(0) {}
  __device__ __forceinline__ bool take(const FwdParams& p, Piece& out) {
    const int n = aux->run_pieces;
    if (k < n) {
      out = aux->run_piece[k];
    } else {
      const int item = int(blockIdx.x) + (k - n) * int(gridDim.x);
      if (item >= aux->whole_items) return false;
      out.item = item;
      out.t0 = 0;
      out.t1 = p.kv_tiles;
    }
    ++k;
    return true;
  }
};

// The same walk worked out from the launch parameters alone (the cuts sit in the constant bank, so
// every value here is uniform across the warp as far as the compiler can see, which a value read
// from shared memory is not): for the roles whose tile loop is the hot one.
struct ParamPieceWalk {
  int u, k;  // next unit of the run; whole items taken so far
  __device__ __forceinline__ ParamPieceWalk(const FwdParams& p, const WsAux*)
      : u(split_cut(p, int(blockIdx.x))), k(0) {}
  __device__ __forceinline__ bool take(const FwdParams& p, Piece& out) {
    const int grid = int(gridDim.x);
    const int first = split_first_item(p, grid);
    const int u_end = split_cut(p, int(blockIdx.x) + 1);
    if (u < u_end) {
      const int j = u / p.kv_tiles;
      out.item = first + j;
      out.t0 = u - j * p.kv_tiles;
      out.t1 = min(p.kv_tiles, out.t0 + (u_end - u));
      u += out.t1 - out.t0;
      return true;
    }
    const int item = int(blockIdx.x) + k * grid;
    if (item >= first) return false;
    out.item = item;
    out.t0 = 0;
    out.t1 = p.kv_tiles;
    ++k;
    return true;
  }
};

// With a causal mask: the groups of heads one after the other; a group's items (numbered by
// falling length, see decode_item) are dealt in rounds of one item per CTA, back and forth: in
// every other round the CTAs take theirs in reverse order, and every other group takes the CTAs
// themselves in reverse order, so whoever drew long items draws short ones next and the sums even
// out (busiest CTA 1.6 % above the mean at B4 H16 L8192 on 148 CTAs; 11 % when every group is
// simply dealt longest first).
struct CausalWalk {
  int g, r;  // head group, round inside the group
  __device__ __forceinline__ CausalWalk(const FwdParams&, const WsAux*) : g(0), r(0) {}
  __device__ __forceinline__ bool take(const FwdParams& p, Piece& out) {
    const int grid = int(gridDim.x);
    const int nbh = p.batch * p.heads;
    const int group_heads = causal_group_heads(p);
    while (g * group_heads < nbh) {
      const int n = min(group_heads, nbh - g * group_heads) * p.m_blocks;  // items of the group
      const int base = r * grid;
      if (base < n) {
        const int in_round = min(grid, n - base);
        const int c = (g & 1) ? grid - 1 - int(blockIdx.x) : int(blockIdx.x);
        if (c < in_round) {
          out.item = g * group_heads * p.m_blocks + base + ((r & 1) ? in_round - 1 - c : c);
          out.t0 = 0;
          out.t1 = p.kv_tiles;
          ++r;
          return true;
        }
      }
      ++g;
      r = 0;
    }
    return false;
  }
};

template <bool kCausal, bool kSplit>
struct WalkOf {
  using type = PieceWalk<kSplit>;
  using hot = PieceWalk<kSplit>;
};
template <>
struct WalkOf<true, false> {
  using type = CausalWalk;
  using hot = CausalWalk;
};
template <>
struct WalkOf<false, true> {
  using type = PieceWalk<true>;  // the epilogue also looks the run's pieces up for the merges
  using hot = ParamPieceWalk;
};

// Thread 0, before the roles start: this CTA's run through the last round, as pieces.
__device__ __forceinline__ void plan_run(const FwdParams& p, WsAux* aux) {
  const int grid = int(gridDim.x);
  const int whole_items = split_first_item(p, grid);
  int u = split_cut(p, int(blockIdx.x));
  const int u_end = split_cut(p, int(blockIdx.x) + 1);
  int n = 0;
  while (u < u_end && n < kMaxRunPieces) {
    const int k = u / p.kv_tiles;
    Piece pc;
    pc.item = whole_items + k;
    pc.t0 = u - k * p.kv_tiles;
    const int left = u_end - u;
    pc.t1 = (left < p.kv_tiles - pc.t0) ? pc.t0 + left : p.kv_tiles;
    aux->run_piece[n++] = pc;
    u += pc.t1 - pc.t0;
  }
  aux->run_pieces = n;
  aux->whole_items = whole_items;
}

// ---- TMA producer -------------------------------------------------------------------------
__device__ __forceinline__ void load_tile(uint32_t lead, uint32_t dst, const CUtensorMap* map,
                                          int row, int h, int b, uint32_t bar) {
  mbar_arrive_expect_tx_lead(lead, bar, kTileBytes);
  tma_load_4d_lead(lead, dst, map, 0, row, h, b, bar);
  tma_load_4d_lead(lead, dst + kBoxBytes, map, 64, row, h, b, bar);
}

template <bool kCausal, bool kSplit>
__device__ void ws_load_role(const FwdParams& p, const WsAux* aux, const CUtensorMap* tq,
                             const CUtensorMap* tk, const CUtensorMap* tv, uint32_t smem_q,
                             uint32_t smem_kv, uint32_t bar0, uint32_t lead, WaitCtx& w) {
  // Run by the whole warp with uniform control flow; `lead` marks the one lane that issues.
  //
  // K/V travel in pairs: pair j holds V of tile j-1 and K of tile j (tiles numbered through all
  // of this CTA's items), because that is what the MMA warp consumes together: PV of tile j-1
  // and then QK of tile j. One "full" and one "empty" barrier phase per pair halves the
  // barrier work of the MMA warp against one phase per tile. The first pair has no V, the last
  // one no K.
  uint32_t slot = 0, empty_parity = 1;  // parity 1 passes on a fresh barrier
  uint32_t q_empty_parity = 1;
  // For the early-exit path: which "full" barriers were armed, and with which parity last.
  uint32_t armed = 0, armed_parity = 0;
  uint32_t q_full_parity = 0;
  bool ok = true;

  auto bar = [&](int i) { return bar0 + 8u * uint32_t(i); };
  auto push_pair = [&](bool has_v, int v_row, const ItemCoord& vc, bool has_k, int k_row,
                       const ItemCoord& kc, int site) -> bool {
    if (!w.wait_issue(bar(kBarPairEmpty + slot), empty_parity, site)) return false;
    const uint32_t full_parity = empty_parity ^ 1u;
    armed |= 1u << slot;
    armed_parity = (armed_parity & ~(1u << slot)) | (full_parity << slot);
    const uint32_t full = bar(kBarPairFull + slot);
    const uint32_t dst = smem_kv + slot * kPairBytes;
    mbar_arrive_expect_tx_lead(lead, full, (has_v ? kTileBytes : 0) + (has_k ? kTileBytes : 0));
    if (has_v) {
      tma_load_4d_lead(lead, dst, tv, 0, v_row, vc.h, vc.b, full);
      tma_load_4d_lead(lead, dst + kBoxBytes, tv, 64, v_row, vc.h, vc.b, full);
    }
    if (has_k) {
      tma_load_4d_lead(lead, dst + kTileBytes, tk, 0, k_row, kc.h, kc.b, full);
      tma_load_4d_lead(lead, dst + kTileBytes + kBoxBytes, tk, 64, k_row, kc.h, kc.b, full);
    }
    slot ^= 1u;
    if (slot == 0) empty_parity ^= 1u;
    return true;
  };

  bool first = true;
  typename WalkOf<kCausal, kSplit>::hot pw(p, aux);
  Piece pc;
  while (ok && pw.take(p, pc)) {
    const int item = pc.item;
    const ItemCoord c = decode_item<kCausal>(p, item);
    // tiles [tb, tb + T) of the item's K/V stream
    const int tb = kSplit ? pc.t0 : 0;
    const int T = kSplit ? pc.t1 - pc.t0 : item_tiles<kCausal>(p, c.row0);
    // K/V coordinates: grouped-query attention maps kv_group query heads onto one K/V head
    ItemCoord kvc = c;
    kvc.h = c.h / p.kv_group;
    w.item = item;
    w.tile = 0;
    if (first) {
      ok = push_pair(false, 0, kvc, true, tb * kBlockN, kvc, 110);  // the first K tile travels alone
      first = false;
      if (!ok) break;
    }
    for (int q = 0; ok && q < kQTilesPerItem; ++q) {
      ok = w.wait_issue(bar(kBarQEmpty + q), q_empty_parity, 100 + q);
      if (!ok) break;
      armed |= 1u << (kPairSlots + q);
      armed_parity = (armed_parity & ~(1u << (kPairSlots + q))) | (q_full_parity << (kPairSlots + q));
      load_tile(lead, smem_q + q * kTileBytes, tq, c.row0 + q * kBlockM, c.h, c.b,
                bar(kBarQFull + q));
    }
    q_empty_parity ^= 1u;
    q_full_parity ^= 1u;
    for (int i = 0; ok && i < T; ++i) {
      w.tile = i;
      if (i + 1 < T) {
        ok = push_pair(true, (tb + i) * kBlockN, kvc, true, (tb + i + 1) * kBlockN, kvc, 111);
      } else {
        // the last V of this piece shares its pair with the first K of the CTA's next piece, if any
        typename WalkOf<kCausal, kSplit>::hot ahead = pw;
        Piece np;
        const bool has_next_piece = ahead.take(p, np);
        ItemCoord next_kvc = kvc;
        if (has_next_piece) {
          next_kvc = decode_item<kCausal>(p, np.item);
          next_kvc.h /= p.kv_group;
        }
        ok = push_pair(true, (tb + i) * kBlockN, kvc, has_next_piece,
                       (kSplit && has_next_piece ? np.t0 : 0) * kBlockN, next_kvc, 112);
      }
    }
  }

  if (!ok || w.aborted()) {
    // Leaving early: wait (bounded) for every copy still in flight, so no TMA write lands in
    // shared memory after the CTA is gone.
    for (int s = 0; s < kPairSlots + kQTilesPerItem; ++s) {
      if (!((armed >> s) & 1u)) continue;
      const uint32_t b =
          (s < kPairSlots) ? bar(kBarPairFull + s) : bar(kBarQFull + (s - kPairSlots));
      const uint64_t t0 = global_timer_ns();
      while (!mbar_try_wait(b, (armed_parity >> s) & 1u, 1000)) {
        if (global_timer_ns() - t0 > w.limit_ns) break;
      }
    }
  }
}

// ---- MMA issuer ---------------------------------------------------------------------------
// Causal form of the MMA issuer (below is the dense one, which it follows step by step). The two
// Q tiles of an item walk the same K/V stream, but the first one stops a tile earlier when the
// stream's last tile lies wholly behind its diagonal: it then takes no part in that tile (no
// scores, no softmax, no PV), and its accumulator is handed to the epilogue a tile earlier.
__device__ void ws_mma_role_causal(const FwdParams& p, uint32_t smem_q, uint32_t smem_kv,
                                   uint32_t bar0, uint32_t tmem_base, uint32_t lead, WaitCtx& w) {
  auto bar = [&](int i) { return bar0 + 8u * uint32_t(i); };
  uint32_t slot = 0, full_parity = 0;  // the (V, K) pair to wait for next: see ws_load_role
  uint32_t q_full_parity = 0;
  uint32_t p_parity[kQTilesPerItem] = {0, 0};  // one phase per tile the Q tile takes part in
  uint32_t o_free_parity = 1;  // passes on the fresh barrier: both accumulators start out free
  bool ok = true;
  bool k_ready = false;

  CausalWalk pw(p, nullptr);
  Piece pc;
  while (ok && pw.take(p, pc)) {
    const int item = pc.item;
    const int row0 = decode_item<true>(p, item).row0;
    int Tq[kQTilesPerItem];
#pragma unroll
    for (int q = 0; q < kQTilesPerItem; ++q) Tq[q] = q_tile_tiles<true>(p, row0, q);
    const int T = Tq[kQTilesPerItem - 1];
    w.item = item;
    w.tile = 0;
    // ---- tile 0 scores for both Q tiles
    if (!k_ready) {
      if (!(ok = w.wait_issue(bar(kBarPairFull + slot), full_parity, 200))) break;
      slot ^= 1u;
      if (slot == 0) full_parity ^= 1u;
      k_ready = true;
    }
    {
      const uint32_t k_smem = smem_kv + (slot ^ 1u) * kPairBytes + kTileBytes;
#pragma unroll
      for (int q = 0; q < kQTilesPerItem; ++q) {
        if (!(ok = w.wait_issue(bar(kBarQFull + q), q_full_parity, 201 + q))) break;
        tc_fence_after_sync();
        issue_qk(lead, tmem_base + q * kBlockN, smem_q + q * kTileBytes, k_smem);
        umma_commit_lead(lead, bar(kBarSFull + q));
        if (Tq[q] == 1) umma_commit_lead(lead, bar(kBarQEmpty + q));
      }
    }
    if (!ok) break;
    // also covers the PV of the previous item that read the V half of this pair
    umma_commit_lead(lead, bar(kBarPairEmpty + (slot ^ 1u)));
    q_full_parity ^= 1u;

    for (int i = 0; ok && i < T; ++i) {
      w.tile = i;
      // V_i and K_{i+1} (or K_0 of this CTA's next item) in one phase
      if (!(ok = w.wait_issue(bar(kBarPairFull + slot), full_parity, 210))) break;
      const uint32_t v_smem = smem_kv + slot * kPairBytes;
      const uint32_t k_smem = v_smem + kTileBytes;
      const uint32_t pair_empty = bar(kBarPairEmpty + slot);
      slot ^= 1u;
      if (slot == 0) full_parity ^= 1u;
#pragma unroll
      for (int q = 0; q < kQTilesPerItem; ++q) {
        if (i < Tq[q]) {
          const uint32_t s_tmem = tmem_base + q * kBlockN;
          const uint32_t o_tmem = tmem_base + kQTilesPerItem * kBlockN + q * kHeadDim;
          if (i == 0) {
            // the previous item's epilogue must have read O_q out before it is overwritten
            if (!(ok = w.wait_issue(bar(kBarOFree + q), o_free_parity, 240 + q))) break;
          }
          if (!(ok = w.wait_issue(bar(kBarPReady + q), p_parity[q], 220 + q))) break;
          tc_fence_after_sync();
          issue_pv(lead, o_tmem, s_tmem, v_smem, /*accumulate=*/i > 0);
          p_parity[q] ^= 1u;
          if (i + 1 < Tq[q]) {
            issue_qk(lead, s_tmem, smem_q + q * kTileBytes, k_smem);
            umma_commit_lead(lead, bar(kBarSFull + q));
            if (i + 2 == Tq[q]) umma_commit_lead(lead, bar(kBarQEmpty + q));
          } else {
            umma_commit_lead(lead, bar(kBarPvDone + q));
          }
        }
        // the pair is free once the longer Q tile is through with it (K_{i+1} only if there is one)
        if (q == kQTilesPerItem - 1 && i + 1 < T) umma_commit_lead(lead, pair_empty);
      }
    }
    o_free_parity ^= 1u;
  }

  if (!ok || w.aborted()) {
    // Leaving early: make sure nothing this warp issued is still running before TMEM goes.
    umma_commit_lead(lead, bar(kBarDrain));
    const uint64_t t0 = global_timer_ns();
    while (!mbar_try_wait(bar(kBarDrain), 0, 1000)) {
      if (global_timer_ns() - t0 > w.limit_ns) break;
    }
  }
}

template <bool kCausal, bool kSplit>
__device__ void ws_mma_role(const FwdParams& p, const WsAux* aux, uint32_t smem_q, uint32_t smem_kv,
                            uint32_t bar0, uint32_t tmem_base, uint32_t lead, WaitCtx& w) {
  if (kCausal) {
    ws_mma_role_causal(p, smem_q, smem_kv, bar0, tmem_base, lead, w);
    return;
  }
  // Run by the whole warp with uniform control flow; `lead` marks the one lane that issues.
  auto bar = [&](int i) { return bar0 + 8u * uint32_t(i); };
  // K/V arrive in pairs (V of one tile with K of the next): see ws_load_role.
  uint32_t slot = 0, full_parity = 0;  // the pair to wait for next
  uint32_t q_full_parity = 0;
  uint32_t p_parity = 0;       // kBarPReady: both Q tiles see one phase per K/V tile
  uint32_t o_free_parity = 1;  // passes on the fresh barrier: both accumulators start out free
  bool ok = true;
  // The pair in use is always the one waited for last, slot ^ 1. After the first item, K_0 of
  // an item has already arrived with the last V of the item before.
  bool k_ready = false;

  PROF_DECL(8);  // 0 other, 1 wait pair, 3 wait P (+O_FREE), 4 issue PV, 5 issue QK, 6 commits

  typename WalkOf<kCausal, kSplit>::hot pw(p, aux);
  Piece pc;
  while (ok && pw.take(p, pc)) {
    const int item = pc.item;
    const int T = kSplit ? pc.t1 - pc.t0 : p.kv_tiles;
    w.item = item;
    w.tile = 0;
    // ---- first scores of the piece for both Q tiles
    if (!k_ready) {
      if (!(ok = w.wait_issue(bar(kBarPairFull + slot), full_parity, 200))) break;
      slot ^= 1u;
      if (slot == 0) full_parity ^= 1u;
      k_ready = true;
    }
    {
      const uint32_t k_smem = smem_kv + (slot ^ 1u) * kPairBytes + kTileBytes;
#pragma unroll
    for (int q = 0; q < kQTilesPerItem; ++q) {
      if (!(ok = w.wait_issue(bar(kBarQFull + q), q_full_parity, 201 + q))) break;
      tc_fence_after_sync();
      issue_qk(lead, tmem_base + q * kBlockN, smem_q + q * kTileBytes, k_smem);
      umma_commit_lead(lead, bar(kBarSFull + q));
      if (T == 1) umma_commit_lead(lead, bar(kBarQEmpty + q));
    }
    }
    if (!ok) break;
    // also covers the PV of the previous item that read the V half of this pair
    umma_commit_lead(lead, bar(kBarPairEmpty + (slot ^ 1u)));
    q_full_parity ^= 1u;

    for (int i = 0; ok && i < T; ++i) {
      w.tile = i;
      PROF_LAP(0);
      // V_i and K_{i+1} (or K_0 of this CTA's next item) in one phase
      if (!(ok = w.wait_issue(bar(kBarPairFull + slot), full_parity, 210))) break;
      PROF_LAP(1);
      const uint32_t v_smem = smem_kv + slot * kPairBytes;
      const uint32_t k_smem = v_smem + kTileBytes;
      const uint32_t pair_empty = bar(kBarPairEmpty + slot);
      slot ^= 1u;
      if (slot == 0) full_parity ^= 1u;
      const bool has_next = (i + 1 < T);
#pragma unroll
      for (int q = 0; q < kQTilesPerItem; ++q) {
        const uint32_t s_tmem = tmem_base + q * kBlockN;
        const uint32_t o_tmem = tmem_base + kQTilesPerItem * kBlockN + q * kHeadDim;
        PROF_LAP(0);
        if (lead) B200ATTN_TRACE_EVENT(p, 2, item, i, q, 0);
        if (i == 0) {
          // the previous item's epilogue must have read O_q out before it is overwritten
          if (!(ok = w.wait_issue(bar(kBarOFree + q), o_free_parity, 240 + q))) break;
        }
        if (!(ok = w.wait_issue(bar(kBarPReady + q), p_parity, 220 + q))) break;
        tc_fence_after_sync();
        PROF_LAP(3);
        if (lead) B200ATTN_TRACE_EVENT(p, 2, item, i, q, 1);
        issue_pv(lead, o_tmem, s_tmem, v_smem, /*accumulate=*/i > 0);
        PROF_LAP(4);
        if (lead) B200ATTN_TRACE_EVENT(p, 2, item, i, q, 2);
        if (!has_next) {
          umma_commit_lead(lead, bar(kBarPvDone + q));
        } else {
          if (lead) B200ATTN_TRACE_EVENT(p, 2, item, i, q, 3);
          PROF_LAP(0);
          issue_qk(lead, s_tmem, smem_q + q * kTileBytes, k_smem);
          PROF_LAP(5);
          if (lead) B200ATTN_TRACE_EVENT(p, 2, item, i, q, 4);
          umma_commit_lead(lead, bar(kBarSFull + q));
          if (i + 2 == T) umma_commit_lead(lead, bar(kBarQEmpty + q));
          if (q == kQTilesPerItem - 1) umma_commit_lead(lead, pair_empty);
        }
        PROF_LAP(6);
        if (lead) B200ATTN_TRACE_EVENT(p, 2, item, i, q, 5);
      }
      p_parity ^= 1u;
    }
    o_free_parity ^= 1u;
  }
  PROF_LAP(0);
  if (lead) PROF_FLUSH(p, 0, 8);

  if (!ok || w.aborted()) {
    // Leaving early: make sure nothing this warp issued is still running before TMEM goes.
    umma_commit_lead(lead, bar(kBarDrain));
    const uint64_t t0 = global_timer_ns();
    while (!mbar_try_wait(bar(kBarDrain), 0, 1000)) {
      if (global_timer_ns() - t0 > w.limit_ns) break;
    }
  }
}

// ---- softmax: one query row per thread ---------------------------------------------------
// 2^(s * c - m) for one 32-column chunk: 16 packed bf16 pairs out, row-sum pairs accumulated.
__device__ __forceinline__ void exp_chunk(const uint32_t (&s)[32], f2 scale2, f2 neg_m2,
                                          uint32_t (&packed)[16], f2& sum_a, f2& sum_b) {
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const f2 x = f2_fma(f2_make(__uint_as_float(s[2 * j]), __uint_as_float(s[2 * j + 1])), scale2,
                        neg_m2);
    float x0, x1;
    f2_split(x, x0, x1);
    const float e0 = ex2_approx(x0), e1 = ex2_approx(x1);
    const f2 e = f2_make(e0, e1);
    if (j & 1) sum_b = f2_add(sum_b, e); else sum_a = f2_add(sum_a, e);
    packed[j] = pack_bf16x2(e0, e1);
  }
}

__device__ __forceinline__ float f2_hsum(f2 a, f2 b) {
  float lo, hi;
  f2_split(f2_add(a, b), lo, hi);
  return lo + hi;
}

// Per K/V tile a thread turns its row of 128 scores into bf16 probabilities relative to the
// row's reference maximum m and adds them to the running sum l.
//
// Tiles after the first do not start with a row-maximum pass. The tile is exponentiated
// speculatively against the current m; the speculation holds if the row's sum of the tile stays
// below 2^kRebase (then no single probability reached 2^kRebase). Otherwise, and always on the
// first tile, the warp takes the exact path: fetch the scores again (S is still intact in TMEM,
// nothing has been stored over it yet), take the true maximum, move m, multiply l and the row's
// O accumulator in TMEM by 2^(m_old - m_new) (O is stable here: the scores of this tile exist, so
// the previous PV has finished, and the next PV has not been released yet), and redo the tile.
// P is stored and P_READY signalled only after the decision, so there is never anything to
// retract. All exponentials run on the MUFU unit and P is handed over in one piece: handing the
// first columns over early, an FMA-pipe polynomial for part of the exponentials, and storing P
// chunk by chunk as it is produced each measured slower in this kernel.
template <bool kCausal, bool kSplit>
__device__ void ws_softmax_role(const FwdParams& p, WsAux* aux, uint32_t bar0, uint32_t tmem_base,
                                int q, int warp_in_group, int lane, WaitCtx& w) {
  auto bar = [&](int i) { return bar0 + 8u * uint32_t(i); };
  constexpr float kRebase = B200ATTN_REBASE_LOG2;
  const float sum_limit = exp2f(kRebase);
  const uint32_t lane_field = uint32_t(warp_in_group * 32) << 16;
  const uint32_t s_tmem = tmem_base + q * kBlockN + lane_field;
  const uint32_t p_tmem = s_tmem;  // bf16 P overwrites S columns 0..63
  const uint32_t o_tmem = tmem_base + kQTilesPerItem * kBlockN + q * kHeadDim + lane_field;
  const int r = warp_in_group * 32 + lane;
  const float scale_log2 = p.scale_log2;
  const f2 scale2 = f2_splat(scale_log2);
  const int last_tile = p.kv_tiles - 1;
  const int tail_valid = p.len_kv - last_tile * kBlockN;  // keys in the last tile, 1..128
#ifdef B200ATTN_TRACE
  const bool tr = (warp_in_group == B200ATTN_TRACE_WARP && lane == 0);
#else
  const bool tr = false;
#endif
  uint32_t s_parity = 0;
  uint32_t fin_free_parity = 1;  // passes on the fresh barrier: nothing to consume yet
  PROF_DECL(8);  // 0 other, 1 wait S, 2 TMEM load, 3 exponentials + check, 4 store + signal

  typename WalkOf<kCausal, kSplit>::hot pw(p, aux);
  Piece pc;
  while (pw.take(p, pc)) {
    const int item = pc.item;
    w.item = item;
    w.tile = 0;
    // The epilogue warps must have consumed the previous item's final (max, sum) before this
    // group publishes the next pair: it protects the two shared-memory slots and keeps kBarFin
    // from completing twice before its waiters looked (parity waits would alias) when an item
    // has a single K/V tile. It costs nothing: the scores of the next item cannot exist before
    // the previous item's last PV has finished, which is what the epilogue waits for.
    if (!w.wait_warp(bar(kBarFinFree + q), fin_free_parity, 310 + q)) return;
    fin_free_parity ^= 1u;
    float m = kNegInf;  // reference maximum, log2 units
    float l = 0.0f;     // running sum of 2^(s - m)
    // causal: this row sees keys 0 .. row + causal_off; its Q tile's first row sees the fewest
    const int row0 = kCausal ? decode_item<true>(p, item).row0 : 0;
    // this piece's tiles are tiles [tb, tb + T) of the item (a piece starts its own partial result)
    const int tb = kSplit ? pc.t0 : 0;
    const int T = kSplit ? pc.t1 - pc.t0 : q_tile_tiles<kCausal>(p, row0, q);
    const int ragged_i = last_tile - tb;  // the piece's tile that holds the ragged end of the keys, if any
    const int tile_limit = row0 + q * kBlockM + p.causal_off;  // last key the tile's first row sees
    const int row_limit = tile_limit + r;                      // last key this row sees
    for (int i = 0; i < T; ++i) {
      w.tile = i;
      if (tr) B200ATTN_TRACE_EVENT(p, q, item, i, 0, 0);
      PROF_LAP(0);
      if (!w.wait_warp(bar(kBarSFull + q), s_parity, 300 + q)) return;
      s_parity ^= 1u;
      tc_fence_after_sync();
      PROF_LAP(1);
      if (tr) B200ATTN_TRACE_EVENT(p, q, item, i, 0, 1);

      uint32_t s[4][32];
      tmem_ld32(s_tmem + 0, s[0]);
      tmem_wait_ld();  // chunk 0 alone, so that its exponentials overlap the other three loads
      tmem_ld32(s_tmem + 32, s[1]);
      tmem_ld32(s_tmem + 64, s[2]);
      tmem_ld32(s_tmem + 96, s[3]);
      PROF_LAP(2);
      if (tr) B200ATTN_TRACE_EVENT(p, q, item, i, 0, 2);
      // keys of this tile that exist for this row: all 128, fewer in a ragged last tile, and with
      // a causal mask fewer (possibly none) in the tiles the diagonal crosses
      bool tail = (i == ragged_i && tail_valid < kBlockN);
      int valid = tail ? tail_valid : kBlockN;
      if (kCausal && i * kBlockN + kBlockN - 1 > tile_limit) {
        tail = true;
        valid = min(valid, row_limit - i * kBlockN + 1);
      }
      if (tail || i == 0) tmem_wait_ld();  // these paths look at all chunks at once
      if (tail) mask_tail(s, valid);

      uint32_t packed[4][16];
      f2 sum_a = f2_splat(0.0f), sum_b = f2_splat(0.0f);
      float tile_sum = 0.0f;
      bool exact = (i == 0);
      if (!exact) {
        const f2 neg_m2 = f2_splat(-m);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          exp_chunk(s[c], scale2, neg_m2, packed[c], sum_a, sum_b);
          if (c == 0) tmem_wait_ld();
        }
        tile_sum = f2_hsum(sum_a, sum_b);
        // written so that a NaN sum also lands on the exact path
        exact = __any_sync(0xffffffffu, !(tile_sum < sum_limit));
      }
      if (tr) B200ATTN_TRACE_EVENT_AFTER(p, q, item, i, 0, 6, tile_sum);
      if (__builtin_expect(exact, 0)) {
        if (i > 0) {
          // the score registers were consumed by the speculation: fetch them again
#pragma unroll
          for (int c = 0; c < 4; ++c) tmem_ld32(s_tmem + c * 32, s[c]);
          tmem_wait_ld();
          if (tail) mask_tail(s, valid);
        }
        const float tile_max = row_max(s) * scale_log2;
        if (i == 0) {
          m = tile_max;
        } else {
          const float m_new = fmaxf(m, tile_max);
          const float f = ex2_approx(m - m_new);
          m = m_new;
          l *= f;
          if (__any_sync(0xffffffffu, f != 1.0f)) {
#pragma unroll 1
            for (int c = 0; c < kHeadDim / 16; ++c) {
              uint32_t acc[16];
              tmem_ld16(o_tmem + c * 16, acc);
              tmem_wait_ld();
#pragma unroll
              for (int j = 0; j < 16; ++j) acc[j] = __float_as_uint(__uint_as_float(acc[j]) * f);
              tmem_st16(o_tmem + c * 16, acc);
            }
            tmem_wait_st();
          }
        }
        const f2 neg_m2 = f2_splat(-m);
        sum_a = f2_splat(0.0f);
        sum_b = f2_splat(0.0f);
#pragma unroll
        for (int c = 0; c < 4; ++c) exp_chunk(s[c], scale2, neg_m2, packed[c], sum_a, sum_b);
        tile_sum = f2_hsum(sum_a, sum_b);
      }
      if (tr) B200ATTN_TRACE_EVENT_AFTER(p, q, item, i, 0, 3, tile_sum);
#ifdef B200ATTN_PROFILE
      asm volatile("" ::"f"(tile_sum), "r"(packed[3][15]));
#endif
      PROF_LAP(3);

#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_st16(p_tmem + c * 16, packed[c]);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
#ifdef B200ATTN_TEST_DROP_P_READY
      // Test builds only (never the shipped library): one warp withholds one arrival, so that the
      // bounded waits of every role run out and the CTA leaves with a recorded timeout.
      const bool withheld = (q == 0 && warp_in_group == 0 && item == 0 && i == 1);
      mbar_arrive_lead((lane == 0 && !withheld) ? 1u : 0u, bar(kBarPReady + q));
#else
      mbar_arrive_lead(lane == 0 ? 1u : 0u, bar(kBarPReady + q));
#endif
      PROF_LAP(4);
      if (tr) B200ATTN_TRACE_EVENT(p, q, item, i, 0, 4);
      l += tile_sum;
      if (tr) B200ATTN_TRACE_EVENT(p, q, item, i, 0, 5);
    }
    aux->row_max[q][r] = m;
    aux->row_sum[q][r] = l;
    __syncwarp();
    if (lane == 0) mbar_arrive(bar(kBarFin + q));
  }
  PROF_LAP(0);
  if (warp_in_group == 0 && lane == 0) PROF_FLUSH(p, 8 + 8 * q, 8);
}

// ---- epilogue -------------------------------------------------------------------------------
// A cut piece's partial result and, for the piece that finishes last, the merge of the item.
// Called by one epilogue warp for its 32 rows of Q tile q, after the piece's partial (normalised
// fp32 O and LSE) has been stored to this CTA's slot. Nobody waits for another CTA: every piece
// stores, fences and takes a ticket; whoever draws the last ticket finds every partial in memory
// and writes the item's bf16 O and LSE.
//
// The pieces of an item belong to consecutive CTAs c_first .. c_last (runs strictly inside an item
// are never empty), in slot 0 of each except possibly c_first, whose run may have begun before
// the item. The merge first finds every row's total LSE (one row per lane), then walks the rows
// with the whole warp on one row at a time, so that partial rows are read and the output row is
// written as whole 512- and 256-byte lines.
__device__ void split_merge_rows(const FwdParams& p, const Piece& pc, const ItemCoord& c, int q,
                                 int warp_in_group, int lane) {
  const int grid = int(gridDim.x);
  const int T = p.kv_tiles;
  const int item_u0 = (pc.item - split_first_item(p, grid)) * T;
  const int c_first = split_owner(p, item_u0);
  const int c_last = split_owner(p, item_u0 + T - 1);
  const int pieces = c_last - c_first + 1;

  // every lane's stores are ordered before the ticket
  __threadfence();
  __syncwarp();
  int32_t* ticket = p.split_tickets + c_first * kSplitTicketsPerCta + q * 4 + warp_in_group;
  int drawn = 0;
  if (lane == 0) drawn = atomicAdd(ticket, 1);
  drawn = __shfl_sync(0xffffffffu, drawn, 0);
  if (drawn != pieces - 1) return;
  if (lane == 0) *ticket = 0;  // ready for the next launch
  __threadfence();

  const int first_which = split_cut(p, c_first) < item_u0 ? 1 : 0;
  const float* slot0 = p.split_scratch + (size_t(c_first) * 2 + first_which) * kSplitSlotFloats;
  auto slot_of = [&](int k) -> const float* {  // k-th piece of the item
    return k == 0 ? slot0 : p.split_scratch + size_t(c_first + k) * 2 * kSplitSlotFloats;
  };
  const int rs0 = q * kBlockM + warp_in_group * 32;  // first of this warp's rows inside a slot
  // pass 1 (one row per lane): the row's total LSE and the weights of its first four pieces
  float top = kNegInf, sum = 0.0f;
  float lse_k[4] = {kNegInf, kNegInf, kNegInf, kNegInf};
#pragma unroll
  for (int k = 0; k < 4; ++k)
    if (k < pieces) lse_k[k] = __ldcg(slot_of(k) + kItemRows * kHeadDim + rs0 + lane);
#pragma unroll
  for (int k = 0; k < 4; ++k) top = fmaxf(top, lse_k[k]);
  for (int k = 4; k < pieces; ++k) top = fmaxf(top, __ldcg(slot_of(k) + kItemRows * kHeadDim + rs0 + lane));
#pragma unroll
  for (int k = 0; k < 4; ++k) sum += expf(lse_k[k] - top);  // exp(-inf) = 0 for absent pieces
  for (int k = 4; k < pieces; ++k) sum += expf(__ldcg(slot_of(k) + kItemRows * kHeadDim + rs0 + lane) - top);
  const float lse_mine = top + logf(sum);
  float w_k[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) w_k[k] = expf(lse_k[k] - lse_mine);
  const int row_mine = c.row0 + rs0 + lane;
  if (row_mine < p.len_q && p.lse != nullptr)
    p.lse[(int64_t(c.b) * p.heads + c.h) * p.len_q + row_mine] = lse_mine;

  // pass 2: four rows per step, the whole warp on each row (lane l holds columns 4l .. 4l+3), every
  // load of a step in flight before the first use
  __nv_bfloat16* o_base = p.o + int64_t(c.b) * p.o_stride_b + int64_t(c.h) * p.o_stride_h;
#pragma unroll 1
  for (int rr = 0; rr < 32; rr += 4) {
    float4 acc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < pieces; ++k) {
      const float* slot = slot_of(k);
      float4 a[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        a[j] = __ldcg(reinterpret_cast<const float4*>(slot + size_t(rs0 + rr + j) * kHeadDim) + lane);
      float wgt[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float w0 = __shfl_sync(0xffffffffu, w_k[0], rr + j), w1 = __shfl_sync(0xffffffffu, w_k[1], rr + j);
        const float w2 = __shfl_sync(0xffffffffu, w_k[2], rr + j), w3 = __shfl_sync(0xffffffffu, w_k[3], rr + j);
        const float lt = __shfl_sync(0xffffffffu, lse_mine, rr + j);
        wgt[j] = k == 0 ? w0 : k == 1 ? w1 : k == 2 ? w2 : k == 3 ? w3
                 : expf(__ldcg(slot + kItemRows * kHeadDim + rs0 + rr + j) - lt);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[j].x = fmaf(a[j].x, wgt[j], acc[j].x);
        acc[j].y = fmaf(a[j].y, wgt[j], acc[j].y);
        acc[j].z = fmaf(a[j].z, wgt[j], acc[j].z);
        acc[j].w = fmaf(a[j].w, wgt[j], acc[j].w);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int row = c.row0 + rs0 + rr + j;
      if (row >= p.len_q) continue;  // uniform across the warp
      uint2 out;
      out.x = pack_bf16x2(acc[j].x, acc[j].y);
      out.y = pack_bf16x2(acc[j].z, acc[j].w);
      *reinterpret_cast<uint2*>(o_base + int64_t(row) * p.o_stride_l + lane * 4) = out;
    }
  }
}

// Once per piece and Q tile: take the final (max, sum) from the softmax group, read the
// accumulator out of TMEM, normalise, optionally merge with a stored partial, store O / LSE.
template <bool kCausal, bool kSplit>
__device__ void ws_epilogue_role(const FwdParams& p, WsAux* aux, uint32_t bar0, uint32_t tmem_base,
                                 int warp_in_group, int lane, WaitCtx& w) {
  auto bar = [&](int i) { return bar0 + 8u * uint32_t(i); };
  const uint32_t lane_field = uint32_t(warp_in_group * 32) << 16;
  const int r = warp_in_group * 32 + lane;
  uint32_t fin_parity = 0;

  typename WalkOf<kCausal, kSplit>::type pw(p, aux);
  Piece pc;
  while (pw.take(p, pc)) {
    const int item = pc.item;
    w.item = item;
    w.tile = p.kv_tiles;
    const ItemCoord c = decode_item<kCausal>(p, item);
    const bool cut = kSplit && (pc.t0 > 0 || pc.t1 < p.kv_tiles);
    for (int q = 0; q < kQTilesPerItem; ++q) {
      if (!w.wait_warp(bar(kBarFin + q), fin_parity, 410 + q)) return;
      if (!w.wait_warp(bar(kBarPvDone + q), fin_parity, 420 + q)) return;
      tc_fence_after_sync();
      const float fin_m = aux->row_max[q][r];
      const float fin_l = aux->row_sum[q][r];
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarFinFree + q));
      const int row = c.row0 + q * kBlockM + r;
      RowOut out;
      if (cut) {
        // this piece covers only part of the item's keys: leave a partial in this CTA's slot
        // (slot 0 if the piece opens the CTA's run, else slot 1)
        const int unit = (item - split_first_item(p, int(gridDim.x))) * p.kv_tiles + pc.t0;
        const bool opens_run = unit == split_cut(p, int(blockIdx.x));
        float* slot = p.split_scratch + (size_t(blockIdx.x) * 2 + (opens_run ? 0 : 1)) * kSplitSlotFloats;
        const int rs = q * kBlockM + r;
        out.valid = row < p.len_q;
        out.o_row = nullptr;
        out.part_row = slot + size_t(rs) * kHeadDim;
        out.w_cur = 1.0f / fin_l;
        out.w_prev = 0.0f;
        out.emit_partial = true;
        if (out.valid) slot[kItemRows * kHeadDim + rs] = (fin_m + log2f(fin_l)) * kLn2;
      } else {
        out = make_row_out(p, c.b, c.h, row, fin_m, fin_l);
      }
      const uint32_t o_tmem = tmem_base + kQTilesPerItem * kBlockN + q * kHeadDim + lane_field;
      store_row(out, o_tmem, [&]() {
        // O_q is in registers: the next piece's first PV may overwrite it.
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(kBarOFree + q));
      });
    }
    // Tickets and merges of the run's cut pieces wait until the run's last piece has handed both
    // accumulators back: they then run beside the CTA's whole items (or, with none, at the end)
    // and never between two short pieces, where they would hold up the next hand-back.
    if constexpr (kSplit) {
      if (pw.k == aux->run_pieces) {
        for (int j = 0; j < aux->run_pieces; ++j) {
          const Piece done = aux->run_piece[j];
          if (done.t0 == 0 && done.t1 == p.kv_tiles) continue;
          const ItemCoord dc = decode_item<kCausal>(p, done.item);
          for (int q = 0; q < kQTilesPerItem; ++q) {
            split_merge_rows(p, done, dc, q, warp_in_group, lane);
            __syncwarp();
          }
        }
      }
    }
    fin_parity ^= 1u;
  }
}

// kShortKv: the variant for items of few K/V tiles (see attn_fwd_ws_short_kernel).
template <bool kCausal, bool kSplit, bool kShortKv>
__device__ __forceinline__ void ws_kernel_body(const CUtensorMap& tmap_q, const CUtensorMap& tmap_k,
                                               const CUtensorMap& tmap_v, const FwdParams& p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const uint32_t smem_q = smem_u32(smem);
  const uint32_t smem_kv = smem_q + kQTilesPerItem * kTileBytes;
  WsAux* aux = reinterpret_cast<WsAux*>(smem + kQTilesPerItem * kTileBytes + kPairSlots * kPairBytes);
  const uint32_t bar0 = smem_u32(&aux->bar[0]);

  WaitCtx w;
  w.abort_addr = smem_u32(&aux->abort_flag);
  w.status = p.status;
  w.limit_ns = uint64_t(p.wait_limit_ms) * 1000000ull;
  w.item = -1;
  w.tile = -1;

  const bool misaligned = (smem_q & 1023u) != 0;  // uniform across the CTA
  if (threadIdx.x == 0) {
    aux->abort_flag = 0;
    if (misaligned) {
      w.raise(kDevSmemMisaligned, 1, 0);
    } else {
      for (int q = 0; q < kQTilesPerItem; ++q) {
        mbar_init(bar0 + 8u * (kBarQFull + q), 1);
        mbar_init(bar0 + 8u * (kBarQEmpty + q), 1);
        mbar_init(bar0 + 8u * (kBarSFull + q), 1);
        mbar_init(bar0 + 8u * (kBarPReady + q), 4);
        mbar_init(bar0 + 8u * (kBarSpare + q), 1);
        mbar_init(bar0 + 8u * (kBarPvDone + q), 1);
        mbar_init(bar0 + 8u * (kBarFin + q), 4);
        mbar_init(bar0 + 8u * (kBarFinFree + q), 4);
        mbar_init(bar0 + 8u * (kBarOFree + q), 4);
      }
      mbar_init(bar0 + 8u * kBarDrain, 1);
      mbar_init(bar0 + 8u * (kBarDrain + 1), 1);
      for (int s = 0; s < kPairSlots; ++s) {
        mbar_init(bar0 + 8u * (kBarPairFull + s), 1);
        mbar_init(bar0 + 8u * (kBarPairEmpty + s), 1);
      }
      mbar_init_fence();
      fence_proxy_async_smem();
      if (kSplit) plan_run(p, aux);
    }
  }
  if (misaligned) return;
  if (warp == 12) {
    tmem_alloc(smem_u32(&aux->tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = aux->tmem_base;

  if (warp < 8) {
    reg_grow<kRegsSoftmax>();
    ws_softmax_role<kCausal, kSplit>(p, aux, bar0, tmem_base, warp >> 2, warp & 3, lane, w);
  } else if (warp < 12) {
    reg_shrink<kRegsEpilogue>();
    ws_epilogue_role<kCausal, kSplit>(p, aux, bar0, tmem_base, warp & 3, lane, w);
  } else {
    reg_shrink<kRegsOther>();
    const uint32_t lead = (lane == 0) ? 1u : 0u;
    if (warp == 12) {
      // kShortKv: the TMEM base (read from shared memory above) goes through a warp-wide
      // reduction first, whose result the compiler knows to be the same in every lane. Measured
      // +2.1 % at 4 K/V tiles per item, +0.8 % at 8, -0.5 % at 64.
      ws_mma_role<kCausal, kSplit>(p, aux, smem_q, smem_kv, bar0,
                                   kShortKv ? __reduce_or_sync(0xffffffffu, tmem_base) : tmem_base, lead, w);
    } else if (warp == 13) {
      if (lead) {
        tma_prefetch_desc(&tmap_q);
        tma_prefetch_desc(&tmap_k);
        tma_prefetch_desc(&tmap_v);
      }
      __syncwarp();
        ws_load_role<kCausal, kSplit>(p, aux, &tmap_q, &tmap_k, &tmap_v, smem_q, smem_kv, bar0, lead, w);
    }
    __syncwarp();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 12) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <bool kCausal, bool kSplit>
__global__ void __launch_bounds__(kWsThreads, 1)
attn_fwd_ws_kernel(const __grid_constant__ CUtensorMap tmap_q,
                   const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const FwdParams p) {
  ws_kernel_body<kCausal, kSplit, false>(tmap_q, tmap_k, tmap_v, p);
}

// The dense, unsplit kernel as launched for items of at most kShortKvTiles K/V tiles.
constexpr int kShortKvTiles = 8;
__global__ void __launch_bounds__(kWsThreads, 1)
attn_fwd_ws_short_kernel(const __grid_constant__ CUtensorMap tmap_q,
                         const __grid_constant__ CUtensorMap tmap_k,
                         const __grid_constant__ CUtensorMap tmap_v, const FwdParams p) {
  ws_kernel_body<false, false, true>(tmap_q, tmap_k, tmap_v, p);
}

// ==========================================================================================
// Serial bring-up kernel: one CTA per 128 query rows, 4 warps, thread 0 issues TMA and MMA.
// ==========================================================================================
struct alignas(16) SerialAux {
  uint64_t bar_q, bar_k, bar_v, bar_mma, bar_drain;
  uint32_t tmem_base;
  uint32_t abort_flag;
};
constexpr int kSerialSmemBytes = 3 * kTileBytes + int(sizeof(SerialAux));

__global__ void __launch_bounds__(128, 1)
attn_fwd_serial_kernel(const __grid_constant__ CUtensorMap tmap_q,
                       const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v, const FwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_q = smem_u32(smem);
  const uint32_t smem_k = smem_q + kTileBytes;
  const uint32_t smem_v = smem_k + kTileBytes;
  SerialAux* aux = reinterpret_cast<SerialAux*>(smem + 3 * kTileBytes);
  const uint32_t bar_q = smem_u32(&aux->bar_q), bar_k = smem_u32(&aux->bar_k),
                 bar_v = smem_u32(&aux->bar_v), bar_mma = smem_u32(&aux->bar_mma);

  WaitCtx w;
  w.abort_addr = smem_u32(&aux->abort_flag);
  w.status = p.status;
  w.limit_ns = uint64_t(p.wait_limit_ms) * 1000000ull;
  w.item = int(blockIdx.x);
  w.tile = -1;

  const bool misaligned = (smem_q & 1023u) != 0;
  if (threadIdx.x == 0) {
    aux->abort_flag = 0;
    if (misaligned) {
      w.raise(kDevSmemMisaligned, 2, 0);
    } else {
      mbar_init(bar_q, 1);
      mbar_init(bar_k, 1);
      mbar_init(bar_v, 1);
      mbar_init(bar_mma, 1);
      mbar_init(smem_u32(&aux->bar_drain), 1);
      mbar_init_fence();
      fence_proxy_async_smem();
    }
  }
  if (misaligned) return;
  if (warp == 0) {
    tmem_alloc(smem_u32(&aux->tmem_base), 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = aux->tmem_base;
  const uint32_t lane_field = uint32_t(warp * 32) << 16;
  const uint32_t s_tmem = tmem_base + lane_field;          // S, then P in columns 0..63
  const uint32_t o_tmem = tmem_base + kBlockN + lane_field;

  // The serial kernel's m-blocks are single 128-row tiles.
  const int m_tiles = (p.len_q + kBlockM - 1) / kBlockM;
  const int bh = int(blockIdx.x) / m_tiles;
  const int row0 = (int(blockIdx.x) - bh * m_tiles) * kBlockM;
  const int b = bh / p.heads, h = bh - b * p.heads;
  const int T = p.kv_tiles;
  const int tail_valid = p.len_kv - (T - 1) * kBlockN;
  const bool issuer = threadIdx.x == 0;

  uint32_t kv_parity = 0, mma_parity = 0;
  uint32_t armed_parity = 0;  // parity of the K/V phase armed most recently (issuer only)
  float m = kNegInf, l = 0.0f;
  bool ok = true;

  if (issuer) load_tile(1u, smem_q, &tmap_q, row0, h, b, bar_q);

  for (int i = 0; i < T; ++i) {
    w.tile = i;
    if (issuer) {
      load_tile(1u, smem_k, &tmap_k, i * kBlockN, h, b, bar_k);
      load_tile(1u, smem_v, &tmap_v, i * kBlockN, h, b, bar_v);
      armed_parity = kv_parity;
      ok = (i > 0) || w.wait(bar_q, 0, 500);
      ok = ok && w.wait(bar_k, kv_parity, 501);
      if (ok) {
        tc_fence_after_sync();
        issue_qk(1u, tmem_base, smem_q, smem_k);
      }
      umma_commit(bar_mma);  // always commit so nobody is left waiting for a missing arrival
    }
    __syncwarp();
    if (!w.wait_warp(bar_mma, mma_parity, 502)) break;
    mma_parity ^= 1u;
    tc_fence_after_sync();

    uint32_t s[4][32];
    tmem_ld32(s_tmem + 0, s[0]);
    tmem_ld32(s_tmem + 32, s[1]);
    tmem_ld32(s_tmem + 64, s[2]);
    tmem_ld32(s_tmem + 96, s[3]);
    tmem_wait_ld();
    if (i == T - 1 && tail_valid < kBlockN) mask_tail(s, tail_valid);

    const float m_new = fmaxf(m, row_max(s) * p.scale_log2);
    if (i > 0) {
      const float alpha = ex2_approx(m - m_new);
      l *= alpha;
#pragma unroll 1
      for (int c = 0; c < kHeadDim / 32; ++c) {
        uint32_t acc[32];
        tmem_ld32(o_tmem + c * 32, acc);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = __float_as_uint(__uint_as_float(acc[j]) * alpha);
        tmem_st32(o_tmem + c * 32, acc);
      }
    }
    m = m_new;
    float sum = 0.0f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t packed[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float e0 = ex2_approx(fmaf(__uint_as_float(s[c][2 * j]), p.scale_log2, -m));
        const float e1 = ex2_approx(fmaf(__uint_as_float(s[c][2 * j + 1]), p.scale_log2, -m));
        sum += e0 + e1;
        packed[j] = pack_bf16x2(e0, e1);
      }
      tmem_st16(s_tmem + c * 16, packed);
    }
    l += sum;
    tmem_wait_st();
    tc_fence_before_sync();
    __syncthreads();

    if (issuer) {
      tc_fence_after_sync();
      ok = w.wait(bar_v, kv_parity, 503);
      if (ok) {
        tc_fence_after_sync();
        issue_pv(1u, tmem_base + kBlockN, tmem_base, smem_v, i > 0);
      }
      umma_commit(bar_mma);
    }
    kv_parity ^= 1u;
    __syncwarp();
    if (!w.wait_warp(bar_mma, mma_parity, 504)) break;
    mma_parity ^= 1u;
    tc_fence_after_sync();
  }

  if (!w.aborted()) {
    const RowOut out = make_row_out(p, b, h, row0 + warp * 32 + lane, m, l);
    store_row(out, o_tmem, []() {});
  } else if (issuer) {
    // Bounded drain of the copies and MMAs still in flight before shared memory and TMEM go.
    const uint64_t t0 = global_timer_ns();
    const uint32_t bar_drain = smem_u32(&aux->bar_drain);
    umma_commit(bar_drain);
    while (!(mbar_try_wait(bar_q, 0, 1000) && mbar_try_wait(bar_k, armed_parity, 1000) &&
             mbar_try_wait(bar_v, armed_parity, 1000) && mbar_try_wait(bar_drain, 0, 1000))) {
      if (global_timer_ns() - t0 > w.limit_ns) break;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 256);
  }
}

}  // namespace

// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------
cudaError_t prepare_kernels() {
  // The warp-specialised kernel re-partitions registers between its roles. A growing role
  // blocks in hardware until the CTA's pool has room, so refuse to run unless the pool the
  // launch reserves (registers per thread x 512 threads) covers what the roles ask for.
  constexpr int kPoolNeeded = 128 * (2 * kRegsSoftmax + kRegsEpilogue + kRegsOther);
  const void* ws_kernels[4] = {reinterpret_cast<const void*>(&attn_fwd_ws_kernel<false, false>),
                               reinterpret_cast<const void*>(&attn_fwd_ws_kernel<true, false>),
                               reinterpret_cast<const void*>(&attn_fwd_ws_kernel<false, true>),
                               reinterpret_cast<const void*>(&attn_fwd_ws_short_kernel)};
  for (const void* kernel : ws_kernels) {
    cudaFuncAttributes fa;
    cudaError_t e = cudaFuncGetAttributes(&fa, kernel);
    if (e != cudaSuccess) return e;
    if (fa.numRegs * kWsThreads < kPoolNeeded) return cudaErrorLaunchOutOfResources;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kWsSmemBytes);
    if (e != cudaSuccess) return e;
  }
  return cudaFuncSetAttribute(attn_fwd_serial_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              kSerialSmemBytes);
}

SplitPlan split_plan(const FwdParams& p, int sm_count) {
  const SplitPlan none{0, 0};
  if (p.causal || p.partial.merge || p.partial.emit || p.kv_tiles < 2 * kSplitMinPieceTiles) return none;
  if (static_cast<long long>(p.total_items) * p.kv_tiles >= (1ll << 31)) return none;
  // the last, partly filled round of whole items is what gets cut into equal runs
  const int tail_items = p.total_items % sm_count;
  if (tail_items == 0) return none;
  const bool full_rounds = p.total_items >= sm_count;
  const long long tail_units = static_cast<long long>(tail_items) * p.kv_tiles;
  long long runs = tail_units / kSplitMinPieceTiles;
  if (runs > sm_count) runs = sm_count;
  if (runs > kSplitMaxRuns) runs = kSplitMaxRuns;
  // Without full rounds behind it the merge of a cut item stands at the end of the launch, and it
  // costs about six tile periods per piece: keep the pieces per item few.
  constexpr int kExposedPiecesPerItem = 4, kMergeTilesPerPiece = 6;
  if (!full_rounds && runs > static_cast<long long>(tail_items) * kExposedPiecesPerItem)
    runs = static_cast<long long>(tail_items) * kExposedPiecesPerItem;
  if (runs < 1) return none;
  const int grid = full_rounds ? sm_count : int(runs);
  // tiles on the busiest CTA: whole items dealt round-robin, against full rounds plus one even run
  // per CTA (which pays for up to two cut pieces: their extra Q loads and partial stores, about
  // three tile periods, and for an exposed merge)
  const int rounds_grid = full_rounds ? sm_count : p.total_items;
  const long long legacy = static_cast<long long>((p.total_items + rounds_grid - 1) / rounds_grid) * p.kv_tiles;
  const long long pieces_per_item = (runs + tail_items - 1) / tail_items + 1;
  const long long split = static_cast<long long>(p.total_items / sm_count) * p.kv_tiles + (tail_units + runs - 1) / runs +
                          3 + (full_rounds ? 0 : kMergeTilesPerPiece * pieces_per_item);
  return (split * 100 < legacy * 97) ? SplitPlan{grid, int(runs)} : none;
}

// The cuts: run c ends where an even share of what is left would end, moved down to the nearest
// admissible place (an item boundary, or at least kSplitMinPieceTiles away from both ends of the
// item), so no run grows beyond the even share by more than the rounding and the slack spreads over
// the runs that follow; a run is at least kSplitMinPieceTiles long.
void split_fill_cuts(FwdParams& p, int sm_count, const SplitPlan& plan) {
  const int T = p.kv_tiles;
  const int total = (p.total_items % sm_count) * T;
  const int runs = plan.runs < kSplitMaxRuns ? plan.runs : kSplitMaxRuns;
  auto admissible = [&](int u) {
    const int r = u % T;
    return r == 0 || (r >= kSplitMinPieceTiles && r <= T - kSplitMinPieceTiles);
  };
  p.split_runs = runs;
  p.split_cut[0] = 0;
  for (int c = 0; c < runs; ++c) {
    const int from = p.split_cut[c], left = runs - c;
    int u = total;
    if (left > 1 && from < total) {
      int lowest = from + kSplitMinPieceTiles;
      while (!admissible(lowest)) ++lowest;
      u = from + (total - from + left - 1) / left;
      while (u > lowest && !admissible(u)) --u;
      if (u < lowest) u = lowest;
      if (total - u < kSplitMinPieceTiles) u = total;
    }
    p.split_cut[c + 1] = u;
  }
}

cudaError_t launch_fwd_ws(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                          const FwdParams& p, int sm_count, cudaStream_t stream) {
  const int grid = p.total_items < sm_count ? p.total_items : sm_count;
  if (p.causal) {
    attn_fwd_ws_kernel<true, false><<<grid, kWsThreads, kWsSmemBytes, stream>>>(tq, tk, tv, p);
  } else if (p.split_scratch != nullptr) {
    attn_fwd_ws_kernel<false, true><<<split_plan(p, sm_count).grid, kWsThreads, kWsSmemBytes, stream>>>(tq, tk, tv, p);
  } else {
    if (p.kv_tiles <= kShortKvTiles) {
      attn_fwd_ws_short_kernel<<<grid, kWsThreads, kWsSmemBytes, stream>>>(tq, tk, tv, p);
    } else {
      attn_fwd_ws_kernel<false, false><<<grid, kWsThreads, kWsSmemBytes, stream>>>(tq, tk, tv, p);
    }
  }
  return cudaGetLastError();
}

cudaError_t launch_fwd_serial(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                              const FwdParams& p, cudaStream_t stream) {
  const int m_tiles = (p.len_q + kBlockM - 1) / kBlockM;
  const int grid = p.batch * p.heads * m_tiles;
  attn_fwd_serial_kernel<<<grid, 128, kSerialSmemBytes, stream>>>(tq, tk, tv, p);
  return cudaGetLastError();
}

}  // namespace b200attn
