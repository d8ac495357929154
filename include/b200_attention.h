/*
 * b200_attention.h — C ABI of libb200attn.so: dense forward scaled-dot-product attention for
 * NVIDIA B200 (sm_100a): non-causal, or with a causal mask; optionally with grouped K/V heads.
 * bf16 Q/K/V in, bf16 O out, optional fp32 LSE, head_dim 128. Plain pointers and sizes only; no torch types. Every entry point returns
 * a b200attn_status (0 = success) and never throws or aborts.
 *
 * Which entry point replaces which interface of the reference project
 * (IaroslavElistratov/b200-attention, paths relative to its root):
 *
 *   b200attn_bhld_launch   the per-checkpoint launcher symbol bound by the benchmark
 *                          registry's generated glue,
 *                          `void <launch_symbol>(const nv_bfloat16* Q, K, V, nv_bfloat16* O,
 *                          int batch_heads, int len_q, int len_kv, cudaStream_t)`
 *                          (benchmarks/registry.py:272-282; implemented by
 *                          kernels/5_minor/18_tma_l2_promotion.cu:1007-1059), which is also
 *                          what the capstone op calls (capstone-project/kernel/binding.cpp:13-23).
 *   b200attn_bshd_launch   the direct-BSHD launcher
 *                          `attention_tcgen05_v18_bshd_launch(Q, K, V, O, batch, heads, len_q,
 *                          len_kv, stream)` (benchmarks/benchmark_bshd.py:151-160;
 *                          kernels/variants/18_tma_l2_promotion_bshd.cu:1076-1133).
 *   b200attn_forward       superset of both: arbitrary (batch, head, row) strides, runtime
 *                          softmax scale, LSE output, partial-result chaining for a
 *                          sequence-parallel K/V ring. The reference has no counterpart for
 *                          the extra arguments (its scale is fixed at 1/sqrt(128),
 *                          18_tma_l2_promotion.cu:654, and it has no LSE or multi-GPU path).
 *                          Its `causal` / `heads_kv` fields cover the operator of the
 *                          reference's research launcher
 *                          `attention_tcgen05_causal_gqa_2cta_launch(Q, K, V, O, LSE, counter, B,
 *                          Sq, Skv, Hq, Hkv, softmax_scale, stream)`
 *                          (research/causal_gqa_2cta.cu:1131-1137).
 */
#ifndef B200_ATTENTION_H_
#define B200_ATTENTION_H_

#include <stdint.h>

#if defined(__GNUC__)
#define B200ATTN_API __attribute__((visibility("default")))
#else
#define B200ATTN_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum b200attn_status {
  B200ATTN_OK = 0,
  B200ATTN_ERR_INVALID_ARGUMENT = 1,  /* null pointer, non-positive size, bad stride, bad struct */
  B200ATTN_ERR_UNSUPPORTED = 2,       /* head_dim != 128, sizes beyond the kernel's limits */
  B200ATTN_ERR_ARCH = 3,              /* device is not compute capability 10.0 */
  B200ATTN_ERR_CUDA = 4,              /* a CUDA runtime call failed; see b200attn_last_error */
  B200ATTN_ERR_DRIVER = 5,            /* tensor-map encoding failed or driver entry point missing */
  B200ATTN_ERR_DEVICE_TIMEOUT = 6,    /* a bounded device-side wait ran out (kernel left early) */
  B200ATTN_ERR_DEVICE_FAULT = 7       /* device-side self check failed (e.g. misaligned smem) */
} b200attn_status;

enum { B200ATTN_KERNEL_WARP_SPECIALIZED = 0, B200ATTN_KERNEL_SERIAL = 1 };

/* One operand: base pointer (device memory) and strides in ELEMENTS for the batch, head and
 * row (sequence) axes. The head_dim axis is contiguous. Every stride times 2 bytes must be a
 * multiple of 16 bytes and the base 16-byte aligned (TMA requirements). */
typedef struct b200attn_operand {
  const void* ptr;
  int64_t stride_batch;
  int64_t stride_head;
  int64_t stride_row;
} b200attn_operand;

typedef struct b200attn_forward_args {
  uint32_t struct_bytes; /* sizeof(b200attn_forward_args), checked */
  int32_t batch, heads, len_q, len_kv, head_dim;
  b200attn_operand q, k, v; /* bf16 */
  b200attn_operand o;       /* bf16, written; ptr is cast to mutable */
  float* lse;               /* [batch, heads, len_q] fp32 contiguous, natural log; may be NULL */
  float softmax_scale;      /* <= 0 selects 1/sqrt(head_dim) */
  int32_t kernel;           /* B200ATTN_KERNEL_* */
  /* Partial-result chaining (sequence-parallel K/V ring). Scratch owned by the caller:
   *   partial_o   [batch, heads, len_q, 128] fp32 contiguous
   *   partial_lse [batch, heads, len_q]      fp32 contiguous
   * partial_merge != 0: the epilogue merges the (O, LSE) pair already stored there with this
   *                     call's result (in registers, no extra kernel);
   * partial_emit  != 0: the (merged) pair is written back there instead of to o / lse. */
  float* partial_o;
  float* partial_lse;
  int32_t partial_merge;
  int32_t partial_emit;
  void* stream; /* cudaStream_t; NULL = the legacy default stream */
  /* Causal mask and grouped-query attention (warp-specialised kernel only). The reference's
   * shipped kernels are dense and ungrouped; its research kernel
   * (research/causal_gqa_2cta.cu:1131-1137: always causal, square, heads == 4 * heads_kv, BSHD)
   * is the adjacent operator these two fields cover.
   *   causal   != 0: key j is visible to query row i iff j <= i + (len_kv - len_q), i.e. the mask
   *                  is aligned to the bottom-right corner; needs len_kv >= len_q.
   *   heads_kv  > 0: k and v have heads_kv heads (their strides and extents refer to that many);
   *                  query head h reads K/V head h / (heads / heads_kv); heads % heads_kv == 0.
   *                  0 means heads_kv == heads. */
  int32_t causal;
  int32_t heads_kv;
  /* Optional workspace for the tile-stream split (no counterpart in the reference, whose
   * scheduler deals whole 256-row work items round-robin, 18_tma_l2_promotion.cu:1039-1046).
   * With at least b200attn_workspace_bytes() of ZEROED, 16-byte aligned device memory here, a
   * dense call whose work items do not fill the SMs evenly (e.g. 256 items on 148 SMs) is cut
   * into one equal run of K/V tiles per SM instead; work items cut by a run boundary are merged
   * in the kernel through this memory (fp32 partial O and LSE, arrival counters that return to
   * zero). The call decides by itself whether splitting pays; results are the same up to
   * rounding. The memory may be reused by later calls on the SAME stream; calls whose kernels
   * can overlap (other streams) need workspaces of their own. After a call that ended in
   * B200ATTN_ERR_DEVICE_TIMEOUT, zero it again. NULL: never split. */
  void* workspace;
  uint64_t workspace_bytes;
} b200attn_forward_args;

/* Asynchronous on args->stream. The device that is current when the call is made is used. */
B200ATTN_API int b200attn_forward(const b200attn_forward_args* args);

/* Size of b200attn_forward_args.workspace for the current device (depends on its SM count). */
B200ATTN_API int b200attn_workspace_bytes(uint64_t* bytes);

/* How a dense, unmasked call of `work_items` 256-row work items (batch * heads * ceil(len_q / 256))
 * over `kv_tiles` K/V tiles (ceil(len_kv / 128)) would be laid out on `sm_count` SMs when given a
 * workspace; host arithmetic only, needs no device (no counterpart in the reference). *grid = CTAs
 * launched, 0 if the call would not be split (then *runs = 0). Otherwise the first *runs CTAs share
 * the items of the last, partly filled round: numbering that round's (item, tile) pairs item-major,
 * CTA c works on units [cuts[c], cuts[c + 1]); cuts (may be NULL) receives *runs + 1 entries. */
B200ATTN_API int b200attn_split_layout(int32_t work_items, int32_t kv_tiles, int32_t sm_count, int32_t* grid,
                                       int32_t* runs, int32_t* cuts, int32_t max_cuts);

/* Q [batch_heads, len_q, 128], K/V [batch_heads, len_kv, 128], O like Q; all contiguous bf16.
 * Unlike the reference launcher there is no len_q % 256 / len_kv % 128 restriction. */
B200ATTN_API int b200attn_bhld_launch(const void* q, const void* k, const void* v, void* o, int batch_heads,
                         int len_q, int len_kv, void* stream);

/* Q [batch, len_q, heads, 128], K/V [batch, len_kv, heads, 128], O like Q; contiguous bf16,
 * read and written in place (no layout copies). */
B200ATTN_API int b200attn_bshd_launch(const void* q, const void* k, const void* v, void* o, int batch,
                         int heads, int len_q, int len_kv, void* stream);

/* The kernels never spin without a limit: a wait that exceeds the limit makes the CTA record
 * where it stopped and leave. After synchronising the stream(s) you launched on, call this to
 * learn whether that happened on `device` (-1 = current). On a non-zero result `record`
 * (8 ints, may be NULL) receives {code, site, block, warp, parity, item, tile, 0}; the record
 * is cleared by the call. */
B200ATTN_API int b200attn_device_check(int device, int32_t record[8]);

/* Limit for device-side waits, milliseconds (default 2000). Applies to later launches. */
B200ATTN_API int b200attn_set_wait_limit_ms(uint32_t ms);

/* Measurement aid (no counterpart in the reference project): records, for every SM a block of this
 * tiny kernel lands on, the SM's cycle counter and the global nanosecond timer, on `stream`.
 * `out` is device memory for 2 * max_sms int64 values: out[2 * smid] = clock64, out[2 * smid + 1]
 * = globaltimer (SMs with smid >= max_sms are skipped; entries of SMs no block ran on keep their
 * old contents, so clear the buffer first). Two samples around a timed region give the average
 * SM clock over exactly that region: (clock64_after - clock64_before) / (timer_after -
 * timer_before) per SM. Does not count towards b200attn_launch_count. */
B200ATTN_API int b200attn_sample_sm_clocks(int64_t* out, int32_t max_sms, void* stream);

/* Number of kernels this library has launched in this process (all devices, all streams). */
B200ATTN_API uint64_t b200attn_launch_count(void);

/* Peer access for the sequence-parallel ring, one process per GPU: export a handle for device
 * memory owned by this process / map a peer's handle. A handle names a whole allocation;
 * `offset_bytes` receives where device_ptr lies inside it (add it to the mapped base). */
B200ATTN_API int b200attn_ipc_export(const void* device_ptr, unsigned char handle[64],
                                     uint64_t* offset_bytes);
B200ATTN_API int b200attn_ipc_open(const unsigned char handle[64], void** mapped_ptr);
B200ATTN_API int b200attn_ipc_close(void* mapped_ptr);
/* Copy `bytes` from a peer-mapped (or local) pointer into local memory on `stream`. */
B200ATTN_API int b200attn_copy_async(void* dst_local, const void* src, uint64_t bytes, void* stream);

/* Forward pass for callers that must not allocate (no counterpart in the reference project).
 * Same arguments as b200attn_forward with partial_* unset; the key/value sequence is processed
 * in up to `kv_splits` chunks of whole 128-key tiles whose (O, LSE) partials are chained through
 * a fixed device array built into the library instead of caller scratch, and the wait watchdog
 * record lives there too, so neither this call nor its first-use set-up calls cudaMalloc,
 * cudaHostAlloc or any other allocating routine.
 *   - Limit: batch * heads * len_q <= B200ATTN_NOALLOC_MAX_ROWS query rows (the array is
 *     8,454,400 bytes and every GPU that loads the library holds it until process exit);
 *     larger problems return B200ATTN_ERR_UNSUPPORTED.
 *   - The first call on a device looks up the array's device address and sets kernel
 *     attributes; make that call before any stream capture.
 *   - All calls on a device share the array: calls whose kernels overlap on the GPU race.
 *   - A launching call (kv_splits >= 1) never queries, copies from or waits for the stream. A
 *     device-side wait that ran out is reported by a kv_splits == 0 call, which launches nothing,
 *     synchronises args->stream and reads the record back; it returns
 *     B200ATTN_ERR_INVALID_ARGUMENT on a stream that is being captured. */
#define B200ATTN_NOALLOC_MAX_ROWS 16384
B200ATTN_API int b200attn_forward_kv_split_noalloc(const b200attn_forward_args* args, int32_t kv_splits);

B200ATTN_API const char* b200attn_status_string(int status);
/* Message of the last failing call on this thread ("" if none). */
B200ATTN_API const char* b200attn_last_error(void);
B200ATTN_API const char* b200attn_version(void);

#ifdef __cplusplus
}
#endif
#endif /* B200_ATTENTION_H_ */
