// b200attn_forward_kv_split_noalloc: the forward pass for callers that must not allocate.
//
// The ordinary entry points allocate: the first b200attn_forward on a device reserves a pinned,
// device-mapped record for the kernels' wait watchdog, and chaining calls over K/V shards needs
// caller-allocated fp32 scratch for the partial (O, LSE). Some hosts cannot do either at call
// time: a serving process that handed the whole HBM to its own pool at start-up (so a fresh
// cudaMalloc fails or fragments the pool), or a latency-critical loop that cannot afford the
// device-wide synchronisation cudaMalloc / cudaFree / cudaHostAlloc imply. For them this file
// keeps everything the kernel needs besides its inputs and outputs in ONE file-scope device
// array of fixed size, part of the library image, held by every GPU that loads the library
// until the process exits.
//
// What the array holds and its limit: the fp32 partial O and LSE for at most
// B200ATTN_NOALLOC_MAX_ROWS = 16384 query rows (batch * heads * len_q) plus the watchdog record,
// 8,454,400 bytes in all. Larger problems are refused with B200ATTN_ERR_UNSUPPORTED.
//
// In host code the array's name is only a host-side stand-in for the symbol, never a device
// address, so the address the kernel gets is obtained with cudaGetSymbolAddress, once per
// device, with that device current, on the first call made on that device. That first call
// also sets kernel attributes; make it before any stream capture.
//
// Every call on a device shares the array and it keeps the previous call's contents. Nothing in
// the partial-state region has to start at zero (the first K/V chunk of a call overwrites it
// before any later chunk reads it); the watchdog record must: it is zero when the library image
// is loaded (file-scope device memory starts out zeroed) and is cleared again whenever a
// non-zero record has been reported. Two calls whose kernels overlap on the GPU (different
// streams, or different host threads) race on the array: serialise them.
//
// A launching call (kv_splits >= 1) only checks arguments and enqueues kernels: no stream query,
// no copy, no synchronisation. The watchdog record is read back only by a kv_splits == 0 call,
// which synchronises the stream; that call is refused on a stream that is being captured.
//
// The entry point calls no cudaMalloc, cudaFree, cudaHostAlloc or any other allocating routine.

#include "attn_kernels.cuh"
#include "host_common.cuh"

#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>

namespace {

using namespace b200attn;
using namespace b200attn::host;

constexpr int64_t kMaxRows = B200ATTN_NOALLOC_MAX_ROWS;
constexpr size_t kPartialOFloats = size_t(kMaxRows) * kHeadDim;
constexpr size_t kPartialLseFloats = size_t(kMaxRows);
constexpr size_t kStatusFloats = 64;  // 256 bytes; the first kStatusInts words are the record
constexpr size_t kScratchFloats = kPartialOFloats + kPartialLseFloats + kStatusFloats;

static __device__ __align__(256) float g_noalloc_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;

struct NoAllocDevice {
  std::once_flag once;
  int init_status = B200ATTN_OK;
  std::string init_error;
  float* scratch = nullptr;  // device address of g_noalloc_scratch on this device
  int sm_count = 0;
};
NoAllocDevice g_dev[kMaxDevices];

void setup_device(int device, NoAllocDevice* st) {
  auto cuda_fail = [&](const char* what, cudaError_t e) {
    st->init_status = B200ATTN_ERR_CUDA;
    st->init_error = std::string(what) + ": " + cudaGetErrorString(e);
    (void)cudaGetLastError();
  };
  int major = 0, minor = 0;
  cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&st->sm_count, cudaDevAttrMultiProcessorCount, device);
  if (e != cudaSuccess) return cuda_fail("device attribute query", e);
  if (major != 10 || minor != 0) {
    st->init_status = B200ATTN_ERR_ARCH;
    st->init_error = "device is not compute capability 10.0 (sm_100a required)";
    return;
  }
  if ((e = prepare_kernels()) != cudaSuccess) return cuda_fail("kernel attribute set-up", e);
  // The symbol's device address on the current device. Passing `g_noalloc_scratch` itself to a
  // kernel from host code would hand it a host-side shadow address.
  float* base = nullptr;
  if ((e = cudaGetSymbolAddress(reinterpret_cast<void**>(&base), g_noalloc_scratch)) != cudaSuccess)
    return cuda_fail("cudaGetSymbolAddress(scratch)", e);
  if (base == nullptr || (reinterpret_cast<uintptr_t>(base) & 255u) != 0) {
    st->init_status = B200ATTN_ERR_CUDA;
    st->init_error = "scratch symbol address is null or not 256-byte aligned";
    return;
  }
  st->scratch = base;
}

}  // namespace

extern "C" B200ATTN_API int b200attn_forward_kv_split_noalloc(const b200attn_forward_args* a,
                                                                int32_t kv_splits) {
  if (a == nullptr) return fail(B200ATTN_ERR_INVALID_ARGUMENT, "args is null");
  if (a->struct_bytes != sizeof(b200attn_forward_args))
    return fail(B200ATTN_ERR_INVALID_ARGUMENT, "struct_bytes does not match this library's b200attn_forward_args");
  if (a->head_dim != kHeadDim) return fail(B200ATTN_ERR_UNSUPPORTED, "head_dim must be 128");
  if (a->batch < 1 || a->heads < 1 || a->len_q < 1 || a->len_kv < 1)
    return fail(B200ATTN_ERR_INVALID_ARGUMENT, "batch, heads, len_q and len_kv must be positive");
  if (kv_splits < 0 || kv_splits > 64)
    return fail(B200ATTN_ERR_INVALID_ARGUMENT, "kv_splits must be in 0..64 (0 = only report the watchdog record)");
  if (a->kernel != B200ATTN_KERNEL_WARP_SPECIALIZED)
    return fail(B200ATTN_ERR_INVALID_ARGUMENT, "the no-allocation entry point runs the warp-specialised kernel only");
  if (a->partial_o != nullptr || a->partial_lse != nullptr || a->partial_merge != 0 || a->partial_emit != 0)
    return fail(B200ATTN_ERR_INVALID_ARGUMENT, "partial_* must be unset: the partial state lives in the built-in scratch");
  if (a->causal != 0 || (a->heads_kv != 0 && a->heads_kv != a->heads))
    return fail(B200ATTN_ERR_UNSUPPORTED, "the no-allocation entry point has no causal mask and no grouped K/V heads");
  const int64_t rows = int64_t(a->batch) * a->heads * a->len_q;
  if (rows > kMaxRows) {
    char buf[200];
    snprintf(buf, sizeof buf,
             "batch * heads * len_q = %lld query rows exceed the built-in scratch of %lld rows "
             "(B200ATTN_NOALLOC_MAX_ROWS); use b200attn_forward with caller-provided scratch",
             static_cast<long long>(rows), static_cast<long long>(kMaxRows));
    return fail(B200ATTN_ERR_UNSUPPORTED, buf);
  }
  int rc;
  if ((rc = check_operand("q", a->q, a->batch, a->heads, a->len_q)) != 0) return rc;
  if ((rc = check_operand("k", a->k, a->batch, a->heads, a->len_kv)) != 0) return rc;
  if ((rc = check_operand("v", a->v, a->batch, a->heads, a->len_kv)) != 0) return rc;
  if ((rc = check_operand("o", a->o, a->batch, a->heads, a->len_q)) != 0) return rc;
  if (!(a->softmax_scale == a->softmax_scale) || std::isinf(a->softmax_scale))
    return fail(B200ATTN_ERR_INVALID_ARGUMENT, "softmax_scale must be finite");

  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return fail_cuda("cudaGetDevice", e);
  if (device < 0 || device >= kMaxDevices) return fail(B200ATTN_ERR_UNSUPPORTED, "device index too large");
  NoAllocDevice* st = &g_dev[device];
  std::call_once(st->once, setup_device, device, st);
  if (st->init_status != B200ATTN_OK) return fail(st->init_status, st->init_error);

  float* part_o = st->scratch;
  float* part_lse = st->scratch + kPartialOFloats;
  int32_t* status = reinterpret_cast<int32_t*>(st->scratch + kPartialOFloats + kPartialLseFloats);
  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);

  if (kv_splits == 0) {
    // Report what earlier calls left in the watchdog record. This is the one place the entry point
    // waits for the GPU, so it is never done on a stream that is being captured (querying or
    // synchronising such a stream would invalidate the capture).
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    if ((e = cudaStreamIsCapturing(stream, &capture)) != cudaSuccess) return fail_cuda("cudaStreamIsCapturing", e);
    if (capture != cudaStreamCaptureStatusNone)
      return fail(B200ATTN_ERR_INVALID_ARGUMENT,
                  "kv_splits == 0 reads the watchdog record back and cannot run on a capturing stream");
    int32_t rec[kStatusInts] = {0};
    e = cudaMemcpyAsync(rec, status, sizeof rec, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return fail_cuda("watchdog read-back", e);
    if (rec[0] != kDevOk) {
      e = cudaMemsetAsync(status, 0, kStatusInts * sizeof(int32_t), stream);
      if (e != cudaSuccess) return fail_cuda("watchdog clear", e);
      char buf[200];
      snprintf(buf, sizeof buf,
               "an earlier no-allocation call left early: code %d, site %d, block %d, warp %d, item %d, tile %d",
               rec[0], rec[1], rec[2], rec[3], rec[5], rec[6]);
      return fail(rec[0] == kDevWaitTimeout ? B200ATTN_ERR_DEVICE_TIMEOUT : B200ATTN_ERR_DEVICE_FAULT, buf);
    }
    return B200ATTN_OK;
  }

  // K/V chunks of whole tiles, as even as possible.
  const int32_t tiles = (a->len_kv + kBlockN - 1) / kBlockN;
  const int32_t tiles_per_chunk = (tiles + kv_splits - 1) / kv_splits;
  const int32_t chunk_keys = tiles_per_chunk * kBlockN;
  const int32_t chunks = (a->len_kv + chunk_keys - 1) / chunk_keys;

  FwdParams p;
  memset(&p, 0, sizeof p);
  p.o = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(a->o.ptr));
  p.lse = a->lse;
  p.o_stride_b = a->o.stride_batch;
  p.o_stride_h = a->o.stride_head;
  p.o_stride_l = a->o.stride_row;
  p.batch = a->batch;
  p.heads = a->heads;
  p.len_q = a->len_q;
  p.m_blocks = (a->len_q + kItemRows - 1) / kItemRows;
  p.total_items = int32_t(int64_t(a->batch) * a->heads * p.m_blocks);
  p.kv_group = 1;
  const float scale = a->softmax_scale > 0.0f ? a->softmax_scale : 1.0f / std::sqrt(float(kHeadDim));
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  p.wait_limit_ms = g_wait_limit_ms.load(std::memory_order_relaxed);

  CUtensorMap tq;
  const MapKey kq{a->q.ptr, a->q.stride_batch, a->q.stride_head, a->q.stride_row, a->batch, a->heads, a->len_q, device};
  if ((rc = make_tensor_map(kq, &tq)) != 0) return rc;

  for (int32_t c = 0; c < chunks; ++c) {
    const int32_t key0 = c * chunk_keys;
    const int32_t keys = (a->len_kv - key0 < chunk_keys) ? a->len_kv - key0 : chunk_keys;
    const char* kptr = static_cast<const char*>(a->k.ptr) + int64_t(key0) * a->k.stride_row * 2;
    const char* vptr = static_cast<const char*>(a->v.ptr) + int64_t(key0) * a->v.stride_row * 2;
    CUtensorMap tk, tv;
    const MapKey kk{kptr, a->k.stride_batch, a->k.stride_head, a->k.stride_row, a->batch, a->heads, keys, device};
    const MapKey kv{vptr, a->v.stride_batch, a->v.stride_head, a->v.stride_row, a->batch, a->heads, keys, device};
    if ((rc = make_tensor_map(kk, &tk)) != 0) return rc;
    if ((rc = make_tensor_map(kv, &tv)) != 0) return rc;
    p.len_kv = keys;
    p.kv_tiles = (keys + kBlockN - 1) / kBlockN;
    p.partial.o = chunks > 1 ? part_o : nullptr;
    p.partial.lse = chunks > 1 ? part_lse : nullptr;
    p.partial.merge = c > 0;
    p.partial.emit = c + 1 < chunks;
    e = launch_fwd_ws(tq, tk, tv, p, st->sm_count, stream);
    if (e != cudaSuccess) return fail_cuda("kernel launch", e);
    g_launches.fetch_add(1, std::memory_order_relaxed);
  }
  return B200ATTN_OK;
}
