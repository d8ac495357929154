// C ABI of libb200attn.so: argument checking, per-device set-up, tensor-map construction
// (cached), launch, and the device watchdog record. See include/b200_attention.h.

#include "../../include/b200_attention.h"
#include "attn_kernels.cuh"
#include "host_common.cuh"

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>

namespace b200attn {
namespace host {

thread_local std::string g_last_error;
std::atomic<uint64_t> g_launches{0};
std::atomic<uint32_t> g_wait_limit_ms{2000};

int fail(int status, const std::string& msg) {
  g_last_error = msg;
  return status;
}

int fail_cuda(const char* what, cudaError_t e) {
  // Clear the sticky-free error so a later call does not see it again.
  (void)cudaGetLastError();
  return fail(B200ATTN_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

}  // namespace host
}  // namespace b200attn

namespace {

using namespace b200attn;
using namespace b200attn::host;

constexpr int kMaxDevices = 64;
constexpr const char* kVersion = "b200attn 0.1 (sm_100a)";

// ---- driver entry point for tensor-map encoding (resolved at run time: no link against libcuda)
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// ---- per-device state
struct DeviceState {
  std::once_flag once;
  int init_status = B200ATTN_OK;
  std::string init_error;
  int sm_count = 0;
  int32_t* status_host = nullptr;  // pinned, mapped; the kernels write here only on trouble
  int32_t* status_dev = nullptr;
};
DeviceState g_dev[kMaxDevices];

void init_device(int device, DeviceState* st) {
  int major = 0, minor = 0;
  cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&st->sm_count, cudaDevAttrMultiProcessorCount, device);
  if (e != cudaSuccess) {
    st->init_status = B200ATTN_ERR_CUDA;
    st->init_error = std::string("device attribute query: ") + cudaGetErrorString(e);
    (void)cudaGetLastError();
    return;
  }
  if (major != 10 || minor != 0) {
    st->init_status = B200ATTN_ERR_ARCH;
    char buf[128];
    snprintf(buf, sizeof buf, "device %d has compute capability %d.%d; sm_100a (10.0) required",
             device, major, minor);
    st->init_error = buf;
    return;
  }
  e = prepare_kernels();
  if (e != cudaSuccess) {
    st->init_status = B200ATTN_ERR_CUDA;
    st->init_error = std::string("kernel attribute set-up: ") + cudaGetErrorString(e);
    (void)cudaGetLastError();
    return;
  }
  e = cudaHostAlloc(reinterpret_cast<void**>(&st->status_host), kStatusInts * sizeof(int32_t),
                    cudaHostAllocMapped | cudaHostAllocPortable);
  if (e == cudaSuccess) {
    memset(st->status_host, 0, kStatusInts * sizeof(int32_t));
    e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&st->status_dev), st->status_host, 0);
  }
  if (e != cudaSuccess) {
    st->init_status = B200ATTN_ERR_CUDA;
    st->init_error = std::string("status record allocation: ") + cudaGetErrorString(e);
    (void)cudaGetLastError();
  }
}

int get_device(int* device_out, DeviceState** st_out) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return fail_cuda("cudaGetDevice", e);
  if (device < 0 || device >= kMaxDevices) return fail(B200ATTN_ERR_UNSUPPORTED, "device index too large");
  DeviceState* st = &g_dev[device];
  std::call_once(st->once, init_device, device, st);
  if (st->init_status != B200ATTN_OK) return fail(st->init_status, st->init_error);
  *device_out = device;
  *st_out = st;
  return B200ATTN_OK;
}

}  // namespace

namespace b200attn {
namespace host {

// ---- tensor maps
static bool same_key(const MapKey& a, const MapKey& o) {
  return a.ptr == o.ptr && a.sb == o.sb && a.sh == o.sh && a.sl == o.sl && a.batch == o.batch &&
         a.heads == o.heads && a.len == o.len && a.device == o.device;
}

struct MapCache {
  static constexpr int kSlots = 96;
  std::mutex mu;
  MapKey keys[kSlots];
  CUtensorMap maps[kSlots];
  int used = 0, next = 0;
};
MapCache g_maps;

// 4-D view (head_dim, row, head, batch) of one bf16 operand; box = 64 x 128 x 1 x 1 with the
// 128-byte swizzle, out-of-range rows read as zero.
int make_tensor_map(const MapKey& key, CUtensorMap* out) {
  {
    std::lock_guard<std::mutex> lock(g_maps.mu);
    for (int i = 0; i < g_maps.used; ++i) {
      if (same_key(g_maps.keys[i], key)) {
        *out = g_maps.maps[i];
        return B200ATTN_OK;
      }
    }
  }
  EncodeTiledFn enc = encode_fn();
  if (enc == nullptr) return fail(B200ATTN_ERR_DRIVER, "cuTensorMapEncodeTiled entry point not available");
  // A size-1 axis may come with any stride; give TMA a legal one.
  auto legal = [](int64_t stride, int32_t extent) -> cuuint64_t {
    return cuuint64_t((extent == 1 && stride <= 0) ? kHeadDim : stride) * 2u;
  };
  const cuuint64_t dims[4] = {cuuint64_t(kHeadDim), cuuint64_t(key.len), cuuint64_t(key.heads),
                              cuuint64_t(key.batch)};
  const cuuint64_t strides[3] = {legal(key.sl, key.len), legal(key.sh, key.heads),
                                 legal(key.sb, key.batch)};
  const cuuint32_t box[4] = {64, cuuint32_t(kBlockN), 1, 1};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  CUtensorMap map;
  const CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(key.ptr), dims,
                         strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[160];
    snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed with CUresult %d (len %d heads %d batch %d)",
             int(r), key.len, key.heads, key.batch);
    return fail(B200ATTN_ERR_DRIVER, buf);
  }
  {
    std::lock_guard<std::mutex> lock(g_maps.mu);
    const int slot = g_maps.used < MapCache::kSlots ? g_maps.used++ : (g_maps.next++ % MapCache::kSlots);
    g_maps.keys[slot] = key;
    g_maps.maps[slot] = map;
  }
  *out = map;
  return B200ATTN_OK;
}

int check_operand(const char* name, const b200attn_operand& t, int32_t batch, int32_t heads,
                  int32_t len) {
  if (t.ptr == nullptr) return fail(B200ATTN_ERR_INVALID_ARGUMENT, std::string(name) + ": null pointer");
  if ((reinterpret_cast<uintptr_t>(t.ptr) & 15u) != 0)
    return fail(B200ATTN_ERR_INVALID_ARGUMENT, std::string(name) + ": pointer must be 16-byte aligned");
  const int64_t s[3] = {t.stride_batch, t.stride_head, t.stride_row};
  const int32_t ext[3] = {batch, heads, len};
  for (int i = 0; i < 3; ++i) {
    if (ext[i] == 1 && s[i] <= 0) continue;
    if (s[i] < kHeadDim || (s[i] % 8) != 0 || s[i] >= (int64_t(1) << 38))
      return fail(B200ATTN_ERR_INVALID_ARGUMENT,
                  std::string(name) + ": strides must be >= 128, multiples of 8 elements and < 2^38");
  }
  return B200ATTN_OK;
}

}  // namespace host
}  // namespace b200attn

// One block per SM (more or less): each writes its SM's cycle counter and the global timer.
__global__ void sample_sm_clocks_kernel(long long* out, int max_sms) {
  if (threadIdx.x != 0) return;
  uint32_t smid;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
  if (int(smid) >= max_sms) return;
  unsigned long long timer;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(timer));
  out[2 * smid] = clock64();
  out[2 * smid + 1] = static_cast<long long>(timer);
}

#if defined(B200ATTN_TRACE) || defined(B200ATTN_PROFILE)
// Timeline studies only (never compiled into the shipped library): where block 0 records clock64.
static long long* g_trace_buffer = nullptr;
extern "C" B200ATTN_API void b200attn_debug_set_trace(void* device_buffer) {
  g_trace_buffer = static_cast<long long*>(device_buffer);
}
#endif

extern "C" {

int b200attn_forward(const b200attn_forward_args* a) {
  if (a == nullptr) return fail(B200ATTN_ERR_INVALID_ARGUMENT, "args is null");
  if (a->struct_bytes != sizeof(b200attn_forward_args))
    return fail(B200ATTN_ERR_INVALID_ARGUMENT, "struct_bytes does not match this library's b200attn_forward_args");
  if (a->head_dim != kHeadDim) return fail(B200ATTN_ERR_UNSUPPORTED, "head_dim must be 128");
  if (a->batch < 1 || a->heads < 1 || a->len_q < 1 || a->len_kv < 1)
    return fail(B200ATTN_ERR_INVALID_ARGUMENT, "batch, heads, len_q and len_kv must be positive");
  if (a->kernel != B200ATTN_KERNEL_WARP_SPECIALIZED && a->kernel != B200ATTN_KERNEL_SERIAL)
    return fail(B200ATTN_ERR_INVALID_ARGUMENT, "unknown kernel selector");
  if (int64_t(a->batch) * a->heads > 65535 * 16)
    return fail(B200ATTN_ERR_UNSUPPORTED, "batch * heads too large");
  const int heads_kv = a->heads_kv > 0 ? a->heads_kv : a->heads;
  if (a->heads_kv < 0 || a->heads % heads_kv != 0)
    return fail(B200ATTN_ERR_INVALID_ARGUMENT, "heads must be a positive multiple of heads_kv");
  if (a->causal != 0 && a->len_kv < a->len_q)
    return fail(B200ATTN_ERR_UNSUPPORTED,
                "causal attention needs len_kv >= len_q (the mask is aligned to the bottom-right corner)");
  if ((a->causal != 0 || heads_kv != a->heads) && a->kernel != B200ATTN_KERNEL_WARP_SPECIALIZED)
    return fail(B200ATTN_ERR_UNSUPPORTED, "causal masks and grouped K/V heads need the warp-specialised kernel");
  int rc;
  if ((rc = check_operand("q", a->q, a->batch, a->heads, a->len_q)) != 0) return rc;
  if ((rc = check_operand("k", a->k, a->batch, heads_kv, a->len_kv)) != 0) return rc;
  if ((rc = check_operand("v", a->v, a->batch, heads_kv, a->len_kv)) != 0) return rc;
  if ((rc = check_operand("o", a->o, a->batch, a->heads, a->len_q)) != 0) return rc;
  if ((a->partial_merge != 0 || a->partial_emit != 0) &&
      (a->partial_o == nullptr || a->partial_lse == nullptr))
    return fail(B200ATTN_ERR_INVALID_ARGUMENT, "partial_merge / partial_emit need partial_o and partial_lse");
  // The kernel derives the mask's diagonal from this call's own len_kv; a chain over K/V shards
  // would mask every shard as if it started at key 0.
  if (a->causal != 0 && (a->partial_merge != 0 || a->partial_emit != 0))
    return fail(B200ATTN_ERR_UNSUPPORTED, "a causal mask cannot be combined with partial_merge / partial_emit");
  if (a->partial_o != nullptr && (reinterpret_cast<uintptr_t>(a->partial_o) & 15u) != 0)
    return fail(B200ATTN_ERR_INVALID_ARGUMENT, "partial_o must be 16-byte aligned");
  if (!(a->softmax_scale == a->softmax_scale) || std::isinf(a->softmax_scale))
    return fail(B200ATTN_ERR_INVALID_ARGUMENT, "softmax_scale must be finite");

  int device = 0;
  DeviceState* st = nullptr;
  if ((rc = get_device(&device, &st)) != 0) return rc;

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
  p.len_kv = a->len_kv;
  p.m_blocks = (a->len_q + kItemRows - 1) / kItemRows;
  p.kv_tiles = (a->len_kv + kBlockN - 1) / kBlockN;
  const int64_t items = int64_t(a->batch) * a->heads * p.m_blocks;
  const int64_t serial_ctas = int64_t(a->batch) * a->heads * ((a->len_q + kBlockM - 1) / kBlockM);
  if (items >= (int64_t(1) << 30) || serial_ctas >= (int64_t(1) << 30))
    return fail(B200ATTN_ERR_UNSUPPORTED, "too many work items");
  p.total_items = int32_t(items);
  p.kv_group = a->heads / heads_kv;
  p.causal = a->causal != 0;
  p.causal_off = a->len_kv - a->len_q;
  const float scale = a->softmax_scale > 0.0f ? a->softmax_scale : 1.0f / std::sqrt(float(kHeadDim));
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = st->status_dev;
  p.wait_limit_ms = g_wait_limit_ms.load(std::memory_order_relaxed);
  p.partial.o = a->partial_o;
  p.partial.lse = a->partial_lse;
  p.partial.merge = a->partial_merge != 0;
  p.partial.emit = a->partial_emit != 0;
#if defined(B200ATTN_TRACE) || defined(B200ATTN_PROFILE)
  p.trace = g_trace_buffer;
#endif
  if (a->workspace != nullptr && a->kernel == B200ATTN_KERNEL_WARP_SPECIALIZED) {
    if ((reinterpret_cast<uintptr_t>(a->workspace) & 15u) != 0)
      return fail(B200ATTN_ERR_INVALID_ARGUMENT, "workspace must be 16-byte aligned");
    if (a->workspace_bytes < split_workspace_bytes(st->sm_count))
      return fail(B200ATTN_ERR_INVALID_ARGUMENT, "workspace is smaller than b200attn_workspace_bytes()");
    const SplitPlan plan = split_plan(p, st->sm_count);
    if (plan.grid > 0) {
      split_fill_cuts(p, st->sm_count, plan);
      p.split_scratch = static_cast<float*>(a->workspace);
      p.split_tickets = reinterpret_cast<int32_t*>(static_cast<char*>(a->workspace) +
                                                   size_t(st->sm_count) * 2 * kSplitSlotFloats * sizeof(float));
    }
  }

  CUtensorMap tq, tk, tv;
  const MapKey kq{a->q.ptr, a->q.stride_batch, a->q.stride_head, a->q.stride_row, a->batch, a->heads, a->len_q, device};
  const MapKey kk{a->k.ptr, a->k.stride_batch, a->k.stride_head, a->k.stride_row, a->batch, heads_kv, a->len_kv, device};
  const MapKey kv{a->v.ptr, a->v.stride_batch, a->v.stride_head, a->v.stride_row, a->batch, heads_kv, a->len_kv, device};
  if ((rc = make_tensor_map(kq, &tq)) != 0) return rc;
  if ((rc = make_tensor_map(kk, &tk)) != 0) return rc;
  if ((rc = make_tensor_map(kv, &tv)) != 0) return rc;

  cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
  const cudaError_t e = (a->kernel == B200ATTN_KERNEL_SERIAL)
                            ? launch_fwd_serial(tq, tk, tv, p, stream)
                            : launch_fwd_ws(tq, tk, tv, p, st->sm_count, stream);
  if (e != cudaSuccess) return fail_cuda("kernel launch", e);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return B200ATTN_OK;
}

int b200attn_workspace_bytes(uint64_t* bytes) {
  if (bytes == nullptr) return fail(B200ATTN_ERR_INVALID_ARGUMENT, "null argument");
  int device = 0;
  DeviceState* st = nullptr;
  const int rc = get_device(&device, &st);
  if (rc != 0) return rc;
  *bytes = split_workspace_bytes(st->sm_count);
  return B200ATTN_OK;
}

int b200attn_split_layout(int32_t work_items, int32_t kv_tiles, int32_t sm_count, int32_t* grid,
                          int32_t* runs, int32_t* cuts, int32_t max_cuts) {
  if (grid == nullptr || runs == nullptr || work_items < 1 || kv_tiles < 1 || sm_count < 1)
    return fail(B200ATTN_ERR_INVALID_ARGUMENT, "work_items, kv_tiles and sm_count must be positive, grid and runs non-null");
  FwdParams p;
  memset(&p, 0, sizeof p);
  p.total_items = work_items;
  p.kv_tiles = kv_tiles;
  const SplitPlan plan = split_plan(p, sm_count);
  *grid = plan.grid;
  *runs = 0;
  if (plan.grid == 0) return B200ATTN_OK;
  split_fill_cuts(p, sm_count, plan);
  *runs = p.split_runs;
  if (cuts != nullptr) {
    if (max_cuts < p.split_runs + 1) return fail(B200ATTN_ERR_INVALID_ARGUMENT, "cuts holds fewer than runs + 1 entries");
    memcpy(cuts, p.split_cut, sizeof(int32_t) * size_t(p.split_runs + 1));
  }
  return B200ATTN_OK;
}

int b200attn_bhld_launch(const void* q, const void* k, const void* v, void* o, int batch_heads,
                         int len_q, int len_kv, void* stream) {
  b200attn_forward_args a;
  memset(&a, 0, sizeof a);
  a.struct_bytes = sizeof a;
  a.batch = 1;
  a.heads = batch_heads;
  a.len_q = len_q;
  a.len_kv = len_kv;
  a.head_dim = kHeadDim;
  a.q = {q, 0, int64_t(len_q) * kHeadDim, kHeadDim};
  a.k = {k, 0, int64_t(len_kv) * kHeadDim, kHeadDim};
  a.v = {v, 0, int64_t(len_kv) * kHeadDim, kHeadDim};
  a.o = {o, 0, int64_t(len_q) * kHeadDim, kHeadDim};
  a.stream = stream;
  return b200attn_forward(&a);
}

int b200attn_bshd_launch(const void* q, const void* k, const void* v, void* o, int batch,
                         int heads, int len_q, int len_kv, void* stream) {
  b200attn_forward_args a;
  memset(&a, 0, sizeof a);
  a.struct_bytes = sizeof a;
  a.batch = batch;
  a.heads = heads;
  a.len_q = len_q;
  a.len_kv = len_kv;
  a.head_dim = kHeadDim;
  const int64_t row = int64_t(heads) * kHeadDim;
  a.q = {q, int64_t(len_q) * row, kHeadDim, row};
  a.k = {k, int64_t(len_kv) * row, kHeadDim, row};
  a.v = {v, int64_t(len_kv) * row, kHeadDim, row};
  a.o = {o, int64_t(len_q) * row, kHeadDim, row};
  a.stream = stream;
  return b200attn_forward(&a);
}

int b200attn_device_check(int device, int32_t record[8]) {
  if (device < 0) {
    const cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return fail_cuda("cudaGetDevice", e);
  }
  if (device >= kMaxDevices) return fail(B200ATTN_ERR_INVALID_ARGUMENT, "device index too large");
  DeviceState* st = &g_dev[device];
  if (st->status_host == nullptr) return B200ATTN_OK;  // nothing was ever launched there
  volatile int32_t* h = st->status_host;
  const int32_t code = h[0];
  if (code == kDevOk) return B200ATTN_OK;
  int32_t rec[kStatusInts];
  for (int i = 0; i < kStatusInts; ++i) rec[i] = h[i];
  if (record != nullptr) memcpy(record, rec, sizeof rec);
  for (int i = kStatusInts - 1; i >= 0; --i) h[i] = 0;
  char buf[200];
  snprintf(buf, sizeof buf,
           "device-side %s: site %d, block %d, warp %d, parity %d, item %d, tile %d",
           code == kDevWaitTimeout ? "wait timed out" : "self check failed", rec[1], rec[2], rec[3],
           rec[4], rec[5], rec[6]);
  return fail(code == kDevWaitTimeout ? B200ATTN_ERR_DEVICE_TIMEOUT : B200ATTN_ERR_DEVICE_FAULT, buf);
}

int b200attn_set_wait_limit_ms(uint32_t ms) {
  if (ms == 0 || ms > 60000) return fail(B200ATTN_ERR_INVALID_ARGUMENT, "wait limit must be in 1..60000 ms");
  g_wait_limit_ms.store(ms, std::memory_order_relaxed);
  return B200ATTN_OK;
}

uint64_t b200attn_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int b200attn_sample_sm_clocks(int64_t* out, int32_t max_sms, void* stream) {
  if (out == nullptr || max_sms < 1) return fail(B200ATTN_ERR_INVALID_ARGUMENT, "null buffer or max_sms < 1");
  int device = 0;
  DeviceState* st = nullptr;
  const int rc = get_device(&device, &st);
  if (rc != 0) return rc;
  // twice as many blocks as SMs, one warp each: every SM that is not completely full gets one
  sample_sm_clocks_kernel<<<2 * st->sm_count, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<long long*>(out), max_sms);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda("clock sample launch", e);
  return B200ATTN_OK;
}

int b200attn_ipc_export(const void* device_ptr, unsigned char handle[64], uint64_t* offset_bytes) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  if (device_ptr == nullptr || handle == nullptr || offset_bytes == nullptr)
    return fail(B200ATTN_ERR_INVALID_ARGUMENT, "null argument");
  // An IPC handle names a whole allocation: find its base and report where device_ptr sits in it.
  using RangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
  static RangeFn range_fn = []() -> RangeFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    return reinterpret_cast<RangeFn>(p);
  }();
  if (range_fn == nullptr) return fail(B200ATTN_ERR_DRIVER, "cuMemGetAddressRange entry point not available");
  CUdeviceptr base = 0;
  size_t size = 0;
  const CUresult r = range_fn(&base, &size, reinterpret_cast<CUdeviceptr>(device_ptr));
  if (r != CUDA_SUCCESS) return fail(B200ATTN_ERR_DRIVER, "cuMemGetAddressRange failed: not a device allocation?");
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base));
  if (e != cudaSuccess) return fail_cuda("cudaIpcGetMemHandle", e);
  memcpy(handle, &h, 64);
  *offset_bytes = uint64_t(reinterpret_cast<CUdeviceptr>(device_ptr) - base);
  return B200ATTN_OK;
}

int b200attn_ipc_open(const unsigned char handle[64], void** mapped_ptr) {
  if (handle == nullptr || mapped_ptr == nullptr) return fail(B200ATTN_ERR_INVALID_ARGUMENT, "null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  const cudaError_t e = cudaIpcOpenMemHandle(mapped_ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail_cuda("cudaIpcOpenMemHandle", e);
  return B200ATTN_OK;
}

int b200attn_ipc_close(void* mapped_ptr) {
  if (mapped_ptr == nullptr) return fail(B200ATTN_ERR_INVALID_ARGUMENT, "null argument");
  const cudaError_t e = cudaIpcCloseMemHandle(mapped_ptr);
  if (e != cudaSuccess) return fail_cuda("cudaIpcCloseMemHandle", e);
  return B200ATTN_OK;
}

int b200attn_copy_async(void* dst_local, const void* src, uint64_t bytes, void* stream) {
  if (dst_local == nullptr || src == nullptr) return fail(B200ATTN_ERR_INVALID_ARGUMENT, "null argument");
  const cudaError_t e =
      cudaMemcpyAsync(dst_local, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail_cuda("cudaMemcpyAsync", e);
  return B200ATTN_OK;
}

const char* b200attn_status_string(int status) {
  switch (status) {
    case B200ATTN_OK: return "ok";
    case B200ATTN_ERR_INVALID_ARGUMENT: return "invalid argument";
    case B200ATTN_ERR_UNSUPPORTED: return "unsupported shape or size";
    case B200ATTN_ERR_ARCH: return "device is not sm_100 (compute capability 10.0)";
    case B200ATTN_ERR_CUDA: return "CUDA runtime error";
    case B200ATTN_ERR_DRIVER: return "CUDA driver / tensor-map error";
    case B200ATTN_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
    case B200ATTN_ERR_DEVICE_FAULT: return "device-side self check failed";
    default: return "unknown status";
  }
}

const char* b200attn_last_error(void) { return g_last_error.c_str(); }
const char* b200attn_version(void) { return kVersion; }

}  // extern "C"
