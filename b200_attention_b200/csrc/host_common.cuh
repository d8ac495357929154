// Host-side helpers shared by the translation units that implement the C ABI.
#pragma once

#include <atomic>
#include <cstdint>
#include <string>

#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/b200_attention.h"

namespace b200attn {
namespace host {

// Records `msg` as this thread's last error and returns `status`.
int fail(int status, const std::string& msg);
int fail_cuda(const char* what, cudaError_t e);

extern thread_local std::string g_last_error;
extern std::atomic<uint64_t> g_launches;       // kernels launched by this process
extern std::atomic<uint32_t> g_wait_limit_ms;  // limit of device-side waits

// Identity of one 4-D tensor map: (head_dim, row, head, batch) view of a bf16 operand.
struct MapKey {
  const void* ptr;
  int64_t sb, sh, sl;  // strides in elements: batch, head, row
  int32_t batch, heads, len;
  int32_t device;
};

// Returns the cached map for `key`, encoding it on a miss (host-only work, no device memory).
int make_tensor_map(const MapKey& key, CUtensorMap* out);

// Pointer / stride rules of one operand; reports through fail().
int check_operand(const char* name, const b200attn_operand& t, int32_t batch, int32_t heads,
                  int32_t len);

}  // namespace host
}  // namespace b200attn
