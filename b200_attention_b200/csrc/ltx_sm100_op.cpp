// Drop-in for the capstone's custom-op library: registers `torch.ops.ltx_sm100.attention`
// with the same schema, dispatch key and tensor contract as the reference binding
// (capstone-project/kernel/binding.cpp:27-110), backed by libb200attn.so. Point the
// reference loader's LTX_SM100_ATTENTION_LIB (capstone-project/src/ltx_sm100/build.py:147-184)
// at the built libltx_sm100_attention.so to use it without touching the capstone code.
//
// Differences, all relaxations: query length need not be a multiple of 256 and key/value
// length need not be a multiple of 128. The argument checks below restate the reference
// binding's own list (binding.cpp:31-76: device, dtype, rank, head dimension, matching batch and
// K/V shapes, contiguity, sizes within int), in its order and with its message texts, because
// callers of the op match on those messages.

#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <climits>

#include "../../include/b200_attention.h"

namespace {

at::Tensor attention(const at::Tensor& query, const at::Tensor& key, const at::Tensor& value) {
  const char* op = "ltx_sm100.attention";
  TORCH_CHECK(query.is_cuda() && key.is_cuda() && value.is_cuda(), op,
              " requires CUDA query/key/value tensors");
  TORCH_CHECK(query.device() == key.device() && query.device() == value.device(), op,
              " requires query/key/value on the same CUDA device");
  TORCH_CHECK(query.scalar_type() == at::kBFloat16 && key.scalar_type() == at::kBFloat16 &&
                  value.scalar_type() == at::kBFloat16,
              op, " requires BF16 query/key/value tensors");
  TORCH_CHECK(query.dim() == 3 && key.dim() == 3 && value.dim() == 3, op,
              " expects query/key/value shaped [BH, L, 128]");
  TORCH_CHECK(query.is_contiguous() && key.is_contiguous() && value.is_contiguous(), op,
              " requires contiguous query/key/value tensors");
  const int64_t bh = query.size(0), lq = query.size(1), lk = key.size(1);
  TORCH_CHECK(key.size(0) == bh && value.size(0) == bh, op,
              " requires matching query/key/value BH dimensions");
  TORCH_CHECK(key.size(2) == query.size(2) && value.size(2) == query.size(2), op,
              " requires matching query/key/value head dimensions");
  TORCH_CHECK(value.size(1) == lk, op, " requires matching key/value sequence lengths");
  TORCH_CHECK(query.size(2) == 128, op, " only supports head dimension 128");
  TORCH_CHECK(bh > 0 && lq > 0 && lk > 0, op, " dimensions must be non-zero");
  TORCH_CHECK(bh <= INT_MAX && lq <= INT_MAX && lk <= INT_MAX, op,
              " dimensions exceed launcher integer limits");

  c10::cuda::CUDAGuard guard(query.device());
  at::Tensor out = at::empty_like(query);
  void* stream = c10::cuda::getCurrentCUDAStream(query.get_device()).stream();
  const int rc = b200attn_bhld_launch(query.data_ptr(), key.data_ptr(), value.data_ptr(),
                                      out.data_ptr(), int(bh), int(lq), int(lk), stream);
  // B200ATTN_ERR_ARCH carries the "needs compute capability 10.0" message of the reference.
  TORCH_CHECK(rc == B200ATTN_OK, op, ": ", b200attn_status_string(rc), ": ", b200attn_last_error());
  return out;
}

}  // namespace

TORCH_LIBRARY(ltx_sm100, library) {
  library.def("attention(Tensor query, Tensor key, Tensor value) -> Tensor");
}

TORCH_LIBRARY_IMPL(ltx_sm100, CUDA, library) { library.impl("attention", &attention); }
