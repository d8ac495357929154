// Thin torch-op shim over the C ABI (include/b200_attention.h). PyTorch is used only for
// tensor plumbing: argument checks, output allocation, current stream and device guard.
//
// Ops registered in namespace `b200_attention_b200` mirror the generated glue of the reference
// benchmark registry (benchmarks/registry.py:258-356: checks, empty_like output, launch on the
// current stream, op name `sdpa`) and of its direct-BSHD benchmark
// (benchmarks/benchmark_bshd.py:139-214: contiguous [B, L, H, 128] in and out, no input copy).

#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <limits>
#include <tuple>

#include "../../include/b200_attention.h"

namespace {

void check_rc(int rc) {
  TORCH_CHECK(rc == B200ATTN_OK, "b200attn: ", b200attn_status_string(rc), ": ",
              b200attn_last_error());
}

void check_common(const at::Tensor& Q, const at::Tensor& K, const at::Tensor& V) {
  TORCH_CHECK(Q.is_cuda() && K.is_cuda() && V.is_cuda(), "Q, K, V must be CUDA tensors");
  TORCH_CHECK(Q.scalar_type() == at::kBFloat16 && K.scalar_type() == at::kBFloat16 &&
                  V.scalar_type() == at::kBFloat16,
              "Q, K, V must be bfloat16");
  TORCH_CHECK(Q.dim() == 4 && K.dim() == 4 && V.dim() == 4, "Q, K, V must be 4D tensors");
  TORCH_CHECK(Q.device() == K.device() && Q.device() == V.device(),
              "Q, K, V must be on the same device");
  TORCH_CHECK(K.sizes() == V.sizes(), "K and V must have the same shape");
}

b200attn_operand operand(const at::Tensor& t, bool bshd) {
  // strides in elements for (batch, head, row)
  if (bshd) return {t.data_ptr(), t.stride(0), t.stride(2), t.stride(1)};
  return {t.data_ptr(), t.stride(0), t.stride(1), t.stride(2)};
}

// Shared body: Q [B,H,Lq,128] (bhld) or [B,Lq,H,128] (bshd); returns (O, LSE or undefined).
std::tuple<at::Tensor, at::Tensor> run(const at::Tensor& Q_in, const at::Tensor& K_in,
                                       const at::Tensor& V_in, double scale, bool bshd,
                                       bool want_lse, int64_t kernel, bool causal = false) {
  check_common(Q_in, K_in, V_in);
  const int l_axis = bshd ? 1 : 2, h_axis = bshd ? 2 : 1;
  TORCH_CHECK(Q_in.size(0) == K_in.size(0), "Q and K/V must have the same batch size");
  TORCH_CHECK(K_in.size(h_axis) >= 1 && Q_in.size(h_axis) % K_in.size(h_axis) == 0,
              "the number of Q heads must be a multiple of the number of K/V heads");
  TORCH_CHECK(!causal || K_in.size(l_axis) >= Q_in.size(l_axis),
              "causal attention needs at least as many keys as queries (bottom-right aligned mask)");
  TORCH_CHECK(Q_in.size(3) == 128 && K_in.size(3) == 128, "head_dim must be 128");
  TORCH_CHECK(Q_in.size(l_axis) >= 1 && K_in.size(l_axis) >= 1, "sequence lengths must be positive");
  constexpr int64_t kMaxInt = std::numeric_limits<int>::max();
  TORCH_CHECK(Q_in.size(0) <= kMaxInt && Q_in.size(h_axis) <= kMaxInt &&
                  Q_in.size(l_axis) <= kMaxInt && K_in.size(l_axis) <= kMaxInt,
              "a dimension exceeds int range");

  c10::cuda::CUDAGuard guard(Q_in.device());
  at::Tensor Q = Q_in, K = K_in, V = V_in;
  if (bshd) {
    // direct-BSHD contract: no input copy
    TORCH_CHECK(Q.is_contiguous() && K.is_contiguous() && V.is_contiguous(),
                "BSHD inputs must be contiguous [B, L, H, 128]");
  } else {
    // the innermost axis must be dense; other axes may be strided (multiples of 8 elements)
    auto usable = [](const at::Tensor& t) {
      if (t.stride(3) != 1) return false;
      for (int d = 0; d < 3; ++d)
        if (t.size(d) > 1 && (t.stride(d) % 8 != 0 || t.stride(d) < 128)) return false;
      return (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15u) == 0;
    };
    if (!usable(Q)) Q = Q.contiguous();
    if (!usable(K)) K = K.contiguous();
    if (!usable(V)) V = V.contiguous();
  }
  at::Tensor O = at::empty(Q.sizes(), Q.options());  // contiguous in the input's axis order
  at::Tensor LSE;
  const int64_t B = Q.size(0), H = Q.size(h_axis), Lq = Q.size(l_axis), Lk = K.size(l_axis);
  if (want_lse) LSE = at::empty({B, H, Lq}, Q.options().dtype(at::kFloat));

  b200attn_forward_args a{};
  a.struct_bytes = sizeof a;
  a.batch = int(B);
  a.heads = int(H);
  a.len_q = int(Lq);
  a.len_kv = int(Lk);
  a.head_dim = 128;
  a.q = operand(Q, bshd);
  a.k = operand(K, bshd);
  a.v = operand(V, bshd);
  a.o = operand(O, bshd);
  a.lse = want_lse ? LSE.data_ptr<float>() : nullptr;
  a.softmax_scale = float(scale);
  a.kernel = int(kernel);
  a.causal = causal ? 1 : 0;
  a.heads_kv = int(K.size(h_axis));
  a.stream = c10::cuda::getCurrentCUDAStream(Q.device().index()).stream();
  check_rc(b200attn_forward(&a));
  return {O, LSE};
}

at::Tensor sdpa(const at::Tensor& Q, const at::Tensor& K, const at::Tensor& V) {
  return std::get<0>(run(Q, K, V, 0.0, /*bshd=*/false, /*want_lse=*/false, 0));
}

at::Tensor sdpa_bshd(const at::Tensor& Q, const at::Tensor& K, const at::Tensor& V) {
  return std::get<0>(run(Q, K, V, 0.0, /*bshd=*/true, /*want_lse=*/false, 0));
}

std::tuple<at::Tensor, at::Tensor> sdpa_lse(const at::Tensor& Q, const at::Tensor& K,
                                            const at::Tensor& V, double scale, bool bshd,
                                            int64_t kernel) {
  return run(Q, K, V, scale, bshd, /*want_lse=*/true, kernel);
}

// Causal attention with grouped K/V heads on token-major tensors, the call shape of the
// reference's research launcher (research/causal_gqa_2cta.cu:1131-1137): Q [B, Sq, Hq, 128],
// K, V [B, Skv, Hkv, 128], returns (O [B, Sq, Hq, 128], LSE [B, Hq, Sq]).
std::tuple<at::Tensor, at::Tensor> sdpa_causal_gqa(const at::Tensor& Q, const at::Tensor& K,
                                                   const at::Tensor& V, double scale) {
  return run(Q, K, V, scale, /*bshd=*/true, /*want_lse=*/true, 0, /*causal=*/true);
}

// Raises if a kernel launched earlier on the current device left early. The caller must have
// synchronised the stream it launched on.
void device_check() {
  int32_t rec[8];
  check_rc(b200attn_device_check(-1, rec));
}

}  // namespace

TORCH_LIBRARY(b200_attention_b200, m) {
  m.def("sdpa(Tensor Q, Tensor K, Tensor V) -> Tensor", &sdpa);
  m.def("sdpa_bshd(Tensor Q, Tensor K, Tensor V) -> Tensor", &sdpa_bshd);
  m.def("sdpa_lse(Tensor Q, Tensor K, Tensor V, float scale, bool bshd, int kernel) -> (Tensor, Tensor)",
        &sdpa_lse);
  m.def("sdpa_causal_gqa(Tensor Q, Tensor K, Tensor V, float scale) -> (Tensor, Tensor)", &sdpa_causal_gqa);
  m.def("device_check() -> ()", &device_check);
}
