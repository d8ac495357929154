// Thin inline-PTX wrappers for the sm_100a features the attention kernels use:
// mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (MMA, TMEM alloc / ld / st,
// commit, fences), packed f32x2 arithmetic and register re-partitioning.
//
// Every spin on an mbarrier in this library goes through WaitCtx::wait(), which
// gives up after a wall-clock limit, records where it gave up and lets the CTA
// leave cleanly (no unbounded device-side wait exists anywhere in the library).
#pragma once

#include <cstdint>
#include <cuda_runtime.h>
#include <cuda_bf16.h>

namespace b200attn {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ----------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(arrivals) : "memory");
}

__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}

// Arrival by the lane with lead != 0 only, by predication (no branch).
__device__ __forceinline__ void mbar_arrive_lead(uint32_t lead, uint32_t bar) {
  asm volatile(
      "{\n\t"
      ".reg .pred p_lead;\n\t"
      "setp.ne.u32 p_lead, %1, 0;\n\t"
      "@p_lead mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];\n\t"
      "}\n" ::"r"(bar),
      "r"(lead)
      : "memory");
}

// One poll; the hardware may suspend the thread for up to `hint_ns` before answering.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p_w;\n\t"
      "mbarrier.try_wait.parity.acquire.cta.shared::cta.b64 p_w, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p_w;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return done != 0;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
  return t;
}

// ----------------------------------------------------------------------------- proxies / fences
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
}

// ----------------------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];\n" ::"l"(tmap) : "memory");
}

// ----------------------------------------------------------------------------- TMEM management
// Whole-warp collectives. `ncols` is a power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                   smem_result),
               "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols)
               : "memory");
}

// ----------------------------------------------------------------------------- UMMA
// Shared-memory operand descriptor, SWIZZLE_128B, descriptor version 1 (Blackwell).
//   bits  0..13  start address >> 4
//   bits 16..29  leading-dimension byte offset >> 4
//   bits 32..45  stride-dimension byte offset >> 4
//   bits 46..47  version (1)
//   bits 61..63  layout type (2 = 128-byte swizzle)
// The kernels keep the two 32-bit halves apart (umma_desc_lo / umma_desc_hi_sw128 below): the
// high half is a compile-time constant and the low half is one add away from the tile base.

// Instruction descriptor for kind::f16, bf16 x bf16 -> fp32, A K-major.
//   bit 4: D is fp32; bit 7: A is bf16; bit 10: B is bf16; bit 16: B is MN-major;
//   bits 17..22: N / 8; bits 24..28: M / 16.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) |
         (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

// The kernels keep descriptors as two 32-bit halves: the high half is a compile-time constant
// per operand kind, the low half carries the address (and LBO) and is what changes per step.
__host__ __device__ constexpr uint32_t umma_desc_hi_sw128(uint32_t sbo_bytes) {
  return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
}
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t smem_addr, uint32_t lbo_bytes) {
  return ((smem_addr & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi,
                                        uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p_acc;\n\t"
      ".reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "setp.ne.u32 p_acc, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p_acc;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]   (A: packed bf16 pairs, one pair per 32-bit TMEM cell)
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                        uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p_acc;\n\t"
      ".reg .b64 db;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.u32 p_acc, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p_acc;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Warp-uniform issue: every lane of the warp executes these with identical operands and only the
// lane with `lead != 0` issues the instruction, so the surrounding control flow stays uniform.
__device__ __forceinline__ void umma_commit_lead(uint32_t lead, uint32_t bar) {
  asm volatile(
      "{\n\t"
      ".reg .pred p_lead;\n\t"
      "setp.ne.u32 p_lead, %1, 0;\n\t"
      "@p_lead tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
      "}\n" ::"r"(bar),
      "r"(lead)
      : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx_lead(uint32_t lead, uint32_t bar,
                                                           uint32_t bytes) {
  asm volatile(
      "{\n\t"
      ".reg .pred p_lead;\n\t"
      "setp.ne.u32 p_lead, %2, 0;\n\t"
      "@p_lead mbarrier.arrive.expect_tx.release.cta.shared::cta.b64 _, [%0], %1;\n\t"
      "}\n" ::"r"(bar),
      "r"(bytes), "r"(lead)
      : "memory");
}

// 4-D tiled load: coordinates are (innermost .. outermost) = (c0, c1, c2, c3).
// c0 * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_4d_lead(uint32_t lead, uint32_t dst_smem, const void* tmap,
                                                 int c0, int c1, int c2, int c3, uint32_t bar) {
  asm volatile(
      "{\n\t"
      ".reg .pred p_lead;\n\t"
      "setp.ne.u32 p_lead, %7, 0;\n\t"
      "@p_lead cp.async.bulk.tensor.4d.shared::cta.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4, %5}], [%6];\n\t"
      "}\n" ::"r"(dst_smem),
      "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar), "r"(lead)
      : "memory");
}

// The mbarrier receives one arrival once every MMA this thread issued so far has finished.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar)
      : "memory");
}

// ----------------------------------------------------------------------------- TMEM <-> registers
// 32x32b shape: lane i of the warp addresses TMEM lane (base_lane + i); each thread
// moves N consecutive 32-bit columns. Warp w of a 4-warp group may only touch TMEM
// lanes 32*(w%4) .. 32*(w%4)+31.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(
          taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
      "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
      "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
      "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
      "r"(r[15])
      : "memory");
}

__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}

// ----------------------------------------------------------------------------- register budget
template <int kRegs>
__device__ __forceinline__ void reg_grow() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(kRegs));
}

template <int kRegs>
__device__ __forceinline__ void reg_shrink() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(kRegs));
}

// ----------------------------------------------------------------------------- arithmetic
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}

// Packed pairs of fp32 in one 64-bit register.
struct f2 {
  uint64_t bits;
};

__device__ __forceinline__ f2 f2_make(float lo, float hi) {
  f2 r;
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(r.bits) : "f"(lo), "f"(hi));
  return r;
}

__device__ __forceinline__ f2 f2_splat(float v) { return f2_make(v, v); }

__device__ __forceinline__ void f2_split(f2 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(v.bits));
}

__device__ __forceinline__ f2 f2_fma(f2 a, f2 b, f2 c) {
  f2 r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(r.bits) : "l"(a.bits), "l"(b.bits), "l"(c.bits));
  return r;
}

__device__ __forceinline__ f2 f2_add(f2 a, f2 b) {
  f2 r;
  asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(r.bits) : "l"(a.bits), "l"(b.bits));
  return r;
}

// Two bf16 in one 32-bit word: `lo` in bits 0..15, `hi` in bits 16..31.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;\n" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

}  // namespace ptx
}  // namespace b200attn
