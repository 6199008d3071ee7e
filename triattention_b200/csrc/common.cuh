// Shared device helpers for the TriAttention B200 kernels: packed fp32x2 arithmetic,
// bf16 unpacking, bulk async copy (TMA 1-D) and bounded mbarrier waits.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/triattn_b200.h"

namespace triattn {

constexpr int kSMs = 148;  // B200

// ---------------------------------------------------------------- packed fp32x2 (sm_100)
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<uint64_t&>(a)), "l"(reinterpret_cast<uint64_t&>(b)),
        "l"(reinterpret_cast<uint64_t&>(c)));
  return d;
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  float2 d;
  asm("mul.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<uint64_t&>(a)), "l"(reinterpret_cast<uint64_t&>(b)));
  return d;
}
__device__ __forceinline__ float sqrt_approx(float x) {
  float r;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
// two bf16 packed in a 32-bit word -> (low element, high element) as fp32 (exact)
__device__ __forceinline__ float2 bf16x2_to_float2(uint32_t w) {
  return make_float2(__uint_as_float(__byte_perm(w, 0u, 0x1044u)), __uint_as_float(__byte_perm(w, 0u, 0x3244u)));
}
// |k|^2 of two frequencies at once: `re` and `im` hold the bf16 pairs (re_f, re_f') and (im_f, im_f').
// fma.rn.f32.bf16 multiplies two bf16 values exactly and accumulates in fp32, so the pairs need no unpacking
// (re*re is rounded once, im*im is fused into it - the same two roundings as an fp32 mul followed by an fma).
__device__ __forceinline__ float2 sq_mag_bf16x2(uint32_t re, uint32_t im) {
  float2 m;
  asm("{\n\t.reg .b16 rl, rh, il, ih;\n\t"
      "mov.b32 {rl, rh}, %2;\n\tmov.b32 {il, ih}, %3;\n\t"
      "fma.rn.f32.bf16 %0, rl, rl, 0f00000000;\n\tfma.rn.f32.bf16 %0, il, il, %0;\n\t"
      "fma.rn.f32.bf16 %1, rh, rh, 0f00000000;\n\tfma.rn.f32.bf16 %1, ih, ih, %1;\n\t}"
      : "=f"(m.x), "=f"(m.y)
      : "r"(re), "r"(im));
  return m;
}
// |k|^2 of ONE frequency whose (re, im) sit in the two halves of `w` (interleaved RoPE layout).
__device__ __forceinline__ float sq_mag_bf16_pair(uint32_t w) {
  float m;
  asm("{\n\t.reg .b16 r, i;\n\t"
      "mov.b32 {r, i}, %1;\n\t"
      "fma.rn.f32.bf16 %0, r, r, 0f00000000;\n\tfma.rn.f32.bf16 %0, i, i, %0;\n\t}"
      : "=f"(m)
      : "r"(w));
  return m;
}
// Split two non-negative fp32 values into bf16 pairs (hi, lo) with m = hi + lo + e, |e| <= 2^-18 m: hi is m rounded
// to nearest bf16 (one packed convert), the remainder m - hi is exact in fp32 and is formed by the mixed-precision
// FMA straight from the packed halves of hi (hi * -1 + m), lo is its bf16 rounding.  Four instructions per pair.
__device__ __forceinline__ void split_bf16x2_hi_lo(float m0, float m1, uint32_t& hi, uint32_t& lo) {
  asm("{\n\t.reg .b16 hl, hh, neg1;\n\t.reg .f32 r0, r1;\n\t"
      "cvt.rn.bf16x2.f32 %0, %3, %2;\n\t"
      "mov.b32 {hl, hh}, %0;\n\tmov.b16 neg1, 0xBF80;\n\t"
      "fma.rn.f32.bf16 r0, hl, neg1, %2;\n\tfma.rn.f32.bf16 r1, hh, neg1, %3;\n\t"
      "cvt.rn.bf16x2.f32 %1, r1, r0;\n\t}"
      : "=&r"(hi), "=r"(lo)
      : "f"(m0), "f"(m1));
}
__device__ __forceinline__ float2 fsub2(float2 a, float2 b) {
  float2 d;
  asm("sub.rn.f32x2 %0, %1, %2;"
      : "=l"(reinterpret_cast<uint64_t&>(d))
      : "l"(reinterpret_cast<uint64_t&>(a)), "l"(reinterpret_cast<uint64_t&>(b)));
  return d;
}
__device__ __forceinline__ float bf16_to_float(uint16_t h) { return __uint_as_float(((uint32_t)h) << 16); }

// ---------------------------------------------------------------- mbarrier + bulk copy
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// orders earlier generic-proxy accesses to shared memory before later async-proxy (bulk copy) writes
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t suspend_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(suspend_ns)
      : "memory");
  return ok != 0;
}
// Bounded wait: each poll may suspend the thread in hardware for up to kWaitSuspendNs (so a wait that is
// satisfied within that time costs one instruction); after kWaitLimit polls it gives up and reports failure
// instead of spinning forever (worst case about kWaitLimit * kWaitSuspendNs = 1 s).  A build with
// TRIATTN_TEST_SHORT_WAIT (tests only) gives up after about a millisecond and makes every barrier expect
// kTestExtraTxBytes more than is ever copied, so that the wait runs out after all real copies have landed.
constexpr uint32_t kWaitSuspendNs = 1u << 14;
#ifdef TRIATTN_TEST_SHORT_WAIT
constexpr uint32_t kWaitLimit = 1u << 6;
constexpr uint32_t kTestExtraTxBytes = 16u;
#else
constexpr uint32_t kWaitLimit = 1u << 16;
constexpr uint32_t kTestExtraTxBytes = 0u;
#endif
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait_hint(bar, parity, kWaitSuspendNs)) return true;
  for (uint32_t i = 1; i < kWaitLimit; ++i) {
    if (mbar_try_wait_hint(bar, parity, kWaitSuspendNs)) return true;
  }
  return false;
}
// Same, but also gives up as soon as `*abort_flag` (shared memory) is non-zero: once one warp of a CTA has
// timed out the stages it would have released are never refilled, and the others need not wait a second each.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, const volatile int* abort_flag) {
  if (mbar_try_wait_hint(bar, parity, kWaitSuspendNs)) return true;
  for (uint32_t i = 1; i < kWaitLimit; ++i) {
    if (*abort_flag != 0) return false;
    if (mbar_try_wait_hint(bar, parity, kWaitSuspendNs)) return true;
  }
  return false;
}
// "Last reader refills": the warps that read a shared-memory buffer count themselves out on an mbarrier whose
// expected count is the number of reader warps.  A warp that is done calls __syncwarp() (orders its lanes' reads
// before lane 0) and lane 0 arrives with release semantics.  The state an arrive returns describes the barrier
// BEFORE that arrive, so a pending count of 1 means this arrive completed the phase: that warp is the last
// reader.  Its test_wait on the completed phase (acquire) then orders every reader's loads before what follows:
// fence.proxy.async and the bulk copy that overwrites the buffer.  The barrier re-arms itself for the next round.
__device__ __forceinline__ uint64_t mbar_arrive_release(uint32_t bar) {
  uint64_t state;
  asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 %0, [%1];" : "=l"(state) : "r"(bar) : "memory");
  return state;
}
__device__ __forceinline__ uint32_t mbar_pending_count(uint64_t state) {
  uint32_t n;
  asm volatile("mbarrier.pending_count.b64 %0, %1;" : "=r"(n) : "l"(state));
  return n;
}
__device__ __forceinline__ bool mbar_test_wait_acquire(uint32_t bar, uint64_t state) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.acquire.cta.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "l"(state)
      : "memory");
  return ok != 0;
}
// true for exactly one caller per round: the reader whose arrive was the last of the round
__device__ __forceinline__ bool release_and_check_last(uint32_t empty_bar) {
  const uint64_t state = mbar_arrive_release(empty_bar);
  if (mbar_pending_count(state) != 1u) return false;
  mbar_test_wait_acquire(empty_bar, state);  // the phase this arrive completed: acquires the other readers' releases
  return true;
}

// ---------------------------------------------------------------- programmatic dependent launch
// A kernel launched with the programmatic-stream-serialization attribute may start while its predecessor in
// the stream is still running; it must call grid_dependency_wait() before it touches anything the predecessor
// wrote (the wait returns once the predecessor has completed and its memory is visible).  A predecessor calls
// trigger_dependents() once its CTA no longer needs the SM resources the successor competes for.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void trigger_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// 1-D bulk copy global -> this CTA's shared memory, completion counted in bytes on `bar`.
// Both addresses 16-byte aligned, bytes a multiple of 16.  No multicast.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// order-preserving map fp32 -> uint32 (larger float <=> larger key; +inf near the top)
__device__ __forceinline__ uint32_t float_to_ordered(float x) {
  uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ void flag_status(uint32_t* status, uint32_t bit) {
  if (status != nullptr) atomicOr(status, bit);
}

}  // namespace triattn
