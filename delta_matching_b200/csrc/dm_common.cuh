// Shared definitions of the delta-matching B200 kernels: status codes, UE8M0 scale arithmetic, role abort protocol.
#pragma once
#include <stdint.h>
#include "dm_ptx.cuh"

namespace dm {

// Status word values a kernel may leave in its int* status argument (0 = no problem seen).  A non-zero value means a
// bounded wait ran out; the output of that launch is not valid.
enum : int {
  kStatusOk = 0,
  kStatusTimeoutProducer = 1,   // TMA producer gave up waiting for a free stage
  kStatusTimeoutMma = 2,        // MMA issuer gave up waiting for operands or for the compute warps
  kStatusTimeoutCompute = 3,    // compute warps gave up waiting for an accumulator
  kStatusTimeoutProbe = 4,
};

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// ---------------------------------------------------------------------------------------------- UE8M0 scale bytes
// Byte b <-> scale 2^(b - 127).  Follows delta_matching/sm100/fp8_e8m0_scale_sm100.py:48-124 (pow2_sb, add_sb_clamp,
// inv_pow2_from_sb) and the producers' rule in delta_matching/sm100/quant.py:160-176.
// Byte of the smallest power of two s with amax <= 448 * s; `zero_byte` is returned for amax == 0.
__device__ __forceinline__ uint32_t pow2_sb(float amax, uint32_t zero_byte) {
  uint32_t bits = __float_as_uint(amax);
  int eb = static_cast<int>((bits >> 23) & 0xFF) - 8 + ((bits & 0x7FFFFF) > 0x600000 ? 1 : 0);
  eb = max(1, min(eb, 254));
  return amax > 0.f ? static_cast<uint32_t>(eb) : zero_byte;
}
__device__ __forceinline__ float sb_to_scale(uint32_t b) { return __uint_as_float(b << 23); }          // 2^(b-127), b>=1
__device__ __forceinline__ float sb_to_inv(uint32_t b) { return __uint_as_float((254u - b) << 23); }   // 2^(127-b)
__device__ __forceinline__ uint32_t scale_to_sb(float s) { return (__float_as_uint(s) >> 23) & 0xFF; }
// Byte of the product of two power-of-two scales.
__device__ __forceinline__ uint32_t sb_mul(uint32_t a, uint32_t b) {
  int s = static_cast<int>(a) + static_cast<int>(b) - 127;
  return static_cast<uint32_t>(max(0, min(s, 254)));
}
__device__ __forceinline__ uint32_t pack4(uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3) {
  return b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
}

// (hi, lo) += x with the rounding error of the addition kept in lo (Knuth TwoSum; no fast-math reassociation is enabled).
__device__ __forceinline__ void two_sum_acc(float& hi, float& lo, float x) {
  const float s = __fadd_rn(hi, x);
  const float bb = __fsub_rn(s, hi);
  const float err = __fadd_rn(__fsub_rn(hi, __fsub_rn(s, bb)), __fsub_rn(x, bb));
  hi = s;
  lo = __fadd_rn(lo, err);
}

// ---------------------------------------------------------------------------------------------- persistent schedule
// Work items are numbered heaviest first.  Round k hands items k * n_ctas ... k * n_ctas + n_ctas - 1 to the CTAs in
// ascending CTA order when k is even and in descending order when k is odd, so that the totals of the CTAs stay close to
// each other (a CTA that got the heaviest item of one round gets the lightest of the next).  A CTA whose item of round k
// does not exist has no item in any later round either.
__device__ __forceinline__ int sched_item(int k, int cta, int n_ctas) {
  return k * n_ctas + ((k & 1) ? (n_ctas - 1 - cta) : cta);
}

// ---------------------------------------------------------------------------------------------- bounded waits
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Wait on an mbarrier phase for at most `limit_ns` of wall time (~2 s unless the caller passes its own limit), giving up
// early when another role of the CTA has already raised the abort flag.  Returns false on give-up; the caller records a
// status code, raises the flag and leaves its loop.
constexpr uint64_t kWaitLimitNs = 2000000000ull;
#ifndef DM_POLL_NS
#define DM_POLL_NS 40        // sleep between two polls of a phase that is not complete yet
#endif
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                              uint64_t limit_ns = kWaitLimitNs) {
  if (mbar_test_wait(bar, parity)) return true;      // the common case in a pipeline that runs ahead: already complete
  if (mbar_try_wait(bar, parity)) return true;
  // A waiting warp must not eat the issue slots of the warps it waits for: after a few immediate retries it sleeps
  // between polls, and it looks at the abort flag and the clock only every 256 polls (every poll under a short limit).
#pragma unroll 1
  for (int i = 0; i < 4; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  const uint64_t t0 = global_ns();
  const uint32_t check_mask = (limit_ns < 100000000ull) ? 0u : 255u;
#pragma unroll 1
  for (uint32_t spins = 1;; ++spins) {
    __nanosleep(DM_POLL_NS);
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & check_mask) == 0u) {
      if (*abort_flag != 0) return false;
      if (global_ns() - t0 > limit_ns) return false;
    }
  }
}
// Whole-warp form for the compute warps: every lane polls, the verdict is made uniform so that the warp-wide tcgen05.ld /
// tcgen05.st that follow are never executed by a part of the warp.
__device__ __forceinline__ bool wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (__all_sync(0xffffffffu, mbar_test_wait(bar, parity) ? 1 : 0) != 0) return true;   // ~30 cycles when complete
  return __all_sync(0xffffffffu, wait_or_abort(bar, parity, abort_flag) ? 1 : 0) != 0;
}
// The status word may live in pinned host memory that the GPU writes directly (the host then sees a give-up without a
// copy): a plain store of the first code seen, no atomic; two roles racing here both hold a non-zero code.
__device__ __forceinline__ void raise_abort(volatile int* abort_flag, int* status, int code) {
  *abort_flag = 1;
  if (status != nullptr) {
    volatile int* s = status;
    if (*s == 0) *s = code;
    __threadfence_system();
  }
}

// Producer side of a named barrier: count towards the barrier without waiting (the consumers call bar_sync with the
// same id and total thread count).
__device__ __forceinline__ void bar_arrive(int id, int nthreads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Named barrier for the compute warps (id 1..15; id 0 is __syncthreads).
__device__ __forceinline__ void bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

}  // namespace dm
