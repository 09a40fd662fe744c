// Inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (TMEM alloc / mma / ld / st / commit).
// Every wait is bounded: a wait that runs out returns false and the caller records a status code and drains.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <math_constants.h>

namespace dm {

// ------------------------------------------------------------------------------------------------ generic helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.release.cta.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 100000;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking phase test: about 20 cycles when the phase is complete, against about 50 for try_wait with a time hint.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// 16-byte load from shared memory through the shared window (pointers derived from the dynamic shared-memory base by
// integer arithmetic are generic to the compiler, which would emit generic loads for them).
__device__ __forceinline__ float4 lds_f4(uint32_t saddr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(saddr));
  return v;
}
__device__ __forceinline__ float4 lds_f4(const float* p) { return lds_f4(smem_u32(p)); }
__device__ __forceinline__ float lds_f(uint32_t saddr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(saddr));
  return v;
}
__device__ __forceinline__ void sts_f(uint32_t saddr, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(saddr), "f"(v) : "memory");
}
__device__ __forceinline__ void sts_u4(uint32_t saddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void sts_u4(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  sts_u4(smem_u32(p), a, b, c, d);
}
// ------------------------------------------------------------------------------------------------ fences
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ------------------------------------------------------------------------------------------------ TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tiled load: coordinates (x = innermost, y).  x * elemsize must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// 2-D tiled store shared -> global (bulk async group of the issuing thread).  The writers of the shared tile fence it
// for the async proxy (fence_async_smem) before they signal the issuing thread.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until at most N of this thread's bulk groups still read their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Wait until at most N of this thread's bulk groups are incomplete (their global writes done).
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// 1-D bulk copy global -> shared: both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
               "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// ------------------------------------------------------------------------------------------------ TMEM
// Allocation: one warp, all lanes; the base address lands in shared memory.
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 columns: thread t of the warp reads lane (base lane + t), 32 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(a), "r"(b), "r"(c),
               "r"(d)
               : "memory");
}

// ------------------------------------------------------------------------------------------------ descriptors
// Shared-memory matrix descriptor of a 128-byte-swizzled tile whose rows are 128 bytes wide (row r at byte r * 128 of a
// 1024-byte aligned tile, 16-byte chunks XOR-swizzled with r % 8: exactly what a TMA box of 128 inner bytes with
// CU_TENSOR_MAP_SWIZZLE_128B writes).  The same bytes serve both majors:
//   K-major  (rows = M/N index, the 128 bytes = contraction): step k of 32 bytes = start + 32 * k
//   MN-major (rows = contraction index, the 128 bytes = M/N): step k of 32 rows  = start + 4096 * k
// sbo = byte distance between 8-row groups (1024); lbo = byte distance between 128-byte column blocks of an MN-major
// operand wider than 128 (ignored otherwise).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;   // descriptor version of sm_100
  d |= static_cast<uint64_t>(2) << 61;   // 128-byte swizzle
  return d;
}

// Instruction descriptor, kind::f8f6f4, e4m3 x e4m3 -> fp32.  a_mn / b_mn: operand is MN-major (else K-major).
__host__ __device__ constexpr uint32_t idesc_f8(int M, int N, bool a_mn, bool b_mn) {
  return (1u << 4)                                  // D format fp32
         | (0u << 7) | (0u << 10)                   // A, B = e4m3
         | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16)
         | (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}
// Block-scaled kind::mxf8f6f4 with UE8M0 scale bytes: byte a_id of the SFA word and b_id of the SFB word.
__host__ __device__ constexpr uint32_t idesc_mxf8(int M, int N, bool a_mn, bool b_mn, int a_id, int b_id) {
  return (static_cast<uint32_t>(b_id & 3) << 4) | (0u << 7) | (0u << 10)
         | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16)
         | (static_cast<uint32_t>(N >> 3) << 17) | (1u << 23)
         | (static_cast<uint32_t>(M >> 4) << 24) | (static_cast<uint32_t>(a_id & 3) << 29);
}

// ------------------------------------------------------------------------------------------------ MMA issue (one thread)
// The issuing thread is alone in its warp, so every instruction between two MMAs is exposed latency.  The 64-bit
// shared-memory descriptors are therefore kept as a constant high word (kDescHi: 1024-byte group stride, version 1,
// 128-byte swizzle) and a 32-bit low word (start address >> 4 plus the 16-byte leading offset field) that advances by a
// compile-time constant per step: (bytes >> 4) for a K-major 32-byte step is 2, for an MN-major 32-row step 256.
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr) { return ((saddr & 0x3FFFFu) >> 4) | (1u << 16); }

template <bool kAcc>
__device__ __forceinline__ void mma_f8_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "n"(kAcc ? 1 : 0), "r"(kDescHi)
      : "memory");
}
__device__ __forceinline__ void mma_f8_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, bool acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(acc ? 1u : 0u), "r"(kDescHi)
      : "memory");
}
__device__ __forceinline__ void mma_f8_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc, bool acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], db, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(acc ? 1u : 0u), "r"(kDescHi)
      : "memory");
}
__device__ __forceinline__ void mma_mxf8_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                            uint32_t sfa_tmem, uint32_t sfb_tmem, bool acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 da, {%1, %7};\n\tmov.b64 db, {%2, %7};\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], da, db, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(acc ? 1u : 0u), "r"(kDescHi)
      : "memory");
}
__device__ __forceinline__ void mma_mxf8_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                            uint32_t sfa_tmem, uint32_t sfb_tmem, bool acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 db, {%2, %7};\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], [%1], db, %3, [%4], [%5], p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(acc ? 1u : 0u), "r"(kDescHi)
      : "memory");
}

// ------------------------------------------------------------------------------------------------ numerics helpers
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2_approx(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Two fp32 -> two e4m3 codes (RNE, saturating): lo in bits 0-7, hi in bits 8-15.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t cvt_e4m3x4(float a, float b, float c, float d) {
  uint32_t w;
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
      "mov.b32 %0, {lo, hi};\n\t}"
      : "=r"(w)
      : "f"(a), "f"(b), "f"(c), "f"(d));
  return w;
}

// ------------------------------------------------------------------------------------------------ packed fp32 pairs
// sm_100 executes fma / mul / add on two fp32 lanes per instruction (same rounding as the scalar forms), which halves
// the issue slots of the softmax arithmetic.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 splat2(float a) { return make_float2(a, a); }
__device__ __forceinline__ float2 ex2_2(float2 x) { return make_float2(ex2_approx(x.x), ex2_approx(x.y)); }
__device__ __forceinline__ float max3(float a, float b, float c) {
  float m;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(m) : "f"(a), "f"(b), "f"(c));
  return m;
}
// 2^x on the FMA and integer pipes for a part of the forward's exponentials (the MUFU pipe, 16 results per clock and SM,
// is the floor of the attention kernels; pass 0 and the backward kernels must produce one and the same P and therefore
// all use ex2.approx): round-to-nearest split x = n + f with f in [-0.5, 0.5] through the 1.5 * 2^23 trick,
// degree-5 polynomial for 2^f (2.4e-7 relative error in fp32, the accuracy of ex2.approx), n added to the exponent field.
// Arguments below -120 are clamped (the result, < 1e-36, is zero for every use here); arguments must stay below 120.
__device__ __forceinline__ float2 ex2_poly2(float2 x) {
  x = make_float2(fmaxf(x.x, -120.0f), fmaxf(x.y, -120.0f));
  const float2 big = splat2(12582912.0f);
  const float2 t = add2(x, big);
  const float2 n = add2(t, splat2(-12582912.0f));
  const float2 f = add2(x, make_float2(-n.x, -n.y));
  float2 q = fma2(f, splat2(0.0013390863314270973f), splat2(0.009676031768321991f));
  q = fma2(q, f, splat2(0.055503569543361664f));
  q = fma2(q, f, splat2(0.2402210682630539f));
  q = fma2(q, f, splat2(0.6931471824645996f));
  q = fma2(q, f, splat2(1.0000001192092896f));
  return make_float2(__uint_as_float(__float_as_uint(q.x) + (__float_as_uint(t.x) << 23)),
                     __uint_as_float(__float_as_uint(q.y) + (__float_as_uint(t.y) << 23)));
}
// max over 32 floats held as 16 pairs (exact, order-free)
__device__ __forceinline__ float max32(const float2 (&v)[16]) {
  float m0 = max3(v[0].x, v[0].y, v[1].x), m1 = max3(v[1].y, v[2].x, v[2].y);
  float m2 = max3(v[3].x, v[3].y, v[4].x), m3 = max3(v[4].y, v[5].x, v[5].y);
#pragma unroll
  for (int i = 6; i < 14; i += 4) {
    m0 = max3(m0, v[i].x, v[i].y);
    m1 = max3(m1, v[i + 1].x, v[i + 1].y);
    m2 = max3(m2, v[i + 2].x, v[i + 2].y);
    m3 = max3(m3, v[i + 3].x, v[i + 3].y);
  }
  m0 = max3(m0, v[14].x, v[14].y);
  m1 = max3(m1, v[15].x, v[15].y);
  return fmaxf(max3(m0, m1, m2), m3);
}
// 32 floats (16 pairs) times a common factor -> 8 words of four e4m3 codes
__device__ __forceinline__ void codes32(const float2 (&v)[16], float inv, uint32_t (&w)[8]) {
  const float2 i2 = make_float2(inv, inv);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float2 a = mul2(v[2 * i], i2), b = mul2(v[2 * i + 1], i2);
    w[i] = cvt_e4m3x4(a.x, a.y, b.x, b.y);
  }
}

}  // namespace dm
