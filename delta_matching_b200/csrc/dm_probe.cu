// One-tile tcgen05 building-block check: a 128 x 128 x (32 * nk) e4m3 product through exactly the operand paths the
// attention kernels use (TMA 128-byte-swizzled tiles as K-major or MN-major shared-memory operands, A from TMEM, plain
// kind::f8f6f4 and block-scaled kind::mxf8f6f4 with caller-supplied scale words).  Used by the unit tests to pin the
// descriptor encodings and the TMEM scale-word placement against a host matmul, and (skip_commit) to show what a bounded
// wait does when it runs out: every thread gives up after wait_limit_ns, one of them records the status code, nobody
// reads the accumulator, TMEM is freed and the kernel returns.
#include "dm_common.cuh"
#include "dm_kernels.h"
#include "dm_probe.h"

namespace dm {

__global__ void __launch_bounds__(128, 1)
probe_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const ProbeParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + 16384;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 32768);
  uint64_t* bar_load = bars + 0;
  uint64_t* bar_mma = bars + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 3);
  const int tid = threadIdx.x, warp = tid >> 5;

  if (tid == 0) {
    mbar_init(bar_load, 1);
    mbar_init(bar_mma, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  constexpr uint32_t kColD = 0, kColA = 128, kColSfa = 160, kColSfb = 164;

  if (tid == 0) {
    mbar_expect_tx(bar_load, 32768);
    tma_load_2d(sA, &tm_a, bar_load, 0, 0);
    tma_load_2d(sB, &tm_b, bar_load, 0, 0);
  }
  if (p.a_tmem) {
    // row t of A (K contiguous) -> TMEM lane t, 32 columns of 4 codes
    uint32_t r[32];
    const uint4* src = reinterpret_cast<const uint4*>(p.a_codes + static_cast<size_t>(tid) * 128);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint4 v = src[i];
      r[4 * i] = v.x; r[4 * i + 1] = v.y; r[4 * i + 2] = v.z; r[4 * i + 3] = v.w;
    }
    tmem_st32(tmem + lane_base + kColA, r);
  }
  if (p.scaled) {
    const uint32_t* a = p.sfa_words + tid * 4;
    const uint32_t* bw = p.sfb_words + tid * 4;
    tmem_st4(tmem + lane_base + kColSfa, a[0], a[1], a[2], a[3]);
    tmem_st4(tmem + lane_base + kColSfb, bw[0], bw[1], bw[2], bw[3]);
  }
  tmem_wait_st();
  tc_fence_before();
  __syncthreads();

  bool ok = true;
  if (tid == 0) {
    ok = wait_or_abort(bar_load, 0, abort_flag);
    if (ok) {
      tc_fence_after();
      for (int ks = 0; ks < p.nk; ++ks) {
        const uint32_t da = desc_lo(smem_u32(sA)) + (p.a_mn ? ks * 256 : ks * 2);
        const uint32_t db = desc_lo(smem_u32(sB)) + (p.b_mn ? ks * 256 : ks * 2);
        const bool acc = ks > 0;
        if (p.scaled) {
          const uint32_t id = idesc_mxf8(128, 128, p.a_mn != 0, p.b_mn != 0, ks, ks);
          if (p.a_tmem) mma_mxf8_ts(tmem + kColD, tmem + kColA + ks * 8, db, id, tmem + kColSfa, tmem + kColSfb, acc);
          else mma_mxf8_ss(tmem + kColD, da, db, id, tmem + kColSfa, tmem + kColSfb, acc);
        } else {
          const uint32_t id = idesc_f8(128, 128, p.a_mn != 0, p.b_mn != 0);
          if (p.a_tmem) mma_f8_ts(tmem + kColD, tmem + kColA + ks * 8, db, id, acc);
          else mma_f8_ss(tmem + kColD, da, db, id, acc);
        }
      }
      // skip_commit: the arrival everybody below waits for never comes, which makes their bounded wait run out
      if (!p.skip_commit) tc_commit(bar_mma);
    } else {
      raise_abort(abort_flag, p.status, kStatusTimeoutProbe);
    }
  }
  __syncwarp();
  ok = wait_or_abort(bar_mma, 0, abort_flag, p.wait_limit_ns != 0 ? p.wait_limit_ns : kWaitLimitNs);
  if (ok) {
    tc_fence_after();
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld32(tmem + lane_base + kColD + 32 * c, r);
      tmem_wait_ld();
      float* dst = p.out + static_cast<size_t>(tid) * 128 + 32 * c;
#pragma unroll
      for (int e = 0; e < 32; ++e) dst[e] = __uint_as_float(r[e]);
    }
  } else if (tid == 32) {
    raise_abort(abort_flag, p.status, kStatusTimeoutProbe);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

cudaError_t launch_probe(const CUtensorMap& ta, const CUtensorMap& tb, const ProbeParams& p, cudaStream_t stream) {
  constexpr int kSmem = 32768 + 64 + 1024;
  cudaError_t e = cudaFuncSetAttribute(probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  if (e != cudaSuccess) return e;
  probe_kernel<<<1, 128, kSmem, stream>>>(ta, tb, p);
  count_launch();
  return cudaGetLastError();
}

}  // namespace dm
