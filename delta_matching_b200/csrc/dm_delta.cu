// Pass 0 of the backward: the matched delta.  For every query row, delta_i = sum_j P_ij dP_ij / sum_j P_ij with P and dP
// recomputed from the fp8 codes exactly as the backward recomputes them, so that rowsum(dS) = 0 holds at fp32 round-off.
//
// Arithmetic shared with the backward (delta_matching/sm100/attention_math_sm100.py:26-45; emulation
// delta_matching/reference.py:483, 491, 526-535):
//   c = (ks_b * qs) * log2e;  l2 = lse * log2e;  P = ex2(fma(S_acc, c, -l2));  a = vs_b * dos;  dP = dP_acc * a.
// Sums: four fp32 FMA chains of 8 elements per 32-key block, folded into fp64 per row (the power-of-two factor a is
// applied once per block, which is exact); one fp64 divide and one fp32 store per row.
//
// CTA = one 128-query tile of one (batch, query head); S = Q8 K8^T and dP = dO8 V8^T on tcgen05 (kind::f8f6f4) into
// two 128-column TMEM accumulators.  Warps 0-3 compute (thread t = TMEM lane t = query row t), warp 4 TMA, warp 5 MMA.
#include "dm_common.cuh"
#include "dm_kernels.h"

namespace dm {

template <int D>
struct DeltaCfg {
  static constexpr int kSub = D / 128;
  static constexpr int kTileBytes = 128 * D;
  static constexpr int kStages = 2;
  static constexpr int kTmemCols = 256;
  static constexpr int kColS = 0, kColDp = 128;
  static constexpr int kSmemQ = 0;
  static constexpr int kSmemDo = kTileBytes;
  static constexpr int kSmemK = 2 * kTileBytes;
  static constexpr int kSmemV = kSmemK + kStages * kTileBytes;
  static constexpr int kSmemBar = kSmemV + kStages * kTileBytes;
  static constexpr int kSmemBytes = kSmemBar + 256 + 1024;
};

template <int D>
__global__ void __launch_bounds__(192, (D == 128) ? 2 : 1)
delta_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
             const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do, const DeltaParams p) {
  using C = DeltaCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + C::kSmemQ;
  uint8_t* sDo = smem + C::kSmemDo;
  uint8_t* sK = smem + C::kSmemK;
  uint8_t* sV = smem + C::kSmemV;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kSmemBar);
  uint64_t* bar_q = bars + 0;
  uint64_t* bar_s = bars + 1;      // S and dP accumulators ready
  uint64_t* bar_c = bars + 2;      // compute warps have read them (128 arrivals)
  uint64_t* full = bars + 4;       // [kStages] K and V of the stage landed
  uint64_t* empty = bars + 6;      // [kStages]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 11);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int n_qt = p.N / 128;
  const int qt = n_qt - 1 - static_cast<int>(blockIdx.x);
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int bhk = b * p.Hk + h / (p.H / p.Hk);
  const int n_it = p.causal ? (qt + 1) : n_qt;

  if (tid == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_c, 128);
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 4) {
    if (elect_one()) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_do);
      mbar_expect_tx(bar_q, 2 * C::kTileBytes);
      for (int s = 0; s < C::kSub; ++s) {
        tma_load_2d(sQ + s * 16384, &tm_q, bar_q, s * 128, bh * p.N + qt * 128);
        tma_load_2d(sDo + s * 16384, &tm_do, bar_q, s * 128, bh * p.N + qt * 128);
      }
      for (int it = 0; it < n_it; ++it) {
        const int st = it % C::kStages;
        if (it >= C::kStages) {
          if (!wait_or_abort(empty + st, ((it / C::kStages) - 1) & 1, abort_flag)) {
            raise_abort(abort_flag, p.status, kStatusTimeoutProducer);
            break;
          }
        }
        const int row = bhk * p.N + it * 128;            // key tiles in ascending order
        mbar_expect_tx(full + st, 2 * C::kTileBytes);
        for (int s = 0; s < C::kSub; ++s) {
          tma_load_2d(sK + st * C::kTileBytes + s * 16384, &tm_k, full + st, s * 128, row);
          tma_load_2d(sV + st * C::kTileBytes + s * 16384, &tm_v, full + st, s * 128, row);
        }
      }
    }
  } else if (warp == 5) {
    if (elect_one()) {
      constexpr uint32_t kIdesc = idesc_f8(128, 128, false, false);
      bool ok = wait_or_abort(bar_q, 0, abort_flag);
      for (int it = 0; ok && it < n_it; ++it) {
        const int st = it % C::kStages;
        if (!(ok = wait_or_abort(full + st, (it / C::kStages) & 1, abort_flag))) break;
        if (it > 0 && !(ok = wait_or_abort(bar_c, (it - 1) & 1, abort_flag))) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < D / 32; ++ks) {
          const uint32_t off = (ks / 4) * 16384 + (ks % 4) * 32;
          mma_f8_ss(tmem + C::kColS, smem_desc_sw128(smem_u32(sQ) + off, 16, 1024),
                    smem_desc_sw128(smem_u32(sK + st * C::kTileBytes) + off, 16, 1024), kIdesc, ks > 0);
        }
#pragma unroll
        for (int ks = 0; ks < D / 32; ++ks) {
          const uint32_t off = (ks / 4) * 16384 + (ks % 4) * 32;
          mma_f8_ss(tmem + C::kColDp, smem_desc_sw128(smem_u32(sDo) + off, 16, 1024),
                    smem_desc_sw128(smem_u32(sV + st * C::kTileBytes) + off, 16, 1024), kIdesc, ks > 0);
        }
        tc_commit(empty + st);
        tc_commit(bar_s);
      }
      if (!ok) raise_abort(abort_flag, p.status, kStatusTimeoutMma);
    }
  } else {
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const int row = qt * 128 + tid;
    const int nblk = p.N / 32;
    const float qs = p.qs[static_cast<size_t>(bh) * nblk + row / 32];
    const float dos = p.dos[static_cast<size_t>(bh) * nblk + row / 32];
    const float neg_l2 = -(p.lse[static_cast<size_t>(bh) * p.N + row] * kLog2e);
    double num = 0.0, den = 0.0;
    bool ok = true;
    const float* ks_base = p.ks + static_cast<size_t>(bhk) * nblk;
    const float* vs_base = p.vs + static_cast<size_t>(bhk) * nblk;
    float4 ks4 = *reinterpret_cast<const float4*>(ks_base);
    float4 vs4 = *reinterpret_cast<const float4*>(vs_base);
    const float2 nl2 = splat2(neg_l2);
    for (int it = 0; it < n_it; ++it) {
      const float cb[4] = {(ks4.x * qs) * kLog2e, (ks4.y * qs) * kLog2e, (ks4.z * qs) * kLog2e, (ks4.w * qs) * kLog2e};
      // a = vs * dos is a power of two, so P * (dP_acc * a) == (P * dP_acc) * a exactly: a is applied once per block
      const double ab[4] = {static_cast<double>(vs4.x * dos), static_cast<double>(vs4.y * dos),
                            static_cast<double>(vs4.z * dos), static_cast<double>(vs4.w * dos)};
      if (it + 1 < n_it) {
        ks4 = *reinterpret_cast<const float4*>(ks_base + (it + 1) * 4);
        vs4 = *reinterpret_cast<const float4*>(vs_base + (it + 1) * 4);
      }
      const bool diag = p.causal && (it == qt);
      if (!(ok = wait_warp(bar_s, it & 1, abort_flag))) break;
      tc_fence_after();
      uint32_t rs[2][32], rd[2][32];
      tmem_ld32(tmem + lane_base + C::kColS, rs[0]);
      tmem_ld32(tmem + lane_base + C::kColDp, rd[0]);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        tmem_wait_ld();
        if (c < 3) {
          tmem_ld32(tmem + lane_base + C::kColS + 32 * (c + 1), rs[(c + 1) & 1]);
          tmem_ld32(tmem + lane_base + C::kColDp + 32 * (c + 1), rd[(c + 1) & 1]);
        }
        uint32_t(&s)[32] = rs[c & 1];
        const uint32_t(&dp)[32] = rd[c & 1];
        if (diag) {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (32 * c + e > tid) s[e] = 0xff800000u;
        }
        const float2 c2 = splat2(cb[c]);
        float2 n0 = make_float2(0.f, 0.f), n1 = n0, d0 = n0, d1 = n0;
#pragma unroll
        for (int e = 0; e < 16; e += 2) {
          const float2 p0 = ex2_2(fma2(make_float2(__uint_as_float(s[2 * e]), __uint_as_float(s[2 * e + 1])), c2, nl2));
          const float2 p1 = ex2_2(fma2(make_float2(__uint_as_float(s[2 * e + 2]), __uint_as_float(s[2 * e + 3])), c2, nl2));
          n0 = fma2(p0, make_float2(__uint_as_float(dp[2 * e]), __uint_as_float(dp[2 * e + 1])), n0);
          n1 = fma2(p1, make_float2(__uint_as_float(dp[2 * e + 2]), __uint_as_float(dp[2 * e + 3])), n1);
          d0 = add2(d0, p0);
          d1 = add2(d1, p1);
        }
        num += (static_cast<double>(n0.x) + static_cast<double>(n0.y) + static_cast<double>(n1.x) +
                static_cast<double>(n1.y)) * ab[c];
        den += static_cast<double>(d0.x) + static_cast<double>(d0.y) + static_cast<double>(d1.x) +
               static_cast<double>(d1.y);
      }
      tc_fence_before();
      mbar_arrive(bar_c);
    }
    if (!ok) {
      raise_abort(abort_flag, p.status, kStatusTimeoutCompute);
    } else {
      p.delta[static_cast<size_t>(bh) * p.N + row] = static_cast<float>(num / den);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem, C::kTmemCols);
}

template <int D>
static cudaError_t launch_delta_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                                  const CUtensorMap& tdo, const DeltaParams& p, cudaStream_t stream) {
  using C = DeltaCfg<D>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(delta_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  dim3 grid(p.N / 128, p.B * p.H);
  delta_kernel<D><<<grid, 192, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError();
}

cudaError_t launch_delta(int D, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                         const CUtensorMap& tdo, const DeltaParams& p, cudaStream_t stream) {
  return D == 128 ? launch_delta_t<128>(tq, tk, tv, tdo, p, stream) : launch_delta_t<256>(tq, tk, tv, tdo, p, stream);
}

}  // namespace dm
