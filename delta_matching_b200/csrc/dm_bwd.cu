// Backward of delta-matching fp8 attention on sm_100a: all matmuls on tcgen05 with TMEM accumulators, bit-deterministic
// (one writer per output element, fixed loop orders, no atomics, no O(N^2) workspace).
//
//   kernel 1 (dK/dV, key-stationary): CTA = (128-key tile, kv head, batch); loops over the query heads of the GQA group
//     and their 128-query tiles: S^T = K8 Q8^T, dP^T = V8 dO8^T (kind::f8f6f4), P^T codes and dS^T codes written to TMEM,
//     dV += P^T dO and dK += dS^T Q as block-scaled chains (kind::mxf8f6f4).  The group is reduced in TMEM, dK / dV are
//     rounded to bf16 once per KV head.
//   kernel 2 (dQ, query-stationary): CTA = (128-query tile, query head, batch); loops over key tiles: S, dP recomputed,
//     dS codes staged in shared memory, dQ += dS K block-scaled; dQ * softmax_scale rounded to bf16 once.
//
// Numerics (delta_matching/reference.py:476-518 with preset "sm100-mx", :612-613; kernel-side rules
// delta_matching/sm100/dm_bwd_sm100.py:5413-5433, 6175-6224 and attention_math_sm100.py:26-45):
//   P = ex2(fma(S_acc, (ks*qs)*log2e, -lse*log2e));  dP = dP_acc * (vs*dos);  dS = P * (dP - delta)   (fp32)
//   P^T codes: power-of-two scale per (key, 32 queries), amax 0 -> byte 0;   SFA_dV = p_sb (+) dos_sb
//   dS codes:  power-of-two scale per (128 queries x 32 keys), amax 0 -> scale 1;  SFA_dK = ds_sb (+) qs_sb,
//              dQ's scale along keys = ds_sb (+) ks_sb;  dQ = (dS K) * D^-0.5.
// Both kernels evaluate P and dS with the same operations on the same accumulators, so the dS codes of kernel 2 are the
// codes of kernel 1 whenever the two MMA orientations return the same fp32 sums.
#include <cuda_bf16.h>
#include "dm_common.cuh"
#include "dm_kernels.h"

namespace dm {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}

// Row of an fp32 TMEM accumulator (32-column chunk c) -> bf16, 64 bytes to global.
__device__ __forceinline__ void store_bf16_chunk(const uint32_t (&r)[32], float mul, __nv_bfloat16* dst) {
  uint32_t w[16];
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * e]) * mul, __uint_as_float(r[2 * e + 1]) * mul);
    w[e] = *reinterpret_cast<uint32_t*>(&v);
  }
  uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int e = 0; e < 4; ++e) d4[e] = make_uint4(w[4 * e], w[4 * e + 1], w[4 * e + 2], w[4 * e + 3]);
}

// ================================================================================================ dK / dV
template <int D, bool DV, bool DK>
struct KvCfg {
  static constexpr int kSub = D / 128;
  static constexpr int kTileBytes = 128 * D;
  static constexpr int kStages = 2;
  static constexpr int kTmemCols = 512;
  static constexpr int kColS = 0;            // S^T fp32; P^T codes reuse columns 0-31
  static constexpr int kColSfaV = 32;        // 4 columns: SFA word of the dV chain (written after S^T is consumed)
  static constexpr int kColOne = 36;         // 4 columns of 0x7F7F7F7F: scale 1.0 for the B operand
  static constexpr int kColDp = 128;         // dP^T fp32; dS^T codes reuse columns 128-159
  static constexpr int kColSfaK = 160;       // 4 columns: SFA word of the dK chain
  static constexpr int kColDv = 256;                         // D columns when DV
  static constexpr int kColDk = DV ? 256 + D : 256;          // D columns when DK
  static_assert(kColDk + (DK ? D : 0) <= 512, "TMEM budget");
  static constexpr int kSmemK = 0;
  static constexpr int kSmemV = kTileBytes;
  static constexpr int kSmemQ = 2 * kTileBytes;                      // [kStages]
  static constexpr int kSmemDo = kSmemQ + kStages * kTileBytes;      // [kStages]
  static constexpr int kSmemVec = kSmemDo + kStages * kTileBytes;    // 2 x (l2[128], delta[128]) floats
  static constexpr int kSmemBar = kSmemVec + 2 * 2 * 128 * 4;
  static constexpr int kSmemBytes = kSmemBar + 256 + 1024;
};

template <int D, bool DV, bool DK>
__global__ void __launch_bounds__(192, 1)
bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do, const BwdParams p) {
  using C = KvCfg<D, DV, DK>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + C::kSmemK;
  uint8_t* sV = smem + C::kSmemV;
  uint8_t* sQ = smem + C::kSmemQ;
  uint8_t* sDo = smem + C::kSmemDo;
  float* sVec = reinterpret_cast<float*>(smem + C::kSmemVec);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kSmemBar);
  uint64_t* bar_kv = bars + 0;
  uint64_t* bar_s = bars + 1;       // S^T, dP^T ready
  uint64_t* bar_p = bars + 2;       // codes and scale words written (128 arrivals)
  uint64_t* bar_done = bars + 3;    // dV / dK chains of the iteration done
  uint64_t* full = bars + 4;        // [kStages]
  uint64_t* empty = bars + 6;       // [kStages]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 11);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int n_t = p.N / 128;
  const int kt = blockIdx.x;                          // causal: tile 0 has the most query tiles and starts first
  const int bhk = blockIdx.y;
  const int b = bhk / p.Hk, hk = bhk % p.Hk;
  const int rep = p.H / p.Hk;
  const int qt0 = p.causal ? kt : 0;
  const int n_qi = n_t - qt0;
  const int n_it = rep * n_qi;                        // iteration = (query head of the group, query tile)

  if (tid == 0) {
    mbar_init(bar_kv, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_p, 128);
    mbar_init(bar_done, 1);
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
    // ------------------------------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_do);
      mbar_expect_tx(bar_kv, 2 * C::kTileBytes);
      for (int s = 0; s < C::kSub; ++s) {
        tma_load_2d(sK + s * 16384, &tm_k, bar_kv, s * 128, bhk * p.N + kt * 128);
        tma_load_2d(sV + s * 16384, &tm_v, bar_kv, s * 128, bhk * p.N + kt * 128);
      }
      for (int it = 0; it < n_it; ++it) {
        const int st = it % C::kStages;
        if (it >= C::kStages) {
          if (!wait_or_abort(empty + st, ((it / C::kStages) - 1) & 1, abort_flag)) {
            raise_abort(abort_flag, p.status, kStatusTimeoutProducer);
            break;
          }
        }
        const int h = hk * rep + it / n_qi;
        const int row = (b * p.H + h) * p.N + (qt0 + it % n_qi) * 128;
        mbar_expect_tx(full + st, 2 * C::kTileBytes);
        for (int s = 0; s < C::kSub; ++s) {
          tma_load_2d(sQ + st * C::kTileBytes + s * 16384, &tm_q, full + st, s * 128, row);
          tma_load_2d(sDo + st * C::kTileBytes + s * 16384, &tm_do, full + st, s * 128, row);
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t kIdesc = idesc_f8(128, 128, false, false);
      bool ok = wait_or_abort(bar_kv, 0, abort_flag);
      for (int it = 0; ok && it < n_it; ++it) {
        const int st = it % C::kStages;
        if (!(ok = wait_or_abort(full + st, (it / C::kStages) & 1, abort_flag))) break;
        // the previous chains still read the code and scale columns that the next S^T / dP^T overwrite
        if (it > 0 && !(ok = wait_or_abort(bar_done, (it - 1) & 1, abort_flag))) break;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQ + st * C::kTileBytes), do_addr = smem_u32(sDo + st * C::kTileBytes);
#pragma unroll
        for (int ks = 0; ks < D / 32; ++ks) {
          const uint32_t off = (ks / 4) * 16384 + (ks % 4) * 32;
          mma_f8_ss(tmem + C::kColS, smem_desc_sw128(smem_u32(sK) + off, 16, 1024),
                    smem_desc_sw128(q_addr + off, 16, 1024), kIdesc, ks > 0);
        }
        if (DK) {
#pragma unroll
          for (int ks = 0; ks < D / 32; ++ks) {
            const uint32_t off = (ks / 4) * 16384 + (ks % 4) * 32;
            mma_f8_ss(tmem + C::kColDp, smem_desc_sw128(smem_u32(sV) + off, 16, 1024),
                      smem_desc_sw128(do_addr + off, 16, 1024), kIdesc, ks > 0);
          }
        }
        tc_commit(bar_s);
        if (!(ok = wait_or_abort(bar_p, it & 1, abort_flag))) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
          for (int s = 0; s < C::kSub; ++s) {
            // contraction over the 128 queries of the tile: B = dO / Q tile read MN-major, 32 query rows per step
            if (DV)
              mma_mxf8_ts(tmem + C::kColDv + s * 128, tmem + C::kColS + ks * 8,
                          smem_desc_sw128(do_addr + s * 16384 + ks * 4096, 16, 1024),
                          idesc_mxf8(128, 128, false, true, ks, ks), tmem + C::kColSfaV, tmem + C::kColOne,
                          (it > 0) || (ks > 0));
            if (DK)
              mma_mxf8_ts(tmem + C::kColDk + s * 128, tmem + C::kColDp + ks * 8,
                          smem_desc_sw128(q_addr + s * 16384 + ks * 4096, 16, 1024),
                          idesc_mxf8(128, 128, false, true, ks, ks), tmem + C::kColSfaK, tmem + C::kColOne,
                          (it > 0) || (ks > 0));
          }
        }
        tc_commit(empty + st);
        tc_commit(bar_done);
      }
      if (!ok) raise_abort(abort_flag, p.status, kStatusTimeoutMma);
    }
  } else {
    // ------------------------------------------------------------------------------------------ compute warps
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const int key = kt * 128 + tid;
    const int nblk = p.N / 32;
    const float ks_row = p.ks[static_cast<size_t>(bhk) * nblk + key / 32];
    const float vs_row = p.vs[static_cast<size_t>(bhk) * nblk + key / 32];
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int h = hk * rep + it / n_qi;
      const int qt = qt0 + it % n_qi;
      const int bh = b * p.H + h;
      float* l2 = sVec + (it & 1) * 256;
      float* dl = l2 + 128;
      l2[tid] = p.lse[static_cast<size_t>(bh) * p.N + qt * 128 + tid] * kLog2e;
      dl[tid] = p.delta[static_cast<size_t>(bh) * p.N + qt * 128 + tid];
      const float4 qs4 = *reinterpret_cast<const float4*>(p.qs + static_cast<size_t>(bh) * nblk + qt * 4);
      const float4 dos4 = *reinterpret_cast<const float4*>(p.dos + static_cast<size_t>(bh) * nblk + qt * 4);
      const float qsv[4] = {qs4.x, qs4.y, qs4.z, qs4.w};
      const float dosv[4] = {dos4.x, dos4.y, dos4.z, dos4.w};
      const bool diag = p.causal && (qt == kt);
      bar_sync(1, 128);
      // after a failed wait the warp keeps meeting the others at the named barrier (it only skips the work)
      if (ok) ok = wait_warp(bar_s, it & 1, abort_flag);
      if (!ok) continue;
      tc_fence_after();
      float ds[DK ? 128 : 1];
      float ds_amax = 0.f;
      uint32_t sfa_v[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float cc = (ks_row * qsv[c]) * kLog2e;
        const float aa = vs_row * dosv[c];
        uint32_t rs[32];
        tmem_ld32(tmem + lane_base + C::kColS + 32 * c, rs);
        tmem_wait_ld();
        float pr[32];
        float pmax = 0.f;
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          float s = __uint_as_float(rs[e]);
          if (diag && (tid > 32 * c + e)) s = -INFINITY;          // key index above the query index
          pr[e] = ex2_approx(fmaf(s, cc, -l2[32 * c + e]));
          pmax = fmaxf(pmax, pr[e]);
        }
        if (DV) {
          const uint32_t psb = pow2_sb(pmax, 0u);
          const float inv = sb_to_inv(psb);
          uint32_t codes[8];
#pragma unroll
          for (int e = 0; e < 32; e += 4)
            codes[e / 4] = cvt_e4m3x4(pr[e] * inv, pr[e + 1] * inv, pr[e + 2] * inv, pr[e + 3] * inv);
          tmem_st8(tmem + lane_base + C::kColS + 8 * c, codes);
          sfa_v[c] = sb_mul(psb, scale_to_sb(dosv[c]));
        }
        if (DK) {
          uint32_t rd[32];
          tmem_ld32(tmem + lane_base + C::kColDp + 32 * c, rd);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const float v = pr[e] * (__uint_as_float(rd[e]) * aa - dl[32 * c + e]);
            ds[32 * c + e] = v;
            ds_amax = fmaxf(ds_amax, fabsf(v));
          }
        }
      }
      if (DV) {
        const uint32_t w = pack4(sfa_v[0], sfa_v[1], sfa_v[2], sfa_v[3]);
        tmem_st4(tmem + lane_base + C::kColSfaV, w, w, w, w);
      }
      tmem_st4(tmem + lane_base + C::kColOne, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu);
      if (DK) {
        // one scale for the (128 queries x this warp's 32 keys) block
        const uint32_t dsb = pow2_sb(warp_max(ds_amax), 127u);
        const float inv = sb_to_inv(dsb);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t codes[8];
#pragma unroll
          for (int e = 0; e < 32; e += 4)
            codes[e / 4] = cvt_e4m3x4(ds[32 * c + e] * inv, ds[32 * c + e + 1] * inv, ds[32 * c + e + 2] * inv,
                                      ds[32 * c + e + 3] * inv);
          tmem_st8(tmem + lane_base + C::kColDp + 8 * c, codes);
        }
        const uint32_t w = pack4(sb_mul(dsb, scale_to_sb(qsv[0])), sb_mul(dsb, scale_to_sb(qsv[1])),
                                 sb_mul(dsb, scale_to_sb(qsv[2])), sb_mul(dsb, scale_to_sb(qsv[3])));
        tmem_st4(tmem + lane_base + C::kColSfaK, w, w, w, w);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar_p);
    }
    if (ok) ok = wait_warp(bar_done, (n_it - 1) & 1, abort_flag);
    if (!ok) {
      raise_abort(abort_flag, p.status, kStatusTimeoutCompute);
    } else {
      tc_fence_after();
      if (DV) {
        __nv_bfloat16* dst = p.dv + static_cast<int64_t>(b) * p.dv_sb + static_cast<int64_t>(key) * p.dv_sn +
                             static_cast<int64_t>(hk) * p.dv_sh;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem + lane_base + C::kColDv + 32 * c, r);
          tmem_wait_ld();
          store_bf16_chunk(r, 1.0f, dst + 32 * c);
        }
      }
      if (DK) {
        __nv_bfloat16* dst = p.dk + static_cast<int64_t>(b) * p.dk_sb + static_cast<int64_t>(key) * p.dk_sn +
                             static_cast<int64_t>(hk) * p.dk_sh;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem + lane_base + C::kColDk + 32 * c, r);
          tmem_wait_ld();
          store_bf16_chunk(r, 1.0f, dst + 32 * c);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem, C::kTmemCols);
}

// ================================================================================================ dQ
template <int D>
struct DqCfg {
  static constexpr int kSub = D / 128;
  static constexpr int kTileBytes = 128 * D;
  static constexpr int kStages = 2;
  static constexpr int kTmemCols = 512;
  static constexpr int kColS = 0;
  static constexpr int kColSfa = 32;         // written after S is consumed: bytes = ds_sb (+) ks_sb per 32-key step
  static constexpr int kColOne = 36;
  static constexpr int kColDp = 128;
  static constexpr int kColDq = 256;
  static constexpr int kSmemQ = 0;
  static constexpr int kSmemDo = kTileBytes;
  static constexpr int kSmemK = 2 * kTileBytes;                      // [kStages]
  static constexpr int kSmemV = kSmemK + kStages * kTileBytes;       // [kStages]
  static constexpr int kSmemDs = kSmemV + kStages * kTileBytes;      // 128 x 128 dS codes, rows = queries
  static constexpr int kSmemRed = kSmemDs + 16384;                   // 2 x [4 warps][4 blocks] floats
  static constexpr int kSmemBar = kSmemRed + 2 * 16 * 4;
  static constexpr int kSmemBytes = kSmemBar + 256 + 1024;
};

template <int D>
__global__ void __launch_bounds__(192, 1)
bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do, const BwdParams p) {
  using C = DqCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + C::kSmemQ;
  uint8_t* sDo = smem + C::kSmemDo;
  uint8_t* sK = smem + C::kSmemK;
  uint8_t* sV = smem + C::kSmemV;
  uint8_t* sDs = smem + C::kSmemDs;
  float* sRed = reinterpret_cast<float*>(smem + C::kSmemRed);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kSmemBar);
  uint64_t* bar_q = bars + 0;
  uint64_t* bar_s = bars + 1;
  uint64_t* bar_p = bars + 2;
  uint64_t* bar_done = bars + 3;
  uint64_t* full = bars + 4;
  uint64_t* empty = bars + 6;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 11);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int n_t = p.N / 128;
  const int qt = n_t - 1 - static_cast<int>(blockIdx.x);
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const int bhk = b * p.Hk + h / (p.H / p.Hk);
  const int n_it = p.causal ? (qt + 1) : n_t;

  if (tid == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_p, 128);
    mbar_init(bar_done, 1);
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
        const int row = bhk * p.N + it * 128;
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
        if (it > 0 && !(ok = wait_or_abort(bar_done, (it - 1) & 1, abort_flag))) break;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + st * C::kTileBytes), v_addr = smem_u32(sV + st * C::kTileBytes);
#pragma unroll
        for (int ks = 0; ks < D / 32; ++ks) {
          const uint32_t off = (ks / 4) * 16384 + (ks % 4) * 32;
          mma_f8_ss(tmem + C::kColS, smem_desc_sw128(smem_u32(sQ) + off, 16, 1024),
                    smem_desc_sw128(k_addr + off, 16, 1024), kIdesc, ks > 0);
        }
#pragma unroll
        for (int ks = 0; ks < D / 32; ++ks) {
          const uint32_t off = (ks / 4) * 16384 + (ks % 4) * 32;
          mma_f8_ss(tmem + C::kColDp, smem_desc_sw128(smem_u32(sDo) + off, 16, 1024),
                    smem_desc_sw128(v_addr + off, 16, 1024), kIdesc, ks > 0);
        }
        tc_commit(bar_s);
        if (!(ok = wait_or_abort(bar_p, it & 1, abort_flag))) break;
        tc_fence_after();
        // dQ += dS K: A = dS codes in shared memory (rows = queries, K-major), B = K tile MN-major (32 key rows per step)
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
          for (int s = 0; s < C::kSub; ++s) {
            mma_mxf8_ss(tmem + C::kColDq + s * 128, smem_desc_sw128(smem_u32(sDs) + ks * 32, 16, 1024),
                        smem_desc_sw128(k_addr + s * 16384 + ks * 4096, 16, 1024),
                        idesc_mxf8(128, 128, false, true, ks, ks), tmem + C::kColSfa, tmem + C::kColOne,
                        (it > 0) || (ks > 0));
          }
        }
        tc_commit(empty + st);
        tc_commit(bar_done);
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
    const float dlt = p.delta[static_cast<size_t>(bh) * p.N + row];
    const bool probe = p.rowsum_ds != nullptr;
    double rs_acc = 0.0, ap_acc = 0.0;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const float4 ks4 = *reinterpret_cast<const float4*>(p.ks + static_cast<size_t>(bhk) * nblk + it * 4);
      const float4 vs4 = *reinterpret_cast<const float4*>(p.vs + static_cast<size_t>(bhk) * nblk + it * 4);
      const float ksv[4] = {ks4.x, ks4.y, ks4.z, ks4.w};
      const float vsv[4] = {vs4.x, vs4.y, vs4.z, vs4.w};
      const bool diag = p.causal && (it == qt);
      if (ok) ok = wait_warp(bar_s, it & 1, abort_flag);
      tc_fence_after();
      float ds[128];
      float bmax[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; ok && c < 4; ++c) {
        const float cc = (ksv[c] * qs) * kLog2e;
        const float aa = vsv[c] * dos;
        uint32_t rs[32], rd[32];
        tmem_ld32(tmem + lane_base + C::kColS + 32 * c, rs);
        tmem_ld32(tmem + lane_base + C::kColDp + 32 * c, rd);
        tmem_wait_ld();
        float am = 0.f, rsum = 0.f, asum = 0.f;
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          float s = __uint_as_float(rs[e]);
          if (diag && (32 * c + e > tid)) s = -INFINITY;
          const float pe = ex2_approx(fmaf(s, cc, neg_l2));
          const float dp = __uint_as_float(rd[e]) * aa;
          const float v = pe * (dp - dlt);
          ds[32 * c + e] = v;
          am = fmaxf(am, fabsf(v));
          if (probe) {
            rsum += v;
            asum += fabsf(pe * dp);
          }
        }
        bmax[c] = am;
        if (probe) {
          rs_acc += static_cast<double>(rsum);
          ap_acc += static_cast<double>(asum);
        }
      }
      // one scale per (this tile's 128 queries x 32 keys): reduce the block maxima over the four warps
      float* red = sRed + (it & 1) * 16;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float wm = warp_max(bmax[c]);
        if ((tid & 31) == 0) red[warp * 4 + c] = wm;
      }
      bar_sync(1, 128);          // reached by every compute warp in every iteration, also after a failed wait
      if (!ok) continue;
      uint32_t sfw[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float am = fmaxf(fmaxf(red[c], red[4 + c]), fmaxf(red[8 + c], red[12 + c]));
        const uint32_t dsb = pow2_sb(am, 127u);
        const float inv = sb_to_inv(dsb);
        sfw[c] = sb_mul(dsb, scale_to_sb(ksv[c]));
        // row tid of the dS tile: 16-byte chunk j of the row lands at chunk (j ^ (tid % 8)) (128-byte swizzle)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int e0 = 32 * c + 16 * j;
          uint4 w;
          w.x = cvt_e4m3x4(ds[e0 + 0] * inv, ds[e0 + 1] * inv, ds[e0 + 2] * inv, ds[e0 + 3] * inv);
          w.y = cvt_e4m3x4(ds[e0 + 4] * inv, ds[e0 + 5] * inv, ds[e0 + 6] * inv, ds[e0 + 7] * inv);
          w.z = cvt_e4m3x4(ds[e0 + 8] * inv, ds[e0 + 9] * inv, ds[e0 + 10] * inv, ds[e0 + 11] * inv);
          w.w = cvt_e4m3x4(ds[e0 + 12] * inv, ds[e0 + 13] * inv, ds[e0 + 14] * inv, ds[e0 + 15] * inv);
          const int chunk = (2 * c + j) ^ (tid & 7);
          *reinterpret_cast<uint4*>(sDs + tid * 128 + chunk * 16) = w;
        }
      }
      const uint32_t w = pack4(sfw[0], sfw[1], sfw[2], sfw[3]);
      tmem_st4(tmem + lane_base + C::kColSfa, w, w, w, w);
      tmem_st4(tmem + lane_base + C::kColOne, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu);
      tmem_wait_st();
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(bar_p);
    }
    if (ok) ok = wait_warp(bar_done, (n_it - 1) & 1, abort_flag);
    if (!ok) {
      raise_abort(abort_flag, p.status, kStatusTimeoutCompute);
    } else {
      tc_fence_after();
      __nv_bfloat16* dst = p.dq + static_cast<int64_t>(b) * p.dq_sb + static_cast<int64_t>(row) * p.dq_sn +
                           static_cast<int64_t>(h) * p.dq_sh;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem + lane_base + C::kColDq + 32 * c, r);
        tmem_wait_ld();
        store_bf16_chunk(r, p.sm_scale, dst + 32 * c);
      }
      if (probe) {
        p.rowsum_ds[static_cast<size_t>(bh) * p.N + row] = static_cast<float>(rs_acc);
        p.sum_abs_pdp[static_cast<size_t>(bh) * p.N + row] = static_cast<float>(ap_acc);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem, C::kTmemCols);
}

// ================================================================================================ launchers
template <typename K>
static cudaError_t set_smem(K kernel, int bytes, bool* done) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return e;
    done[dev] = true;
  }
  return cudaSuccess;
}

template <int D, bool DV, bool DK>
static cudaError_t launch_kv_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                               const CUtensorMap& tdo, const BwdParams& p, cudaStream_t stream) {
  using C = KvCfg<D, DV, DK>;
  static bool done[64] = {};
  cudaError_t e = set_smem(bwd_dkdv_kernel<D, DV, DK>, C::kSmemBytes, done);
  if (e != cudaSuccess) return e;
  dim3 grid(p.N / 128, p.B * p.Hk);
  bwd_dkdv_kernel<D, DV, DK><<<grid, 192, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError();
}

cudaError_t launch_bwd_dkdv(int D, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                            const CUtensorMap& tdo, const BwdParams& p, cudaStream_t stream) {
  if (D == 128) return launch_kv_t<128, true, true>(tq, tk, tv, tdo, p, stream);
  // head_dim 256: S^T + dP^T + dK + dV exceed the 512 TMEM columns, so dV and dK run as two launches
  cudaError_t e = launch_kv_t<256, true, false>(tq, tk, tv, tdo, p, stream);
  if (e != cudaSuccess) return e;
  return launch_kv_t<256, false, true>(tq, tk, tv, tdo, p, stream);
}

template <int D>
static cudaError_t launch_dq_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                               const CUtensorMap& tdo, const BwdParams& p, cudaStream_t stream) {
  using C = DqCfg<D>;
  static bool done[64] = {};
  cudaError_t e = set_smem(bwd_dq_kernel<D>, C::kSmemBytes, done);
  if (e != cudaSuccess) return e;
  dim3 grid(p.N / 128, p.B * p.H);
  bwd_dq_kernel<D><<<grid, 192, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError();
}

cudaError_t launch_bwd_dq(int D, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                          const CUtensorMap& tdo, const BwdParams& p, cudaStream_t stream) {
  return D == 128 ? launch_dq_t<128>(tq, tk, tv, tdo, p, stream) : launch_dq_t<256>(tq, tk, tv, tdo, p, stream);
}

}  // namespace dm
