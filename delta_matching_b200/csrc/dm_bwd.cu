// Backward of delta-matching fp8 attention on sm_100a: all matmuls on tcgen05 with TMEM accumulators, bit-deterministic
// (one writer per output element, fixed loop orders, no atomics, no O(N^2) workspace).
//
//   kernel 1 (dK/dV, key-stationary): CTA = (128-key tile, kv head, batch); loops over the query heads of the GQA group
//     and their 128-query tiles: S^T = K8 Q8^T, dP^T = V8 dO8^T (kind::f8f6f4), P^T codes and dS^T codes written to TMEM,
//     dV += P^T dO and dK += dS^T Q as block-scaled chains (kind::mxf8f6f4).  The group is reduced in TMEM, dK / dV are
//     rounded to bf16 once per KV head.  With a workspace it also leaves the dS^T code tiles there for the streaming dQ
//     kernel (dm_bwd_p2.cu).  Head_dim 256 runs it as two launches, one per accumulator.
//   kernel 2 (dQ, query-stationary, the form without a workspace): CTA = (128-query tile, query head, batch); loops over
//     key tiles: S, dP recomputed, dS codes staged in shared memory, dQ += dS K block-scaled; dQ * softmax_scale rounded
//     to bf16 once.
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

// Maximum over the warp of a non-negative value: non-negative floats order like their bit patterns, so one integer
// redux.sync does the work of a five-step shuffle butterfly.
__device__ __forceinline__ float warp_max(float v) {
  return __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(v)));
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

// ================================================================================================ dK / dV, pipelined
// One CTA per SM: G compute groups of four warps (G = 2 or 4; group g owns the query blocks [g * 4/G, (g+1) * 4/G) of
// every tile, 32 query columns per block; thread t % 128 = key row = TMEM lane), then one TMA warp and one MMA warp.
// TMEM: one 128-column region is time-shared by S^T and dP^T (each is pulled into registers as soon as it lands, which
// frees the region for the other), P^T codes, dS^T codes and the scale words have columns of their own, dV and dK
// accumulate over all (query head of the group, query tile) iterations.  The tensor pipe therefore runs dP^T(i) and
// S^T(i+1) while the compute warps work on tile i, then dV(i) and dK(i) once both code sets of the tile are written.
//
// Head_dim 128 runs the kernel with both accumulators (DV and DK).  At head_dim 256 one accumulator fills 256 columns,
// so the same kernel runs twice: a DV launch (S^T, P^T codes, dV: no dP^T, no dS) and a DK launch (S^T, dP^T, dS codes,
// dK, and the dS tiles for the workspace), each with the other half of the work compiled out.
template <int G, int D = 128, bool DV = true, bool DK = true>
struct KvPipeCfg {
  static_assert(D == 128 ? (DV && DK) : (D == 256 && DV != DK), "128: both accumulators; 256: one per launch");
  static constexpr int kSub = D / 128;                 // 128-byte-wide sub-tiles of an operand row
  static constexpr int kTileBytes = 128 * D;           // K, V, Q, dO tile
  static constexpr int kCodeBytes = 128 * 128;         // dS^T code tile (does not depend on head_dim)
  static constexpr int kStages = (D == 128) ? 4 : 2;
  static constexpr int kWsBufs = (D == 128) ? 2 : 1;
  static constexpr int kGroups = G;
  static constexpr int kChunks = 4 / G;      // 32-column query blocks per thread and tile
  static constexpr int kThreads = kGroups * 128 + 64;
  static constexpr int kTmemCols = 512;
  static constexpr int kColSd = 0;           // S^T, then dP^T (fp32)
  static constexpr int kColPc = 128;         // P^T codes: 8 columns per query block
  static constexpr int kColDc = 160;         // dS^T codes
  static constexpr int kColXv = 192;         // 4 x 4 columns: dV scale word of query block b (byte 0)
  static constexpr int kColXk = 208;         // 4 x 4 columns: dK scale word of query block b
  static constexpr int kColOne = 224;        // 4 columns of 0x7F7F7F7F
  static constexpr int kColDv = 256, kColDk = (D == 128) ? 384 : 256;
  static constexpr int kSmemK = 0;
  static constexpr int kSmemV = kTileBytes;
  static constexpr int kSmemQ = 2 * kTileBytes;                      // [kStages]
  static constexpr int kSmemDo = kSmemQ + kStages * kTileBytes;      // [kStages]
  static constexpr int kSmemVec = kSmemDo + kStages * kTileBytes;    // [kStages] x (lse[128], delta[128]) floats
  static constexpr int kSmemWs = kSmemVec + kStages * 1024;          // 2 staging tiles of dS^T codes for the workspace
  static constexpr int kSmemXch = kSmemWs + kWsBufs * kCodeBytes;    // 2 x [16 warps] floats
  static constexpr int kSmemBar = kSmemXch + 2 * 16 * 4;
  static constexpr int kSmemBytes = kSmemBar + 256 + 1024;
  static_assert(kSmemBytes <= 232448, "shared memory budget");
};

// DS32: the dS scale is taken per (32 queries x 32 keys), which is one warp's block of a tile (each thread holds one
// 32-query block per tile), instead of the contract's (128 queries x 32 keys), for which the four groups' warps of a
// key quadrant exchange their maxima.
template <int G, int D, bool DV, bool DK, bool DS32>
__global__ void __launch_bounds__(KvPipeCfg<G, D, DV, DK>::kThreads, 1)
bwd_dkdv_pipe_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                     const __grid_constant__ CUtensorMap tm_ds, const BwdParams p) {
  using C = KvPipeCfg<G, D, DV, DK>;
  constexpr int kW = C::kGroups * 4;                 // compute warps; warp kW = TMA, kW + 1 = MMA
  constexpr int CH = C::kChunks;
  static_assert(!DS32 || CH == 1, "per-block dS scales need one 32-query block per thread and tile");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem + C::kSmemK;
  uint8_t* sV = smem + C::kSmemV;
  uint8_t* sQ = smem + C::kSmemQ;
  uint8_t* sDo = smem + C::kSmemDo;
  float* sVec = reinterpret_cast<float*>(smem + C::kSmemVec);
  float* sXch = reinterpret_cast<float*>(smem + C::kSmemXch);
  uint8_t* sWs = smem + C::kSmemWs;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kSmemBar);
  uint64_t* bar_kv = bars + 0;
  uint64_t* bar_s = bars + 1;        // S^T landed in the shared region (MMA commit)
  uint64_t* bar_sfree = bars + 2;    // every compute warp holds its S^T columns (one arrival per warp)
  uint64_t* bar_dp = bars + 3;       // dP^T landed
  uint64_t* bar_dpfree = bars + 4;   // every compute warp holds its dP^T columns
  uint64_t* bar_pv = bars + 5;       // P^T codes + dV scale words written
  uint64_t* bar_pk = bars + 6;       // dS^T codes + dK scale words written
  uint64_t* bar_done = bars + 7;     // dV and dK chains of the iteration done (MMA commit)
  uint64_t* full = bars + 8;         // [kStages] Q, dO, lse, delta of the stage landed
  uint64_t* empty = bars + 12;       // [kStages]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 17);

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
    mbar_init(bar_dp, 1);
    mbar_init(bar_done, 1);
    mbar_init(bar_sfree, kW);
    mbar_init(bar_dpfree, kW);
    mbar_init(bar_pv, kW);
    mbar_init(bar_pk, kW);
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kW + 1) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == kW) {
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
      int h = hk * rep, qi = 0;
      for (int it = 0; it < n_it; ++it) {
        const int st = it % C::kStages;
        if (it >= C::kStages) {
          if (!wait_or_abort(empty + st, ((it / C::kStages) - 1) & 1, abort_flag)) {
            raise_abort(abort_flag, p.status, kStatusTimeoutProducer);
            break;
          }
        }
        const size_t row = static_cast<size_t>(b * p.H + h) * p.N + (qt0 + qi) * 128;
        mbar_expect_tx(full + st, 2 * C::kTileBytes + 1024);
        for (int s = 0; s < C::kSub; ++s) {
          tma_load_2d(sQ + st * C::kTileBytes + s * 16384, &tm_q, full + st, s * 128, static_cast<int>(row));
          tma_load_2d(sDo + st * C::kTileBytes + s * 16384, &tm_do, full + st, s * 128, static_cast<int>(row));
        }
        bulk_load_1d(sVec + st * 256, p.lse + row, 512, full + st);
        bulk_load_1d(sVec + st * 256 + 128, p.delta + row, 512, full + st);
        if (++qi == n_qi) {
          qi = 0;
          ++h;
        }
      }
    }
  } else if (warp == kW + 1) {
    // ------------------------------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t kIdesc = idesc_f8(128, 128, false, false);
      constexpr uint32_t kIdescBs = idesc_mxf8(128, 128, false, true, 0, 0);
      const uint32_t k_lo = desc_lo(smem_u32(sK)), v_lo = desc_lo(smem_u32(sV));
      const uint32_t q_lo0 = desc_lo(smem_u32(sQ)), do_lo0 = desc_lo(smem_u32(sDo));
      // a first matmul of the tile: both operands K-major, D / 32 steps of 32 bytes inside the 128-byte swizzle rows
      auto chain_kmajor = [&](uint32_t a_lo, uint32_t b_lo) {
#pragma unroll
        for (int ks = 0; ks < D / 32; ++ks) {
          const uint32_t off = (ks / 4) * 1024 + (ks % 4) * 2;        // descriptor units of 16 bytes
          mma_f8_ss(tmem + C::kColSd, a_lo + off, b_lo + off, kIdesc, ks > 0);
        }
      };
      // a second matmul: A = codes in TMEM (8 columns per 32-query step), B = dO / Q tile MN-major (32 query rows per
      // step), one 128-column accumulator slice per sub-tile of head_dim
      auto chain_acc = [&](uint32_t d_col, uint32_t a_col, uint32_t b_lo, uint32_t x_col, bool first) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
          for (int s = 0; s < C::kSub; ++s)
            mma_mxf8_ts(tmem + d_col + s * 128, tmem + a_col + ks * 8, b_lo + s * 1024 + ks * 256, kIdescBs,
                        tmem + x_col + 4 * ks, tmem + C::kColOne, !first || (ks > 0));
        }
      };
      bool ok = wait_or_abort(bar_kv, 0, abort_flag);
      if (ok) ok = wait_or_abort(full + 0, 0, abort_flag);
      if (ok) {
        tc_fence_after();
        chain_kmajor(k_lo, q_lo0);
        tc_commit(bar_s);
      }
      for (int it = 0; ok && it < n_it; ++it) {
        const int st = it % C::kStages;
        const uint32_t q_lo = q_lo0 + st * (C::kTileBytes >> 4), do_lo = do_lo0 + st * (C::kTileBytes >> 4);
        const uint32_t ph = it & 1;
        auto next_st = [&]() -> bool {                         // S^T of the next iteration into the shared region
          if (it + 1 >= n_it) return true;
          const int sn = (it + 1) % C::kStages;
          if (!wait_or_abort(full + sn, ((it + 1) / C::kStages) & 1, abort_flag)) return false;
          tc_fence_after();
          chain_kmajor(k_lo, q_lo0 + sn * (C::kTileBytes >> 4));
          tc_commit(bar_s);
          return true;
        };
        if (!(ok = wait_or_abort(bar_sfree, ph, abort_flag))) break;
        tc_fence_after();
        if (DK) {
          chain_kmajor(v_lo, do_lo);                           // dP^T = V dO^T into the region S^T has just left
          tc_commit(bar_dp);
        } else {
          if (!(ok = next_st())) break;                        // no dP^T in a DV launch: the region is free at once
        }
        if (DV && !DK) {
          if (!(ok = wait_or_abort(bar_pv, ph, abort_flag))) break;
          tc_fence_after();
          chain_acc(C::kColDv, C::kColPc, do_lo, C::kColXv, it == 0);       // dV += P^T dO
        }
        if (DK) {
          if (!(ok = wait_or_abort(bar_dpfree, ph, abort_flag))) break;
          if (!(ok = next_st())) break;
          // With both accumulators the compute warps hand P^T and dS^T codes over together (one tcgen05.wait::st and
          // one arrival per tile instead of two): the dV chain moves behind the same barrier.  Both chains are long
          // finished when the warps, after the exponentials of the next tile, want to overwrite the codes.
          if (!(ok = wait_or_abort(bar_pk, ph, abort_flag))) break;
          tc_fence_after();
          if (DV) chain_acc(C::kColDv, C::kColPc, do_lo, C::kColXv, it == 0);  // dV += P^T dO
          chain_acc(C::kColDk, C::kColDc, q_lo, C::kColXk, it == 0);        // dK += dS^T Q
          if (p.ds_codes != nullptr) {
            // The compute warps also left the dS^T codes of this iteration in a staging tile: send it to the workspace.
            // Before the commit of bar_done below every earlier store has read its tile (with two tiles, all but this
            // one), and a warp waits for bar_done of iteration it before it writes the staging tile of it + 1.
            const int hq_it = hk * rep + it / n_qi, qt_it = qt0 + it % n_qi;
            const int ws_tile = ((b * p.H + hq_it) * n_t + qt_it) * n_t + kt;
            tma_store_2d(&tm_ds, sWs + (it % C::kWsBufs) * C::kCodeBytes, 0, ws_tile * 128);
            bulk_commit_group();
            bulk_wait_group_read<C::kWsBufs - 1>();
          }
        }
        tc_commit(empty + st);
        tc_commit(bar_done);
      }
      if (p.ds_codes != nullptr) bulk_wait_group<0>();
      if (!ok) raise_abort(abort_flag, p.status, kStatusTimeoutMma);
    }
  } else {
    // ------------------------------------------------------------------------------------------ compute groups
    const int wg = warp >> 2;                          // query blocks [wg * CH, wg * CH + CH) of every tile
    const int quad = warp & 3;                         // lane quadrant = 32-key block of the dS scale
    const int r = tid & 127;                           // key row inside the tile = TMEM lane
    const int blk0 = wg * CH;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const int key = kt * 128 + r;
    const int nblk = p.N / 32;
    const float ks_row = p.ks[static_cast<size_t>(bhk) * nblk + key / 32];
    const float vs_row = p.vs[static_cast<size_t>(bhk) * nblk + key / 32];
    const float2 nlog2e = splat2(-kLog2e);
    const uint32_t vec_a = smem_u32(sVec), xch_a = smem_u32(sXch), ws_a = smem_u32(sWs);
    bool ok = true;
    // iteration state kept incrementally: stage and its phase, query tile, and the scale pointers of (head, tile)
    int st = 0, qi = 0;
    uint32_t st_ph = 0;
    const float* qs_ptr = p.qs + static_cast<size_t>(b * p.H + hk * rep) * nblk + qt0 * 4 + blk0;
    const float* dos_ptr = p.dos + static_cast<size_t>(b * p.H + hk * rep) * nblk + qt0 * 4 + blk0;
    float qs_n[CH], dos_n[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      qs_n[c] = qs_ptr[c];
      dos_n[c] = dos_ptr[c];
    }
    int hq = hk * rep;                                   // query head of the iteration
    for (int it = 0; it < n_it; ++it) {
      const uint32_t ph = it & 1;
      const bool diag = p.causal && (qi == 0);           // the first query tile of a causal sweep is the diagonal one
      // workspace tile of this iteration (pass 2 reads it back as dS of query tile qt0 + qi, key tile kt)
      const size_t ws_tile = (static_cast<size_t>(b * p.H + hq) * n_t + (qt0 + qi)) * n_t + kt;
      float qs_c[CH], dos_c[CH];
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        qs_c[c] = qs_n[c];
        dos_c[c] = dos_n[c];
      }
      {                                                  // advance to the next (head, tile) and prefetch its scales
        const int step = (qi + 1 == n_qi) ? (nblk - (n_qi - 1) * 4) : 4;
        qs_ptr += step;
        dos_ptr += step;
        if (it + 1 < n_it) {
#pragma unroll
          for (int c = 0; c < CH; ++c) {
            qs_n[c] = qs_ptr[c];
            dos_n[c] = dos_ptr[c];
          }
        }
      }
      const uint32_t lse_a = vec_a + st * 1024 + 128 * blk0;       // shared-window addresses of lse / delta of the stage
      const uint32_t dl_a = lse_a + 512;
      float2 pr[CH][16];
      if (ok) ok = wait_warp(full + st, st_ph, abort_flag);       // lse / delta of the tile are in smem
      if (ok) ok = wait_warp(bar_s, ph, abort_flag);
      if (ok) {
        tc_fence_after();
        uint32_t rs[CH][32];
#pragma unroll
        for (int c = 0; c < CH; ++c) tmem_ld32(tmem + lane_base + C::kColSd + 32 * (blk0 + c), rs[c]);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if ((tid & 31) == 0) mbar_arrive(bar_sfree);
        uint32_t w[DV ? CH : 1][8], xv[DV ? CH : 1];
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          if (diag) {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (r > 32 * (blk0 + c) + e) rs[c][e] = 0xff800000u;   // -inf: key index above the query index
          }
          const float2 cc = splat2((ks_row * qs_c[c]) * kLog2e);
          float pm0 = 0.f, pm1 = 0.f;
#pragma unroll
          for (int e = 0; e < 16; e += 2) {
            const float4 l4 = lds_f4(lse_a + 4 * (32 * c + 2 * e));
            const float2 x0 = fma2(make_float2(__uint_as_float(rs[c][2 * e]), __uint_as_float(rs[c][2 * e + 1])), cc,
                                   mul2(make_float2(l4.x, l4.y), nlog2e));
            const float2 x1 = fma2(make_float2(__uint_as_float(rs[c][2 * e + 2]), __uint_as_float(rs[c][2 * e + 3])), cc,
                                   mul2(make_float2(l4.z, l4.w), nlog2e));
            pr[c][e] = ex2_2(x0);
            pr[c][e + 1] = ex2_2(x1);
            pm0 = max3(pm0, pr[c][e].x, pr[c][e].y);
            pm1 = max3(pm1, pr[c][e + 1].x, pr[c][e + 1].y);
          }
          if (DV) {
            // P^T codes: one power-of-two scale per (key row, 32 queries) = per thread, block and tile
            const uint32_t psb = pow2_sb(fmaxf(pm0, pm1), 0u);
            codes32(pr[c], sb_to_inv(psb), w[c]);
            xv[c] = sb_mul(psb, scale_to_sb(dos_c[c]));
          }
        }
        if (it > 0) ok = wait_warp(bar_done, ph ^ 1, abort_flag);   // the previous chains have read codes and words
        if (ok) {
          if (DV) {
#pragma unroll
            for (int c = 0; c < CH; ++c) {
              tmem_st8(tmem + lane_base + C::kColPc + 8 * (blk0 + c), w[c]);
              tmem_st4(tmem + lane_base + C::kColXv + 4 * (blk0 + c), xv[c], xv[c], xv[c], xv[c]);
            }
          }
          if (wg == 0) tmem_st4(tmem + lane_base + C::kColOne, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu);
          if (!DK) {                                       // a DV launch has no second half: the codes are the hand-off
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if ((tid & 31) == 0) mbar_arrive(bar_pv);
          }
        }
      }
      if (!DK) {                                           // DV launch: on to the next tile
        if (++st == C::kStages) {
          st = 0;
          st_ph ^= 1;
        }
        if (++qi == n_qi) {
          qi = 0;
          ++hq;
        }
        continue;
      }
      // dP^T (its chain was issued when S^T was handed back) is requested while the code stores are still in flight
      float wm = 0.f;
      if (ok) ok = wait_warp(bar_dp, ph, abort_flag);
      if (ok) {
        tc_fence_after();
        uint32_t rd[CH][32];
#pragma unroll
        for (int c = 0; c < CH; ++c) tmem_ld32(tmem + lane_base + C::kColSd + 32 * (blk0 + c), rd[c]);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if ((tid & 31) == 0) mbar_arrive(bar_dpfree);
        float am0 = 0.f, am1 = 0.f;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          // -dS = P (delta - dP_acc a): a is a power of two, so the product is exact; the sign is undone by the scale
          const float2 naa = splat2(-(vs_row * dos_c[c]));
#pragma unroll
          for (int e = 0; e < 16; e += 2) {
            const float4 d4 = lds_f4(dl_a + 4 * (32 * c + 2 * e));
            const float2 t0 = fma2(make_float2(__uint_as_float(rd[c][2 * e]), __uint_as_float(rd[c][2 * e + 1])), naa,
                                   make_float2(d4.x, d4.y));
            const float2 t1 = fma2(make_float2(__uint_as_float(rd[c][2 * e + 2]), __uint_as_float(rd[c][2 * e + 3])), naa,
                                   make_float2(d4.z, d4.w));
            pr[c][e] = mul2(pr[c][e], t0);
            pr[c][e + 1] = mul2(pr[c][e + 1], t1);
            am0 = max3(am0, fabsf(pr[c][e].x), fabsf(pr[c][e].y));
            am1 = max3(am1, fabsf(pr[c][e + 1].x), fabsf(pr[c][e + 1].y));
          }
        }
        wm = warp_max(fmaxf(am0, am1));
        if (!DS32 && (tid & 31) == 0) sts_f(xch_a + 4 * (ph * 16 + warp), wm);
      }
      // one dS scale per (128 queries x this quadrant's 32 keys): the groups' warps of the quadrant meet here (reached
      // in every iteration, also after a failed wait).  With 32 x 32 blocks the warp's own maximum is the block's.
      if (!DS32) bar_sync(1 + quad, 32 * C::kGroups);
      const int st_cur = st;
      if (++st == C::kStages) {
        st = 0;
        st_ph ^= 1;
      }
      if (++qi == n_qi) {
        qi = 0;
        ++hq;
      }
      (void)st_cur;
      if (!ok) continue;
      float am = wm;
      if (!DS32) {
        const uint32_t x_a = xch_a + 4 * (ph * 16 + quad);
        am = fmaxf(lds_f(x_a), lds_f(x_a + 16));
        if (C::kGroups == 4) am = fmaxf(am, fmaxf(lds_f(x_a + 32), lds_f(x_a + 48)));
      }
      const uint32_t dsb = pow2_sb(am, 127u);
      const float ninv = -sb_to_inv(dsb);
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        uint32_t w[8];
        codes32(pr[c], ninv, w);
        tmem_st8(tmem + lane_base + C::kColDc + 8 * (blk0 + c), w);
        const uint32_t xk = sb_mul(dsb, scale_to_sb(qs_c[c]));
        tmem_st4(tmem + lane_base + C::kColXk + 4 * (blk0 + c), xk, xk, xk, xk);
        if (p.ds_codes != nullptr) {
          // the same codes as a [key][query] tile in 128-byte-swizzled shared memory (16-byte chunk j of row r at
          // chunk j ^ (r % 8)); the MMA warp's thread stores the tile to the workspace for pass 2
          const uint32_t ws_row = ws_a + (it % C::kWsBufs) * C::kCodeBytes + r * 128;
          const int j = 2 * (blk0 + c);
          sts_u4(ws_row + ((j ^ (r & 7)) << 4), w[0], w[1], w[2], w[3]);
          sts_u4(ws_row + (((j + 1) ^ (r & 7)) << 4), w[4], w[5], w[6], w[7]);
        }
      }
      if (p.ds_codes != nullptr) fence_async_smem();
      // scale bytes of the tile for pass 2, [query block][key block]
      if (p.ds_codes != nullptr && (tid & 31) == 0) {
        if (DS32) {
          p.ds_words[ws_tile * 16 + blk0 * 4 + quad] = static_cast<uint8_t>(dsb);
        } else if (wg == 0) {
#pragma unroll
          for (int qb = 0; qb < 4; ++qb) p.ds_words[ws_tile * 16 + qb * 4 + quad] = static_cast<uint8_t>(dsb);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if ((tid & 31) == 0) mbar_arrive(bar_pk);
    }
    if (ok) ok = wait_warp(bar_done, (n_it - 1) & 1, abort_flag);
    if (!ok) {
      raise_abort(abort_flag, p.status, kStatusTimeoutCompute);
    } else {
      tc_fence_after();
      // every group writes its 32-column blocks of each 128-column slice of the accumulators
#pragma unroll 1
      for (int cc = 0; cc < C::kSub * CH; ++cc) {
        const int col = 128 * (cc / CH) + 32 * (blk0 + cc % CH);
        uint32_t rr[32];
        if (DV) {
          tmem_ld32(tmem + lane_base + C::kColDv + col, rr);
          tmem_wait_ld();
          store_bf16_chunk(rr, 1.0f, p.dv + static_cast<int64_t>(b) * p.dv_sb + static_cast<int64_t>(key) * p.dv_sn +
                                         static_cast<int64_t>(hk) * p.dv_sh + col);
        }
        if (DK) {
          tmem_ld32(tmem + lane_base + C::kColDk + col, rr);
          tmem_wait_ld();
          store_bf16_chunk(rr, 1.0f, p.dk + static_cast<int64_t>(b) * p.dk_sb + static_cast<int64_t>(key) * p.dk_sn +
                                         static_cast<int64_t>(hk) * p.dk_sh + col);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kW + 1) tmem_dealloc(tmem, C::kTmemCols);
}

// ================================================================================================ dQ
template <int D>
struct DqSerialCfg {
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
bwd_dq_serial_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do, const BwdParams p) {
  using C = DqSerialCfg<D>;
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
      const uint32_t q_lo = desc_lo(smem_u32(sQ)), do_lo = desc_lo(smem_u32(sDo)), ds_lo = desc_lo(smem_u32(sDs));
      const uint32_t k_lo0 = desc_lo(smem_u32(sK)), v_lo0 = desc_lo(smem_u32(sV));
      bool ok = wait_or_abort(bar_q, 0, abort_flag);
      for (int it = 0; ok && it < n_it; ++it) {
        const int st = it % C::kStages;
        if (!(ok = wait_or_abort(full + st, (it / C::kStages) & 1, abort_flag))) break;
        if (it > 0 && !(ok = wait_or_abort(bar_done, (it - 1) & 1, abort_flag))) break;
        tc_fence_after();
        const uint32_t k_lo = k_lo0 + st * (C::kTileBytes >> 4), v_lo = v_lo0 + st * (C::kTileBytes >> 4);
#pragma unroll
        for (int ks = 0; ks < D / 32; ++ks) {
          const uint32_t off = (ks / 4) * 1024 + (ks % 4) * 2;      // descriptor units of 16 bytes
          mma_f8_ss(tmem + C::kColS, q_lo + off, k_lo + off, kIdesc, ks > 0);
        }
#pragma unroll
        for (int ks = 0; ks < D / 32; ++ks) {
          const uint32_t off = (ks / 4) * 1024 + (ks % 4) * 2;
          mma_f8_ss(tmem + C::kColDp, do_lo + off, v_lo + off, kIdesc, ks > 0);
        }
        tc_commit(bar_s);
        if (!(ok = wait_or_abort(bar_p, it & 1, abort_flag))) break;
        tc_fence_after();
        // dQ += dS K: A = dS codes in shared memory (rows = queries, K-major), B = K tile MN-major (32 key rows per step)
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
          for (int s = 0; s < C::kSub; ++s) {
            mma_mxf8_ss(tmem + C::kColDq + s * 128, ds_lo + ks * 2, k_lo + s * 1024 + ks * 256,
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
      // (with 32 x 32 dS blocks the warp's own maximum is the block's)
      float* red = sRed + (it & 1) * 16;
      float wmx[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        wmx[c] = warp_max(bmax[c]);
        if ((tid & 31) == 0) red[warp * 4 + c] = wmx[c];
      }
      bar_sync(1, 128);          // reached by every compute warp in every iteration, also after a failed wait
      if (!ok) continue;
      uint32_t sfw[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float am = p.ds32 ? wmx[c] : fmaxf(fmaxf(red[c], red[4 + c]), fmaxf(red[8 + c], red[12 + c]));
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


// ================================================================================================ dQ, pipelined (D = 128)
// One CTA per SM, 576 threads.  Warps 0-15: four compute groups of four warps; group g owns key block g of every tile
// (32 key columns = one whole dS scale block of 128 queries x 32 keys; thread t % 128 = query row = TMEM lane), which
// puts four compute warps on every scheduler.  Warp 16: TMA.  Warp 17: MMA.  The groups pull S and dP of tile i into
// registers and hand the accumulators back at once, so the tensor pipe computes S, dP of tile i+1 while the groups take
// the exponentials of tile i; dS codes go to shared memory (double-buffered), the scale words to TMEM columns of their
// own, and dQ += dS K runs behind the next tile's compute.
struct DqCfg {
  static constexpr int kTileBytes = 128 * 128;
  static constexpr int kStages = 4;
  static constexpr int kGroups = 4;
  static constexpr int kThreads = kGroups * 128 + 64;
  static constexpr int kTmemCols = 512;
  static constexpr int kColS = 0, kColDp = 128, kColDq = 256;
  static constexpr int kColX = 384;          // 4 x 4 columns: scale word of key block g at kColX + 4 g (byte 0)
  static constexpr int kColOne = 400;        // 4 columns of 0x7F7F7F7F: scale 1.0 for the B operand
  static constexpr int kSmemQ = 0;
  static constexpr int kSmemDo = kTileBytes;
  static constexpr int kSmemK = 2 * kTileBytes;
  static constexpr int kSmemV = kSmemK + kStages * kTileBytes;
  static constexpr int kSmemDs = kSmemV + kStages * kTileBytes;      // 2 x (128 x 128 dS codes, rows = queries)
  static constexpr int kSmemRed = kSmemDs + 2 * kTileBytes;          // 2 x [16 warps] block maxima, then probe sums
  static constexpr int kSmemProbe = kSmemRed + 2 * 16 * 4;           // 3 slots x 3 groups x 128 rows x 2 doubles
  static constexpr int kSmemBar = kSmemProbe + 3 * 3 * 128 * 16;
  static constexpr int kSmemBytes = kSmemBar + 256 + 1024;
};

// Work item = one 128-query tile of one (batch, query head); persistent CTAs (one per SM) walk the item list with stride
// gridDim.x, heaviest items first, and the TMA / MMA pipeline runs across item boundaries.
struct DqWalk {                      // position of a role in the CTA's sequence of (item, key tile) pairs
  int item, it, n_it, qt, bh;
  uint32_t n_done;                   // items finished before the current one
};
__device__ __forceinline__ void dq_walk_set(DqWalk& w, const BwdParams& p, int n_t, int bh_count) {
  w.qt = n_t - 1 - w.item / bh_count;
  w.bh = w.item % bh_count;
  w.n_it = p.causal ? (w.qt + 1) : n_t;
  w.it = 0;
}

__global__ void __launch_bounds__(DqCfg::kThreads, 1)
bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do, const BwdParams p) {
  using C = DqCfg;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + C::kSmemQ;
  uint8_t* sDo = smem + C::kSmemDo;
  uint8_t* sK = smem + C::kSmemK;
  uint8_t* sV = smem + C::kSmemV;
  uint8_t* sDs = smem + C::kSmemDs;
  float* sRed = reinterpret_cast<float*>(smem + C::kSmemRed);
  double* sProbe = reinterpret_cast<double*>(smem + C::kSmemProbe);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kSmemBar);
  uint64_t* bar_q = bars + 0;        // Q and dO of the item landed
  uint64_t* bar_qfree = bars + 1;    // every MMA that reads Q / dO of the item is done
  uint64_t* bar_s = bars + 2;        // S and dP of the tile ready (MMA commit)
  uint64_t* bar_free = bars + 3;     // every compute warp holds its part of the tile in registers (16 arrivals)
  uint64_t* bar_p = bars + 4;        // dS codes and scale words written (16 arrivals)
  uint64_t* bar_done = bars + 5;     // dQ chain of the tile done (MMA commit)
  uint64_t* bar_dqfree = bars + 6;   // the item's dQ accumulator has been read out (16 arrivals)
  uint64_t* full = bars + 7;         // [kStages]
  uint64_t* empty = bars + 7 + C::kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7 + 2 * C::kStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 8 + 2 * C::kStages);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int n_t = p.N / 128;
  const int bh_count = p.B * p.H;
  const int n_items = n_t * bh_count;

  if (tid == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_qfree, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_free, C::kGroups * 4);
    mbar_init(bar_p, C::kGroups * 4);
    mbar_init(bar_done, 1);
    mbar_init(bar_dqfree, C::kGroups * 4);
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 17) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 16) {
    // ------------------------------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_do);
      uint32_t g = 0, n_done = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x, ++n_done) {
        const int qt = n_t - 1 - item / bh_count, bh = item % bh_count;
        const int bhk = (bh / p.H) * p.Hk + (bh % p.H) / (p.H / p.Hk);
        const int n_it = p.causal ? (qt + 1) : n_t;
        if (n_done > 0 && !(ok = wait_or_abort(bar_qfree, (n_done - 1) & 1, abort_flag))) break;
        mbar_expect_tx(bar_q, 2 * C::kTileBytes);
        tma_load_2d(sQ, &tm_q, bar_q, 0, bh * p.N + qt * 128);
        tma_load_2d(sDo, &tm_do, bar_q, 0, bh * p.N + qt * 128);
        for (int it = 0; it < n_it; ++it, ++g) {
          const uint32_t st = g % C::kStages;
          if (g >= C::kStages && !(ok = wait_or_abort(empty + st, ((g / C::kStages) - 1) & 1, abort_flag))) break;
          const int row = bhk * p.N + it * 128;
          mbar_expect_tx(full + st, 2 * C::kTileBytes);
          tma_load_2d(sK + st * C::kTileBytes, &tm_k, full + st, 0, row);
          tma_load_2d(sV + st * C::kTileBytes, &tm_v, full + st, 0, row);
        }
      }
      if (!ok) raise_abort(abort_flag, p.status, kStatusTimeoutProducer);
    }
  } else if (warp == 17) {
    // ------------------------------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t kIdesc = idesc_f8(128, 128, false, false);
      const uint32_t q_lo = desc_lo(smem_u32(sQ)), do_lo = desc_lo(smem_u32(sDo)), ds_lo0 = desc_lo(smem_u32(sDs));
      const uint32_t k_lo0 = desc_lo(smem_u32(sK)), v_lo0 = desc_lo(smem_u32(sV));
      bool ok = true;
      // `nx` runs one tile ahead of `cur`: S / dP of the next tile (possibly the first tile of the next item) are
      // issued as soon as the compute warps hold the current tile in registers.
      DqWalk cur{static_cast<int>(blockIdx.x), 0, 0, 0, 0, 0}, nx = cur;
      uint32_t g_nx = 0;                                // tiles whose S / dP have been issued
      auto issue_s_dp = [&]() -> bool {                 // for the tile `nx` points at; advances nx
        if (nx.it == 0 && !wait_or_abort(bar_q, nx.n_done & 1, abort_flag)) return false;
        const uint32_t st = g_nx % C::kStages;
        if (!wait_or_abort(full + st, (g_nx / C::kStages) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t k_lo = k_lo0 + st * (C::kTileBytes >> 4), v_lo = v_lo0 + st * (C::kTileBytes >> 4);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) mma_f8_ss(tmem + C::kColS, q_lo + ks * 2, k_lo + ks * 2, kIdesc, ks > 0);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) mma_f8_ss(tmem + C::kColDp, do_lo + ks * 2, v_lo + ks * 2, kIdesc, ks > 0);
        tc_commit(bar_s);
        ++g_nx;
        if (++nx.it == nx.n_it) {                       // last tile of the item: its Q / dO may be replaced
          tc_commit(bar_qfree);
          nx.item += gridDim.x;
          ++nx.n_done;
          if (nx.item < n_items) dq_walk_set(nx, p, n_t, bh_count);
        }
        return true;
      };
      if (cur.item < n_items) {
        dq_walk_set(cur, p, n_t, bh_count);
        nx = cur;
        ok = issue_s_dp();
      }
      uint32_t g = 0;                                   // tiles whose dQ chain has been issued
      while (ok && cur.item < n_items) {
        const uint32_t st = g % C::kStages;
        if (!(ok = wait_or_abort(bar_free, g & 1, abort_flag))) break;
        if (nx.item < n_items && !(ok = issue_s_dp())) break;
        if (!(ok = wait_or_abort(bar_p, g & 1, abort_flag))) break;
        // the first chain of an item overwrites the accumulator: the previous item's dQ must have been read out
        if (cur.it == 0 && cur.n_done > 0 && !(ok = wait_or_abort(bar_dqfree, (cur.n_done - 1) & 1, abort_flag))) break;
        tc_fence_after();
        // dQ += dS K: A = dS codes in shared memory (rows = queries, K-major), B = K tile MN-major (32 key rows per step)
        const uint32_t ds_lo = ds_lo0 + (g & 1) * (C::kTileBytes >> 4), k_lo = k_lo0 + st * (C::kTileBytes >> 4);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_mxf8_ss(tmem + C::kColDq, ds_lo + ks * 2, k_lo + ks * 256, idesc_mxf8(128, 128, false, true, 0, 0),
                      tmem + C::kColX + 4 * ks, tmem + C::kColOne, (cur.it > 0) || (ks > 0));
        tc_commit(empty + st);
        tc_commit(bar_done);
        ++g;
        if (++cur.it == cur.n_it) {
          cur.item += gridDim.x;
          ++cur.n_done;
          if (cur.item < n_items) dq_walk_set(cur, p, n_t, bh_count);
        }
      }
      if (!ok) raise_abort(abort_flag, p.status, kStatusTimeoutMma);
    }
  } else {
    // ------------------------------------------------------------------------------------------ compute groups
    const int wg = warp >> 2;
    const int r = tid & 127;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int nblk = p.N / 32;
    const bool probe = p.rowsum_ds != nullptr;
    uint32_t g = 0, n_done = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++n_done) {
      const int qt = n_t - 1 - item / bh_count, bh = item % bh_count;
      const int b = bh / p.H, h = bh % p.H;
      const int bhk = b * p.Hk + h / (p.H / p.Hk);
      const int n_it = p.causal ? (qt + 1) : n_t;
      const int row = qt * 128 + r;
      const float qs = p.qs[static_cast<size_t>(bh) * nblk + row / 32];
      const float dos = p.dos[static_cast<size_t>(bh) * nblk + row / 32];
      const float2 nl2 = splat2(-(p.lse[static_cast<size_t>(bh) * p.N + row] * kLog2e));
      const float2 ndl = splat2(-p.delta[static_cast<size_t>(bh) * p.N + row]);
      const float* ks_base = p.ks + static_cast<size_t>(bhk) * nblk + wg;
      const float* vs_base = p.vs + static_cast<size_t>(bhk) * nblk + wg;
      float ks1 = *ks_base, vs1 = *vs_base;
      double rs_acc = 0.0, ap_acc = 0.0;
      for (int it = 0; it < n_it; ++it, ++g) {
        const float ksv = ks1, vsv = vs1;
        if (it + 1 < n_it) {
          ks1 = ks_base[(it + 1) * 4];
          vs1 = vs_base[(it + 1) * 4];
        }
        const bool diag = p.causal && (it == qt);
        float2 v[16];
        float wm = 0.f;
        if (ok) ok = wait_warp(bar_s, g & 1, abort_flag);
        if (ok) {
          tc_fence_after();
          uint32_t rs[32], rd[32];
          tmem_ld32(tmem + lane_base + C::kColS + 32 * wg, rs);
          tmem_ld32(tmem + lane_base + C::kColDp + 32 * wg, rd);
          tmem_wait_ld();
          tc_fence_before();
          __syncwarp();
          if ((tid & 31) == 0) mbar_arrive(bar_free);    // this warp's part of the accumulators may be overwritten now
          if (diag) {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (32 * wg + e > r) rs[e] = 0xff800000u;  // -inf: key index above the query index
          }
          const float2 cc = splat2((ksv * qs) * kLog2e), aa = splat2(vsv * dos);
          float am0 = 0.f, am1 = 0.f;
          float2 rsum = make_float2(0.f, 0.f), asum = rsum;
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float2 pe = ex2_2(fma2(make_float2(__uint_as_float(rs[2 * e]), __uint_as_float(rs[2 * e + 1])), cc, nl2));
            const float2 dp = make_float2(__uint_as_float(rd[2 * e]), __uint_as_float(rd[2 * e + 1]));
            const float2 t = fma2(dp, aa, ndl);          // dP_acc * a - delta: a is a power of two, the product is exact
            const float2 d = mul2(pe, t);
            v[e] = d;
            if (e & 1) am1 = max3(am1, fabsf(d.x), fabsf(d.y));
            else am0 = max3(am0, fabsf(d.x), fabsf(d.y));
            if (probe) {
              rsum = add2(rsum, d);
              const float2 pd = mul2(pe, mul2(dp, aa));
              asum = add2(asum, make_float2(fabsf(pd.x), fabsf(pd.y)));
            }
          }
          if (probe) {
            rs_acc += static_cast<double>(rsum.x) + static_cast<double>(rsum.y);
            ap_acc += static_cast<double>(asum.x) + static_cast<double>(asum.y);
          }
          // one scale per (128 queries x 32 keys): the maxima of this group's four warps meet in shared memory
          // (with 32 x 32 dS blocks the warp's own maximum is the block's)
          wm = warp_max(fmaxf(am0, am1));
          if ((tid & 31) == 0) sRed[(g & 1) * 16 + warp] = wm;
        }
        bar_sync(1 + wg, 128);        // reached by every warp of the group in every iteration, also after a failed wait
        if (ok && g > 0) ok = wait_warp(bar_done, (g - 1) & 1, abort_flag);   // the previous chain has read its scale words
        if (!ok) continue;
        const float* red = sRed + (g & 1) * 16 + wg * 4;
        const uint32_t dsb = pow2_sb(p.ds32 ? wm : fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3])), 127u);
        uint32_t w[8];
        codes32(v, sb_to_inv(dsb), w);
        // row r of the dS tile: 16-byte chunk j of the row lands at chunk (j ^ (r % 8)) (128-byte swizzle)
        uint8_t* ds_row = sDs + (g & 1) * C::kTileBytes + r * 128;
        sts_u4(ds_row + (((2 * wg) ^ (r & 7)) << 4), w[0], w[1], w[2], w[3]);
        sts_u4(ds_row + (((2 * wg + 1) ^ (r & 7)) << 4), w[4], w[5], w[6], w[7]);
        const uint32_t word = sb_mul(dsb, scale_to_sb(ksv));
        tmem_st4(tmem + lane_base + C::kColX + 4 * wg, word, word, word, word);
        if (wg == 0) tmem_st4(tmem + lane_base + C::kColOne, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu);
        tmem_wait_st();
        fence_async_smem();
        tc_fence_before();
        __syncwarp();
        if ((tid & 31) == 0) mbar_arrive(bar_p);
      }
      // item epilogue: dQ of the item out of TMEM, then hand the accumulator to the next item
      if (ok) ok = wait_warp(bar_done, (g - 1) & 1, abort_flag);
      if (ok) {
        tc_fence_after();
        __nv_bfloat16* dst = p.dq + static_cast<int64_t>(b) * p.dq_sb + static_cast<int64_t>(row) * p.dq_sn +
                             static_cast<int64_t>(h) * p.dq_sh + 32 * wg;
        uint32_t rr[32];
        tmem_ld32(tmem + lane_base + C::kColDq + 32 * wg, rr);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if ((tid & 31) == 0) mbar_arrive(bar_dqfree);
        store_bf16_chunk(rr, p.sm_scale, dst);
      }
      if (probe) {                     // identity probe: the groups' partial row sums meet in shared memory
        const int slot = n_done % 3;   // slots and barriers rotate: a warp is at most two items ahead of another
        double* pr = sProbe + slot * (3 * 128 * 2);
        if (wg > 0) {
          pr[((wg - 1) * 128 + r) * 2] = rs_acc;
          pr[((wg - 1) * 128 + r) * 2 + 1] = ap_acc;
          bar_arrive(5 + slot, C::kGroups * 128);
        } else {
          bar_sync(5 + slot, C::kGroups * 128);
          for (int gi = 0; gi < C::kGroups - 1; ++gi) {
            rs_acc += pr[(gi * 128 + r) * 2];
            ap_acc += pr[(gi * 128 + r) * 2 + 1];
          }
          if (ok) {
            p.rowsum_ds[static_cast<size_t>(bh) * p.N + row] = static_cast<float>(rs_acc);
            p.sum_abs_pdp[static_cast<size_t>(bh) * p.N + row] = static_cast<float>(ap_acc);
          }
        }
      }
    }
    if (!ok) raise_abort(abort_flag, p.status, kStatusTimeoutCompute);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 17) tmem_dealloc(tmem, C::kTmemCols);
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

template <int D, bool DV, bool DK, bool DS32>
static cudaError_t launch_kv_pipe_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                                    const CUtensorMap& tdo, const CUtensorMap& tds, const BwdParams& p,
                                    cudaStream_t stream) {
  using C = KvPipeCfg<4, D, DV, DK>;
  static bool done[64] = {};
  cudaError_t e = set_smem(bwd_dkdv_pipe_kernel<4, D, DV, DK, DS32>, C::kSmemBytes, done);
  if (e != cudaSuccess) return e;
  dim3 grid(p.N / 128, p.B * p.Hk);
  bwd_dkdv_pipe_kernel<4, D, DV, DK, DS32><<<grid, C::kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, tds, p);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_bwd_dkdv(int D, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                            const CUtensorMap& tdo, const CUtensorMap* tds_or_null, const BwdParams& p,
                            cudaStream_t stream) {
  const CUtensorMap* tds = (tds_or_null != nullptr) ? tds_or_null : &tq;     // unused by the kernel without a workspace
  if (D == 128) {
    return p.ds32 ? launch_kv_pipe_t<128, true, true, true>(tq, tk, tv, tdo, *tds, p, stream)
                  : launch_kv_pipe_t<128, true, true, false>(tq, tk, tv, tdo, *tds, p, stream);
  }
  // head_dim 256: one accumulator fills 256 of the 512 TMEM columns, so dV and dK run as two launches of the same kernel
  cudaError_t e = launch_kv_pipe_t<256, true, false, false>(tq, tk, tv, tdo, *tds, p, stream);
  if (e != cudaSuccess) return e;
  return p.ds32 ? launch_kv_pipe_t<256, false, true, true>(tq, tk, tv, tdo, *tds, p, stream)
                : launch_kv_pipe_t<256, false, true, false>(tq, tk, tv, tdo, *tds, p, stream);
}

template <int D>
static cudaError_t launch_dq_serial_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                                      const CUtensorMap& tdo, const BwdParams& p, cudaStream_t stream) {
  using C = DqSerialCfg<D>;
  static bool done[64] = {};
  cudaError_t e = set_smem(bwd_dq_serial_kernel<D>, C::kSmemBytes, done);
  if (e != cudaSuccess) return e;
  dim3 grid(p.N / 128, p.B * p.H);
  bwd_dq_serial_kernel<D><<<grid, 192, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_bwd_dq(int D, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                          const CUtensorMap& tdo, const BwdParams& p, cudaStream_t stream) {
  // head_dim 256: dQ alone fills 256 TMEM columns, which leaves no room for the pipelined kernel's separate scale-word
  // columns; it keeps the kernel that serialises MMA and compute inside a CTA.
  if (D != 128) return launch_dq_serial_t<256>(tq, tk, tv, tdo, p, stream);
  static bool done[64] = {};
  cudaError_t e = set_smem(bwd_dq_kernel, DqCfg::kSmemBytes, done);
  if (e != cudaSuccess) return e;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int n_items = (p.N / 128) * p.B * p.H;
  bwd_dq_kernel<<<n_items < sms ? n_items : sms, DqCfg::kThreads, DqCfg::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);
  count_launch();
  return cudaGetLastError();
}

}  // namespace dm
