// Pass 0 of the backward: the matched delta.  For every query row, delta_i = sum_j P_ij dP_ij / sum_j P_ij with P and dP
// recomputed from the fp8 codes exactly as the backward recomputes them, so that rowsum(dS) = 0 holds at fp32 round-off.
//
// Arithmetic shared with the backward (delta_matching/sm100/attention_math_sm100.py:26-45; emulation
// delta_matching/reference.py:483, 491, 526-535):
//   c = (ks_b * qs) * log2e;  l2 = lse * log2e;  P = ex2(fma(S_acc, c, -l2));  a = vs_b * dos;  dP = dP_acc * a.
// Sums: four fp32 FMA chains of 8 elements per 32-key block (the power-of-two factor a is applied once per block,
// which is exact), block sums accumulated across key tiles as compensated fp32 pairs (TwoSum), folded in fp64 at the
// end; one fp64 divide and one fp32 store per row.
//
// One persistent CTA per SM; a work item is one 128-query tile of one (batch, query head).  S = Q8 K8^T and dP = dO8 V8^T run on tcgen05
// (kind::f8f6f4) into TMEM accumulators that are double-buffered (2 x (128 + 128) columns), so the tensor pipe works on
// key tile i+1 while the compute warps take the exponentials of tile i.  Four compute groups of four warps (warps 0-15)
// split the 128 key columns of a tile, 32 each, i.e. one K/V scale block per group (thread t of every group = TMEM lane
// t % 128 = query row), which puts four compute warps on every scheduler: enough to keep the MUFU pipe fed while one
// warp waits for TMEM or an mbarrier.  Warp 16 issues TMA loads, warp 17 the MMAs.  The four partial sums of a row meet
// once, at the end, in shared memory.
#include "dm_common.cuh"
#include "dm_kernels.h"

namespace dm {

template <int D>
struct DeltaCfg {
  static constexpr int kSub = D / 128;
  static constexpr int kTileBytes = 128 * D;
  static constexpr int kStages = (D == 128) ? 5 : 2;
  static constexpr int kTmemCols = 512;
  static constexpr int kSmemQ = 0;
  static constexpr int kSmemDo = kTileBytes;
  static constexpr int kSmemK = 2 * kTileBytes;
  static constexpr int kSmemV = kSmemK + kStages * kTileBytes;
  static constexpr int kGroups = 4;                                     // compute groups, 32 key columns each
  static constexpr int kThreads = kGroups * 128 + 64;
  static constexpr int kSmemRed = kSmemV + kStages * kTileBytes;        // 3 slots x 3 groups x 128 rows x (num, den) doubles
  static constexpr int kSmemBar = kSmemRed + 3 * 3 * 128 * 16;
  static constexpr int kSmemBytes = kSmemBar + 256 + 1024;
};

// Work item = one 128-query tile of one (batch, query head).  The kernel is persistent: gridDim.x CTAs (one per SM) walk
// the item list with stride gridDim.x.  Items are ordered by decreasing length (causal: the last query tile of every
// head first), so the static round-robin split is balanced to within one item, and the TMA / MMA pipeline runs across
// item boundaries: the next item's Q / dO and first key tiles are in flight while the current item's last tiles are
// still being reduced.
__device__ __forceinline__ void delta_item(int item, int n_qt, int bh_count, int& qt, int& bh) {
  qt = n_qt - 1 - item / bh_count;
  bh = item % bh_count;
}

template <int D>
__global__ void __launch_bounds__(DeltaCfg<D>::kThreads, 1)
delta_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
             const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do, const DeltaParams p) {
  using C = DeltaCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + C::kSmemQ;
  uint8_t* sDo = smem + C::kSmemDo;
  uint8_t* sK = smem + C::kSmemK;
  uint8_t* sV = smem + C::kSmemV;
  double* sRed = reinterpret_cast<double*>(smem + C::kSmemRed);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kSmemBar);
  uint64_t* bar_q = bars + 0;      // Q and dO of the item landed
  uint64_t* bar_qfree = bars + 1;  // every MMA that reads Q / dO of the item is done
  uint64_t* bar_s = bars + 2;      // [2] S and dP of the buffer ready (MMA commit)
  uint64_t* bar_c = bars + 4;      // [2] every compute warp has loaded its part of the buffer (one arrival per warp)
  uint64_t* full = bars + 6;       // [kStages] K and V of the stage landed
  uint64_t* empty = bars + 6 + C::kStages;   // [kStages] the MMAs reading the stage are done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6 + 2 * C::kStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 7 + 2 * C::kStages);
  uint64_t* bar_pub = bars + 20;   // [3] parts 1-3 have published their partial sums of the item (rotating slots)
  uint64_t* bar_read = bars + 23;  // [3] part 0 has read the slot
  static_assert(7 + 2 * C::kStages < 20, "barrier block layout");

  const int tid = threadIdx.x, warp = tid >> 5;
  const int n_qt = p.N / 128;
  const int bh_count = p.B * p.H;
  const int n_items = n_qt * bh_count;

  if (tid == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_qfree, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_s + s, 1);
      mbar_init(bar_c + s, C::kGroups * 2);              // one arrival per warp of the team that owns the tile
    }
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int s = 0; s < 3; ++s) {
      mbar_init(bar_pub + s, (C::kGroups - 1) * 4);
      mbar_init(bar_read + s, 4);
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
      uint32_t g = 0, n_done = 0;                      // key tiles issued so far; items started so far
      bool ok = true;
      for (int k = 0, item; ok && (item = sched_item(k, blockIdx.x, gridDim.x)) < n_items; ++k, ++n_done) {
        int qt, bh;
        delta_item(item, n_qt, bh_count, qt, bh);
        const int bhk = (bh / p.H) * p.Hk + (bh % p.H) / (p.H / p.Hk);
        const int n_it = p.causal ? (qt + 1) : n_qt;
        if (n_done > 0 && !(ok = wait_or_abort(bar_qfree, (n_done - 1) & 1, abort_flag))) break;
        mbar_expect_tx(bar_q, 2 * C::kTileBytes);
        for (int s = 0; s < C::kSub; ++s) {
          tma_load_2d(sQ + s * 16384, &tm_q, bar_q, s * 128, bh * p.N + qt * 128);
          tma_load_2d(sDo + s * 16384, &tm_do, bar_q, s * 128, bh * p.N + qt * 128);
        }
        for (int it = 0; it < n_it; ++it, ++g) {
          const uint32_t st = g % C::kStages;
          if (g >= C::kStages && !(ok = wait_or_abort(empty + st, ((g / C::kStages) - 1) & 1, abort_flag))) break;
          const int row = bhk * p.N + it * 128;          // key tiles in ascending order
          mbar_expect_tx(full + st, 2 * C::kTileBytes);
          for (int s = 0; s < C::kSub; ++s) {
            tma_load_2d(sK + st * C::kTileBytes + s * 16384, &tm_k, full + st, s * 128, row);
            tma_load_2d(sV + st * C::kTileBytes + s * 16384, &tm_v, full + st, s * 128, row);
          }
        }
      }
      if (!ok) raise_abort(abort_flag, p.status, kStatusTimeoutProducer);
    }
  } else if (warp == 17) {
    // ------------------------------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t kIdesc = idesc_f8(128, 128, false, false);
      const uint32_t q_lo = desc_lo(smem_u32(sQ)), do_lo = desc_lo(smem_u32(sDo));
      const uint32_t k_lo0 = desc_lo(smem_u32(sK)), v_lo0 = desc_lo(smem_u32(sV));
      uint32_t g = 0, n_done = 0;
      bool ok = true;
      for (int k = 0, item; ok && (item = sched_item(k, blockIdx.x, gridDim.x)) < n_items; ++k, ++n_done) {
        int qt, bh;
        delta_item(item, n_qt, bh_count, qt, bh);
        const int n_it = p.causal ? (qt + 1) : n_qt;
        if (!(ok = wait_or_abort(bar_q, n_done & 1, abort_flag))) break;
        for (int it = 0; it < n_it; ++it, ++g) {
          const uint32_t st = g % C::kStages, buf = g & 1;
          // the accumulator pair `buf` was last used two tiles ago: wait until every compute warp has read it
          if (g >= 2 && !(ok = wait_or_abort(bar_c + buf, ((g - 2) >> 1) & 1, abort_flag))) break;
          if (!(ok = wait_or_abort(full + st, (g / C::kStages) & 1, abort_flag))) break;
          tc_fence_after();
          const uint32_t k_lo = k_lo0 + st * (C::kTileBytes >> 4), v_lo = v_lo0 + st * (C::kTileBytes >> 4);
          const uint32_t t_s = tmem + buf * 256, t_dp = t_s + 128;
#pragma unroll
          for (int ks = 0; ks < D / 32; ++ks) {
            const uint32_t off = (ks / 4) * 1024 + (ks % 4) * 2;      // descriptor units of 16 bytes
            mma_f8_ss(t_s, q_lo + off, k_lo + off, kIdesc, ks > 0);
          }
#pragma unroll
          for (int ks = 0; ks < D / 32; ++ks) {
            const uint32_t off = (ks / 4) * 1024 + (ks % 4) * 2;
            mma_f8_ss(t_dp, do_lo + off, v_lo + off, kIdesc, ks > 0);
          }
          tc_commit(empty + st);
          tc_commit(bar_s + buf);
        }
        tc_commit(bar_qfree);
      }
      if (!ok) raise_abort(abort_flag, p.status, kStatusTimeoutMma);
    }
  } else {
    // ------------------------------------------------------------------------------------------ compute groups
    const int r = tid & 127;                           // query row inside the tile = TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    // Two teams of eight warps alternate over the key tiles, so that one team's waits and TMEM loads run behind the other
    // team's exponentials.  A team owns one S / dP buffer, i.e. the tiles of one parity of the CTA's running tile count
    // (it waits on every phase of that buffer's barriers, so the phase parity is never ambiguous).  A thread takes 64
    // key columns of a tile as two 32-column blocks.  Inside an item the team's tiles are those of one parity q of the
    // tile index; the partial sums are filed under (q, column half), so that what is summed, and in which order, depends
    // on the item only and not on which team did it.
    const int team = warp >> 3;
    const int half = (warp >> 2) & 1;
    const int blk0 = 2 * half;                          // first of the thread's two key blocks (32 keys each)
    const int nblk = p.N / 32;
    uint32_t g = 0, n_done = 0;
    bool ok = true;
    for (int k = 0, item; (item = sched_item(k, blockIdx.x, gridDim.x)) < n_items; ++k, ++n_done) {
      int qt, bh;
      delta_item(item, n_qt, bh_count, qt, bh);
      const int bhk = (bh / p.H) * p.Hk + (bh % p.H) / (p.H / p.Hk);
      const int n_it = p.causal ? (qt + 1) : n_qt;
      const int row = qt * 128 + r;
      const float qs = p.qs[static_cast<size_t>(bh) * nblk + row / 32];
      const float dos = p.dos[static_cast<size_t>(bh) * nblk + row / 32];
      const float2 nl2 = splat2(-(p.lse[static_cast<size_t>(bh) * p.N + row] * kLog2e));
      const float* ks_base = p.ks + static_cast<size_t>(bhk) * nblk + blk0;
      const float* vs_base = p.vs + static_cast<size_t>(bhk) * nblk + blk0;
      const int q = team ^ static_cast<int>(g & 1);    // parity of this team's tile indices inside the item
      const int part = 2 * q + half;                   // index of this thread's partial sums in the item fold
      float2 ks1 = make_float2(0.f, 0.f), vs1 = ks1;
      if (q < n_it) {
        ks1 = *reinterpret_cast<const float2*>(ks_base + q * 4);
        vs1 = *reinterpret_cast<const float2*>(vs_base + q * 4);
      }
      // running sums as unevaluated fp32 pairs (hi + lo, TwoSum): exact to ~2^-48 relative without the fp64 pipe
      float num_hi = 0.f, num_lo = 0.f, den_hi = 0.f, den_lo = 0.f;
      for (int it = q; ok && it < n_it; it += 2) {
        const uint32_t gt = g + it;                    // the CTA's running tile count selects buffer and barrier phase
        const uint32_t buf = gt & 1;
        const float kss[2] = {ks1.x, ks1.y}, vss[2] = {vs1.x, vs1.y};
        if (it + 2 < n_it) {                           // scales of the team's next key tile, in flight during this one
          ks1 = *reinterpret_cast<const float2*>(ks_base + (it + 2) * 4);
          vs1 = *reinterpret_cast<const float2*>(vs_base + (it + 2) * 4);
        }
        const bool diag = p.causal && (it == qt);
        if (!(ok = wait_warp(bar_s + buf, (gt >> 1) & 1, abort_flag))) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int blk = blk0 + c;
          const float2 c2 = splat2((kss[c] * qs) * kLog2e);
          // a = vs * dos is a power of two, so P * (dP_acc * a) == (P * dP_acc) * a exactly: a is applied once per block
          const float a = vss[c] * dos;
          uint32_t s[32], dp[32];
          tmem_ld32(tmem + lane_base + buf * 256 + 32 * blk, s);
          tmem_ld32(tmem + lane_base + buf * 256 + 128 + 32 * blk, dp);
          tmem_wait_ld();
          if (c == 1) {                                // both blocks of this warp are in registers: hand the buffer back
            tc_fence_before();
            __syncwarp();
            if ((tid & 31) == 0) mbar_arrive(bar_c + buf);
          }
          if (diag) {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (32 * blk + e > r) s[e] = 0xff800000u;   // -inf: key index above the query index
          }
          float2 n0 = make_float2(0.f, 0.f), n1 = n0, d0 = n0, d1 = n0;
#pragma unroll
          for (int e = 0; e < 16; e += 2) {
            // every exponential is ex2.approx of the same fma as in the backward kernels: P is bitwise the backward's P
            const float2 p0 = ex2_2(fma2(make_float2(__uint_as_float(s[2 * e]), __uint_as_float(s[2 * e + 1])), c2, nl2));
            const float2 p1 = ex2_2(fma2(make_float2(__uint_as_float(s[2 * e + 2]), __uint_as_float(s[2 * e + 3])), c2, nl2));
            n0 = fma2(p0, make_float2(__uint_as_float(dp[2 * e]), __uint_as_float(dp[2 * e + 1])), n0);
            n1 = fma2(p1, make_float2(__uint_as_float(dp[2 * e + 2]), __uint_as_float(dp[2 * e + 3])), n1);
            d0 = add2(d0, p0);
            d1 = add2(d1, p1);
          }
          const float nb = ((n0.x + n0.y) + (n1.x + n1.y)) * a;
          const float db = (d0.x + d0.y) + (d1.x + d1.y);
          two_sum_acc(num_hi, num_lo, nb);
          two_sum_acc(den_hi, den_lo, db);
        }
      }
      g += static_cast<uint32_t>(n_it);
      // Fold the four partial sums of a row in fp64: parts 1-3 publish, part 0 adds in part order and stores.  The slots
      // (shared memory and two mbarriers each) rotate over three items: a publisher writes slot n % 3 only after part 0
      // has read item n - 3 out of it, which also bounds how far a team can run ahead (it has no tile in a one-tile item).
      const int slot = n_done % 3;
      const uint32_t slot_phase = (n_done / 3) & 1;
      double* red = sRed + slot * (3 * 128 * 2);
      const double num = static_cast<double>(num_hi) + static_cast<double>(num_lo);
      const double den = static_cast<double>(den_hi) + static_cast<double>(den_lo);
      if (part > 0) {
        if (ok && n_done >= 3) ok = wait_warp(bar_read + slot, slot_phase ^ 1, abort_flag);
        red[((part - 1) * 128 + r) * 2] = num;
        red[((part - 1) * 128 + r) * 2 + 1] = den;
        __syncwarp();
        if ((tid & 31) == 0) mbar_arrive(bar_pub + slot);
      } else {
        if (ok) ok = wait_warp(bar_pub + slot, slot_phase, abort_flag);
        double n = num, dd = den;
#pragma unroll
        for (int gi = 0; gi < C::kGroups - 1; ++gi) {
          n += red[(gi * 128 + r) * 2];
          dd += red[(gi * 128 + r) * 2 + 1];
        }
        __syncwarp();
        if ((tid & 31) == 0) mbar_arrive(bar_read + slot);
        if (ok) p.delta[static_cast<size_t>(bh) * p.N + row] = static_cast<float>(p.norm ? n / dd : n);
      }
    }
    if (!ok) raise_abort(abort_flag, p.status, kStatusTimeoutCompute);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 17) tmem_dealloc(tmem, C::kTmemCols);
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
  static int sm_count[64] = {};
  if (dev >= 0 && dev < 64 && sm_count[dev] == 0) {
    cudaError_t e = cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
  }
  const int n_items = (p.N / 128) * p.B * p.H;
  const int ctas = (dev >= 0 && dev < 64) ? sm_count[dev] : 148;
  delta_kernel<D><<<n_items < ctas ? n_items : ctas, C::kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_delta(int D, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                         const CUtensorMap& tdo, const DeltaParams& p, cudaStream_t stream) {
  return D == 128 ? launch_delta_t<128>(tq, tk, tv, tdo, p, stream) : launch_delta_t<256>(tq, tk, tv, tdo, p, stream);
}

}  // namespace dm
