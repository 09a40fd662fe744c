// Backward pass 2: dQ = dS K from the quantised dS tiles that the dK / dV kernel left in a workspace.
//
// Reference structure: pass 1 writes dS codes, pass 2 multiplies them with K
// (csrc/fq8_dq_pass2_hd128.h:407-442, launched from csrc/flash_bwd_fp8v10_launch.h:158-163).  The alternative without a
// workspace (dm_bwd.cu: bwd_dq_kernel) recomputes S, dP and the exponentials per tile; this kernel only streams
// 16 KiB dS^T tiles and K tiles through one block-scaled MMA chain per tile, so it is bound by the L2 / HBM stream.
//
// Workspace: tile (head bh, query tile qt, key tile kt) at index (bh * n_t + qt) * n_t + kt holds 128 x 128 e4m3 codes
// as [key][query] (the layout the dK chain consumes), followed after all tiles by four 32-bit words per tile: word b
// belongs to query block b (32 queries) and its byte j is the UE8M0 scale of key block j (32 keys).  With the contract's
// dS blocks of 128 queries x 32 keys the four words of a tile are equal; with 32 x 32 blocks they differ.  The tile is the A operand of dQ in MN-major form
// (M = queries contiguous); K is the B operand in MN-major form as in the other kernels.
//
// One persistent CTA per SM, 320 threads: warps 0-3 write the per-tile scale words into TMEM (byte j = dS scale x K
// scale of key block j; warp b writes the word of query block b into its 32 rows), warps 4-7 write dQ out (at head_dim 128 two accumulators alternate
// between items; at head_dim 256 one accumulator fills the columns, and an item's first chain waits for the read-out
// of the previous item), warp 8 TMA, warp 9 MMA.  Items = (query tile, head), most key tiles first.
#include <cuda_bf16.h>
#include "dm_common.cuh"
#include "dm_kernels.h"
#include "dm_ptx.cuh"

namespace dm {

template <int D>
struct DqP2Cfg {
  static constexpr int kSub = D / 128;           // 128-byte-wide sub-tiles of a K row
  static constexpr int kDsBytes = 128 * 128;     // dS^T tile
  static constexpr int kKBytes = 128 * D;        // K tile
  static constexpr int kStages = (D == 128) ? 7 : 4;   // dS^T tile + K tile + scale word per stage (224 / 192 KiB)
  static constexpr int kAccs = (D == 128) ? 2 : 1;     // dQ accumulators of D fp32 columns
  static constexpr int kThreads = 320;
  static constexpr int kTmemCols = 512;
  static constexpr int kColDq = 0;
  static constexpr int kColSf = 256;           // kStages x 4 columns: the tile's scale word
  static constexpr int kColOne = 256 + 4 * kStages;   // 4 columns of 0x7F7F7F7F: scale 1.0 for the B operand
  static constexpr int kSmemDs = 0;
  static constexpr int kSmemK = kStages * kDsBytes;
  static constexpr int kSmemBar = kStages * (kDsBytes + kKBytes);
  static constexpr int kSmemBytes = kSmemBar + 256 + 1024;
  static_assert(kSmemBytes <= 232448, "shared memory budget");
};

template <int D>
__global__ void __launch_bounds__(DqP2Cfg<D>::kThreads, 1)
bwd_dq_p2_kernel(const __grid_constant__ CUtensorMap tm_ds, const __grid_constant__ CUtensorMap tm_k, const BwdParams p) {
  using C = DqP2Cfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sDs = smem + C::kSmemDs;
  uint8_t* sK = smem + C::kSmemK;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kSmemBar);
  // One barrier pair per stage keeps the MMA thread's loop short (one wait, four MMAs, one commit per tile): `full`
  // collects the TMA transaction and one arrival per scale warp, `empty` (MMA commit) releases the stage's shared memory
  // to the TMA warp and its scale-word columns to the scale warps.
  uint64_t* full = bars + 0;          // [kStages] tiles landed and scale word written
  uint64_t* empty = bars + C::kStages;          // [kStages] the stage's chain has read them (MMA commit)
  uint64_t* dq_full = bars + 2 * C::kStages;     // [2] last chain of the item done (MMA commit)
  uint64_t* dq_free = bars + 2 * C::kStages + 2; // [2] accumulator read out (one arrival per epilogue warp)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * C::kStages + 5);
  static_assert(2 * C::kStages + 6 <= 32, "barrier block is 256 bytes");

  const int tid = threadIdx.x, warp = tid >> 5;
  const int n_t = p.N / 128;
  const int BH = p.B * p.H;
  const int n_items = n_t * BH;
  const int rep = p.H / p.Hk;
  const int nblk = p.N / 32;
  const int first_item = static_cast<int>(blockIdx.x), item_step = static_cast<int>(gridDim.x);

  if (tid == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(full + s, 1 + 4);
      mbar_init(empty + s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(dq_full + s, 1);
      mbar_init(dq_free + s, 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 8) {
    // ------------------------------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tm_ds);
      tma_prefetch_desc(&tm_k);
      bool ok = true;
      uint32_t g = 0;
      for (int k = 0, item; ok && (item = sched_item(k, first_item, item_step)) < n_items; ++k) {
        const int qt = n_t - 1 - item / BH, bh = item % BH;
        const int bhk = (bh / p.H) * p.Hk + (bh % p.H) / rep;
        const int n_it = p.causal ? (qt + 1) : n_t;
        const int tile0 = (bh * n_t + qt) * n_t;
        for (int it = 0; it < n_it; ++it, ++g) {
          const uint32_t st = g % C::kStages;
          if (g >= C::kStages && !(ok = wait_or_abort(empty + st, ((g / C::kStages) - 1) & 1, abort_flag))) break;
          mbar_expect_tx(full + st, C::kDsBytes + C::kKBytes);
          tma_load_2d(sDs + st * C::kDsBytes, &tm_ds, full + st, 0, (tile0 + it) * 128);
          for (int sub = 0; sub < C::kSub; ++sub)
            tma_load_2d(sK + st * C::kKBytes + sub * 16384, &tm_k, full + st, sub * 128, bhk * p.N + it * 128);
        }
      }
      if (!ok) raise_abort(abort_flag, p.status, kStatusTimeoutProducer);
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t ds_lo0 = desc_lo(smem_u32(sDs)), k_lo0 = desc_lo(smem_u32(sK));
      bool ok = true;
      uint32_t g = 0, n_done = 0;
      for (int k = 0, item; ok && (item = sched_item(k, first_item, item_step)) < n_items; ++k, ++n_done) {
        const int qt = n_t - 1 - item / BH;
        const int n_it = p.causal ? (qt + 1) : n_t;
        const uint32_t acc = n_done % C::kAccs;
        // the accumulator was last used kAccs items ago: its read-out must be complete
        if (n_done >= C::kAccs && !(ok = wait_or_abort(dq_free + acc, ((n_done / C::kAccs) - 1) & 1, abort_flag))) break;
        for (int it = 0; it < n_it; ++it, ++g) {
          const uint32_t st = g % C::kStages;
          if (!(ok = wait_or_abort(full + st, (g / C::kStages) & 1, abort_flag))) break;
          tc_fence_after();
          // dQ += dS K over the tile's 128 keys: A = dS^T tile read MN-major, B = K tile read MN-major; both advance
          // by 32 key rows (4096 bytes) per step; byte ks of the scale word belongs to key block ks
          const uint32_t ds_lo = ds_lo0 + st * (C::kDsBytes >> 4), k_lo = k_lo0 + st * (C::kKBytes >> 4);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
            for (int sub = 0; sub < C::kSub; ++sub)
              mma_mxf8_ss(tmem + C::kColDq + D * acc + 128 * sub, ds_lo + ks * 256, k_lo + sub * 1024 + ks * 256,
                          idesc_mxf8(128, 128, true, true, ks, 0), tmem + C::kColSf + 4 * st, tmem + C::kColOne,
                          (it > 0) || (ks > 0));
          }
          tc_commit(empty + st);
          if (it == n_it - 1) tc_commit(dq_full + acc);
        }
      }
      if (!ok) raise_abort(abort_flag, p.status, kStatusTimeoutMma);
    }
  } else if (warp < 4) {
    // ------------------------------------------------------------------------------------------ scale words
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t* words = reinterpret_cast<const uint32_t*>(p.ds_words);
    tmem_st4(tmem + lane_base + C::kColOne, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu);
    bool ok = true;
    // The tile's dS scale word and its four K scales come from global memory: they are requested kAhead tiles before
    // they are used, through a walk over the CTA's (item, key tile) sequence that runs ahead of the consuming one.
    constexpr int kAhead = 4;
    struct Walk {
      int k, item, it, n_it;
      const uint32_t* w_ptr;
      const float4* ks_ptr;
    };
    auto walk_set = [&](Walk& wk) {
      if (wk.item >= n_items) return;
      const int qt = n_t - 1 - wk.item / BH, bh = wk.item % BH;
      const int bhk = (bh / p.H) * p.Hk + (bh % p.H) / rep;
      wk.it = 0;
      wk.n_it = p.causal ? (qt + 1) : n_t;
      wk.w_ptr = words + static_cast<size_t>(bh * n_t + qt) * n_t * 4 + warp;   // this warp's query block of each tile
      wk.ks_ptr = reinterpret_cast<const float4*>(p.ks + static_cast<size_t>(bhk) * nblk);
    };
    auto walk_next = [&](Walk& wk) {
      if (++wk.it == wk.n_it) {
        wk.item = sched_item(++wk.k, first_item, item_step);
        walk_set(wk);
      }
    };
    Walk pre{0, first_item, 0, 0, nullptr, nullptr};
    walk_set(pre);
    uint32_t w_q[kAhead];
    float4 k_q[kAhead];
#pragma unroll
    for (int i = 0; i < kAhead; ++i) {
      w_q[i] = 0;
      k_q[i] = make_float4(1.f, 1.f, 1.f, 1.f);
      if (pre.item < n_items) {
        w_q[i] = pre.w_ptr[4 * pre.it];
        k_q[i] = pre.ks_ptr[pre.it];
        walk_next(pre);
      }
    }
    uint32_t g = 0;
    for (int k = 0, item; ok && (item = sched_item(k, first_item, item_step)) < n_items; ++k) {
      const int qt = n_t - 1 - item / BH;
      const int n_it = p.causal ? (qt + 1) : n_t;
      for (int it = 0; it < n_it; ++it, ++g) {
        const uint32_t w = w_q[0];
        const float4 k4 = k_q[0];
#pragma unroll
        for (int i = 0; i + 1 < kAhead; ++i) {
          w_q[i] = w_q[i + 1];
          k_q[i] = k_q[i + 1];
        }
        if (pre.item < n_items) {
          w_q[kAhead - 1] = pre.w_ptr[4 * pre.it];
          k_q[kAhead - 1] = pre.ks_ptr[pre.it];
          walk_next(pre);
        }
        const uint32_t word = pack4(sb_mul(w & 0xFF, scale_to_sb(k4.x)), sb_mul((w >> 8) & 0xFF, scale_to_sb(k4.y)),
                                    sb_mul((w >> 16) & 0xFF, scale_to_sb(k4.z)), sb_mul(w >> 24, scale_to_sb(k4.w)));
        const uint32_t st = g % C::kStages;
        if (g >= C::kStages && !(ok = wait_warp(empty + st, ((g / C::kStages) - 1) & 1, abort_flag))) break;
        tc_fence_after();
        tmem_st4(tmem + lane_base + C::kColSf + 4 * st, word, word, word, word);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if ((tid & 31) == 0) mbar_arrive(full + st);
      }
    }
    if (!ok) raise_abort(abort_flag, p.status, kStatusTimeoutCompute);
  } else {
    // ------------------------------------------------------------------------------------------ dQ read-out
    const int quad = warp & 3;
    const int r = quad * 32 + (tid & 31);
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    bool ok = true;
    uint32_t n_done = 0;
    for (int k = 0, item; ok && (item = sched_item(k, first_item, item_step)) < n_items; ++k, ++n_done) {
      const int qt = n_t - 1 - item / BH, bh = item % BH;
      const int b = bh / p.H, h = bh % p.H;
      const uint32_t acc = n_done % C::kAccs;
      if (!(ok = wait_warp(dq_full + acc, (n_done / C::kAccs) & 1, abort_flag))) break;
      tc_fence_after();
      __nv_bfloat16* dst = p.dq + static_cast<int64_t>(b) * p.dq_sb + static_cast<int64_t>(qt * 128 + r) * p.dq_sn +
                           static_cast<int64_t>(h) * p.dq_sh;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t rr[32];
        tmem_ld32(tmem + lane_base + C::kColDq + D * acc + 32 * c, rr);
        tmem_wait_ld();
        uint32_t w[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(rr[2 * e]) * p.sm_scale,
                                                   __uint_as_float(rr[2 * e + 1]) * p.sm_scale);
          w[e] = *reinterpret_cast<uint32_t*>(&v);
        }
        uint4* d4 = reinterpret_cast<uint4*>(dst + 32 * c);
#pragma unroll
        for (int e = 0; e < 4; ++e) d4[e] = make_uint4(w[4 * e], w[4 * e + 1], w[4 * e + 2], w[4 * e + 3]);
      }
      tc_fence_before();
      __syncwarp();
      if ((tid & 31) == 0) mbar_arrive(dq_free + acc);
    }
    if (!ok) raise_abort(abort_flag, p.status, kStatusTimeoutCompute);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, C::kTmemCols);
}

template <int D>
static cudaError_t launch_p2_t(const CUtensorMap& tds, const CUtensorMap& tk, const BwdParams& p, cudaStream_t stream) {
  using C = DqP2Cfg<D>;
  static bool attr_set[64] = {};
  static int sm_count[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(bwd_dq_p2_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return e;
    e = cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  const int sms = (dev >= 0 && dev < 64) ? sm_count[dev] : 148;
  const int items = (p.N / 128) * p.B * p.H;
  bwd_dq_p2_kernel<D><<<items < sms ? items : sms, C::kThreads, C::kSmemBytes, stream>>>(tds, tk, p);
  count_launch();
  return cudaGetLastError();
}

cudaError_t launch_bwd_dq_p2(int D, const CUtensorMap& tds, const CUtensorMap& tk, const BwdParams& p, cudaStream_t stream) {
  return D == 128 ? launch_p2_t<128>(tds, tk, p, stream) : launch_p2_t<256>(tds, tk, p, stream);
}

}  // namespace dm
