// Forward of delta-matching fp8 attention on sm_100a: S = Q8 K8^T on tcgen05 (kind::f8f6f4) with the accumulator in TMEM,
// per-(row, 32-key block) power-of-two P basis, P codes and UE8M0 scale words written back to TMEM, O += P V as one
// block-scaled tcgen05 chain (kind::mxf8f6f4), O bf16 and natural-log LSE.
//
// Numerics follow the reference's Blackwell contract ("sm100-mx"): delta_matching/reference.py:159-171 (mx_pfwd),
// :454-471 (forward engine) and the op list in delta_matching/sm100/dm_fwd_sm100.py:3685-3757:
//   c_b = (qs * log2e) * ks_b;  xb = max_b(S_acc) * c_b;  k_b = max(floor(xb), -1e30);  p = ex2(fma(S_acc, c_b, 7 - k_b))
//   (ex2 = ex2.approx, or a polynomial of the same accuracy on the FMA pipe for three of sixteen element pairs)
//   code = e4m3(p);  m integer-valued running max (ceil), moved only when the candidate exceeds it by more than 32;
//   SFA_b = UE8M0(k_b - 7 - m), SFB_b = V scale byte;  l += sum_b (sum of the unquantised p of block b) * 2^(k_b - 7 - m)
//   O = bf16(O_acc / l);  LSE = (m + log2 l) * ln2.  Key tiles are visited from the highest index down.
//
// Work item = one 128-query tile of one (batch, query head); a CTA walks a list of items.  Warps 0-3: softmax / epilogue
// (thread t owns TMEM lane t = query row t).  Warp 4: TMA producer.  Warp 5: MMA issuer and TMEM owner.  Every mbarrier wait is bounded.
#include <type_traits>
#include <cuda_bf16.h>
#include "dm_common.cuh"
#include "dm_kernels.h"

namespace dm {

template <int D>
struct FwdCfg {
  static constexpr int kSub = D / 128;                 // 128-byte-wide sub-tiles per operand row
  static constexpr int kTileBytes = 128 * D;           // one 128-row operand tile
  static constexpr int kStages = 2;
  static constexpr int kTmemCols = (D == 128) ? 256 : 512;
  // At head_dim 256 one CTA owns the SM's 512 columns, and S is double-buffered (S0 0-127, S1 128-255, O 256-511): the
  // S chain of key tile i + 1 runs while the softmax warps work on tile i.  At head_dim 128 two CTAs share the SM with 256
  // columns each (S 0-127, O 128-255) and take turns instead.
  static constexpr bool kDoubleS = (D == 256);
  static constexpr int kColS = 0;                      // S accumulator, 128 fp32 columns; P codes reuse columns 0-31
  static constexpr int kColSfa = 32;                   // 4 columns, each this row's SFA word
  static constexpr int kColSfb = 36;                   // 4 columns, each the tile's V scale word
  static constexpr int kColO = kDoubleS ? 256 : 128;   // O accumulator, D fp32 columns
  // shared memory: Q | K stages | V stages | barriers
  static constexpr int kSmemQ = 0;
  static constexpr int kSmemK = kTileBytes;
  static constexpr int kSmemV = kSmemK + kStages * kTileBytes;
  static constexpr int kSmemOut = kSmemV + kStages * kTileBytes;   // 4 warps x 32 rows x 80 bytes: O write-out staging
  static constexpr int kOutRow = 80;                               // 64 bytes of a row + 16 of padding (bank spread)
  static constexpr int kSmemBar = kSmemOut + 4 * 32 * kOutRow;
  static constexpr int kSmemBytes = kSmemBar + 256 + 1024;   // + slack for the 1024-byte alignment of the tile base
};

// Persistent: the grid is (CTAs per SM) x (SMs); CTA j processes the work items sched_item(0, j), sched_item(1, j), ...
// of a list ordered by decreasing number of key tiles (item -> query tile n_qt - 1 - item / (B H), head item % (B H)).  The three roles keep
// running tile / item counters for the barrier phases, so the K / V ring, the next Q tile and the next S run ahead into
// the following item while the softmax warps still write out O of the current one.
// kOrdered: the MMA thread waits for the completion of the PV chain of tile i before it issues S of tile i + 1.  That S
// chain overwrites the TMEM columns from which the PV chain reads its scale-factor words; the PTX ISA orders a later
// MMA's accumulator writes behind an earlier MMA's operand reads, but does not say so for scale-factor reads (the
// reference met the same question and answers it with a commit and a wait, delta_matching/sm100/dm_fwd_sm100.py:636-645).
// kOrdered = false issues S(i + 1) straight behind PV(i) and relies on issue order alone.
template <int D, bool kOrdered>
__global__ void __launch_bounds__(192, (D == 128) ? 2 : 1)
fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
           const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  using C = FwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + C::kSmemQ;
  uint8_t* sK = smem + C::kSmemK;
  uint8_t* sV = smem + C::kSmemV;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kSmemBar);
  uint64_t* bar_q = bars + 0;
  uint64_t* bar_s = bars + 1;     // S accumulator ready (MMA commit); with two S buffers: buffer 0
  uint64_t* bar_s1 = bars + 11;   // S buffer 1 ready
  uint64_t* bar_p1 = bars + 16;   // two S buffers: P codes of buffer 1 written
  uint64_t* bar_o1 = bars + 17;   // two S buffers: PV chain out of buffer 1 done
  uint64_t* bar_p = bars + 2;     // P codes + scale words written (one arrival per softmax warp)
  uint64_t* bar_o = bars + 3;     // PV chain done (MMA commit)
  uint64_t* full_k = bars + 4;    // [kStages]
  uint64_t* full_v = bars + 6;    // [kStages]
  uint64_t* empty_k = bars + 8;   // [kStages] K stage free again (MMA commit behind the S chain)
  uint64_t* empty_v = bars + 14;  // [kStages] V stage free again (MMA commit behind the PV chain)
  uint64_t* bar_qfree = bars + 10; // the item's last S chain has read Q (MMA commit)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 13);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int n_qt = p.N / 128;
  const int BH = p.B * p.H;
  const int n_items = n_qt * BH;
  const int rep = p.H / p.Hk;
  const int first_item = static_cast<int>(blockIdx.x), item_step = static_cast<int>(gridDim.x);

  if (tid == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_s1, 1);
    mbar_init(bar_p1, 4);
    mbar_init(bar_o1, 1);
    mbar_init(bar_p, 4);
    mbar_init(bar_o, 1);
    mbar_init(bar_qfree, 1);
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(full_k + s, 1);
      mbar_init(full_v + s, 1);
      mbar_init(empty_k + s, 1);
      mbar_init(empty_v + s, 1);
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
  // Barrier and phase of running tile g.  With two S buffers the S / P / PV barriers exist once per buffer and tile g is
  // phase g / 2 of its buffer's barrier: a waiter is then never more than one phase away from the barrier it tests (with
  // one barrier for both buffers the softmax warps, which run a tile ahead of the PV chains, could test the phase bit of
  // chain g while chain g - 1 was still pending, and the test would pass at once).
  auto s_bar = [&](int g) { return (C::kDoubleS && (g & 1)) ? bar_s1 : bar_s; };
  auto p_bar = [&](int g) { return (C::kDoubleS && (g & 1)) ? bar_p1 : bar_p; };
  auto o_bar = [&](int g) { return (C::kDoubleS && (g & 1)) ? bar_o1 : bar_o; };
  auto tile_ph = [&](int g) -> uint32_t { return static_cast<uint32_t>(C::kDoubleS ? (g >> 1) : g) & 1u; };

  if (warp == 4) {
    // ------------------------------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      bool ok = true;
      int gt = 0, ic = 0;                                 // tiles and items issued so far by this CTA
      for (int k = 0, item; ok && (item = sched_item(k, first_item, item_step)) < n_items; ++k, ++ic) {
        const int qt = n_qt - 1 - item / BH, bh = item % BH;
        const int bhk = (bh / p.H) * p.Hk + (bh % p.H) / rep;
        const int n_it = p.causal ? (qt + 1) : n_qt;
        const int kt_first = p.causal ? qt : (n_qt - 1);
        if (ic > 0 && !(ok = wait_or_abort(bar_qfree, (ic - 1) & 1, abort_flag))) break;
        mbar_expect_tx(bar_q, C::kTileBytes);
        for (int s = 0; s < C::kSub; ++s) tma_load_2d(sQ + s * 16384, &tm_q, bar_q, s * 128, bh * p.N + qt * 128);
        for (int it = 0; it < n_it; ++it, ++gt) {
          const int st = gt % C::kStages;
          const uint32_t eph = ((gt / C::kStages) - 1) & 1;
          if (gt >= C::kStages && !(ok = wait_or_abort(empty_k + st, eph, abort_flag))) break;
          const int row = bhk * p.N + (kt_first - it) * 128;
          mbar_expect_tx(full_k + st, C::kTileBytes);
          for (int s = 0; s < C::kSub; ++s)
            tma_load_2d(sK + st * C::kTileBytes + s * 16384, &tm_k, full_k + st, s * 128, row);
          if (gt >= C::kStages && !(ok = wait_or_abort(empty_v + st, eph, abort_flag))) break;
          mbar_expect_tx(full_v + st, C::kTileBytes);
          for (int s = 0; s < C::kSub; ++s)
            tma_load_2d(sV + st * C::kTileBytes + s * 16384, &tm_v, full_v + st, s * 128, row);
        }
      }
      if (!ok) raise_abort(abort_flag, p.status, kStatusTimeoutProducer);
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t kIdescS = idesc_f8(128, 128, false, false);
      const uint32_t q_lo = desc_lo(smem_u32(sQ)), k_lo0 = desc_lo(smem_u32(sK)), v_lo0 = desc_lo(smem_u32(sV));
      bool ok = true;
      int gt = 0, ic = 0;
      for (int k = 0, item; ok && (item = sched_item(k, first_item, item_step)) < n_items; ++k, ++ic) {
        const int qt = n_qt - 1 - item / BH;
        const int n_it = p.causal ? (qt + 1) : n_qt;
        if (!(ok = wait_or_abort(bar_q, ic & 1, abort_flag))) break;
        // S = Q K^T of running tile g of the CTA into S buffer `buf`: both operands K-major, k-step of 32 bytes inside
        // the 128-byte swizzle row
        // `prev`: a PV chain that has to be complete first (none if negative).  With one S buffer that is the chain of tile
        // g - 1 (see kOrdered above).  With two, the chain of tile g - 2 read its codes and scale words out of this buffer;
        // the caller names the latest chain it has issued, which is g - 2 for a look-ahead and g - 1 for the first tile of
        // an item, which finished behind the chain of g - 2.
        auto issue_s = [&](int g, int buf, int prev) -> bool {
          const int st = g % C::kStages;
          if (!wait_or_abort(full_k + st, (g / C::kStages) & 1, abort_flag)) return false;
          if (prev >= 0 && !wait_or_abort(o_bar(prev), tile_ph(prev), abort_flag)) return false;
          tc_fence_after();
          const uint32_t k_lo = k_lo0 + st * (C::kTileBytes >> 4);
#pragma unroll
          for (int ks = 0; ks < D / 32; ++ks) {
            const uint32_t off = (ks / 4) * 1024 + (ks % 4) * 2;      // descriptor units of 16 bytes
            mma_f8_ss(tmem + C::kColS + 128 * buf, q_lo + off, k_lo + off, kIdescS, ks > 0);
          }
          tc_commit(s_bar(g));
          tc_commit(empty_k + st);                             // the K stage is free as soon as this chain has read it
          return true;
        };
        for (int it = 0; it < n_it; ++it, ++gt) {
          const int st = gt % C::kStages;
          const uint32_t ph = (gt / C::kStages) & 1;
          const int buf = C::kDoubleS ? (gt & 1) : 0;
          if (!C::kDoubleS || it == 0) {
            if (!(ok = issue_s(gt, buf, (kOrdered || C::kDoubleS) ? gt - 1 : -1))) break;
            if (it == n_it - 1) tc_commit(bar_qfree);
          }
          if (C::kDoubleS && it + 1 < n_it) {                  // the next tile of the item into the other buffer, now
            if (!(ok = issue_s(gt + 1, buf ^ 1, gt - 1))) break;
            if (it + 1 == n_it - 1) tc_commit(bar_qfree);
          }
          if (!(ok = wait_or_abort(p_bar(gt), tile_ph(gt), abort_flag))) break;
          if (!(ok = wait_or_abort(full_v + st, ph, abort_flag))) break;
          tc_fence_after();
          const uint32_t v_lo = v_lo0 + st * (C::kTileBytes >> 4);
          // O += P V: A = P codes in TMEM (8 columns per 32-key step), B = V tile MN-major (32 key rows per step).  The
          // first chain of an item overwrites O: the softmax warps signal bar_p of that tile only after they have read
          // the previous item's O.
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
            for (int s = 0; s < C::kSub; ++s) {
              mma_mxf8_ts(tmem + C::kColO + s * 128, tmem + C::kColS + 128 * buf + ks * 8, v_lo + s * 1024 + ks * 256,
                          idesc_mxf8(128, 128, false, true, ks, ks), tmem + C::kColSfa + 128 * buf,
                          tmem + C::kColSfb + 128 * buf, (it > 0) || (ks > 0));
            }
          }
          tc_commit(empty_v + st);
          tc_commit(o_bar(gt));
        }
      }
      if (!ok) raise_abort(abort_flag, p.status, kStatusTimeoutMma);
    }
  } else {
    // ------------------------------------------------------------------------------------------ softmax / epilogue
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const int nblk = p.N / 32;
    bool ok = true;
    int gt = 0;
    // scalars of an item: head, query row, first key tile; the scales of item + 1 are requested one item ahead
    auto item_qs = [&](int item) -> const float* {
      const int qt = n_qt - 1 - item / BH, bh = item % BH;
      return p.qs + static_cast<size_t>(bh) * nblk + (qt * 128 + tid) / 32;
    };
    auto item_kv = [&](int item, const float* base) -> const float* {
      const int qt = n_qt - 1 - item / BH, bh = item % BH;
      const int bhk = (bh / p.H) * p.Hk + (bh % p.H) / rep;
      return base + static_cast<size_t>(bhk) * nblk + (p.causal ? qt : (n_qt - 1)) * 4;
    };
    float qs_next = 0.f;
    float4 ks4 = make_float4(0.f, 0.f, 0.f, 0.f), vs4 = ks4;
    if (first_item < n_items) {
      qs_next = *item_qs(first_item);
      ks4 = *reinterpret_cast<const float4*>(item_kv(first_item, p.ks));
      vs4 = *reinterpret_cast<const float4*>(item_kv(first_item, p.vs));
    }
    for (int k = 0, item; (item = sched_item(k, first_item, item_step)) < n_items; ++k) {
      const int qt = n_qt - 1 - item / BH, bh = item % BH;
      const int b = bh / p.H, h = bh % p.H;
      const int n_it = p.causal ? (qt + 1) : n_qt;
      const int row = qt * 128 + tid;                                       // query index inside the head
      const float qsl = qs_next * kLog2e;
      const int item_n = sched_item(k + 1, first_item, item_step);
      const bool has_next = item_n < n_items;
      if (has_next) qs_next = *item_qs(item_n);
      const float* ks_ptr = item_kv(item, p.ks);                            // scales of the tile being processed
      const float* vs_ptr = item_kv(item, p.vs);
      float m = 0.f, l = 0.f;
      // One key tile.  kDiag: the tile on the diagonal of a causal problem (always the first one visited), where keys
      // above the query index are masked; a compile-time variant so that the other tiles carry no select per element.
      auto tile = [&](int it, auto diag_tag) -> bool {
        constexpr bool kDiag = decltype(diag_tag)::value;
        const float cb[4] = {qsl * ks4.x, qsl * ks4.y, qsl * ks4.z, qsl * ks4.w};
        const uint32_t sfb = pack4(scale_to_sb(vs4.x), scale_to_sb(vs4.y), scale_to_sb(vs4.z), scale_to_sb(vs4.w));
        // scales of the next key tile (of this item or of the next one): in flight while this tile is processed
        if (it + 1 < n_it) {
          ks_ptr -= 4;
          vs_ptr -= 4;
          ks4 = *reinterpret_cast<const float4*>(ks_ptr);
          vs4 = *reinterpret_cast<const float4*>(vs_ptr);
        } else if (has_next) {
          ks4 = *reinterpret_cast<const float4*>(item_kv(item_n, p.ks));
          vs4 = *reinterpret_cast<const float4*>(item_kv(item_n, p.vs));
        }
        const int sbuf = C::kDoubleS ? (gt & 1) : 0;                         // S buffer of this tile
        const uint32_t s_col = C::kColS + 128 * sbuf;
        if (!wait_warp(s_bar(gt), tile_ph(gt), abort_flag)) return false;
        tc_fence_after();
        float bsum[4], kb[4], bmax[4];
        uint32_t r[2][32];
        tmem_ld32(tmem + lane_base + s_col, r[0]);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t (&rc)[32] = r[c & 1];
          tmem_wait_ld();
          if (c < 3) tmem_ld32(tmem + lane_base + s_col + 32 * (c + 1), r[(c + 1) & 1]);   // next chunk in flight
          if (kDiag) {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (32 * c + e > tid) rc[e] = 0xff800000u;       // -inf: key index above the query index
          }
          float2 s2[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) s2[e] = make_float2(__uint_as_float(rc[2 * e]), __uint_as_float(rc[2 * e + 1]));
          bmax[c] = max32(s2) * cb[c];
          kb[c] = fmaxf(floorf(bmax[c]), -1e30f);
          const float2 c2 = splat2(cb[c]), bias2 = splat2(7.0f - kb[c]);
          float2 sum0 = make_float2(0.f, 0.f), sum1 = make_float2(0.f, 0.f);
          uint32_t codes[8];
#pragma unroll
          for (int e = 0; e < 16; e += 2) {
            const float2 p0 = ex2_2(fma2(s2[e], c2, bias2));
            // three of the sixteen pairs take the polynomial: the MUFU pipe is the floor of this loop, the FMA pipe has room
            const float2 p1 = (e == 2 || e == 8 || e == 14) ? ex2_poly2(fma2(s2[e + 1], c2, bias2)) : ex2_2(fma2(s2[e + 1], c2, bias2));
            sum0 = add2(sum0, p0);
            sum1 = add2(sum1, p1);
            codes[e / 2] = cvt_e4m3x4(p0.x, p0.y, p1.x, p1.y);
          }
          sum0 = add2(sum0, sum1);
          bsum[c] = sum0.x + sum0.y;
          tmem_st8(tmem + lane_base + s_col + 8 * c, codes);
        }
        const float mcand = ceilf(fmaxf(fmaxf(bmax[0], bmax[1]), fmaxf(bmax[2], bmax[3])));
        float acc_scale = 1.0f;
        if (it == 0) {
          m = mcand;
        } else if (mcand > m + 32.0f) {
          acc_scale = sb_to_scale(static_cast<uint32_t>(max(0, min(__float2int_rn(m - mcand) + 127, 254))));
          m = mcand;
        }
        if (it > 0 && __any_sync(0xffffffffu, acc_scale != 1.0f)) {
          // rare: the running max moved by more than 32 binades; rescale this warp's O rows in place.  With two S
          // buffers this tile's S was issued ahead of the previous PV chain, so that chain is waited for by name.
          if (C::kDoubleS) {
            if (!wait_warp(o_bar(gt - 1), tile_ph(gt - 1), abort_flag)) return false;
            tc_fence_after();
          }
          for (int c = 0; c < D / 32; ++c) {
            uint32_t ro[32];
            tmem_ld32(tmem + lane_base + C::kColO + 32 * c, ro);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) ro[e] = __float_as_uint(__uint_as_float(ro[e]) * acc_scale);
            tmem_st32(tmem + lane_base + C::kColO + 32 * c, ro);
          }
        }
        l *= acc_scale;
        uint32_t sb[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int e = __float2int_rn(kb[c] - 7.0f - m);      // saturates for fully masked blocks
          sb[c] = static_cast<uint32_t>(max(0, min(max(e, -1000) + 127, 254)));
          l = fmaf(bsum[c], __uint_as_float(sb[c] << 23), l);
        }
        const uint32_t sfa = pack4(sb[0], sb[1], sb[2], sb[3]);
        tmem_st4(tmem + lane_base + C::kColSfa + 128 * sbuf, sfa, sfa, sfa, sfa);
        tmem_st4(tmem + lane_base + C::kColSfb + 128 * sbuf, sfb, sfb, sfb, sfb);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if ((tid & 31) == 0) mbar_arrive(p_bar(gt));
        ++gt;
        return true;
      };
      ok = p.causal ? tile(0, std::true_type{}) : tile(0, std::false_type{});
      for (int it = 1; ok && it < n_it; ++it) ok = tile(it, std::false_type{});
      if (ok) ok = wait_warp(o_bar(gt - 1), tile_ph(gt - 1), abort_flag);
      if (!ok) break;
      tc_fence_after();
      const float inv_l = 1.0f / l;
      // A thread holds one row of O; written row by row, a warp's store would touch 32 rows with 16 bytes each.  Each
      // 32-column chunk (64 bytes per row) goes through a per-warp staging area instead, from which four lanes write
      // the 64 contiguous bytes of a row: a store instruction covers 8 rows completely.
      const int lane = tid & 31;
      const uint32_t stage_a = smem_u32(smem + C::kSmemOut) + warp * (32 * C::kOutRow);
      const int out_row0 = qt * 128 + warp * 32;                    // first row of this warp
      __nv_bfloat16* obase = p.o + static_cast<int64_t>(b) * p.o_sb + static_cast<int64_t>(h) * p.o_sh + 8 * (lane & 3);
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem + lane_base + C::kColO + 32 * c, r);
        tmem_wait_ld();
        uint32_t w[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * e]) * inv_l, __uint_as_float(r[2 * e + 1]) * inv_l);
          w[e] = *reinterpret_cast<uint32_t*>(&v);
        }
        __syncwarp();                                               // the previous chunk has been read out of the stage
#pragma unroll
        for (int e = 0; e < 4; ++e) sts_u4(stage_a + lane * C::kOutRow + 16 * e, w[4 * e], w[4 * e + 1], w[4 * e + 2], w[4 * e + 3]);
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int rr = 8 * i + (lane >> 2);                       // row of the warp this lane writes a quarter of
          const float4 v = lds_f4(stage_a + rr * C::kOutRow + 16 * (lane & 3));
          *reinterpret_cast<float4*>(obase + static_cast<int64_t>(out_row0 + rr) * p.o_sn + 32 * c) = v;
        }
      }
      p.lse[static_cast<size_t>(bh) * p.N + row] = (m + log2f(l)) * kLn2;
    }
    if (!ok) raise_abort(abort_flag, p.status, kStatusTimeoutCompute);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem, C::kTmemCols);
}

template <int D, bool kOrdered>
static cudaError_t launch_fwd_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FwdParams& p,
                                cudaStream_t stream) {
  using C = FwdCfg<D>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(fwd_kernel<D, kOrdered>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  static int sm_count[64] = {};
  if (dev >= 0 && dev < 64 && sm_count[dev] == 0) {
    cudaError_t e = cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
  }
  const int sms = (dev >= 0 && dev < 64) ? sm_count[dev] : 148;
  const int items = (p.N / 128) * p.B * p.H;
  const int ctas = sms * ((D == 128) ? 2 : 1);              // co-resident CTAs: 256 of the 512 TMEM columns each at D = 128
  fwd_kernel<D, kOrdered><<<items < ctas ? items : ctas, 192, C::kSmemBytes, stream>>>(tq, tk, tv, p);
  count_launch();
  return cudaGetLastError();
}


cudaError_t launch_fwd(int D, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FwdParams& p,
                       cudaStream_t stream) {
  // One kernel for both head dims: S (128 columns) plus O (head_dim columns) per CTA, two CTAs per SM at head_dim 128.
  if (p.unordered) {
    if (D != 128) return launch_fwd_t<256, false>(tq, tk, tv, p, stream);
    return launch_fwd_t<128, false>(tq, tk, tv, p, stream);
  }
  if (D != 128) return launch_fwd_t<256, true>(tq, tk, tv, p, stream);
  return launch_fwd_t<128, true>(tq, tk, tv, p, stream);
}

}  // namespace dm
