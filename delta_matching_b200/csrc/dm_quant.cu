// Quantisation producers: bf16 Q / K / V / dO -> e4m3 codes with one power-of-two scale per 32 tokens over all of
// head_dim, K centred by its per-(batch, kv head) mean over tokens, optional stale delta rowsum(dO * O).
//
// Rule (delta_matching/sm100/quant.py:1-12, 160-176; emulation delta_matching/reference.py:96-107):
//   y = (x - mean) * prescale (fp32);  amax over the 32 x D block = m * 2^E;
//   scale = 2^(E-8) if m <= 1.75 else 2^(E-7)  (the smallest power of two with amax <= 448 * scale; 1 if amax == 0);
//   code = e4m3_rne(y * 2^-e)  (exact scaling, never saturates).
// K mean (delta_matching/reference.py:328-338): fp32 sums of 64-token chunks folded serially in chunk order, / N.
// HBM-bound kernels: 16-byte loads, 16-byte code stores, one 32-token block per 128-thread CTA.
#include <cuda_bf16.h>
#include "dm_common.cuh"
#include "dm_kernels.h"

namespace dm {

__device__ __forceinline__ void bf16x8_to_float(const uint4& v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

// ------------------------------------------------------------------------------------------------ K mean
// Stage 1: one CTA per (64-token chunk, batch * kv head): column sums of the chunk, rows folded in a fixed order.
template <int D>
struct KMeanTile {
  static constexpr int kTpr = D / 8;            // threads per token row (16 bytes each)
  static constexpr int kRpp = 128 / kTpr;       // rows per pass
};

template <int D>
__device__ __forceinline__ void kmean_block(const KMeanParams& p, int chunk, int bh, float (*red)[D]) {
  constexpr int kTpr = KMeanTile<D>::kTpr, kRpp = KMeanTile<D>::kRpp;
  const int b = bh / p.Hk, h = bh % p.Hk;
  const int tid = threadIdx.x;
  const int c8 = tid % kTpr, r0 = tid / kTpr;
  const __nv_bfloat16* base = p.k + b * p.sb + h * p.sh + static_cast<int64_t>(chunk) * 64 * p.sn + c8 * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
  for (int r = r0; r < 64; r += kRpp) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(base + r * p.sn));
    float f[8];
    bf16x8_to_float(v, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += f[i];
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[r0][c8 * 8 + i] = acc[i];
  __syncthreads();
  for (int c = tid; c < D; c += 128) {
    float s = red[0][c];
#pragma unroll
    for (int r = 1; r < kRpp; ++r) s += red[r][c];
    p.partial[(static_cast<size_t>(bh) * (p.N / 64) + chunk) * D + c] = s;
  }
}

template <int D>
__global__ void __launch_bounds__(128) kmean_partial_kernel(const KMeanParams p) {
  __shared__ float red[KMeanTile<D>::kRpp][D];
  kmean_block<D>(p, blockIdx.x, blockIdx.y, red);
}

// Stage 2: one CTA per (batch, kv head): serial fold of the chunk sums in chunk order, divided by N.
__global__ void kmean_fold_kernel(const KMeanParams p) {
  const int bh = blockIdx.x;
  const int nchunk = p.N / 64;
  for (int c = threadIdx.x; c < p.D; c += blockDim.x) {
    const float* src = p.partial + static_cast<size_t>(bh) * nchunk * p.D + c;
    float s = 0.f;
    int j = 0;
    for (; j + 8 <= nchunk; j += 8) {               // eight loads in flight, added in chunk order
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = src[static_cast<size_t>(j + u) * p.D];
#pragma unroll
      for (int u = 0; u < 8; ++u) s += v[u];
    }
    for (; j < nchunk; ++j) s += src[static_cast<size_t>(j) * p.D];
    p.mean[static_cast<size_t>(bh) * p.D + c] = s / static_cast<float>(p.N);
  }
}

cudaError_t launch_kmean(const KMeanParams& p, cudaStream_t stream) {
  dim3 grid(p.N / 64, p.B * p.Hk);
  if (p.D == 128) kmean_partial_kernel<128><<<grid, 128, 0, stream>>>(p);
  else kmean_partial_kernel<256><<<grid, 128, 0, stream>>>(p);
  kmean_fold_kernel<<<p.B * p.Hk, 128, 0, stream>>>(p);
  count_launch(2);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ quantiser
cudaError_t launch_quant(const QuantParams& p, cudaStream_t stream);
// kMean / kStale: the K tensor alone subtracts a mean and the dO tensor of the stale mode alone reads O; compiled out
// elsewhere, the kernel needs fewer registers and more of its small CTAs fit an SM (more loads in flight).
template <int D, bool kMean, bool kStale>
__device__ __forceinline__ void quant_block(const QuantParams& p, int blk, int bh, float* wmax) {
  constexpr int kTpr = D / 16;           // threads per token row (16 elements each)
  constexpr int kRpp = 128 / kTpr;       // rows per pass
  constexpr int kPass = 32 / kRpp;
  const int b = bh / p.H, h = bh % p.H;
  const int tid = threadIdx.x;
  const int c16 = tid % kTpr, r0 = tid / kTpr;
  const __nv_bfloat16* xb = p.x + b * p.sb + h * p.sh + static_cast<int64_t>(blk) * 32 * p.sn + c16 * 16;

  float mean[kMean ? 16 : 1];
  if (kMean) {
    const float4* mp = reinterpret_cast<const float4*>(p.mean + static_cast<size_t>(bh) * D + c16 * 16);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 v = __ldg(mp + i);
      mean[4 * i] = v.x; mean[4 * i + 1] = v.y; mean[4 * i + 2] = v.z; mean[4 * i + 3] = v.w;
    }
  }

  float y[kPass][16];
  float amax = 0.f;
#pragma unroll
  for (int ps = 0; ps < kPass; ++ps) {
    const int r = r0 + ps * kRpp;
    const uint4* src = reinterpret_cast<const uint4*>(xb + r * p.sn);
    const uint4 v0 = __ldg(src), v1 = __ldg(src + 1);
    bf16x8_to_float(v0, &y[ps][0]);
    bf16x8_to_float(v1, &y[ps][8]);
    if (kStale) {
      // stale delta = sum_d dO * O on the raw bf16 values (delta_matching/reference.py:500-501)
      const __nv_bfloat16* ob = p.o + b * p.o_sb + h * p.o_sh + (static_cast<int64_t>(blk) * 32 + r) * p.o_sn + c16 * 16;
      const uint4 o0 = __ldg(reinterpret_cast<const uint4*>(ob)), o1 = __ldg(reinterpret_cast<const uint4*>(ob) + 1);
      float of[16];
      bf16x8_to_float(o0, &of[0]);
      bf16x8_to_float(o1, &of[8]);
      float d = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) d = fmaf(y[ps][i], of[i], d);
#pragma unroll
      for (int off = kTpr / 2; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
      if (c16 == 0) p.delta[static_cast<size_t>(bh) * p.N + blk * 32 + r] = d;
    }
    // (x - 0) * prescale and x * prescale are the same fp32 value, so leaving the subtraction out changes no bit
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      y[ps][i] = kMean ? (y[ps][i] - mean[i]) * p.prescale : y[ps][i] * p.prescale;
      amax = fmaxf(amax, fabsf(y[ps][i]));
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if ((tid & 31) == 0) wmax[tid >> 5] = amax;
  __syncthreads();
  amax = fmaxf(fmaxf(wmax[0], wmax[1]), fmaxf(wmax[2], wmax[3]));
  const uint32_t sb = pow2_sb(amax, 127u);
  const float inv = sb_to_inv(sb);
  if (tid == 0) p.scales[static_cast<size_t>(bh) * (p.N / 32) + blk] = sb_to_scale(sb);

  uint8_t* cb = p.codes + (static_cast<size_t>(bh) * p.N + static_cast<size_t>(blk) * 32) * D + c16 * 16;
#pragma unroll
  for (int ps = 0; ps < kPass; ++ps) {
    const int r = r0 + ps * kRpp;
    uint4 w;
    w.x = cvt_e4m3x4(y[ps][0] * inv, y[ps][1] * inv, y[ps][2] * inv, y[ps][3] * inv);
    w.y = cvt_e4m3x4(y[ps][4] * inv, y[ps][5] * inv, y[ps][6] * inv, y[ps][7] * inv);
    w.z = cvt_e4m3x4(y[ps][8] * inv, y[ps][9] * inv, y[ps][10] * inv, y[ps][11] * inv);
    w.w = cvt_e4m3x4(y[ps][12] * inv, y[ps][13] * inv, y[ps][14] * inv, y[ps][15] * inv);
    *reinterpret_cast<uint4*>(cb + static_cast<size_t>(r) * D) = w;
  }
}

template <int D, bool kMean, bool kStale>
__global__ void __launch_bounds__(128) quant_kernel(const QuantParams p) {
  __shared__ float wmax[4];
  quant_block<D, kMean, kStale>(p, blockIdx.x, blockIdx.y, wmax);
}

// Q, V and the chunk sums of the K mean in one launch: the three need nothing from each other, and as separate launches
// of a few microseconds each they spend a good part of their time filling and draining the GPU.  The grid is the
// concatenation [K-mean chunks | Q blocks | V blocks] (the chunk sums first: the fold and the K quantiser wait for them).
template <int D>
__global__ void __launch_bounds__(128) quant_qv_kmean_kernel(const QuantParams pq, const QuantParams pv, const KMeanParams pk) {
  __shared__ float wmax[4];
  __shared__ float red[KMeanTile<D>::kRpp][D];
  const int n_km = (pk.N / 64) * pk.B * pk.Hk;
  const int n_q = (pq.N / 32) * pq.B * pq.H;
  int i = static_cast<int>(blockIdx.x);
  if (i < n_km) {
    kmean_block<D>(pk, i % (pk.N / 64), i / (pk.N / 64), red);
  } else if ((i -= n_km) < n_q) {
    quant_block<D, false, false>(pq, i % (pq.N / 32), i / (pq.N / 32), wmax);
  } else {
    i -= n_q;
    quant_block<D, false, false>(pv, i % (pv.N / 32), i / (pv.N / 32), wmax);
  }
}

cudaError_t launch_quant_qkv(const QuantParams& pq, const QuantParams& pk, const QuantParams& pv, const KMeanParams& pm,
                             cudaStream_t stream) {
  const long long blocks = static_cast<long long>(pm.N / 64) * pm.B * pm.Hk + static_cast<long long>(pq.N / 32) * pq.B * pq.H +
                           static_cast<long long>(pv.N / 32) * pv.B * pv.H;
  if (blocks > 0x7fffffffll) return cudaErrorInvalidValue;
  if (pq.D == 128) quant_qv_kmean_kernel<128><<<static_cast<unsigned>(blocks), 128, 0, stream>>>(pq, pv, pm);
  else quant_qv_kmean_kernel<256><<<static_cast<unsigned>(blocks), 128, 0, stream>>>(pq, pv, pm);
  kmean_fold_kernel<<<pm.B * pm.Hk, 128, 0, stream>>>(pm);
  count_launch(2);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  return launch_quant(pk, stream);                      // K, centred by the mean that the fold has just written
}

cudaError_t launch_quant(const QuantParams& p, cudaStream_t stream) {
  dim3 grid(p.N / 32, p.B * p.H);
  const bool mean = p.mean != nullptr, stale = p.o != nullptr;
  if (p.D == 128) {
    if (stale) quant_kernel<128, false, true><<<grid, 128, 0, stream>>>(p);
    else if (mean) quant_kernel<128, true, false><<<grid, 128, 0, stream>>>(p);
    else quant_kernel<128, false, false><<<grid, 128, 0, stream>>>(p);
  } else {
    if (stale) quant_kernel<256, false, true><<<grid, 128, 0, stream>>>(p);
    else if (mean) quant_kernel<256, true, false><<<grid, 128, 0, stream>>>(p);
    else quant_kernel<256, false, false><<<grid, 128, 0, stream>>>(p);
  }
  count_launch();
  return cudaGetLastError();
}

}  // namespace dm
