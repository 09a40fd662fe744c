// Internal launch interface between the C-ABI layer (dm_abi.cu) and the kernel translation units.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dm {

// Codes are e4m3 bytes in (B, H, N, D) order, dense; scales fp32 powers of two in (B, H, N / 32) order.
struct FwdParams {
  const float* qs;
  const float* ks;
  const float* vs;
  __nv_bfloat16* o;            // element strides for (batch, token, head); head_dim is contiguous
  int64_t o_sb, o_sn, o_sh;
  float* lse;                  // (B, H, N) natural log
  int B, H, Hk, N;
  int causal;
  int* status;
  int unordered;               // S of the next tile issued without waiting for the PV chain (see fwd_kernel's kOrdered)
};

struct DeltaParams {
  const float* qs;
  const float* ks;
  const float* vs;
  const float* dos;
  const float* lse;            // (B, H, N)
  float* delta;                // (B, H, N)
  int B, H, Hk, N;
  int causal;
  int* status;
  int norm;                    // 1: delta = sum P dP / sum P (the contract); 0: sum P dP (numerics arm "sm100-mx-nonorm")
};

struct BwdParams {
  const float* qs;
  const float* ks;
  const float* vs;
  const float* dos;
  const float* lse;            // (B, H, N)
  const float* delta;          // (B, H, N)
  __nv_bfloat16* dq;           // (batch, token, head) element strides, head_dim contiguous; dq has H heads
  int64_t dq_sb, dq_sn, dq_sh;
  __nv_bfloat16* dk;           // Hk heads
  int64_t dk_sb, dk_sn, dk_sh;
  __nv_bfloat16* dv;
  int64_t dv_sb, dv_sn, dv_sh;
  float* rowsum_ds;            // optional (B, H, N): sum_j dS_ij before quantisation (identity probe); may be null
  float* sum_abs_pdp;          // optional (B, H, N): sum_j |P_ij dP_ij|; may be null
  uint8_t* ds_codes;           // optional dS workspace: tile (bh, qt, kt) at ((bh n_t + qt) n_t + kt) x 16384
  uint8_t* ds_words;           // bytes, [key][query] e4m3 codes; then per tile 16 UE8M0 bytes [query block][key block]
  float sm_scale;
  int B, H, Hk, N;
  int causal;
  int* status;
  int ds32;                    // dS scale per (32 queries x 32 keys) instead of (128 x 32): numerics arm "sm100-mx-ds32"
};

struct QuantParams {
  const __nv_bfloat16* x;      // element strides for (batch, head, token); head_dim contiguous
  int64_t sb, sh, sn;
  const float* mean;           // optional (B, H, D): subtracted before the prescale
  const __nv_bfloat16* o;      // optional, same logical shape as x with its own strides: stale delta = sum_d x * o
  int64_t o_sb, o_sh, o_sn;
  float prescale;
  uint8_t* codes;              // (B, H, N, D)
  float* scales;               // (B, H, N / 32)
  float* delta;                // optional (B, H, N)
  int B, H, N, D;
};

struct KMeanParams {
  const __nv_bfloat16* k;
  int64_t sb, sh, sn;
  float* partial;              // (B * Hk, N / 64, D) scratch
  float* mean;                 // (B, Hk, D)
  int B, Hk, N, D;
};

// Kernel launches made by the library in this process (every launcher counts its own).
void count_launch(int n = 1);
long long launch_count();

cudaError_t launch_fwd(int D, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FwdParams& p,
                       cudaStream_t stream);
cudaError_t launch_delta(int D, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                         const CUtensorMap& tdo, const DeltaParams& p, cudaStream_t stream);
cudaError_t launch_bwd_dkdv(int D, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                            const CUtensorMap& tdo, const CUtensorMap* tds_or_null, const BwdParams& p,
                            cudaStream_t stream);
cudaError_t launch_bwd_dq(int D, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                          const CUtensorMap& tdo, const BwdParams& p, cudaStream_t stream);
cudaError_t launch_bwd_dq_p2(int D, const CUtensorMap& tds, const CUtensorMap& tk, const BwdParams& p, cudaStream_t stream);
cudaError_t launch_quant(const QuantParams& p, cudaStream_t stream);
// Q, K, V in three launches: [K-mean chunk sums | Q | V], the fold of the chunk sums, K (pk.mean = pm.mean).
cudaError_t launch_quant_qkv(const QuantParams& pq, const QuantParams& pk, const QuantParams& pv, const KMeanParams& pm,
                             cudaStream_t stream);
cudaError_t launch_kmean(const KMeanParams& p, cudaStream_t stream);

}  // namespace dm
