/* C ABI of the delta-matching fp8 attention kernels for NVIDIA B200 (sm_100a).
 *
 * Plain pointers and sizes only; no torch types.  Every entry point
 *   - returns 0 on success and a negative DM_ERR_* code otherwise (dm_last_error gives the message of the calling
 *     thread's last failure), and validates its arguments before any launch,
 *   - launches on the given stream of the CURRENT device and never synchronises, allocates or exits,
 *   - takes device pointers that the caller owns.
 *
 * Layouts.  "codes": e4m3 bytes, dense (B, H, N, D).  "scales": fp32 powers of two, dense (B, H, N / 32): one scale per
 * 32 tokens over all of head_dim (dequantised value = code * scale).  q codes carry the softmax scale D^-0.5; k codes
 * are centred by the per-(batch, kv head) mean over tokens.  lse / delta: fp32 (B, H, N); lse is the natural log in
 * the centred-K convention.  bf16 inputs and outputs are addressed by element strides with head_dim contiguous.
 * Constraints: D in {128, 256}; N a positive multiple of 128; H a positive multiple of Hk; B * H <= 65535; code, scale
 * and bf16 base pointers 16-byte aligned and bf16 strides multiples of 8 elements.
 *
 * `status` (may be NULL) is a device int the kernels set to a non-zero DM_STATUS_* value when one of their bounded
 * waits runs out; the outputs of that launch are then invalid.  The caller zeroes it and reads it after a sync.
 */
#ifndef DM_B200_H_
#define DM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DM_ERR_ARG (-1)      /* bad argument (message names it) */
#define DM_ERR_CUDA (-2)     /* a CUDA runtime / driver call failed */
#define DM_ERR_DEVICE (-3)   /* current device is not sm_100 */

#define DM_STATUS_OK 0
#define DM_STATUS_TIMEOUT_PRODUCER 1
#define DM_STATUS_TIMEOUT_MMA 2
#define DM_STATUS_TIMEOUT_COMPUTE 3
#define DM_STATUS_TIMEOUT_PROBE 4

/* Library identity.  Replaces the build-sanity ops build_gt() / build_hd128() / build_bf16dp() of
 * csrc/delta_matching_api.cpp:683-715: dm_version() is MAJOR * 10000 + MINOR * 100 + PATCH; dm_numerics() names the
 * quantisation contract the kernels implement (the reference emulation preset, delta_matching/reference.py:612-629). */
int dm_version(void);
const char* dm_numerics(void);
int dm_last_error(char* buf, int n);

/* Scratch bytes dm_quant_qkv needs (the K-mean chunk sums).  The reference allocates its producer scratch inside
 * quant_qkv2 (delta_matching/sm100/quant.py:300-312); here the caller allocates. */
size_t dm_quant_qkv_workspace_bytes(int B, int N, int Hk, int D);

/* K mean over tokens per (batch, kv head): fp32 sums of 64-token chunks folded serially in chunk order, / N.
 * Replaces kmean_strided / _kmean_kernel (delta_matching/producers.py:127-135, delta_matching/quant.py:17-29).
 * k strides are element strides for (batch, head, token).  mean: (B, Hk, D) fp32. */
int dm_kmean(const void* k, int64_t k_sb, int64_t k_sh, int64_t k_sn, int B, int N, int Hk, int D, float* mean,
             void* workspace, void* stream);

/* One tensor through the quantiser: y = (x - mean[b, h]) * prescale -> codes, scales; when `o` is given also
 * delta[b, h, n] = sum_d x * o (the stale delta).  mean, o, delta may be NULL.
 * Replaces _quant_strided_kernel / _doq_m17_kernel (delta_matching/producers.py:73-103, 367-429) and quant_rows
 * (delta_matching/sm100/quant.py:1-12). */
int dm_quant_rows(const void* x, int64_t x_sb, int64_t x_sh, int64_t x_sn, const float* mean, float prescale,
                  const void* o, int64_t o_sb, int64_t o_sh, int64_t o_sn, int B, int N, int H, int D,
                  void* codes, float* scales, float* delta, void* stream);

/* Q, K, V producers in one call: q * D^-0.5, k - mean(k), v.  Replaces quant_qkv_m17 (delta_matching/producers.py:
 * 244-306) and quant_qkv2 (delta_matching/sm100/quant.py:278-323).  kmean: (B, Hk, D) fp32 output. */
int dm_quant_qkv(const void* q, int64_t q_sb, int64_t q_sh, int64_t q_sn,
                 const void* k, int64_t k_sb, int64_t k_sh, int64_t k_sn,
                 const void* v, int64_t v_sb, int64_t v_sh, int64_t v_sn,
                 int B, int N, int H, int Hk, int D,
                 void* q8, void* k8, void* v8, float* qs, float* ks, float* vs, float* kmean,
                 void* workspace, void* stream);

/* dO producer; with `o` non-NULL also the stale delta rowsum(dO * O).  Replaces doq_m17 (delta_matching/producers.py:
 * 432-461) and quant_do_delta (delta_matching/sm100/quant.py:326-341). */
int dm_quant_do(const void* d_o, int64_t do_sb, int64_t do_sh, int64_t do_sn,
                const void* o, int64_t o_sb, int64_t o_sh, int64_t o_sn,
                int B, int N, int H, int D, void* do8, float* dos, float* delta, void* stream);

/* Forward: O (bf16, element strides for (batch, token, head)) and LSE.  Replaces the fwd_fp8 op
 * (csrc/delta_matching_api.cpp:105-205). */
int dm_fwd(const void* q8, const void* k8, const void* v8, const float* qs, const float* ks, const float* vs,
           int B, int N, int H, int Hk, int D, int causal,
           void* o, int64_t o_sb, int64_t o_sn, int64_t o_sh, float* lse, int* status, void* stream);

/* dm_fwd with the S chain of the next key tile issued straight behind the PV chain of the current one, without the
 * commit-and-wait that dm_fwd puts between them (the next S overwrites the TMEM columns the PV chain reads its scale
 * words from; the reference documents the hazard and orders the two, delta_matching/sm100/dm_fwd_sm100.py:636-645).
 * Test hook: the unit tests demand bitwise equal O and LSE from both forms and the benchmark reports what the ordering
 * costs.  Not a production entry point. */
int dm_dbg_fwd_unordered(const void* q8, const void* k8, const void* v8, const float* qs, const float* ks, const float* vs,
                         int B, int N, int H, int Hk, int D, int causal,
                         void* o, int64_t o_sb, int64_t o_sn, int64_t o_sh, float* lse, int* status, void* stream);

/* Matched delta (pass 0): delta_i = sum_j P_ij dP_ij / sum_j P_ij from the backward's own P / dP recompute.
 * Replaces the delta_fp8 op (csrc/delta_matching_api.cpp:470-609). */
int dm_delta(const void* q8, const void* k8, const void* v8, const void* do8,
             const float* qs, const float* ks, const float* vs, const float* dos, const float* lse,
             int B, int N, int H, int Hk, int D, int causal, float* delta, int* status, void* stream);

/* dm_delta without the division: delta_i = sum_j P_ij dP_ij.  The matched delta of the reference emulation's numerics
 * arm "sm100-mx-nonorm" (delta_matching/reference.py:526-535 with delta_norm = False, preset at :620). */
int dm_delta_sum(const void* q8, const void* k8, const void* v8, const void* do8,
                 const float* qs, const float* ks, const float* vs, const float* dos, const float* lse,
                 int B, int N, int H, int Hk, int D, int causal, float* delta, int* status, void* stream);

/* Backward: dQ (H heads), dK and dV (Hk heads: the GQA group is reduced inside the kernel), bf16 with element strides
 * for (batch, token, head).  rowsum_ds / sum_abs_pdp (fp32 (B, H, N), may be NULL) receive the identity probe
 * sum_j dS_ij and sum_j |P_ij dP_ij| taken before dS is quantised.  Replaces the bwd_fp8_t op
 * (csrc/delta_matching_api.cpp:223-391, 428-437) and the GQA fold of delta_matching/attn.py:114-117. */
int dm_bwd(const void* q8, const void* k8, const void* v8, const void* do8,
           const float* qs, const float* ks, const float* vs, const float* dos,
           const float* lse, const float* delta,
           int B, int N, int H, int Hk, int D, int causal,
           void* dq, int64_t dq_sb, int64_t dq_sn, int64_t dq_sh,
           void* dk, int64_t dk_sb, int64_t dk_sn, int64_t dk_sh,
           void* dv, int64_t dv_sb, int64_t dv_sn, int64_t dv_sh,
           float* rowsum_ds, float* sum_abs_pdp, int* status, void* stream);

/* dm_bwd with a choice of kernels: parts = 1 runs only the dK / dV kernel, 2 only the dQ kernel, 3 both (what dm_bwd
 * does).  The reference launches its pass 1 and pass 2 from one op (csrc/flash_bwd_fp8v10_launch.h:158-163); the split
 * exists so that each kernel can be timed and profiled alone.
 * Adding DM_DS_BLOCK32 (4) to parts quantises dS with one power-of-two scale per (32 queries x 32 keys) instead of
 * the contract's (128 queries x 32 keys): the reference emulation's numerics arm "sm100-mx-ds32"
 * (delta_matching/reference.py:110-116, preset at :625; "sm100-mx-d256-ds32" at head_dim 256, :630).  Both kernels
 * of a backward must get the same value. */
#define DM_PARTS_DKDV 1
#define DM_PARTS_DQ 2
#define DM_DS_BLOCK32 4
int dm_bwd_parts(const void* q8, const void* k8, const void* v8, const void* do8,
                 const float* qs, const float* ks, const float* vs, const float* dos,
                 const float* lse, const float* delta,
                 int B, int N, int H, int Hk, int D, int causal,
                 void* dq, int64_t dq_sb, int64_t dq_sn, int64_t dq_sh,
                 void* dk, int64_t dk_sb, int64_t dk_sn, int64_t dk_sh,
                 void* dv, int64_t dv_sb, int64_t dv_sn, int64_t dv_sh,
                 float* rowsum_ds, float* sum_abs_pdp, int parts, int* status, void* stream);

/* The backward in the reference's two-pass form: the dK / dV kernel (pass 1) also leaves the quantised dS tiles in
 * `workspace`, and dQ = dS K is a streaming kernel over them (pass 2) instead of a kernel that recomputes S, dP and the
 * exponentials (csrc/flash_bwd_fp8v10_launch.h:158-163, csrc/fq8_dq_pass2_hd128.h:407-442; the reference allocates the
 * dS buffer inside the op and bounds it with its head-group split, delta_matching/attn.py:88-112,
 * delta_matching/split.py:37-97; its Blackwell head_dim-256 route has the same two kernels,
 * delta_matching/sm100/attention_bwd_hd256_sm100.py:1-10).
 * Outputs are bit-identical to dm_bwd.  workspace: device buffer of at least dm_bwd_workspace_bytes(B, N, H, D) bytes,
 * 16-byte aligned; contents on entry are ignored.  parts as in dm_bwd_parts; parts = 2 alone reads what an earlier
 * parts = 1 call with the same arguments wrote.  Limit: B * H * (N / 128)^2 < 2^24 tiles per call (split the heads
 * beyond that).  There is no identity probe on this path (use dm_bwd). */
int64_t dm_bwd_workspace_bytes(int B, int N, int H, int D);     /* 0 for a shape the kernels do not take */
int dm_bwd_ws(const void* q8, const void* k8, const void* v8, const void* do8,
              const float* qs, const float* ks, const float* vs, const float* dos,
              const float* lse, const float* delta,
              int B, int N, int H, int Hk, int D, int causal,
              void* dq, int64_t dq_sb, int64_t dq_sn, int64_t dq_sh,
              void* dk, int64_t dk_sb, int64_t dk_sn, int64_t dk_sh,
              void* dv, int64_t dv_sb, int64_t dv_sn, int64_t dv_sh,
              void* workspace, int64_t workspace_bytes, int parts, int* status, void* stream);

/* One 128 x 128 x (32 * nk) e4m3 tile product through the operand paths the kernels use (unit-test hook; the
 * reference has per-kernel debug ops instead, csrc/delta_matching_api.cpp:611-661).  a, b: 128 x 128 e4m3 row-major
 * device buffers; sfa / sfb: 128 x 4 uint32 scale words (block-scaled runs only); out: 128 x 128 fp32. */
int dm_dbg_mma_tile(const void* a, const void* b, const uint32_t* sfa, const uint32_t* sfb, int a_tmem, int a_mn,
                    int b_mn, int scaled, int nk, float* out, int* status, void* stream);

/* The same one-tile kernel with the arrival its threads wait for left out, and with `limit_ns` as the limit of that
 * wait: shows what every bounded wait of the library does when it runs out (the reference's kernels spin without a
 * bound; this has no counterpart there).  The kernel returns by itself after about limit_ns, *status becomes
 * DM_STATUS_TIMEOUT_PROBE (4), out is left unwritten, the context stays usable.  a, b as in dm_dbg_mma_tile. */
int dm_dbg_wait_expiry(const void* a, const void* b, float* out, long long limit_ns, int* status, void* stream);

/* Kernel launches this library has made in this process so far (all devices, all streams). */
long long dm_launch_count(void);

/* K mean without a workspace argument, for callers that cannot allocate device memory themselves (code inside a
 * no-allocation region of its host framework, or a plugin that owns no memory pool): same inputs, same kernels and
 * bit-identical result as dm_kmean, but the chunk-sum scratch is an array built into the library (4 MiB on every GPU
 * that loads it, held until the process exits).  This entry point has no counterpart in the reference.
 *   - Limit: B * Hk * (N / 64) * D <= 1048576; larger problems are refused with a message (use dm_kmean).
 *   - The first call on each device looks up the array's device address; make that call before any stream capture.
 *   - It calls no allocation routine of any kind and does not synchronise.
 *   - All calls on a device share the one array, which keeps the previous call's contents (nothing needs clearing:
 *     every value read is written first by the same call); two calls that overlap on the GPU race on it, so issue them
 *     on one stream or order them yourself.
 * Returns 0, or a negative code with a message in err (may be NULL). */
int dm_kmean_static(const void* k, int64_t k_sb, int64_t k_sh, int64_t k_sn, int B, int N, int Hk, int D, float* mean,
                    void* stream, char* err, int err_len);

/* Asynchronous strided copy between pinned host memory and device memory on a stream: `height` rows of `width` bytes,
 * rows `spitch` / `dpitch` bytes apart; to_device != 0 copies host -> device.  A helper for callers that keep their
 * tensors in host memory and feed (batch, head-range) slices of them to the entry points above (one cudaMemcpy2DAsync;
 * the reference has no host-memory path).  Returns 0 or a negative code. */
int dm_copy_2d_async(void* dst, int64_t dpitch, const void* src, int64_t spitch, int64_t width, int64_t height,
                     int to_device, void* stream);

#ifdef __cplusplus
}
#endif
#endif  /* DM_B200_H_ */
