// C-ABI layer: argument validation, TMA descriptor construction, kernel launches.  No torch headers, no allocation,
// no synchronisation.  Validation mirrors the op-level checks of csrc/delta_matching_api.cpp:73-98, 126-148 (device
// memory, alignment, shape constraints, causal => equal sequence lengths by construction) and reports through
// dm_last_error instead of TORCH_CHECK.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/dm_b200.h"
#include "dm_kernels.h"
#include "dm_probe.h"

namespace dm {
static std::atomic<long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launch_count() { return g_launches.load(std::memory_order_relaxed); }
}  // namespace dm

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(DM_ERR_CUDA, "delta_matching: %s failed: %s", what, cudaGetErrorString(e));
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

// 2-D map over dense e4m3 codes viewed as [rows][D]: boxes of 128 rows x 128 bytes, 128-byte swizzle.
int make_code_map(CUtensorMap* m, const void* base, uint64_t rows, int D) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(DM_ERR_CUDA, "delta_matching: cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(D), rows};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(D)};
  const cuuint32_t box[2] = {128, 128};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(DM_ERR_CUDA, "delta_matching: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int check_device_ptr(const void* p, const char* name) {
  if (p == nullptr) return fail(DM_ERR_ARG, "delta_matching: %s is NULL (every tensor must be a CUDA buffer)", name);
  cudaPointerAttributes a;
  cudaError_t e = cudaPointerGetAttributes(&a, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(DM_ERR_ARG, "delta_matching: %s must be CUDA memory", name);
  }
  if (a.type != cudaMemoryTypeDevice && a.type != cudaMemoryTypeManaged)
    return fail(DM_ERR_ARG, "delta_matching: %s must be CUDA memory (got a host pointer)", name);
  int dev = -1;
  cudaGetDevice(&dev);
  if (a.type == cudaMemoryTypeDevice && a.device != dev)
    return fail(DM_ERR_ARG, "delta_matching: %s is on device %d but the current device is %d (every tensor must be on the "
                            "same device)", name, a.device, dev);
  if (!aligned16(p)) return fail(DM_ERR_ARG, "delta_matching: %s must be 16-byte aligned", name);
  return 0;
}

int check_shape(int B, int N, int H, int Hk, int D) {
  if (D != 128 && D != 256) return fail(DM_ERR_ARG, "delta_matching: head_dim must be 128 or 256 (got %d)", D);
  if (B <= 0 || N <= 0 || H <= 0 || Hk <= 0) return fail(DM_ERR_ARG, "delta_matching: empty tensor (B=%d N=%d H=%d Hk=%d)", B, N, H, Hk);
  if (N % 128) return fail(DM_ERR_ARG, "delta_matching: seqlen must be a multiple of 128 (got %d)", N);
  if (H % Hk) return fail(DM_ERR_ARG, "delta_matching: nheads (%d) must be a multiple of nheads_k (%d)", H, Hk);
  if (static_cast<long long>(B) * H > 65535) return fail(DM_ERR_ARG, "delta_matching: batch * nheads must be at most 65535 (got %lld)", static_cast<long long>(B) * H);
  return 0;
}

int check_strides(const char* name, int64_t a, int64_t b, int64_t c) {
  if ((a % 8) || (b % 8) || (c % 8))
    return fail(DM_ERR_ARG, "delta_matching: %s strides must be multiples of 8 elements (16-byte aligned rows)", name);
  return 0;
}

int check_sm100() {
  static int cached[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev < 64 && cached[dev] == 1) return 0;
  int major = 0;
  e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
  if (major != 10) return fail(DM_ERR_DEVICE, "delta_matching: needs a Blackwell GPU (sm_100); device %d is sm_%d*", dev, major);
  if (dev < 64) cached[dev] = 1;
  return 0;
}

#define DM_TRY(expr)            \
  do {                          \
    int _r = (expr);            \
    if (_r != 0) return _r;     \
  } while (0)

}  // namespace

extern "C" {

int dm_version(void) { return 100; }   // 0.1.0

const char* dm_numerics(void) { return "sm100-mx"; }

int dm_last_error(char* buf, int n) {
  if (buf == nullptr || n <= 0) return static_cast<int>(strlen(g_err));
  strncpy(buf, g_err, n - 1);
  buf[n - 1] = 0;
  return static_cast<int>(strlen(g_err));
}

size_t dm_quant_qkv_workspace_bytes(int B, int N, int Hk, int D) {
  if (B <= 0 || N <= 0 || Hk <= 0 || D <= 0) return 0;
  return static_cast<size_t>(B) * Hk * (N / 64) * D * sizeof(float);
}

int dm_kmean(const void* k, int64_t k_sb, int64_t k_sh, int64_t k_sn, int B, int N, int Hk, int D, float* mean,
             void* workspace, void* stream) {
  DM_TRY(check_shape(B, N, Hk, Hk, D));
  DM_TRY(check_device_ptr(k, "k"));
  DM_TRY(check_device_ptr(mean, "kmean"));
  DM_TRY(check_device_ptr(workspace, "workspace"));
  DM_TRY(check_strides("k", k_sb, k_sh, k_sn));
  dm::KMeanParams p{static_cast<const __nv_bfloat16*>(k), k_sb, k_sh, k_sn, static_cast<float*>(workspace), mean, B, Hk, N, D};
  cudaError_t e = dm::launch_kmean(p, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : cuda_fail(e, "k-mean launch");
}

// checks the arguments of one quantiser call and fills its parameter block
static int quant_params(dm::QuantParams& p, const void* x, int64_t x_sb, int64_t x_sh, int64_t x_sn, const float* mean,
                        float prescale, const void* o, int64_t o_sb, int64_t o_sh, int64_t o_sn, int B, int N, int H, int D,
                        void* codes, float* scales, float* delta) {
  DM_TRY(check_shape(B, N, H, H, D));
  DM_TRY(check_device_ptr(x, "input"));
  DM_TRY(check_device_ptr(codes, "codes"));
  DM_TRY(check_device_ptr(scales, "scales"));
  DM_TRY(check_strides("input", x_sb, x_sh, x_sn));
  if (mean != nullptr) DM_TRY(check_device_ptr(mean, "mean"));
  if (o != nullptr) {
    DM_TRY(check_device_ptr(o, "o"));
    DM_TRY(check_device_ptr(delta, "delta"));
    DM_TRY(check_strides("o", o_sb, o_sh, o_sn));
  }
  p = dm::QuantParams{};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.sb = x_sb; p.sh = x_sh; p.sn = x_sn;
  p.mean = mean;
  p.o = static_cast<const __nv_bfloat16*>(o);
  p.o_sb = o_sb; p.o_sh = o_sh; p.o_sn = o_sn;
  p.prescale = prescale;
  p.codes = static_cast<uint8_t*>(codes);
  p.scales = scales;
  p.delta = (o != nullptr) ? delta : nullptr;
  p.B = B; p.H = H; p.N = N; p.D = D;
  return 0;
}

int dm_quant_rows(const void* x, int64_t x_sb, int64_t x_sh, int64_t x_sn, const float* mean, float prescale,
                  const void* o, int64_t o_sb, int64_t o_sh, int64_t o_sn, int B, int N, int H, int D,
                  void* codes, float* scales, float* delta, void* stream) {
  dm::QuantParams p;
  DM_TRY(quant_params(p, x, x_sb, x_sh, x_sn, mean, prescale, o, o_sb, o_sh, o_sn, B, N, H, D, codes, scales, delta));
  cudaError_t e = dm::launch_quant(p, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : cuda_fail(e, "quantiser launch");
}

int dm_quant_qkv(const void* q, int64_t q_sb, int64_t q_sh, int64_t q_sn,
                 const void* k, int64_t k_sb, int64_t k_sh, int64_t k_sn,
                 const void* v, int64_t v_sb, int64_t v_sh, int64_t v_sn,
                 int B, int N, int H, int Hk, int D,
                 void* q8, void* k8, void* v8, float* qs, float* ks, float* vs, float* kmean,
                 void* workspace, void* stream) {
  DM_TRY(check_shape(B, N, H, Hk, D));
  // the softmax scale is baked into the Q codes as an fp32 multiply (delta_matching/reference.py:408)
  const float sm = static_cast<float>(1.0 / sqrt(static_cast<double>(D)));
  DM_TRY(check_device_ptr(kmean, "kmean"));
  DM_TRY(check_device_ptr(workspace, "workspace"));
  dm::QuantParams pq, pk, pv;
  DM_TRY(quant_params(pq, q, q_sb, q_sh, q_sn, nullptr, sm, nullptr, 0, 0, 0, B, N, H, D, q8, qs, nullptr));
  DM_TRY(quant_params(pk, k, k_sb, k_sh, k_sn, kmean, 1.0f, nullptr, 0, 0, 0, B, N, Hk, D, k8, ks, nullptr));
  DM_TRY(quant_params(pv, v, v_sb, v_sh, v_sn, nullptr, 1.0f, nullptr, 0, 0, 0, B, N, Hk, D, v8, vs, nullptr));
  dm::KMeanParams pm{static_cast<const __nv_bfloat16*>(k), k_sb, k_sh, k_sn, static_cast<float*>(workspace), kmean, B, Hk, N, D};
  // three launches: [chunk sums of the K mean | Q | V] in one grid, the fold of the chunk sums, then K
  cudaError_t e = dm::launch_quant_qkv(pq, pk, pv, pm, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : cuda_fail(e, "producer launch");
}

int dm_quant_do(const void* d_o, int64_t do_sb, int64_t do_sh, int64_t do_sn,
                const void* o, int64_t o_sb, int64_t o_sh, int64_t o_sn,
                int B, int N, int H, int D, void* do8, float* dos, float* delta, void* stream) {
  return dm_quant_rows(d_o, do_sb, do_sh, do_sn, nullptr, 1.0f, o, o_sb, o_sh, o_sn, B, N, H, D, do8, dos, delta, stream);
}

static int fwd_impl(const void* q8, const void* k8, const void* v8, const float* qs, const float* ks, const float* vs,
                    int B, int N, int H, int Hk, int D, int causal,
                    void* o, int64_t o_sb, int64_t o_sn, int64_t o_sh, float* lse, int* status, void* stream,
                    int unordered) {
  DM_TRY(check_shape(B, N, H, Hk, D));
  DM_TRY(check_sm100());
  DM_TRY(check_device_ptr(q8, "q8")); DM_TRY(check_device_ptr(k8, "k8")); DM_TRY(check_device_ptr(v8, "v8"));
  DM_TRY(check_device_ptr(qs, "q scales")); DM_TRY(check_device_ptr(ks, "k scales")); DM_TRY(check_device_ptr(vs, "v scales"));
  DM_TRY(check_device_ptr(o, "o")); DM_TRY(check_device_ptr(lse, "lse"));
  DM_TRY(check_strides("o", o_sb, o_sn, o_sh));
  CUtensorMap tq, tk, tv;
  DM_TRY(make_code_map(&tq, q8, static_cast<uint64_t>(B) * H * N, D));
  DM_TRY(make_code_map(&tk, k8, static_cast<uint64_t>(B) * Hk * N, D));
  DM_TRY(make_code_map(&tv, v8, static_cast<uint64_t>(B) * Hk * N, D));
  dm::FwdParams p{qs, ks, vs, static_cast<__nv_bfloat16*>(o), o_sb, o_sn, o_sh, lse, B, H, Hk, N, causal ? 1 : 0, status,
                  unordered};
  cudaError_t e = dm::launch_fwd(D, tq, tk, tv, p, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : cuda_fail(e, "forward launch");
}

int dm_fwd(const void* q8, const void* k8, const void* v8, const float* qs, const float* ks, const float* vs,
           int B, int N, int H, int Hk, int D, int causal,
           void* o, int64_t o_sb, int64_t o_sn, int64_t o_sh, float* lse, int* status, void* stream) {
  return fwd_impl(q8, k8, v8, qs, ks, vs, B, N, H, Hk, D, causal, o, o_sb, o_sn, o_sh, lse, status, stream, 0);
}

int dm_dbg_fwd_unordered(const void* q8, const void* k8, const void* v8, const float* qs, const float* ks, const float* vs,
                         int B, int N, int H, int Hk, int D, int causal,
                         void* o, int64_t o_sb, int64_t o_sn, int64_t o_sh, float* lse, int* status, void* stream) {
  return fwd_impl(q8, k8, v8, qs, ks, vs, B, N, H, Hk, D, causal, o, o_sb, o_sn, o_sh, lse, status, stream, 1);
}

static int delta_impl(const void* q8, const void* k8, const void* v8, const void* do8,
                      const float* qs, const float* ks, const float* vs, const float* dos, const float* lse,
                      int B, int N, int H, int Hk, int D, int causal, float* delta, int* status, void* stream, int norm) {
  DM_TRY(check_shape(B, N, H, Hk, D));
  DM_TRY(check_sm100());
  DM_TRY(check_device_ptr(q8, "q8")); DM_TRY(check_device_ptr(k8, "k8")); DM_TRY(check_device_ptr(v8, "v8"));
  DM_TRY(check_device_ptr(do8, "do8"));
  DM_TRY(check_device_ptr(qs, "q scales")); DM_TRY(check_device_ptr(ks, "k scales")); DM_TRY(check_device_ptr(vs, "v scales"));
  DM_TRY(check_device_ptr(dos, "do scales")); DM_TRY(check_device_ptr(lse, "lse")); DM_TRY(check_device_ptr(delta, "delta"));
  CUtensorMap tq, tk, tv, td;
  DM_TRY(make_code_map(&tq, q8, static_cast<uint64_t>(B) * H * N, D));
  DM_TRY(make_code_map(&tk, k8, static_cast<uint64_t>(B) * Hk * N, D));
  DM_TRY(make_code_map(&tv, v8, static_cast<uint64_t>(B) * Hk * N, D));
  DM_TRY(make_code_map(&td, do8, static_cast<uint64_t>(B) * H * N, D));
  dm::DeltaParams p{qs, ks, vs, dos, lse, delta, B, H, Hk, N, causal ? 1 : 0, status, norm};
  cudaError_t e = dm::launch_delta(D, tq, tk, tv, td, p, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : cuda_fail(e, "matched-delta launch");
}

int dm_delta(const void* q8, const void* k8, const void* v8, const void* do8,
             const float* qs, const float* ks, const float* vs, const float* dos, const float* lse,
             int B, int N, int H, int Hk, int D, int causal, float* delta, int* status, void* stream) {
  return delta_impl(q8, k8, v8, do8, qs, ks, vs, dos, lse, B, N, H, Hk, D, causal, delta, status, stream, 1);
}

int dm_delta_sum(const void* q8, const void* k8, const void* v8, const void* do8,
                 const float* qs, const float* ks, const float* vs, const float* dos, const float* lse,
                 int B, int N, int H, int Hk, int D, int causal, float* delta, int* status, void* stream) {
  return delta_impl(q8, k8, v8, do8, qs, ks, vs, dos, lse, B, N, H, Hk, D, causal, delta, status, stream, 0);
}

static int bwd_impl(const void* q8, const void* k8, const void* v8, const void* do8,
                    const float* qs, const float* ks, const float* vs, const float* dos,
                    const float* lse, const float* delta,
                    int B, int N, int H, int Hk, int D, int causal,
                    void* dq, int64_t dq_sb, int64_t dq_sn, int64_t dq_sh,
                    void* dk, int64_t dk_sb, int64_t dk_sn, int64_t dk_sh,
                    void* dv, int64_t dv_sb, int64_t dv_sn, int64_t dv_sh,
                    float* rowsum_ds, float* sum_abs_pdp, void* workspace, int64_t workspace_bytes, int parts,
                    int* status, void* stream) {
  if ((parts & 3) == 0 || (parts & ~7))
    return fail(DM_ERR_ARG, "delta_matching: parts must be 1 (dK/dV), 2 (dQ) or 3, plus 4 for 32 x 32 dS blocks (got %d)", parts);
  DM_TRY(check_shape(B, N, H, Hk, D));
  DM_TRY(check_sm100());
  DM_TRY(check_device_ptr(q8, "q8")); DM_TRY(check_device_ptr(k8, "k8")); DM_TRY(check_device_ptr(v8, "v8"));
  DM_TRY(check_device_ptr(do8, "do8"));
  DM_TRY(check_device_ptr(qs, "q scales")); DM_TRY(check_device_ptr(ks, "k scales")); DM_TRY(check_device_ptr(vs, "v scales"));
  DM_TRY(check_device_ptr(dos, "do scales")); DM_TRY(check_device_ptr(lse, "lse")); DM_TRY(check_device_ptr(delta, "delta"));
  DM_TRY(check_device_ptr(dq, "dq")); DM_TRY(check_device_ptr(dk, "dk")); DM_TRY(check_device_ptr(dv, "dv"));
  DM_TRY(check_strides("dq", dq_sb, dq_sn, dq_sh));
  DM_TRY(check_strides("dk", dk_sb, dk_sn, dk_sh));
  DM_TRY(check_strides("dv", dv_sb, dv_sn, dv_sh));
  if ((rowsum_ds == nullptr) != (sum_abs_pdp == nullptr))
    return fail(DM_ERR_ARG, "delta_matching: rowsum_ds and sum_abs_pdp must be given together");
  CUtensorMap tq, tk, tv, td;
  DM_TRY(make_code_map(&tq, q8, static_cast<uint64_t>(B) * H * N, D));
  DM_TRY(make_code_map(&tk, k8, static_cast<uint64_t>(B) * Hk * N, D));
  DM_TRY(make_code_map(&tv, v8, static_cast<uint64_t>(B) * Hk * N, D));
  DM_TRY(make_code_map(&td, do8, static_cast<uint64_t>(B) * H * N, D));
  dm::BwdParams p{};
  p.qs = qs; p.ks = ks; p.vs = vs; p.dos = dos; p.lse = lse; p.delta = delta;
  p.dq = static_cast<__nv_bfloat16*>(dq); p.dq_sb = dq_sb; p.dq_sn = dq_sn; p.dq_sh = dq_sh;
  p.dk = static_cast<__nv_bfloat16*>(dk); p.dk_sb = dk_sb; p.dk_sn = dk_sn; p.dk_sh = dk_sh;
  p.dv = static_cast<__nv_bfloat16*>(dv); p.dv_sb = dv_sb; p.dv_sn = dv_sn; p.dv_sh = dv_sh;
  p.rowsum_ds = rowsum_ds; p.sum_abs_pdp = sum_abs_pdp;
  p.sm_scale = static_cast<float>(1.0 / sqrt(static_cast<double>(D)));
  p.B = B; p.H = H; p.Hk = Hk; p.N = N; p.causal = causal ? 1 : 0; p.status = status;
  p.ds32 = (parts & 4) ? 1 : 0;
  CUtensorMap tds;
  if (workspace != nullptr) {
    const int64_t need = dm_bwd_workspace_bytes(B, N, H, D);
    if (need == 0) return fail(DM_ERR_ARG, "delta_matching: no dS workspace size for this shape (head_dim %d, seqlen %d)", D, N);
    if (workspace_bytes < need)
      return fail(DM_ERR_ARG, "delta_matching: dS workspace of %lld bytes given, %lld needed", (long long)workspace_bytes, (long long)need);
    DM_TRY(check_device_ptr(workspace, "workspace"));
    if (!aligned16(workspace)) return fail(DM_ERR_ARG, "delta_matching: workspace must be 16-byte aligned");
    const uint64_t tiles = static_cast<uint64_t>(B) * H * (N / 128) * (N / 128);
    if (tiles * 128 >= (1ull << 31))
      return fail(DM_ERR_ARG, "delta_matching: B * H * (N / 128)^2 = %llu tiles exceed one workspace (split the heads)", (unsigned long long)tiles);
    p.ds_codes = static_cast<uint8_t*>(workspace);
    p.ds_words = p.ds_codes + tiles * 16384;
    DM_TRY(make_code_map(&tds, workspace, tiles * 128, 128));
  }
  if (parts & 1) {
    cudaError_t e = dm::launch_bwd_dkdv(D, tq, tk, tv, td, (workspace != nullptr) ? &tds : nullptr, p,
                                        static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(e, "backward dK/dV launch");
  }
  if (parts & 2) {
    cudaError_t e = (workspace != nullptr) ? dm::launch_bwd_dq_p2(D, tds, tk, p, static_cast<cudaStream_t>(stream))
                                           : dm::launch_bwd_dq(D, tq, tk, tv, td, p, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(e, "backward dQ launch");
  }
  return 0;
}

int64_t dm_bwd_workspace_bytes(int B, int N, int H, int D) {
  if ((D != 128 && D != 256) || B <= 0 || H <= 0 || N <= 0 || (N % 128) != 0) return 0;
  const int64_t tiles = static_cast<int64_t>(B) * H * (N / 128) * (N / 128);
  return tiles * (16384 + 16);
}

int dm_bwd_ws(const void* q8, const void* k8, const void* v8, const void* do8,
              const float* qs, const float* ks, const float* vs, const float* dos,
              const float* lse, const float* delta,
              int B, int N, int H, int Hk, int D, int causal,
              void* dq, int64_t dq_sb, int64_t dq_sn, int64_t dq_sh,
              void* dk, int64_t dk_sb, int64_t dk_sn, int64_t dk_sh,
              void* dv, int64_t dv_sb, int64_t dv_sn, int64_t dv_sh,
              void* workspace, int64_t workspace_bytes, int parts, int* status, void* stream) {
  if (workspace == nullptr) return fail(DM_ERR_ARG, "delta_matching: workspace is NULL (dm_bwd is the entry point without one)");
  return bwd_impl(q8, k8, v8, do8, qs, ks, vs, dos, lse, delta, B, N, H, Hk, D, causal, dq, dq_sb, dq_sn, dq_sh,
                  dk, dk_sb, dk_sn, dk_sh, dv, dv_sb, dv_sn, dv_sh, nullptr, nullptr, workspace, workspace_bytes, parts,
                  status, stream);
}

int dm_bwd_parts(const void* q8, const void* k8, const void* v8, const void* do8,
                 const float* qs, const float* ks, const float* vs, const float* dos,
                 const float* lse, const float* delta,
                 int B, int N, int H, int Hk, int D, int causal,
                 void* dq, int64_t dq_sb, int64_t dq_sn, int64_t dq_sh,
                 void* dk, int64_t dk_sb, int64_t dk_sn, int64_t dk_sh,
                 void* dv, int64_t dv_sb, int64_t dv_sn, int64_t dv_sh,
                 float* rowsum_ds, float* sum_abs_pdp, int parts, int* status, void* stream) {
  return bwd_impl(q8, k8, v8, do8, qs, ks, vs, dos, lse, delta, B, N, H, Hk, D, causal, dq, dq_sb, dq_sn, dq_sh,
                  dk, dk_sb, dk_sn, dk_sh, dv, dv_sb, dv_sn, dv_sh, rowsum_ds, sum_abs_pdp, nullptr, 0, parts, status,
                  stream);
}

int dm_bwd(const void* q8, const void* k8, const void* v8, const void* do8,
           const float* qs, const float* ks, const float* vs, const float* dos,
           const float* lse, const float* delta,
           int B, int N, int H, int Hk, int D, int causal,
           void* dq, int64_t dq_sb, int64_t dq_sn, int64_t dq_sh,
           void* dk, int64_t dk_sb, int64_t dk_sn, int64_t dk_sh,
           void* dv, int64_t dv_sb, int64_t dv_sn, int64_t dv_sh,
           float* rowsum_ds, float* sum_abs_pdp, int* status, void* stream) {
  return dm_bwd_parts(q8, k8, v8, do8, qs, ks, vs, dos, lse, delta, B, N, H, Hk, D, causal, dq, dq_sb, dq_sn, dq_sh,
                      dk, dk_sb, dk_sn, dk_sh, dv, dv_sb, dv_sn, dv_sh, rowsum_ds, sum_abs_pdp, 3, status, stream);
}

int dm_dbg_mma_tile(const void* a, const void* b, const uint32_t* sfa, const uint32_t* sfb, int a_tmem, int a_mn,
                    int b_mn, int scaled, int nk, float* out, int* status, void* stream) {
  DM_TRY(check_sm100());
  DM_TRY(check_device_ptr(a, "a")); DM_TRY(check_device_ptr(b, "b")); DM_TRY(check_device_ptr(out, "out"));
  if (nk < 1 || nk > 4) return fail(DM_ERR_ARG, "delta_matching: nk must be in 1..4 (got %d)", nk);
  if (a_tmem && a_mn) return fail(DM_ERR_ARG, "delta_matching: an A operand in TMEM has no major mode (a_mn must be 0)");
  if (scaled) { DM_TRY(check_device_ptr(sfa, "sfa")); DM_TRY(check_device_ptr(sfb, "sfb")); }
  CUtensorMap ta, tb;
  DM_TRY(make_code_map(&ta, a, 128, 128));
  DM_TRY(make_code_map(&tb, b, 128, 128));
  dm::ProbeParams p{static_cast<const uint8_t*>(a), sfa, sfb, out, a_tmem, a_mn, b_mn, scaled, nk, status, 0, 0};
  cudaError_t e = dm::launch_probe(ta, tb, p, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : cuda_fail(e, "probe launch");
}

int dm_dbg_wait_expiry(const void* a, const void* b, float* out, long long limit_ns, int* status, void* stream) {
  DM_TRY(check_sm100());
  DM_TRY(check_device_ptr(a, "a")); DM_TRY(check_device_ptr(b, "b")); DM_TRY(check_device_ptr(out, "out"));
  if (status == nullptr) return fail(DM_ERR_ARG, "delta_matching: the expiry probe needs a status word");
  if (limit_ns < 1000 || limit_ns > 1000000000ll)
    return fail(DM_ERR_ARG, "delta_matching: limit_ns must be between 1 microsecond and 1 second (got %lld)", limit_ns);
  CUtensorMap ta, tb;
  DM_TRY(make_code_map(&ta, a, 128, 128));
  DM_TRY(make_code_map(&tb, b, 128, 128));
  dm::ProbeParams p{static_cast<const uint8_t*>(a), nullptr, nullptr, out, 0, 0, 0, 0, 4, status, 1,
                    static_cast<uint64_t>(limit_ns)};
  cudaError_t e = dm::launch_probe(ta, tb, p, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : cuda_fail(e, "probe launch");
}

long long dm_launch_count(void) { return dm::launch_count(); }

int dm_copy_2d_async(void* dst, int64_t dpitch, const void* src, int64_t spitch, int64_t width, int64_t height,
                     int to_device, void* stream) {
  if (dst == nullptr || src == nullptr) return fail(DM_ERR_ARG, "delta_matching: dm_copy_2d_async: NULL pointer");
  if (width < 0 || height < 0 || dpitch < width || spitch < width)
    return fail(DM_ERR_ARG, "delta_matching: dm_copy_2d_async: pitches must be at least the row width");
  if (width == 0 || height == 0) return 0;
  cudaError_t e = cudaMemcpy2DAsync(dst, static_cast<size_t>(dpitch), src, static_cast<size_t>(spitch),
                                    static_cast<size_t>(width), static_cast<size_t>(height),
                                    to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost,
                                    static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : cuda_fail(e, "strided copy");
}

}  // extern "C"
