// dm_kmean_static: the K mean for callers that must not allocate.
//
// dm_kmean needs a scratch buffer for its per-chunk column sums, and someone has to allocate it.  Some callers cannot:
// code running inside a region where the allocator is off limits (a framework's no-allocation section, a real-time loop,
// a plugin that was handed a fixed arena and nothing else) or code that simply has no handle on the host program's
// memory pool.  For them this entry point keeps the scratch inside the library itself, as a fixed array in device
// global memory.  The price: the array is created on every GPU that loads the library and stays until the process ends,
// so it is kept small (kScratchFloats below), and problems that need more are refused instead of served.
//
// The array's name is only meaningful to device code.  Host code that wants to hand the array to a kernel has to ask the
// runtime for its device address (cudaGetSymbolAddress) with the right device current; passing the name itself would
// give the kernel a host-side placeholder.  That lookup happens here on the first call per device and is cached.
#include <cstdio>
#include <mutex>

#include "dm_kernels.h"

namespace {

// 4 MiB: B * Hk * (N / 64) * D floats.  Enough for B * Hk * N <= 524288 tokens at head_dim 128 (e.g. 4 x 8 x 16384).
constexpr size_t kScratchFloats = 1u << 20;
static __device__ __align__(256) float g_kmean_scratch[kScratchFloats];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {};
std::mutex g_setup_mutex;

int refuse(char* err, int err_len, int code, const char* msg) {
  if (err != nullptr && err_len > 0) snprintf(err, err_len, "%s", msg);
  return code;
}

// Device or managed memory that the current device owns, 16-byte aligned: the same demand dm_kmean makes of its
// pointers.  cudaPointerGetAttributes allocates nothing.  Returns nullptr when the pointer passes, else the complaint.
const char* bad_pointer(const void* ptr, int dev, const char* what, char* msg, size_t msg_len) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, ptr) != cudaSuccess) {
    cudaGetLastError();
    snprintf(msg, msg_len, "delta_matching: %s must be CUDA memory", what);
    return msg;
  }
  if (a.type != cudaMemoryTypeDevice && a.type != cudaMemoryTypeManaged) {
    snprintf(msg, msg_len, "delta_matching: %s must be CUDA memory (got a host pointer)", what);
    return msg;
  }
  if (a.type == cudaMemoryTypeDevice && a.device != dev) {
    snprintf(msg, msg_len, "delta_matching: %s is on device %d but the current device is %d", what, a.device, dev);
    return msg;
  }
  if (reinterpret_cast<uintptr_t>(ptr) & 15) {
    snprintf(msg, msg_len, "delta_matching: %s must be 16-byte aligned", what);
    return msg;
  }
  return nullptr;
}

}  // namespace

extern "C" int dm_kmean_static(const void* k, int64_t k_sb, int64_t k_sh, int64_t k_sn, int B, int N, int Hk, int D,
                               float* mean, void* stream, char* err, int err_len) {
  if (k == nullptr || mean == nullptr) return refuse(err, err_len, -1, "delta_matching: k and mean must be CUDA buffers (got NULL)");
  if (D != 128 && D != 256) return refuse(err, err_len, -1, "delta_matching: head_dim must be 128 or 256");
  if (B <= 0 || Hk <= 0 || N <= 0 || N % 128) return refuse(err, err_len, -1, "delta_matching: B, Hk must be positive and seqlen a positive multiple of 128");
  if ((k_sb % 8) || (k_sh % 8) || (k_sn % 8) || (reinterpret_cast<uintptr_t>(k) & 15))
    return refuse(err, err_len, -1, "delta_matching: k must be 16-byte aligned with strides that are multiples of 8 elements");
  const size_t need = static_cast<size_t>(B) * Hk * (N / 64) * D;
  if (need > kScratchFloats) {
    char msg[256];
    snprintf(msg, sizeof(msg), "delta_matching: dm_kmean_static needs %zu scratch floats but its built-in scratch holds %zu "
             "(B * Hk * (N / 64) * D must not exceed it); use dm_kmean with a caller-provided workspace", need, kScratchFloats);
    return refuse(err, err_len, -1, msg);
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0) return refuse(err, err_len, -2, "delta_matching: cudaGetDevice failed");
  if (dev >= kMaxDevices) {
    char msg[160];
    snprintf(msg, sizeof(msg), "delta_matching: dm_kmean_static keeps its scratch address for devices 0..%d; the current "
             "device is %d (use dm_kmean)", kMaxDevices - 1, dev);
    return refuse(err, err_len, -1, msg);
  }
  {
    char msg[200];
    if (bad_pointer(k, dev, "k", msg, sizeof(msg)) != nullptr) return refuse(err, err_len, -1, msg);
    if (bad_pointer(mean, dev, "mean", msg, sizeof(msg)) != nullptr) return refuse(err, err_len, -1, msg);
  }
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_addr[dev] == nullptr) {
      // once per device, with that device current: the device address of the array as this GPU sees it
      float* p = nullptr;
      e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_kmean_scratch);
      if (e != cudaSuccess || p == nullptr) {
        char msg[256];
        snprintf(msg, sizeof(msg), "delta_matching: cudaGetSymbolAddress for the built-in scratch failed: %s", cudaGetErrorString(e));
        return refuse(err, err_len, -2, msg);
      }
      g_scratch_addr[dev] = p;
    }
    scratch = g_scratch_addr[dev];
  }
  // Nothing in the scratch has to start at zero: stage 1 writes every chunk sum that stage 2 reads.
  dm::KMeanParams p{static_cast<const __nv_bfloat16*>(k), k_sb, k_sh, k_sn, scratch, mean, B, Hk, N, D};
  e = dm::launch_kmean(p, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    char msg[256];
    snprintf(msg, sizeof(msg), "delta_matching: k-mean launch failed: %s", cudaGetErrorString(e));
    return refuse(err, err_len, -2, msg);
  }
  return 0;
}
