// Parameters of the one-tile tcgen05 building-block check (dm_probe.cu).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dm {

struct ProbeParams {
  const uint8_t* a_codes;      // 128 x 128 e4m3, row-major (used directly when A is staged in TMEM)
  const uint32_t* sfa_words;   // 128 lanes x 4 columns of 32-bit scale words (block-scaled runs)
  const uint32_t* sfb_words;
  float* out;                  // 128 x 128 fp32, row-major
  int a_tmem;                  // A operand from TMEM (rows = lanes) instead of shared memory
  int a_mn, b_mn;              // shared-memory operand is MN-major (tile rows = contraction index)
  int scaled;                  // kind::mxf8f6f4.block_scale instead of kind::f8f6f4
  int nk;                      // 32-wide contraction steps (1..4); step k uses scale byte k
  int* status;
  int skip_commit;             // the MMA role leaves out its commit: the waits of every thread run out (expiry check)
  uint64_t wait_limit_ns;      // limit of those waits; 0 = the kernels' own limit
};

cudaError_t launch_probe(const CUtensorMap& ta, const CUtensorMap& tb, const ProbeParams& p, cudaStream_t stream);

}  // namespace dm
