// Sequential host driver around the reference's Morton-code kernel
// (warpconvnet/csrc/morton_code.cu).  REF_SRC is the absolute path of that file.
#include "cuda_cpu_shim.h"
#include REF_SRC

// Launch shape of morton_code() in coords/ops/serialization.py:245-250:
// ceil(N / (256*4)) blocks of 256 threads, 4 points per thread.
extern "C" int ref_morton20(const int* coords_xyz, int num_points, long long* codes) {
  const int threads = 256;
  blockDim = {(unsigned)threads, 1, 1};
  long long blocks = ((long long)num_points + threads * 4 - 1) / (threads * 4);
  gridDim = {(unsigned)blocks, 1, 1};
  for (long long b = 0; b < blocks; ++b) {
    blockIdx = {(unsigned)b, 0, 0};
    for (int t = 0; t < threads; ++t) {
      threadIdx = {(unsigned)t, 0, 0};
      assign_order_discrete_20bit_kernel_4points(coords_xyz, num_points, (int64_t*)codes);
    }
  }
  return 0;
}
