// Host-side stand-ins for the few CUDA builtins used by the reference's
// self-contained kernel sources, so that g++ can compile those sources as
// plain C++ where they lie.  Test infrastructure only: nothing in the product
// links against this.
//
// A "launch" is emulated by the drivers in this folder: they loop over every
// (block, thread) index, store it in the thread-local variables below and call
// the kernel body as an ordinary function.  Execution is sequential, so
// atomicCAS needs no real atomicity.
#pragma once
#define __global__
#define __device__
#define __host__
#define __forceinline__ inline
#ifndef __restrict__
#define __restrict__
#endif

struct wcn_shim_dim3 { unsigned int x, y, z; };
static thread_local wcn_shim_dim3 blockIdx = {0, 0, 0};
static thread_local wcn_shim_dim3 threadIdx = {0, 0, 0};
static thread_local wcn_shim_dim3 blockDim = {1, 1, 1};
static thread_local wcn_shim_dim3 gridDim = {1, 1, 1};

static inline int atomicCAS(int* address, int compare, int val) {
  int old = *address;
  if (old == compare) *address = val;
  return old;
}
