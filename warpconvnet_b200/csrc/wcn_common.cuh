// Shared device helpers for libwcn_b200.so (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <limits.h>
#include <stdint.h>

#include "../../include/wcn_b200.h"

#define WCN_EMPTY_BATCH INT_MIN  // key.x of an empty slot (reserved batch value)

#define WCN_CHECK_LAUNCH()                                     \
  do {                                                         \
    cudaError_t e_ = cudaGetLastError();                       \
    if (e_ != cudaSuccess) return WCN_ERR_EXECUTION;           \
  } while (0)

static inline cudaStream_t wcn_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// ------------------------------------------------------------------ hashing
// Three public 32-bit mixing schemes folded over the four key ints.  Slot
// placement is internal to this library; only lookups are observable.

__device__ __forceinline__ uint32_t wcn_fmix32(uint32_t h) {
  h ^= h >> 16;
  h *= 0x85EBCA6Bu;
  h ^= h >> 13;
  h *= 0xC2B2AE35u;
  h ^= h >> 16;
  return h;
}

template <int METHOD>
__device__ __forceinline__ uint32_t wcn_hash4(int4 k) {
  const uint32_t v[4] = {(uint32_t)k.x, (uint32_t)k.y, (uint32_t)k.z, (uint32_t)k.w};
  if (METHOD == WCN_HASH_FNV1A) {
    uint32_t h = 2166136261u;
#pragma unroll
    for (int i = 0; i < 4; ++i) h = (h ^ v[i]) * 16777619u;
    return wcn_fmix32(h);  // FNV's low bits are its good ones; the slot uses the high ones
  } else if (METHOD == WCN_HASH_MURMUR) {
    uint32_t h = 0x9747B28Cu;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t x = v[i] * 0xCC9E2D51u;
      x = (x << 15) | (x >> 17);
      x *= 0x1B873593u;
      h ^= x;
      h = (h << 13) | (h >> 19);
      h = h * 5u + 0xE6546B64u;
    }
    return wcn_fmix32(h ^ 16u);
  } else {
    uint32_t h = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) h = wcn_fmix32(h + v[i] * 0x9E3779B9u);
    return h;
  }
}

// Multiply-shift range reduction: [0, 2^32) -> [0, cap) without a division.
__device__ __forceinline__ uint32_t wcn_slot(uint32_t h, uint32_t cap) { return __umulhi(h, cap); }

__device__ __forceinline__ bool wcn_key_eq(int4 a, int4 b) {
  return a.x == b.x && a.y == b.y && a.z == b.z && a.w == b.w;
}

__device__ __forceinline__ int wcn_floordiv(int a, int s) {
  int q = a / s;
  return q - ((a % s != 0) && (a < 0));
}

// Probe for `key`; returns its value or -1.  Keys and values live in two arrays
// of the same table buffer: keys[cap] (int4) followed by vals[cap] (int).
template <int METHOD>
__device__ __forceinline__ int wcn_lookup(const int4* __restrict__ tkeys,
                                          const int* __restrict__ tvals, uint32_t cap, int4 key) {
  uint32_t slot = wcn_slot(wcn_hash4<METHOD>(key), cap);
  for (uint32_t p = 0; p < cap; ++p) {
    const int4 cur = __ldg(&tkeys[slot]);
    if (cur.x == WCN_EMPTY_BATCH) return -1;
    if (wcn_key_eq(cur, key)) return __ldg(&tvals[slot]);
    slot = (slot + 1 == cap) ? 0u : slot + 1;
  }
  return -1;
}

// ------------------------------------------------------------------ element types

template <typename T> __device__ __forceinline__ float wcn_to_float(T v);
template <> __device__ __forceinline__ float wcn_to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float wcn_to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float wcn_to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T wcn_from_float(float v);
template <> __device__ __forceinline__ float wcn_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half wcn_from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 wcn_from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Epilogue affine step, written with explicit roundings so that every kernel produces the same
// bits whatever the compiler would have contracted: fma when both are present.
__device__ __forceinline__ float wcn_affine(float y, const float* scale, const float* shift, int n) {
  if (scale && shift) return fmaf(y, scale[n], shift[n]);
  if (scale) return __fmul_rn(y, scale[n]);
  if (shift) return __fadd_rn(y, shift[n]);
  return y;
}

static inline int wcn_dtype_size(int dtype) { return dtype == WCN_F32 ? 4 : 2; }

// An index that names no row was skipped: say so in the status word, unless it already holds
// something (the first report stays; an expired wait is stored unconditionally and wins).
__device__ __forceinline__ void wcn_report_bounds(int32_t* dev_status) {
  if (dev_status) atomicCAS(dev_status, 0, (int)WCN_ERR_BOUNDS);
}
