// Row gather and owner scatter-add used by the explicit-GEMM algorithm
// (gather rows -> dense GEMM -> add into the owning output rows).
#include "wcn_common.cuh"

namespace {

// 16-byte vectors when a row is a whole number of them, else element-wise.
__global__ void gather_rows_vec_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ idx,
                                       uint4* __restrict__ dst, int64_t rows, int vec_per_row) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows * vec_per_row) return;
  const int64_t r = t / vec_per_row;
  const int v = (int)(t - r * vec_per_row);
  dst[t] = __ldg(&src[(int64_t)__ldg(&idx[r]) * vec_per_row + v]);
}

template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ src, const int32_t* __restrict__ idx,
                                   T* __restrict__ dst, int64_t rows, int channels) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows * channels) return;
  const int64_t r = t / channels;
  const int c = (int)(t - r * channels);
  dst[t] = src[(int64_t)idx[r] * channels + c];
}

template <typename T>
__global__ void scatter_add_rows_kernel(const T* __restrict__ src, const int32_t* __restrict__ idx,
                                        T* __restrict__ dst, int64_t rows, int channels) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows * channels) return;
  const int64_t r = t / channels;
  const int c = (int)(t - r * channels);
  T* d = dst + (int64_t)idx[r] * channels + c;
  // the add is rounded once to the storage type, like `dst[idx] += src` in that type
  *d = wcn_from_float<T>(wcn_to_float<T>(*d) + wcn_to_float<T>(src[t]));
}

}  // namespace

extern "C" int wcn_gather_rows(const void* src, const int32_t* idx, void* dst, int64_t num_rows,
                               int32_t channels, int dtype, void* stream) {
  if (num_rows < 0 || channels <= 0 || dtype < WCN_F32 || dtype > WCN_BF16) return WCN_ERR_INVALID_PARAMETERS;
  if (num_rows == 0) return WCN_OK;
  if (!src || !idx || !dst) return WCN_ERR_INVALID_PARAMETERS;
  cudaStream_t st = wcn_stream(stream);
  const int64_t row_bytes = (int64_t)channels * wcn_dtype_size(dtype);
  const bool vec = row_bytes % 16 == 0 && !(reinterpret_cast<uintptr_t>(src) & 15) &&
                   !(reinterpret_cast<uintptr_t>(dst) & 15);
  if (vec) {
    const int vpr = (int)(row_bytes / 16);
    const int64_t total = num_rows * vpr;
    gather_rows_vec_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
        reinterpret_cast<const uint4*>(src), idx, reinterpret_cast<uint4*>(dst), num_rows, vpr);
  } else {
    const int64_t total = num_rows * channels;
    const unsigned grid = (unsigned)((total + 255) / 256);
    if (dtype == WCN_F32)
      gather_rows_kernel<float><<<grid, 256, 0, st>>>((const float*)src, idx, (float*)dst, num_rows, channels);
    else  // 16-bit types move as raw bits
      gather_rows_kernel<uint16_t><<<grid, 256, 0, st>>>((const uint16_t*)src, idx, (uint16_t*)dst, num_rows, channels);
  }
  WCN_CHECK_LAUNCH();
  return WCN_OK;
}

extern "C" int wcn_scatter_add_rows(const void* src, const int32_t* idx, void* dst, int64_t num_rows,
                                    int32_t channels, int dtype, void* stream) {
  if (num_rows < 0 || channels <= 0) return WCN_ERR_INVALID_PARAMETERS;
  if (num_rows == 0) return WCN_OK;
  if (!src || !idx || !dst) return WCN_ERR_INVALID_PARAMETERS;
  cudaStream_t st = wcn_stream(stream);
  const int64_t total = num_rows * channels;
  const unsigned grid = (unsigned)((total + 255) / 256);
  switch (dtype) {
    case WCN_F32: scatter_add_rows_kernel<float><<<grid, 256, 0, st>>>((const float*)src, idx, (float*)dst, num_rows, channels); break;
    case WCN_F16: scatter_add_rows_kernel<__half><<<grid, 256, 0, st>>>((const __half*)src, idx, (__half*)dst, num_rows, channels); break;
    case WCN_BF16: scatter_add_rows_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)src, idx, (__nv_bfloat16*)dst, num_rows, channels); break;
    default: return WCN_ERR_INVALID_PARAMETERS;
  }
  WCN_CHECK_LAUNCH();
  return WCN_OK;
}
