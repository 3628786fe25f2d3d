// Row gather and owner scatter-add used by the explicit-GEMM algorithm
// (gather rows -> dense GEMM -> add into the owning output rows).
#include "wcn_common.cuh"

namespace {

// 16-byte vectors when a row is a whole number of them, else element-wise.
// An index outside [0, limit) is not followed: the caller's policy (zero row / skipped add)
// applies and the status word, when there is one, receives WCN_ERR_BOUNDS.
__device__ __forceinline__ bool row_in_range(int64_t i, int64_t limit, int32_t* dev_status) {
  if (i >= 0 && i < limit) return true;
  wcn_report_bounds(dev_status);
  return false;
}

__global__ void gather_rows_vec_kernel(const uint4* __restrict__ src, int64_t num_src, const int32_t* __restrict__ idx,
                                       uint4* __restrict__ dst, int64_t rows, int vec_per_row, int32_t* dev_status) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows * vec_per_row) return;
  const int64_t r = t / vec_per_row;
  const int v = (int)(t - r * vec_per_row);
  const int64_t i = __ldg(&idx[r]);
  dst[t] = row_in_range(i, num_src, dev_status) ? __ldg(&src[i * vec_per_row + v]) : make_uint4(0, 0, 0, 0);
}

template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ src, int64_t num_src, const int32_t* __restrict__ idx,
                                   T* __restrict__ dst, int64_t rows, int channels, int32_t* dev_status) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows * channels) return;
  const int64_t r = t / channels;
  const int c = (int)(t - r * channels);
  const int64_t i = idx[r];
  dst[t] = row_in_range(i, num_src, dev_status) ? src[i * channels + c] : T(0);
}

template <typename T>
__global__ void scatter_add_rows_kernel(const T* __restrict__ src, const int32_t* __restrict__ idx,
                                        T* __restrict__ dst, int64_t num_dst, int64_t rows, int channels,
                                        int32_t* dev_status) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= rows * channels) return;
  const int64_t r = t / channels;
  const int c = (int)(t - r * channels);
  const int64_t i = idx[r];
  if (!row_in_range(i, num_dst, dev_status)) return;
  T* d = dst + i * channels + c;
  // the add is rounded once to the storage type, like `dst[idx] += src` in that type
  *d = wcn_from_float<T>(wcn_to_float<T>(*d) + wcn_to_float<T>(src[t]));
}

}  // namespace

extern "C" int wcn_gather_rows(const void* src, int64_t num_src, const int32_t* idx, void* dst, int64_t num_rows,
                               int32_t channels, int dtype, int32_t* dev_status, void* stream) {
  if (num_rows < 0 || num_src < 0 || channels <= 0 || dtype < WCN_F32 || dtype > WCN_BF16) return WCN_ERR_INVALID_PARAMETERS;
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
        reinterpret_cast<const uint4*>(src), num_src, idx, reinterpret_cast<uint4*>(dst), num_rows, vpr, dev_status);
  } else {
    const int64_t total = num_rows * channels;
    const unsigned grid = (unsigned)((total + 255) / 256);
    if (dtype == WCN_F32)
      gather_rows_kernel<float><<<grid, 256, 0, st>>>((const float*)src, num_src, idx, (float*)dst, num_rows, channels, dev_status);
    else  // 16-bit types move as raw bits
      gather_rows_kernel<uint16_t><<<grid, 256, 0, st>>>((const uint16_t*)src, num_src, idx, (uint16_t*)dst, num_rows, channels, dev_status);
  }
  WCN_CHECK_LAUNCH();
  return WCN_OK;
}

extern "C" int wcn_scatter_add_rows(const void* src, const int32_t* idx, void* dst, int64_t num_dst, int64_t num_rows,
                                    int32_t channels, int dtype, int32_t* dev_status, void* stream) {
  if (num_rows < 0 || num_dst < 0 || channels <= 0) return WCN_ERR_INVALID_PARAMETERS;
  if (num_rows == 0) return WCN_OK;
  if (!src || !idx || !dst) return WCN_ERR_INVALID_PARAMETERS;
  cudaStream_t st = wcn_stream(stream);
  const int64_t total = num_rows * channels;
  const unsigned grid = (unsigned)((total + 255) / 256);
  switch (dtype) {
    case WCN_F32: scatter_add_rows_kernel<float><<<grid, 256, 0, st>>>((const float*)src, idx, (float*)dst, num_dst, num_rows, channels, dev_status); break;
    case WCN_F16: scatter_add_rows_kernel<__half><<<grid, 256, 0, st>>>((const __half*)src, idx, (__half*)dst, num_dst, num_rows, channels, dev_status); break;
    case WCN_BF16: scatter_add_rows_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)src, idx, (__nv_bfloat16*)dst, num_dst, num_rows, channels, dev_status); break;
    default: return WCN_ERR_INVALID_PARAMETERS;
  }
  WCN_CHECK_LAUNCH();
  return WCN_OK;
}

// ------------------------------------------------------------------ pooling

namespace {

// out[m, :] = reduce over the offsets k that have a neighbour (nbr[k*M + m] >= 0) of
// feats[nbr[k*M + m], :]; rows without any neighbour become 0.  One thread owns VEC consecutive
// channels of one output row, walks the offsets in order and accumulates in fp32.
template <typename T, int VEC>
__global__ void row_reduce_kernel(const T* __restrict__ feats, int num_in, const int32_t* __restrict__ nbr, int64_t M,
                                  int K, int channels, int op, T* __restrict__ out, int32_t* dev_status) {
  const int vpr = channels / VEC;
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t m = t / vpr;
  if (m >= M) return;
  const int c0 = (int)(t - m * vpr) * VEC;
  float acc[VEC];
  int count = 0;
  bool bad = false;
  for (int k = 0; k < K; ++k) {
    const int src = __ldg(&nbr[(int64_t)k * M + m]);
    if (src < 0) continue;
    if (src >= num_in) {  // not a feature row: counts as absent, reported once when the thread is done
      bad = true;
      continue;
    }
    __align__(16) T v[VEC];
    if (VEC > 1) {
      constexpr int PIECES = (int)(VEC * sizeof(T) / 16);
#pragma unroll
      for (int q = 0; q < PIECES; ++q)
        reinterpret_cast<uint4*>(v)[q] = __ldg(reinterpret_cast<const uint4*>(feats + (int64_t)src * channels + c0) + q);
    } else {
      v[0] = feats[(int64_t)src * channels + c0];
    }
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const float x = wcn_to_float<T>(v[i]);
      if (count == 0) acc[i] = x;
      else if (op == WCN_REDUCE_MIN) acc[i] = fminf(acc[i], x);
      else if (op == WCN_REDUCE_MAX) acc[i] = fmaxf(acc[i], x);
      else if (op == WCN_REDUCE_MUL) acc[i] = __fmul_rn(acc[i], x);
      else acc[i] = __fadd_rn(acc[i], x);  // sum, mean
    }
    ++count;
  }
  __align__(16) T o[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    float y = count ? acc[i] : 0.f;
    if (op == WCN_REDUCE_MEAN && count) y = __fdiv_rn(y, (float)count);
    o[i] = wcn_from_float<T>(y);
  }
  if (VEC > 1) {
    constexpr int PIECES = (int)(VEC * sizeof(T) / 16);
#pragma unroll
    for (int q = 0; q < PIECES; ++q)
      reinterpret_cast<uint4*>(out + m * channels + c0)[q] = reinterpret_cast<uint4*>(o)[q];
  } else {
    out[m * channels + c0] = o[0];
  }
  if (bad) wcn_report_bounds(dev_status);
}

template <typename T>
int launch_row_reduce(const void* feats, int num_in, const int32_t* nbr, int64_t M, int K, int channels, int op,
                      void* out, int32_t* dev_status, cudaStream_t st) {
  constexpr int VEC = (int)(16 / sizeof(T));
  const bool vec = channels % VEC == 0 && !(reinterpret_cast<uintptr_t>(feats) & 15) &&
                   !(reinterpret_cast<uintptr_t>(out) & 15);
  if (vec) {
    const int64_t total = M * (channels / VEC);
    row_reduce_kernel<T, VEC><<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const T*)feats, num_in, nbr, M, K,
                                                                              channels, op, (T*)out, dev_status);
  } else {
    const int64_t total = M * channels;
    row_reduce_kernel<T, 1><<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const T*)feats, num_in, nbr, M, K,
                                                                            channels, op, (T*)out, dev_status);
  }
  return cudaGetLastError() == cudaSuccess ? WCN_OK : WCN_ERR_EXECUTION;
}

}  // namespace

extern "C" int wcn_row_reduce(const void* feats, int64_t num_in, const int32_t* nbr, int64_t num_out,
                              int32_t num_offsets, int32_t channels, int dtype, int op, void* out,
                              int32_t* dev_status, void* stream) {
  if (num_out < 0 || num_in < 0 || num_offsets <= 0 || channels <= 0 || op < WCN_REDUCE_MIN || op > WCN_REDUCE_MUL)
    return WCN_ERR_INVALID_PARAMETERS;
  const int nin = (int)(num_in < 0x7FFFFFFFll ? num_in : 0x7FFFFFFFll);
  if (num_out == 0) return WCN_OK;
  if (!nbr || !out) return WCN_ERR_INVALID_PARAMETERS;
  if ((int64_t)num_out * channels >= (int64_t)0x7FFFFFFF * 256) return WCN_ERR_INVALID_PARAMETERS;
  cudaStream_t st = wcn_stream(stream);
  switch (dtype) {
    case WCN_F32: return launch_row_reduce<float>(feats, nin, nbr, num_out, num_offsets, channels, op, out, dev_status, st);
    case WCN_F16: return launch_row_reduce<__half>(feats, nin, nbr, num_out, num_offsets, channels, op, out, dev_status, st);
    case WCN_BF16: return launch_row_reduce<__nv_bfloat16>(feats, nin, nbr, num_out, num_offsets, channels, op, out, dev_status, st);
    default: return WCN_ERR_INVALID_PARAMETERS;
  }
}
