// Output-stationary sparse convolution on the FP32 pipes.  This is the kernel
// for fp32 tensors (where tensor-core formats would lose the 1e-4 accuracy
// bound) and for shapes the tcgen05 kernel does not take.  One block owns a
// 64-row x 64-column output tile, walks the kernel offsets that have at least
// one neighbour in the tile, gathers the neighbour rows into shared memory and
// accumulates in fp32 registers; every output element is written once.
#include "wcn_common.cuh"

namespace {

constexpr int TM = 64;   // output rows per block
constexpr int TN = 64;   // output columns per block
constexpr int TK = 16;   // input channels per step
constexpr int NT = 256;  // threads: 16 x 16, each a 4 x 4 micro-tile

// Row strides (elements) of the three matrices, the number of feature rows an index may name
// and where to report one that does not (null: such an index is skipped silently).
struct RowLayout {
  int64_t in_ld, out_ld, res_ld;
  int num_in;
  int32_t* dev_status;
};

template <typename T, typename TO>
__global__ void __launch_bounds__(NT)
conv_simt_kernel(const T* __restrict__ feats, const T* __restrict__ weight, const int32_t* __restrict__ nbr,
                 const int32_t* __restrict__ out_rows, int64_t M, int K, int c_in, int c_out, const float* __restrict__ scale,
                 const float* __restrict__ shift, const TO* __restrict__ residual, int relu,
                 TO* __restrict__ out, const RowLayout lay) {
  __shared__ float As[TK][TM + 4];
  __shared__ float Ws[TK][TN + 4];
  __shared__ int rows[TM];

  const int64_t m0 = (int64_t)blockIdx.x * TM;
  const int n0 = blockIdx.y * TN;
  const int tx = threadIdx.x & 15;  // column group
  const int ty = threadIdx.x >> 4;  // row group
  float acc[4][4] = {};
  bool bad = false;

  for (int k = 0; k < K; ++k) {
    int r = -1;
    if (threadIdx.x < TM) {
      const int64_t m = m0 + threadIdx.x;
      r = m < M ? __ldg(&nbr[(int64_t)k * M + m]) : -1;
      if (r >= lay.num_in) {  // not a feature row: treated as absent, reported once when the thread is done
        r = -1;
        bad = true;
      }
      rows[threadIdx.x] = r;
    }
    if (!__syncthreads_or(r >= 0)) continue;  // no neighbour at this offset in the tile
    const T* wk = weight + (int64_t)k * c_in * c_out;
    for (int c0 = 0; c0 < c_in; c0 += TK) {
      // A: TM x TK gathered rows (zero where the neighbour is absent)
#pragma unroll
      for (int e = threadIdx.x; e < TM * TK; e += NT) {
        const int rr = e / TK, cc = e % TK;
        const int src = rows[rr];
        float v = 0.f;
        if (src >= 0 && c0 + cc < c_in) v = wcn_to_float<T>(feats[(int64_t)src * lay.in_ld + c0 + cc]);
        As[cc][rr] = v;
      }
      // W: TK x TN slice of weight[k]
#pragma unroll
      for (int e = threadIdx.x; e < TK * TN; e += NT) {
        const int cc = e / TN, nn = e % TN;
        float v = 0.f;
        if (c0 + cc < c_in && n0 + nn < c_out) v = wcn_to_float<T>(wk[(int64_t)(c0 + cc) * c_out + n0 + nn]);
        Ws[cc][nn] = v;
      }
      __syncthreads();
#pragma unroll
      for (int cc = 0; cc < TK; ++cc) {
        float a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = As[cc][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = Ws[cc][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
      __syncthreads();
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t slot = m0 + ty * 4 + i;
    if (slot >= M) continue;
    const int64_t m = out_rows ? (int64_t)__ldg(&out_rows[slot]) : slot;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= c_out) continue;
      float y = acc[i][j];
      y = wcn_affine(y, scale, shift, n);
      if (residual) y = __fadd_rn(y, wcn_to_float<TO>(residual[m * lay.res_ld + n]));
      if (relu) y = fmaxf(y, 0.f);
      out[m * lay.out_ld + n] = wcn_from_float<TO>(y);
    }
  }
  if (bad) wcn_report_bounds(lay.dev_status);
}

template <typename T, typename TO>
int launch_simt(const void* feats, const void* weight, const int32_t* nbr, const int32_t* out_rows, int64_t M, int K, int c_in,
                int c_out, const float* scale, const float* shift, const void* residual, int relu, void* out,
                const RowLayout& lay, cudaStream_t st) {
  dim3 grid((unsigned)((M + TM - 1) / TM), (unsigned)((c_out + TN - 1) / TN));
  conv_simt_kernel<T, TO><<<grid, NT, 0, st>>>((const T*)feats, (const T*)weight, nbr, out_rows, M, K, c_in, c_out, scale,
                                              shift, (const TO*)residual, relu, (TO*)out, lay);
  return cudaGetLastError() == cudaSuccess ? WCN_OK : WCN_ERR_EXECUTION;
}


// ------------------------------------------------------------------ narrow inputs
//
// Layers with a handful of input channels (the 3 -> 32 stem of a network) are pure
// streaming: a few bytes in, a row of c_out values out.  One thread owns 8 output channels of
// one output row, the whole weight tensor sits in shared memory as fp32, and consecutive
// threads write consecutive 16-byte (32-byte for fp32) pieces, so the output is written in
// full lines.  Accumulation order (offset-major, then input channel, fused multiply-add) is
// the one of conv_simt_kernel, so fp32 results are bit-identical to it.
constexpr int NARROW_MAX_CIN = 8;
constexpr int NARROW_MAX_WEIGHTS = 8192;  // floats of shared memory

template <typename T, typename TO>
__global__ void __launch_bounds__(NT)
conv_narrow_kernel(const T* __restrict__ feats, const T* __restrict__ weight, const int32_t* __restrict__ nbr,
                   const int32_t* __restrict__ out_rows, int64_t M, int K, int c_in, int c_out,
                   const float* __restrict__ scale, const float* __restrict__ shift,
                   const TO* __restrict__ residual, int relu, TO* __restrict__ out, const RowLayout lay) {
  __shared__ __align__(16) float w_s[NARROW_MAX_WEIGHTS];
  for (int i = threadIdx.x; i < K * c_in * c_out; i += NT) w_s[i] = wcn_to_float<T>(weight[i]);
  __syncthreads();
  const int groups = c_out >> 3;
  const int64_t t = (int64_t)blockIdx.x * NT + threadIdx.x;
  const int64_t slot = t / groups;
  const int n0 = (int)(t - slot * groups) * 8;
  if (slot >= M) return;
  float acc[8] = {};
  bool bad = false;
  for (int k = 0; k < K; ++k) {
    const int src = __ldg(&nbr[(int64_t)k * M + slot]);
    if (src < 0) continue;
    if (src >= lay.num_in) {
      bad = true;
      continue;
    }
    const T* x = feats + (int64_t)src * lay.in_ld;
    for (int c = 0; c < c_in; ++c) {
      const float xv = wcn_to_float<T>(x[c]);
      const float4 w0 = *reinterpret_cast<const float4*>(&w_s[(k * c_in + c) * c_out + n0]);
      const float4 w1 = *reinterpret_cast<const float4*>(&w_s[(k * c_in + c) * c_out + n0 + 4]);
      acc[0] = fmaf(xv, w0.x, acc[0]); acc[1] = fmaf(xv, w0.y, acc[1]);
      acc[2] = fmaf(xv, w0.z, acc[2]); acc[3] = fmaf(xv, w0.w, acc[3]);
      acc[4] = fmaf(xv, w1.x, acc[4]); acc[5] = fmaf(xv, w1.y, acc[5]);
      acc[6] = fmaf(xv, w1.z, acc[6]); acc[7] = fmaf(xv, w1.w, acc[7]);
    }
  }
  const int64_t m = out_rows ? (int64_t)__ldg(&out_rows[slot]) : slot;
  constexpr int VEC = (int)(8 * sizeof(TO) / 16);  // 16-byte pieces of 8 outputs
  __align__(16) TO tmp[8];
  if (residual) {
#pragma unroll
    for (int v = 0; v < VEC; ++v)
      reinterpret_cast<uint4*>(tmp)[v] = __ldg(reinterpret_cast<const uint4*>(residual + m * lay.res_ld + n0) + v);
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float y = acc[j];
    y = wcn_affine(y, scale, shift, n0 + j);
    if (residual) y = __fadd_rn(y, wcn_to_float<TO>(tmp[j]));
    if (relu) y = fmaxf(y, 0.f);
    tmp[j] = wcn_from_float<TO>(y);
  }
#pragma unroll
  for (int v = 0; v < VEC; ++v) reinterpret_cast<uint4*>(out + m * lay.out_ld + n0)[v] = reinterpret_cast<uint4*>(tmp)[v];
  if (bad) wcn_report_bounds(lay.dev_status);
}

template <typename T, typename TO>
int launch_narrow(const void* feats, const void* weight, const int32_t* nbr, const int32_t* out_rows, int64_t M,
                  int K, int c_in, int c_out, const float* scale, const float* shift, const void* residual,
                  int relu, void* out, const RowLayout& lay, cudaStream_t st) {
  const int64_t threads = M * (c_out >> 3);
  conv_narrow_kernel<T, TO><<<(unsigned)((threads + NT - 1) / NT), NT, 0, st>>>(
      (const T*)feats, (const T*)weight, nbr, out_rows, M, K, c_in, c_out, scale, shift, (const TO*)residual, relu,
      (TO*)out, lay);
  return cudaGetLastError() == cudaSuccess ? WCN_OK : WCN_ERR_EXECUTION;
}

// ------------------------------------------------------------------ narrow outputs
//
// Layers with at most 32 output channels that the tensor-core kernel does not take (a
// 96 -> 20 classification head): one thread owns ROWS consecutive output rows, reads their input
// rows with 16-byte loads, keeps all outputs in registers and takes the weights (fp32, padded to NP
// columns) from shared memory, where every lane reads the same address.  A weight quad fetched
// from shared memory feeds ROWS x 4 multiply-adds, which is what keeps the kernel off the
// shared-memory pipe (with one row per thread it was bound by it).  Accumulation order per output
// is the one of conv_simt_kernel.
template <typename T, typename TO, int NP, int ROWS>
__global__ void __launch_bounds__(NT)
conv_narrow_out_kernel(const T* __restrict__ feats, const T* __restrict__ weight, const int32_t* __restrict__ nbr,
                       const int32_t* __restrict__ out_rows, int64_t M, int K, int c_in, int c_out,
                       const float* __restrict__ scale, const float* __restrict__ shift,
                       const TO* __restrict__ residual, int relu, TO* __restrict__ out, const RowLayout lay) {
  __shared__ __align__(16) float w_s[NARROW_MAX_WEIGHTS];  // [K][c_in][NP]
  for (int i = threadIdx.x; i < K * c_in * NP; i += NT) {
    const int n = i % NP, kc = i / NP;
    w_s[i] = n < c_out ? wcn_to_float<T>(weight[(int64_t)kc * c_out + n]) : 0.f;
  }
  __syncthreads();
  const int64_t slot0 = ((int64_t)blockIdx.x * NT + threadIdx.x) * ROWS;
  if (slot0 >= M) return;
  constexpr int EPV = 16 / (int)sizeof(T);  // input elements per 16-byte load
  float acc[ROWS][NP];
  bool bad = false;
#pragma unroll
  for (int r = 0; r < ROWS; ++r)
#pragma unroll
    for (int j = 0; j < NP; ++j) acc[r][j] = 0.f;
  for (int k = 0; k < K; ++k) {
    const uint4* x[ROWS];
    bool any = false;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      int src = slot0 + r < M ? __ldg(&nbr[(int64_t)k * M + slot0 + r]) : -1;
      if (src >= lay.num_in) {
        bad = true;
        src = -1;
      }
      x[r] = src >= 0 ? reinterpret_cast<const uint4*>(feats + (int64_t)src * lay.in_ld) : nullptr;
      any = any || src >= 0;
    }
    if (!any) continue;
    const float* wk = w_s + (int64_t)k * c_in * NP;
    for (int c0 = 0; c0 < c_in; c0 += EPV) {
      uint4 raw[ROWS];
#pragma unroll
      for (int r = 0; r < ROWS; ++r) raw[r] = x[r] ? __ldg(x[r] + c0 / EPV) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int e = 0; e < EPV; ++e) {
        float xf[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) xf[r] = wcn_to_float<T>(reinterpret_cast<const T*>(&raw[r])[e]);
        const float4* w4 = reinterpret_cast<const float4*>(wk + (c0 + e) * NP);
#pragma unroll
        for (int q = 0; q < NP / 4; ++q) {
          const float4 w = w4[q];
#pragma unroll
          for (int r = 0; r < ROWS; ++r) {
            if (x[r]) {  // an absent neighbour adds nothing (and keeps -0.0 sums exactly as the row-wise kernel does)
              acc[r][4 * q + 0] = fmaf(xf[r], w.x, acc[r][4 * q + 0]);
              acc[r][4 * q + 1] = fmaf(xf[r], w.y, acc[r][4 * q + 1]);
              acc[r][4 * q + 2] = fmaf(xf[r], w.z, acc[r][4 * q + 2]);
              acc[r][4 * q + 3] = fmaf(xf[r], w.w, acc[r][4 * q + 3]);
            }
          }
        }
      }
    }
  }
  constexpr int PER8 = (int)(8 / sizeof(TO));  // outputs per 8-byte store
  const bool wide = (c_out % PER8) == 0 && (lay.out_ld % PER8) == 0 &&
                    (reinterpret_cast<uintptr_t>(out) & 7) == 0;  // rows start 8-byte aligned
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int64_t slot = slot0 + r;
    if (slot >= M) break;
    const int64_t m = out_rows ? (int64_t)__ldg(&out_rows[slot]) : slot;
    TO* orow = out + m * lay.out_ld;
    const TO* rrow = residual ? residual + m * lay.res_ld : nullptr;
#pragma unroll
    for (int j0 = 0; j0 < NP; j0 += PER8) {
      __align__(8) TO o[PER8];
#pragma unroll
      for (int i = 0; i < PER8; ++i) {
        const int j = j0 + i;
        float y = acc[r][j];
        if (j < c_out) {
          y = wcn_affine(y, scale, shift, j);
          if (rrow) y = __fadd_rn(y, wcn_to_float<TO>(rrow[j]));
          if (relu) y = fmaxf(y, 0.f);
        }
        o[i] = wcn_from_float<TO>(y);
      }
      if (wide) {
        if (j0 < c_out) *reinterpret_cast<uint2*>(orow + j0) = *reinterpret_cast<const uint2*>(o);
      } else {
#pragma unroll
        for (int i = 0; i < PER8; ++i)
          if (j0 + i < c_out) orow[j0 + i] = o[i];
      }
    }
  }
  if (bad) wcn_report_bounds(lay.dev_status);
}

template <typename T, typename TO>
int launch_narrow_out(const void* feats, const void* weight, const int32_t* nbr, const int32_t* out_rows, int64_t M,
                      int K, int c_in, int c_out, const float* scale, const float* shift, const void* residual,
                      int relu, void* out, const RowLayout& lay, cudaStream_t st) {
#define WCN_NOUT(NPV, ROWSV)                                                                                        \
  conv_narrow_out_kernel<T, TO, NPV, ROWSV><<<(unsigned)((M + (int64_t)NT * ROWSV - 1) / ((int64_t)NT * ROWSV)), NT, 0, st>>>( \
      (const T*)feats, (const T*)weight, nbr, out_rows, M, K, c_in, c_out, scale, shift, (const TO*)residual, relu,   \
      (TO*)out, lay)
  if (c_out <= 8) WCN_NOUT(8, 4);
  else if (c_out <= 16) WCN_NOUT(16, 4);
  else if (c_out <= 24) WCN_NOUT(24, 4);
  else WCN_NOUT(32, 2);
#undef WCN_NOUT
  return cudaGetLastError() == cudaSuccess ? WCN_OK : WCN_ERR_EXECUTION;
}

}  // namespace

static RowLayout make_layout(int64_t num_in, int64_t feats_ld, int64_t out_ld, int64_t residual_ld, int32_t* dev_status) {
  RowLayout lay;
  lay.in_ld = feats_ld; lay.out_ld = out_ld; lay.res_ld = residual_ld;
  lay.num_in = (int)(num_in < 0x7FFFFFFFll ? num_in : 0x7FFFFFFFll);
  lay.dev_status = dev_status;
  return lay;
}

int wcn_conv_simt_fwd(const void* feats, int64_t num_in, int64_t feats_ld, const void* weight, const int32_t* nbr,
                      const int32_t* out_rows, int64_t M, int K, int c_in, int c_out, int dtype, const float* scale,
                      const float* shift, const void* residual, int64_t residual_ld, int relu, void* out,
                      int64_t out_ld, int out_dtype, int32_t* dev_status, cudaStream_t st) {
  const RowLayout lay = make_layout(num_in, feats_ld, out_ld, residual_ld, dev_status);
#define WCN_SIMT_CASE(DT, T, ODT, TO) \
  if (dtype == DT && out_dtype == ODT) \
    return launch_simt<T, TO>(feats, weight, nbr, out_rows, M, K, c_in, c_out, scale, shift, residual, relu, out, lay, st);
  WCN_SIMT_CASE(WCN_F32, float, WCN_F32, float)
  WCN_SIMT_CASE(WCN_F16, __half, WCN_F16, __half)
  WCN_SIMT_CASE(WCN_BF16, __nv_bfloat16, WCN_BF16, __nv_bfloat16)
  WCN_SIMT_CASE(WCN_F16, __half, WCN_F32, float)
  WCN_SIMT_CASE(WCN_BF16, __nv_bfloat16, WCN_F32, float)
  WCN_SIMT_CASE(WCN_F32, float, WCN_F16, __half)
  WCN_SIMT_CASE(WCN_F32, float, WCN_BF16, __nv_bfloat16)
#undef WCN_SIMT_CASE
  return WCN_ERR_UNSUPPORTED_CONFIG;
}

// Rows of `out` and `residual` must start on 16-byte boundaries for the vector stores.
bool wcn_conv_narrow_supported(int K, int c_in, int c_out, const void* out, int64_t out_ld, const void* residual,
                               int64_t residual_ld, int out_dtype) {
  const int64_t osz = out_dtype == WCN_F32 ? 4 : 2;
  return c_in <= NARROW_MAX_CIN && c_out % 8 == 0 && (int64_t)K * c_in * c_out <= NARROW_MAX_WEIGHTS &&
         (reinterpret_cast<uintptr_t>(out) & 15) == 0 && (reinterpret_cast<uintptr_t>(residual) & 15) == 0 &&
         (out_ld * osz) % 16 == 0 && (!residual || (residual_ld * osz) % 16 == 0);
}

int wcn_conv_narrow_fwd(const void* feats, int64_t num_in, int64_t feats_ld, const void* weight, const int32_t* nbr,
                        const int32_t* out_rows, int64_t M, int K, int c_in, int c_out, int dtype,
                        const float* scale, const float* shift, const void* residual, int64_t residual_ld, int relu,
                        void* out, int64_t out_ld, int out_dtype, int32_t* dev_status, cudaStream_t st) {
  const RowLayout lay = make_layout(num_in, feats_ld, out_ld, residual_ld, dev_status);
#define WCN_NARROW_CASE(DT, T, ODT, TO) \
  if (dtype == DT && out_dtype == ODT) \
    return launch_narrow<T, TO>(feats, weight, nbr, out_rows, M, K, c_in, c_out, scale, shift, residual, relu, out, lay, st);
  WCN_NARROW_CASE(WCN_F32, float, WCN_F32, float)
  WCN_NARROW_CASE(WCN_F16, __half, WCN_F16, __half)
  WCN_NARROW_CASE(WCN_BF16, __nv_bfloat16, WCN_BF16, __nv_bfloat16)
  WCN_NARROW_CASE(WCN_F16, __half, WCN_F32, float)
  WCN_NARROW_CASE(WCN_BF16, __nv_bfloat16, WCN_F32, float)
#undef WCN_NARROW_CASE
  return WCN_ERR_UNSUPPORTED_CONFIG;
}

// Feature rows must start on 16-byte boundaries for the vector loads.
bool wcn_conv_narrow_out_supported(int K, int c_in, int c_out, int dtype, const void* feats, int64_t feats_ld) {
  const int np = (c_out + 7) / 8 * 8;
  return c_out <= 32 && (int64_t)K * c_in * np <= NARROW_MAX_WEIGHTS && (c_in * wcn_dtype_size(dtype)) % 16 == 0 &&
         (feats_ld * wcn_dtype_size(dtype)) % 16 == 0 && (reinterpret_cast<uintptr_t>(feats) & 15) == 0;
}

int wcn_conv_narrow_out_fwd(const void* feats, int64_t num_in, int64_t feats_ld, const void* weight,
                            const int32_t* nbr, const int32_t* out_rows, int64_t M, int K, int c_in, int c_out,
                            int dtype, const float* scale, const float* shift, const void* residual,
                            int64_t residual_ld, int relu, void* out, int64_t out_ld, int out_dtype,
                            int32_t* dev_status, cudaStream_t st) {
  const RowLayout lay = make_layout(num_in, feats_ld, out_ld, residual_ld, dev_status);
#define WCN_NOUT_CASE(DT, T, ODT, TO) \
  if (dtype == DT && out_dtype == ODT) \
    return launch_narrow_out<T, TO>(feats, weight, nbr, out_rows, M, K, c_in, c_out, scale, shift, residual, relu, out, lay, st);
  WCN_NOUT_CASE(WCN_F32, float, WCN_F32, float)
  WCN_NOUT_CASE(WCN_F16, __half, WCN_F16, __half)
  WCN_NOUT_CASE(WCN_BF16, __nv_bfloat16, WCN_BF16, __nv_bfloat16)
  WCN_NOUT_CASE(WCN_F16, __half, WCN_F32, float)
  WCN_NOUT_CASE(WCN_BF16, __nv_bfloat16, WCN_F32, float)
#undef WCN_NOUT_CASE
  return WCN_ERR_UNSUPPORTED_CONFIG;
}
