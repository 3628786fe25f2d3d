// Entry points that do not belong to one kernel family: version, status text and
// the convolution dispatcher.
#include "wcn_common.cuh"

// conv_simt.cu
int wcn_conv_simt_fwd(const void* feats, int64_t num_in, int64_t feats_ld, const void* weight, const int32_t* nbr,
                      const int32_t* out_rows, int64_t M, int K, int c_in, int c_out, int dtype, const float* scale,
                      const float* shift, const void* residual, int64_t residual_ld, int relu, void* out,
                      int64_t out_ld, int out_dtype, int32_t* dev_status, cudaStream_t st);
bool wcn_conv_narrow_supported(int K, int c_in, int c_out, const void* out, int64_t out_ld, const void* residual,
                               int64_t residual_ld, int out_dtype);
int wcn_conv_narrow_fwd(const void* feats, int64_t num_in, int64_t feats_ld, const void* weight, const int32_t* nbr,
                        const int32_t* out_rows, int64_t M, int K, int c_in, int c_out, int dtype,
                        const float* scale, const float* shift, const void* residual, int64_t residual_ld, int relu,
                        void* out, int64_t out_ld, int out_dtype, int32_t* dev_status, cudaStream_t st);
bool wcn_conv_narrow_out_supported(int K, int c_in, int c_out, int dtype, const void* feats, int64_t feats_ld);
int wcn_conv_narrow_out_fwd(const void* feats, int64_t num_in, int64_t feats_ld, const void* weight,
                            const int32_t* nbr, const int32_t* out_rows, int64_t M, int K, int c_in, int c_out,
                            int dtype, const float* scale, const float* shift, const void* residual,
                            int64_t residual_ld, int relu, void* out, int64_t out_ld, int out_dtype,
                            int32_t* dev_status, cudaStream_t st);
// conv_tcgen05.cu
bool wcn_conv_tcgen05_supported(int K, int c_in, int c_out, int dtype, int out_dtype);
int64_t wcn_conv_tcgen05_packed_bytes(int K, int c_in, int c_out);
int64_t wcn_conv_tcgen05_workspace_bytes(int64_t M, int K, int c_in, int c_out, int split_k);
int wcn_conv_tcgen05_pack(const void* weight, int K, int c_in, int c_out, void* packed, cudaStream_t st);
int wcn_conv_tcgen05_fwd(const void* feats, int64_t num_in, int64_t feats_ld, const void* packed, const int32_t* nbr,
                         const int32_t* out_rows, int64_t M, int K, int c_in, int c_out, int dtype,
                         const float* scale, const float* shift, const void* residual, int64_t residual_ld, int relu,
                         void* out, int64_t out_ld, int out_dtype, int split_k, void* workspace,
                         int64_t workspace_bytes, int32_t* dev_status, cudaStream_t st);
// conv_wgrad_tcgen05.cu
bool wcn_conv_wgrad_tcgen05_supported(int K, int c_in, int c_out, int dtype);
int wcn_conv_wgrad_tcgen05(const void* feats, int64_t num_in, const void* grad_out, const int32_t* nbr,
                           const int32_t* out_rows, const uint32_t* tile_masks, int64_t M, int K, int c_in, int c_out, int dtype,
                           float* grad_weight, int32_t* dev_status, cudaStream_t st);

extern "C" int wcn_version(void) { return 100; }

extern "C" const char* wcn_status_string(int status) {
  switch (status) {
    case WCN_OK: return "success";
    case WCN_ERR_PROBLEM_NOT_SUPPORTED: return "problem not supported";
    case WCN_ERR_INITIALIZATION: return "kernel initialization failed";
    case WCN_ERR_EXECUTION: return "kernel launch or execution failed";
    case WCN_ERR_UNSUPPORTED_CONFIG: return "unsupported configuration";
    case WCN_ERR_INVALID_PARAMETERS: return "invalid parameters";
    case WCN_ERR_HASH_OVERFLOW: return "hash table overflow";
    case WCN_ERR_WAIT_EXPIRED: return "a bounded device-side wait expired";
    case WCN_ERR_BOUNDS: return "index out of bounds";
    case WCN_ERR_SCRATCH_TOO_SMALL: return "problem larger than the library's built-in scratch array";
    default: return "unknown status";
  }
}

extern "C" int wcn_conv_packed_weight_bytes(int algo, int32_t num_offsets, int32_t c_in, int32_t c_out,
                                            int dtype, int64_t* bytes) {
  if (!bytes || num_offsets <= 0 || c_in <= 0 || c_out <= 0) return WCN_ERR_INVALID_PARAMETERS;
  *bytes = 0;
  if (algo == WCN_CONV_SIMT) return WCN_OK;
  const bool ok = wcn_conv_tcgen05_supported(num_offsets, c_in, c_out, dtype, dtype);
  if (!ok) return algo == WCN_CONV_TCGEN05 ? WCN_ERR_UNSUPPORTED_CONFIG : WCN_OK;
  *bytes = wcn_conv_tcgen05_packed_bytes(num_offsets, c_in, c_out);
  return WCN_OK;
}

extern "C" int wcn_conv_pack_weight(int algo, const void* weight, int32_t num_offsets, int32_t c_in,
                                    int32_t c_out, int dtype, void* packed, void* stream) {
  if (!weight || !packed) return WCN_ERR_INVALID_PARAMETERS;
  if (algo == WCN_CONV_SIMT || !wcn_conv_tcgen05_supported(num_offsets, c_in, c_out, dtype, dtype))
    return WCN_ERR_UNSUPPORTED_CONFIG;
  return wcn_conv_tcgen05_pack(weight, num_offsets, c_in, c_out, packed, wcn_stream(stream));
}

static bool conv_takes_tcgen05(int algo, bool tc_ok, const void* packed_weight, const int32_t* dev_status,
                               int64_t num_in) {
  return algo == WCN_CONV_TCGEN05 || (algo == WCN_CONV_AUTO && tc_ok && packed_weight && dev_status && num_in > 0);
}

extern "C" int wcn_conv_workspace_bytes(int algo, int64_t num_out, int32_t num_offsets, int32_t c_in, int32_t c_out,
                                        int dtype, int out_dtype, int32_t split_k, int64_t* bytes) {
  if (!bytes || num_out < 0 || num_offsets <= 0 || c_in <= 0 || c_out <= 0) return WCN_ERR_INVALID_PARAMETERS;
  *bytes = 0;
  if (algo == WCN_CONV_SIMT || !wcn_conv_tcgen05_supported(num_offsets, c_in, c_out, dtype, out_dtype)) return WCN_OK;
  *bytes = wcn_conv_tcgen05_workspace_bytes(num_out, num_offsets, c_in, c_out, split_k);
  return WCN_OK;
}

extern "C" int wcn_conv_fwd(int algo, const void* feats, int64_t num_in, int64_t feats_ld, const void* weight,
                            const void* packed_weight, const int32_t* nbr, const int32_t* out_rows,
                            int64_t num_out, int32_t num_offsets, int32_t c_in, int32_t c_out, int dtype,
                            const float* scale, const float* shift, const void* residual, int64_t residual_ld,
                            int relu, void* out, int64_t out_ld, int out_dtype, int32_t split_k, void* workspace,
                            int64_t workspace_bytes, int32_t* dev_status, void* stream) {
  if (num_in < 0 || num_out < 0 || num_offsets <= 0 || c_in <= 0 || c_out <= 0) return WCN_ERR_INVALID_PARAMETERS;
  if (num_in >= 0x7FFFFFFFll || num_out >= 0x7FFFFFFFll) return WCN_ERR_INVALID_PARAMETERS;  // row numbers are 32-bit
  if (dtype < WCN_F32 || dtype > WCN_BF16 || out_dtype < WCN_F32 || out_dtype > WCN_BF16)
    return WCN_ERR_INVALID_PARAMETERS;
  if (feats_ld == 0) feats_ld = c_in;  // 0: rows are dense
  if (out_ld == 0) out_ld = c_out;
  if (residual_ld == 0) residual_ld = c_out;
  if (feats_ld < c_in || out_ld < c_out || residual_ld < c_out) return WCN_ERR_INVALID_PARAMETERS;
  if (num_out == 0) return WCN_OK;
  if (!nbr || !out || (num_in > 0 && !feats)) return WCN_ERR_INVALID_PARAMETERS;
  cudaStream_t st = wcn_stream(stream);
  const bool tc_ok = wcn_conv_tcgen05_supported(num_offsets, c_in, c_out, dtype, out_dtype);
  if (conv_takes_tcgen05(algo, tc_ok, packed_weight, dev_status, num_in)) {
    if (!tc_ok) return WCN_ERR_UNSUPPORTED_CONFIG;
    return wcn_conv_tcgen05_fwd(feats, num_in, feats_ld, packed_weight, nbr, out_rows, num_out, num_offsets, c_in,
                                c_out, dtype, scale, shift, residual, residual_ld, relu, out, out_ld, out_dtype,
                                split_k, workspace, workspace_bytes, dev_status, st);
  }
  if (algo != WCN_CONV_SIMT && algo != WCN_CONV_AUTO) return WCN_ERR_INVALID_PARAMETERS;
  if (!weight) return WCN_ERR_INVALID_PARAMETERS;
  if (algo == WCN_CONV_AUTO && wcn_conv_narrow_supported(num_offsets, c_in, c_out, out, out_ld, residual, residual_ld, out_dtype)) {
    // a few input channels: the streaming kernel (same numbers as the FP32-pipe kernel)
    const int rc = wcn_conv_narrow_fwd(feats, num_in, feats_ld, weight, nbr, out_rows, num_out, num_offsets, c_in,
                                       c_out, dtype, scale, shift, residual, residual_ld, relu, out, out_ld,
                                       out_dtype, dev_status, st);
    if (rc != WCN_ERR_UNSUPPORTED_CONFIG) return rc;
  }
  if (algo == WCN_CONV_AUTO && num_in > 0 && wcn_conv_narrow_out_supported(num_offsets, c_in, c_out, dtype, feats, feats_ld)) {
    // a few output channels (a classification head): one thread per output row
    const int rc = wcn_conv_narrow_out_fwd(feats, num_in, feats_ld, weight, nbr, out_rows, num_out, num_offsets, c_in,
                                           c_out, dtype, scale, shift, residual, residual_ld, relu, out, out_ld,
                                           out_dtype, dev_status, st);
    if (rc != WCN_ERR_UNSUPPORTED_CONFIG) return rc;
  }
  return wcn_conv_simt_fwd(feats, num_in, feats_ld, weight, nbr, out_rows, num_out, num_offsets, c_in, c_out, dtype,
                           scale, shift, residual, residual_ld, relu, out, out_ld, out_dtype, dev_status, st);
}

bool wcn_conv_rows_shape_supported(int K, int c_in, int c_out_packed, int dtype, int out_dtype);
int wcn_conv_rows_tcgen05_fwd(const void* feats, int64_t num_in, int64_t feats_ld, const void* packed,
                              const int32_t* dst_rows, int64_t num_out, int K, int c_in, int c_out_packed, int c_out,
                              int dtype, const float* scale, const float* shift, const void* residual,
                              int64_t residual_ld, int relu, void* out, int64_t out_ld, int out_dtype,
                              int32_t* dev_status, cudaStream_t st);

extern "C" int wcn_conv_rows_supported(int32_t num_offsets, int32_t c_in, int32_t c_out_packed, int dtype, int out_dtype,
                                       int32_t* supported) {
  if (!supported) return WCN_ERR_INVALID_PARAMETERS;
  *supported = wcn_conv_rows_shape_supported(num_offsets, c_in, c_out_packed, dtype, out_dtype) ? 1 : 0;
  return WCN_OK;
}

extern "C" int wcn_conv_rows_fwd(const void* feats, int64_t num_in, int64_t feats_ld, const void* packed_weight,
                                 const int32_t* dst_rows, int64_t num_out, int32_t num_offsets, int32_t c_in,
                                 int32_t c_out_packed, int32_t c_out, int dtype, const float* scale, const float* shift,
                                 const void* residual, int64_t residual_ld, int relu, void* out, int64_t out_ld,
                                 int out_dtype, int32_t* dev_status, void* stream) {
  if (num_in < 0 || num_out < 0 || num_offsets <= 0 || c_in <= 0 || c_out <= 0) return WCN_ERR_INVALID_PARAMETERS;
  if (feats_ld == 0) feats_ld = c_in;
  if (out_ld == 0) out_ld = c_out;
  if (residual_ld == 0) residual_ld = c_out;
  if (feats_ld < c_in || out_ld < c_out || residual_ld < c_out) return WCN_ERR_INVALID_PARAMETERS;
  if (num_in == 0 || num_out == 0) return WCN_OK;
  return wcn_conv_rows_tcgen05_fwd(feats, num_in, feats_ld, packed_weight, dst_rows, num_out, num_offsets, c_in,
                                   c_out_packed, c_out, dtype, scale, shift, residual, residual_ld, relu, out, out_ld,
                                   out_dtype, dev_status, wcn_stream(stream));
}

extern "C" int wcn_conv_wgrad(const void* feats, int64_t num_in, const void* grad_out, const int32_t* nbr,
                              const int32_t* out_rows, const uint32_t* tile_masks, int64_t num_out, int32_t num_offsets, int32_t c_in, int32_t c_out, int dtype,
                              float* grad_weight, int32_t* dev_status, void* stream) {
  if (num_in < 0 || num_out < 0 || num_offsets <= 0 || c_in <= 0 || c_out <= 0) return WCN_ERR_INVALID_PARAMETERS;
  if (!wcn_conv_wgrad_tcgen05_supported(num_offsets, c_in, c_out, dtype)) return WCN_ERR_UNSUPPORTED_CONFIG;
  if (num_out == 0 || num_in == 0) return WCN_OK;
  if (!feats || !grad_out || !nbr || !grad_weight || !dev_status) return WCN_ERR_INVALID_PARAMETERS;
  return wcn_conv_wgrad_tcgen05(feats, num_in, grad_out, nbr, out_rows, tile_masks, num_out, num_offsets, c_in, c_out, dtype, grad_weight,
                                dev_status, wcn_stream(stream));
}
