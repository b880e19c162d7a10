#include "host_util.h"

#include <mutex>

namespace syn {

static thread_local char g_cuda_err[512] = "";

void set_cuda_error(const char* what, const char* detail) {
  snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", what, detail ? detail : "?");
}

int device_sm_count(int* out) {
  static int cached[64];
  int dev = 0;
  SYN_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && cached[dev] > 0) {
    *out = cached[dev];
    return SYN_OK;
  }
  int n = 0;
  SYN_CUDA_TRY(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
  if (dev >= 0 && dev < 64) cached[dev] = n;
  *out = n;
  return SYN_OK;
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

static encode_tiled_fn get_encode_tiled() {
  static encode_tiled_fn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<encode_tiled_fn>(p);
    }
  });
  return fn;
}

int encode_tmap_2d_sw128(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                         uint32_t box_rows, uint32_t box_cols) {
  encode_tiled_fn fn = get_encode_tiled();
  if (fn == nullptr) {
    set_cuda_error("cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)", "not available");
    return SYN_ERR_CUDA;
  }
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[64];
    snprintf(buf, sizeof(buf), "CUresult %d", static_cast<int>(r));
    set_cuda_error("cuTensorMapEncodeTiled(2d)", buf);
    return SYN_ERR_CUDA;
  }
  return SYN_OK;
}

int encode_tmap_2d_plain(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                         uint32_t box_rows, uint32_t box_cols) {
  encode_tiled_fn fn = get_encode_tiled();
  if (fn == nullptr) {
    set_cuda_error("cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)", "not available");
    return SYN_ERR_CUDA;
  }
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[64];
    snprintf(buf, sizeof(buf), "CUresult %d", static_cast<int>(r));
    set_cuda_error("cuTensorMapEncodeTiled(2d plain)", buf);
    return SYN_ERR_CUDA;
  }
  return SYN_OK;
}

int encode_tmap_3d_sw128(CUtensorMap* out, const void* base, uint64_t d2, uint64_t rows, uint64_t cols,
                         uint64_t stride2, uint64_t ld, uint32_t box_rows, uint32_t box_cols) {
  encode_tiled_fn fn = get_encode_tiled();
  if (fn == nullptr) {
    set_cuda_error("cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)", "not available");
    return SYN_ERR_CUDA;
  }
  cuuint64_t gdim[3] = {cols, rows, d2};
  cuuint64_t gstride[2] = {ld * 2, stride2 * 2};
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[64];
    snprintf(buf, sizeof(buf), "CUresult %d", static_cast<int>(r));
    set_cuda_error("cuTensorMapEncodeTiled(3d)", buf);
    return SYN_ERR_CUDA;
  }
  return SYN_OK;
}

int encode_tmap_4d_sw128(CUtensorMap* out, const void* base, uint64_t d3, uint64_t d2, uint64_t rows, uint64_t cols,
                         uint64_t s3, uint64_t s2, uint64_t ld, uint32_t box_rows, uint32_t box_cols) {
  encode_tiled_fn fn = get_encode_tiled();
  if (fn == nullptr) {
    set_cuda_error("cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)", "not available");
    return SYN_ERR_CUDA;
  }
  cuuint64_t gdim[4] = {cols, rows, d2, d3};
  cuuint64_t gstride[3] = {ld * 2, s2 * 2, s3 * 2};
  cuuint32_t box[4] = {box_cols, box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[64];
    snprintf(buf, sizeof(buf), "CUresult %d", static_cast<int>(r));
    set_cuda_error("cuTensorMapEncodeTiled(4d)", buf);
    return SYN_ERR_CUDA;
  }
  return SYN_OK;
}

int status_to_err(int dev_code) {
  switch (dev_code) {
    case 0: return SYN_OK;
    case 1: return SYN_ERR_TIMEOUT_FLAG;
    case 2: return SYN_ERR_TIMEOUT_MBAR;
    case 3: return SYN_ERR_TIMEOUT_COUNTER;
    default: return SYN_ERR_INVALID;
  }
}

}  // namespace syn

extern "C" {

const char* syn_strerror(int code) {
  switch (code) {
    case SYN_OK: return "ok";
    case SYN_ERR_INVALID: return "invalid argument";
    case SYN_ERR_SHAPE: return "schedule entry out of bounds or not a multiple of the block";
    case SYN_ERR_CUDA: return "CUDA call failed (see syn_last_cuda_error)";
    case SYN_ERR_TIMEOUT_FLAG: return "device wait on a signal flag timed out";
    case SYN_ERR_TIMEOUT_MBAR: return "device pipeline wait timed out";
    case SYN_ERR_TIMEOUT_COUNTER: return "device wait on a grid counter timed out";
    case SYN_ERR_RENDEZVOUS: return "peer rendezvous timed out";
    case SYN_ERR_UNSUPPORTED: return "unsupported configuration";
    case SYN_ERR_TOO_LARGE: return "too many waves / ops / bytes for the fixed limits";
    default: return "unknown error";
  }
}

const char* syn_last_cuda_error(void) { return syn::g_cuda_err; }

const char* syn_version(void) { return "syncopate_b200 0.1 (sm_100a)"; }

}  // extern "C"
