// Host-side helpers shared by the C-ABI translation units: error plumbing, driver entry points
// (resolved at run time so that the library links without libcuda), tensor-map encoding.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/syncopate_b200.h"

namespace syn {

void set_cuda_error(const char* what, const char* detail);
int device_sm_count(int* out);

#define SYN_CUDA_TRY(expr)                                  \
  do {                                                      \
    cudaError_t _e = (expr);                                \
    if (_e != cudaSuccess) {                                \
      ::syn::set_cuda_error(#expr, cudaGetErrorString(_e)); \
      return SYN_ERR_CUDA;                                  \
    }                                                       \
  } while (0)

// 2-D row-major 16-bit tensor [rows, cols] with leading dimension ld (elements); box = [box_rows, 64]
// elements with the 128-byte swizzle the UMMA shared-memory descriptors expect.
int encode_tmap_2d_sw128(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                         uint32_t box_rows, uint32_t box_cols);
// Same tensor without swizzle (rows of box_cols elements laid out back to back in shared memory).
int encode_tmap_2d_plain(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                         uint32_t box_rows, uint32_t box_cols);
// 3-D variant: [d2, rows, cols] with strides (stride2, ld, 1) in elements.
int encode_tmap_3d_sw128(CUtensorMap* out, const void* base, uint64_t d2, uint64_t rows, uint64_t cols,
                         uint64_t stride2, uint64_t ld, uint32_t box_rows, uint32_t box_cols);

// 4-D 16-bit tensor [d3, d2, rows, cols] with element strides (s3, s2, ld, 1); box = [1, 1, box_rows, box_cols].
int encode_tmap_4d_sw128(CUtensorMap* out, const void* base, uint64_t d3, uint64_t d2, uint64_t rows, uint64_t cols,
                         uint64_t s3, uint64_t s2, uint64_t ld, uint32_t box_rows, uint32_t box_cols);

// Kernel loading, one function per translation unit (see syn_preload): each loads the code of its
// kernels on the current device.
int preload_symm_kernels();
int preload_copy_kernels();
int preload_fused_kernels();
int preload_gemm_kernels();
int preload_attn_kernels();

// Maps a device status code (ptx.cuh) to the negative C-ABI code.
int status_to_err(int dev_code);

}  // namespace syn
