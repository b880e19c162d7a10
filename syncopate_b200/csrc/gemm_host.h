// Internal interface between the GEMM host code and the fused-operator entry points.
#pragma once
#include "gemm_sm100.cuh"
#include "host_util.h"

namespace syn {

// `multiple`: the tile width must be a multiple of this (32; 64 when tiles leave through TMA stores).
int pick_block_n(const syn_schedule* s, int M, int N, int num_sms, int multiple = 32, bool* pair_out = nullptr);
int validate_schedule_2d(const syn_schedule* s, int M, int N, int bn);
// Checks `a`, encodes the tensor maps and fills the wave table (all routes -1).
int gemm_fill_common(GemmParams* p, const syn_gemm_args* a, const syn_schedule* sched, int bn);
int gemm_resolve_grid_and_bn(const syn_gemm_args* a, const syn_schedule* sched, int* grid, int* bn, int multiple = 32,
                             bool* pair_out = nullptr);
int gemm_launch(const GemmParams& p, int bn, bool fused, int grid, cudaStream_t stream);
// CTA-pair form (gemm2_kernel): usable when pair_eligible() says so for the filled parameters.
bool pair_eligible(const GemmParams& p, int bn, int grid);
int gemm_launch_pair(const GemmParams& p, const syn_gemm_args* a, int bn, int grid, bool fused, cudaStream_t stream);

}  // namespace syn
