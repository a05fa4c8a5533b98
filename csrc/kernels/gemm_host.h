// Host-side helpers of the GEMM launchers, shared between gemm_tcgen05.cu and the
// fused collective kernels in csrc/comm/.
#pragma once
#include "../../include/cogito_kernels.h"
#include "gemm_tc_body.cuh"
#include "host_common.h"

namespace cgk {

// Tensor maps of both operands for a tile width BN (box shapes depend on the
// operand's storage order).
int make_gemm_tmaps(const cgk_gemm_args& a, int BN, CUtensorMap* tmA, CUtensorMap* tmB);
// Tensor maps of the bf16 output and the pre-activation output for the epilogue's bulk stores;
// *ok = 0 (and cleared maps) when the output's layout or the epilogue's terms rule them out.
// tmIn / *in_kind: the one epilogue input fetched by bulk loads (1 = activation-derivative operand,
// 2 = residual, 0 = none).
int make_gemm_out_tmaps(const cgk_gemm_args& a, CUtensorMap* tmC, CUtensorMap* tmAux, CUtensorMap* tmIn, int* ok,
                        int* in_kind);
// Copies the argument struct into the device-side parameter block (hooks cleared).
int fill_gemm_dev(const cgk_gemm_args& a, GemmDev* g);
// True when both operands satisfy TMA's alignment rules.
bool gemm_tma_ok(const cgk_gemm_args& a);
// Checks the arguments of the rotary epilogue (0 or CGK_E_ARG).
int gemm_rope_ok(const cgk_gemm_args& a);
// Tile width (256 / 128 / 64) for a problem run by `ctas` persistent CTAs.
int pick_bn(const cgk_gemm_args& a, int ctas);

}  // namespace cgk
