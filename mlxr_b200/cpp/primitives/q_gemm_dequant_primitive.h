// Drop-in for core/kernels/primitives/q_gemm_dequant_primitive.h: everything lives in mlxr_kernels.h.
#pragma once
#include "mlxr_kernels.h"
