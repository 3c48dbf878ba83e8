// Drop-in for core/kernels/primitives/swiglu_mlp_primitive.h: everything lives in mlxr_kernels.h.
#pragma once
#include "mlxr_kernels.h"
