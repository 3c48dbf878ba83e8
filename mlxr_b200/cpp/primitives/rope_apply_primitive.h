// Drop-in for core/kernels/primitives/rope_apply_primitive.h: everything lives in mlxr_kernels.h.
#pragma once
#include "mlxr_kernels.h"
