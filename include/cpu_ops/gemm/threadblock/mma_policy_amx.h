// Drop-in path of the reference header of the same name.  The CPU library's policy types
// choose a packing and micro-kernel; on the GPU they are tag types that the operators
// accept and ignore (cpu_ops/b200/device_gemm.h).
#pragma once
#include "cpu_ops/b200/device_gemm.h"
