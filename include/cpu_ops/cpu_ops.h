// Umbrella header of the quantized-GEMM surface (the reference umbrella also pulls in
// its float GEMMs and ops, which stay with the CPU library).
#pragma once
#include "cpu_ops/b200/device_gemm.h"
