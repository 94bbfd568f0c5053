// Scan kernels for element type int32_t (one translation unit per type keeps the build parallel).
#include "scan_launch.cuh"

KF_SCAN_INSTANTIATE(i32, int32_t)
