// Scan kernels for element type uint32_t (one translation unit per type keeps the build parallel).
#include "scan_launch.cuh"

KF_SCAN_INSTANTIATE(u32, uint32_t)
