// Scan kernels for element type float (one translation unit per type keeps the build parallel).
#include "scan_launch.cuh"

KF_SCAN_INSTANTIATE(f32, float)
