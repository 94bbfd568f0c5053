// Scan kernels for element type int8_t (one translation unit per type keeps the build parallel).
#include "scan_launch.cuh"

KF_SCAN_INSTANTIATE(i8, int8_t)
