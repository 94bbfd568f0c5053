// Scan kernels for element type int16_t (one translation unit per type keeps the build parallel).
#include "scan_launch.cuh"

KF_SCAN_INSTANTIATE(i16, int16_t)
