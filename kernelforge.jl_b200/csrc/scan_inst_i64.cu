// Scan kernels for element type long long (one translation unit per type keeps the build parallel).
#include "scan_launch.cuh"

KF_SCAN_INSTANTIATE(i64, long long)
