// Scan kernels for element type kf::u64 (one translation unit per type keeps the build parallel).
#include "scan_launch.cuh"

KF_SCAN_INSTANTIATE(u64, kf::u64)
