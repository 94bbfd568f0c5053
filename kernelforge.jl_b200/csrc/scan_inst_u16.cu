// Scan kernels for element type uint16_t (one translation unit per type keeps the build parallel).
#include "scan_launch.cuh"

KF_SCAN_INSTANTIATE(u16, uint16_t)
