// Scan kernels for element type uint8_t (one translation unit per type keeps the build parallel).
#include "scan_launch.cuh"

KF_SCAN_INSTANTIATE(u8, uint8_t)
