// Onesweep and histogram kernels for uint32_t keys (keys-only and 4-/8-byte payloads).
#include "sort_impl.cuh"

KF_SORT_INSTANTIATE(k32, uint32_t)
