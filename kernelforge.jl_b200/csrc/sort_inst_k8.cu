// Onesweep and histogram kernels for 1-byte keys: a single pass (keys-only and 4-/8-byte payloads).
#include "sort_impl.cuh"

KF_SORT_INSTANTIATE_INT(k8, uint8_t)
