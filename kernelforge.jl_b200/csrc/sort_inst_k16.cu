// Onesweep and histogram kernels for 2-byte keys: two passes (keys-only and 4-/8-byte payloads).
#include "sort_impl.cuh"

KF_SORT_INSTANTIATE_INT(k16, uint16_t)
