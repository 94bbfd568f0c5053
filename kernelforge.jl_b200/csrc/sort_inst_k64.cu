// Onesweep and histogram kernels for kf::u64 keys (keys-only and 4-/8-byte payloads).
#include "sort_impl.cuh"

KF_SORT_INSTANTIATE(k64, kf::u64)
