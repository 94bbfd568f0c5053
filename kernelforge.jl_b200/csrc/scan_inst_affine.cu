// Scan kernels for the non-commutative affine-composition operator on Float32 (a, b) pairs, in
// the interleaved (NTuple{2,Float32}) and the two-array layouts.
#include "scan_launch.cuh"

namespace kf {

int scan_dispatch_affine_aos(int variant, const float *src, float *dst, const ScanArgs &args, cudaStream_t s) {
    PlainAccess<Affine> acc{reinterpret_cast<const Affine *>(src), reinterpret_cast<Affine *>(dst)};
    PlainArrays<Affine> arr;
    arr.src[0] = reinterpret_cast<const char *>(src);
    arr.dst[0] = reinterpret_cast<char *>(dst);
    return scan_launch<Affine, OpAffine>(variant, acc, arr, args, s);
}

int scan_dispatch_affine_soa(int variant, const float *a_src, const float *b_src, float *a_dst, float *b_dst,
                             const ScanArgs &args, cudaStream_t s) {
    AffineSoaAccess acc{a_src, b_src, a_dst, b_dst};
    AffineSoaArrays arr;
    arr.src[0] = reinterpret_cast<const char *>(a_src);
    arr.src[1] = reinterpret_cast<const char *>(b_src);
    arr.dst[0] = reinterpret_cast<char *>(a_dst);
    arr.dst[1] = reinterpret_cast<char *>(b_dst);
    return scan_launch<Affine, OpAffine>(variant, acc, arr, args, s);
}

}  // namespace kf
