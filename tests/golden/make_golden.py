"""Generates tests/golden/golden_small.npz: seeded inputs of every configuration of the path at a
small size, with the CPU oracle's outputs. The reference's own tests store no vectors for this
path (they compare with Julia Base at run time, and Julia is not available here), so these
fixtures freeze the oracle: inputs come from numpy's PCG64 with the seeds below, outputs from
oracle/kf_oracle.c, cross-checked against the numpy restatement before they are written.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import oracle as O  # noqa: E402


def main():
    rng = np.random.default_rng(0)
    n = 4099
    out = {}
    out["mr_x"] = rng.random(n, dtype=np.float32)                       # mapreduce(abs2, +, x), x ~ U[0,1)
    out["mr_abs2_sum"] = np.float64(O.c_mapreduce(O.MAP_ABS2, O.OP_ADD, out["mr_x"]))
    assert abs(out["mr_abs2_sum"] - np.sum(out["mr_x"].astype(np.float64) ** 2)) < 1e-9
    out["scan_u32_x"] = rng.integers(0, 256, n).astype(np.uint32)        # U{0..255}, wrapping add
    out["scan_u32_x"][:8] = 0xFFFFFFF0                                   # force wrap-around early
    out["scan_u32_out"] = O.c_scan(0, O.OP_ADD, out["scan_u32_x"])
    assert (out["scan_u32_out"] == np.cumsum(out["scan_u32_x"], dtype=np.uint32)).all()
    out["scan_u8_x"] = rng.integers(0, 256, n).astype(np.uint8)
    out["scan_u8_out"] = O.c_scan(0, O.OP_ADD, out["scan_u8_x"])
    out["scan_f32_x"] = rng.random(n, dtype=np.float32)
    out["scan_f32_out"] = O.c_scan(0, O.OP_ADD, out["scan_f32_x"])      # float64 left fold
    out["aff_a"] = (0.5 + 0.5 * rng.random(n)).astype(np.float32)        # a ~ U[0.5,1), b ~ U[-1,1)
    out["aff_b"] = (2.0 * rng.random(n) - 1.0).astype(np.float32)
    out["aff_oa"], out["aff_ob"] = O.c_scan_affine(out["aff_a"], out["aff_b"])
    x = rng.standard_normal(n).astype(np.float32)                        # N(0,1) with +-0 and subnormals injected
    x[::97] = 0.0
    x[1::97] = -0.0
    x[2::97] = (rng.integers(1, 1 << 23, x[2::97].size).astype(np.uint32)).view(np.float32)
    x[3::97] = (rng.integers(1, 1 << 23, x[3::97].size).astype(np.uint32) | np.uint32(1 << 31)).view(np.float32)
    out["sort_f32_x"] = x
    out["sort_f32_out"] = O.c_sort(x)
    assert (out["sort_f32_out"].view(np.uint32) == O.np_sort(x).view(np.uint32)).all()
    out["sort_u32_x"] = rng.integers(0, 1 << 32, n, dtype=np.uint64).astype(np.uint32)
    out["sort_u32_out"] = O.c_sort(out["sort_u32_x"])
    out["pairs_keys"] = rng.integers(0, 64, n).astype(np.uint32)         # heavy duplicates: stability shows
    out["pairs_perm"] = O.c_sortperm(out["pairs_keys"])                  # payload = original index (0-based)
    assert (out["pairs_perm"].astype(np.int64) == O.np_sortperm(out["pairs_keys"])).all()
    np.savez_compressed(os.path.join(HERE, "golden_small.npz"), **out)
    print("wrote golden_small.npz with", len(out), "arrays")


if __name__ == "__main__":
    main()
