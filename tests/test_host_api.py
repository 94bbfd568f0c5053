"""CPU tests of the host layer that mirrors the Julia API: closure -> enum mapping, argument
checks and error behaviour. Nothing here computes: tensors on the CPU are rejected (there is no CPU
path), exactly like a non-device array would be in the reference."""
import math
import operator

import pytest
import torch


def test_closure_mapping(kf):
    from kernelforge_jl_b200 import _cabi as C, ops
    assert ops.map_code(kf.identity) == C.MAP_IDENTITY and ops.map_code(kf.abs2) == C.MAP_ABS2
    assert ops.map_code(abs) == C.MAP_ABS and ops.map_code("abs2") == C.MAP_ABS2
    assert ops.op_code(operator.add) == C.OP_ADD and ops.op_code("+") == C.OP_ADD
    assert ops.op_code(min) == C.OP_MIN and ops.op_code(max) == C.OP_MAX and ops.op_code(operator.mul) == C.OP_MUL
    assert ops.op_code(operator.and_) == C.OP_AND and ops.op_code(operator.or_) == C.OP_OR
    assert ops.op_code(operator.xor) == C.OP_XOR and ops.op_code("⊻") == C.OP_XOR
    assert ops.op_code(kf.AffineCompose()) == C.OP_AFFINE and kf.AffineCompose() is kf.AffineCompose()
    assert ops.post_code(math.sqrt) == C.POST_SQRT and ops.post_code(kf.identity) == C.POST_IDENTITY
    for bad in (lambda x: x + 1, print, 3):
        with pytest.raises(kf.ArgumentError):
            ops.map_code(bad)
        with pytest.raises(kf.ArgumentError):
            ops.op_code(bad)
    # the operator itself, on the host: (a1,b1) o (a2,b2) = (a1*a2, a2*b1 + b2)
    assert kf.AffineCompose()((2.0, 1.0), (0.5, -1.0)) == (1.0, -0.5)


def test_no_cpu_path(kf):
    x = torch.ones(16)
    for call in (lambda: kf.mapreduce(kf.identity, "+", x), lambda: kf.scan("+", x), lambda: kf.sort(x),
                 lambda: kf.get_allocation(kf.Scan1D, kf.identity, "+", x)):
        with pytest.raises(kf.ArgumentError):
            call()


def test_argument_checks_that_need_no_device(kf):
    x = torch.ones(16)
    with pytest.raises(kf.ArgumentError):
        kf.mapreduce(kf.identity, "+", x, dims=1)
    with pytest.raises(kf.ArgumentError):
        kf.mapreduce(kf.identity, "+", (x, x))
    with pytest.raises(kf.ArgumentError):
        kf.sort(x, rev=True)
    with pytest.raises(kf.ArgumentError):
        kf.sort(x, by=lambda v: -v)
    with pytest.raises(kf.ArgumentError):
        kf.scan("+", x, g=math.sqrt)
    with pytest.raises(TypeError):
        kf.scan_("+", x)
    with pytest.raises(kf.KernelForgeError):
        kf.get_allocation(object, x)


def test_names_follow_the_reference(kf):
    for name in ("mapreduce", "mapreduce_", "mapreduce1d", "mapreduce1d_", "scan", "scan_", "sort", "sort_",
                 "sortperm", "get_allocation", "KernelBuffer", "MapReduce1D", "Scan1D", "Sort1D", "AffineCompose"):
        assert hasattr(kf, name)
