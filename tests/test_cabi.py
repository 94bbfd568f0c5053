"""CPU tests of the C-ABI boundary: the library loads, exports every symbol include/kf_b200.h
declares, answers size queries and rejects bad arguments before touching a device."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "kf_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kf_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound(kf):
    from kernelforge_jl_b200 import _cabi as C
    syms = declared_symbols()
    assert len(syms) >= 17
    raw = ctypes.CDLL(C.LIB_PATH)
    for name in syms:
        assert hasattr(raw, name), "libkf_b200.so does not export %s" % name
        assert name in C.PROTOTYPES, "%s is declared in the header but not bound in _cabi.py" % name
    assert set(C.PROTOTYPES) == set(syms)


def test_header_cites_reference_for_every_entry(kf):
    text = open(HEADER).read()
    for name in declared_symbols():
        m = re.search(r"^(?:int32_t|uint64_t|size_t|const char \*)\s*" + name + r"\(", text, flags=re.M)  # the declaration itself
        assert m, name
        i = m.start()
        comment = text[text.rfind("/*", 0, i):i]
        assert re.search(r"\.jl:\d+|no\s+counterpart|ABI version|last KF_ERR|SMs of the current", comment, flags=re.I), name


def test_version_and_error_strings(kf):
    lib = kf.lib
    assert lib.kf_abi_version() == 2
    texts = {lib.kf_error_string(i).decode() for i in range(7)}
    assert len(texts) == 7 and "ok" in texts
    assert "unknown" in lib.kf_error_string(99).decode()
    assert lib.kf_num_sms() >= 1


def test_workspace_queries(kf):
    from kernelforge_jl_b200 import _cabi as C
    lib = kf.lib
    n = 1 << 28
    assert lib.kf_mapreduce_workspace_bytes(C.F32, n, None) >= 256 + 4
    scan_b = lib.kf_scan_workspace_bytes(C.F32, 0, n, None)
    assert 256 < scan_b < (8 << 20)  # descriptors only: a few hundred KB
    assert lib.kf_scan_workspace_bytes(C.F32, 1, 1 << 26, None) > 0
    assert lib.kf_scan_workspace_bytes(C.F64, 1, 1 << 26, None) == 0  # affine pairs are Float32 only
    keys = lib.kf_sort_workspace_bytes(C.U32, 0, n, None)
    pairs = lib.kf_sort_workspace_bytes(C.U32, 4, n, None)
    assert keys >= 4 * n and pairs >= 8 * n and pairs > keys  # n-element ping-pong scratch inside
    assert lib.kf_sort_workspace_bytes(C.U16, 0, n, None) >= 2 * n  # every element type is a key type
    assert lib.kf_sort_workspace_bytes(42, 0, n, None) == 0
    assert lib.kf_sort_workspace_bytes(C.U32, 3, n, None) == 0
    bad = ctypes.pointer(C.LaunchCfg(96, 3, 0, 0))
    assert lib.kf_scan_workspace_bytes(C.F32, 0, n, bad) == 0
    assert lib.kf_mapreduce_workspace_bytes(99, n, None) == 0


def test_launch_table(kf):
    from kernelforge_jl_b200 import _cabi as C
    lib = kf.lib
    for prim, eb in ((C.PRIM_MAPREDUCE, 4), (C.PRIM_SCAN, 4), (C.PRIM_SCAN, 8), (C.PRIM_SORT_KEYS, 4), (C.PRIM_SORT_PAIRS, 8)):
        for log2n in (10, 20, 28, 32):
            cfg = C.LaunchCfg()
            assert lib.kf_launch_table_lookup(prim, eb, 1 << log2n, ctypes.byref(cfg)) == C.OK
            assert cfg.threads % 32 == 0 and cfg.threads >= 128 and cfg.items >= 1
    assert lib.kf_launch_table_lookup(17, 4, 1000, ctypes.byref(C.LaunchCfg())) == C.ERR_UNSUPPORTED
    assert lib.kf_launch_table_lookup(0, 4, 1000, None) == C.ERR_INVALID_ARG


def test_argument_errors_before_any_device_work(kf):
    """Every rejection below happens on the host: no CUDA call is made, so this runs without a GPU."""
    from kernelforge_jl_b200 import _cabi as C
    lib = kf.lib
    fake = ctypes.c_void_p(0x1000)  # never dereferenced
    assert lib.kf_mapreduce(0, 0, 0, C.F32, fake, 0, fake, fake, 1 << 20, None, None) == C.ERR_EMPTY
    assert lib.kf_mapreduce(0, 0, 0, C.F32, None, 10, fake, fake, 1 << 20, None, None) == C.ERR_INVALID_ARG
    assert lib.kf_mapreduce(7, 0, 0, C.F32, fake, 10, fake, fake, 1 << 20, None, None) == C.ERR_UNSUPPORTED
    assert lib.kf_mapreduce(0, 0, 1, C.I32, fake, 10, fake, fake, 1 << 20, None, None) == C.ERR_UNSUPPORTED  # sqrt of ints
    assert lib.kf_mapreduce(0, 0, 0, C.F32, fake, 1 << 20, fake, fake, 16, None, None) == C.ERR_WORKSPACE_TOO_SMALL
    assert lib.kf_mapreduce(0, 0, 0, C.F32, ctypes.c_void_p(0x1002), 10, fake, fake, 1 << 20, None, None) == C.ERR_INVALID_ARG
    assert lib.kf_scan(0, 0, 0, C.F32, fake, fake, 0, None, 0, fake, 0, None, None) == C.OK  # n == 0 is a no-op
    assert lib.kf_scan(0, C.OP_AFFINE, 0, C.F32, fake, fake, 10, None, 0, fake, 1 << 20, None, None) == C.ERR_UNSUPPORTED
    assert lib.kf_scan(0, 0, 0, C.F32, fake, fake, 1 << 20, None, 0, fake, 8, None, None) == C.ERR_WORKSPACE_TOO_SMALL
    assert lib.kf_scan(0, 0, 0, 42, fake, fake, 10, None, 0, fake, 1 << 20, None, None) == C.ERR_INVALID_ARG
    assert lib.kf_sort_keys(C.U32, fake, fake, 0, fake, 0, None, None) == C.OK
    assert lib.kf_sort_keys(42, fake, fake, 10, fake, 1 << 20, None, None) == C.ERR_INVALID_ARG
    assert lib.kf_sort_pairs(C.U8, fake, fake, 2, fake, fake, 10, fake, 1 << 20, None, None) == C.ERR_UNSUPPORTED  # 2-byte payload
    assert lib.kf_sort_keys(C.U32, fake, fake, 1 << 20, fake, 1024, None, None) == C.ERR_WORKSPACE_TOO_SMALL
    assert lib.kf_sort_pairs(C.U32, fake, fake, 0, fake, fake, 10, fake, 1 << 20, None, None) == C.ERR_INVALID_ARG
    assert lib.kf_sort_pairs(C.U32, fake, fake, 4, None, fake, 10, fake, 1 << 30, None, None) == C.ERR_INVALID_ARG
    assert lib.kf_check(None, None) == C.ERR_INVALID_ARG


def test_missing_library_fails_loudly(kf, tmp_path):
    from kernelforge_jl_b200 import _cabi as C
    with pytest.raises(C.KernelForgeError):
        C.load(str(tmp_path / "libkf_b200.so"))
