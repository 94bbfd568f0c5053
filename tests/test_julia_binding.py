"""CPU check that the Julia layer (kernelforge.jl_b200/julia/*.jl) still matches the C ABI.

Julia is not installed where these tests run, so the `.jl` files cannot be executed; what can drift
silently is the `ccall` signatures. Every `ccall((:kf_x, libkf), Ret, (ArgTypes...), ...)` is parsed
out of the Julia sources, its types are mapped to ctypes, and return type, arity and argument widths
are compared with the ctypes prototypes of `_cabi.py` (which test_cabi.py ties to include/kf_b200.h
and to the exported symbols). Every symbol of the header must be bound by the Julia layer.
"""
import ctypes
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
JULIA = os.path.join(ROOT, "kernelforge.jl_b200", "julia")

# Julia C types -> (kind, size in bytes). Pointers of any flavour are one kind.
JL = {"Cint": ("int", 4), "Int32": ("int", 4), "UInt32": ("int", 4), "Cuint": ("int", 4), "UInt64": ("int", 8), "Int64": ("int", 8),
      "Csize_t": ("int", ctypes.sizeof(ctypes.c_size_t)), "Cstring": ("ptr", ctypes.sizeof(ctypes.c_void_p))}


def jl_type(t):
    t = t.strip()
    if t.startswith(("CuPtr{", "Ptr{")) or t == "Cstring":
        return ("ptr", ctypes.sizeof(ctypes.c_void_p))
    return JL[t]


def c_type(t):
    if t is None:
        return None
    if t in (ctypes.c_void_p, ctypes.c_char_p) or isinstance(t, type(ctypes.POINTER(ctypes.c_int))) and hasattr(t, "contents"):
        return ("ptr", ctypes.sizeof(ctypes.c_void_p))
    return ("int", ctypes.sizeof(t))


def split_top(s):
    """Splits a comma-separated type list, leaving braces intact."""
    out, depth, cur = [], 0, ""
    for ch in s:
        if ch in "{(":
            depth += 1
        elif ch in "})":
            depth -= 1
        if ch == "," and depth == 0:
            out.append(cur)
            cur = ""
        else:
            cur += ch
    if cur.strip():
        out.append(cur)
    return [x.strip() for x in out if x.strip()]


def julia_ccalls():
    found = {}
    for path in sorted(glob.glob(os.path.join(JULIA, "**", "*.jl"), recursive=True)):
        text = open(path).read()
        for m in re.finditer(r"ccall\(\(:(kf_[a-z0-9_]+),\s*libkf\),\s*([A-Za-z0-9_{}]+),\s*\(", text):
            name, ret = m.group(1), m.group(2)
            i, depth = m.end(), 1
            while depth:  # the argument-type tuple ends at its matching parenthesis
                depth += {"(": 1, ")": -1}.get(text[i], 0)
                i += 1
            args = split_top(text[m.end():i - 1])
            found.setdefault(name, []).append((ret, args, os.path.basename(path)))
    return found


def test_every_ccall_matches_the_ctypes_prototype(kf):
    from kernelforge_jl_b200 import _cabi as C
    calls = julia_ccalls()
    assert len(calls) >= 25
    for name, sites in calls.items():
        assert name in C.PROTOTYPES, "%s is called from Julia but not declared in the C ABI" % name
        res, argtypes = C.PROTOTYPES[name]
        for ret, args, where in sites:
            assert jl_type(ret) == c_type(res), (name, where, "return type", ret)
            assert len(args) == len(argtypes), (name, where, "arity", args)
            for k, (a, c) in enumerate(zip(args, argtypes)):
                assert jl_type(a) == c_type(c), (name, where, "argument %d" % k, a)


def test_every_header_symbol_is_bound_in_julia(kf):
    from kernelforge_jl_b200 import _cabi as C
    missing = sorted(set(C.PROTOTYPES) - set(julia_ccalls()))
    assert not missing, "declared in include/kf_b200.h but not bound in julia/: %s" % missing


def test_julia_abi_version_matches(kf):
    from kernelforge_jl_b200 import _cabi as C
    text = open(os.path.join(JULIA, "ext", "KernelForgeB200CUDAExt.jl")).read()
    assert "v == %d ||" % C.ABI_VERSION in text
