# Backend glue, the counterpart of ext/KernelForgeCUDAExt.jl:13-53 of KernelForge.jl, rewired to the
# ccall layer: no architecture detection and no tuning files to load (the launch table is compiled
# into libkf_b200.so, single target sm_100a); `num_sms` asks the library; buffers are CuArrays and
# are freed like any other.
module KernelForgeB200CUDAExt

using CUDA
import ..KernelForgeB200: KernelBuffer, libkf

function __init__()
    CUDA.functional() || return
    v = ccall((:kf_abi_version, libkf), Cint, ())
    v == 2 || error("libkf_b200.so has ABI version $v, expected 2")
    for dev in CUDA.devices()
        cap = CUDA.capability(dev)
        cap >= v"10.0" || @warn "libkf_b200.so is built for sm_100a only; device $(CUDA.name(dev)) is $(cap)"
    end
end

num_sms() = Int(ccall((:kf_num_sms, libkf), Cint, ()))

_unsafe_free!(buf::KernelBuffer) = foreach(CUDA.unsafe_free!, buf.arrays)

# The reference's compile-only hook (src/tuning/precompile.jl:10) has nothing to do here: every
# kernel is precompiled into the shared library.
compile_kernel_only(args...; kwargs...) = nothing

end # module
