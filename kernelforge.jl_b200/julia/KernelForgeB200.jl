# KernelForgeB200.jl — Julia host layer over libkf_b200.so (C ABI in include/kf_b200.h).
#
# Drop-in for the memory-bound primitive core of KernelForge.jl: the same qualified names and
# call signatures (`KernelForgeB200.mapreduce`, `scan`, `scan!`, `sort`, `sort!`, `get_allocation`,
# `KernelBuffer`, `@allocate`), with the kernels replaced by `ccall`s into hand-written sm_100a
# CUDA. Replaces src/mapreduce/mapreduce.jl:51-62,151-162, src/mapreduce/1D/mapreduce1d.jl:177-346,
# src/scan/scan.jl:218-284,414-479, src/sort/sort1d.jl:307-502,780-874,1006-1090 and
# src/allocations.jl:16-49 of KernelForge.jl v0.2.0.
#
# The operator set is fixed: identity/abs2/abs as `f` (over tuples of arrays: `*`, `SqDiff()`,
# `WeightedSq()`), + * min max & | xor as `op`, identity/sqrt as `g`, plus `AffineCompose()` for scans.
# Any other closure, `by`, `lt`, `rev`, a custom `uint_map` or `dims` raises `ArgumentError`; there is
# no fallback path of any kind. Also here: argmax / argmin / findfirst / findlast / vcopy! / setvalue!
# (src/search/highlevel.jl:1-52, src/copy/copy.jl:24-56), with Julia's 1-based indices.
#
# This file cannot be executed where it was written (no Julia toolchain); its executable twin is the
# Python package next to it, which binds the same C entry points with the same argument order.
module KernelForgeB200

using CUDA

const libkf = get(ENV, "KF_B200_LIB", joinpath(@__DIR__, "..", "libkf_b200.so"))

# ---- enums (must match include/kf_b200.h) -----------------------------------------------------
const KF_OK = Cint(0)
const DTYPES = Dict{DataType,Cint}(UInt8 => 0, Int8 => 1, UInt16 => 2, Int16 => 3, UInt32 => 4, Int32 => 5,
                                   UInt64 => 6, Int64 => 7, Float32 => 8, Float64 => 9, Bool => 0)

"Composition of affine maps x -> a*x + b: (a1,b1) ∘ (a2,b2) = (a1*a2, a2*b1 + b2). Scan only."
struct AffineCompose <: Function end
(::AffineCompose)(l::NTuple{2,Float32}, r::NTuple{2,Float32}) = (l[1] * r[1], r[1] * l[2] + r[2])

map_code(::typeof(identity)) = Cint(0)
map_code(::typeof(abs2)) = Cint(1)
map_code(::typeof(abs)) = Cint(2)
map_code(f) = throw(ArgumentError("unsupported map function $f: this library implements identity, abs2 and abs only"))
op_code(::typeof(+)) = Cint(0)
op_code(::typeof(*)) = Cint(1)
op_code(::typeof(min)) = Cint(2)
op_code(::typeof(max)) = Cint(3)
op_code(::typeof(&)) = Cint(4)
op_code(::typeof(|)) = Cint(5)
op_code(::typeof(xor)) = Cint(6)
op_code(::AffineCompose) = Cint(7)
op_code(op) = throw(ArgumentError("unsupported operator $op: this library implements + * min max & | xor and AffineCompose()"))
post_code(::typeof(identity)) = Cint(0)
post_code(::typeof(sqrt)) = Cint(1)
post_code(g) = throw(ArgumentError("unsupported post-map $g: this library implements identity and sqrt only"))
dtype_code(::Type{T}) where {T} = get(DTYPES, T) do
    throw(ArgumentError("unsupported element type $T"))
end

struct LaunchCfg
    threads::Cint
    items::Cint
    blocks::Cint
    reserved::Cint
end
make_cfg(workgroup, Nitem, blocks) =
    (workgroup === nothing && Nitem === nothing && blocks === nothing) ? nothing :
    Ref(LaunchCfg(something(workgroup, 0), something(Nitem, 0), something(blocks, 0), 0))
cfg_ptr(::Nothing) = Ptr{LaunchCfg}(C_NULL)
cfg_ptr(r::Ref{LaunchCfg}) = Base.unsafe_convert(Ptr{LaunchCfg}, r)

function check(code::Cint, what)
    code == KF_OK && return nothing
    msg = unsafe_string(ccall((:kf_error_string, libkf), Cstring, (Cint,), code))
    code in (1, 2, 6, 7) ? throw(ArgumentError("$what: $msg")) : error("$what: $msg")
end

stream_handle() = reinterpret(Ptr{Cvoid}, CUDA.stream().handle)

# ---- workspaces (src/allocations.jl:16-49) ------------------------------------------------------
abstract type ForgeAlgorithm end
struct MapReduce1D <: ForgeAlgorithm end
struct Scan1D <: ForgeAlgorithm end
struct Sort1D <: ForgeAlgorithm end

"Pre-allocated workspace; `arrays.workspace` is the byte buffer handed to the C library."
struct KernelBuffer{Arrays<:NamedTuple}
    arrays::Arrays
end
_alloc(nbytes) = nbytes == 0 ? throw(ArgumentError("no workspace layout for these arguments")) :
                 KernelBuffer((; workspace=CUDA.zeros(UInt8, nbytes)))

mapreduce_bytes(::Type{T}, n, cfg) where {T} =
    ccall((:kf_mapreduce_workspace_bytes, libkf), Csize_t, (Cint, UInt64, Ptr{LaunchCfg}), dtype_code(T), n, cfg_ptr(cfg))
scan_bytes(::Type{T}, pair, n, cfg) where {T} =
    ccall((:kf_scan_workspace_bytes, libkf), Csize_t, (Cint, Cint, UInt64, Ptr{LaunchCfg}), dtype_code(T), pair, n, cfg_ptr(cfg))
sort_bytes(::Type{K}, valbytes, n, cfg) where {K} =
    ccall((:kf_sort_workspace_bytes, libkf), Csize_t, (Cint, Cint, UInt64, Ptr{LaunchCfg}), dtype_code(K), valbytes, n, cfg_ptr(cfg))

function get_allocation(::Type{MapReduce1D}, f, op, src::CuArray{T}, workgroup=nothing, blocks=nothing, arch=nothing) where {T}
    _alloc(mapreduce_bytes(T, length(src), make_cfg(workgroup, nothing, blocks)))
end
function get_allocation(::Type{Scan1D}, f, op, src::CuArray{T}, workgroup=nothing, blocks=nothing, arch=nothing) where {T}
    _alloc(scan_bytes(T, 0, length(src), make_cfg(workgroup, nothing, nothing)))
end
function get_allocation(::Type{Scan1D}, f, op::AffineCompose, src, workgroup=nothing, blocks=nothing, arch=nothing)
    n = src isa Tuple ? length(src[1]) : length(src)
    _alloc(scan_bytes(Float32, 1, n, make_cfg(workgroup, nothing, nothing)))
end
function get_allocation(::Type{Sort1D}, src::CuArray{T}; Nitem=nothing, Nchunks=nothing, workgroup=nothing, arch=nothing,
                        by=identity, uint_map=nothing, keys=nothing) where {T}
    cfg = make_cfg(workgroup, Nitem, nothing)
    keys === nothing ? _alloc(sort_bytes(T, 0, length(src), cfg)) : _alloc(sort_bytes(eltype(keys), sizeof(T), length(src), cfg))
end

const KERNEL_TAGS = Dict(:mapreduce1d => MapReduce1D, :scan1d => Scan1D, :sort1d => Sort1D)
macro allocate(expr)
    @assert expr.head == :call "expected a function call"
    tag = get(KERNEL_TAGS, expr.args[1], nothing)
    tag === nothing && error("Unknown ForgeAlgorithm: $(expr.args[1])")
    rest = expr.args[2:end]
    args = Any[GlobalRef(@__MODULE__, :get_allocation)]
    if !isempty(rest) && rest[1] isa Expr && rest[1].head == :parameters
        push!(args, rest[1]); push!(args, tag); append!(args, rest[2:end])
    else
        push!(args, tag); append!(args, rest)
    end
    esc(Expr(:call, args...))
end

function _resolve_tmp(tmp, need)
    need == 0 && throw(ArgumentError("unsupported element type or launch override for this primitive"))
    tmp === nothing && return _alloc(need)
    length(tmp.arrays.workspace) < need && error("tmp holds $(length(tmp.arrays.workspace)) bytes but this call needs $need")
    tmp
end

# ---- mapreduce (src/mapreduce/mapreduce.jl:51-62,151-162) -----------------------------------------
function mapreduce!(f, op, dst::CuArray{T}, src::CuArray{T}; dims=nothing, g=identity, tmp=nothing, Nitem=nothing,
                    workgroup=nothing, blocks=nothing, arch=nothing) where {T}
    (dims === nothing || dims === Colon()) || throw(ArgumentError("only full reductions (dims=nothing) are implemented"))
    op isa AffineCompose && throw(ArgumentError("AffineCompose is not commutative: use scan"))
    n = length(src)
    n == 0 && throw(ArgumentError("reducing over an empty collection is not allowed"))
    cfg = make_cfg(workgroup, Nitem, blocks)
    buf = _resolve_tmp(tmp, mapreduce_bytes(T, n, cfg))
    ws = buf.arrays.workspace
    GC.@preserve cfg begin
        check(ccall((:kf_mapreduce, libkf), Cint,
                    (Cint, Cint, Cint, Cint, CuPtr{Cvoid}, UInt64, CuPtr{Cvoid}, CuPtr{Cvoid}, Csize_t, Ptr{LaunchCfg}, Ptr{Cvoid}),
                    map_code(f), op_code(op), post_code(g), dtype_code(T), pointer(src), n, pointer(dst), pointer(ws), length(ws),
                    cfg_ptr(cfg), stream_handle()), "mapreduce!")
    end
    dst
end
function mapreduce(f, op, src::CuArray{T}; g=identity, to_cpu::Bool=true, kwargs...) where {T}
    dst = CUDA.zeros(T, 1)
    mapreduce!(f, op, dst, src; g, kwargs...)
    to_cpu ? Array(dst)[1] : dst   # the only host<->device crossing, as in mapreduce1d.jl:203
end

# Tuple form mapreduce(f, op, (x, y, ...)) (src/mapreduce/1D/mapreduce1d.jl:186-204): f is one of `*`
# (product of 2 to 4 arrays; the dot product for two), SqDiff() ((x - y)^2) or WeightedSq() (w * x^2).
"(x, y) -> (x - y)^2 over a pair of arrays"
struct SqDiff <: Function end
(::SqDiff)(x, y) = (x - y)^2
"(w, x) -> w * x^2 over a pair of arrays"
struct WeightedSq <: Function end
(::WeightedSq)(w, x) = w * x * x
mapn_code(::typeof(*)) = Cint(0)
mapn_code(::SqDiff) = Cint(1)
mapn_code(::WeightedSq) = Cint(2)
mapn_code(f) = throw(ArgumentError("unsupported map over a tuple of arrays $f: this library implements *, SqDiff() and WeightedSq()"))

function mapreduce!(f, op, dst::CuArray{T}, srcs::NTuple{N,CuArray{T}}; dims=nothing, g=identity, tmp=nothing, Nitem=nothing,
                    workgroup=nothing, blocks=nothing, arch=nothing) where {T,N}
    N == 1 && return mapreduce!(f, op, dst, srcs[1]; dims, g, tmp, Nitem, workgroup, blocks, arch)
    (dims === nothing || dims === Colon()) || throw(ArgumentError("only full reductions (dims=nothing) are implemented"))
    2 <= N <= 4 || throw(ArgumentError("the tuple form takes 2 to 4 arrays"))
    n = length(srcs[1])
    all(x -> length(x) == n, srcs) || throw(ArgumentError("the arrays of the tuple form must have equal lengths"))
    n == 0 && throw(ArgumentError("reducing over an empty collection is not allowed"))
    cfg = make_cfg(workgroup, Nitem, blocks)
    buf = _resolve_tmp(tmp, mapreduce_bytes(T, n, cfg))
    ws = buf.arrays.workspace
    ptrs = CuPtr{Cvoid}[pointer(x) for x in srcs]   # host array of device pointers
    GC.@preserve cfg ptrs begin
        check(ccall((:kf_mapreduce_multi, libkf), Cint,
                    (Cint, Cint, Cint, Cint, Ptr{CuPtr{Cvoid}}, Cint, UInt64, CuPtr{Cvoid}, CuPtr{Cvoid}, Csize_t, Ptr{LaunchCfg}, Ptr{Cvoid}),
                    mapn_code(f), op_code(op), post_code(g), dtype_code(T), ptrs, N, n, pointer(dst), pointer(ws), length(ws),
                    cfg_ptr(cfg), stream_handle()), "mapreduce!")
    end
    dst
end
function mapreduce(f, op, srcs::NTuple{N,CuArray{T}}; g=identity, to_cpu::Bool=true, kwargs...) where {T,N}
    dst = CUDA.zeros(T, 1)
    mapreduce!(f, op, dst, srcs; g, kwargs...)
    to_cpu ? Array(dst)[1] : dst
end
const mapreduce1d = mapreduce
const mapreduce1d! = mapreduce!

# ---- scan (src/scan/scan.jl:218-284) ---------------------------------------------------------------
scan!(op, dst, src; kwargs...) = scan!(identity, op, dst, src; kwargs...)
function scan!(f, op, dst::CuArray{T}, src::CuArray{T}; g=identity, tmp=nothing, Nitem=nothing, workgroup=nothing,
               family=nothing, arch=nothing, init=nothing) where {T}
    # g is applied to every output element (src/scan/scan_kernel.jl:463,470,474); `init` is a device
    # array whose elements are folded left to right and seed the scan (one element, or the totals of
    # the shards before this one in a sharded scan)
    if _quat_component(T) !== nothing  # Quaternion{Float32|Float64}: `*` is the Hamilton product
        (op === (*) && f === identity && g === identity) ||
            throw(ArgumentError("quaternion arrays support scan!(*, dst, src) with f = g = identity only"))
        return scan_quaternion!(dst, src; tmp=tmp, Nitem=Nitem, workgroup=workgroup, init=init)
    end
    n = length(src)
    n == 0 && return dst
    length(dst) == n || throw(ArgumentError("dst and src must have equal lengths"))
    cfg = make_cfg(workgroup, Nitem, nothing)
    buf = _resolve_tmp(tmp, scan_bytes(T, 0, n, cfg))
    ws = buf.arrays.workspace
    GC.@preserve cfg begin
        check(ccall((:kf_scan, libkf), Cint,
                    (Cint, Cint, Cint, Cint, CuPtr{Cvoid}, CuPtr{Cvoid}, UInt64, CuPtr{Cvoid}, UInt32, CuPtr{Cvoid}, Csize_t,
                     Ptr{LaunchCfg}, Ptr{Cvoid}),
                    map_code(f), op_code(op), post_code(g), dtype_code(T), pointer(src), pointer(dst), n,
                    init === nothing ? CU_NULL : pointer(init), init === nothing ? 0 : length(init),
                    pointer(ws), length(ws), cfg_ptr(cfg), stream_handle()), "scan!")
    end
    dst
end
# Affine pairs stored as two Float32 arrays: scan!(AffineCompose(), (a_dst, b_dst), (a_src, b_src))
function scan!(f, op::AffineCompose, dst::NTuple{2,CuArray{Float32}}, src::NTuple{2,CuArray{Float32}}; tmp=nothing, Nitem=nothing,
               workgroup=nothing, init=nothing, kwargs...)
    f === identity || throw(ArgumentError("AffineCompose supports f=identity only"))
    n = length(src[1])
    n == 0 && return dst
    cfg = make_cfg(workgroup, Nitem, nothing)
    buf = _resolve_tmp(tmp, scan_bytes(Float32, 1, n, cfg))
    ws = buf.arrays.workspace
    GC.@preserve cfg begin
        check(ccall((:kf_scan_affine_soa, libkf), Cint,
                    (CuPtr{Cfloat}, CuPtr{Cfloat}, CuPtr{Cfloat}, CuPtr{Cfloat}, UInt64, CuPtr{Cfloat}, UInt32, CuPtr{Cvoid}, Csize_t,
                     Ptr{LaunchCfg}, Ptr{Cvoid}),
                    pointer(src[1]), pointer(src[2]), pointer(dst[1]), pointer(dst[2]), n,
                    init === nothing ? CU_NULL : pointer(init), init === nothing ? 0 : length(init) ÷ 2,
                    pointer(ws), length(ws), cfg_ptr(cfg), stream_handle()), "scan!")
    end
    dst
end
# The reference's own form: a vector of NTuple{2,Float32} on the split-descriptor kernel (scan_kernel.jl:94-299)
function scan!(f, op::AffineCompose, dst::CuArray{NTuple{2,Float32}}, src::CuArray{NTuple{2,Float32}}; tmp=nothing,
               Nitem=nothing, workgroup=nothing, init=nothing, kwargs...)
    n = length(src)
    n == 0 && return dst
    cfg = make_cfg(workgroup, Nitem, nothing)
    buf = _resolve_tmp(tmp, scan_bytes(Float32, 1, n, cfg))
    ws = buf.arrays.workspace
    GC.@preserve cfg begin
        check(ccall((:kf_scan_affine_aos, libkf), Cint,
                    (CuPtr{Cfloat}, CuPtr{Cfloat}, UInt64, CuPtr{Cfloat}, UInt32, CuPtr{Cvoid}, Csize_t, Ptr{LaunchCfg}, Ptr{Cvoid}),
                    pointer(src), pointer(dst), n, init === nothing ? CU_NULL : pointer(init),
                    init === nothing ? 0 : length(init) ÷ 2, pointer(ws), length(ws), cfg_ptr(cfg), stream_handle()), "scan!")
    end
    dst
end
# Quaternions (Quaternions.jl's Quaternion{Float32|Float64}: four components s, v1, v2, v3) under `*`, the
# reference's non-commutative scan case (test/tests/scan/scan_test.jl:22-33). Any isbits struct named
# Quaternion with four equal Float32 or Float64 fields is accepted, so Quaternions.jl is not a dependency.
function _quat_component(::Type{Q}) where {Q}
    (isbitstype(Q) && nameof(Q) === :Quaternion && fieldcount(Q) == 4) || return nothing
    C = fieldtype(Q, 1)
    (C === Float32 || C === Float64) && all(i -> fieldtype(Q, i) === C, 2:4) ? C : nothing
end
function get_allocation(::Type{Scan1D}, f, op::typeof(*), src::CuArray{Q}, workgroup=nothing, blocks=nothing, arch=nothing) where {Q}
    C = _quat_component(Q)
    C === nothing && return _alloc(scan_bytes(Q, 0, length(src), make_cfg(workgroup, nothing, nothing)))
    _alloc(ccall((:kf_scan_quaternion_workspace_bytes, libkf), Csize_t, (Cint, UInt64), dtype_code(C), length(src)))
end
function scan_quaternion!(dst::CuArray{Q}, src::CuArray{Q}; tmp=nothing, Nitem=nothing, workgroup=nothing, init=nothing) where {Q}
    C = _quat_component(Q)
    C === nothing && throw(ArgumentError("scan_quaternion!: element type $Q is not a Quaternion{Float32|Float64}"))
    n = length(src)
    n == 0 && return dst
    cfg = make_cfg(workgroup, Nitem, nothing)
    need = ccall((:kf_scan_quaternion_workspace_bytes, libkf), Csize_t, (Cint, UInt64), dtype_code(C), n)
    buf = _resolve_tmp(tmp, need)
    ws = buf.arrays.workspace
    GC.@preserve cfg begin
        check(ccall((:kf_scan_quaternion, libkf), Cint,
                    (Cint, CuPtr{Cvoid}, CuPtr{Cvoid}, UInt64, CuPtr{Cvoid}, UInt32, CuPtr{Cvoid}, Csize_t, Ptr{LaunchCfg}, Ptr{Cvoid}),
                    dtype_code(C), pointer(src), pointer(dst), n, init === nothing ? CU_NULL : pointer(init),
                    init === nothing ? 0 : length(init), pointer(ws), length(ws), cfg_ptr(cfg), stream_handle()), "scan!")
    end
    dst
end
scan(op, src; kwargs...) = scan(identity, op, src; kwargs...)
scan(f, op, src::CuArray; kwargs...) = scan!(f, op, similar(src), src; kwargs...)
scan(f, op, src::Tuple; kwargs...) = scan!(f, op, map(similar, src), src; kwargs...)

# ---- sort (src/sort/sort1d.jl:307-502) ---------------------------------------------------------------
function _reject(by, uint_map, lt, rev, algorithm)
    by === identity || throw(ArgumentError("sort: `by` other than identity is not supported"))
    uint_map === nothing || throw(ArgumentError("sort: a custom `uint_map` is not supported"))
    (lt === nothing && !rev) || throw(ArgumentError("sort: `lt` / `rev` need a comparison sort, which this library does not have"))
    algorithm in (nothing, :radix, :onesweep) || throw(ArgumentError("sort: only the radix onesweep algorithm is implemented"))
end
sort!(src::CuArray; kwargs...) = sort!(src, src; kwargs...)
function sort!(dst::CuArray{T}, src::CuArray{T}; keys=nothing, keys_dst=nothing, by=identity, uint_map=nothing, lt=nothing,
               rev::Bool=false, algorithm=nothing, tmp=nothing, Nitem=nothing, Nchunks=nothing, workgroup=nothing,
               arch=nothing, family=nothing, rr=nothing) where {T}
    _reject(by, uint_map, lt, rev, algorithm)
    n = length(src)
    length(dst) == n || throw(ArgumentError("dst and src must have the same length"))
    cfg = make_cfg(workgroup, Nitem, nothing)
    if keys === nothing
        n == 0 && return dst
        buf = _resolve_tmp(tmp, sort_bytes(T, 0, n, cfg))
        ws = buf.arrays.workspace
        GC.@preserve cfg begin
            check(ccall((:kf_sort_keys, libkf), Cint,
                        (Cint, CuPtr{Cvoid}, CuPtr{Cvoid}, UInt64, CuPtr{Cvoid}, Csize_t, Ptr{LaunchCfg}, Ptr{Cvoid}),
                        dtype_code(T), pointer(src), pointer(dst), n, pointer(ws), length(ws), cfg_ptr(cfg), stream_handle()), "sort!")
        end
        return dst
    end
    length(keys) == n || error("sort!: `keys` must have the same length as `src`")
    sizeof(T) in (4, 8) || throw(ArgumentError("sort: payload elements must be 4 or 8 bytes wide"))
    kd = keys_dst === nothing ? (dst === src ? keys : similar(keys)) : keys_dst
    n == 0 && return (dst, kd)
    buf = _resolve_tmp(tmp, sort_bytes(eltype(keys), sizeof(T), n, cfg))
    ws = buf.arrays.workspace
    GC.@preserve cfg begin
        check(ccall((:kf_sort_pairs, libkf), Cint,
                    (Cint, CuPtr{Cvoid}, CuPtr{Cvoid}, Cint, CuPtr{Cvoid}, CuPtr{Cvoid}, UInt64, CuPtr{Cvoid}, Csize_t,
                     Ptr{LaunchCfg}, Ptr{Cvoid}),
                    dtype_code(eltype(keys)), pointer(keys), pointer(kd), sizeof(T), pointer(src), pointer(dst), n, pointer(ws),
                    length(ws), cfg_ptr(cfg), stream_handle()), "sort!")
    end
    (dst, kd)
end
sort(src::CuArray; kwargs...) = sort!(similar(src), src; kwargs...)

"Stable permutation that sorts `keys` (1-based, like src/sort/sortperm.jl:162-214): iota + key-value sort."
function sortperm(keys::CuArray; kwargs...)
    n = length(keys)
    idx = CuArray{n >= 2^31 ? Int64 : Int32}(undef, n)
    n == 0 && return idx
    check(ccall((:kf_iota, libkf), Cint, (Cint, CuPtr{Cvoid}, UInt64, UInt64, Ptr{Cvoid}),
                dtype_code(eltype(idx)), pointer(idx), n, 1, stream_handle()), "sortperm")
    first(sort!(similar(idx), idx; keys, keys_dst=similar(keys), kwargs...))
end

# ---- search, copy, fill (src/search/highlevel.jl:1-52, src/copy/copy.jl:24-56) ------------------------
argmax_bytes(::Type{T}, n) where {T} =
    ccall((:kf_argmax_workspace_bytes, libkf), Csize_t, (Cint, UInt64), dtype_code(T), n)

"(value, index) of the first extremal f(src[i]) under `rel` (`>` or `<`); ties go to the smallest index. 1-based."
function argmax1d(f, rel, src::CuArray{T}; tmp=nothing) where {T}
    greater = rel === (>) ? Cint(1) : rel === (<) ? Cint(0) : throw(ArgumentError("unsupported relation $rel: argmax takes > or <"))
    n = length(src)
    n == 0 && throw(ArgumentError("argmax over an empty collection is not allowed"))
    ws = tmp === nothing ? CUDA.zeros(UInt8, argmax_bytes(T, n)) : tmp
    val = CuArray{T}(undef, 1)
    idx = CuArray{UInt64}(undef, 1)
    check(ccall((:kf_argmax, libkf), Cint,
                (Cint, Cint, Cint, CuPtr{Cvoid}, UInt64, CuPtr{Cvoid}, CuPtr{UInt64}, CuPtr{Cvoid}, Csize_t, Ptr{Cvoid}),
                map_code(f), greater, dtype_code(T), pointer(src), n, pointer(val), pointer(idx), pointer(ws), length(ws),
                stream_handle()), "argmax")
    (Array(val)[1], Int(Array(idx)[1]) + 1)
end
argmax(src::CuArray) = argmax1d(identity, >, src)[2]
argmax(rel, src::CuArray) = argmax1d(identity, rel, src)[2]
argmin(src::CuArray) = argmax1d(identity, <, src)[2]

# Predicates are Base's partially applied comparisons: >(v), <(v), >=(v), <=(v), ==(v), !=(v).
pred_code(p::Base.Fix2{typeof(>)}) = (Cint(0), p.x)
pred_code(p::Base.Fix2{typeof(<)}) = (Cint(1), p.x)
pred_code(p::Base.Fix2{typeof(>=)}) = (Cint(2), p.x)
pred_code(p::Base.Fix2{typeof(<=)}) = (Cint(3), p.x)
pred_code(p::Base.Fix2{typeof(==)}) = (Cint(4), p.x)
pred_code(p::Base.Fix2{typeof(!=)}) = (Cint(5), p.x)
pred_code(p) = throw(ArgumentError("unsupported predicate $p: use >(v), <(v), >=(v), <=(v), ==(v) or !=(v)"))

function _find(pred, src::CuArray{T}, last::Bool) where {T}
    code, v = pred_code(pred)
    operand = Ref(convert(T, v))           # host scalar
    out = CuArray{UInt64}(undef, 1)
    n = length(src)
    GC.@preserve operand begin
        check(ccall((:kf_find, libkf), Cint,
                    (Cint, Cint, Cint, CuPtr{Cvoid}, UInt64, Ptr{Cvoid}, CuPtr{UInt64}, Ptr{Cvoid}),
                    code, Cint(last), dtype_code(T), pointer(src), n, operand, pointer(out), stream_handle()), "findfirst")
    end
    r = Array(out)[1]
    last ? (r == 0 ? nothing : Int(r)) : (r >= n ? nothing : Int(r) + 1)   # C side: 0-based / index + 1
end
findfirst(pred, src::CuArray) = _find(pred, src, false)
findlast(pred, src::CuArray) = _find(pred, src, true)

"Vectorised device copy (src/copy/copy.jl:24-28)."
function vcopy!(dst::CuArray{T}, src::CuArray{T}) where {T}
    length(dst) == length(src) || throw(ArgumentError("dst and src must have the same length"))
    check(ccall((:kf_vcopy, libkf), Cint, (CuPtr{Cvoid}, CuPtr{Cvoid}, UInt64, Ptr{Cvoid}),
                pointer(dst), pointer(src), sizeof(T) * length(src), stream_handle()), "vcopy!")
    dst
end
"Vectorised fill (src/copy/copy.jl:30-55)."
function setvalue!(dst::CuArray{T}, val) where {T}
    v = Ref(convert(T, val))
    GC.@preserve v begin
        check(ccall((:kf_setvalue, libkf), Cint, (Cint, CuPtr{Cvoid}, UInt64, Ptr{Cvoid}, Ptr{Cvoid}),
                    dtype_code(T), pointer(dst), length(dst), v, stream_handle()), "setvalue!")
    end
    dst
end

# ---- scan without a workspace (no counterpart in KernelForge.jl) -----------------------------------------
# For callers that cannot allocate device memory where they call: the descriptors live in a fixed 1 MiB
# device array of the library. Calls on one device must not overlap; the first call per device should
# come before any stream capture.
function scan_static!(f, op, dst::CuArray{T}, src::CuArray{T}; g=identity, init=nothing) where {T}
    n = length(src)
    length(dst) == n || throw(ArgumentError("dst and src must have equal lengths"))
    check(ccall((:kf_scan_static, libkf), Cint,
                (Cint, Cint, Cint, Cint, CuPtr{Cvoid}, CuPtr{Cvoid}, UInt64, CuPtr{Cvoid}, UInt32, Ptr{Cvoid}),
                map_code(f), op_code(op), post_code(g), dtype_code(T), pointer(src), pointer(dst), n,
                init === nothing ? CU_NULL : pointer(init), init === nothing ? 0 : length(init), stream_handle()), "scan_static!")
    dst
end
scan_static_max_n(::Type{T}) where {T} = ccall((:kf_scan_static_max_n, libkf), UInt64, (Cint,), dtype_code(T))
scan_static_check() = ccall((:kf_scan_static_check, libkf), Cint, (Ptr{Cvoid},), stream_handle())

# ---- helpers of a sharded sample sort (no counterpart in KernelForge.jl) ---------------------------------
"For each splitter, the index (0-based count) of the first element of the sorted `keys` that is greater."
function upper_bounds(keys::CuArray{K}, splitters::CuArray{K}) where {K}
    out = CuArray{UInt64}(undef, length(splitters))
    check(ccall((:kf_upper_bounds, libkf), Cint, (Cint, CuPtr{Cvoid}, UInt64, CuPtr{Cvoid}, Cint, CuPtr{UInt64}, Ptr{Cvoid}),
                dtype_code(K), pointer(keys), length(keys), pointer(splitters), length(splitters), pointer(out), stream_handle()),
          "upper_bounds")
    out
end
"Destination piece (UInt8) of every key: the number of splitters below it in the sort's key order."
function bucket_ids(keys::CuArray{K}, splitters::CuArray{K}) where {K}
    out = CuArray{UInt8}(undef, length(keys))
    check(ccall((:kf_bucket_ids, libkf), Cint, (Cint, CuPtr{Cvoid}, UInt64, CuPtr{Cvoid}, Cint, CuPtr{UInt8}, Ptr{Cvoid}),
                dtype_code(K), pointer(keys), length(keys), pointer(splitters), length(splitters), pointer(out), stream_handle()),
          "bucket_ids")
    out
end

# Peer-memory exchange of a sharded sample sort (one process per GPU): allocate / export / map / pull.
function xbuf_alloc(nbytes::Integer)
    out = Ref{CuPtr{Cvoid}}(CU_NULL)
    check(ccall((:kf_xbuf_alloc, libkf), Cint, (Csize_t, Ptr{CuPtr{Cvoid}}), nbytes, out), "xbuf_alloc")
    out[]
end
xbuf_free(p::CuPtr{Cvoid}) = check(ccall((:kf_xbuf_free, libkf), Cint, (CuPtr{Cvoid},), p), "xbuf_free")
function ipc_export(p::CuPtr{Cvoid})
    h = Vector{UInt8}(undef, 64)
    check(ccall((:kf_ipc_export, libkf), Cint, (CuPtr{Cvoid}, Ptr{UInt8}), p, h), "ipc_export")
    h
end
function ipc_open(h::Vector{UInt8})
    out = Ref{CuPtr{Cvoid}}(CU_NULL)
    check(ccall((:kf_ipc_open, libkf), Cint, (Ptr{UInt8}, Ptr{CuPtr{Cvoid}}), h, out), "ipc_open")
    out[]
end
ipc_close(p::CuPtr{Cvoid}) = check(ccall((:kf_ipc_close, libkf), Cint, (CuPtr{Cvoid},), p), "ipc_close")
copy_d2d(dst::CuPtr{Cvoid}, src::CuPtr{Cvoid}, nbytes::Integer) =
    check(ccall((:kf_copy_d2d, libkf), Cint, (CuPtr{Cvoid}, CuPtr{Cvoid}, UInt64, Ptr{Cvoid}), dst, src, nbytes, stream_handle()), "copy_d2d")

peer_region_bytes() = ccall((:kf_peer_region_bytes, libkf), Csize_t, ())
"One element per rank, gathered over peer memory by a kernel of the library (see include/kf_b200.h)."
function peer_allgather!(out::CuArray{T}, value::CuArray{T}, peers::CuArray{CuPtr{Cvoid}}, region::CuPtr{Cvoid},
                         world::Integer, rank::Integer, epoch::Integer, status::CuArray{UInt8}) where {T}
    check(ccall((:kf_peer_allgather, libkf), Cint,
                (CuPtr{Cvoid}, CuPtr{Cvoid}, Cint, Cint, UInt32, CuPtr{Cvoid}, Cint, CuPtr{Cvoid}, CuPtr{Cvoid}, Ptr{LaunchCfg}, Ptr{Cvoid}),
                pointer(peers), region, world, rank, epoch, pointer(value), sizeof(T), pointer(out), pointer(status),
                cfg_ptr(nothing), stream_handle()), "peer_allgather!")
    out
end

# ---- library -------------------------------------------------------------------------------------------
launch_count() = ccall((:kf_launch_count, libkf), UInt64, ())
num_sms() = Int(ccall((:kf_num_sms, libkf), Cint, ()))
last_cuda_error() = ccall((:kf_last_cuda_error, libkf), Cint, ())
abi_version() = ccall((:kf_abi_version, libkf), Cint, ())
function launch_table_lookup(primitive::Integer, elem_bytes::Integer, n::Integer)
    out = Ref(LaunchCfg(0, 0, 0, 0))
    check(ccall((:kf_launch_table_lookup, libkf), Cint, (Cint, Cint, UInt64, Ptr{LaunchCfg}), primitive, elem_bytes, n, out),
          "launch_table_lookup")
    out[]
end

"Device-side status of a workspace after synchronising the stream (KF_ERR_TIMEOUT if a bounded wait ran out)."
kf_check(buf::KernelBuffer) =
    ccall((:kf_check, libkf), Cint, (CuPtr{Cvoid}, Ptr{Cvoid}), pointer(buf.arrays.workspace), stream_handle())

end # module
