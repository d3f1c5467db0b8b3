# B200 softmax / logsoftmax methods for dense CuArrays.
#
# Add `include("softmax.jl")` to ext/NNlibCUDAExt/NNlibCUDAExt.jl after `include("attention.jl")`
# (it uses `libnnlib_b200`, `B200Float` and `_b200_dtype` from there).  The methods replace what
# ext/NNlibCUDACUDNNExt/softmax.jl routes to cuDNN (leading dims) or to the generic broadcasts
# (non-leading dims, benchmark/cuda_softmax/README.md:80-85): one kernel family in libnnlib_b200.so
# handles every run of consecutive dims, the array being seen as (inner, n, outer).
#
# NOTE: like attention.jl this mirrors the tested Python caller (nnlib_jl_b200/softmax.py) and has not
# been executed (no Julia toolchain where the library was developed).

import NNlib: softmax!, logsoftmax!, ∇softmax!, ∇logsoftmax!

Base.@kwdef struct B200SoftmaxParams
    struct_size::Csize_t = 0
    dtype::Int32 = 0
    log::Int32 = 0
    inner::Int64 = 0; n::Int64 = 0; outer::Int64 = 0
    x::CuPtr{Cvoid} = CU_NULL
    dy::CuPtr{Cvoid} = CU_NULL
    out::CuPtr{Cvoid} = CU_NULL
end

# (inner, n, outer) for a run of consecutive dims (or `:`); nothing when the dims have gaps
function _b200_softmax_split(x, dims)
    dims === Colon() && return (1, length(x), 1)
    ds = sort(unique(collect(Int, dims)))
    (isempty(ds) || ds[1] < 1 || ds != collect(ds[1]:ds[end])) && return nothing
    inner = prod(size(x, i) for i in 1:ds[1]-1; init=1)
    n = prod(size(x, i) for i in ds; init=1)
    return (inner, n, length(x) ÷ max(inner * n, 1))
end

function _b200_softmax!(out::DenseCuArray{T}, x::DenseCuArray{T}, dy, split, log::Bool, backward::Bool) where {T<:B200Float}
    inner, n, outer = split
    p = B200SoftmaxParams(; struct_size=sizeof(B200SoftmaxParams), dtype=_b200_dtype(T), log=Int32(log),
                          inner, n, outer, x=reinterpret(CuPtr{Cvoid}, pointer(x)),
                          dy=dy === nothing ? CU_NULL : reinterpret(CuPtr{Cvoid}, pointer(dy)),
                          out=reinterpret(CuPtr{Cvoid}, pointer(out)))
    GC.@preserve out x dy begin
        rc = backward ?
            ccall((:nnlib_b200_softmax_bwd, libnnlib_b200[]), Cint, (Ref{B200SoftmaxParams}, Ptr{Cvoid}), p, stream().handle) :
            ccall((:nnlib_b200_softmax_fwd, libnnlib_b200[]), Cint, (Ref{B200SoftmaxParams}, Ptr{Cvoid}), p, stream().handle)
    end
    rc == 0 || error("nnlib_b200 softmax failed with code $rc")
    return out
end

for (f, f_generic, islog) in ((:softmax!, :_softmax!, false), (:logsoftmax!, :_logsoftmax!, true))
    @eval function NNlib.$f(y::DenseCuArray{T}, x::DenseCuArray{T}; dims=1) where {T<:B200Float}
        s = _b200_softmax_split(x, dims)
        (s === nothing || size(y) != size(x)) && return NNlib.$f_generic(y, x; dims)
        return _b200_softmax!(y, x, nothing, s, $islog, false)
    end
end
for (f, f_generic, islog) in ((:∇softmax!, :_∇softmax!, false), (:∇logsoftmax!, :_∇logsoftmax!, true))
    @eval function NNlib.$f(dx::DenseCuArray{T}, dy::DenseCuArray{T}, y::DenseCuArray{T}; dims=1) where {T<:B200Float}
        s = _b200_softmax_split(y, dims)
        (s === nothing || size(dx) != size(y) || size(dy) != size(y)) && return NNlib.$f_generic(dx, dy, y; dims)
        return _b200_softmax!(dx, y, dy, s, $islog, true)
    end
end
