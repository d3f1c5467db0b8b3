# B200 attention methods for NNlibCUDAExt.
#
# Add `include("attention.jl")` to ext/NNlibCUDAExt/NNlibCUDAExt.jl (after
# `include("utils.jl")`).  The methods below are strictly more specific than the
# generic ones in src/attention.jl (:52 and :112), so dense `CuArray`s of
# Float16 / BFloat16 / Float32 dispatch here and everything else (views,
# PermutedDimsArray, Float64, complex) keeps running the generic code.  The N-d
# wrapper (src/attention.jl:40-50) reaches the 3-d method unchanged because
# `reshape(::CuArray)` is a `CuArray`.
#
# All arithmetic happens in libnnlib_b200.so (C ABI: include/nnlib_b200.h),
# called with device pointers on the task's current stream.  No cuBLAS, cuDNN
# or KernelAbstractions on this path.
#
# NOTE: this file mirrors, statement for statement, the Python ctypes caller
# (nnlib_jl_b200/attention.py), which is the tested one: no Julia toolchain was
# available where the library was developed, so this source has not been
# executed.  test/ext_cuda/attention.jl is the test to run first.

using CUDA: CuArray, DenseCuArray, CuPtr, CU_NULL, stream, device, device!, devices
import NNlib: dot_product_attention, dot_product_attention_scores, make_causal_mask

# BFloat16 lives in Core from Julia 1.11 on; with BFloat16s.jl loaded on 1.10 use its type instead.
const _BF16 = isdefined(Core, :BFloat16) ? Core.BFloat16 : Union{}
const B200Float = Union{Float16,_BF16,Float32}

const libnnlib_b200 = Ref{String}(get(ENV, "NNLIB_B200_LIB", "libnnlib_b200"))

_b200_dtype(::Type{Float16}) = Int32(0)
_b200_dtype(::Type{Float32}) = Int32(2)
_b200_dtype(::Type{T}) where {T} = T === _BF16 ? Int32(1) : throw(ArgumentError("unsupported eltype $T"))

# Mirror of `nnlib_b200_attn_params` (include/nnlib_b200.h): same order, same types.
Base.@kwdef struct B200AttnParams
    struct_size::Csize_t = 0
    dtype::Int32 = 0
    bias_dtype::Int32 = 0
    d::Int64 = 0; dv::Int64 = 0; H::Int64 = 0; Lq::Int64 = 0; Lkv::Int64 = 0; B::Int64 = 0
    q::CuPtr{Cvoid} = CU_NULL; k::CuPtr{Cvoid} = CU_NULL; v::CuPtr{Cvoid} = CU_NULL; x::CuPtr{Cvoid} = CU_NULL
    q_stride_l::Int64 = 0; q_stride_b::Int64 = 0
    k_stride_l::Int64 = 0; k_stride_b::Int64 = 0
    v_stride_l::Int64 = 0; v_stride_b::Int64 = 0
    x_stride_l::Int64 = 0; x_stride_b::Int64 = 0
    bias::CuPtr{Cvoid} = CU_NULL
    bias_stride::NTuple{4,Int64} = (0, 0, 0, 0)
    mask::CuPtr{UInt8} = CU_NULL
    mask_stride::NTuple{4,Int64} = (0, 0, 0, 0)
    causal::Int32 = 0
    nan_on_fully_masked::Int32 = 1
    scale::Float32 = 0f0
    dropout_p::Float32 = 0f0
    philox_seed::UInt64 = 0
    philox_offset::UInt64 = 0
    rng_h0::Int64 = 0; rng_b0::Int64 = 0; rng_H::Int64 = 0
    lse::CuPtr{Float32} = CU_NULL
    lse_stride_b::Int64 = 0
    alpha::CuPtr{Cvoid} = CU_NULL
    alpha_stride_b::Int64 = 0
    status::CuPtr{Int32} = CU_NULL
    allow_tf32::Int32 = 0
    reserved0::Int32 = 0
    causal_offset::Int64 = 0
end

# One Int32 per device that every launch reports to: a kernel that gave up on a bounded wait, and every launch
# the library skipped on that device afterwards, writes NNLIB_B200_TIMEOUT there (include/nnlib_b200.h,
# "fail-stop behaviour").  Looked at where this file synchronises anyway (`Array(α)`), and by `b200_check_status`.
const _status_words = Dict{Int,CuArray{Int32,1}}()
const _status_lock = ReentrantLock()
function _status_word()
    id = CUDA.deviceid(device())
    lock(_status_lock) do
        get!(() -> CUDA.zeros(Int32, 1), _status_words, id)
    end
end
"Throw if a kernel launched through these methods on the current device gave up on a bounded wait."
function b200_check_status()
    w = lock(() -> get(_status_words, CUDA.deviceid(device()), nothing), _status_lock)
    w === nothing && return nothing
    v = Array(w)[1]
    if v != 0
        fill!(w, 0)
        _b200_check(Cint(v), "a kernel of an earlier call")
    end
    nothing
end

# Float32 arrays: exact fp32 arithmetic unless CUDA.jl's math mode allows reduced precision — the switch that
# lets cuBLAS use TF32 for the reference's own batched_mul.
_allow_tf32(::Type{Float32}) = CUDA.math_mode() == CUDA.FAST_MATH
_allow_tf32(::Type) = false

function _b200_check(rc::Cint, where::String)
    rc == 0 && return nothing
    msg = unsafe_string(ccall((:nnlib_b200_strerror, libnnlib_b200[]), Cstring, (Cint,), rc))
    rc == -1 ? throw(ArgumentError("$where: $msg")) : error("$where: $msg [$rc]")
end

for name in (:attn_fwd, :attn_stats, :attn_scores, :attn_apply)
    fn = Symbol(:_b200_, name)
    sym = QuoteNode(Symbol(:nnlib_b200_, name))
    @eval function $fn(p::B200AttnParams)
        rc = ccall(($sym, libnnlib_b200[]), Cint, (Ref{B200AttnParams}, Ptr{Cvoid}), p, stream().handle)
        _b200_check(rc, $(string(name)))
    end
end

# x and lse.  Few queries against many keys: the library splits the keys of a unit over several CTAs when that
# pays and tells how much scratch memory the partial results need (0: the ordinary forward).
function _b200_forward(p::B200AttnParams)
    need = p.Lq <= 128 ? ccall((:nnlib_b200_attn_decode_workspace_bytes, libnnlib_b200[]), Csize_t,
                               (Ref{B200AttnParams},), p) : Csize_t(0)
    need == 0 && return _b200_attn_fwd(p)
    ws = CuArray{UInt8}(undef, need)
    GC.@preserve ws begin
        rc = ccall((:nnlib_b200_attn_decode, libnnlib_b200[]), Cint,
                   (Ref{B200AttnParams}, CuPtr{Cvoid}, Csize_t, Ptr{Cvoid}), p, pointer(ws), need, stream().handle)
        _b200_check(rc, "attn_decode")
    end
end

"""
    PhiloxDropout(p; seed, offset=0)

`fdrop` that the fused kernels run in place: whether score `(j, i, h, b)` survives
is a pure function of `(seed, offset)` and the position (Philox4x32-10), with the
keep rule of `NNlib.dropout` (keep iff `u > p`, survivors scaled by `1/(1-p)`).
Every use consumes one offset.
"""
mutable struct PhiloxDropout
    p::Float32
    seed::UInt64
    offset::UInt64
    function PhiloxDropout(p::Real; seed::Integer=rand(UInt64), offset::Integer=0)
        0 <= p < 1 || throw(ArgumentError("PhiloxDropout expects a probability 0 <= p < 1"))
        new(Float32(p), UInt64(seed), UInt64(offset))
    end
end
_take_offset!(d::PhiloxDropout) = (o = d.offset; d.offset += 1; o)

"""
    CausalMask(offset=0)

Sentinel for `mask=`: the causal pattern `kv <= query + offset` without the Bool matrix.  `offset = 0` is
`make_causal_mask`'s square pattern; `offset = kv_len - q_len` aligns the last query with the last key (new
queries against a longer key / value history).
"""
struct CausalMask
    offset::Int
end
CausalMask() = CausalMask(0)

# Julia arrays carry no modification counter, so a matrix cannot be proven untouched after
# `make_causal_mask` returned it (`m[1, 3] = true` must change the result).  Every square Bool matrix is
# therefore read on the device each time it is passed: one pass over L*L bytes and a 4-byte copy back.
# Callers who want the causal pattern at no cost pass `mask = CausalMask()`.
function make_causal_mask(x::CuArray; dims::Int=2)
    len = size(x, dims)
    mask = similar(x, Bool, (len, len))
    rc = ccall((:nnlib_b200_causal_fill, libnnlib_b200[]), Cint, (CuPtr{UInt8}, Int64, Ptr{Cvoid}),
               reinterpret(CuPtr{UInt8}, pointer(mask)), len, stream().handle)
    _b200_check(rc, "causal_fill")
    return mask
end

function _is_causal_matrix(mask::DenseCuArray{Bool,2}, Lq, Lkv)
    (Lq == Lkv && size(mask) == (Lkv, Lq)) || return false
    flag = CUDA.zeros(Int32, 1)
    rc = ccall((:nnlib_b200_causal_check, libnnlib_b200[]), Cint, (CuPtr{UInt8}, Int64, CuPtr{Int32}, Ptr{Cvoid}),
               reinterpret(CuPtr{UInt8}, pointer(mask)), Lq, pointer(flag), stream().handle)
    _b200_check(rc, "causal_check")
    return Array(flag)[1] == 1
end
_is_causal_matrix(mask, Lq, Lkv) = false

# element strides of a bias/mask against the (Lkv, Lq, H, B) scores; 0 where it broadcasts
function _bcast_strides(name, t::AbstractArray, full::NTuple{4,Int})
    ndims(t) <= 4 || throw(ArgumentError("$name has $(ndims(t)) dimensions; scores have 4"))
    ntuple(4) do dim
        sz = size(t, dim)
        sz == 1 ? 0 : sz == full[dim] ? Int64(stride(t, dim)) :
            throw(ArgumentError("$name of size $(size(t)) does not broadcast to scores of size $full"))
    end
end

function _b200_params(q::DenseCuArray{T,3}, k::DenseCuArray{T,3}, v, bias, mask, nheads, dropout;
                      rng_origin=nothing) where {T}
    E, Lq, B = size(q); Lkv = size(k, 2); H = nheads
    Ev = v === nothing ? E : size(v, 1)
    full = (Lkv, Lq, H, B)
    causal = false
    coff = 0
    mptr = CuPtr{UInt8}(0); mstr = (0, 0, 0, 0)
    if mask isa CausalMask
        causal = true
        coff = mask.offset
    elseif mask !== nothing
        eltype(mask) === Bool || throw(ArgumentError("mask must be a Bool array"))
        if _is_causal_matrix(mask, Lq, Lkv)
            causal = true
        else
            mstr = _bcast_strides("mask", mask, full)
            mptr = reinterpret(CuPtr{UInt8}, pointer(mask))
        end
    end
    bptr = CuPtr{Cvoid}(0); bstr = (0, 0, 0, 0); bdt = Int32(0)
    if bias !== nothing
        bstr = _bcast_strides("bias", bias, full)
        bptr = reinterpret(CuPtr{Cvoid}, pointer(bias)); bdt = _b200_dtype(eltype(bias))
    end
    p, seed, off = 0f0, UInt64(0), UInt64(0)
    if dropout !== nothing && dropout.p > 0
        p, seed, off = dropout.p, dropout.seed, _take_offset!(dropout)
    end
    h0, b0, Htot = rng_origin === nothing ? (0, 0, 0) : rng_origin
    B200AttnParams(; struct_size=sizeof(B200AttnParams), dtype=_b200_dtype(T), bias_dtype=bdt,
        d=E ÷ H, dv=Ev ÷ H, H, Lq, Lkv, B,
        q=reinterpret(CuPtr{Cvoid}, pointer(q)), k=reinterpret(CuPtr{Cvoid}, pointer(k)),
        v=v === nothing ? CuPtr{Cvoid}(0) : reinterpret(CuPtr{Cvoid}, pointer(v)),
        bias=bptr, bias_stride=bstr, mask=mptr, mask_stride=mstr, causal=Int32(causal), causal_offset=coff,
        dropout_p=p, philox_seed=seed, philox_offset=off, rng_h0=h0, rng_b0=b0, rng_H=Htot,
        status=pointer(_status_word()), allow_tf32=Int32(_allow_tf32(T)))
end

_with(p::B200AttnParams; kw...) = B200AttnParams(; (f => getfield(p, f) for f in fieldnames(B200AttnParams))..., kw...)

"""
    LazyAttnScores{T} <: AbstractArray{T,N}

The `α` of `(x, α) = dot_product_attention(...)` on the B200 path.  The fused
kernel keeps one log-sum-exp per query; the `(kv_len, q_len, nheads, batch...)`
array is rebuilt from it (with the same dropout mask) by a second kernel the
first time an element is needed.  `x, _ = dot_product_attention(...)` never
pays for it.
"""
mutable struct LazyAttnScores{T,N} <: AbstractArray{T,N}
    dims::NTuple{N,Int}
    params::B200AttnParams
    keep::Any                                  # q, k, bias, mask, lse: kept alive for the rebuild
    value::Union{Nothing,CuArray{T,4}}
end
Base.size(a::LazyAttnScores) = a.dims
function materialize!(a::LazyAttnScores{T}) where {T}
    if a.value === nothing
        p = a.params
        α = CuArray{T}(undef, p.Lkv, p.Lq, p.H, p.B)
        GC.@preserve a α _b200_attn_scores(_with(p; alpha=reinterpret(CuPtr{Cvoid}, pointer(α))))
        a.value = α
    end
    return reshape(a.value, a.dims)
end
Base.reshape(a::LazyAttnScores{T}, dims::Dims{N}) where {T,N} =
    (prod(dims) == prod(a.dims) || throw(DimensionMismatch()); LazyAttnScores{T,N}(dims, a.params, (a.keep, a), a.value))
Base.getindex(a::LazyAttnScores, I...) = CUDA.@allowscalar materialize!(a)[I...]
Base.Array(a::LazyAttnScores) = (h = Array(materialize!(a)); b200_check_status(); h)   # the copy synchronised anyway
Base.collect(a::LazyAttnScores) = Array(a)
CUDA.CuArray(a::LazyAttnScores) = materialize!(a)
Base.Broadcast.broadcastable(a::LazyAttnScores) = materialize!(a)
Base.sum(a::LazyAttnScores; kw...) = sum(materialize!(a); kw...)

function dot_product_attention(q::DenseCuArray{T,3}, k::DenseCuArray{T,3}, v::DenseCuArray{T,3}, bias=nothing;
                               fdrop=identity, mask=nothing, nheads=1) where {T<:B200Float}
    # the reference's four checks, same order and text (src/attention.jl:55-78)
    (all(size.((q, k, v), 1) .% nheads .== 0)) || throw(ArgumentError("""
    First dimension in query, key and value must be divisible by `nheads`.
    Instead:
    - size(q): $(size(q))
    - size(k): $(size(k))
    - size(v): $(size(v))
    - nheads: $nheads
    """))
    (size(q, 3) == size(k, 3) == size(v, 3)) || throw(ArgumentError("""
    Batch dimensions have to be the same. Instead:
    - size(q): $(size(q))
    - size(k): $(size(k))
    - size(v): $(size(v))
    """))
    size(q, 1) == size(k, 1) || throw(ArgumentError("""
    First dimension in query and key has to be the same. Instead:
    - size(q): $(size(q))
    - size(k): $(size(k))
    """))
    size(k, 2) == size(v, 2) || throw(ArgumentError("""
    Second dimension in key and value has to be the same. Instead:
    - size(k): $(size(k))
    - size(v): $(size(v))
    """))
    Ev, Lq, B = size(v, 1), size(q, 2), size(q, 3); Lkv = size(k, 2)
    x = similar(q, T, (Ev, Lq, B))
    lse = CuArray{Float32}(undef, Lq, nheads, B)
    if fdrop === identity || fdrop isa PhiloxDropout
        p = _b200_params(q, k, v, bias, mask, nheads, fdrop isa PhiloxDropout ? fdrop : nothing)
        p = _with(p; x=reinterpret(CuPtr{Cvoid}, pointer(x)), lse=pointer(lse))
        GC.@preserve q k v x lse bias mask (Lq > 0 && B > 0 && _b200_forward(p))
        α = LazyAttnScores{T,4}((Lkv, Lq, nheads, B), p, (q, k, bias, mask, lse), nothing)
        return x, α
    else
        # opaque fdrop: materialise α, let the caller's function transform it, x = V·α′ (src/attention.jl:91-98)
        p = _b200_params(q, k, v, bias, mask, nheads, nothing)
        α = CuArray{T}(undef, Lkv, Lq, nheads, B)
        p = _with(p; x=reinterpret(CuPtr{Cvoid}, pointer(x)), lse=pointer(lse), alpha=reinterpret(CuPtr{Cvoid}, pointer(α)))
        GC.@preserve q k v x lse α bias mask begin
            if Lq > 0 && B > 0
                _b200_attn_stats(p); _b200_attn_scores(p)
            end
            α′ = convert(CuArray{T,4}, fdrop(α))
            size(α′) == size(α) || throw(ArgumentError("fdrop must return an array of the scores' size"))
            GC.@preserve α′ (Lq > 0 && B > 0 &&
                _b200_attn_apply(_with(p; alpha=reinterpret(CuPtr{Cvoid}, pointer(α′)))))
            return x, α′
        end
    end
end

function dot_product_attention_scores(q::DenseCuArray{T,4}, k::DenseCuArray{T,4}, bias=nothing;
                                      fdrop=identity, mask=nothing) where {T<:B200Float}
    d, H, Lq, B = size(q); Lkv = size(k, 3)
    q3, k3 = reshape(q, d * H, Lq, B), reshape(k, d * H, Lkv, B)
    dropout = fdrop isa PhiloxDropout ? fdrop : nothing
    α = CuArray{T}(undef, Lkv, Lq, H, B)
    lse = CuArray{Float32}(undef, Lq, H, B)
    p = _with(_b200_params(q3, k3, nothing, bias, mask, H, dropout);
              lse=pointer(lse), alpha=reinterpret(CuPtr{Cvoid}, pointer(α)))
    GC.@preserve q k α lse bias mask if Lq > 0 && B > 0 && Lkv > 0
        _b200_attn_stats(p); _b200_attn_scores(p)
    end
    return (dropout === nothing && fdrop !== identity) ? fdrop(α) : α
end

# ---------------------------------------------------------------------------
# multi-GPU driver: the independent (batch, head) units over the devices of one box,
# one Julia task per device, no collective (every unit is a separate problem,
# src/attention.jl:87-99).
# ---------------------------------------------------------------------------
"Contiguous, balanced unit ranges (unit u = b*H + h) as (b0, nb, h0, nh) rectangles, one list per shard."
function partition_units(B::Int, H::Int, n::Int)
    total = B * H; base, extra = divrem(total, n)
    plan = Vector{Vector{NTuple{4,Int}}}(); u = 0
    for r in 0:n-1
        cnt = base + (r < extra ? 1 : 0); rects = NTuple{4,Int}[]; stop = u + cnt
        while u < stop
            b, h = divrem(u, H)
            if h == 0 && stop - u >= H
                nb = (stop - u) ÷ H; push!(rects, (b, nb, 0, H)); u += nb * H
            else
                nh = min(H - h, stop - u); push!(rects, (b, 1, h, nh)); u += nh
            end
        end
        push!(plan, rects)
    end
    return plan
end

"""
    sharded_attention(q, k, v; nheads, mask=nothing, fdrop=identity, devs=collect(devices()))

`dot_product_attention` of host arrays `q, k, v` with the units spread over `devs`.
Returns `x` on the host and a vector of per-device `(ok, error)` status; a failing
device does not disturb the slices of the others.
"""
function sharded_attention(q::Array{T,3}, k::Array{T,3}, v::Array{T,3}; nheads=1, mask=nothing,
                           fdrop=identity, devs=collect(devices())) where {T}
    E, Lq, B = size(q); Ev = size(v, 1); d, dv = E ÷ nheads, Ev ÷ nheads
    x = Array{T}(undef, Ev, Lq, B)
    drop = fdrop isa PhiloxDropout ? PhiloxDropout(fdrop.p; seed=fdrop.seed, offset=_take_offset!(fdrop)) : nothing
    plan = partition_units(B, nheads, length(devs))
    status = Vector{Any}(undef, length(devs))
    @sync for (r, dev) in enumerate(devs)
        Threads.@spawn try
            device!(dev)
            for (b0, nb, h0, nh) in plan[r]
                bs = b0+1:b0+nb
                qd = CuArray(q[h0*d+1:(h0+nh)*d, :, bs]); kd = CuArray(k[h0*d+1:(h0+nh)*d, :, bs])
                vd = CuArray(v[h0*dv+1:(h0+nh)*dv, :, bs])
                xd = similar(qd, T, (nh * dv, Lq, nb)); lse = CuArray{Float32}(undef, Lq, nh, nb)
                dr = drop === nothing ? nothing : PhiloxDropout(drop.p; seed=drop.seed, offset=drop.offset)
                p = _b200_params(qd, kd, vd, nothing, mask, nh, dr; rng_origin=(h0, b0, nheads))
                p = _with(p; x=reinterpret(CuPtr{Cvoid}, pointer(xd)), lse=pointer(lse))
                GC.@preserve qd kd vd xd lse _b200_attn_fwd(p)
                x[h0*dv+1:(h0+nh)*dv, :, bs] .= Array(xd)
            end
            status[r] = (true, nothing)
        catch err
            status[r] = (false, err)
        end
    end
    return x, status
end

# ---------------------------------------------------------------------------
# Reverse rule.  The generic path is differentiated by Zygote through rrule(batched_mul),
# rrule(softmax) and rrule(dropout); an opaque ccall has no adjoint, so the B200 method brings its
# own: nnlib_b200_attn_bwd recomputes the scores from the saved log-sum-exp and replays the Philox
# dropout mask (tcgen05 kernels for Float16 / BFloat16 with head sizes 64 and 128 — causal flag, Bool
# masks, dropout and bias / dbias included —, CUDA-core kernels otherwise; nnlib_b200_attn_bwd_path
# tells which).  fdrop must be `identity` or a `PhiloxDropout`; other callables keep the generic rules
# (Zygote differentiates the materialise → fdrop → attn_apply sequence only if those steps have rules,
# so such calls should go through the generic method when gradients are needed).
# ---------------------------------------------------------------------------
using ChainRulesCore: ChainRulesCore, NoTangent, ZeroTangent, unthunk

Base.@kwdef struct B200AttnGrads
    struct_size::Csize_t = 0
    dx::CuPtr{Cvoid} = CU_NULL
    dx_stride_l::Int64 = 0; dx_stride_b::Int64 = 0
    dq::CuPtr{Cvoid} = CU_NULL; dk::CuPtr{Cvoid} = CU_NULL; dv::CuPtr{Cvoid} = CU_NULL
    dbias::CuPtr{Float32} = CU_NULL
    dbias_stride::NTuple{4,Int64} = (0, 0, 0, 0)
    delta::CuPtr{Float32} = CU_NULL
end

function ChainRulesCore.rrule(::typeof(dot_product_attention), q::DenseCuArray{T,3}, k::DenseCuArray{T,3},
                              v::DenseCuArray{T,3}, bias=nothing; fdrop=identity, mask=nothing,
                              nheads=1) where {T<:B200Float}
    (fdrop === identity || fdrop isa PhiloxDropout) ||
        throw(ArgumentError("the B200 attention rrule needs fdrop = identity or a PhiloxDropout"))
    x, α = dot_product_attention(q, k, v, bias; fdrop, mask, nheads)
    p = α.params                     # forward description incl. x, lse and the dropout offset that was used
    function attention_pullback(Δ)
        dx = convert(CuArray{T,3}, unthunk(Δ[1]))   # the cotangent of α is not supported (α is lazy)
        dq, dk, dv = similar(q), similar(k), similar(v)
        delta = CuArray{Float32}(undef, p.Lq * p.H * p.B)
        dbias32 = bias === nothing ? nothing : CUDA.zeros(Float32, size(bias))
        g = B200AttnGrads(; struct_size=sizeof(B200AttnGrads), dx=reinterpret(CuPtr{Cvoid}, pointer(dx)),
            dq=reinterpret(CuPtr{Cvoid}, pointer(dq)), dk=reinterpret(CuPtr{Cvoid}, pointer(dk)),
            dv=reinterpret(CuPtr{Cvoid}, pointer(dv)), delta=pointer(delta),
            dbias=dbias32 === nothing ? CuPtr{Float32}(0) : pointer(dbias32),
            dbias_stride=dbias32 === nothing ? (0, 0, 0, 0) : _bcast_strides("bias", dbias32, (p.Lkv, p.Lq, p.H, p.B)))
        GC.@preserve q k v x α dx dq dk dv delta dbias32 bias mask begin
            rc = ccall((:nnlib_b200_attn_bwd, libnnlib_b200[]), Cint,
                       (Ref{B200AttnParams}, Ref{B200AttnGrads}, Ptr{Cvoid}), p, g, stream().handle)
            _b200_check(rc, "attn_bwd")
        end
        dbias = bias === nothing ? NoTangent() : convert(typeof(bias), dbias32)
        return (NoTangent(), dq, dk, dv, dbias)
    end
    return (x, α), attention_pullback
end
