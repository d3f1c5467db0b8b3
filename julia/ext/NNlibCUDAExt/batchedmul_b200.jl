# batched_mul for Float16 / BFloat16 CuArrays on the B200 tensor cores.
#
# Add `include("batchedmul_b200.jl")` to ext/NNlibCUDAExt/NNlibCUDAExt.jl next to `include("batchedmul.jl")`.
#
# The reference routes `batched_mul!` to BLAS only for `BlasFloat` element types
# (src/batched/batchedmul.jl:256-259); Float16 and BFloat16 CuArrays fall to `batched_mul_generic!`
# (:306-325), a per-slice `mul!`.  The two methods below send them through the same stride analysis the
# BLAS route uses (`_batched_try_gemm!`, :261-303, reproduced for the real case) and then to
# `nnlib_b200_batched_gemm` (include/nnlib_b200.h): tcgen05 kernel when A and B are 16-byte aligned with
# leading dimensions / batch strides that are multiples of 8 elements, a CUDA-core kernel otherwise.
#
# NOTE: like attention.jl this file mirrors the tested Python caller (nnlib_jl_b200/batched.py) and has not
# been executed: no Julia toolchain was available where the library was developed.

import NNlib: _batched_mul!, _batched_gemm!, batched_transpose, batched_mul_generic!, BatchedAdjoint, BatchedTranspose,
              is_strided, _unbatch

const B200Half = Union{Float16,_BF16}

Base.@kwdef struct B200GemmParams
    struct_size::Csize_t = 0
    dtype::Int32 = 0
    transA::Int32 = 0
    transB::Int32 = 0
    reserved::Int32 = 0
    M::Int64 = 0; N::Int64 = 0; K::Int64 = 0; batch::Int64 = 0
    A::CuPtr{Cvoid} = CU_NULL; lda::Int64 = 0; strideA::Int64 = 0
    B::CuPtr{Cvoid} = CU_NULL; ldb::Int64 = 0; strideB::Int64 = 0
    C::CuPtr{Cvoid} = CU_NULL; ldc::Int64 = 0; strideC::Int64 = 0
    alpha::Float32 = 1f0
    beta::Float32 = 0f0
    status::CuPtr{Int32} = CU_NULL
end

# C = alpha * op(A) * op(B) + beta * C per batch, the contract of batched_gemm! (src/gemm.jl:89-188)
function NNlib._batched_gemm!(::Type{<:CuArray{T}}, transA::Char, transB::Char, alpha::Number, A, B, beta::Number,
                              C) where {T<:B200Half}
    m = size(A, transA == 'N' ? 1 : 2); ka = size(A, transA == 'N' ? 2 : 1)
    kb = size(B, transB == 'N' ? 1 : 2); n = size(B, transB == 'N' ? 2 : 1)
    (ka == kb && m == size(C, 1) && n == size(C, 2)) ||
        throw(DimensionMismatch("A1 has size ($m,$ka), B1 has size ($kb,$n), C1 has size $(size(C)[1:2])"))
    (size(A, 3) == 1 || size(A, 3) == size(C, 3)) || throw(DimensionMismatch("batch size mismatch: A != C"))
    (size(B, 3) == 1 || size(B, 3) == size(C, 3)) || throw(DimensionMismatch("batch size mismatch: B != C"))
    p = B200GemmParams(; struct_size=sizeof(B200GemmParams), dtype=_b200_dtype(T),
        transA=Int32(transA != 'N'), transB=Int32(transB != 'N'), M=m, N=n, K=ka, batch=size(C, 3),
        A=reinterpret(CuPtr{Cvoid}, pointer(A)), lda=max(1, stride(A, 2)), strideA=size(A, 3) == 1 ? 0 : stride(A, 3),
        B=reinterpret(CuPtr{Cvoid}, pointer(B)), ldb=max(1, stride(B, 2)), strideB=size(B, 3) == 1 ? 0 : stride(B, 3),
        C=reinterpret(CuPtr{Cvoid}, pointer(C)), ldc=max(1, stride(C, 2)), strideC=stride(C, 3),
        alpha=Float32(alpha), beta=Float32(beta), status=pointer(_status_word()))
    GC.@preserve A B C begin
        rc = ccall((:nnlib_b200_batched_gemm, libnnlib_b200[]), Cint, (Ref{B200GemmParams}, Ptr{Cvoid}), p, stream().handle)
        _b200_check(rc, "batched_gemm")
    end
    C
end

# The stride analysis of `_batched_try_gemm!` (src/batched/batchedmul.jl:261-303) for real 16-bit element types:
# a factor with unit first stride goes in as 'N', one with unit second stride as 'T' of its parent.
function NNlib._batched_mul!(::Type{DT}, C, A, B, alpha::Number, beta::Number) where {DT<:CuArray{T}} where {T<:B200Half}
    (is_strided(_unbatch(A)) && is_strided(_unbatch(B)) && C isa StridedArray && stride(C, 1) == 1) ||
        return batched_mul_generic!(C, A, B, alpha, beta)
    function flag(X)
        X = X isa BatchedAdjoint ? batched_transpose(parent(X)) : X          # real: adjoint == transpose
        if stride(X, 2) == 1 && size(X, 1) > 1
            batched_transpose(X), 'T'
        elseif stride(X, 1) == 1
            X, 'N'
        elseif stride(X, 2) == 1
            batched_transpose(X), 'T'
        else
            nothing, 'X'
        end
    end
    blasA, tA = flag(A); blasB, tB = flag(B)
    (tA == 'X' || tB == 'X') && return batched_mul_generic!(C, A, B, alpha, beta)
    _batched_gemm!(DT, tA, tB, alpha, blasA, blasB, beta, C)
    C
end
