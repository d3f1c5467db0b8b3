# batched_mul of Float16 / BFloat16 CuArrays through libnnlib_b200 (ext/NNlibCUDAExt/batchedmul_b200.jl),
# modelled on the reference's test/batchedmul.jl:6-16, 40-49: every case is compared with the slice-by-slice
# product of the same (rounded) inputs in Float32 on the host.
using NNlib, CUDA, Test
using NNlib: batched_mul, batched_mul!, batched_transpose

function bmm_host(a, b; transA=false, transB=false)
    transA && (a = permutedims(a, (2, 1, 3)))
    transB && (b = permutedims(b, (2, 1, 3)))
    cat((a[:, :, size(a, 3) == 1 ? 1 : i] * b[:, :, size(b, 3) == 1 ? 1 : i] for i in 1:max(size(a, 3), size(b, 3)))...; dims=3)
end

@testset "batched_mul: $T on tcgen05" for T in (Float16,)
    for (M, N, K, nb) in ((128, 128, 64, 1), (200, 136, 72, 3), (520, 264, 200, 2), (7, 6, 5, 3))
        A = Float32.(T.(randn(Float32, M, K, nb))); B = Float32.(T.(randn(Float32, K, N, nb)))
        dA, dB = cu(T.(A)), cu(T.(B))
        tol = 1f-3 * maximum(abs, bmm_host(A, B))
        @test maximum(abs, Float32.(Array(batched_mul(dA, dB))) .- bmm_host(A, B)) <= tol
        At, Bt = permutedims(A, (2, 1, 3)), permutedims(B, (2, 1, 3))
        dAt, dBt = cu(T.(At)), cu(T.(Bt))
        @test maximum(abs, Float32.(Array(batched_mul(batched_transpose(dAt), dB))) .- bmm_host(A, B)) <= tol
        @test maximum(abs, Float32.(Array(batched_mul(dA, batched_transpose(dBt)))) .- bmm_host(A, B)) <= tol
        @test maximum(abs, Float32.(Array(batched_mul(batched_transpose(dAt), batched_transpose(dBt)))) .- bmm_host(A, B)) <= tol
    end
    # batch of one on one side, alpha / beta
    A = Float32.(T.(randn(Float32, 136, 96, 3))); B = Float32.(T.(randn(Float32, 96, 200, 1)))
    C = Float32.(T.(randn(Float32, 136, 200, 3)))
    dC = cu(T.(C))
    batched_mul!(dC, cu(T.(A)), cu(T.(B)), 0.5f0, -2f0)
    want = 0.5f0 .* bmm_host(A, B) .- 2f0 .* C
    @test maximum(abs, Float32.(Array(dC)) .- want) <= 2f-3 * maximum(abs, want)
    @test_throws DimensionMismatch batched_mul(cu(T.(rand(Float32, 2, 2, 2))), cu(T.(rand(Float32, 2, 2, 10))))
end
