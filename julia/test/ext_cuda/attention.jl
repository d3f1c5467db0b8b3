# CUDA attention tests for the B200 methods of NNlibCUDAExt (ext/NNlibCUDAExt/attention.jl).
# Add `include("attention.jl")` to test/ext_cuda/runtests.jl.  Same strategy as the other
# ext_cuda tests: run on Array and on CuArray and compare (test/ext_cuda/test_utils.jl).
# Not executed where the library was developed (no Julia there); the Python tests under
# tests/ of the library's repository exercise the same C ABI with the same cases.

@testset "attention: CPU vs B200 kernels" begin
    n, lenq, lenkv = 15, 3, 4
    for batch_size in [(), 1, 2, (2, 1, 3)], nheads in [1, 3, 5]
        qh = rand(Float32, n, lenq, batch_size...)
        kh = rand(Float32, n, lenkv, batch_size...)
        vh = rand(Float32, n, lenkv, batch_size...)
        q, k, v = cu(qh), cu(kh), cu(vh)
        y, α = dot_product_attention(q, k, v; nheads)
        @test y isa CuArray{Float32}
        @test size(y) == (n, lenq, batch_size...)
        @test size(α) == (lenkv, lenq, nheads, batch_size...)
        @test sum(Array(α), dims=1) ≈ ones(1, lenq, nheads, batch_size...)
        yh, αh = dot_product_attention(qh, kh, vh; nheads)
        @test Array(y) ≈ yh atol=1f-5
        @test Array(α) ≈ αh atol=1f-5
    end
end

@testset "attention: golden values on the device" begin
    q = k = v = cu(Float32.(reshape([1:12;], 4, 3, 1) ./ 12))
    y, α = dot_product_attention(q, k, v; nheads=2)
    ytrue = [0.429754, 0.513087, 0.613791, 0.697125, 0.46431, 0.547644, 0.647876, 0.73121, 0.49773, 0.581064, 0.680455, 0.763788]
    @test vec(Array(y)) ≈ ytrue atol=1e-5
end

@testset "attention: tensor-core path (Float16, d = 64 / 128)" begin
    for (E, H) in [(128, 2), (256, 2)], causal in (false, true)
        L = 300
        qh, kh, vh = (Float32.(Float16.(randn(Float32, E, L, 2))) for _ in 1:3)
        mask = causal ? make_causal_mask(qh) : nothing
        yh, αh = dot_product_attention(qh, kh, vh; nheads=H, mask)
        q, k, v = (cu(Float16.(a)) for a in (qh, kh, vh))
        y, α = dot_product_attention(q, k, v; nheads=H, mask=causal ? make_causal_mask(q) : nothing)
        @test maximum(abs, Float32.(Array(y)) .- yh) <= 3f-3
        @test maximum(abs, Float32.(Array(α)) .- αh) <= 3f-3
    end
end

@testset "attention: mask" begin
    x = CUDA.rand(Float32, 4, 2, 3, 1)
    mask = make_causal_mask(x, dims=3)
    @test mask isa CuArray{Bool}
    α = dot_product_attention_scores(x, x; mask)
    α_host, mask_host = Array.((α, mask))
    @test all((α_host[:, :, 1, 1] .> 0) .== mask_host)
    @test all((α_host[:, :, 2, 1] .> 0) .== mask_host)
end

@testset "attention: a modified causal matrix is an ordinary mask" begin
    q = CUDA.rand(Float32, 8, 6, 1)
    mask = make_causal_mask(q)
    CUDA.@allowscalar mask[5, 2] = true            # key 5 now visible to query 2
    α = Array(dot_product_attention(q, q, q; nheads=2, mask)[2])
    @test all(α[5, 2, :, 1] .> 0)
    αh = dot_product_attention(Array(q), Array(q), Array(q); nheads=2, mask=Array(mask))[2]
    @test α ≈ αh atol=1f-5
end

@testset "attention: dropout" begin
    q = k = v = CUDA.rand(Float32, 10, 10, 10)
    y, α = dot_product_attention(q, k, v; nheads=2, fdrop=x -> dropout(x, 0.5))      # opaque callable
    @test 0.6 > mean(>(0), Array(α)) > 0.4
    ext = Base.get_extension(NNlib, :NNlibCUDAExt)
    y, α = dot_product_attention(q, k, v; nheads=2, fdrop=ext.PhiloxDropout(0.5; seed=1))  # fused
    @test 0.6 > mean(>(0), Array(α)) > 0.4
end
