// Host-side launch functions of every kernel family, shared between the
// translation units and the C ABI in api.cu.
#pragma once
#include <cuda_runtime.h>
#include "common.cuh"

namespace nb200 {

// argument check of the x + alpha composites (api.cu): everything attn_fwd and attn_scores would reject
int attention_validate(const nnlib_b200_attn_params* p, bool launching = true);
int attention_both(const nnlib_b200_attn_params* p, void* stream);

// CUDA-core kernels (attn_simt.cu)
bool simt_supports(int d, int dv);
cudaError_t simt_fwd(const AttnArgs& a, int dtype, cudaStream_t st);
cudaError_t simt_stats(const AttnArgs& a, int dtype, cudaStream_t st);
cudaError_t simt_scores(const AttnArgs& a, int dtype, cudaStream_t st);
cudaError_t simt_apply(const AttnArgs& a, int dtype, cudaStream_t st);
cudaError_t causal_fill(unsigned char* m, long long L, cudaStream_t st);
cudaError_t causal_check(const unsigned char* m, long long L, int* flag, cudaStream_t st);

// backward on CUDA cores (attn_bwd_simt.cu)
bool simt_bwd_supports(int d, int dv);
cudaError_t simt_bwd(const AttnArgs& a, const BwdArgs& g, int dtype, cudaStream_t st);

// tcgen05 + TMA kernels (attn_umma.cu)
const char* umma_fwd_reject_reason(const AttnArgs& a, int dtype, bool need_v);
cudaError_t umma_fwd(const AttnArgs& a, int dtype, bool stats_only, cudaStream_t st);
cudaError_t umma_scores(const AttnArgs& a, int dtype, cudaStream_t st);
bool umma_apply_supports(const AttnArgs& a, int dtype);
cudaError_t umma_apply(const AttnArgs& a, int dtype, cudaStream_t st);
cudaError_t umma_take_abort(int* out, cudaStream_t st);
cudaError_t umma_wait_runout(unsigned long long limit_ns, int* status, cudaStream_t st);

// tcgen05 + TMA kernels for other head sizes and for Float32 arrays on the TF32 path (attn_tile.cu)
const char* tile_reject_reason(const AttnArgs& a, int dtype, bool need_v, bool allow_tf32);
cudaError_t tile_fwd(const AttnArgs& a, int dtype, cudaStream_t st);
cudaError_t tile_stats(const AttnArgs& a, int dtype, cudaStream_t st);
cudaError_t tile_scores(const AttnArgs& a, int dtype, cudaStream_t st);
cudaError_t tile_take_abort(int* out, cudaStream_t st);
int tile_split_count(const AttnArgs& a);                 // 0: the split-key forward does not apply (Lq > 128)
size_t tile_split_workspace_bytes(const AttnArgs& a);
cudaError_t tile_split(const AttnArgs& a, int dtype, cudaStream_t st);   // a.ws holds the workspace

// x and alpha in one pass when a query's whole score row fits in tensor memory (attn_short.cu)
bool short_supports(const AttnArgs& a, int dtype);
cudaError_t short_attention(const AttnArgs& a, int dtype, cudaStream_t st);
cudaError_t short_take_abort(int* out, cudaStream_t st);

// tcgen05 backward kernels (attn_bwd_umma.cu)
bool umma_bwd_supports(const AttnArgs& a, const BwdArgs& g, int dtype);
cudaError_t umma_bwd(const AttnArgs& a, const BwdArgs& g, int dtype, cudaStream_t st);
cudaError_t umma_bwd_take_abort(int* out, cudaStream_t st);

// strided-batched matrix product (gemm_umma.cu): tcgen05 kernel for 16-bit arrays, CUDA-core kernel for the rest
const char* gemm_umma_reject_reason(const GemmArgs& g, int dtype);
cudaError_t gemm_umma(const GemmArgs& g, int dtype, cudaStream_t st);
cudaError_t gemm_simt(const GemmArgs& g, int dtype, cudaStream_t st);
cudaError_t gemm_take_abort(int* out, cudaStream_t st);

// softmax / logsoftmax over one dimension (softmax.cu)
cudaError_t softmax_forward(int dtype, bool log, const void* x, void* y, long long inner, long long n, long long outer,
                            cudaStream_t st);
cudaError_t softmax_backward(int dtype, bool log, const void* dy, const void* y, void* dx, long long inner, long long n,
                             long long outer, cudaStream_t st);

}  // namespace nb200
