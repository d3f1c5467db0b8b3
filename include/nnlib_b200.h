/*
 * libnnlib_b200.so — C ABI of the B200 (sm_100a) multi-head attention path
 * that stands behind NNlib.jl's
 *     dot_product_attention / dot_product_attention_scores / make_causal_mask
 * (NNlib.jl src/attention.jl:40-159).
 *
 * The boundary is plain C: pointers, sizes, strides, one params struct.  Every
 * pointer in the struct is a DEVICE pointer of the CUDA context that is current
 * on the calling thread; `stream` is a cudaStream_t / CUstream passed as
 * void*.  All entry points enqueue work on that stream and return without
 * synchronising; they never allocate device memory, never change the current
 * device and never throw.  They are re-entrant: several host threads, one per
 * device, may call them at once.  q and x (every pointer when the environment
 * variable NNLIB_B200_CHECK_POINTERS=1 is set) must be memory of the current
 * device, else NNLIB_B200_INVALID_ARG.
 *
 * Fail-stop behaviour of the tensor-core kernels.  Every wait inside them
 * (on a copy, on the tensor core, on another warp) is bounded: after 1 s
 * without progress the thread block gives up, releases what it holds and
 * returns, so a fault in this library cannot hang the GPU.  From then on the
 * DEVICE is marked: every later tensor-core launch of this library on it
 * returns at once WITHOUT writing its outputs, while the entry points keep
 * returning NNLIB_B200_OK (they never synchronise).  The mark shows in two
 * places: p->status, when the caller passes one, is set to
 * NNLIB_B200_TIMEOUT by the launch that gave up and by every launch that was
 * skipped; nnlib_b200_device_health reports and clears it.  Callers should
 * pass a status word and look at it (or call device_health) wherever they
 * synchronise anyway.  It has never fired in a correct run.
 *
 * NNLIB_B200_LOG=1 prints one line per call on stderr: entry point, sizes,
 * options, kernel family (tcgen05 / cuda-core) and, for a call that could
 * not take the tensor-core kernels, the reason (for instance a pointer that
 * is not 16-byte aligned).
 *
 * Memory layout = the reference's column-major arrays:
 *   q      (E , Lq , B)   element (e, i, b) at  q[e + q_stride_l*i + q_stride_b*b]
 *   k      (E , Lkv, B)
 *   v      (Ev, Lkv, B)
 *   x      (Ev, Lq , B)   output
 *   alpha  (Lkv, Lq, H, B) element (j, i, h, b) at alpha[j + Lkv*i + Lkv*Lq*h + alpha_stride_b*b]
 *   lse    (Lq, H, B) float32, natural-log sum of exponentials of the scaled,
 *          biased, masked logits of each query; −inf for a query with nothing
 *          to attend to; NaN for a query with a NaN logit; for a query whose
 *          largest logit is +Inf (a +Inf bias: the reference's softmax then
 *          gives equal shares to the +Inf keys, src/softmax.jl:73-75) a NaN
 *          with the quiet bit clear whose low 22 bits count those keys, which
 *          is what attn_scores needs to rebuild that query's scores
 * with E = H*d, Ev = H*dv; head h owns features h*d .. h*d+d-1
 * (split_heads is a pure reshape, src/attention.jl:158).
 */
#ifndef NNLIB_B200_H_
#define NNLIB_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NNLIB_B200_VERSION 200 /* major*10000 + minor*100 + patch */

#if defined(__GNUC__)
#define NNLIB_B200_API __attribute__((visibility("default")))
#else
#define NNLIB_B200_API
#endif

/* element types of q, k, v, x, alpha (one type for all five) and of bias */
enum {
  NNLIB_B200_F16 = 0,
  NNLIB_B200_BF16 = 1,
  NNLIB_B200_F32 = 2
};

/* return codes: 0 = enqueued, negative = nothing was enqueued */
enum {
  NNLIB_B200_OK = 0,
  NNLIB_B200_INVALID_ARG = -1,       /* null pointer, bad size, bad stride, bad dtype, p outside [0,1) */
  NNLIB_B200_UNSUPPORTED_SHAPE = -2, /* head dimension beyond what any kernel here handles */
  NNLIB_B200_CUDA_ERROR = -3,        /* a CUDA runtime/driver call failed; see nnlib_b200_last_cuda_error */
  NNLIB_B200_TIMEOUT = -4,           /* reported through *status by a kernel whose bounded wait ran out */
  NNLIB_B200_WORKSPACE_TOO_SMALL = -5
};

/* which kernel family a call would use (nnlib_b200_attn_path) */
enum {
  NNLIB_B200_PATH_SIMT = 1,   /* CUDA-core kernel: any dtype, any d <= 1024, dv <= 512, any stride */
  NNLIB_B200_PATH_UMMA = 2,   /* tcgen05 + TMA kernel, two query tiles per CTA: f16/bf16, d = dv any multiple
                                 of 8 up to 128, 16-byte aligned rows */
  NNLIB_B200_PATH_TILE = 3    /* tcgen05 + TMA kernel, one query tile per CTA: f16/bf16 with d, dv any multiples
                                 of 8 up to 256 (dv may differ from d); f32 with allow_tf32 and d, dv multiples
                                 of 4 up to 128; 16-byte aligned rows */
};

typedef struct nnlib_b200_attn_params {
  size_t struct_size;   /* = sizeof(nnlib_b200_attn_params); versions the struct */

  int32_t dtype;        /* NNLIB_B200_F16 / BF16 / F32 */
  int32_t bias_dtype;   /* element type of bias (ignored when bias == NULL) */

  int64_t d;            /* qk features per head  (size(q,1) / nheads) */
  int64_t dv;           /* v  features per head  (size(v,1) / nheads) */
  int64_t H;            /* nheads */
  int64_t Lq;           /* size(q,2) */
  int64_t Lkv;          /* size(k,2) == size(v,2) */
  int64_t B;            /* product of the batch dimensions */

  const void* q;
  const void* k;
  const void* v;        /* unused by attn_stats / attn_scores */
  void* x;              /* unused by attn_stats / attn_scores */

  /* strides in ELEMENTS; the feature stride is 1.  0 means dense:
     stride_l = H*d (or H*dv), stride_b = stride_l * L. */
  int64_t q_stride_l, q_stride_b;
  int64_t k_stride_l, k_stride_b;
  int64_t v_stride_l, v_stride_b;
  int64_t x_stride_l, x_stride_b;

  /* bias added to the scaled logits before masking (apply_attn_bias,
     src/attention.jl:129-131).  Element (j, i, h, b) at
     bias[j*s[0] + i*s[1] + h*s[2] + b*s[3]]; a stride of 0 broadcasts. */
  const void* bias;
  int64_t bias_stride[4];

  /* Bool mask, one byte per element, non-zero = attend (apply_attn_mask,
     src/attention.jl:133-138).  Same indexing/broadcast rule as bias. */
  const uint8_t* mask;
  int64_t mask_stride[4];

  int32_t causal;              /* 1: additionally keep only j <= i + causal_offset (make_causal_mask,
                                  src/attention.jl:149-153, is the case causal_offset = 0) */
  int32_t nan_on_fully_masked; /* 1 (reference behaviour, src/softmax.jl:71-76): a query with nothing to
                                  attend to yields NaN in x and alpha; 0: zeros */

  float scale;                 /* multiplies q·k; 0 means 1/sqrt(d) (src/attention.jl:118) */

  /* dropout on alpha (fdrop, src/attention.jl:126; keep-rule of src/dropout.jl:77-87: keep iff
     rand > p, kept entries scaled by 1/(1-p)).  The random number of element (j,i,h,b) is a 16-bit
     lane of Philox4x32-10(key = seed): counter (j/8, r_lo, r_hi + offset_hi, offset_lo), lane j%8 =
     the low (even j) or high (odd j) half of output word (j%8)/2; the element is dropped iff its lane
     is < floor(p * 2^16).  p = 0 disables.  r = i + Lq*((h + rng_h0) + rng_H*(b + rng_b0)), so that a
     shard holding a sub-range of heads or batches draws the same mask as the whole problem.
     rng_H = 0 means H. */
  float dropout_p;
  uint64_t philox_seed;
  uint64_t philox_offset;
  int64_t rng_h0, rng_b0, rng_H;

  float* lse;                  /* attn_fwd/attn_stats: written when non-NULL; attn_scores: read (required) */
  int64_t lse_stride_b;        /* 0 = dense (Lq*H) */

  void* alpha;                 /* attn_scores: written; attn_apply: read; attn_fwd: ignored */
  int64_t alpha_stride_b;      /* 0 = dense (Lkv*Lq*H) */

  int32_t* status;             /* optional device int32: set to NNLIB_B200_TIMEOUT by a kernel whose
                                  bounded wait ran out (never happens in a correct run); else untouched */

  int32_t allow_tf32;          /* Float32 arrays only.  0 (default): exact fp32 arithmetic on the CUDA-core
                                  kernels, within 1e-5 of the reference's CPU result like the reference's own
                                  GPU tests ask (test/ext_amdgpu/attention.jl:19-21).  1: both products run on
                                  the tensor cores with TF32 operands (10-bit mantissa; max-abs error about
                                  3e-3 on unit-variance inputs), what CUDA.jl's FAST_MATH math mode allows
                                  cuBLAS to do for the reference's batched_mul */
  int32_t reserved0;

  int64_t causal_offset;       /* with causal = 1: query i keeps the keys j <= i + causal_offset.  0 is
                                  make_causal_mask's square pattern; Lkv - Lq aligns the last query with the
                                  last key (new queries against a longer key / value history).  A query that
                                  keeps no key at all is one with nothing to attend to. */
} nnlib_b200_attn_params;

/* x = attention(q,k,v) and, when lse != NULL, lse.  Replaces the whole of
   dot_product_attention's arithmetic (src/attention.jl:86-101,112-127 and the
   softmax of src/softmax.jl:69-79) without materialising alpha. */
NNLIB_B200_API int nnlib_b200_attn_fwd(const nnlib_b200_attn_params* p, void* stream);

/* The same result as nnlib_b200_attn_fwd for a call with few queries against many keys (Lq <= 128; typically
   one new token, or a handful, against a long key / value history, with causal_offset = Lkv - Lq).  attn_fwd
   gives such a call one CTA per (head, batch) unit, which leaves most of the GPU idle when H*B is small; here
   the key tiles of a unit are dealt to several CTAs and a second kernel merges their running maxima, sums and
   partial outputs.  The partial results live in `workspace` (device memory, 16-byte aligned, at least
   nnlib_b200_attn_decode_workspace_bytes(p)); when that function returns 0 the call gains nothing from
   splitting (or its shape is outside the tensor-core kernels) and is simply forwarded to attn_fwd.
   The reference has no counterpart: make_causal_mask is square only (src/attention.jl:149-153). */
NNLIB_B200_API size_t nnlib_b200_attn_decode_workspace_bytes(const nnlib_b200_attn_params* p);
NNLIB_B200_API int nnlib_b200_attn_decode(const nnlib_b200_attn_params* p, void* workspace, size_t workspace_bytes,
                                          void* stream);

/* lse only: the first half of dot_product_attention_scores
   (src/attention.jl:117-125) reduced to one float per query. */
NNLIB_B200_API int nnlib_b200_attn_stats(const nnlib_b200_attn_params* p, void* stream);

/* alpha (after dropout) from q, k, bias, mask and a previously computed lse:
   the array dot_product_attention_scores returns (src/attention.jl:112-127). */
NNLIB_B200_API int nnlib_b200_attn_scores(const nnlib_b200_attn_params* p, void* stream);

/* x = V · alpha for an alpha the caller already holds, i.e. the second
   batched_mul of _dot_product_attention (src/attention.jl:96-98).  Used when
   fdrop is an arbitrary callable that was applied to alpha outside. */
NNLIB_B200_API int nnlib_b200_attn_apply(const nnlib_b200_attn_params* p, void* stream);

/* x AND alpha in one call: what dot_product_attention returns
   (src/attention.jl:83).  lse goes to p->lse when non-NULL, else to
   `workspace` (device memory, at least nnlib_b200_workspace_bytes(p)). */
NNLIB_B200_API int nnlib_b200_attention(const nnlib_b200_attn_params* p, void* workspace,
                         size_t workspace_bytes, void* stream);
NNLIB_B200_API size_t nnlib_b200_workspace_bytes(const nnlib_b200_attn_params* p);

/* The same result as nnlib_b200_attention (x and alpha), for callers that
   cannot provide a workspace because they cannot allocate device memory where
   they call from: all of the device belongs to a memory pool (a cudaMalloc
   would fail or stall every stream), the call site is one where the host
   language's array allocator must not run, or the caller was handed input and
   output pointers and nothing else.  The log-sum-exp goes to a fixed 4 MiB
   array inside the library's device image instead (held by every GPU that
   loads the library, until exit), so a call may cover at most
   NNLIB_B200_STATIC_MAX_QUERIES queries (Lq*H*B); beyond that it returns
   NNLIB_B200_WORKSPACE_TOO_SMALL and does nothing.  p->lse is ignored.  All
   calls on a device share the array: calls that can overlap on the GPU race
   and must be serialised by the caller; nothing needs clearing between calls.
   The first call on each device resolves the array's address; with CUDA's
   lazy module loading that look-up is also what brings the array into being
   (the driver reserves its 4 MiB then and may synchronise the device), so
   make that first call early: before a memory pool claims the rest of the
   device and before any stream capture.  Later calls do no set-up and reach
   no allocating routine.  The address is remembered per device ordinal for
   the life of the process: it assumes the device's primary context is never
   reset.  This entry point has no counterpart in the reference. */
#define NNLIB_B200_STATIC_MAX_QUERIES 1048576ull
NNLIB_B200_API int nnlib_b200_attention_static(const nnlib_b200_attn_params* p, void* stream);

/* Where that fixed array lives on the current device and how large it is (does the same first-call
   set-up).  For tests and for callers that account for every byte of device memory.  No counterpart in
   the reference. */
NNLIB_B200_API int nnlib_b200_static_scratch(void** device_ptr, size_t* bytes);

/* Gradient buffers of nnlib_b200_attn_bwd.  dx, dq, dk, dv have the element type of the forward
   arrays; dq (E, Lq, B), dk (E, Lkv, B), dv (Ev, Lkv, B) are written dense. */
typedef struct nnlib_b200_attn_grads {
  size_t struct_size;        /* = sizeof(nnlib_b200_attn_grads) */
  const void* dx;            /* cotangent of x, (Ev, Lq, B) */
  int64_t dx_stride_l, dx_stride_b;   /* element strides, 0 = dense */
  void* dq;
  void* dk;
  void* dv;
  float* dbias;              /* optional float32 accumulator, indexed like bias with dbias_stride
                                (a stride of 0 sums over that dimension); the CALLER zeroes it first */
  int64_t dbias_stride[4];
  float* delta;              /* scratch, Lq*H*B float32 */
} nnlib_b200_attn_grads;

/* Pullback of x = dot_product_attention(q, k, v, bias; mask, nheads, fdrop)[1]: what Zygote composes
   from rrule(batched_mul) (src/batched/batchedmul.jl:96-110), the softmax pullback
   (src/softmax.jl:84-116) and the dropout pullback (src/dropout.jl:106-122) on this path.
   p describes the forward call and must carry its outputs x and lse; dropout parameters must be the
   forward's, so that the same scores are dropped. */
NNLIB_B200_API int nnlib_b200_attn_bwd(const nnlib_b200_attn_params* p, const nnlib_b200_attn_grads* g,
                                       void* stream);

/* NNLIB_B200_PATH_* that attn_bwd would take for (p, g), or a negative error.  The tensor-core
   backward covers 16-bit element types with d = dv any multiple of 8 up to 128 and every option of the forward
   (causal flag, Bool mask arrays, dropout, bias with dbias); Float32 arrays and other head sizes
   run on the CUDA-core kernels. */
NNLIB_B200_API int nnlib_b200_attn_bwd_path(const nnlib_b200_attn_params* p, const nnlib_b200_attn_grads* g);

/* softmax / logsoftmax over one dimension of a dense column-major array and their pullbacks
   (src/softmax.jl:69-79 _softmax!, :147-157 _logsoftmax!, :98-101 _∇softmax!, :170-190 ∇logsoftmax;
   CUDA methods in ext/NNlibCUDACUDNNExt/softmax.jl).  The array is seen as (inner, n, outer) with the
   reduction over the middle extent: for `dims = k` of an N-d array, inner = prod(size[1:k-1]),
   n = size[k], outer = prod(size[k+1:N]).  Element type as in attn_params.dtype; arithmetic in fp32.
   Non-finite inputs follow the reference: a column whose maximum is +Inf puts its weight on the +Inf
   entries in equal shares, a column whose maximum is -Inf or that holds a NaN becomes NaN.
   x and y (dy, y and dx) may alias. */
typedef struct nnlib_b200_softmax_params {
  size_t struct_size;        /* = sizeof(nnlib_b200_softmax_params) */
  int32_t dtype;             /* NNLIB_B200_F16 / BF16 / F32 */
  int32_t log;               /* 0: softmax, 1: logsoftmax */
  int64_t inner, n, outer;
  const void* x;             /* forward: input.            backward: y = (log)softmax(x) */
  const void* dy;            /* forward: ignored.          backward: cotangent of y */
  void* out;                 /* forward: y.                backward: dx */
} nnlib_b200_softmax_params;

NNLIB_B200_API int nnlib_b200_softmax_fwd(const nnlib_b200_softmax_params* p, void* stream);
NNLIB_B200_API int nnlib_b200_softmax_bwd(const nnlib_b200_softmax_params* p, void* stream);

/* Strided-batched matrix product of column-major arrays,
       C[:, :, b] = alpha * op(A[:, :, b]) * op(B[:, :, b]) + beta * C[:, :, b],   b = 0 .. batch-1,
   the operation NNlib.batched_mul! reaches through NNlib._batched_gemm!(storage, transA, transB, alpha, A, B,
   beta, C) (src/batched/batchedmul.jl:256-303; CPU kernel batched_gemm!, src/gemm.jl:89-188).  The reference's
   CUDA method (ext/NNlibCUDAExt/batchedmul.jl:3-4) covers BlasFloat element types only; Float16 and BFloat16
   arrays fall to the per-slice generic loop (src/batched/batchedmul.jl:306-325).  op(X) = X for trans = 0 and
   the transpose of the stored matrix for trans = 1 (BLAS 'N' / 'T'); op(A) is M x K, op(B) is K x N.  Element
   (i, j) of a stored matrix sits at X[i + ld*j + stride*b]; a batch stride of 0 for A or B uses one matrix for
   every batch (size(A, 3) == 1 in the reference, src/gemm.jl:116-117).  beta = 0 never reads C.  Accumulation
   is fp32.  16-bit element types with 16-byte aligned A and B and leading dimensions / batch strides that are
   multiples of 8 elements run on the tensor cores (tcgen05), everything else (Float32 included) on a plain
   CUDA-core kernel. */
typedef struct nnlib_b200_gemm_params {
  size_t struct_size;        /* = sizeof(nnlib_b200_gemm_params) */
  int32_t dtype;             /* NNLIB_B200_F16 / BF16 / F32: element type of A, B and C */
  int32_t transA, transB;    /* 0 = 'N', 1 = 'T' */
  int32_t reserved;
  int64_t M, N, K, batch;
  const void* A;
  int64_t lda, strideA;      /* elements; strideA = 0: A has no batch dimension */
  const void* B;
  int64_t ldb, strideB;
  void* C;
  int64_t ldc, strideC;
  float alpha, beta;
  int32_t* status;           /* optional device int32, as in nnlib_b200_attn_params */
} nnlib_b200_gemm_params;

NNLIB_B200_API int nnlib_b200_batched_gemm(const nnlib_b200_gemm_params* p, void* stream);
/* NNLIB_B200_PATH_* that batched_gemm would take for p, or a negative error */
NNLIB_B200_API int nnlib_b200_batched_gemm_path(const nnlib_b200_gemm_params* p);

/* make_causal_mask (src/attention.jl:149-153): fill an (L, L) byte matrix
   with m[i + L*j] = (i <= j). */
NNLIB_B200_API int nnlib_b200_causal_fill(uint8_t* mask, int64_t L, void* stream);

/* *flag (device int32) := 1 if the (L, L) byte matrix equals make_causal_mask's
   result, else 0.  Lets the caller swap a materialised causal mask for the
   `causal` flag. */
NNLIB_B200_API int nnlib_b200_causal_check(const uint8_t* mask, int64_t L, int32_t* flag, void* stream);

/* NNLIB_B200_PATH_* that attn_fwd would take for p, or a negative error. */
NNLIB_B200_API int nnlib_b200_attn_path(const nnlib_b200_attn_params* p);

/* Synchronises `stream`, then returns NNLIB_B200_TIMEOUT if a kernel of this
   library gave up on one of its bounded waits on the current device since the
   previous call (the flag is cleared), else NNLIB_B200_OK.  Meant for tests
   and for callers that want to turn a silent abort into an error. */
NNLIB_B200_API int nnlib_b200_device_health(void* stream);

/* Self-test of the fail-stop path: enqueues one thread block that waits, with the very wait every
   tensor-core kernel here uses, on a barrier nobody arrives at.  After limit_ns (1 .. 10^9) the wait
   gives up and the kernel returns by itself: the device is marked as described at the top of this file
   and *status (optional device int32) is set to NNLIB_B200_TIMEOUT.  Nothing faults or hangs.  Call
   nnlib_b200_device_health afterwards to clear the mark.  No counterpart in the reference. */
NNLIB_B200_API int nnlib_b200_selftest_wait_runout(uint64_t limit_ns, int32_t* status, void* stream);

NNLIB_B200_API const char* nnlib_b200_strerror(int code);
NNLIB_B200_API int nnlib_b200_version(void);
/* the cudaError_t of the last failed CUDA call on this thread (0 if none) */
NNLIB_B200_API int nnlib_b200_last_cuda_error(void);
/* number of kernels this library has launched since it was loaded */
NNLIB_B200_API uint64_t nnlib_b200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* NNLIB_B200_H_ */
