"""B200-native multi-head attention behind NNlib.jl's API.

``dot_product_attention``, ``dot_product_attention_scores`` and
``make_causal_mask`` (NNlib.jl ``src/attention.jl``) for column-major CUDA
tensors, computed by the hand-written sm_100a kernels of ``libnnlib_b200.so``
(``csrc/``; C ABI in ``include/nnlib_b200.h``).  ``shard`` spreads the
independent (batch, head) units of one call over the GPUs of a box.
"""
from .attention import (ArgumentError, CausalMask, LazyAttnScores, PhiloxDropout, check_status, device_health,
                        dot_product_attention, dot_product_attention_pullback, dot_product_attention_scores, identity,
                        make_causal_mask, math_mode, scores_mode, set_math_mode, set_scores_mode)
from . import batched  # batched_mul / batched_mul! on the library's strided-batched product
from .batched import batched_adjoint, batched_mul, batched_mul_, batched_transpose
from . import softmax  # softmax / logsoftmax and pullbacks: nnlib_jl_b200.softmax.softmax(x, dims=...)
from .hostio import HostPipelinedAttention
from .layout import (as_column_major, is_column_major, jl_empty, jl_from_numpy, jl_reshape, jl_to_numpy,
                     jl_zeros)

__all__ = [
    "ArgumentError", "CausalMask", "HostPipelinedAttention", "LazyAttnScores", "PhiloxDropout", "check_status", "device_health",
    "dot_product_attention", "dot_product_attention_pullback", "dot_product_attention_scores", "identity", "make_causal_mask", "math_mode", "scores_mode", "set_math_mode", "set_scores_mode",
    "batched_adjoint", "batched_mul", "batched_mul_", "batched_transpose",
    "as_column_major", "is_column_major", "jl_empty", "jl_from_numpy", "jl_reshape", "jl_to_numpy", "jl_zeros",
]
