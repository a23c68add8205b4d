"""Hand-written sm_100a kernels (tcgen05 GEMM/attention, RMSNorm, RoPE, SwiGLU,
cross-entropy, AdamW, NVLink collectives) and their PyTorch-facing wrappers."""
from . import kernels, reference  # noqa: F401
from .functional import *  # noqa: F401,F403
from .functional import (adamw_, attention_bwd, attention_fwd, cross_entropy_, embedding_bwd_,
                         embedding_fwd, gemm, rmsnorm_bwd, rmsnorm_fwd, rope_, sumsq, swiglu_bwd,
                         swiglu_fwd)
