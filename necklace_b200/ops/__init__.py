"""Operators: hand-written sm_100a kernels with PyTorch fp32 reference paths for CPU."""
from .gemm import gemm, linear, mlp, colsum, Linear, EPI_NONE, EPI_GELU_FWD, EPI_GELU_BWD, EPI_RELU
from .norm import LayerNorm, RMSNorm, norm_fwd, norm_bwd
from .loss import cross_entropy_fwd_bwd, lm_head_loss, Embedding, embed_fwd, embed_bwd
from .optim import adam_step, sgd_step, scale_cast, sumsq
from .quant import (quantize_flat, dequantize_flat, matrix_quantize, matrix_dequantize)
from .attention import attention_qkv, attn_fwd, attn_bwd
from ._common import check_status
