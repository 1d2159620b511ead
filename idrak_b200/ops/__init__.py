"""Operations: the sm_100a kernels behind autograd functions, each with a plain PyTorch CPU statement."""
from .gemm import gemm, gemm_reference, linear
from .rowops import (add, colsum, embedding, gated_activation, gelu, layer_norm, norm_backward, norm_branch,
                     norm_forward,
                     rms_norm, rope, rope_, rope_reference)
from .attention import attention, attention_reference, flash_backward, flash_forward, row_starts_from_spans
from .loss import cross_entropy_logits, softmax_xent_, token_cross_entropy
from .optim import FusedAdamW, FusedSGD

__all__ = [
    "gemm", "gemm_reference", "linear", "add", "colsum", "embedding", "gated_activation", "gelu", "layer_norm",
    "norm_backward", "norm_branch", "norm_forward", "rms_norm", "rope", "rope_", "rope_reference", "attention",
    "attention_reference", "flash_backward", "flash_forward", "row_starts_from_spans", "cross_entropy_logits", "softmax_xent_",
    "token_cross_entropy", "FusedAdamW", "FusedSGD",
]
from .fused import mlp_gated, mlp_gelu, qkv_attention  # noqa: E402

__all__ += ["mlp_gated", "mlp_gelu", "qkv_attention"]
