"""``torch.library`` registration of the FP4 attention operator, so that ``torch.compile`` (and any other
fake-tensor tracing) can carry it as one opaque node instead of tracing into the ctypes calls.

The reference registers its INT8 kernels this way (``sageattention/sm89_compile.py:5-23`` custom ops,
``:69-101`` fake implementations); its FP4 path has no such registration.  Here the whole operator
(smoothing, quantisation, attention) is one op with a shape-only fake; it launches exactly the kernels
``sageattn3_blackwell`` / ``sageattn4_blackwell`` launch and nothing else.
"""
from __future__ import annotations

import torch

from . import api


@torch.library.custom_op("sageattention_b200::fp4_attention", mutates_args=(), device_types="cuda")
def fp4_attention_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tensor_layout: str, is_causal: bool,
                     sm_scale: float, per_block_mean: bool, k_packing: bool) -> torch.Tensor:
    """``sm_scale <= 0`` selects the default ``head_dim ** -0.5``; ``k_packing`` selects the fork's
    K-packing operator (``sageattn4/api.py:250``)."""
    fn = api.sageattn4_blackwell if k_packing else api.sageattn3_blackwell
    return fn(q, k, v, tensor_layout=tensor_layout, is_causal=is_causal,
              sm_scale=sm_scale if sm_scale > 0 else None, per_block_mean=per_block_mean)


@fp4_attention_op.register_fake
def _fp4_attention_fake(q, k, v, tensor_layout, is_causal, sm_scale, per_block_mean, k_packing):
    if tensor_layout not in ("HND", "NHD"):
        raise ValueError(f"unknown tensor_layout {tensor_layout!r}")
    return torch.empty(q.shape, dtype=q.dtype, device=q.device)


def sageattn_compilable(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tensor_layout: str = "HND",
                        is_causal: bool = False, sm_scale: float | None = None, per_block_mean: bool = True,
                        k_packing: bool = False) -> torch.Tensor:
    """``sageattn`` for use inside ``torch.compile``d modules (same arguments, no ``return_lse``)."""
    return fp4_attention_op(q, k, v, tensor_layout, bool(is_causal), float(sm_scale) if sm_scale else 0.0,
                            bool(per_block_mean), bool(k_packing))
