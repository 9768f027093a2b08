"""Model-side hooks for the FP4 attention operator.

The reference wires its operator into diffusion models in two ways: by swapping
``torch.nn.functional.scaled_dot_product_attention`` for it (``example/cogvideox_infer.py:34-35``,
``example/parallel_sageattn_cogvideo.py:89-95``) and by installing attention processors that call an
``attn_func(query, key, value, attn_mask=..., dropout_p=..., is_causal=...)`` on ``[B, H, N, D]`` tensors
(``example/modify_model/modify_wan.py:8-107`` and its siblings).  Both need the same thing from this package: a
callable with the signature of ``scaled_dot_product_attention``.  The reference also recommends, for models that
do not tolerate FP4 everywhere, a hybrid schedule - a higher-precision attention at the first and last denoising
steps, the FP4 operator for all others (``sageattention3_blackwell/README.md:16-22``).

Nothing here touches tensors: the hooks only choose which attention function is called.
"""
from __future__ import annotations

import contextlib
from typing import Callable, Optional

import torch
import torch.nn.functional as F


def as_sdpa(attn_fn: Optional[Callable] = None, precise_fn: Optional[Callable] = None) -> Callable:
    """A function with the signature of ``torch.nn.functional.scaled_dot_product_attention`` that runs ``attn_fn``
    (default :func:`sageattention_b200.sageattn`) on ``[B, H, N, D]`` tensors.

    What the FP4 operator cannot express goes to ``precise_fn`` (default: the original PyTorch function) exactly as
    the reference's operator hands unsupported cases to SDPA (``sageattn4/api.py:253-255``): an ``attn_mask``,
    dropout, head dims above 128, inputs that are not bf16 CUDA tensors."""
    if attn_fn is None:
        from .api import sageattn as attn_fn
    fallback = precise_fn or _ORIGINAL_SDPA

    def sdpa(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, enable_gqa=False, **kw):
        usable = (attn_mask is None and dropout_p == 0.0 and query.dim() == 4 and query.is_cuda
                  and query.dtype == torch.bfloat16 and query.shape[-1] <= 128
                  and query.shape[1] % key.shape[1] == 0 and (enable_gqa or query.shape[1] == key.shape[1]))
        if not usable:
            return fallback(query, key, value, attn_mask=attn_mask, dropout_p=dropout_p, is_causal=is_causal,
                            scale=scale, **({"enable_gqa": True} if enable_gqa else {}))
        return attn_fn(query, key, value, tensor_layout="HND", is_causal=is_causal, sm_scale=scale)

    return sdpa


_ORIGINAL_SDPA = F.scaled_dot_product_attention


@contextlib.contextmanager
def patched_sdpa(sdpa_fn: Optional[Callable] = None):
    """Swap ``torch.nn.functional.scaled_dot_product_attention`` for ``sdpa_fn`` (default :func:`as_sdpa`) inside the
    ``with`` block - the reference's monkey patch (``example/cogvideox_infer.py:34-35``), undone on exit."""
    fn = sdpa_fn or as_sdpa()
    saved = F.scaled_dot_product_attention
    F.scaled_dot_product_attention = fn
    try:
        yield fn
    finally:
        F.scaled_dot_product_attention = saved


class TimestepHybridAttention:
    """The reference's hybrid schedule (``sageattention3_blackwell/README.md:16-22``): ``precise_fn`` at the first
    ``first`` and last ``last`` of ``num_steps`` denoising steps, ``fast_fn`` at all others.  Both take the
    ``scaled_dot_product_attention`` arguments.  The sampler loop calls :meth:`set_step` (or :meth:`next_step`) once
    per denoising step; the object itself is what gets installed as the model's attention function."""

    def __init__(self, num_steps: int, fast_fn: Optional[Callable] = None, precise_fn: Optional[Callable] = None,
                 first: int = 1, last: int = 1):
        if num_steps < 1 or first < 0 or last < 0:
            raise ValueError("num_steps must be positive, first / last non-negative")
        self.num_steps, self.first, self.last = int(num_steps), int(first), int(last)
        self.fast_fn = fast_fn or as_sdpa()
        self.precise_fn = precise_fn or _ORIGINAL_SDPA
        self.step = 0
        self.calls = {"fast": 0, "precise": 0}

    def set_step(self, step: int) -> None:
        self.step = int(step)

    def next_step(self) -> None:
        self.step += 1

    def uses_precise(self, step: Optional[int] = None) -> bool:
        s = self.step if step is None else step
        return s < self.first or s >= self.num_steps - self.last

    def __call__(self, query, key, value, *args, **kwargs):
        if self.uses_precise():
            self.calls["precise"] += 1
            return self.precise_fn(query, key, value, *args, **kwargs)
        self.calls["fast"] += 1
        return self.fast_fn(query, key, value, *args, **kwargs)


def set_attn_func(model: torch.nn.Module, attn_func: Callable, attribute: str = "attn_func") -> int:
    """Point every attention processor of ``model`` that carries an ``attn_func`` attribute (the reference's
    ``Sage*AttnProcessor`` classes, ``example/modify_model/modify_wan.py:8-11``) at ``attn_func``.  Returns how many
    processors were updated."""
    n = 0
    for module in model.modules():
        proc = getattr(module, "processor", None)
        if proc is not None and hasattr(proc, attribute):
            setattr(proc, attribute, attn_func)
            n += 1
    return n
