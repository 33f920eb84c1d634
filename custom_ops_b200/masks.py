"""Additive masks from rules, written on the device at a pitch the forward reads in place.

Callers of the reference build the ``(B, 1, Sq, Sk)`` mask with a handful of tensor operations
(``examples/custom_mask_demo.py:33-65``: causal, sliding window, padding), and when ``Sk`` is not
a multiple of 8 the operator then copies it to an aligned pitch on every call
(``csrc/fa/fa_fwd_op.cu:117-138``).  ``rule_mask`` is one kernel launch
(``fa_mask_build_sm100``) that writes the mask directly with rows padded to a multiple of 8
elements: pass the result to ``ops.mha_fwd_with_mask`` as it is - columns beyond ``Sk`` are
ignored by the operator - and no re-pitch copy runs.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _cabi

__all__ = ["rule_mask"]


def rule_mask(batch: int, seqlen_q: int, seqlen_k: int, *, dtype: torch.dtype = torch.bfloat16,
              causal: bool = False, window: int = 0, valid_lens: Optional[torch.Tensor] = None,
              device=None, pad_to: int = 8) -> torch.Tensor:
    """Returns ``(batch, 1, seqlen_q, pitch)`` with ``pitch = ceil(seqlen_k / pad_to) * pad_to``:
    0 where key j is visible to query i, -inf elsewhere (and in the pad columns).

    visible  <=>  j < seqlen_k  and  j < valid_lens[b]  (if given)
                  and  j <= i + seqlen_k - seqlen_q      (if ``causal``; right-aligned)
                  and  j >  i + seqlen_k - seqlen_q - window   (if ``window`` > 0)
    """
    if dtype not in (torch.bfloat16, torch.float16):
        raise ValueError("mask dtype must be torch.bfloat16 or torch.float16")
    if batch < 0 or seqlen_q < 0 or seqlen_k < 0 or pad_to < 1 or window < 0:
        raise ValueError("batch, seqlen_q, seqlen_k and window must be >= 0 and pad_to >= 1")
    if not torch.cuda.is_available():
        raise RuntimeError("rule_mask writes the mask with a CUDA kernel: there is no CPU path")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    lens_ptr = 0
    if valid_lens is not None:
        if valid_lens.numel() != batch:
            raise ValueError("valid_lens must hold one length per batch element")
        valid_lens = valid_lens.to(device=device, dtype=torch.int32).contiguous()
        lens_ptr = valid_lens.data_ptr()
    pitch = -(-seqlen_k // pad_to) * pad_to
    mask = torch.empty((batch, 1, seqlen_q, pitch), dtype=dtype, device=device)
    stream = torch.cuda.current_stream(device).cuda_stream
    _cabi.build_mask(mask.data_ptr(), batch, seqlen_q, seqlen_k, pitch,
                     _cabi.BF16 if dtype == torch.bfloat16 else _cabi.FP16, int(bool(causal)), int(window),
                     lens_ptr, device.index, stream)
    if valid_lens is not None:
        valid_lens.record_stream(torch.cuda.current_stream(device))
    return mask
