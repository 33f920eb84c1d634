"""Additive masks from rules, written on the device at a pitch the forward reads in place.

Callers of the reference build the ``(B, 1, Sq, Sk)`` mask with a handful of tensor operations
(``examples/custom_mask_demo.py:33-65``: causal, sliding window, padding), and when ``Sk`` is not
a multiple of 8 the operator then copies it to an aligned pitch on every call
(``csrc/fa/fa_fwd_op.cu:117-138``).  ``rule_mask`` is one kernel launch
(``fa_mask_build_sm100``) that writes the mask directly with rows padded to a multiple of 8
elements: pass the result to ``ops.mha_fwd_with_mask`` as it is - columns beyond ``Sk`` are
ignored by the operator - and no re-pitch copy runs.

``rule_attention`` goes one step further: the same rules evaluated inside the attention kernel
(``fa_mask_fwd_sm100_rule``), so that no mask exists in memory at all - no mask traffic, no
tile-skip pre-pass (the visible key range of a unit follows from the rule), no mask add on the
blocks a row sees entirely.  Bit-identical to ``ops.mha_fwd_with_mask(q, k, v, rule_mask(...))``.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _cabi

__all__ = ["rule_mask", "rule_attention"]


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


def rule_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = False, window: int = 0,
                   valid_lens: Optional[torch.Tensor] = None, return_lse: bool = False):
    """Attention forward of q ``(B, H, Sq, d)`` over k, v ``(B, Hk, Sk, d)`` under the mask that
    ``rule_mask(B, Sq, Sk, causal=..., window=..., valid_lens=...)`` would describe, without
    building it.  Returns ``out`` (and the fp32 ``(B, H, Sq)`` natural-log LSE with ``return_lse``).
    A row that sees no key gives 0 (LSE -inf)."""
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("rule_attention is only supported on CUDA")
    if q.dtype not in (torch.bfloat16, torch.float16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("q, k, v must share one dtype, float16 or bfloat16")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4 or k.shape != v.shape:
        raise ValueError("q must be (B, H, Sq, d), k and v (B, Hk, Sk, d)")
    if not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()):
        raise ValueError("q, k, v must be contiguous")
    B, H, Sq, d = q.shape
    Hk, Sk = k.shape[1], k.shape[2]
    if k.shape[0] != B or k.shape[3] != d or Hk <= 0 or H % Hk != 0 or d not in (64, 128) or window < 0:
        raise ValueError("shape mismatch: batch, head_dim (64 or 128), H % Hk == 0, window >= 0")
    if k.device != q.device or v.device != q.device:
        raise ValueError("q, k, v must be on the same device")
    lens_ptr = 0
    if valid_lens is not None:
        if valid_lens.numel() != B:
            raise ValueError("valid_lens must hold one length per batch element")
        valid_lens = valid_lens.to(device=q.device, dtype=torch.int32).contiguous()
        lens_ptr = valid_lens.data_ptr()
    out = torch.empty_like(q)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device) if return_lse else None
    args = _cabi.make_args(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), mask=0, out=out.data_ptr(),
                           lse=lse.data_ptr() if return_lse else 0, batch=B, heads=H, heads_k=Hk, seqlen_q=Sq,
                           seqlen_k=Sk, head_dim=d, dtype=_cabi.BF16 if q.dtype == torch.bfloat16 else _cabi.FP16,
                           device=q.device.index)
    stream = torch.cuda.current_stream(q.device)
    # the counter the CTAs take their units from (any content; private to this call)
    ws = torch.empty(_cabi.RULE_WORKSPACE_BYTES, dtype=torch.uint8, device=q.device)
    _cabi.forward_rule(args, int(bool(causal)), int(window), lens_ptr, stream.cuda_stream, ws.data_ptr(),
                       _cabi.RULE_WORKSPACE_BYTES)
    if valid_lens is not None:
        valid_lens.record_stream(stream)
    return (out, lse) if return_lse else out
