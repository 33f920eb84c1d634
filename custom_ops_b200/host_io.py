"""``mha_fwd_with_mask`` for operands that live in host memory.

The reference operator takes device tensors (``__init__.py:mha_fwd_with_mask`` ->
``csrc/fa/fa_fwd_op.cu:46``); a caller whose Q, K, V and mask sit in (pinned) host memory pays
the PCIe copies around it, and for the benchmark shapes those copies are 15-20x the kernel
time.  Batch elements are independent, so this helper runs them as a three-stage pipeline on
three streams - host->device copy of element b+1, attention of element b, device->host copy of
element b-1 - and the two DMA directions and the kernel overlap.  The attention itself is the
unchanged public operator.
"""
from __future__ import annotations

from typing import Optional

import torch

__all__ = ["mha_fwd_with_mask_from_host"]


class _Streams:
    """Side streams per device, created once."""
    _by_device: dict = {}

    @classmethod
    def get(cls, device: torch.device):
        key = (device.type, device.index)
        if key not in cls._by_device:
            cls._by_device[key] = (torch.cuda.Stream(device), torch.cuda.Stream(device),
                                   torch.cuda.Stream(device))
        return cls._by_device[key]


def mha_fwd_with_mask_from_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor,
                                out: Optional[torch.Tensor] = None, *, device=None,
                                batch_chunk: int = 1) -> torch.Tensor:
    """q (B,H,Sq,d), k/v (B,Hk,Sk,d), mask (B,1,>=Sq,>=Sk): CPU tensors, pinned for the copies
    to be asynchronous.  Returns ``out`` (B,H,Sq,d) in host memory (pinned when allocated here).

    The work is enqueued behind the current stream of ``device`` and the current stream waits
    for it: after the call, synchronising the current stream makes ``out`` valid, exactly as
    for a non-blocking device->host copy.
    """
    from . import ops

    if q.is_cuda or k.is_cuda or v.is_cuda or mask.is_cuda:
        raise ValueError("mha_fwd_with_mask_from_host takes host tensors; use ops.mha_fwd_with_mask")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4 or mask.dim() != 4:
        raise ValueError("q, k, v and mask must be 4-D")
    B = q.shape[0]
    if k.shape[0] != B or v.shape[0] != B or mask.shape[0] != B:
        raise ValueError("q, k, v and mask must have the same batch size")
    if out is not None and (out.is_cuda or out.shape != q.shape or out.dtype != q.dtype):
        raise ValueError("out must be a host tensor of q's shape and dtype")
    if not torch.cuda.is_available():
        raise RuntimeError("mha_fwd_with_mask_from_host needs a CUDA device: there is no CPU path")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype, pin_memory=True)
    batch_chunk = max(1, int(batch_chunk))

    s_in, s_run, s_out = _Streams.get(device)
    current = torch.cuda.current_stream(device)
    fork = torch.cuda.Event()
    fork.record(current)
    for s in (s_in, s_run, s_out):
        s.wait_event(fork)

    keep = []                                   # device tensors stay referenced until the join
    for b0 in range(0, B, batch_chunk):
        b1 = min(B, b0 + batch_chunk)
        with torch.cuda.stream(s_in):
            qd = q[b0:b1].to(device, non_blocking=True)
            kd = k[b0:b1].to(device, non_blocking=True)
            vd = v[b0:b1].to(device, non_blocking=True)
            md = mask[b0:b1].to(device, non_blocking=True)
            copied = torch.cuda.Event()
            copied.record(s_in)
        with torch.cuda.stream(s_run):
            s_run.wait_event(copied)
            od = ops.mha_fwd_with_mask(qd, kd, vd, md)
            done = torch.cuda.Event()
            done.record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            out[b0:b1].copy_(od, non_blocking=True)
        for t in (qd, kd, vd, md):
            t.record_stream(s_run)
        od.record_stream(s_out)
        keep.append((qd, kd, vd, md, od))

    for s in (s_in, s_run, s_out):
        join = torch.cuda.Event()
        join.record(s)
        current.wait_event(join)
    return out
