"""Multi-GPU use of ``mha_fwd_with_mask`` on one box: one process per GPU,
``torch.distributed`` for the plumbing.  The reference has no distributed code at
all; this is new work on top of the single-GPU operator.

Two ways to spread the operator:

* **(batch, kv-head) sharding** -- every (batch, head) pair is independent, so the
  work is cut into ``B * Hk`` units (all query heads of one KV group stay together
  so K/V are never duplicated) and each rank takes a contiguous range.  No
  collective touches the data path.  :func:`shard_units` / :func:`shard_inputs`.

* **cross-GPU Split-KV** for the small-grid long-context shape: rank ``g`` owns keys
  ``[g*Sk/G, (g+1)*Sk/G)`` of every head (slice boundaries are multiples of the
  128-key block), runs the local forward with fp32 output and LSE, the partials are
  all-gathered over NCCL (about 1 MB per rank: latency-bound on NVLink) and merged
  by the same log-sum-exp kernel the single-GPU Split-KV uses
  (``fa_mask_fwd_sm100_combine``).  Data always lands in local HBM through NCCL
  before a kernel touches it.  :func:`splitkv_forward`.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch

KV_BLOCK = 128


def shard_units(B: int, Hk: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous range [lo, hi) of the ``B*Hk`` (batch, kv-head) units for ``rank``.
    Ranges differ in size by at most one unit and cover everything exactly once."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    units = B * Hk
    base, extra = divmod(units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def units_to_slices(lo: int, hi: int, Hk: int) -> List[Tuple[int, int, int]]:
    """Break a unit range into per-batch pieces ``(b, hk_lo, hk_hi)``."""
    out = []
    u = lo
    while u < hi:
        b, hk = divmod(u, Hk)
        take = min(hi - u, Hk - hk)
        out.append((b, hk, hk + take))
        u += take
    return out


def shard_inputs(q, k, v, mask, world: int, rank: int):
    """This rank's independent sub-problems: a list of ``(q, k, v, mask)`` with batch 1,
    covering its (batch, kv-head) units.  The mask has no head dimension, so a rank
    needs only the mask slices of the batches it touches."""
    B, H = q.shape[0], q.shape[1]
    Hk = k.shape[1]
    g = H // Hk
    lo, hi = shard_units(B, Hk, world, rank)
    pieces = []
    for b, h0, h1 in units_to_slices(lo, hi, Hk):
        pieces.append((q[b:b + 1, h0 * g:h1 * g].contiguous(), k[b:b + 1, h0:h1].contiguous(),
                       v[b:b + 1, h0:h1].contiguous(), mask[b:b + 1].contiguous()))
    return pieces


def kv_slice_bounds(Sk: int, world: int, rank: int) -> Tuple[int, int]:
    """Key range of ``rank`` for the cross-GPU Split-KV: whole 128-key blocks, spread
    evenly, the ragged tail going to the last rank that owns any keys.  A rank may get
    an empty range when there are fewer blocks than ranks."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    blocks = (Sk + KV_BLOCK - 1) // KV_BLOCK
    base, extra = divmod(blocks, world)
    b_lo = rank * base + min(rank, extra)
    b_hi = b_lo + base + (1 if rank < extra else 0)
    return min(b_lo * KV_BLOCK, Sk), min(b_hi * KV_BLOCK, Sk)


def _local_partial_cuda(q, k, v, mask):
    """fp32 normalised output and natural-log LSE of the local key slice (C ABI)."""
    from . import _cabi

    B, H, Sq, d = q.shape
    out = torch.empty((B, H, Sq, d), device=q.device, dtype=torch.float32)
    lse = torch.empty((B, H, Sq), device=q.device, dtype=torch.float32)
    args = _cabi.make_args(
        q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), mask=mask.data_ptr(), out=out.data_ptr(),
        lse=lse.data_ptr(), batch=B, heads=H, heads_k=k.shape[1], seqlen_q=Sq,
        seqlen_k=k.shape[2], head_dim=d,
        dtype=_cabi.BF16 if q.dtype == torch.bfloat16 else _cabi.FP16,
        mask_seqlen_q=mask.shape[2], mask_seqlen_k=mask.shape[3],
        mask_batch_stride=mask.stride(0), mask_row_stride=mask.stride(2),
        device=q.device.index or 0, out_fp32=1)
    nbytes = _cabi.workspace_bytes(args)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device)
    _cabi.forward(args, ws.data_ptr(), nbytes, torch.cuda.current_stream(q.device).cuda_stream)
    return out, lse, ws


def _combine_cuda(o_parts, lse_parts, dtype):
    """(G, rows, d) fp32 partials + (G, rows) LSE -> (rows, d) in ``dtype``."""
    from . import _cabi

    G, rows, d = o_parts.shape
    out = torch.empty((rows, d), device=o_parts.device, dtype=dtype)
    _cabi.combine(o_parts.data_ptr(), lse_parts.data_ptr(), out.data_ptr(), 0, G, rows, d,
                  _cabi.BF16 if dtype == torch.bfloat16 else _cabi.FP16, 0,
                  o_parts.device.index or 0,
                  torch.cuda.current_stream(o_parts.device).cuda_stream)
    return out


def splitkv_forward(q, k_local, v_local, mask_local, group=None, *,
                    local_fn: Optional[Callable] = None, combine_fn: Optional[Callable] = None):
    """Cross-GPU Split-KV.  ``q`` is replicated; ``k_local``/``v_local``/``mask_local`` hold
    this rank's key slice (see :func:`kv_slice_bounds`), possibly empty.  Every rank
    returns the full result ``(B, H, Sq, d)`` in q's dtype.

    ``local_fn`` / ``combine_fn`` replace the CUDA entry points in host-logic tests
    that run on CPU ranks; production callers leave them unset.
    """
    import torch.distributed as dist

    world = dist.get_world_size(group)
    B, H, Sq, d = q.shape
    local_fn = local_fn or _local_partial_cuda
    combine_fn = combine_fn or _combine_cuda
    keep = None
    if k_local.shape[2] > 0:
        res = local_fn(q, k_local, v_local, mask_local)
        o_loc, lse_loc = res[0], res[1]
        keep = res[2:] if len(res) > 2 else None      # scratch stays alive until the stream is done
    else:
        o_loc = torch.zeros((B, H, Sq, d), device=q.device, dtype=torch.float32)
        lse_loc = torch.full((B, H, Sq), float("-inf"), device=q.device, dtype=torch.float32)
    rows = B * H * Sq
    # one packed buffer per rank: [O (rows*d) | LSE (rows)] -> a single all_gather
    packed = torch.cat([o_loc.reshape(-1), lse_loc.reshape(-1)])
    flat = torch.empty(world * packed.numel(), device=q.device, dtype=torch.float32)
    dist.all_gather_into_tensor(flat, packed, group=group)      # rank-major
    gathered = flat.view(world, packed.numel())
    o_parts = gathered[:, :rows * d].reshape(world, rows, d).contiguous()
    lse_parts = gathered[:, rows * d:].reshape(world, rows).contiguous()
    out = combine_fn(o_parts, lse_parts, q.dtype)
    del keep
    return out.reshape(B, H, Sq, d)
