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
  128-key block), runs the local forward with fp32 output and LSE into its packed part
  (about 1 MB per rank), and the parts are merged by the same log-sum-exp kernel the
  single-GPU Split-KV uses.  Two ways to exchange the parts (:func:`splitkv_forward`):

  - ``exchange="peer"``: the parts live in symmetric (peer-addressable) memory; the merge
    kernel itself signals the other ranks, waits -- bounded -- for their parts and reads
    them straight over NVLink with plain loads.  One kernel does the exchange and the
    merge; no collective library call sits on the path (a 1 MB NCCL all-gather costs
    about 20 us of latency, more than a rank's share of the attention itself).
  - ``exchange="nccl"``: one ``all_gather_into_tensor`` of the parts, then the merge on
    local memory.  The fallback where symmetric memory cannot be set up.

  No TMA load and no multicast ever touches another GPU's memory.
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
    """This rank's independent sub-problems: a list of ``(q, k, v, mask)`` covering its
    (batch, kv-head) units.  Batch elements of which the rank owns every head stay together
    as one sub-problem (a contiguous view, nothing is copied); a batch element it shares with
    another rank gives a sub-problem of batch 1 with its heads.  The mask has no head
    dimension, so a rank needs only the mask slices of the batches it touches."""
    B, H = q.shape[0], q.shape[1]
    Hk = k.shape[1]
    g = H // Hk
    lo, hi = shard_units(B, Hk, world, rank)
    pieces = []
    run = None            # consecutive batch elements of which this rank owns every head: one launch
    for b, h0, h1 in units_to_slices(lo, hi, Hk):
        if h0 == 0 and h1 == Hk:
            run = (run[0], b + 1) if run is not None and run[1] == b else (b, b + 1)
            if run[0] != b:
                pieces.pop()
            pieces.append((q[run[0]:run[1]], k[run[0]:run[1]], v[run[0]:run[1]], mask[run[0]:run[1]]))
            continue
        run = None
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


class _SplitKVScratch:
    """Buffers of the cross-GPU Split-KV, kept between calls per (device, rows, d, world) so the
    steady state allocates nothing: this rank's packed part ``[O (rows*d) | LSE (rows)]``, the
    gathered parts of all ranks, and the forward's workspace."""

    _cache: dict = {}

    def __init__(self, device, rows: int, d: int, world: int):
        # parts are padded to a multiple of 4 floats so that every part starts 16-byte aligned
        self.part_floats = (rows * (d + 1) + 3) // 4 * 4
        self.part = torch.empty(self.part_floats, device=device, dtype=torch.float32)
        self.gathered = torch.empty(world * self.part_floats, device=device, dtype=torch.float32)
        self.workspace = None

    @classmethod
    def get(cls, device, rows: int, d: int, world: int) -> "_SplitKVScratch":
        key = (device.type, device.index, rows, d, world)
        if key not in cls._cache:
            if len(cls._cache) >= 8:
                cls._cache.clear()
            cls._cache[key] = cls(device, rows, d, world)
        return cls._cache[key]

    def workspace_for(self, nbytes: int, device):
        if self.workspace is None or self.workspace.numel() < max(nbytes, 16):
            self.workspace = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=device)
        return self.workspace


class _PeerScratch:
    """Symmetric-memory buffers of the peer exchange, one set per (device, rows, d, group):
    two part slots (calls alternate, so a rank that is one call ahead never overwrites a part
    another rank still reads), then ``world`` flag words.  Set up collectively on first use."""

    _cache: dict = {}

    def __init__(self, device, rows: int, d: int, group):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        world = dist.get_world_size(group)
        self.part_floats = (rows * (d + 1) + 3) // 4 * 4
        self.flag_offset = 2 * self.part_floats
        total = self.flag_offset + max(64, world)
        self.buf = symm_mem.empty(total, dtype=torch.float32, device=device)
        self.buf.zero_()
        group_name = (group or dist.group.WORLD).group_name
        self.handle = symm_mem.rendezvous(self.buf, group_name)
        torch.cuda.synchronize(device)
        dist.barrier(group)                  # every rank's flags are zero before anyone signals
        self.table = int(self.handle.buffer_ptrs_dev)     # device array of the ranks' buffer bases
        self.rank = dist.get_rank(group)
        self.world = world
        self.seq = 0
        self.workspace = None

    @classmethod
    def get(cls, device, rows: int, d: int, group) -> "_PeerScratch":
        key = (device.type, device.index, rows, d, id(group))
        if key not in cls._cache:
            cls._cache[key] = cls(device, rows, d, group)
        return cls._cache[key]

    def workspace_for(self, nbytes: int, device):
        if self.workspace is None or self.workspace.numel() < max(nbytes, 16):
            self.workspace = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=device)
        return self.workspace


_PEER_FAILED = ""          # why the peer exchange could not be set up in this process (then: NCCL)


class _SetupError(RuntimeError):
    pass


def peer_exchange_available() -> bool:
    """Whether torch offers symmetric memory here (the set-up itself may still fail on
    hardware without peer access; :func:`splitkv_forward` then falls back to NCCL)."""
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
        return torch.cuda.is_available()
    except Exception:  # noqa: BLE001
        return False


def _check_operands(q, k, v, mask):
    """The C ABI addresses q, k and v as contiguous (B, H, S, d) tensors; only the mask carries
    strides.  A sliced view (``k[:, :, lo:hi]``) would silently be read as something else."""
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous (call .contiguous() on a sliced view)")
    for name, t in (("k", k), ("v", v), ("mask", mask)):
        if t.dtype != q.dtype or t.device != q.device:
            raise ValueError(f"{name} must have q's dtype and device")
    if mask.dim() != 4 or mask.stride(3) != 1:
        raise ValueError("mask must be (B, 1, Sq_m, Sk_m) with unit stride along the keys")


def _local_partial_cuda(q, k, v, mask, part: torch.Tensor, scratch: "_SplitKVScratch"):
    """Normalised fp32 output and natural-log LSE of the local key slice, written straight into
    ``part`` = [O (rows*d) | LSE (rows)] (C ABI, out_fp32 = 1)."""
    from . import _cabi

    _check_operands(q, k, v, mask)
    B, H, Sq, d = q.shape
    rows = B * H * Sq
    args = _cabi.make_args(
        q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), mask=mask.data_ptr(), out=part.data_ptr(),
        lse=part.data_ptr() + 4 * rows * d, batch=B, heads=H, heads_k=k.shape[1], seqlen_q=Sq,
        seqlen_k=k.shape[2], head_dim=d,
        dtype=_cabi.BF16 if q.dtype == torch.bfloat16 else _cabi.FP16,
        mask_seqlen_q=mask.shape[2], mask_seqlen_k=mask.shape[3],
        mask_batch_stride=mask.stride(0), mask_row_stride=mask.stride(2),
        device=q.device.index or 0, out_fp32=1)
    nbytes = _cabi.workspace_bytes(args)
    ws = scratch.workspace_for(nbytes, q.device)
    _cabi.forward(args, ws.data_ptr(), nbytes, torch.cuda.current_stream(q.device).cuda_stream)


def _combine_cuda(gathered: torch.Tensor, part_floats: int, world: int, rows: int, d: int, dtype):
    """``world`` packed parts -> (rows, d) in ``dtype``."""
    from . import _cabi

    out = torch.empty((rows, d), device=gathered.device, dtype=dtype)
    _cabi.combine_packed(gathered.data_ptr(), part_floats, out.data_ptr(), 0, world, rows, d,
                         _cabi.BF16 if dtype == torch.bfloat16 else _cabi.FP16, 0,
                         gathered.device.index or 0,
                         torch.cuda.current_stream(gathered.device).cuda_stream)
    return out


def _splitkv_forward_peer(q, k_local, v_local, mask_local, group):
    from . import _cabi

    B, H, Sq, d = q.shape
    rows = B * H * Sq
    sc = _PeerScratch.get(q.device, rows, d, group)
    sc.seq += 1
    slot = sc.seq & 1
    part = sc.buf[slot * sc.part_floats:(slot + 1) * sc.part_floats]
    if k_local.shape[2] > 0:
        _local_partial_cuda(q, k_local, v_local, mask_local, part, sc)
    else:
        part[:rows * d].zero_()
        part[rows * d:rows * (d + 1)].fill_(float("-inf"))
    out = torch.empty((rows, d), device=q.device, dtype=q.dtype)
    _cabi.combine_peers(sc.table, slot * sc.part_floats, sc.flag_offset, sc.rank, sc.world, sc.seq,
                        out.data_ptr(), 0, rows, d,
                        _cabi.BF16 if q.dtype == torch.bfloat16 else _cabi.FP16, 0,
                        q.device.index or 0, torch.cuda.current_stream(q.device).cuda_stream)
    return out.reshape(B, H, Sq, d)


def splitkv_forward(q, k_local, v_local, mask_local, group=None, *, exchange: str = "auto",
                    local_fn: Optional[Callable] = None, combine_fn: Optional[Callable] = None):
    """Cross-GPU Split-KV.  ``q`` is replicated; ``k_local``/``v_local``/``mask_local`` hold
    this rank's key slice (see :func:`kv_slice_bounds`), possibly empty.  Every rank
    returns the full result ``(B, H, Sq, d)`` in q's dtype.

    Per call: one forward that writes its fp32 result and LSE straight into this rank's packed
    part, then either the merge kernel with the exchange built in (``exchange="peer"``, the
    default where symmetric memory is available: parts in peer-addressable memory, read over
    NVLink by the merge itself) or one ``all_gather_into_tensor`` of the parts and the merge on
    local memory (``exchange="nccl"``).  Nothing is concatenated, copied or allocated in the
    steady state (the buffers are kept per shape).  Every rank must make the same sequence of
    calls.

    ``local_fn(q, k, v, mask) -> (O fp32, LSE)`` / ``combine_fn(o_parts, lse_parts, dtype)``
    replace the CUDA entry points in host-logic tests that run on CPU ranks; production
    callers leave them unset.
    """
    import torch.distributed as dist

    if exchange not in ("auto", "peer", "nccl"):
        raise ValueError("exchange must be 'auto', 'peer' or 'nccl'")
    if local_fn is None and combine_fn is None and q.is_cuda and exchange != "nccl":
        global _PEER_FAILED
        if exchange == "peer" or (peer_exchange_available() and not _PEER_FAILED):
            try:
                return _splitkv_forward_peer(q, k_local, v_local, mask_local, group)
            except _SetupError:
                raise
            except (RuntimeError, AttributeError) as e:
                # only the collective set-up may fail softly, and it fails on every rank alike
                if exchange == "peer" or _PeerScratch._cache:
                    raise
                _PEER_FAILED = str(e)
    world = dist.get_world_size(group)
    B, H, Sq, d = q.shape
    rows = B * H * Sq
    scratch = _SplitKVScratch.get(q.device, rows, d, world)
    part, pf = scratch.part, scratch.part_floats
    if k_local.shape[2] > 0:
        if local_fn is None:
            _local_partial_cuda(q, k_local, v_local, mask_local, part, scratch)
        else:
            o_loc, lse_loc = local_fn(q, k_local, v_local, mask_local)[:2]
            part[:rows * d].copy_(o_loc.reshape(-1))
            part[rows * d:rows * (d + 1)].copy_(lse_loc.reshape(-1))
    else:
        part[:rows * d].zero_()
        part[rows * d:rows * (d + 1)].fill_(float("-inf"))
    dist.all_gather_into_tensor(scratch.gathered, part, group=group)      # rank-major
    if combine_fn is None:
        out = _combine_cuda(scratch.gathered, pf, world, rows, d, q.dtype)
    else:
        g = scratch.gathered.view(world, pf)
        out = combine_fn(g[:, :rows * d].reshape(world, rows, d).contiguous(),
                         g[:, rows * d:rows * (d + 1)].contiguous(), q.dtype)
    return out.reshape(B, H, Sq, d)
