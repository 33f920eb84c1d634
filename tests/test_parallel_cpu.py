"""Host logic of the multi-GPU paths on CPU ranks (gloo, world_size 2): the
(batch, kv-head) sharding covers every unit exactly once and reproduces the
unsharded result, and the cross-GPU Split-KV gathers per-rank partials in rank
order and merges them to the single-device answer.  The CUDA entry points are
replaced by the CPU oracle through the hooks ``splitkv_forward`` offers for this."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from custom_ops_b200 import parallel
from oracle import oracle
from tests.fa_testlib import bits, make_case, tag


def test_shard_units_cover_exactly_once():
    for B, Hk, world in [(4, 16, 8), (4, 4, 8), (1, 16, 3), (2, 3, 4), (1, 1, 2), (4, 4, 1)]:
        seen = []
        for r in range(world):
            lo, hi = parallel.shard_units(B, Hk, world, r)
            seen += list(range(lo, hi))
            for b, h0, h1 in parallel.units_to_slices(lo, hi, Hk):
                assert 0 <= b < B and 0 <= h0 < h1 <= Hk
        assert seen == list(range(B * Hk))
        sizes = [parallel.shard_units(B, Hk, world, r) for r in range(world)]
        assert max(h - l for l, h in sizes) - min(h - l for l, h in sizes) <= 1
    with pytest.raises(ValueError):
        parallel.shard_units(1, 1, 2, 2)


def test_kv_slice_bounds():
    for Sk, world in [(32768, 8), (32768, 2), (4099, 4), (130, 4), (100, 2), (0, 2)]:
        prev = 0
        for r in range(world):
            lo, hi = parallel.kv_slice_bounds(Sk, world, r)
            assert lo == prev and lo <= hi <= Sk
            assert lo % 128 == 0 or lo == Sk
            prev = hi
        assert prev == Sk
    assert parallel.kv_slice_bounds(32768, 8, 3) == (12288, 16384)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _oracle_local(q, k, v, mask):
    o, lse = None, None
    qb, kb, vb, mb = bits(q), bits(k), bits(v), bits(mask)
    o = oracle.attn_fp32(qb, kb, vb, mb, tag(q))
    lse = oracle.lse_fp32(qb, kb, mb, tag(q))
    return torch.from_numpy(o), torch.from_numpy(lse)


def _numpy_combine(o_parts, lse_parts, dtype):
    o = o_parts.numpy().astype(np.float64)
    l = lse_parts.numpy().astype(np.float64)
    mx = l.max(axis=0)
    mx = np.where(np.isfinite(mx), mx, 0.0)
    w = np.exp(l - mx)
    den = w.sum(axis=0)
    out = (w[:, :, None] * o).sum(axis=0) / np.where(den > 0, den, 1.0)[:, None]
    return torch.from_numpy(out.astype(np.float32)).to(dtype)


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        # ---- cross-GPU Split-KV: one fully masked row, ragged Sk, a slice whose keys are all masked
        q, k, v, m = make_case(1, 4, 2, 40, 300, 64, torch.bfloat16, "drop_bias", seed=21)
        m[:, :, 3, :] = float("-inf")
        m[:, :, :, 256:] = float("-inf")
        lo, hi = parallel.kv_slice_bounds(300, world, rank)
        out = parallel.splitkv_forward(q, k[:, :, lo:hi].contiguous(), v[:, :, lo:hi].contiguous(),
                                       m[:, :, :, lo:hi].contiguous(), local_fn=_oracle_local,
                                       combine_fn=_numpy_combine)
        want = oracle.attn_fp32(bits(q), bits(k), bits(v), bits(m), "bf16")
        err_split = float(np.abs(out.float().numpy() - want).max())
        row_zero = bool((out[:, :, 3] == 0).all())
        # ---- (batch, kv-head) sharding: every rank computes its pieces, results are gathered
        q, k, v, m = make_case(3, 6, 3, 17, 50, 64, torch.float16, "drop_bias", seed=22)
        full = oracle.attn_fp32(bits(q), bits(k), bits(v), bits(m), "fp16")
        lo_u, hi_u = parallel.shard_units(3, 3, world, rank)
        mine = np.zeros_like(full)
        g = 2
        for (b, h0, h1), (qs, ks, vs, ms) in zip(parallel.units_to_slices(lo_u, hi_u, 3),
                                                 parallel.shard_inputs(q, k, v, m, world, rank)):
            mine[b, h0 * g:h1 * g] = oracle.attn_fp32(bits(qs), bits(ks), bits(vs), bits(ms), "fp16")[0]
        total = torch.from_numpy(mine)
        dist.all_reduce(total)                       # disjoint supports: the sum is the union
        err_shard = float(np.abs(total.numpy() - full).max())
        if rank == 0:
            ret["split"] = err_split
            ret["row_zero"] = row_zero
            ret["shard"] = err_shard
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_splitkv_and_sharding():
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret["split"] < 1e-2, dict(ret)       # result was rounded to bf16 by the merge
    assert ret["row_zero"]
    assert ret["shard"] < 1e-6, dict(ret)
