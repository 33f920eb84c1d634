"""Helpers shared by the GPU parity tests: call the C ABI with torch-owned device
buffers, build the reference test matrix's inputs on the CPU, compare with the
CPU oracle."""
from __future__ import annotations

import numpy as np
import torch

from custom_ops_b200 import _cabi
from oracle import oracle


from custom_ops_b200.workloads import dtype_tag as tag, to_bits as bits  # noqa: E402,F401


def from_bits(b: np.ndarray, dtype: str) -> torch.Tensor:
    t = torch.from_numpy(b.view(np.int16).copy())
    return t.view(torch.bfloat16 if dtype == "bf16" else torch.float16)


def run_cabi(q, k, v, mask, *, num_splits=0, want_lse=False, out_fp32=False, device=0,
             no_tile_skip=0, no_unit_cut=0, no_head_pairs=0, mask_version=0):
    """q, k, v, mask: CUDA tensors.  Returns (out, lse or None, plan)."""
    B, H, Sq, d = q.shape
    Hk, Sk = k.shape[1], k.shape[2]
    out = torch.empty((B, H, Sq, d), device=q.device,
                      dtype=torch.float32 if out_fp32 else q.dtype)
    lse = torch.empty((B, H, Sq), device=q.device, dtype=torch.float32) if want_lse else None
    args = _cabi.make_args(
        q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), mask=mask.data_ptr(), out=out.data_ptr(),
        lse=lse.data_ptr() if want_lse else 0, batch=B, heads=H, heads_k=Hk, seqlen_q=Sq,
        seqlen_k=Sk, head_dim=d, dtype=_cabi.BF16 if q.dtype == torch.bfloat16 else _cabi.FP16,
        mask_seqlen_q=mask.shape[2], mask_seqlen_k=mask.shape[3],
        mask_batch_stride=mask.stride(0), mask_row_stride=mask.stride(2), device=device,
        num_splits=num_splits, out_fp32=1 if out_fp32 else 0, no_tile_skip=no_tile_skip, no_unit_cut=no_unit_cut,
        no_head_pairs=no_head_pairs, mask_version=mask_version)
    plan = _cabi.plan(args)
    nbytes = _cabi.workspace_bytes(args)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device)
    stream = torch.cuda.current_stream(q.device).cuda_stream
    _cabi.forward(args, ws.data_ptr(), nbytes, stream)
    torch.cuda.synchronize(q.device)
    return out, lse, plan


def make_case(B, H, Hk, Sq, Sk, d, dtype, mask_kind, *, seed=0, sigma=0.5, pad_rows=0, pad_cols=0):
    """Inputs in the style of the reference tests (randn*0.5; mask kinds zero /
    causal / random (finite bias) / block / all_masked_row / drop10)."""
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, H, Sq, d, generator=g) * sigma).to(dtype)
    k = (torch.randn(B, Hk, Sk, d, generator=g) * sigma).to(dtype)
    v = (torch.randn(B, Hk, Sk, d, generator=g) * sigma).to(dtype)
    Sqm, Skm = Sq + pad_rows, Sk + pad_cols
    neg = float("-inf")
    if mask_kind == "zero":
        m = torch.zeros(B, 1, Sqm, Skm)
    elif mask_kind == "causal":
        m = torch.triu(torch.full((Sqm, Skm), neg), diagonal=1).expand(B, 1, Sqm, Skm).clone()
    elif mask_kind == "random":
        m = torch.randn(B, 1, Sqm, Skm, generator=g) * 0.3
    elif mask_kind == "block":
        m = torch.zeros(B, 1, Sqm, Skm)
        m[..., Sk // 2:] = neg
    elif mask_kind == "all_masked_row":
        m = torch.zeros(B, 1, Sqm, Skm)
        m[:, :, 0, :] = neg
    elif mask_kind == "drop10":
        m = torch.zeros(B, 1, Sqm, Skm)
        drop = torch.rand(B, 1, Sqm, Skm, generator=g) < 0.1
        drop[..., 0] = False
        m = m.masked_fill(drop, neg)
    elif mask_kind == "drop_bias":
        m = torch.randn(B, 1, Sqm, Skm, generator=g) * 0.3
        drop = torch.rand(B, 1, Sqm, Skm, generator=g) < (1.0 / 7.0)
        drop[..., 0] = False
        m = m.masked_fill(drop, neg)
    else:
        raise ValueError(mask_kind)
    return q, k, v, m.to(dtype).contiguous()


def oracle_pair(q, k, v, mask):
    """(fp32 softmax oracle, ref_attn oracle with P rounding), both fp32 numpy.
    Uses the compiled C restatement when it is built (same maths, much faster)."""
    dt = tag(q)
    qb, kb, vb, mb = bits(q), bits(k), bits(v), bits(mask)
    if oracle.load_port() is not None:
        return (oracle.port_attn(qb, kb, vb, mb, dt, quantize_p=False),
                oracle.port_attn(qb, kb, vb, mb, dt, quantize_p=True))
    return oracle.attn_fp32(qb, kb, vb, mb, dt), oracle._attn(qb, kb, vb, mb, dt, True)


def check_against_oracle(out: torch.Tensor, q, k, v, mask, what=""):
    """Both pass rules: the accuracy bar vs the fp32 oracle (max-abs 2e-2, mean-abs
    2e-3) and the reference test's own rule vs its P-rounding oracle
    (max_err < 1e-2 or max_err/max|ref| < 1e-2)."""
    o = out.detach().float().cpu().numpy()
    assert np.all(np.isfinite(o)), f"{what}: non-finite output"
    ref32, ref_q = oracle_pair(q, k, v, mask)
    mx, mean = oracle.errors(o, ref32)
    assert mx <= oracle.MAX_ABS_TOL and mean <= oracle.MEAN_ABS_TOL, \
        f"{what}: max_abs={mx:.3e} mean_abs={mean:.3e} vs fp32 oracle"
    assert oracle.within_reference_rule(o, oracle.quantize(ref_q, tag(q))), \
        f"{what}: fails the reference rule, max_abs={oracle.errors(o, ref_q)[0]:.3e}"
    return mx, mean
