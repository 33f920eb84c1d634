#!/usr/bin/env python3
"""Write ``tests/golden/ref_attn_cases.npz``: small inputs together with the
outputs of the REFERENCE's own test oracle ``ref_attn``
(``tests/test_mha_fwd_with_mask.py:38-53``) evaluated on them on the CPU.

Run where the reference checkout is mounted:

    python tests/golden/make_golden.py --reference <path to the reference checkout>

The reference's root directory *is* the package ``custom_ops``; its test module
does ``from custom_ops import ops`` at import time (lazy, nothing is compiled),
so the script exposes the checkout under that name through a temporary symlink
and loads the test file by path.  The committed ``.npz`` is what the test-suite
reads; this script is not needed at test time.

The cases mirror the reference's matrix (``tests/test_mha_fwd_with_mask.py:181-230``)
at sizes that keep the file small: mask kinds zero / causal / random finite /
random -inf / one fully masked row, GQA, ragged Sq and Sk, a pre-padded mask
whose pad columns hold trap values.
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import sys
import tempfile

import numpy as np
import torch


def load_reference_ref_attn(ref_root: str):
    tmp = tempfile.mkdtemp(prefix="ref_pkg_")
    os.symlink(ref_root, os.path.join(tmp, "custom_ops"))
    sys.path.insert(0, tmp)
    os.environ.setdefault("TORCH_EXTENSIONS_DIR", os.path.join(tmp, "torch_ext"))
    path = os.path.join(ref_root, "tests", "test_mha_fwd_with_mask.py")
    spec = importlib.util.spec_from_file_location("ref_test_mha_fwd_with_mask", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.ref_attn


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


CASES = [
    # name, dtype, B, H, Hk, Sq, Sk, d, mask kind, pad_rows, pad_cols
    ("bf16_d64_drop10", torch.bfloat16, 1, 2, 2, 48, 72, 64, "drop10", 0, 0),
    ("fp16_d128_gqa_bias", torch.float16, 1, 4, 2, 33, 40, 128, "bias", 0, 0),
    ("bf16_d64_causal_rowmasked", torch.bfloat16, 2, 2, 1, 16, 24, 64, "causal_row0", 0, 0),
    ("fp16_d64_padded_trap", torch.float16, 1, 2, 2, 20, 24, 64, "bias", 8, 8),
    ("bf16_d128_ragged", torch.bfloat16, 1, 2, 2, 5, 13, 128, "drop10", 0, 0),
    ("fp16_d128_zero", torch.float16, 1, 1, 1, 17, 136, 128, "zero", 0, 0),
    ("bf16_d128_multiblock", torch.bfloat16, 1, 2, 1, 130, 300, 128, "drop10_bias", 0, 0),
]


def make_case(gen, dtype, B, H, Hk, Sq, Sk, d, kind, pad_rows, pad_cols):
    q = (torch.randn(B, H, Sq, d, generator=gen) * 0.5).to(dtype)
    k = (torch.randn(B, Hk, Sk, d, generator=gen) * 0.5).to(dtype)
    v = (torch.randn(B, Hk, Sk, d, generator=gen) * 0.5).to(dtype)
    Sqm, Skm = Sq + pad_rows, Sk + pad_cols
    neg = float("-inf")
    if kind == "zero":
        m = torch.zeros(B, 1, Sqm, Skm)
    elif kind == "bias":
        m = torch.randn(B, 1, Sqm, Skm, generator=gen) * 0.3
    elif kind == "drop10":
        m = torch.zeros(B, 1, Sqm, Skm)
        drop = torch.rand(B, 1, Sqm, Skm, generator=gen) < 0.1
        drop[..., 0] = False
        m = m.masked_fill(drop, neg)
    elif kind == "drop10_bias":
        m = torch.randn(B, 1, Sqm, Skm, generator=gen) * 0.3
        drop = torch.rand(B, 1, Sqm, Skm, generator=gen) < 0.1
        drop[..., 0] = False
        m = m.masked_fill(drop, neg)
    elif kind == "causal_row0":
        m = torch.triu(torch.full((Sqm, Skm), neg), diagonal=1).expand(B, 1, Sqm, Skm).clone()
        m[:, :, 0, :] = neg                      # one fully masked row -> output 0
    else:
        raise ValueError(kind)
    return q, k, v, m.to(dtype).contiguous()


def main():
    ap = argparse.ArgumentParser()
    here = os.path.dirname(os.path.abspath(__file__))
    beside = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(here))), "reference")
    ap.add_argument("--reference", default=os.environ.get("CUSTOM_OPS_REFERENCE", beside),
                    help="checkout of the reference (default: $CUSTOM_OPS_REFERENCE, else a directory "
                         "'reference' beside this repository)")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                  "ref_attn_cases.npz"))
    args = ap.parse_args()
    ref_attn = load_reference_ref_attn(args.reference)
    gen = torch.Generator().manual_seed(20240607)
    blob = {}
    names = []
    for name, dtype, B, H, Hk, Sq, Sk, d, kind, pr, pc in CASES:
        q, k, v, m = make_case(gen, dtype, B, H, Hk, Sq, Sk, d, kind, pr, pc)
        rep = H // Hk
        # The reference oracle has no GQA or padded-mask handling of its own: its
        # tests expand K/V with repeat_interleave and crop the mask before calling it
        # (tests/test_mha_fwd_with_mask.py:104,116-123).
        out = ref_attn(q, k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1),
                       m[:, :, :Sq, :Sk].contiguous())
        assert out.dtype == dtype and not torch.isnan(out.float()).any()
        names.append(name)
        blob[name + ".q"] = bits(q)
        blob[name + ".k"] = bits(k)
        blob[name + ".v"] = bits(v)
        blob[name + ".mask"] = bits(m)
        blob[name + ".out"] = bits(out)
        blob[name + ".dtype"] = np.array("bf16" if dtype == torch.bfloat16 else "fp16")
        print(f"{name}: q{tuple(q.shape)} k{tuple(k.shape)} mask{tuple(m.shape)} "
              f"max|out|={out.float().abs().max():.4f}")
    blob["names"] = np.array(names)
    np.savez_compressed(args.out, **blob)
    print("wrote", args.out, os.path.getsize(args.out), "bytes")


if __name__ == "__main__":
    main()
