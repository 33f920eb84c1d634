"""Seeded synthetic inputs for the five benchmark configurations of
``mha_fwd_with_mask``.

They stand in for the reference's ``benchmark/benchmark_fa.py`` suites, whose
shapes and value distributions they follow (``benchmark_fa.py:100-112``: N(0,1)
q/k/v, additive mask that is ``-inf`` with a given probability and 0 elsewhere,
one column forced visible so no row is empty).  Tensors are created on the CPU
from one ``torch.Generator`` per configuration so every implementation sees the
same bytes; the caller moves them to a device.

The mask is one ``(B, 1, Sq, Sk)`` tensor per batch, shared by all heads
(``csrc/fa/fa_fwd_op.cu:96-108``).
"""
from __future__ import annotations

import dataclasses
import math

import numpy as np
import torch


@dataclasses.dataclass(frozen=True)
class Workload:
    name: str
    B: int
    H: int
    Hk: int
    Sq: int
    Sk: int
    d: int
    dtype: torch.dtype
    mask_kind: str          # random10 | causal_window | padding_random | item_sparse
    sigma: float = 1.0

    @property
    def flops(self) -> float:
        """Dense algorithmic FLOPs, mask ignored, unpadded Sk: 4*B*H*Sq*Sk*d
        (``benchmark_fa.py:135-137``)."""
        return 4.0 * self.B * self.H * self.Sq * self.Sk * self.d

    @property
    def bytes(self) -> float:
        """Algorithmic HBM bytes: Q and O once, K and V once per kv head, the mask
        once per batch; 2 bytes per element."""
        return 2.0 * (2 * self.B * self.H * self.Sq * self.d
                      + 2 * self.B * self.Hk * self.Sk * self.d
                      + self.B * self.Sq * self.Sk)

    def with_batch(self, B: int) -> "Workload":
        return dataclasses.replace(self, B=B)


WORKLOADS = {
    "plumbing": Workload("plumbing", 2, 4, 4, 256, 256, 64, torch.bfloat16, "random10"),
    "standard": Workload("standard", 4, 16, 16, 2048, 2048, 128, torch.bfloat16, "random10"),
    "gqa_window": Workload("gqa_window", 4, 16, 4, 2048, 2048, 128, torch.bfloat16, "causal_window"),
    "splitkv_long": Workload("splitkv_long", 1, 16, 16, 128, 32768, 128, torch.bfloat16,
                             "padding_random"),
    "ragged_items": Workload("ragged_items", 4, 16, 4, 1000, 4099, 128, torch.float16,
                             "item_sparse", sigma=0.5),
}


def make_mask(kind: str, B: int, Sq: int, Sk: int, dtype: torch.dtype,
              gen: torch.Generator) -> torch.Tensor:
    neg = float("-inf")
    if kind == "random10":
        drop = torch.rand(B, 1, Sq, Sk, generator=gen) < 0.1
        idx = torch.arange(min(Sq, Sk))
        drop[:, :, idx, idx] = False                      # diagonal stays visible
        drop[..., 0] = False                              # and no row is ever empty
        return torch.zeros(B, 1, Sq, Sk, dtype=dtype).masked_fill(drop, neg)
    if kind == "causal_window":
        i = torch.arange(Sq).view(Sq, 1)
        j = torch.arange(Sk).view(1, Sk)
        vis = (i - j >= 0) & (i - j < 512)
        m = torch.zeros(Sq, Sk, dtype=dtype).masked_fill(~vis, neg)
        return m.view(1, 1, Sq, Sk).expand(B, 1, Sq, Sk).contiguous()
    if kind == "padding_random":
        drop = torch.rand(B, 1, Sq, Sk, generator=gen) < 0.1
        drop[..., int(Sk * 0.9):] = True                  # last 10 % of keys are padding
        drop[..., 0] = False
        return torch.zeros(B, 1, Sq, Sk, dtype=dtype).masked_fill(drop, neg)
    if kind == "item_sparse":
        n_items = math.ceil(Sk / 8)
        drop_item = torch.rand(B, 1, Sq, n_items, generator=gen) < 0.1
        drop = drop_item.repeat_interleave(8, dim=-1)[..., :Sk].clone()
        drop[..., :64] = False                            # first 64 keys always visible
        return torch.zeros(B, 1, Sq, Sk, dtype=dtype).masked_fill(drop, neg)
    raise ValueError(f"unknown mask kind {kind!r}")


def make_inputs(w: Workload, seed: int = 42):
    """q, k, v, mask on the CPU for workload ``w``."""
    gen = torch.Generator().manual_seed(seed)
    q = (torch.randn(w.B, w.H, w.Sq, w.d, generator=gen) * w.sigma).to(w.dtype)
    k = (torch.randn(w.B, w.Hk, w.Sk, w.d, generator=gen) * w.sigma).to(w.dtype)
    v = (torch.randn(w.B, w.Hk, w.Sk, w.d, generator=gen) * w.sigma).to(w.dtype)
    mask = make_mask(w.mask_kind, w.B, w.Sq, w.Sk, w.dtype, gen)
    return q, k, v, mask


def small_analogue(w: Workload, Sq: int, Sk: int, B: int = 1, H: int | None = None) -> Workload:
    """Same head layout, dtype and mask recipe at a size a CPU oracle finishes quickly."""
    H = H or w.H
    Hk = max(1, H // (w.H // w.Hk))
    return dataclasses.replace(w, name=w.name + "_small", B=B, H=H, Hk=Hk, Sq=Sq, Sk=Sk)


def to_bits(t: torch.Tensor) -> np.ndarray:
    """The raw 16-bit patterns of a float16 / bfloat16 tensor as a numpy uint16 array (numpy has
    no bfloat16; checkers that work on bit patterns take this)."""
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def dtype_tag(t: torch.Tensor) -> str:
    return "bf16" if t.dtype == torch.bfloat16 else "fp16"
