"""CPU-only tests of the host side: the C-ABI library loads and exports what the
header declares, the launch planner and argument validation, the Python mirror of
the reference's loader/facade, and the workload generators.  No kernel is launched."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from custom_ops_b200 import _cabi, workloads
from custom_ops_b200.workloads import WORKLOADS, make_inputs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ------------------------------------------------------------------ C ABI
def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "fa_mask_fwd_sm100.h")).read()
    declared = set(re.findall(r"^(?:int|const char\*)\s+(fa_mask_\w+)\s*\(", header, flags=re.M))
    assert declared == set(_cabi.EXPORTS)
    lib = _cabi.load()
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.fa_mask_fwd_sm100_abi_version() == _cabi.ABI_VERSION


def test_struct_sizes_match_header_layout():
    # 2*4 + 6*8 + 8*4 + 2*8 + 4*4 + 8 = 128 ; 16*4 + 8 = 72
    assert ctypes.sizeof(_cabi.FaMaskFwdArgs) == 128
    assert ctypes.sizeof(_cabi.FaMaskFwdPlan) == 72
    a = _cabi.make_args(batch=1, heads=1, heads_k=1, seqlen_q=8, seqlen_k=8, head_dim=64,
                        dtype=_cabi.BF16)
    a.struct_size = 64
    with pytest.raises(_cabi.FaSm100Error) as e:
        _cabi.plan(a)
    assert e.value.code == -11


def _plan(**kw):
    base = dict(batch=1, heads=1, heads_k=1, seqlen_q=128, seqlen_k=128, head_dim=128,
                dtype=_cabi.BF16)
    base.update(kw)
    return _cabi.plan(_cabi.make_args(**base))


def test_mask_planes_must_not_overlap():
    ok = dict(batch=3, heads=2, heads_k=2, seqlen_q=100, seqlen_k=200, mask_seqlen_q=100, mask_seqlen_k=200,
              mask_row_stride=200)
    assert _plan(mask_batch_stride=100 * 200, **ok).num_splits >= 1
    assert _plan(mask_batch_stride=0, **ok).num_splits >= 1             # one plane for every batch element
    for bad in (8, 200, 100 * 200 - 8):
        with pytest.raises(_cabi.FaSm100Error) as e:
            _plan(mask_batch_stride=bad, **ok)
        assert e.value.code == -3
    assert _plan(batch=1, heads=2, heads_k=2, seqlen_q=100, seqlen_k=200, mask_batch_stride=8).num_splits >= 1


def test_plan_of_the_five_configurations():
    sm = _plan().sm_count                      # 148 where no device can be queried
    p = _plan(batch=4, heads=16, heads_k=16, seqlen_q=2048, seqlen_k=2048)
    # 8 * 16 * 4 = 512 units; pair mode is persistent: one CTA per SM takes every grid_x-th unit
    assert (p.num_splits, p.kv_blocks, p.grid_x, p.q_tiles_per_cta) == (1, 16, min(512, sm), 2)
    # block flags (4 * 8 * 16 bytes -> 512) + the unit counter; more units than CTAs: the units of
    # the last, partial round are cut in pieces, which takes per CTA 256 rows of fp32 O + LSE and 8 tags
    pieces = min(sm // (512 % sm), 3) if 512 > sm and 512 % sm else 0      # CTAs per unit of the last round (at most floor(sqrt(0.65 * 16)))
    pieces = pieces if pieces >= 2 else 0
    cut = -(-(p.grid_x * 256 * (128 + 1) * 4 + p.grid_x * 8 * 8) // 256) * 256 if pieces else 0
    assert p.unit_cut == pieces
    assert p.tile_skip == 1 and p.workspace_bytes == 512 + 256 + cut and p.mask_repitched == 0 and p.threads == 384
    assert _plan(batch=4, heads=16, heads_k=16, seqlen_q=2048, seqlen_k=2048, no_tile_skip=1).workspace_bytes == cut
    assert _plan(batch=4, heads=16, heads_k=16, seqlen_q=2048, seqlen_k=2048, no_tile_skip=1,
                 no_unit_cut=1).workspace_bytes == 0
    p = _plan(batch=1, heads=16, heads_k=16, seqlen_q=128, seqlen_k=32768)
    assert p.kv_blocks == 256 and p.num_splits == 2 * max(1, sm // 16) and p.q_tiles_per_cta == 1
    assert p.dual_split == 1 and p.grid_x == 16 * ((p.num_splits + 1) // 2)
    assert p.blocks_per_split == -(-256 // p.num_splits)
    rows = 16 * 128
    assert p.workspace_bytes >= (p.num_splits // 2) * rows * (128 + 1) * 4   # one partial per CTA
    p = _plan(batch=4, heads=16, heads_k=4, seqlen_q=1000, seqlen_k=4099, dtype=_cabi.FP16)
    assert p.num_splits == 1 and p.kv_blocks == 33 and p.mask_repitched == 1
    assert p.workspace_bytes >= 4 * 1000 * 4104 * 2
    p = _plan(batch=2, heads=4, heads_k=4, seqlen_q=256, seqlen_k=256, head_dim=64)
    assert p.num_splits == 1 and p.grid_x == 8 and p.tile_skip == 0
    assert p.smem_bytes <= 232448


def test_plan_pairs_grouped_query_heads():
    """An even group size: a unit is two heads of a KV group over one 128-row tile; the block flags
    of the tile-skip pre-pass are then per 128 rows."""
    sm = _plan().sm_count
    p = _plan(batch=4, heads=16, heads_k=4, seqlen_q=2048, seqlen_k=2048)
    assert p.head_pairs == 1 and p.q_tiles_per_cta == 2 and p.grid_x == min(4 * 8 * 16, sm)
    q = _plan(batch=4, heads=16, heads_k=4, seqlen_q=2048, seqlen_k=2048, no_head_pairs=1)
    assert q.head_pairs == 0 and q.grid_x == p.grid_x
    # flags: 4 batches x 16 tiles x 16 key blocks against 4 x 8 pairs x 16
    assert p.workspace_bytes - q.workspace_bytes == 4 * 16 * 16 - 4 * 8 * 16
    assert _plan(batch=1, heads=6, heads_k=2, seqlen_q=300, seqlen_k=300).head_pairs == 0      # group of 3
    assert _plan(batch=1, heads=8, heads_k=8, seqlen_q=300, seqlen_k=300).head_pairs == 0      # no groups
    # one query tile and few heads: two heads fill the two slots of a CTA
    p = _plan(batch=2, heads=8, heads_k=2, seqlen_q=100, seqlen_k=256)
    assert p.head_pairs == 1 and p.grid_x == 2 * 4 and p.q_tiles_per_cta == 2
    # one query tile with a split key range keeps two splits per CTA instead
    p = _plan(batch=1, heads=16, heads_k=4, seqlen_q=128, seqlen_k=32768)
    assert p.dual_split == 1 and p.head_pairs == 0


def test_plan_split_rules():
    # never an empty split, never more splits than key blocks, forced counts honoured
    for sk, forced in [(1300, 3), (1300, 7), (1300, 40), (1300, 128), (4096, 40), (130, 2)]:
        p = _plan(seqlen_k=sk, num_splits=forced)
        nb = (sk + 127) // 128
        assert p.num_splits == min(forced, nb)
        assert p.blocks_per_split == -(-nb // p.num_splits)
    assert _plan(seqlen_k=8192, num_splits=1).num_splits == 1
    assert _plan(seqlen_k=512).num_splits == 1          # too short to be worth splitting
    assert _plan(seqlen_k=0).num_splits == 1


@pytest.mark.parametrize("kw,code", [
    (dict(dtype=2), -2), (dict(head_dim=96), -4), (dict(heads=6, heads_k=4), -3),
    (dict(seqlen_q=-1), -3), (dict(mask_seqlen_k=64), -3), (dict(mask_seqlen_q=64), -3),
    (dict(num_splits=129), -9), (dict(num_splits=-1), -9), (dict(heads_k=0), -3),
    (dict(mask_row_stride=100), -3),
])
def test_validation_codes(kw, code):
    with pytest.raises(_cabi.FaSm100Error) as e:
        _plan(**kw)
    assert e.value.code == code
    assert _cabi.strerror(code) not in ("ok", "unknown error")


def test_null_arguments_and_strerror():
    lib = _cabi.load()
    assert lib.fa_mask_fwd_sm100_plan(None, None) == -1
    n = ctypes.c_size_t()
    assert lib.fa_mask_fwd_sm100_workspace_bytes(None, ctypes.byref(n)) == -1
    assert _cabi.strerror(0) == "ok"
    assert "head_dim" in _cabi.strerror(-4)
    assert "float16 or bfloat16" in _cabi.strerror(-2)
    assert _cabi.strerror(-12345) == "unknown error"


def test_forward_without_a_gpu_fails_loudly():
    """No CPU fallback: on a machine without a device the call returns an error."""
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    buf = (ctypes.c_uint8 * 4096)()
    addr = (ctypes.addressof(buf) + 15) & ~15
    a = _cabi.make_args(q=addr, k=addr, v=addr, mask=addr, out=addr, batch=1, heads=1, heads_k=1,
                        seqlen_q=8, seqlen_k=8, head_dim=64, dtype=_cabi.BF16)
    with pytest.raises(_cabi.FaSm100Error) as e:
        _cabi.forward(a, addr, 4096, 0)
    assert e.value.code in (-7, -8)


# ------------------------------------------------------------------ loader / facade
def test_group_definition_matches_reference_contract():
    from custom_ops_b200 import FAOps
    assert FAOps.namespace == "recsys_ops"
    assert FAOps.so_name == "recsys_fa_kernel"
    assert FAOps.required_ops == ["mha_fwd_with_mask"]
    # the reference's one operator is the required one; the LSE-returning variant is an extra
    assert FAOps.optional_ops == ["mha_fwd_with_mask_lse", "mha_fwd_rule_mask"]
    assert FAOps.fake_ops == ["mha_fwd_with_mask", "mha_fwd_with_mask_lse", "mha_fwd_rule_mask"]
    assert FAOps.op_schemas["mha_fwd_with_mask"] == \
        "mha_fwd_with_mask(Tensor q, Tensor k, Tensor v, Tensor mask) -> Tensor"
    assert FAOps.requires_cuda is True


def test_facade_lazy_load_schema_and_fake_kernel():
    import custom_ops_b200
    from custom_ops_b200 import RecsysOps
    fresh = RecsysOps()
    assert fresh.groups == {"fa": "not_loaded"}
    assert fresh.load_error() is None
    fresh.ensure_loaded("fa")
    assert fresh.groups == {"fa": "loaded"}, fresh.load_error("fa")
    assert fresh.is_available("fa")
    schema = str(torch._C._get_schema("recsys_ops::mha_fwd_with_mask", ""))
    assert schema == "recsys_ops::mha_fwd_with_mask(Tensor q, Tensor k, Tensor v, Tensor mask) -> Tensor"
    assert torch._C._dispatch_has_kernel_for_dispatch_key("recsys_ops::mha_fwd_with_mask", "Meta")
    q = torch.empty(2, 4, 10, 64, device="meta", dtype=torch.float16)
    kv = torch.empty(2, 2, 24, 64, device="meta", dtype=torch.float16)
    m = torch.empty(2, 1, 10, 24, device="meta", dtype=torch.float16)
    out = torch.ops.recsys_ops.mha_fwd_with_mask(q, kv, kv, m)
    assert out.shape == q.shape and out.dtype == q.dtype
    # a second facade shares the already loaded library
    again = RecsysOps(allow_jit=False).ensure_loaded("fa")
    assert again.is_available("fa")
    assert custom_ops_b200.ops.mha_fwd_with_mask.__doc__


def test_facade_errors():
    from custom_ops_b200 import CustomOpsError, RecsysOps
    ops = RecsysOps()
    x = torch.zeros(1, 1, 8, 64, dtype=torch.bfloat16)
    m = torch.zeros(1, 1, 8, 8, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="only supported on CUDA"):
        ops.mha_fwd_with_mask(x, x, x, m)                  # CPU tensors: the reference's stub message
    with pytest.raises(CustomOpsError):
        ops.mha_fwd_with_mask(x, x, x, m, backend="tilelang")
    with pytest.raises(ValueError):
        ops.mha_fwd_with_mask(x, x, x, m, backend="rocm")
    with pytest.raises(AttributeError):
        ops.fuse_moe
    with pytest.raises(ValueError):
        ops.is_available("moe")


def test_strict_mode_does_not_build(tmp_path, monkeypatch):
    from custom_ops_b200 import FAOps
    g = FAOps(allow_jit=False)
    monkeypatch.setattr(g, "prebuilt_path", lambda: str(tmp_path / "missing.so"))
    with pytest.warns(UserWarning):
        g.load()
    assert not g.is_available()
    assert "allow_jit=False" in g.load_error()
    with pytest.raises(RuntimeError, match="extension not loaded"):
        g.mha_fwd_with_mask


# ------------------------------------------------------------------ workloads
def test_workload_shapes_flops_bytes():
    w = WORKLOADS["standard"]
    assert w.flops == 4 * 4 * 16 * 2048 * 2048 * 128 == 137438953472
    assert w.bytes == 167772160
    assert WORKLOADS["splitkv_long"].bytes == pytest.approx(277.87e6, rel=1e-3)
    assert WORKLOADS["ragged_items"].dtype == torch.float16


def test_mask_recipes():
    g = torch.Generator().manual_seed(0)
    m = workloads.make_mask("random10", 2, 64, 64, torch.bfloat16, g)
    frac = torch.isneginf(m.float()).float().mean().item()
    assert 0.05 < frac < 0.15
    assert torch.all(m[:, 0].diagonal(dim1=-2, dim2=-1) == 0)
    m = workloads.make_mask("causal_window", 1, 1024, 1024, torch.bfloat16, g)[0, 0]
    assert m[600, 600] == 0 and m[600, 89] == 0 and torch.isneginf(m[600, 88]) and torch.isneginf(m[600, 601])
    m = workloads.make_mask("padding_random", 1, 8, 1000, torch.bfloat16, g)[0, 0]
    assert torch.isneginf(m[:, 900:].float()).all() and (m[:, 0] == 0).all()
    m = workloads.make_mask("item_sparse", 1, 16, 83, torch.float16, g)[0, 0]
    assert (m[:, :64] == 0).all()
    items = torch.isneginf(m[:, 64:80].float()).view(16, 2, 8)
    assert (items.all(-1) | (~items).all(-1)).all()        # whole 8-token items
    q, k, v, mm = make_inputs(workloads.small_analogue(WORKLOADS["ragged_items"], 20, 83, H=8))
    assert q.shape == (1, 8, 20, 128) and k.shape == (1, 2, 83, 128) and mm.shape == (1, 1, 20, 83)
    assert abs(q.float().std().item() - 0.5) < 0.05


def test_host_memory_entry_point_checks_its_arguments():
    """Argument errors of ``mha_fwd_with_mask_from_host`` are raised before any CUDA call, and
    without a device the call fails loudly instead of computing on the CPU."""
    from custom_ops_b200 import mha_fwd_with_mask_from_host
    q = torch.zeros(2, 2, 8, 64, dtype=torch.bfloat16)
    k = torch.zeros(2, 2, 8, 64, dtype=torch.bfloat16)
    m = torch.zeros(2, 1, 8, 8, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        mha_fwd_with_mask_from_host(q, k[:1], k, m)
    with pytest.raises(ValueError):
        mha_fwd_with_mask_from_host(q, k, k, m[0])
    with pytest.raises(ValueError):
        mha_fwd_with_mask_from_host(q, k, k, m, torch.zeros(2, 2, 8, 64))
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            mha_fwd_with_mask_from_host(q, k, k, m)


def test_rule_mask_checks_its_arguments():
    from custom_ops_b200.masks import rule_mask
    with pytest.raises(ValueError):
        rule_mask(1, 8, 8, dtype=torch.float32)
    with pytest.raises(ValueError):
        rule_mask(1, 8, -1)
    lib = _cabi.load()
    assert lib.fa_mask_build_sm100(None, 1, 8, 8, 8, _cabi.BF16, 0, 0, None, 0, None) == -1
    buf = (ctypes.c_uint8 * 64)()
    addr = ctypes.addressof(buf)
    assert lib.fa_mask_build_sm100(addr, 1, 8, 8, 4, _cabi.BF16, 0, 0, None, 0, None) == -3     # pitch < Sk
    assert lib.fa_mask_build_sm100(addr, 1, 8, 8, 8, 7, 0, 0, None, 0, None) == -2              # dtype
    assert lib.fa_mask_build_sm100(addr, 0, 8, 8, 8, _cabi.BF16, 0, 0, None, 0, None) == 0      # nothing to write
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            rule_mask(1, 8, 8)


def test_plan_unit_cut_rule():
    """Pieces per unit of a last round that is at most half full: SMs / left-over units, at most
    floor(sqrt(0.65 * key blocks)) (every further piece costs the first one a merge), none below
    six key blocks, none when the rounds are whole or the caller switches it off."""
    sm = _plan().sm_count
    def cut(units, sk, **kw):
        return _plan(batch=1, heads=units, heads_k=units, seqlen_q=256, seqlen_k=sk, **kw).unit_cut
    assert cut(sm + 1, 128 * 16) == 3
    assert cut(sm + 1, 128 * 64) == 6
    assert cut(sm + sm // 2, 128 * 64) == 2
    assert cut(sm + sm // 2 + 1, 128 * 64) == 0          # more than half a round left over
    assert cut(2 * sm, 128 * 16) == 0                    # whole rounds only
    assert cut(sm + 1, 128 * 5) == 0                     # too few key blocks to pay
    assert cut(sm + 1, 128 * 16, no_unit_cut=1) == 0
    assert cut(sm - 1, 128 * 16) == 0                    # one piece per CTA is all there is
    # fewer units than SMs: the only round is a partial one, every unit is cut, the grid grows
    # (key ranges of 24 blocks and more are split over CTAs instead, see test_plan_split_rules)
    assert cut(sm // 2, 128 * 16) == 2 and cut(sm // 3, 128 * 20) == 3 and cut(sm // 2, 128 * 11) == 0
    p = _plan(batch=1, heads=sm // 2, heads_k=sm // 2, seqlen_q=256, seqlen_k=128 * 16)
    assert p.grid_x == 2 * (sm // 2)
    assert _plan(batch=1, heads=sm // 2, heads_k=sm // 2, seqlen_q=256, seqlen_k=128 * 16,
                 no_unit_cut=1).grid_x == sm // 2

