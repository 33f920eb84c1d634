"""The allocation-free entry point, fa_mask_fwd_sm100_static_scratch.

Some callers cannot give the library scratch memory: they run where cudaMalloc is not
allowed (a serving loop that bans allocator calls, a region being captured, a host runtime
that does not own a memory pool) or can only pass the operator's own tensors.  For them the
library carries a fixed scratch array; this test calls that entry point through the C ABI
on inputs that need scratch (Split-KV partials, a re-pitched mask) and checks it against the
ordinary entry point, twice in a row because the array keeps the previous call's contents.
The file sorts last so a run that stops at the first failure has finished everything else.
"""
import pytest
import torch

from custom_ops_b200 import _cabi
from tests.fa_testlib import check_against_oracle, make_case, run_cabi

pytestmark = pytest.mark.gpu


def _args(q, k, v, m, out):
    B, H, Sq, d = q.shape
    return _cabi.make_args(
        q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), mask=m.data_ptr(), out=out.data_ptr(),
        batch=B, heads=H, heads_k=k.shape[1], seqlen_q=Sq, seqlen_k=k.shape[2], head_dim=d,
        dtype=_cabi.BF16 if q.dtype == torch.bfloat16 else _cabi.FP16,
        mask_seqlen_q=m.shape[2], mask_seqlen_k=m.shape[3], mask_batch_stride=m.stride(0),
        mask_row_stride=m.stride(2))


def test_static_scratch_matches_workspace_entry_point_twice():
    stream = torch.cuda.current_stream().cuda_stream
    # call 1: Split-KV (two splits per CTA) with a ragged Sk, so partials, LSE and a re-pitched
    # mask all live in the built-in array; call 2: another shape that leaves different bytes there
    cases = [make_case(1, 4, 2, 128, 4099, 128, torch.bfloat16, "drop_bias", seed=31),
             make_case(1, 2, 2, 100, 8192, 64, torch.float16, "drop_bias", seed=32)]
    for q, k, v, m in cases:
        q, k, v, m = q.cuda(), k.cuda(), v.cuda(), m.cuda()
        want, _, plan = run_cabi(q, k, v, m)
        assert plan.num_splits > 1 and 0 < plan.workspace_bytes <= _cabi.STATIC_SCRATCH_BYTES
        for _ in range(2):                       # two calls in a row on the same array
            got = torch.empty_like(q)
            _cabi.forward_static_scratch(_args(q, k, v, m, got), stream)
            torch.cuda.synchronize()
            # same kernels, same inputs, same order of operations: bit-identical
            assert torch.equal(got, want)
        check_against_oracle(got, q, k, v, m, "static scratch")
    assert _cabi.device_status(0, clear=True) == 0


def test_static_scratch_on_a_dirty_array_unit_cut_and_tile_skip():
    """Run after the Split-KV case above, so the array holds that call's bytes.  The slots of the
    unit cutting are guarded by tags that are compared with a value unique to each launch (they
    are not cleared first), and the tile-skip flags and the unit counter are written by the
    pre-pass kernel before the attention kernel reads them: neither may be fooled by stale
    contents.  Each shape runs twice and is compared with the workspace entry point."""
    stream = torch.cuda.current_stream().cuda_stream
    # (1, 40, 8, 1024, 3000): 160 units on 148 SMs -> the last round is cut in pieces, scratch < 24 MiB
    cut = make_case(1, 40, 8, 1024, 3000, 128, torch.float16, "drop_bias", seed=41)
    # a causal mask over 6 key blocks: the pre-pass finds blocks to skip, units are handed out
    # from the counter in the scratch array
    skip = make_case(2, 4, 2, 768, 768, 128, torch.bfloat16, "causal", seed=42)
    for name, (q, k, v, m) in (("unit cut", cut), ("tile skip", skip)):
        q, k, v, m = q.cuda(), k.cuda(), v.cuda(), m.cuda()
        want, _, plan = run_cabi(q, k, v, m)
        assert 0 < plan.workspace_bytes <= _cabi.STATIC_SCRATCH_BYTES
        assert (plan.unit_cut >= 2) if name == "unit cut" else (plan.tile_skip == 1)
        for _ in range(2):
            got = torch.empty_like(q)
            _cabi.forward_static_scratch(_args(q, k, v, m, got), stream)
            torch.cuda.synchronize()
            assert (got.float() - want.float()).abs().max().item() <= 4e-3, name
        check_against_oracle(got, q, k, v, m, f"static scratch, {name}")
    assert _cabi.device_status(0, clear=True) == 0


def test_static_scratch_rejects_oversized_requests():
    # 64 heads x 128 rows x 128 splits of fp32 partials is far beyond the built-in array
    q = torch.empty(1, 64, 128, 128, device="cuda", dtype=torch.bfloat16)
    a = _cabi.make_args(q=q.data_ptr(), k=q.data_ptr(), v=q.data_ptr(), mask=q.data_ptr(),
                        out=q.data_ptr(), batch=1, heads=64, heads_k=64, seqlen_q=128,
                        seqlen_k=128 * 1024, head_dim=128, dtype=_cabi.BF16, num_splits=128)
    assert _cabi.workspace_bytes(a) > _cabi.STATIC_SCRATCH_BYTES
    with pytest.raises(_cabi.FaSm100Error) as e:
        _cabi.forward_static_scratch(a, 0)
    assert e.value.code == -6
