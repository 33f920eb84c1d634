"""The CPU oracle against the reference's own outputs (committed fixtures written
by tests/golden/make_golden.py from the reference's ``ref_attn``), against the
reference's compiled CPU kernels where they were built, and against itself
(numpy restatement vs plain-C restatement)."""
import math
import os

import numpy as np
import pytest

from oracle import oracle


def _case(golden, name):
    g = lambda k: golden[f"{name}.{k}"]
    return g("q"), g("k"), g("v"), g("mask"), g("out"), str(g("dtype"))


def test_golden_file_lists_cases(golden):
    names = [str(n) for n in golden["names"]]
    assert len(names) >= 7
    for n in names:
        for part in ("q", "k", "v", "mask", "out", "dtype"):
            assert f"{n}.{part}" in golden.files


def test_numpy_oracle_matches_reference_ref_attn(golden):
    """Half an ulp of the 16-bit output is the most two fp32 summation orders differ."""
    for name in (str(n) for n in golden["names"]):
        q, k, v, m, out_bits, dt = _case(golden, name)
        o32, o_bits = oracle.ref_attn(q, k, v, m, dt)
        ref = oracle.to_f32(out_bits, dt)
        ulp = 2.0 ** (-8 if dt == "bf16" else -11)
        tol = ulp * np.maximum(np.abs(ref), 2.0 ** -6) * 1.01 + 1e-6
        assert np.all(np.abs(o32 - ref) <= tol), name
        # and almost every element rounds to the very same bit pattern
        assert (o_bits == out_bits).mean() > 0.98, name


def test_c_port_matches_numpy_oracle(golden):
    if oracle.load_port() is None:
        pytest.skip("oracle/libfa_mask_oracle.so not built")
    for name in (str(n) for n in golden["names"]):
        q, k, v, m, _, dt = _case(golden, name)
        for qp in (True, False):
            a = oracle._attn(q, k, v, m, dt, quantize_p=qp)
            b = oracle.port_attn(q, k, v, m, dt, quantize_p=qp)
            # P rounding can flip on a last-bit difference of exp(); 2^-9 relative on
            # one P entry times |v| is far below the 1e-3 used here.
            assert np.abs(a - b).max() < (1e-3 if qp else 2e-5), (name, qp)


def test_c_port_lse(golden):
    if oracle.load_port() is None:
        pytest.skip("oracle/libfa_mask_oracle.so not built")
    q, k, v, m, _, dt = _case(golden, "bf16_d64_causal_rowmasked")
    _, lse = oracle.port_attn(q, k, v, m, dt, want_lse=True)
    ref = oracle.lse_fp32(q, k, m, dt)
    assert np.all(np.isneginf(lse[:, :, 0]))           # fully masked row
    assert np.array_equal(np.isneginf(lse), np.isneginf(ref))
    fin = np.isfinite(ref)
    assert np.abs(lse[fin] - ref[fin]).max() < 1e-4


def test_fp32_oracle_close_to_ref_attn(golden):
    """The two oracle flavours differ only by the P rounding."""
    for name in (str(n) for n in golden["names"]):
        q, k, v, m, out_bits, dt = _case(golden, name)
        o = oracle.attn_fp32(q, k, v, m, dt)
        assert oracle.within_bar(oracle.to_f32(out_bits, dt), o), name


def test_fully_masked_row_is_zero(golden):
    q, k, v, m, out_bits, dt = _case(golden, "bf16_d64_causal_rowmasked")
    o = oracle.attn_fp32(q, k, v, m, dt)
    assert np.all(o[:, :, 0, :] == 0)
    assert np.all(oracle.to_f32(out_bits, dt)[:, :, 0, :] == 0)
    assert not np.isnan(o).any()


def test_pad_columns_are_ignored(golden):
    q, k, v, m, _, dt = _case(golden, "fp16_d64_padded_trap")
    Sq, Sk = q.shape[2], k.shape[2]
    assert m.shape[2] > Sq and m.shape[3] > Sk
    a = oracle.attn_fp32(q, k, v, m, dt)
    m2 = m.copy()
    m2[:, :, :, Sk:] = 0x7C00      # +inf in the pad columns must change nothing
    m2[:, :, Sq:, :] = 0x7C00
    b = oracle.attn_fp32(q, k, v, m2, dt)
    assert np.array_equal(a, b)


def test_gqa_head_mapping(golden):
    q, k, v, m, _, dt = _case(golden, "fp16_d128_gqa_bias")
    H, Hk = q.shape[1], k.shape[1]
    g = H // Hk
    full = oracle.attn_fp32(q, k, v, m, dt)
    k_rep = np.repeat(k, g, axis=1)
    v_rep = np.repeat(v, g, axis=1)
    assert np.array_equal(full, oracle.attn_fp32(q, k_rep, v_rep, m, dt))


def test_finite_bias_scale_order():
    """score = s*scale + mask, not (s + mask)*scale."""
    rng = np.random.default_rng(0)
    d = 64
    q = oracle.f32_to_bf16_bits(rng.standard_normal((1, 1, 4, d)).astype(np.float32))
    k = oracle.f32_to_bf16_bits(rng.standard_normal((1, 1, 8, d)).astype(np.float32))
    v = oracle.f32_to_bf16_bits(rng.standard_normal((1, 1, 8, d)).astype(np.float32))
    m = oracle.f32_to_bf16_bits((rng.standard_normal((1, 1, 4, 8)) * 2).astype(np.float32))
    o = oracle.attn_fp32(q, k, v, m, "bf16")
    qf, kf, vf, mf = (oracle.bf16_bits_to_f32(x) for x in (q, k, v, m))
    s = qf[0, 0] @ kf[0, 0].T / math.sqrt(d) + mf[0, 0]
    p = np.exp(s - s.max(-1, keepdims=True))
    want = (p / p.sum(-1, keepdims=True)) @ vf[0, 0]
    assert np.abs(o[0, 0] - want).max() < 1e-5


def test_bit_conversions_roundtrip():
    lib = oracle.load_port()
    xs = np.array([0.0, 1.0, -1.0, 0.1, 3.14159, 65504.0, 1e-7, 6e-8, 1e-8, 70000.0,
                   np.inf, -np.inf, 0.33325195], np.float32)
    for dt in ("bf16", "fp16"):
        b = oracle.to_bits(xs, dt)
        back = oracle.to_f32(b, dt)
        assert np.array_equal(oracle.to_bits(back, dt), b)
        if lib is not None:
            import ctypes
            lib.fa_mask_oracle_f32_to_bits.restype = ctypes.c_uint16
            lib.fa_mask_oracle_f32_to_bits.argtypes = [ctypes.c_float, ctypes.c_int]
            lib.fa_mask_oracle_bits_to_f32.restype = ctypes.c_float
            lib.fa_mask_oracle_bits_to_f32.argtypes = [ctypes.c_uint16, ctypes.c_int]
            for x, bb in zip(xs, b):
                assert lib.fa_mask_oracle_f32_to_bits(float(x), dt == "bf16") == int(bb), (x, dt)
                assert lib.fa_mask_oracle_bits_to_f32(int(bb), dt == "bf16") == \
                    float(oracle.to_f32(np.array([bb], np.uint16), dt)[0])


def test_reference_cpu_kernels_agree(golden):
    """The reference's compiled C++ CPU attention (oracle/_ref) against the oracle.
    Its kernels are fp32 end to end (no P rounding), so compare with attn_fp32."""
    if oracle.load_ref() is None:
        pytest.skip("oracle/_ref/libfa_ref_cpu.so not built (needs the reference checkout)")
    for name in (str(n) for n in golden["names"]):
        q, k, v, m, _, dt = _case(golden, name)
        want = oracle.attn_fp32(q, k, v, m, dt)
        for isa in ("scalar", oracle.ref_best_isa()):
            got = oracle.ref_cpu_attn(q, k, v, m, dt, isa=isa)
            assert not np.isnan(got).any(), (name, isa)
            assert np.abs(got - want).max() < 2e-4, (name, isa)
