"""CPU oracle for ``mha_fwd_with_mask`` -- TEST INFRASTRUCTURE, not a product path.

Only the test-suite, the smoke check and the CPU-baseline legs of the benchmark
may import this module.  The shipped operator never routes through it.

Two restatements of the reference semantics in numpy (fp32 arithmetic):

* :func:`ref_attn` follows the reference's own test oracle
  (``tests/test_mha_fwd_with_mask.py:38-53``): scores ``(q*scale) @ k^T + mask``
  in fp32, row max clamped below at ``-1e30`` so a fully masked row yields
  ``exp(-inf) = 0`` instead of NaN, denominator clamped at ``1e-38`` so that row
  becomes exactly 0, **P rounded to the input dtype before the PV product**
  (mirrors the kernel's P quantisation, ``csrc/fa/sm89/fa_fwd_kernel.h:432-435``),
  result rounded to the input dtype.
* :func:`attn_fp32` is the same without the P rounding: the plain
  ``softmax(QK^T * scale + mask) V`` in fp32 that the accuracy bar
  (max-abs 2e-2, mean-abs 2e-3) is stated against.

GQA maps query head ``h`` to kv head ``h // (H // Hk)``
(``csrc/fa/sm89/fa_fwd_kernel.h:114,121``).  A mask larger than ``(Sq, Sk)`` is
cropped: columns ``>= Sk`` are always masked and rows ``>= Sq`` are never read
(``csrc/fa/fa_fwd_op.cu:96-108``).

Parity pin: the functions here are checked against outputs of the reference's
``ref_attn`` itself (fixtures under ``tests/golden/``, written by
``tests/golden/make_golden.py`` which imports the reference test module) and
against the reference's compiled C++ CPU kernels (``oracle/_ref``).

16-bit tensors travel as ``uint16`` bit patterns plus a dtype tag ("bf16" or
"fp16") because numpy has no bfloat16.
"""
from __future__ import annotations

import ctypes
import math
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

# --------------------------------------------------------------------------- #
# 16-bit <-> fp32 conversions (round to nearest even, like torch's .to(dtype)) #
# --------------------------------------------------------------------------- #


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    rounded = (u + (((u >> 16) & 1) + np.uint32(0x7FFF))) >> 16
    # NaN keeps a quiet-NaN pattern instead of rounding into infinity.
    out = np.where(np.isnan(x), np.uint32(0x7FC0), rounded)
    return out.astype(np.uint16)


def fp16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return bits.view(np.float16).astype(np.float32)


def f32_to_fp16_bits(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def to_f32(bits: np.ndarray, dtype: str) -> np.ndarray:
    if dtype == "bf16":
        return bf16_bits_to_f32(bits)
    if dtype == "fp16":
        return fp16_bits_to_f32(bits)
    raise ValueError(f"dtype must be 'bf16' or 'fp16', got {dtype!r}")


def to_bits(x: np.ndarray, dtype: str) -> np.ndarray:
    if dtype == "bf16":
        return f32_to_bf16_bits(x)
    if dtype == "fp16":
        return f32_to_fp16_bits(x)
    raise ValueError(f"dtype must be 'bf16' or 'fp16', got {dtype!r}")


def quantize(x: np.ndarray, dtype: str) -> np.ndarray:
    """fp32 -> dtype -> fp32."""
    return to_f32(to_bits(x, dtype), dtype)


# --------------------------------------------------------------------------- #
# The attention restatements                                                    #
# --------------------------------------------------------------------------- #


def _check_shapes(q, k, v, mask):
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4 or mask.ndim != 4:
        raise ValueError("q, k, v, mask must be 4-D")
    B, H, Sq, d = q.shape
    Bk, Hk, Sk, dk = k.shape
    if Bk != B or v.shape != k.shape or dk != d or mask.shape[0] != B:
        raise ValueError("batch / head_dim / seqlen_k mismatch")
    if H % Hk:
        raise ValueError("n_heads must be divisible by n_kv_heads")
    if mask.shape[1] != 1 or mask.shape[2] < Sq or mask.shape[3] < Sk:
        raise ValueError("mask shape must be (B, 1, >=Sq, >=Sk)")
    return B, H, Hk, Sq, Sk, d


def _attn(qb, kb, vb, mb, dtype: str, quantize_p: bool):
    B, H, Hk, Sq, Sk, d = _check_shapes(qb, kb, vb, mb)
    q = to_f32(qb, dtype)
    k = to_f32(kb, dtype)
    v = to_f32(vb, dtype)
    m = to_f32(mb[:, :, :Sq, :Sk], dtype)
    g = H // Hk
    scale = np.float32(1.0 / math.sqrt(d))
    out = np.zeros((B, H, Sq, d), dtype=np.float32)
    with np.errstate(invalid="ignore", over="ignore"):
        for b in range(B):
            for h in range(H):
                hk = h // g
                s = (q[b, h] * scale) @ k[b, hk].T           # (Sq, Sk) fp32
                s = s + m[b, 0]
                row_max = np.maximum(s.max(axis=-1, keepdims=True), np.float32(-1e30)) \
                    if Sk > 0 else np.full((Sq, 1), -1e30, np.float32)
                p = np.exp(s - row_max)
                denom = np.maximum(p.sum(axis=-1, keepdims=True, dtype=np.float32),
                                   np.float32(1e-38))
                p = p / denom
                if quantize_p:
                    p = quantize(p, dtype)
                out[b, h] = p @ v[b, hk]
    return out


def ref_attn(q_bits, k_bits, v_bits, mask_bits, dtype: str):
    """Reference test-oracle semantics.  Returns (fp32 result, dtype bit patterns)."""
    o = _attn(q_bits, k_bits, v_bits, mask_bits, dtype, quantize_p=True)
    return o, to_bits(o, dtype)


def attn_fp32(q_bits, k_bits, v_bits, mask_bits, dtype: str) -> np.ndarray:
    """Plain fp32 softmax(QK^T*scale + mask) V on the dtype-rounded inputs."""
    return _attn(q_bits, k_bits, v_bits, mask_bits, dtype, quantize_p=False)


def lse_fp32(q_bits, k_bits, mask_bits, dtype: str) -> np.ndarray:
    """Row log-sum-exp ``max*1 + ln(sum)`` of the scaled, masked scores; ``-inf``
    for a fully masked row (``csrc/fa/common/softmax.h:145``).  Shape (B,H,Sq)."""
    B, H, Sq, d = q_bits.shape
    Hk, Sk = k_bits.shape[1], k_bits.shape[2]
    q = to_f32(q_bits, dtype)
    k = to_f32(k_bits, dtype)
    m = to_f32(mask_bits[:, :, :Sq, :Sk], dtype)
    g = H // Hk
    scale = np.float32(1.0 / math.sqrt(d))
    out = np.empty((B, H, Sq), np.float32)
    with np.errstate(invalid="ignore", over="ignore", divide="ignore"):
        for b in range(B):
            for h in range(H):
                s = (q[b, h] * scale) @ k[b, h // g].T + m[b, 0]
                mx = s.max(axis=-1)
                safe = np.where(np.isfinite(mx), mx, np.float32(0))
                out[b, h] = np.where(np.isfinite(mx),
                                     safe + np.log(np.exp(s - safe[:, None]).sum(-1)),
                                     -np.inf)
    return out


# --------------------------------------------------------------------------- #
# Error metrics and the two pass rules                                          #
# --------------------------------------------------------------------------- #

MAX_ABS_TOL = 2e-2    # accuracy bar vs the fp32 oracle, bf16/fp16 outputs
MEAN_ABS_TOL = 2e-3
REF_ATOL = 1e-2       # tests/test_mha_fwd_with_mask.py:32-33
REF_RTOL = 1e-2


def errors(out_f32: np.ndarray, ref_f32: np.ndarray):
    diff = np.abs(out_f32.astype(np.float64) - ref_f32.astype(np.float64))
    return float(diff.max()) if diff.size else 0.0, float(diff.mean()) if diff.size else 0.0


def within_bar(out_f32, ref_f32) -> bool:
    if not np.all(np.isfinite(out_f32)):
        return False
    mx, mean = errors(out_f32, ref_f32)
    return mx <= MAX_ABS_TOL and mean <= MEAN_ABS_TOL


def within_reference_rule(out_f32, ref_f32) -> bool:
    """``max_err < 1e-2 or max_err / max|ref| < 1e-2`` (tests/test_mha_fwd_with_mask.py:61-64)."""
    if not np.all(np.isfinite(out_f32)):
        return False
    mx, _ = errors(out_f32, ref_f32)
    ref_abs = float(np.abs(ref_f32).max()) + 1e-8 if ref_f32.size else 1.0
    return mx < REF_ATOL or mx / ref_abs < REF_RTOL


# --------------------------------------------------------------------------- #
# ctypes access to the compiled checkers                                        #
# --------------------------------------------------------------------------- #

_port_lib = None
_ref_lib = None


def port_lib_path() -> str:
    return os.path.join(_HERE, "libfa_mask_oracle.so")


def ref_lib_path() -> str:
    return os.path.join(_HERE, "_ref", "libfa_ref_cpu.so")


def load_port():
    """The plain-C restatement (oracle/fa_mask_oracle.c); None when not built."""
    global _port_lib
    if _port_lib is None and os.path.exists(port_lib_path()):
        lib = ctypes.CDLL(port_lib_path())
        lib.fa_mask_oracle_fwd.restype = ctypes.c_int
        lib.fa_mask_oracle_fwd.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_void_p, ctypes.c_void_p] + \
            [ctypes.c_int] * 11
        _port_lib = lib
    return _port_lib


def port_attn(q_bits, k_bits, v_bits, mask_bits, dtype: str, quantize_p: bool = True,
              n_threads: int = 0, want_lse: bool = False):
    """Run the C restatement.  Returns fp32 output (and LSE when asked)."""
    lib = load_port()
    if lib is None:
        raise RuntimeError("oracle/libfa_mask_oracle.so is not built (make -C oracle port)")
    B, H, Hk, Sq, Sk, d = _check_shapes(q_bits, k_bits, v_bits, mask_bits)
    q = np.ascontiguousarray(q_bits, np.uint16)
    k = np.ascontiguousarray(k_bits, np.uint16)
    v = np.ascontiguousarray(v_bits, np.uint16)
    m = np.ascontiguousarray(mask_bits, np.uint16)
    out = np.empty((B, H, Sq, d), np.float32)
    lse = np.empty((B, H, Sq), np.float32) if want_lse else None
    rc = lib.fa_mask_oracle_fwd(
        q.ctypes.data, k.ctypes.data, v.ctypes.data, m.ctypes.data, out.ctypes.data,
        lse.ctypes.data if want_lse else None,
        B, H, Hk, Sq, Sk, d, m.shape[2], m.shape[3],
        1 if dtype == "bf16" else 0, 1 if quantize_p else 0, n_threads)
    if rc != 0:
        raise RuntimeError(f"fa_mask_oracle_fwd failed with {rc}")
    return (out, lse) if want_lse else out


def load_ref():
    """The reference's own C++ CPU kernels (csrc/fa/cpu), built by `make -C oracle ref`
    from the sources under the reference checkout; None when not built.  The
    library links libtorch, so torch is imported first."""
    global _ref_lib
    if _ref_lib is None and os.path.exists(ref_lib_path()):
        import torch  # noqa: F401  (brings libtorch/libc10 into the process)
        lib = ctypes.CDLL(ref_lib_path())
        _ref_lib = lib
    return _ref_lib


# C++ symbol names of the reference's raw kernels (csrc/fa/cpu/fa_fwd_cpu.h:171-204):
# void fa_fwd_cpu_kernel_<isa>(const float*, const float*, const float*, const float*,
#                              float*, int, int, int, int, int, float, int)
_REF_SYMS = {
    "scalar": "_Z24fa_fwd_cpu_kernel_scalarPKfS0_S0_S0_Pfiiiiifi",
    "avx2": "_Z22fa_fwd_cpu_kernel_avx2PKfS0_S0_S0_Pfiiiiifi",
    "avx512": "_Z24fa_fwd_cpu_kernel_avx512PKfS0_S0_S0_Pfiiiiifi",
}


def _cpu_flags():
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def ref_best_isa() -> str:
    """Mirror of the reference's run-time choice (csrc/fa/cpu/fa_fwd_cpu.cpp:305-306)."""
    flags = _cpu_flags()
    if {"avx512f", "avx512dq"} <= flags:
        return "avx512"
    if {"avx2", "fma"} <= flags:
        return "avx2"
    return "scalar"


def ref_cpu_attn(q_bits, k_bits, v_bits, mask_bits, dtype: str, isa: str | None = None,
                 n_threads: int = 0) -> np.ndarray:
    """Call the reference's raw fp32 CPU kernel batch by batch.  Inputs are
    widened to fp32 first (the kernels take fp32 buffers, mask exactly (Sq,Sk))."""
    lib = load_ref()
    if lib is None:
        raise RuntimeError("oracle/_ref/libfa_ref_cpu.so is not built (make -C oracle ref)")
    isa = isa or ref_best_isa()
    fn = getattr(lib, _REF_SYMS[isa])
    fn.restype = None
    fn.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 5 + [ctypes.c_float, ctypes.c_int]
    B, H, Hk, Sq, Sk, d = _check_shapes(q_bits, k_bits, v_bits, mask_bits)
    q = to_f32(q_bits, dtype)
    k = to_f32(k_bits, dtype)
    v = to_f32(v_bits, dtype)
    m = np.ascontiguousarray(to_f32(mask_bits[:, :, :Sq, :Sk], dtype))
    out = np.empty((B, H, Sq, d), np.float32)
    nt = n_threads or min(H, os.cpu_count() or 1)
    for b in range(B):
        qb, kb, vb, mb = (np.ascontiguousarray(x) for x in (q[b], k[b], v[b], m[b, 0]))
        fn(qb.ctypes.data, kb.ctypes.data, vb.ctypes.data, mb.ctypes.data,
           out[b].ctypes.data, H, Hk, Sq, Sk, d, ctypes.c_float(1.0 / math.sqrt(d)), nt)
    return out
