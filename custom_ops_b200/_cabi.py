"""ctypes view of the C ABI in ``include/fa_mask_fwd_sm100.h``.

This is the torch-free way into the library: pointers and sizes only.  The
torch operator (``csrc/fa_bindings.cpp``) calls the same entry points from C++;
tests call them from here to check the ABI itself.  There is no fallback: when
the shared library is missing, loading raises.
"""
from __future__ import annotations

import ctypes
import os

from . import build as _build

ABI_VERSION = 2
FP16, BF16 = 0, 1
MAX_SPLITS = 128

ERRORS = {
    0: "OK", -1: "ERR_NULL", -2: "ERR_DTYPE", -3: "ERR_SHAPE", -4: "ERR_HEAD_DIM", -5: "ERR_ALIGN",
    -6: "ERR_WORKSPACE", -7: "ERR_ARCH", -8: "ERR_CUDA", -9: "ERR_SPLITS", -10: "ERR_DEVICE_WAIT",
    -11: "ERR_ABI",
}

EXPORTS = [
    "fa_mask_fwd_sm100_abi_version",
    "fa_mask_fwd_sm100_plan",
    "fa_mask_fwd_sm100_workspace_bytes",
    "fa_mask_fwd_sm100",
    "fa_mask_fwd_sm100_static_scratch",
    "fa_mask_build_sm100",
    "fa_mask_fwd_sm100_rule",
    "fa_mask_fwd_sm100_combine",
    "fa_mask_fwd_sm100_combine_packed",
    "fa_mask_fwd_sm100_combine_peers",
    "fa_mask_fwd_sm100_device_status",
    "fa_mask_fwd_sm100_launch_count",
    "fa_mask_fwd_sm100_strerror",
]


class FaMaskFwdArgs(ctypes.Structure):
    _fields_ = [
        ("struct_size", ctypes.c_uint32),
        ("device", ctypes.c_int32),
        ("q", ctypes.c_void_p),
        ("k", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("mask", ctypes.c_void_p),
        ("out", ctypes.c_void_p),
        ("lse", ctypes.c_void_p),
        ("batch", ctypes.c_int32),
        ("heads", ctypes.c_int32),
        ("heads_k", ctypes.c_int32),
        ("seqlen_q", ctypes.c_int32),
        ("seqlen_k", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("mask_seqlen_q", ctypes.c_int32),
        ("mask_seqlen_k", ctypes.c_int32),
        ("mask_batch_stride", ctypes.c_int64),
        ("mask_row_stride", ctypes.c_int64),
        ("dtype", ctypes.c_int32),
        ("num_splits", ctypes.c_int32),
        ("out_fp32", ctypes.c_int32),
        ("disable", ctypes.c_int32),
        ("mask_version", ctypes.c_uint64),
    ]


class FaMaskFwdPlan(ctypes.Structure):
    _fields_ = [
        ("num_splits", ctypes.c_int32),
        ("kv_blocks", ctypes.c_int32),
        ("blocks_per_split", ctypes.c_int32),
        ("q_tiles_per_cta", ctypes.c_int32),
        ("grid_x", ctypes.c_int32),
        ("grid_y", ctypes.c_int32),
        ("grid_z", ctypes.c_int32),
        ("threads", ctypes.c_int32),
        ("smem_bytes", ctypes.c_int32),
        ("mask_repitched", ctypes.c_int32),
        ("sm_count", ctypes.c_int32),
        ("dual_split", ctypes.c_int32),
        ("tile_skip", ctypes.c_int32),
        ("unit_cut", ctypes.c_int32),
        ("head_pairs", ctypes.c_int32),
        ("reserved0", ctypes.c_int32),
        ("workspace_bytes", ctypes.c_uint64),
    ]


class FaSm100Error(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"fa_mask_fwd_sm100: {text} ({ERRORS.get(code, code)})")
        self.code = code


_lib = None


def library_path() -> str:
    return _build.CABI_SO


def load(path: str | None = None):
    """dlopen the C-ABI library and declare its prototypes.  Raises when absent."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    path = path or library_path()
    if not os.path.exists(path):
        raise FileNotFoundError(
            f"{path} is not built; run `python -m custom_ops_b200.build` (needs nvcc)")
    lib = ctypes.CDLL(path)
    P = ctypes.POINTER
    lib.fa_mask_fwd_sm100_abi_version.restype = ctypes.c_int
    lib.fa_mask_fwd_sm100_abi_version.argtypes = []
    lib.fa_mask_fwd_sm100_plan.restype = ctypes.c_int
    lib.fa_mask_fwd_sm100_plan.argtypes = [P(FaMaskFwdArgs), P(FaMaskFwdPlan)]
    lib.fa_mask_fwd_sm100_workspace_bytes.restype = ctypes.c_int
    lib.fa_mask_fwd_sm100_workspace_bytes.argtypes = [P(FaMaskFwdArgs), P(ctypes.c_size_t)]
    lib.fa_mask_fwd_sm100.restype = ctypes.c_int
    lib.fa_mask_fwd_sm100.argtypes = [P(FaMaskFwdArgs), ctypes.c_void_p, ctypes.c_size_t,
                                      ctypes.c_void_p]
    lib.fa_mask_fwd_sm100_static_scratch.restype = ctypes.c_int
    lib.fa_mask_fwd_sm100_static_scratch.argtypes = [P(FaMaskFwdArgs), ctypes.c_void_p]
    lib.fa_mask_fwd_sm100_combine.restype = ctypes.c_int
    lib.fa_mask_fwd_sm100_combine.argtypes = [
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32,
        ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
        ctypes.c_void_p]
    lib.fa_mask_fwd_sm100_combine_packed.restype = ctypes.c_int
    lib.fa_mask_fwd_sm100_combine_packed.argtypes = [
        ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32,
        ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
        ctypes.c_void_p]
    lib.fa_mask_fwd_sm100_combine_peers.restype = ctypes.c_int
    lib.fa_mask_fwd_sm100_combine_peers.argtypes = [
        ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_uint32,
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
        ctypes.c_int32, ctypes.c_void_p]
    lib.fa_mask_fwd_sm100_rule.restype = ctypes.c_int
    lib.fa_mask_fwd_sm100_rule.argtypes = [P(FaMaskFwdArgs), ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p,
                                           ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
    lib.fa_mask_build_sm100.restype = ctypes.c_int
    lib.fa_mask_build_sm100.argtypes = [
        ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
        ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p]
    lib.fa_mask_fwd_sm100_device_status.restype = ctypes.c_int
    lib.fa_mask_fwd_sm100_device_status.argtypes = [ctypes.c_int32, P(ctypes.c_uint32),
                                                    ctypes.c_int32]
    lib.fa_mask_fwd_sm100_launch_count.restype = ctypes.c_int
    lib.fa_mask_fwd_sm100_launch_count.argtypes = [P(ctypes.c_uint64)]
    lib.fa_mask_fwd_sm100_strerror.restype = ctypes.c_char_p
    lib.fa_mask_fwd_sm100_strerror.argtypes = [ctypes.c_int]
    if lib.fa_mask_fwd_sm100_abi_version() != ABI_VERSION:
        raise RuntimeError("libfa_mask_sm100.so was built from a different ABI version")
    if path == library_path():
        _lib = lib
    return lib


def strerror(code: int) -> str:
    return load().fa_mask_fwd_sm100_strerror(code).decode()


def check(code: int):
    if code != 0:
        raise FaSm100Error(code, strerror(code))


NO_TILE_SKIP = 1      # FaMaskFwdArgs.disable bits (FA_SM100_NO_*)
NO_UNIT_CUT = 2
NO_HEAD_PAIRS = 4
TEST_STALL_MASK = 0x100   # tests only: withhold the mask loads so that a bounded wait runs out


def make_args(*, q=0, k=0, v=0, mask=0, out=0, lse=0, batch, heads, heads_k, seqlen_q, seqlen_k,
              head_dim, dtype, mask_seqlen_q=None, mask_seqlen_k=None, mask_batch_stride=None,
              mask_row_stride=None, device=0, num_splits=0, out_fp32=0,
              no_tile_skip=0, no_unit_cut=0, test_stall_mask=0, no_head_pairs=0, mask_version=0) -> FaMaskFwdArgs:
    a = FaMaskFwdArgs()
    a.struct_size = ctypes.sizeof(FaMaskFwdArgs)
    a.device = device
    a.q, a.k, a.v, a.mask, a.out, a.lse = q or None, k or None, v or None, mask or None, \
        out or None, lse or None
    a.batch, a.heads, a.heads_k = batch, heads, heads_k
    a.seqlen_q, a.seqlen_k, a.head_dim = seqlen_q, seqlen_k, head_dim
    a.mask_seqlen_q = seqlen_q if mask_seqlen_q is None else mask_seqlen_q
    a.mask_seqlen_k = seqlen_k if mask_seqlen_k is None else mask_seqlen_k
    a.mask_row_stride = a.mask_seqlen_k if mask_row_stride is None else mask_row_stride
    a.mask_batch_stride = (a.mask_seqlen_q * a.mask_row_stride if mask_batch_stride is None
                           else mask_batch_stride)
    a.dtype = dtype
    a.num_splits = num_splits
    a.out_fp32 = out_fp32
    a.disable = ((NO_TILE_SKIP if no_tile_skip else 0) | (NO_UNIT_CUT if no_unit_cut else 0)
                 | (NO_HEAD_PAIRS if no_head_pairs else 0)
                 | (TEST_STALL_MASK if test_stall_mask else 0))
    a.mask_version = mask_version
    return a


def plan(args: FaMaskFwdArgs) -> FaMaskFwdPlan:
    p = FaMaskFwdPlan()
    check(load().fa_mask_fwd_sm100_plan(ctypes.byref(args), ctypes.byref(p)))
    return p


def workspace_bytes(args: FaMaskFwdArgs) -> int:
    n = ctypes.c_size_t(0)
    check(load().fa_mask_fwd_sm100_workspace_bytes(ctypes.byref(args), ctypes.byref(n)))
    return int(n.value)


def forward(args: FaMaskFwdArgs, workspace: int, workspace_nbytes: int, stream: int):
    check(load().fa_mask_fwd_sm100(ctypes.byref(args), workspace or None, workspace_nbytes,
                                   stream or None))


STATIC_SCRATCH_BYTES = 24 * 1024 * 1024


def forward_static_scratch(args: FaMaskFwdArgs, stream: int):
    """The forward on the library's built-in scratch: nothing is allocated anywhere.
    Calls that may overlap on the GPU must not share it (they would race)."""
    check(load().fa_mask_fwd_sm100_static_scratch(ctypes.byref(args), stream or None))


def combine(o_parts: int, lse_parts: int, out: int, lse_out: int, num_parts: int, rows: int,
            head_dim: int, dtype: int, out_fp32: int, device: int, stream: int):
    check(load().fa_mask_fwd_sm100_combine(o_parts or None, lse_parts or None, out or None,
                                           lse_out or None, num_parts, rows, head_dim, dtype,
                                           out_fp32, device, stream or None))


def combine_packed(packed: int, part_stride: int, out: int, lse_out: int, num_parts: int, rows: int,
                   head_dim: int, dtype: int, out_fp32: int, device: int, stream: int):
    """Merge of parts laid out [O (rows*d) | LSE (rows)] every ``part_stride`` floats."""
    check(load().fa_mask_fwd_sm100_combine_packed(packed or None, part_stride, out or None,
                                                  lse_out or None, num_parts, rows, head_dim, dtype,
                                                  out_fp32, device, stream or None))


def combine_peers(part_table: int, part_offset: int, flag_offset: int, rank: int, world: int, seq: int,
                  out: int, lse_out: int, rows: int, head_dim: int, dtype: int, out_fp32: int, device: int,
                  stream: int):
    """Merge with the exchange through peer-addressable memory built in (see the header)."""
    check(load().fa_mask_fwd_sm100_combine_peers(part_table or None, part_offset, flag_offset, rank, world,
                                                 seq, out or None, lse_out or None, rows, head_dim, dtype,
                                                 out_fp32, device, stream or None))


def build_mask(mask: int, batch: int, seqlen_q: int, seqlen_k: int, pitch: int, dtype: int, causal: int,
               window: int, valid_lens: int, device: int, stream: int):
    check(load().fa_mask_build_sm100(mask or None, batch, seqlen_q, seqlen_k, pitch, dtype, causal, window,
                                     valid_lens or None, device, stream or None))


def device_status(device: int = 0, clear: bool = True) -> int:
    """Synchronises the device; returns the sticky status word (0 = clean)."""
    st = ctypes.c_uint32(0)
    rc = load().fa_mask_fwd_sm100_device_status(device, ctypes.byref(st), 1 if clear else 0)
    if rc not in (0, -10):
        check(rc)
    return int(st.value)


RULE_WORKSPACE_BYTES = 16


def forward_rule(args: FaMaskFwdArgs, causal: int, window: int, valid_lens: int, stream: int,
                 workspace: int = 0, workspace_nbytes: int = 0):
    """The forward for a mask given by rules (causal / sliding window / valid lengths) instead of
    a tensor; ``valid_lens`` is a device pointer to ``batch`` int32 or 0; ``workspace``:
    ``RULE_WORKSPACE_BYTES`` of device memory private to the call, or 0."""
    check(load().fa_mask_fwd_sm100_rule(ctypes.byref(args), int(causal), int(window), valid_lens or None,
                                        workspace or None, workspace_nbytes, stream or None))


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    n = ctypes.c_uint64(0)
    check(load().fa_mask_fwd_sm100_launch_count(ctypes.byref(n)))
    return int(n.value)
