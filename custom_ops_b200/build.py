"""In-tree build of the two native libraries of the masked-attention group.

* ``libfa_mask_sm100.so`` -- the CUDA kernels and the C ABI
  (``include/fa_mask_fwd_sm100.h``); nvcc, sm_100a only, no torch.
* ``recsys_fa_kernel.so`` -- the torch operator registration
  (``csrc/fa_bindings.cpp``); host compiler against the torch headers, linked to
  the first library.  The name is the reference group's ``so_name``
  (``recsys.py:171``).

Both land next to this file so they travel with the source tree; nothing is
written to a per-user JIT cache.  The reference builds through
``torch.utils.cpp_extension`` with a content-hash stamp and a file lock
(``__init__.py:566-629, 1011-1067``); the same stamp idea is used here so a
second call is a no-op.

Run ``python -m custom_ops_b200.build`` to build both.
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG_DIR), "include")

CABI_SO = os.path.join(PKG_DIR, "libfa_mask_sm100.so")
TORCH_SO = os.path.join(PKG_DIR, "recsys_fa_kernel.so")

CABI_SOURCES = [os.path.join(CSRC, "fa_mask_fwd_sm100.cu")]
CABI_HEADERS = [os.path.join(CSRC, "sm100_ptx.cuh"), os.path.join(CSRC, "arch_targets.h"),
                os.path.join(INCLUDE, "fa_mask_fwd_sm100.h")]
TORCH_SOURCES = [os.path.join(CSRC, "fa_bindings.cpp")]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-DFA_TARGETS=0x8", "-shared", "-Xcompiler", "-fPIC"]


class BuildError(RuntimeError):
    pass


def _cuda_home() -> str:
    return os.environ.get("CUDA_HOME") or os.environ.get("CUDA_PATH") or "/usr/local/cuda"


def _nvcc() -> str:
    cand = os.path.join(_cuda_home(), "bin", "nvcc")
    if os.path.exists(cand):
        return cand
    found = shutil.which("nvcc")
    if not found:
        raise BuildError("nvcc not found (set CUDA_HOME)")
    return found


def _host_cxx() -> str:
    # The image's preset CXX wrapper lacks some link specs; prefer the system g++.
    for cand in (os.environ.get("CUSTOM_OPS_CXX"), "/usr/bin/g++", shutil.which("g++")):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("no host C++ compiler found")


def _fingerprint(paths, extra: str) -> str:
    """Hash of the build inputs: flags, file names and contents -- not the directory the tree
    happens to live in, so a tree that was built in one place and copied to another (with its
    libraries and stamps) is still up to date there and is not rebuilt under a process that
    already holds the old library."""
    h = hashlib.sha256(extra.encode())
    for p in paths:
        with open(p, "rb") as f:
            h.update(os.path.basename(p).encode() + b"\0" + f.read())
    return h.hexdigest()


def _up_to_date(so: str, fp: str) -> bool:
    stamp = so + ".build_stamp"
    if not (os.path.exists(so) and os.path.exists(stamp)):
        return False
    with open(stamp) as f:
        return f.read().strip() == fp


def _run(cmd, what: str, verbose: bool):
    if verbose:
        print("[custom_ops_b200.build]", " ".join(cmd), file=sys.stderr)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"{what} failed ({r.returncode}):\n{r.stdout}\n{r.stderr}")
    return r


def _locked(so: str):
    lock = open(so + ".lock", "w")
    fcntl.flock(lock, fcntl.LOCK_EX)
    return lock


def build_cabi(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    """Compile the kernels + C ABI for sm_100a.  Returns the library path."""
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_info else [])
    fp = _fingerprint(CABI_SOURCES + CABI_HEADERS, " ".join(flags))
    lock = _locked(CABI_SO)
    try:
        if not force and _up_to_date(CABI_SO, fp):
            return CABI_SO
        tmp = CABI_SO + ".tmp"
        r = _run([_nvcc()] + flags + ["-I", INCLUDE, "-I", CSRC, "-o", tmp] + CABI_SOURCES,
                 "nvcc (C-ABI library)", verbose)
        if ptxas_info:
            print(r.stderr, file=sys.stderr)
        os.replace(tmp, CABI_SO)
        with open(CABI_SO + ".build_stamp", "w") as f:
            f.write(fp)
        return CABI_SO
    finally:
        lock.close()


def build_torch_binding(force: bool = False, verbose: bool = False) -> str:
    """Compile the torch operator registration and link it to the C-ABI library."""
    import torch

    build_cabi(verbose=verbose)
    tdir = os.path.dirname(torch.__file__)
    abi = int(torch.compiled_with_cxx11_abi())
    flags = ["-O2", "-std=c++17", "-fPIC", "-shared", "-w",
             f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=recsys_fa_kernel",
             "-DTORCH_API_INCLUDE_EXTENSION_H"]
    fp = _fingerprint(TORCH_SOURCES + [os.path.join(INCLUDE, "fa_mask_fwd_sm100.h")],
                      " ".join(flags) + torch.__version__)
    lock = _locked(TORCH_SO)
    try:
        if not force and _up_to_date(TORCH_SO, fp):
            return TORCH_SO
        inc = ["-I", os.path.join(tdir, "include"),
               "-I", os.path.join(tdir, "include", "torch", "csrc", "api", "include"),
               "-I", sysconfig.get_paths()["include"], "-I", os.path.join(_cuda_home(), "include"),
               "-I", INCLUDE]
        libs = ["-L", os.path.join(tdir, "lib"), "-L", PKG_DIR,
                "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{os.path.join(tdir, 'lib')}",
                "-l:libfa_mask_sm100.so", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda",
                "-ltorch", "-ltorch_python"]
        tmp = TORCH_SO + ".tmp"
        _run([_host_cxx()] + flags + inc + ["-o", tmp] + TORCH_SOURCES + libs,
             "host compile (torch binding)", verbose)
        os.replace(tmp, TORCH_SO)
        with open(TORCH_SO + ".build_stamp", "w") as f:
            f.write(fp)
        return TORCH_SO
    finally:
        lock.close()


def build_all(force: bool = False, verbose: bool = False):
    return build_cabi(force, verbose), build_torch_binding(force, verbose)


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true", help="print registers / spills per kernel")
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    print(build_cabi(a.force, a.verbose, a.ptxas_info))
    print(build_torch_binding(a.force, a.verbose))
