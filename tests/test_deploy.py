"""Offline export + strict loading (the deployment half of the loader contract).

Mirrors what the reference pins in ``tests/test_custom_ops_loading.py`` for its own loader:
an export never loads, a strict load never compiles, and every mismatch between the JSON
sidecar, the Python wrapper, the runtime and the bytes on disk is refused BEFORE dlopen.
No GPU is needed: the operator library loads on a CPU-only machine, only calling it does not.
"""
import json
import os
import shutil
import subprocess
import sys

import pytest
import torch

from custom_ops_b200 import CustomOpsError, FAOps
from custom_ops_b200 import deploy

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def exported(tmp_path_factory):
    """One export shared by the tests below; each test copies what it wants to break."""
    d = tmp_path_factory.mktemp("export")
    path = FAOps().export(str(d))
    return path


def _copy_export(exported, tmp_path):
    src = os.path.dirname(exported)
    dst = tmp_path / "copy"
    shutil.copytree(src, dst)
    return str(dst / os.path.basename(exported))


def _rewrite(path, edit, refingerprint=True):
    side = deploy.sidecar_path(path)
    meta = json.load(open(side))
    edit(meta)
    if refingerprint:
        meta["build_fingerprint"] = deploy.metadata_fingerprint(meta)
    json.dump(meta, open(side, "w"))


def _run_fresh(code, **env_extra):
    env = dict(os.environ)
    env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
    env.update(env_extra)
    return subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=600)


def test_export_describes_both_libraries(exported):
    d = os.path.dirname(exported)
    meta = json.load(open(deploy.sidecar_path(exported)))
    assert meta["producer"] == "custom_ops_b200" and meta["format_version"] == deploy.FORMAT_VERSION
    assert meta["namespace"] == "recsys_ops" and meta["so_name"] == "recsys_fa_kernel"
    assert meta["required_ops"] == ["mha_fwd_with_mask"]
    assert meta["fake_ops"] == ["mha_fwd_rule_mask", "mha_fwd_with_mask", "mha_fwd_with_mask_lse"]
    assert meta["schemas"]["mha_fwd_with_mask"].startswith("recsys_ops::mha_fwd_with_mask(Tensor q")
    assert meta["with_cuda"] is True and meta["cuda_arch_list"] == ["10.0a"]
    assert meta["library"]["filename"] == os.path.basename(exported)
    assert [c["filename"] for c in meta["companions"]] == ["libfa_mask_sm100.so"]
    for entry in [meta["library"]] + meta["companions"]:
        p = os.path.join(d, entry["filename"])
        assert os.path.getsize(p) == entry["size"] and deploy.file_sha256(p) == entry["sha256"]
    assert meta["build_fingerprint"] == deploy.metadata_fingerprint(meta)
    assert not [n for n in os.listdir(d) if n.endswith(".part")]
    assert deploy.check_precompiled(FAOps(), exported)["source_fingerprint"] == meta["source_fingerprint"]


def test_export_does_not_load_and_strict_load_does_not_compile(exported):
    """Fresh processes: (1) after an export the operator is not registered; (2) a strict load of
    the export works with no compiler reachable, registers schema and fake kernel, is idempotent,
    and a second provider of the same operator (the in-tree build) is refused."""
    r = _run_fresh(
        "import torch, tempfile\n"
        "from custom_ops_b200 import FAOps\n"
        "p = FAOps().export(tempfile.mkdtemp())\n"
        "try:\n"
        "    torch._C._get_schema('recsys_ops::mha_fwd_with_mask', '')\n"
        "    print('REGISTERED')\n"
        "except RuntimeError:\n"
        "    print('NOT-LOADED', p)\n")
    assert "NOT-LOADED" in r.stdout, r.stdout + r.stderr
    code = (
        "import os, torch\n"
        "from custom_ops_b200 import FAOps, RecsysOps, CustomOpsError\n"
        "from custom_ops_b200 import build\n"
        "def no_build(*a, **k): raise AssertionError('a strict load must not build')\n"
        "build.build_cabi = build.build_torch_binding = build._run = no_build\n"
        f"path = {exported!r}\n"
        "ops = RecsysOps(allow_jit=False)\n"
        "assert not ops.is_available('fa')\n"
        "ops.load_precompiled('fa', path)\n"
        "assert ops.is_available('fa') and ops.groups == {'fa': 'loaded'}\n"
        "g = ops._group('fa')\n"
        "assert g.library_path == path and g.metadata_path == path + '.json'\n"
        "q = torch.empty(2, 4, 8, 64, dtype=torch.bfloat16, device='meta')\n"
        "m = torch.empty(2, 1, 8, 8, dtype=torch.bfloat16, device='meta')\n"
        "o = torch.ops.recsys_ops.mha_fwd_with_mask(q, q, q, m)\n"
        "assert o.shape == q.shape and o.device.type == 'meta'\n"
        "ops.load_precompiled('fa', path)\n"
        "other = FAOps(allow_jit=False)\n"
        "try:\n"
        "    other.load_precompiled()\n"
        "    print('SECOND-PROVIDER-ACCEPTED')\n"
        "except CustomOpsError as e:\n"
        "    print('OK', e)\n")
    r = _run_fresh(code, PATH="/usr/bin:/bin", CUDA_HOME="/nonexistent")
    assert r.returncode == 0 and "OK" in r.stdout and "ACCEPTED" not in r.stdout, r.stdout + r.stderr


def test_every_mismatch_is_refused_before_dlopen(exported, tmp_path, monkeypatch):
    def forbidden(path):
        raise AssertionError(f"dlopen of {path}: the check should have refused it")
    monkeypatch.setattr(torch.ops, "load_library", forbidden)

    def refused(path, match, group=None, **kw):
        with pytest.raises(CustomOpsError, match=match):
            (group or FAOps(allow_jit=False)).load_precompiled(path, **kw)

    refused(str(tmp_path / "nothing.so"), "library not found")
    p = _copy_export(exported, tmp_path / "a")
    os.remove(deploy.sidecar_path(p))
    refused(p, "metadata not found")
    p = _copy_export(exported, tmp_path / "b")
    open(deploy.sidecar_path(p), "w").write("[1, 2]")
    refused(p, "must be a JSON object")
    p = _copy_export(exported, tmp_path / "c")
    _rewrite(p, lambda m: m.update(so_name="other_kernel"))
    refused(p, "so_name mismatch")
    p = _copy_export(exported, tmp_path / "d")
    _rewrite(p, lambda m: m["schemas"].update(mha_fwd_with_mask="recsys_ops::mha_fwd_with_mask(Tensor q) -> Tensor"))
    refused(p, "schemas mismatch")
    p = _copy_export(exported, tmp_path / "e")
    _rewrite(p, lambda m: m.update(required_ops=["mha_fwd_with_mask", "extra"]))
    refused(p, "required_ops mismatch")
    p = _copy_export(exported, tmp_path / "f")
    _rewrite(p, lambda m: m["compatibility"].update(torch="1.13"))
    refused(p, r"torch mismatch")
    p = _copy_export(exported, tmp_path / "g")
    _rewrite(p, lambda m: m.update(fake_ops=[]), refingerprint=False)
    refused(p, "fake_ops mismatch")
    p = _copy_export(exported, tmp_path / "h")
    _rewrite(p, lambda m: m["library"].update(size=m["library"]["size"] + 1), refingerprint=False)
    refused(p, "build fingerprint is invalid")
    # the wrapper decides whether CUDA is needed: metadata cannot declare it away
    p = _copy_export(exported, tmp_path / "i")
    _rewrite(p, lambda m: m.update(with_cuda=False, cuda_arch_list=[]))
    refused(p, "CUDA requirement")
    p = _copy_export(exported, tmp_path / "j")
    with open(p, "ab") as f:
        f.write(b"\0")
    refused(p, "hash/size mismatch")
    p = _copy_export(exported, tmp_path / "k")
    with open(os.path.join(os.path.dirname(p), "libfa_mask_sm100.so"), "r+b") as f:
        f.seek(4096)
        byte = f.read(1)
        f.seek(4096)
        f.write(bytes([byte[0] ^ 0xFF]))
    refused(p, "hash/size mismatch")
    p = _copy_export(exported, tmp_path / "l")
    os.remove(os.path.join(os.path.dirname(p), "libfa_mask_sm100.so"))
    refused(p, "companion library not found")
    # a sidecar given explicitly, for a library of another name
    p = _copy_export(exported, tmp_path / "m")
    renamed = os.path.join(os.path.dirname(p), "renamed.so")
    os.rename(p, renamed)
    refused(renamed, "describes recsys_fa_kernel.so", metadata_path=deploy.sidecar_path(p))
    # full target strings: sm_90 is not covered, and neither is 10.0 without the ISA suffix
    p = _copy_export(exported, tmp_path / "n")
    monkeypatch.setenv("TORCH_CUDA_ARCH_LIST", "9.0;10.0a")
    refused(p, "CUDA target mismatch")
    monkeypatch.setenv("TORCH_CUDA_ARCH_LIST", "10.0")
    refused(p, "CUDA target mismatch")
    monkeypatch.setenv("TORCH_CUDA_ARCH_LIST", "10.0a")
    deploy.check_precompiled(FAOps(), p)

    class Drifted(FAOps):
        op_schemas = {"mha_fwd_with_mask": "mha_fwd_with_mask(Tensor q, Tensor k, Tensor v, Tensor mask, "
                                           "bool causal=False) -> Tensor"}
    refused(p, "schemas mismatch", group=Drifted(allow_jit=False))


def test_visible_sm_must_be_built_for(exported, monkeypatch):
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "device_count", lambda: 2)
    monkeypatch.setattr(torch.cuda, "get_device_capability", lambda i=None: (10, 0) if i == 0 else (9, 0))
    with pytest.raises(CustomOpsError, match=r"SM mismatch: visible=\[90, 100\], built=\[100\]"):
        deploy.check_precompiled(FAOps(), exported)
    monkeypatch.setattr(torch.cuda, "get_device_capability", lambda i=None: (10, 0))
    deploy.check_precompiled(FAOps(), exported)


def test_offline_build_needs_a_schema_for_every_operator(tmp_path):
    class Undeclared(FAOps):
        optional_ops = ["mha_bwd_with_mask"]
    with pytest.raises(CustomOpsError, match="explicit schema"):
        Undeclared().export(str(tmp_path))
    assert not os.listdir(tmp_path)
