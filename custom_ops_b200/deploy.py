"""Offline export and strict loading of an operator group.

The reference separates *development* (``load()``: JIT-compile when needed) from
*deployment* (``build()`` writes a library plus a JSON description next to it,
``load_precompiled()`` accepts that pair only if everything in the description agrees with
the Python wrapper, the runtime and the bytes on disk - and decides all of that BEFORE the
library is dlopen'ed; reference ``__init__.py:654-979``, pinned by
``tests/test_custom_ops_loading.py``).  This module is that contract for the groups of this
package, written for its two-library layout: the torch operator binding and, beside it, the
C-ABI kernel library it links to (``$ORIGIN`` rpath), both described by one sidecar.

    path = export_group(FAOps(), "/deploy/dir")          # build machine: compiles, never loads
    FAOps(allow_jit=False).load_precompiled(path)        # serving process: never compiles
"""
from __future__ import annotations

import hashlib
import json
import os
import re
import shutil
import sys
from typing import Optional

import torch

FORMAT_VERSION = 1
PRODUCER = "custom_ops_b200"
CUDA_TARGETS = ["10.0a"]            # the only target this package builds for


class CustomOpsError(RuntimeError):
    """Loader / deployment contract violation (reference ``__init__.py:71``)."""


DeployError = CustomOpsError


def file_sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def json_hash(value) -> str:
    return hashlib.sha256(json.dumps(value, sort_keys=True, separators=(",", ":")).encode()).hexdigest()


def metadata_fingerprint(metadata: dict) -> str:
    """Hash of everything in the sidecar except the fingerprint itself."""
    return json_hash({k: v for k, v in metadata.items() if k != "build_fingerprint"})


def runtime_compatibility() -> dict:
    """What a binary built against this runtime depends on (reference ``__init__.py:124-137``)."""
    return {
        "torch": ".".join(torch.__version__.split("+")[0].split(".")[:2]),
        "python": f"{sys.version_info.major}.{sys.version_info.minor}",
        "cxx11_abi": bool(torch.compiled_with_cxx11_abi()),
        "cuda_major": (torch.version.cuda or "").split(".")[0],
        "platform": sys.platform,
    }


def sidecar_path(library: str) -> str:
    return library + ".json"


def _describe(path: str) -> dict:
    return {"filename": os.path.basename(path), "size": os.path.getsize(path), "sha256": file_sha256(path)}


def group_description(group) -> dict:
    """The part of the sidecar that comes from the Python wrapper alone."""
    schemas = group._schema_contract()
    return {
        "format_version": FORMAT_VERSION,
        "producer": PRODUCER,
        "group": type(group).__name__,
        "namespace": group.namespace,
        "so_name": group.so_name,
        "build_version": str(group.build_version),
        "required_ops": sorted(group.required_ops),
        "optional_ops": sorted(group.optional_ops),
        "fake_ops": sorted(group.fake_ops),
        "schemas": schemas,
        "schema_fingerprint": json_hash(schemas),
        "with_cuda": bool(group.requires_cuda),
        "cuda_arch_list": list(CUDA_TARGETS) if group.requires_cuda else [],
    }


def export_group(group, directory: str, *, force: bool = False, verbose: bool = False) -> str:
    """Compile the group's libraries (in-tree, as always), copy them to ``directory`` and
    describe them in ``<library>.json``.  Nothing is loaded into this process.  Returns the path
    of the exported operator library.  An existing export is only replaced as a whole: the
    sidecar is removed first and written last, so a half-written export never validates."""
    if not group.op_schemas or set(group.op_schemas) != set(group.required_ops) | set(group.optional_ops):
        raise DeployError("an offline build needs an explicit schema for every operator of the group")
    built = group.build(force=force, verbose=verbose)
    companions = list(group.companion_libraries())
    os.makedirs(directory, exist_ok=True)
    target = os.path.join(directory, os.path.basename(built))
    sidecar = sidecar_path(target)
    if os.path.exists(sidecar):
        os.remove(sidecar)
    copies = []
    for src in [built] + companions:
        dst = os.path.join(directory, os.path.basename(src))
        tmp = dst + ".part"
        shutil.copyfile(src, tmp)
        os.replace(tmp, dst)
        copies.append(dst)
    metadata = group_description(group)
    metadata["compatibility"] = runtime_compatibility()
    metadata["library"] = _describe(copies[0])
    metadata["companions"] = [_describe(p) for p in copies[1:]]
    metadata["source_fingerprint"] = group.source_fingerprint()
    metadata["build_fingerprint"] = metadata_fingerprint(metadata)
    tmp = sidecar + ".part"
    with open(tmp, "w", encoding="utf-8") as f:
        json.dump(metadata, f, indent=1, sort_keys=True)
    os.replace(tmp, sidecar)
    return target


def _same(metadata: dict, key: str, expected) -> None:
    got = metadata.get(key)
    if got != expected or type(got) is not type(expected):
        raise DeployError(f"precompiled {key} mismatch: built={got!r}, expected={expected!r}")


def check_precompiled(group, library: str, sidecar: Optional[str] = None) -> dict:
    """Every check that can be made without loading the library; raises ``DeployError``.

    Order: the files exist; the sidecar is a JSON object of this format; it describes this
    wrapper (names, operator lists, schema contract) and this runtime; its fingerprints are
    intact; the build targets cover what is requested (``TORCH_CUDA_ARCH_LIST``) and every
    visible GPU, by exact SM; the bytes on disk are the bytes that were described."""
    sidecar = sidecar or sidecar_path(library)
    if not os.path.isfile(library):
        raise DeployError(f"precompiled library not found: {library}")
    if not os.path.isfile(sidecar):
        raise DeployError(f"precompiled metadata not found: {sidecar}")
    try:
        with open(sidecar, encoding="utf-8") as f:
            metadata = json.load(f)
    except (OSError, ValueError) as e:
        raise DeployError(f"precompiled metadata is unreadable: {e}") from None
    if not isinstance(metadata, dict):
        raise DeployError("precompiled metadata must be a JSON object")
    for key, expected in group_description(group).items():
        if key in ("with_cuda", "cuda_arch_list", "group"):     # the class name is informational
            continue
        _same(metadata, key, expected)
    compatibility = metadata.get("compatibility")
    if not isinstance(compatibility, dict):
        raise DeployError("precompiled compatibility information is missing")
    for key, expected in runtime_compatibility().items():
        _same(compatibility, key, expected)
    for key in ("source_fingerprint", "build_fingerprint"):
        if not isinstance(metadata.get(key), str) or not re.fullmatch(r"[0-9a-f]{64}", metadata[key]):
            raise DeployError(f"precompiled {key} is missing or invalid")
    if metadata["build_fingerprint"] != metadata_fingerprint(metadata):
        raise DeployError("precompiled build fingerprint is invalid (the metadata was edited)")
    # the wrapper, not the metadata, says whether the group needs CUDA
    with_cuda, targets = metadata.get("with_cuda"), metadata.get("cuda_arch_list")
    if not isinstance(with_cuda, bool) or not isinstance(targets, list) or \
            any(not isinstance(t, str) for t in targets):
        raise DeployError("precompiled CUDA target information is invalid")
    if with_cuda != bool(group.requires_cuda) or bool(targets) != with_cuda:
        raise DeployError("precompiled CUDA requirement does not match this Python wrapper")
    if with_cuda:
        if torch.version.cuda is None or getattr(torch.version, "hip", None):
            raise DeployError("a CUDA library requires an NVIDIA CUDA build of PyTorch")
        requested = [t.strip() for t in re.split(r"[;\s]+", os.environ.get("TORCH_CUDA_ARCH_LIST", "")) if t.strip()]
        missing = sorted(set(requested) - set(targets))
        if missing:
            raise DeployError(f"precompiled CUDA target mismatch: requested={missing}, built={targets} "
                              f"(ISA suffix and +PTX are significant)")
        if torch.cuda.is_available():
            built_sms = {int(float(re.match(r"[0-9]+\.[0-9]+", t).group(0)) * 10 + 0.5) for t in targets}
            visible = {mj * 10 + mn for mj, mn in (torch.cuda.get_device_capability(i)
                                                   for i in range(torch.cuda.device_count()))}
            if not visible.issubset(built_sms):
                raise DeployError(f"precompiled SM mismatch: visible={sorted(visible)}, built={sorted(built_sms)}")
    entries = [metadata.get("library")] + list(metadata.get("companions") or [])
    directory = os.path.dirname(os.path.abspath(library))
    for i, entry in enumerate(entries):
        if not isinstance(entry, dict) or not isinstance(entry.get("filename"), str) or \
                os.path.basename(entry["filename"]) != entry["filename"]:
            raise DeployError("precompiled library identity information is missing")
        path = library if i == 0 else os.path.join(directory, entry["filename"])
        if i == 0 and entry["filename"] != os.path.basename(library):
            raise DeployError(f"precompiled metadata describes {entry['filename']}, not {os.path.basename(library)}")
        if not os.path.isfile(path):
            raise DeployError(f"precompiled companion library not found: {path}")
        if type(entry.get("size")) is not int or entry["size"] != os.path.getsize(path) or \
                entry.get("sha256") != file_sha256(path):
            raise DeployError(f"precompiled library hash/size mismatch: {path}")
    return metadata
