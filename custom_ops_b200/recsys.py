"""Host-side mirror of the reference's Python entry point for the FA group.

``from custom_ops_b200 import ops; ops.mha_fwd_with_mask(q, k, v, mask)`` is the
drop-in for ``from custom_ops import ops`` (reference ``recsys.py:641-656``):
same group definition (``FAOps``: namespace ``recsys_ops``, library
``recsys_fa_kernel``, schema string, fake implementation ``empty_like(q)``;
reference ``recsys.py:165-202``), same lazy loading, the same loader checks after
``torch.ops.load_library`` (schema equality, a Meta kernel must exist; reference
``__init__.py:910-934, 1069-1150``) and the same query API (``is_available``,
``load_error``, ``ensure_loaded``, ``groups``).

Only the FA group exists here, only for sm_100a, and there is exactly one
backend: hand-written CUDA.  ``backend="tilelang"`` and the automatic fallback of
the reference (``recsys.py:597-620``) are rejected, and a missing or unloadable
native library raises instead of silently computing elsewhere.
"""
from __future__ import annotations

import os
import threading
import warnings
from typing import Optional

import torch

from . import build as _build
from . import deploy as _deploy
from .deploy import CustomOpsError


_LIBRARY_LOCK = threading.RLock()
_LOADED_LIBRARIES: dict = {}


def _schema(qualified: str) -> str:
    return str(torch._C._get_schema(qualified, ""))


def _has_schema(qualified: str) -> bool:
    try:
        torch._C._get_schema(qualified, "")
        return True
    except RuntimeError:
        return False


def _resolve_backend(backend) -> str:
    """Explicit argument > env ``CUSTOM_OPS_BACKEND`` > "auto" (reference
    ``recsys.py:142-158``).  Only "auto" and "cuda" select anything here."""
    if backend is None:
        backend = os.environ.get("CUSTOM_OPS_BACKEND", "auto")
    backend = str(backend).lower()
    if backend not in ("auto", "cuda", "tilelang"):
        raise ValueError(
            f"backend must be 'auto' | 'cuda' | 'tilelang', got {backend!r} "
            f"(or set CUSTOM_OPS_BACKEND env)")
    if backend == "tilelang":
        raise CustomOpsError(
            "this build has a single backend (hand-written sm_100a CUDA); "
            "the Tile-lang backend is not part of it")
    return backend


class CustomOps:
    """Minimal loader for one group of operators living in one shared library.

    Subclasses set ``namespace``, ``so_name``, ``required_ops``, ``op_schemas`` and
    ``fake_ops`` and override :meth:`register_fake_impls`.  ``allow_jit=True``
    builds the library in-tree when it is missing or stale; ``allow_jit=False``
    (deployment) only loads what is already built.
    """

    namespace: str = ""
    so_name: str = ""
    requires_cuda: bool = True
    build_version: str = "1"       # bump when a rebuild must not be mistaken for an older export
    required_ops: list = []
    optional_ops: list = []
    op_schemas: dict = {}
    fake_ops: list = []

    def __init__(self, *, allow_jit: bool = True) -> None:
        self._allow_jit = bool(allow_jit)
        self._loaded = False
        self._load_error: Optional[str] = None
        self._fake_ops_registered: set = set()
        self._library_path: Optional[str] = None
        self._metadata_path: Optional[str] = None

    # -- configuration -------------------------------------------------------
    @property
    def allow_jit(self) -> bool:
        return self._allow_jit

    @allow_jit.setter
    def allow_jit(self, value: bool) -> None:
        self._allow_jit = bool(value)

    def configure(self, *, allow_jit: bool) -> "CustomOps":
        self._allow_jit = bool(allow_jit)
        return self

    def disable_jit(self) -> "CustomOps":
        return self.configure(allow_jit=False)

    @property
    def library_path(self) -> Optional[str]:
        return self._library_path

    # -- hooks ----------------------------------------------------------------
    def get_sources(self) -> list:
        raise NotImplementedError

    def get_include_dirs(self) -> list:
        return []

    def build(self, *, force: bool = False, verbose: bool = False) -> str:
        raise NotImplementedError

    def prebuilt_path(self) -> str:
        raise NotImplementedError

    def companion_libraries(self) -> list:
        """Other shared libraries the operator library needs beside it (``$ORIGIN`` rpath)."""
        return []

    def source_fingerprint(self) -> str:
        """sha256 over the contents of every source and header of the group."""
        files = list(self.get_sources())
        for d in self.get_include_dirs():
            for root, _, names in sorted(os.walk(d)):
                files += [os.path.join(root, n) for n in sorted(names)
                          if n.endswith((".h", ".hpp", ".cuh", ".cu", ".cpp"))]
        return _deploy.json_hash({os.path.basename(p): _deploy.file_sha256(p) for p in sorted(set(files))})

    def export(self, directory: str, *, force: bool = False, verbose: bool = False) -> str:
        """Offline build for deployment: libraries + JSON sidecar into ``directory``; nothing is
        loaded (reference ``__init__.py:654-729``).  Returns the exported library's path."""
        return _deploy.export_group(self, directory, force=force, verbose=verbose)

    @property
    def metadata_path(self) -> Optional[str]:
        return self._metadata_path

    def register_fake_impls(self) -> None:
        pass

    # -- loading ---------------------------------------------------------------
    def _schema_contract(self) -> dict:
        return {name: str(torch._C.parse_schema(f"{self.namespace}::{text}"))
                for name, text in self.op_schemas.items()}

    def _verify_ops(self) -> None:
        missing = [n for n in self.required_ops if not _has_schema(f"{self.namespace}::{n}")]
        if missing:
            raise CustomOpsError(
                f"Required ops not found in torch.ops.{self.namespace}: {missing}.")
        for name, expected in self._schema_contract().items():
            qualified = f"{self.namespace}::{name}"
            if _has_schema(qualified) and _schema(qualified) != expected:
                raise CustomOpsError(
                    f"Loaded schema mismatch for {qualified}: "
                    f"got={_schema(qualified)!r}, expected={expected!r}")

    def register_fake_for(self, op_name: str, fake_fn) -> None:
        qualified = f"{self.namespace}::{op_name}"
        with _LIBRARY_LOCK:
            _schema(qualified)      # a missing schema is an error, never swallowed
            has_meta = torch._C._dispatch_has_kernel_for_dispatch_key
            if not has_meta(qualified, "Meta"):
                torch.library.register_fake(qualified)(fake_fn)
            if not has_meta(qualified, "Meta"):
                raise CustomOpsError(f"Fake registration did not create a Meta kernel: {qualified}")
            self._fake_ops_registered.add(op_name)

    def _dlopen_library(self, path: str) -> None:
        with _LIBRARY_LOCK:
            real = os.path.realpath(path)
            if real in _LOADED_LIBRARIES:
                if _LOADED_LIBRARIES[real] is None:
                    raise CustomOpsError(f"{path} failed to load before; it is not tried again")
                return
            for name in self.required_ops:
                if _has_schema(f"{self.namespace}::{name}"):
                    # also a byte-identical copy under another name: the dispatcher keeps one
                    # registration per operator, a second dlopen would abort the process
                    raise CustomOpsError(
                        f"{self.namespace}::{name} is already registered by another library; "
                        f"two providers of one operator cannot share a process")
            try:
                torch.ops.load_library(path)
            except Exception:
                _LOADED_LIBRARIES[real] = None          # never retried, never replaced
                raise
            _LOADED_LIBRARIES[real] = type(self).__name__

    def load(self) -> "CustomOps":
        """Build if allowed and needed, dlopen, verify schemas, register fakes.
        Never raises: failures are kept for :meth:`load_error` (reference
        ``__init__.py:981-1009``); calling an operator afterwards does raise."""
        with _LIBRARY_LOCK:
            if self._loaded:
                return self
            try:
                if self._allow_jit:
                    path = self.build()
                else:
                    path = self.prebuilt_path()
                    if not os.path.exists(path):
                        raise CustomOpsError(
                            f"{path} is not built and allow_jit=False forbids compiling it")
                self._dlopen_library(path)
                self._verify_ops()
                self.register_fake_impls()
                has_meta = torch._C._dispatch_has_kernel_for_dispatch_key
                for name in self.fake_ops:
                    if not has_meta(f"{self.namespace}::{name}", "Meta"):
                        raise CustomOpsError(f"{self.namespace}::{name} has no Meta kernel")
                self._library_path = path
                self._loaded = True
                self._load_error = None
            except Exception as e:  # noqa: BLE001 - surfaced through load_error()
                self._loaded = False
                self._load_error = f"{type(e).__name__}: {e}"
                warnings.warn(f"[{type(self).__name__}] load failed: {self._load_error}")
        return self

    def load_precompiled(self, path: Optional[str] = None,
                         metadata_path: Optional[str] = None) -> "CustomOps":
        """Strict load of an exported library (see :meth:`export`); raises on any problem and
        never compiles.  Everything the JSON sidecar allows to be checked is checked before the
        library is dlopen'ed (reference ``__init__.py:936-979``).  Without ``path`` the in-tree
        build is loaded, which has no sidecar and is only checked after loading."""
        with _LIBRARY_LOCK:
            if self._loaded:
                same = path is None or os.path.realpath(path) == os.path.realpath(self._library_path or "")
                if not same:
                    raise CustomOpsError(
                        f"{type(self).__name__} already loaded {self._library_path}; a process keeps one "
                        f"provider per operator")
                return self
            metadata = None
            if path is None:
                path = self.prebuilt_path()
                if not os.path.exists(path):
                    raise CustomOpsError(f"precompiled library not found: {path}")
            else:
                metadata = _deploy.check_precompiled(self, path, metadata_path)
            try:
                self._dlopen_library(path)
                self._verify_ops()
                self.register_fake_impls()
                has_meta = torch._C._dispatch_has_kernel_for_dispatch_key
                for name in self.fake_ops:
                    if not has_meta(f"{self.namespace}::{name}", "Meta"):
                        raise CustomOpsError(f"{self.namespace}::{name} has no Meta kernel")
            except Exception as e:
                self._loaded = False
                self._load_error = f"{type(e).__name__}: {e}"
                raise
            self._library_path = path
            self._metadata_path = (metadata_path or _deploy.sidecar_path(path)) if metadata else None
            self._loaded = True
            self._load_error = None
        return self

    # -- public API ------------------------------------------------------------
    def is_available(self) -> bool:
        return self._loaded

    def load_error(self) -> Optional[str]:
        return self._load_error

    def __getattr__(self, name: str):
        if name.startswith("_"):
            raise AttributeError(name)
        if not self._loaded:
            raise RuntimeError(
                f"[{type(self).__name__}] ops.{name}() called but extension not loaded. "
                f"Check is_available(). Error: {self._load_error}")
        ns = getattr(torch.ops, self.namespace, None)
        if ns is None:
            raise AttributeError(f"torch.ops.{self.namespace} not found.")
        op = getattr(ns, name, None)
        if op is None:
            raise AttributeError(f"No op '{name}' in torch.ops.{self.namespace}.")
        return op

    def __repr__(self) -> str:
        state = "loaded" if self._loaded else ("failed" if self._load_error else "not_loaded")
        return f"{type(self).__name__}(namespace={self.namespace!r}, so={self.so_name!r}, {state})"


class FAOps(CustomOps):
    """FA group: ``mha_fwd_with_mask`` (flash attention forward + additive mask),
    sm_100a kernels behind ``include/fa_mask_fwd_sm100.h``."""

    namespace = "recsys_ops"
    requires_cuda = True
    so_name = "recsys_fa_kernel"
    required_ops = ["mha_fwd_with_mask"]
    op_schemas = {
        "mha_fwd_with_mask": "mha_fwd_with_mask(Tensor q, Tensor k, Tensor v, Tensor mask) -> Tensor",
        "mha_fwd_with_mask_lse":
            "mha_fwd_with_mask_lse(Tensor q, Tensor k, Tensor v, Tensor mask) -> (Tensor, Tensor)",
        "mha_fwd_rule_mask":
            "mha_fwd_rule_mask(Tensor q, Tensor k, Tensor v, bool causal, int window, Tensor? valid_lens) -> Tensor",
    }
    fake_ops = ["mha_fwd_with_mask", "mha_fwd_with_mask_lse", "mha_fwd_rule_mask"]
    # not in the reference: the same forward that also returns each row's log-sum-exp, and the
    # forward for a mask given as a rule (causal / sliding window / valid lengths)
    optional_ops = ["mha_fwd_with_mask_lse", "mha_fwd_rule_mask"]

    def get_sources(self) -> list:
        return list(_build.TORCH_SOURCES) + list(_build.CABI_SOURCES)

    def get_include_dirs(self) -> list:
        return [_build.INCLUDE, _build.CSRC]

    def build(self, *, force: bool = False, verbose: bool = False) -> str:
        _build.build_cabi(force=force, verbose=verbose)
        return _build.build_torch_binding(force=force, verbose=verbose)

    def prebuilt_path(self) -> str:
        return _build.TORCH_SO

    def companion_libraries(self) -> list:
        return [_build.CABI_SO]

    def register_fake_impls(self) -> None:
        self.register_fake_for("mha_fwd_with_mask", lambda q, k, v, mask: torch.empty_like(q))
        self.register_fake_for(
            "mha_fwd_with_mask_lse",
            lambda q, k, v, mask: (torch.empty_like(q),
                                   q.new_empty((q.shape[0], q.shape[1], q.shape[2]), dtype=torch.float32)))
        self.register_fake_for("mha_fwd_rule_mask",
                               lambda q, k, v, causal, window, valid_lens: torch.empty_like(q))


class RecsysOps:
    """Lazy facade over the operator groups (here: only "fa").

    The public surface -- ``configure``, ``disable_jit``, ``ensure_loaded``, ``load``, ``groups``,
    ``is_available``, ``load_error``, ``load_precompiled`` and the operators themselves -- is the
    reference facade's (``recsys.py:466-656``), because callers and the loader-contract tests use
    exactly these names, argument meanings and messages.  The bookkeeping behind it is this
    package's own: one table of group states, every public method a query or a transition on it.
    """

    _GROUP_CLASSES = {"fa": FAOps}
    _OP_TO_GROUP = {"mha_fwd_with_mask": "fa", "mha_fwd_with_mask_lse": "fa", "mha_fwd_rule_mask": "fa"}

    def __init__(self, *, allow_jit: bool = True) -> None:
        self._allow_jit = bool(allow_jit)
        self._groups: dict = {}          # name -> CustomOps instance, once somebody asked for it
        self._lock = threading.RLock()

    # ---- policy
    @property
    def allow_jit(self) -> bool:
        return self._allow_jit

    @allow_jit.setter
    def allow_jit(self, value: bool) -> None:
        self.configure(allow_jit=value)

    def configure(self, *, allow_jit: bool) -> "RecsysOps":
        """Sets the build policy for the groups that exist and for those still to come."""
        with self._lock:
            self._allow_jit = bool(allow_jit)
            for inst in list(self._groups.values()):
                inst.configure(allow_jit=self._allow_jit)
            return self

    def disable_jit(self) -> "RecsysOps":
        return self.configure(allow_jit=False)

    # ---- the table of groups
    def _validate_group(self, name: str) -> None:
        if name not in self._GROUP_CLASSES:
            raise ValueError(f"Unknown group {name!r}; available: {sorted(self._GROUP_CLASSES)}")

    def _peek(self, name: str):
        """The group's instance if somebody created it already, else None; never creates."""
        self._validate_group(name)
        return self._groups.get(name)

    def _group(self, name: str) -> CustomOps:
        """The group's instance, created and loaded on first use (a failed load is kept, not
        raised: ``is_available`` / ``load_error`` report it, calling an operator raises)."""
        with self._lock:
            inst = self._peek(name)
            if inst is None:
                inst = self._groups[name] = self._GROUP_CLASSES[name](allow_jit=self._allow_jit)
                inst.load()
            return inst

    def _state(self, name: str) -> str:
        inst = self._groups.get(name)
        if inst is None:
            return "not_loaded"
        return "loaded" if inst.is_available() else "failed"

    def load_precompiled(self, group: str = "fa", path: Optional[str] = None,
                         metadata_path: Optional[str] = None) -> "RecsysOps":
        with self._lock:
            inst = self._peek(group)
            if inst is None:
                inst = self._GROUP_CLASSES[group](allow_jit=False)
            inst.load_precompiled(path, metadata_path)
            self._groups[group] = inst
            return self

    def ensure_loaded(self, *names) -> "RecsysOps":
        """Loads the named groups (all of them when none is named); unknown names are refused
        before anything is loaded."""
        wanted = list(names) or list(self._GROUP_CLASSES)
        with self._lock:
            for name in wanted:
                self._validate_group(name)
            for name in wanted:
                self._group(name)
            return self

    def load(self) -> "RecsysOps":
        return self.ensure_loaded()

    @property
    def groups(self) -> dict:
        with self._lock:
            return {name: self._state(name) for name in self._GROUP_CLASSES}

    def is_available(self, group: Optional[str] = None) -> bool:
        """One group: whether it is loaded and usable (loading it now unless building is off and
        nobody loaded it).  No group named: whether everything that was loaded so far works."""
        with self._lock:
            if group is None:
                if not torch.cuda.is_available() or (not self._allow_jit and not self._groups):
                    return False
                return all(state == "loaded" for state in (self._state(n) for n in self._groups))
            inst = self._peek(group) if not self._allow_jit else self._group(group)
            return inst is not None and inst.is_available()

    def load_error(self, group: Optional[str] = None):
        """The kept load error of one group, or of the first group that failed."""
        with self._lock:
            if group is not None:
                inst = self._peek(group)
                return None if inst is None else inst.load_error()
            failed = [inst for inst in self._groups.values() if not inst.is_available()]
            return failed[0].load_error() if failed else None

    def _dispatch(self, backend, group: str) -> CustomOps:
        _resolve_backend(backend)
        inst = self._group(group)
        if not inst.is_available():
            raise CustomOpsError(
                f"CUDA group '{group}' failed to load and there is no other backend: "
                f"{inst.load_error()}")
        return inst

    def __getattr__(self, name: str):
        if name.startswith("_"):
            raise AttributeError(name)
        group = self._OP_TO_GROUP.get(name)
        if group is None:
            raise AttributeError(
                f"No op '{name}' in recsys_ops. Available ops: {sorted(self._OP_TO_GROUP)} "
                f"(groups: {sorted(self._GROUP_CLASSES)})")
        return getattr(self._group(group), name)

    def __repr__(self) -> str:
        return (f"RecsysOps(lazy, allow_jit={self.allow_jit}, namespace='recsys_ops', "
                f"groups={self.groups})")

    def mha_fwd_with_mask(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                          mask: torch.Tensor, backend: Optional[str] = None) -> torch.Tensor:
        """Flash-attention forward with an arbitrary additive fp16/bf16 mask.

        q ``(B, H, Sq, d)``, k/v ``(B, Hk, Sk, d)``, mask ``(B, 1, >=Sq, >=Sk)`` of q's
        dtype (0 visible, -inf masked, finite = bias); all CUDA and contiguous;
        ``d`` in {64, 128}; ``H % Hk == 0``; any ``Sq`` and ``Sk``.  Returns
        ``(B, H, Sq, d)`` in q's dtype; a fully masked row is 0.
        """
        return self._dispatch(backend, "fa").mha_fwd_with_mask(q, k, v, mask)

    def mha_fwd_with_mask_lse(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                              mask: torch.Tensor, backend: Optional[str] = None):
        """``mha_fwd_with_mask`` that also returns the natural-log log-sum-exp of every row's
        scaled, masked scores: ``(out, lse)`` with ``lse`` fp32 of shape ``(B, H, Sq)``, ``-inf``
        for a fully masked row (the reference computes it, ``csrc/fa/common/softmax.h:145``, but
        its operator does not return it)."""
        return self._dispatch(backend, "fa").mha_fwd_with_mask_lse(q, k, v, mask)

    def mha_fwd_rule_mask(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False,
                          window: int = 0, valid_lens: Optional[torch.Tensor] = None,
                          backend: Optional[str] = None) -> torch.Tensor:
        """The forward for a mask given as a rule instead of a tensor: key ``j`` is visible to query
        ``i`` when ``j < valid_lens[b]`` (if given), ``j <= i + Sk - Sq`` (if ``causal``) and
        ``j > i + Sk - Sq - window`` (if ``window > 0``) - the recipes callers build their additive
        masks from (``examples/custom_mask_demo.py:33-65``), evaluated inside the kernel.
        Bit-identical to ``mha_fwd_with_mask`` on ``masks.rule_mask`` of the same rule."""
        return self._dispatch(backend, "fa").mha_fwd_rule_mask(q, k, v, bool(causal), int(window), valid_lens)
