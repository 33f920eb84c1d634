"""B200-native drop-in for the ``mha_fwd_with_mask`` path of Defyli/custom_ops.

    from custom_ops_b200 import ops
    out = ops.mha_fwd_with_mask(q, k, v, mask)

mirrors ``from custom_ops import ops`` of the reference (``__init__.py:1222``,
``recsys.py:641-656``).  Importing the package compiles and loads nothing; the
native libraries are built (in-tree) and loaded on first use.
``mha_fwd_with_mask_from_host`` is the same operator for operands in host memory;
``rule_mask`` writes causal / sliding-window / padding masks on the device.
"""
from .host_io import mha_fwd_with_mask_from_host  # noqa: F401
from .masks import rule_mask  # noqa: F401
from .recsys import CustomOps, CustomOpsError, FAOps, RecsysOps  # noqa: F401

ops = RecsysOps()

__all__ = ["ops", "RecsysOps", "FAOps", "CustomOps", "CustomOpsError", "mha_fwd_with_mask_from_host", "rule_mask"]
