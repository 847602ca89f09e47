"""B200-native masked incremental inference: the ``incr_modules`` operator surface of
sankeerth95/MaskedIncrementEval on hand-written sm_100a kernels behind a C ABI (``include/mie.h``).

    from maskedincrementeval_b200.incr_modules.mask_incr_modules import nnConvIncr, nnReluIncr
    from maskedincrementeval_b200.incr_modules.e2depth_incr import E2VIDRecurrentIncr

or, to run code written against the reference unchanged, call ``install_aliases()`` once and keep
``from incr_modules... import ...`` / ``import ext.pointops.pointops_functional``.
"""
import importlib
import sys

from . import _native  # noqa: F401  (raises if libmie.so is missing: there is no fallback)
from .fields import IncrConfig, TileMask, config  # noqa: F401

__all__ = ["config", "IncrConfig", "TileMask", "install_aliases"]


def install_aliases() -> None:
    """Register this package's ``incr_modules`` and ``ext.pointops`` under the reference's top-level names."""
    for ref_name, ours in (("incr_modules", "maskedincrementeval_b200.incr_modules"),
                           ("ext", "maskedincrementeval_b200.ext"),
                           ("ext.pointops", "maskedincrementeval_b200.ext.pointops")):
        sys.modules[ref_name] = importlib.import_module(ours)
    for sub in ("masked_types", "mask_incr_functional", "mask_incr_modules", "utils", "e2depth_incr",
                "evflownet_incr", "fireflownet_incr", "delayedevflownet_incr", "obj_detection_incr",
                "event_representation_incr"):
        try:
            sys.modules["incr_modules." + sub] = importlib.import_module("maskedincrementeval_b200.incr_modules." + sub)
        except ModuleNotFoundError:
            pass
    for sub in ("pointops_functional", "pointops_modules"):
        sys.modules["ext.pointops." + sub] = importlib.import_module("maskedincrementeval_b200.ext.pointops." + sub)
