"""Load the reference's own Python modules on a CPU-only machine.  TEST INFRASTRUCTURE ONLY.

This file is part of the oracle: it is imported by the fixture generator in
``tests/golden/`` and by CPU tests that pin the restatement in
``oracle/restatement.py`` against the reference itself.  Nothing in the
product package may import it.

The reference's hot-path modules (``incr_modules/*``) import three things that
do not exist on a CPU box or in a bare checkout:

* its compiled extension ``ext.pointops._C_ext.pointops.pointops_ext``
  (five pybind functions, ``ext/pointops/_C_ext/pointops/ops.cpp:117-123``) --
  never called on the network path because ``nnConvIncr.forward`` always takes
  the dense branch (``incr_modules/mask_incr_modules.py:175-178``);
* ``ev_projs.rpg_e2depth.model.model.BaseE2VID`` (an un-vendored git submodule,
  ``.gitmodules:1-3``) which only parses a config dict into attributes that
  ``E2VIDRecurrentIncr.__init__`` reads (``incr_modules/e2depth_incr.py:471-490``);
* a CUDA device: ``torch.cuda.Stream()`` in ``incr_modules/mask_incr_functional.py:18``,
  ``.cuda()`` in ``incr_modules/mask_incr_modules.py:156`` and
  ``torch.cuda.sparse.FloatTensor`` in ``incr_modules/masked_types.py:8``.

``load_reference`` installs minimal stand-ins for those, puts the reference
root on ``sys.path`` and imports the modules unmodified.  No reference source
is copied.
"""
from __future__ import annotations

import importlib
import os
import sys
import types

import torch
import torch.nn as nn

# where a checkout of the reference lives: named by the caller or by MIE_REFERENCE_ROOT, never guessed
DEFAULT_ROOT = os.environ.get("MIE_REFERENCE_ROOT", "")


def reference_available(root: str = DEFAULT_ROOT) -> bool:
    return bool(root) and os.path.isfile(os.path.join(root, "incr_modules", "mask_incr_modules.py"))


class _NullStream:
    """Stand-in for ``torch.cuda.Stream`` on a machine without CUDA."""

    def __init__(self, *a, **k):
        pass


def _install_stubs() -> None:
    # 1. the compiled extension: five names, never called on the network path.
    name = "ext.pointops._C_ext.pointops.pointops_ext"
    if name not in sys.modules:
        m = types.ModuleType(name)

        def _unreachable(*a, **k):
            raise RuntimeError("pointops_ext stub called: the reference never reaches it at HEAD")

        for fn in ("activation_increment", "conv1x1_increment_ext", "conv3x3_increment_ext",
                   "conv5x5_increment_ext", "conv7x7_increment_ext"):
            setattr(m, fn, _unreachable)
        sys.modules[name] = m

    # 2. BaseE2VID: config parsing only.
    if "ev_projs.rpg_e2depth.model.model" not in sys.modules:
        class BaseE2VID(nn.Module):
            def __init__(self, config):
                super().__init__()
                self.num_bins = int(config["num_bins"])
                self.skip_type = str(config.get("skip_type", "sum"))
                self.num_encoders = int(config.get("num_encoders", 4))
                self.base_num_channels = int(config.get("base_num_channels", 32))
                self.num_residual_blocks = int(config.get("num_residual_blocks", 2))
                self.norm = config.get("norm", None)
                self.use_upsample_conv = bool(config.get("use_upsample_conv", True))

        chain = ["ev_projs", "ev_projs.rpg_e2depth", "ev_projs.rpg_e2depth.model",
                 "ev_projs.rpg_e2depth.model.model"]
        for n in chain:
            if n not in sys.modules:
                mod = types.ModuleType(n)
                mod.__path__ = []  # mark as package so sub-imports resolve through sys.modules
                sys.modules[n] = mod
        sys.modules["ev_projs.rpg_e2depth.model.model"].BaseE2VID = BaseE2VID

    # 2b. the learned quantisation layer of the un-vendored rpg_event_representation_learning project: two names
    # imported by incr_modules/event_representation_incr.py:5 and only used by its ClassifierIncrEval wrapper.
    if "ev_projs.rpg_event_representation_learning.utils.models" not in sys.modules:
        for n in ["ev_projs.rpg_event_representation_learning", "ev_projs.rpg_event_representation_learning.utils",
                  "ev_projs.rpg_event_representation_learning.utils.models"]:
            mod = types.ModuleType(n)
            mod.__path__ = []
            sys.modules[n] = mod
        models = sys.modules["ev_projs.rpg_event_representation_learning.utils.models"]
        models.Classifier = type("Classifier", (nn.Module,), {})
        models.QuantizationLayer = type("QuantizationLayer", (nn.Module,), {})

    # 3. CUDA-only calls, when there is no CUDA device.
    if not torch.cuda.is_available():
        torch.cuda.Stream = _NullStream  # type: ignore[assignment]
        torch.Tensor.cuda = lambda self, *a, **k: self  # type: ignore[assignment]


def load_reference(root: str = DEFAULT_ROOT):
    """Import the reference's ``incr_modules`` package and return a namespace of its modules."""
    if not reference_available(root):
        raise FileNotFoundError(f"reference checkout not found at {root}")
    _install_stubs()
    if root not in sys.path:
        sys.path.insert(0, root)
    ns = types.SimpleNamespace()
    ns.masked_types = importlib.import_module("incr_modules.masked_types")
    ns.functional = importlib.import_module("incr_modules.mask_incr_functional")
    ns.modules = importlib.import_module("incr_modules.mask_incr_modules")
    ns.utils = importlib.import_module("incr_modules.utils")
    ns.e2depth = importlib.import_module("incr_modules.e2depth_incr")
    ns.evflownet = importlib.import_module("incr_modules.evflownet_incr")
    ns.fireflownet = importlib.import_module("incr_modules.fireflownet_incr")
    ns.delayedevflownet = importlib.import_module("incr_modules.delayedevflownet_incr")
    ns.obj_detection = importlib.import_module("incr_modules.obj_detection_incr")
    ns.event_representation = importlib.import_module("incr_modules.event_representation_incr")
    # UNetRecurrentIncr.forward calls print_sparsity on a list and raises TypeError at HEAD
    # (incr_modules/e2depth_incr.py:404 -> incr_modules/utils.py:10); silence it.
    ns.e2depth.print_sparsity = lambda *a, **k: None
    return ns


E2DEPTH_CONFIG = dict(num_bins=5, skip_type="sum", recurrent_block_type="convlstm", num_encoders=3,
                      base_num_channels=32, num_residual_blocks=2, norm=None, use_upsample_conv=True)
