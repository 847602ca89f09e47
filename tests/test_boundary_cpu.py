"""CPU checks of the drop-in boundary: the C-ABI library loads and exports every symbol that
include/mie.h declares, argument validation happens on the host, and the module surface mirrors the
reference's names.  No kernel is launched."""
import os
import re

import pytest
import torch

import maskedincrementeval_b200 as mie
from maskedincrementeval_b200 import _native as nat
from maskedincrementeval_b200 import fields as fl

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "mie.h")).read()
    declared = set(re.findall(r"\b(mie_[a-z0-9_]+)\s*\(", header))
    declared.discard("mie_conv_args")
    assert declared, "no declarations found"
    for name in sorted(declared):
        assert hasattr(nat.lib, name), f"libmie.so does not export {name}"
    assert declared == set(nat.SIGNATURES), (declared ^ set(nat.SIGNATURES))
    assert nat.lib.mie_version() >= 1
    assert nat.lib.mie_status_string(nat.EINVAL).decode() == "invalid argument"


def test_host_side_argument_checks_need_no_gpu():
    # null pointers and bad sizes are rejected before any CUDA call
    assert nat.lib.mie_mask_from_delta(None, 4, 1, 4, 8, 8, 0.0, None, None) == nat.EINVAL
    assert nat.lib.mie_activation_increment(None, None, None, 16, nat.ACT_RELU, None) == nat.EINVAL
    assert nat.lib.mie_tiles_dilate(None, 1, 8, 8, 8, 8, 3, 1, 1, None, None, None, None, None, None, None) == nat.EINVAL
    assert nat.lib.mie_conv_tiles(None, None) == nat.EINVAL
    a = nat.ConvArgs()
    assert nat.lib.mie_conv_tiles(a, None) == nat.EINVAL
    with pytest.raises(nat.MieError):
        nat.check(nat.EINVAL, "x")
    with pytest.raises(NotImplementedError):
        nat.check(nat.EUNSUPPORTED, "x")
    import ctypes as C
    cp, op, nf = C.c_int(), C.c_int(), C.c_int64()
    assert nat.lib.mie_conv_pack_dims(5, 33, 3, C.byref(cp), C.byref(op), C.byref(nf)) == 0
    assert (cp.value, op.value, nf.value) == (8, 64, 9 * 8 * 64)
    assert nat.lib.mie_conv_increment_workspace_bytes(1, 32, 260, 346, 32, 3, 1) > 0


def test_geometry_helpers():
    assert fl.n_tiles(1, 260, 346) == 33 * 44
    assert fl.conv_out_hw(264, 352, 5, 2, 2) == (132, 176)
    x = torch.zeros(2, 6, 5, 7).contiguous(memory_format=torch.channels_last)
    assert fl.pixel_stride(x) == 6
    assert fl.pixel_stride(x[:, 2:4]) == 6
    with pytest.raises(RuntimeError):
        fl.pixel_stride(torch.zeros(2, 6, 5, 7))
    assert fl.act_code(torch.relu) == nat.ACT_RELU and fl.act_code(torch.tanh) == nat.ACT_TANH
    with pytest.raises(NotImplementedError):
        fl.act_code(torch.exp)


def test_surface_mirrors_reference_names():
    from maskedincrementeval_b200.incr_modules import (e2depth_incr, evflownet_incr, fireflownet_incr,
                                                       mask_incr_functional, mask_incr_modules, masked_types, utils)
    for n in ("Masked", "DenseT", "Sp", "SpOrDense", "_device"):
        assert hasattr(masked_types, n)
    for n in ("AccumStreamManager", "IncrementReserve", "IncrPointwiseMultiply", "conv2d_from_module",
              "transposed_conv2d_from_module", "bn2d_from_module", "interpolate_from_module"):
        assert hasattr(mask_incr_functional, n)
    for n in ("IncrementMaskModule", "KFencedMaskModule", "PointwiseMultiplyIncr", "nnReservedMultiplication",
              "NonlinearPointOpIncr", "nnLinearIncr", "nnConvIncrBase", "nnConvIncr", "nnBatchNorm2dIncr",
              "nnMaxPool2dIncr", "nnAdaptiveAvgPool2dIncr", "nnSequentialIncr", "nnReservedActivation",
              "nnReluIncr", "nnSigmoidIncr", "nnTanhIncr"):
        assert hasattr(mask_incr_modules, n)
    for n in ("ConvLayerIncr", "ConvLSTMIncr", "RecurrentConvLayerIncr", "ResidualBlockIncr",
              "UpsampleConvLayerIncr", "TransposedConvLayerIncr", "BaseUNetIncr", "UNetRecurrentIncr",
              "E2VIDRecurrentIncr"):
        assert hasattr(e2depth_incr, n)
    for n in ("skip_concat", "ConvGRUIncr", "ConvLayerIncr", "RecurrentConvLayerIncr", "ResidualBlockIncr",
              "UpsampleConvLayerIncr", "MultiResUNetRecurrentIncr"):
        assert hasattr(evflownet_incr, n)
    assert hasattr(fireflownet_incr, "FireFlowNetIncr")
    assert hasattr(utils, "compute_mask")
    from maskedincrementeval_b200.ext.pointops import pointops_functional as pf, pointops_modules as pm
    for n in ("activation_increment", "conv1x1_increment_ext", "conv3x3_increment_ext", "conv5x5_increment_ext",
              "conv7x7_increment_ext", "activation_incr", "convert_filter_out_channels_last", "functional_conv_module"):
        assert hasattr(pf, n)
    for n in ("ActivationIncr", "IncrementMaskConvModule", "Conv3x3Incr", "Conv5x5Incr", "Conv1x1Incr"):
        assert hasattr(pm, n)


def test_state_dict_keys_match_reference_layout():
    from test_oracle import e2depth_shapes, flow_shapes_ev, flow_shapes_fire
    from maskedincrementeval_b200.incr_modules.e2depth_incr import E2VIDRecurrentIncr
    from maskedincrementeval_b200.incr_modules.evflownet_incr import MultiResUNetRecurrentIncr
    from maskedincrementeval_b200.incr_modules.fireflownet_incr import FireFlowNetIncr
    net = E2VIDRecurrentIncr(dict(num_bins=5, num_encoders=3, base_num_channels=8))
    assert {k: tuple(v.shape) for k, v in net.state_dict().items()} == e2depth_shapes(8)
    f = FireFlowNetIncr(dict(base_num_channels=8, kernel_size=3, mask_output=False), 2)
    assert {k: tuple(v.shape) for k, v in f.state_dict().items()} == flow_shapes_fire(8)
    with torch.device("meta"):
        e = MultiResUNetRecurrentIncr()
    assert {k: tuple(v.shape) for k, v in e.state_dict().items()} == flow_shapes_ev()


def test_ops_refuse_cpu_tensors():
    from maskedincrementeval_b200.incr_modules.mask_incr_modules import nnReluIncr
    a = nnReluIncr()
    a.forward_refresh_reservoirs(torch.zeros(1, 2, 8, 8))
    with pytest.raises(RuntimeError):
        a([torch.zeros(1, 2, 8, 8), None])


def test_install_aliases():
    mie.install_aliases()
    import incr_modules.mask_incr_modules as m  # noqa
    import ext.pointops.pointops_functional as pf  # noqa
    assert m.nnConvIncr.__module__.startswith("maskedincrementeval_b200")
    # leave the interpreter clean for the oracle loader used by other tests
    import sys
    for k in [k for k in sys.modules if k == "ext" or k.startswith("ext.") or k == "incr_modules" or k.startswith("incr_modules.")]:
        del sys.modules[k]
