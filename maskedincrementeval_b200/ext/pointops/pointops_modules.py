"""Stand-alone operator modules over the native boundary (reference: ``ext/pointops/pointops_modules.py:8-63``,
the wrappers its micro-benchmarks time: ``ActivationIncr``, ``IncrementMaskConvModule`` and the three fixed-size
convolutions ``Conv3x3Incr``, ``Conv5x5Incr``, ``Conv1x1Incr``).

The surface is the reference's: an activation module that owns a reservoir of a given shape, and convolution modules
built from ``(in_shape, c_in, c_out, weight[, stride, padding, device])`` that keep the filter in both layouts plus
a random per-element mask of about 10 % (the benchmarks' stand-in for an activity mask) and map an input delta to a
freshly allocated channels-last output delta.  Three deliberate differences:

* the kernel size is a property of the class (``KERNEL_SIZE``) and one ``forward`` serves all of them;
* the mask is honoured (the reference's kernels ignore it, ``ext_conv.cu:74-76``): it selects the 8x8 output tiles
  that are computed -- those a pixel with any mask element set reaches through the filter -- and every other tile is
  zero; for a delta that is zero off-mask that is the plain convolution;
* ``ActivationIncr.forward`` returns the activation delta (the reference computes it and drops it, ``:14``).
"""
from typing import Sequence

import torch
import torch.nn.functional as F

from ...incr_modules.mask_incr_modules import IncrementMaskModule
from . import pointops_functional as pf


class ActivationIncr(IncrementMaskModule):
    """Incremental ReLU over a dense reservoir of a fixed shape."""

    def __init__(self, shape: Sequence[int], device="cuda"):
        super().__init__()
        self.reservoir = torch.zeros(tuple(shape), dtype=torch.float32, device=device)

    def forward(self, x_incr):
        delta = x_incr[0] if isinstance(x_incr, (list, tuple)) else x_incr
        return pf.activation_incr(self.reservoir, delta.contiguous())

    def forward_refresh_reservoir(self, x):
        self.reservoir = x.detach().clone().contiguous()
        return torch.relu(x)

    forward_refresh_reservoirs = forward_refresh_reservoir     # the name the rest of the operator surface uses


class IncrementMaskConvModule(IncrementMaskModule):
    """Masked delta convolution with a fixed square kernel; subclasses set ``KERNEL_SIZE``."""

    KERNEL_SIZE = None          # taken from the weight when a subclass leaves it open
    MASK_DENSITY = 0.1

    @staticmethod
    def convert_filter_out_channels_last(filter, transposed=True):
        """[Cout,Cin,kH,kW] -> contiguous [Cin,kH,kW,Cout], the layout the native entry points read."""
        return pf.convert_filter_out_channels_last(filter)

    def __init__(self, in_shape, c_in, c_out, weight, stride=1, padding=0, device="cuda"):
        super().__init__()
        k = self.KERNEL_SIZE or int(weight.shape[-1])
        if tuple(weight.shape) != (c_out, c_in, k, k):
            raise RuntimeError(f"weight must be [{c_out},{c_in},{k},{k}], got {tuple(weight.shape)}")
        self.kernel_size, self.c_in, self.c_out, self.stride = k, int(c_in), int(c_out), int(stride)
        self.weight = weight
        self.weight_t = self.convert_filter_out_channels_last(weight)
        self.mask = torch.rand(tuple(in_shape), device=device) <= self.MASK_DENSITY

    def out_shape(self, x_incr):
        k, s = self.kernel_size, self.stride
        n, _, h, w = x_incr.shape
        return n, self.c_out, (h + 2 * (k // 2) - k) // s + 1, (w + 2 * (k // 2) - k) // s + 1

    def forward(self, x_incr):
        x = x_incr.contiguous(memory_format=torch.channels_last)
        out = torch.empty(self.out_shape(x), dtype=torch.float32, device=x.device, memory_format=torch.channels_last)
        native = getattr(pf, f"conv{self.kernel_size}x{self.kernel_size}_increment_ext")
        native(x, self.mask, self.weight_t, out, self.stride)
        return out

    def forward_refresh_reservoir(self, x):
        return F.conv2d(x, self.weight, stride=self.stride, padding=self.kernel_size // 2)

    forward_refresh_reservoirs = forward_refresh_reservoir


class Conv3x3Incr(IncrementMaskConvModule):
    KERNEL_SIZE = 3


class Conv5x5Incr(IncrementMaskConvModule):
    KERNEL_SIZE = 5


class Conv1x1Incr(IncrementMaskConvModule):
    KERNEL_SIZE = 1
