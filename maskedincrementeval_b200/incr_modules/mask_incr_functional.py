"""Persistent state and functional operators of the masked incremental path
(reference: ``incr_modules/mask_incr_functional.py:1-81``), running on libmie kernels."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _native as nat
from .. import fields as fl
from ..fields import Scratch, TileMask
from .masked_types import DenseT, Masked


class AccumStreamManager:
    """Singleton side stream (reference ``:9-21``; unused there too)."""
    instance = None

    @classmethod
    def createAccumStream(cls):
        if cls.instance is None:
            cls.instance = cls()
        return cls.instance

    def __init__(self):
        self.s = torch.cuda.Stream()

    def get_stream(self):
        return self.s


class IncrementReserve:
    """Persistent accumulator ``x_prev`` of one operator input (reference ``:26-48``).

    Unlike the reference, ``update_reservoir`` copies into the existing buffer when the shape is
    unchanged, so the device address is stable across refreshes (needed to replay steps as CUDA graphs)."""

    def __init__(self, x_init=None):
        self.reservoir = None
        if x_init is not None:
            self.update_reservoir(x_init)

    def _adjust_mem_format(self):
        if self.reservoir is not None and self.reservoir.dim() == 4:
            self.reservoir = self.reservoir.contiguous(memory_format=torch.channels_last)

    def accumulate(self, incr: Masked):
        d, m = incr[0], incr[1]
        if isinstance(m, TileMask) and self.reservoir.dim() == 4:
            fl.accumulate(self.reservoir, fl.as_channels_last(d), m)
        else:
            self.reservoir.add_(d)

    def update_reservoir(self, x: DenseT):
        x = x.detach()
        r = self.reservoir
        if r is not None and r.shape == x.shape and r.device == x.device and r.dtype == x.dtype:
            r.copy_(x)
        else:
            self.reservoir = x.clone()
            self._adjust_mem_format()


_scratch = Scratch()


def IncrPointwiseMultiply(x1_incr: Masked, x1: IncrementReserve, x2_incr: Masked, x2: IncrementReserve) -> Masked:
    """d(x1*x2) = (dx2 + x2)*dx1 + x1*dx2; the reservoirs are only read (reference ``:52-54``)."""
    d1, m1 = fl.resolve(x1_incr, _scratch, "ipm1")
    d2, m2 = fl.resolve(x2_incr, _scratch, "ipm2")
    n, c, h, w = d1.shape
    out = fl.new_field(n, c, h, w, d1.device)
    bits = fl.new_bits(n, h, w, d1.device)
    m = fl.mul_incr(d1, m1, fl.as_channels_last(x1.reservoir), d2, m2, fl.as_channels_last(x2.reservoir), out, bits,
                    accumulate=False)
    return [out, m]


def conv2d_from_module(x: Masked, conv_weights, stride=(1, 1), padding=(1, 1)) -> Masked:
    """Masked delta convolution with a [Cin,kH,kW,Cout] filter (reference ``:60-61``)."""
    from ..ext.pointops import pointops_functional as pf
    return pf.functional_conv_module(x[0], conv_weights, mask=x[1], stride=stride, padding=padding)


def transposed_conv2d_from_module(x: Masked, gates: nn.ConvTranspose2d, bias=True) -> Masked:
    """Transposed convolution of a delta, no bias (reference ``:64-66``; returns a bare tensor there too).
    Dense library call: no network in scope reaches it."""
    return F.conv_transpose2d(x[0], gates.weight, bias=None, stride=gates.stride, padding=gates.padding,
                              output_padding=gates.output_padding, dilation=gates.dilation, groups=gates.groups)


def bn2d_from_module(x: Masked, bnm: nn.BatchNorm2d) -> Masked:
    """Eval batch-norm of a delta: mean forced to zero and bias omitted, i.e. a per-channel scale
    (reference ``:69-73``).  A scale keeps zeros zero, so the mask passes through."""
    scale = (bnm.weight if bnm.weight is not None else 1.0) / torch.sqrt(bnm.running_var + bnm.eps)
    return x[0] * scale.view(1, -1, 1, 1), x[1] if isinstance(x[1], TileMask) else None


def interpolate_from_module(x: Masked) -> Masked:
    """x2 bilinear upsample (align_corners=False) of a delta (reference ``:76-78``)."""
    d, m = fl.resolve(x, _scratch, "interp")
    n, c, h, w = d.shape
    out = fl.new_field(n, c, 2 * h, 2 * w, d.device)
    bits = fl.new_bits(n, 2 * h, 2 * w, d.device)
    mo = fl.upsample2x(d, m, None, None, out, bits, nat.UP_BILINEAR)
    return out, mo
