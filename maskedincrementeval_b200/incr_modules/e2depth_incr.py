"""Incremental E2Depth: recurrent UNet with ConvLSTM encoders (reference: ``incr_modules/e2depth_incr.py:1-500``).

Same class names, constructor arguments, ``state_dict`` keys and two-entry-point protocol as the reference.  Each class
states its topology once (``_run``) and is evaluated by the dense or the incremental interpreter of ``_algebra``:
``forward_refresh_reservoirs`` is the dense pass that refills the persistent state, ``forward`` the fused incremental
pass over the active tiles.

``compat`` ("reference" | "exact", default ``fields.config.compat``) selects how the incremental pass is wired.  The
reference sums two ``[delta, mask]`` lists with ``+`` where it means a tensor sum (``:333`` used at ``:430``/``:434``,
and ``:113``), which concatenates them: the decoder skips and the head skip are lost and the LSTM cell delta is the
product m1 alone.  "reference" reproduces that; "exact" sums the deltas, which makes the accumulated output equal to a
dense recompute.
"""
from typing import Optional

import torch
import torch.nn as nn

from .. import _native as nat
from .. import fields as fl
from ..fields import Scratch, TileMask, config
from ._algebra import DENSE, INCR, NATIVE, dense_ops
from .masked_types import DenseT, Masked
from .mask_incr_modules import (IncrementReserve, KFencedMaskModule, PointwiseMultiplyIncr, nnBatchNorm2dIncr,  # noqa: F401
                                nnConvIncr, nnReluIncr, nnReservedActivation, nnReservedMultiplication,
                                nnSigmoidIncr, nnTanhIncr)
from .mask_incr_functional import interpolate_from_module  # noqa: F401  (imported by the reference too)
from .utils import print_sparsity  # noqa: F401  (imported by the reference too)


def _compat(module) -> str:
    c = getattr(module, "compat", None) or config.compat
    if c not in ("reference", "exact"):
        raise ValueError("compat must be 'reference' or 'exact'")
    return c


def _conv_block(owner: nn.Module, cin: int, cout: int, k: int, stride: int, padding: int, activation, norm):
    """The members every convolution layer of this network has: ``conv2d``, ``activation`` (or None), ``norm`` and,
    for norm == 'BN', ``norm_layer`` (reference ``:12-29``, ``:281-299``)."""
    if norm == 'IN':
        raise NotImplementedError
    owner.conv2d = nnConvIncr(cin, cout, k, stride, padding, bias=norm != 'BN')
    owner.activation = None if activation is None else nnReservedActivation(getattr(torch, activation, 'relu'))
    owner.norm = norm
    if norm == 'BN':
        owner.norm_layer = nnBatchNorm2dIncr(cout)


class ConvLayerIncr(nn.Module):
    """Convolution, optional eval batch-norm, incremental activation (reference ``:12-52``)."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, activation='relu', norm=None):
        super().__init__()
        _conv_block(self, in_channels, out_channels, kernel_size, stride, padding, activation, norm)

    def _run(self, ops, x, addend=None):
        # The reference tests `self.norm == ['BN', 'IN']` in its incremental pass (``:35``), which is never true:
        # only the dense pass applies the norm layer.  Kept.
        norm = self.norm_layer if (self.norm == 'BN' and not ops.incremental) else None
        return ops.conv(self.conv2d, x, self.activation, addend, norm)

    def forward(self, x_incr: Masked, addend: Optional[Masked] = None) -> Masked:
        return self._run(INCR, x_incr, addend)

    def forward_refresh_reservoirs(self, x: DenseT):
        return self._run(DENSE, x)


class ConvLSTMIncr(nn.Module):
    """ConvLSTM cell on deltas (reference ``:55-166``).

    The incremental pass is two launches after the gate convolution's tile dilation: the 3x3 gate convolution over the
    active tiles, and one point-wise kernel that folds the gate deltas into the pre-activation state and evaluates the
    five nonlinearities and three products of the reference.  State kept between steps: gate pre-activations ``g``
    [N,4C,H,W] (the reference's four activation reservoirs side by side), the accumulated cell ``cell`` and the
    accumulated previous-cell input ``cprev``.  The reference's gate, product and activation sub-modules are created
    for attribute compatibility; the activation ones are given views of ``g`` as reservoirs."""

    def __init__(self, input_size: int, hidden_size: int, kernel_size: int, prev_c_res: IncrementReserve = None):
        super().__init__()
        self.input_size, self.hidden_size, self.kernel_size = input_size, hidden_size, kernel_size
        self.zero_tensors, self.zero_tensors_incr = {}, {}
        self.Gates = nnConvIncr(input_size + hidden_size, 4 * hidden_size, kernel_size, padding=kernel_size // 2)
        self.m1, self.m2, self.m3 = (nnReservedMultiplication() for _ in range(3))
        self.sigmoid1, self.sigmoid2, self.sigmoid3 = (nnSigmoidIncr() for _ in range(3))
        self.tanh1, self.tanh2 = nnTanhIncr(), nnTanhIncr()
        self.compat = None
        self._scratch = Scratch()
        self._g = self._cell = self._cprev = self._hsent = None
        self._cprev_zero, self._hsent_valid = True, False

    def forward(self, input_incr: Masked, prev_state_incr):
        if self._g is None:
            raise RuntimeError("forward_refresh_reservoirs must run before the first incremental step")
        sc = self._scratch
        x, mx = fl.resolve(input_incr, sc, "in")
        n, _, h, w = x.shape
        C, dev = self.hidden_size, x.device
        dcp = mcp = None
        if prev_state_incr is None:
            # zero hidden delta: the gate convolution only sees the first input_size channels
            dg, mg = self.Gates.forward_fused([x, mx], cin_limit=self.input_size)
        else:
            dh_prev, mh = fl.resolve(prev_state_incr[0], sc, "hprev")
            dcp, mcp = fl.resolve(prev_state_incr[1], sc, "cprev")
            dg, mg = self.Gates.forward_fused(INCR.cat([x, mx], [dh_prev, mh], sc, "stacked"))
            self._cprev_zero = False
        dh = sc.get("dh", (n, C, h, w), torch.float32, dev, channels_last=True)
        dc = sc.get("dc", (n, C, h, w), torch.float32, dev, channels_last=True)
        hb = sc.get("dh.bits", (fl.n_tiles(n, h, w),), torch.int64, dev)
        cb = sc.get("dc.bits", (fl.n_tiles(n, h, w),), torch.int64, dev)
        use_cprev = not self._cprev_zero
        thr, hs = self._hidden_carry()
        nat.check(nat.lib.mie_convlstm_point(
            dg.data_ptr(), fl.pixel_stride(dg), mg.bits.data_ptr(), self._g.data_ptr(), fl.pixel_stride(self._g),
            nat.ptr(dcp), fl.pixel_stride(dcp) if dcp is not None else 0, mcp.bits.data_ptr() if mcp is not None else None,
            self._cprev.data_ptr() if use_cprev else None, fl.pixel_stride(self._cprev),
            self._cell.data_ptr(), fl.pixel_stride(self._cell), dh.data_ptr(), fl.pixel_stride(dh), hb.data_ptr(),
            dc.data_ptr(), fl.pixel_stride(dc), cb.data_ptr(), n, C, h, w, 1 if _compat(self) == "exact" else 0,
            thr, nat.ptr(hs), fl.pixel_stride(hs) if hs is not None else 0,
            sc.get("hidden.mask.scratch", (2 * fl.n_tiles(n, h, w),), torch.int64, dev).data_ptr() if hs is not None else None,
            fl.take_tail(hb), nat.stream_ptr(dev)), "convlstm_point")
        return [dh, TileMask(hb, n, h, w)], [dc, TileMask(cb, n, h, w)]

    def _refill_hidden_carry(self, hidden):
        """After a refresh: everything is sent, the carry buffer (if one exists) equals the new hidden state.  Refilled
        in place and at once, not on the next step: that step may be a CUDA-graph replay that runs no host code."""
        if self._hsent is not None and self._hsent.shape == hidden.shape and self._hsent.device == hidden.device:
            self._hsent.copy_(hidden)
            self._hsent_valid = True
        else:
            self._hsent_valid = False

    def _hidden_carry(self):
        """``(threshold, buffer of the hidden state sent so far)`` for a thresholded step, ``(0, None)`` for a lossless
        one.  With ``config.threshold > 0`` and ``config.carry`` the cell's hidden output is thresholded like an
        activation's: its delta is taken against what has been sent, groups of 16 channels whose change stays under
        the threshold are withheld and remain pending.  The buffer is rebuilt from the state (sigmoid(o) * tanh(cell),
        the hidden value itself) whenever a thresholded step follows a refresh or a lossless step; what was pending at
        that moment is sent with it."""
        thr = float(config.threshold)
        if thr <= 0.0 or not config.carry or self.hidden_size % 16:
            self._hsent_valid = False       # a lossless step does not advance the buffer
            return 0.0, None
        if not self._hsent_valid:
            C = self.hidden_size
            hidden = torch.sigmoid(self._g[:, 2 * C:3 * C]) * torch.tanh(self._cell)
            if self._hsent is None or self._hsent.shape != hidden.shape or self._hsent.device != hidden.device:
                self._hsent = hidden.contiguous(memory_format=torch.channels_last)
            else:
                self._hsent.copy_(hidden)   # in place: a captured step keeps pointing at this buffer
            self._hsent_valid = True
        return thr, self._hsent

    def refresh_native(self, x_pair, prev_state):
        """The dense LSTM step on the kernels: with the three state tensors zeroed, the incremental point kernel fed
        the dense gate pre-activations (and the dense previous cell as a delta against zero) computes
        cell = sigmoid(i) * tanh(g) + sigmoid(f) * c_prev and hidden = sigmoid(o) * tanh(cell) -- every "old" term
        of its product rules is sigmoid(0) = 1/2 or tanh(0) = 0 -- and leaves ``g``, ``cell`` and ``cprev`` refilled.
        Returns ``([hidden, mask], [cell, mask])`` in the cell's persistent buffers."""
        sc = self._scratch
        x, mx = x_pair
        n, _, h, w = x.shape
        C, dev = self.hidden_size, x.device
        shapes = ((n, 4 * C, h, w), (n, C, h, w), (n, C, h, w))
        bufs = []
        for buf, shape in zip((self._g, self._cell, self._cprev), shapes):
            if buf is None or tuple(buf.shape) != shape or buf.device != dev:
                buf = fl.new_field(*shape, dev)
            else:
                buf.zero_()
            bufs.append(buf)
        self._g, self._cell, self._cprev = bufs
        dcp = mcp = None
        if prev_state is None:
            dg, mg = self.Gates.forward_fused([x, mx], cin_limit=self.input_size, refresh=True)
        else:
            (h_prev, mh), (dcp, mcp) = prev_state
            dg, mg = self.Gates.forward_fused(INCR.cat([x, mx], [h_prev, mh], sc, "stacked"), refresh=True)
        self._cprev_zero = prev_state is None
        dh = sc.get("dh", (n, C, h, w), torch.float32, dev, channels_last=True)
        dc = sc.get("dc", (n, C, h, w), torch.float32, dev, channels_last=True)
        hb = sc.get("dh.bits", (fl.n_tiles(n, h, w),), torch.int64, dev)
        cb = sc.get("dc.bits", (fl.n_tiles(n, h, w),), torch.int64, dev)
        nat.check(nat.lib.mie_convlstm_point(
            dg.data_ptr(), fl.pixel_stride(dg), mg.bits.data_ptr(), self._g.data_ptr(), fl.pixel_stride(self._g),
            nat.ptr(dcp), fl.pixel_stride(dcp) if dcp is not None else 0, mcp.bits.data_ptr() if mcp is not None else None,
            self._cprev.data_ptr() if dcp is not None else None, fl.pixel_stride(self._cprev),
            self._cell.data_ptr(), fl.pixel_stride(self._cell), dh.data_ptr(), fl.pixel_stride(dh), hb.data_ptr(),
            dc.data_ptr(), fl.pixel_stride(dc), cb.data_ptr(), n, C, h, w, 1, 0.0, None, 0, None, fl.take_tail(hb),
            nat.stream_ptr(dev)), "convlstm_point")
        self._refill_hidden_carry(dh)
        for i, mod in enumerate((self.sigmoid1, self.sigmoid2, self.sigmoid3, self.tanh1)):
            mod.in_res.reservoir = self._g[:, i * C:(i + 1) * C]
        self.tanh2.in_res.reservoir = self._cell
        return [dh, TileMask(hb, n, h, w)], [dc, TileMask(cb, n, h, w)]

    def forward_refresh_reservoirs(self, input_, prev_state):
        """Dense LSTM step; refills ``g``, ``cell`` and ``cprev`` in place (stable addresses across refreshes)."""
        C = self.hidden_size
        zero_state = prev_state is None
        if zero_state:
            key = (input_.shape[0], C) + tuple(input_.shape[2:])
            if key not in self.zero_tensors:
                z = torch.zeros(key, device=input_.device).contiguous(memory_format=torch.channels_last)
                self.zero_tensors[key] = (z, z.clone())
            prev_state = self.zero_tensors[key]
        h_prev, c_prev = prev_state
        gates = self.Gates.forward_refresh_reservoirs(torch.cat((input_, h_prev), 1))
        squashed = torch.sigmoid(gates[:, :3 * C])                      # in, remember, out
        cell = torch.addcmul(squashed[:, C:2 * C] * c_prev, squashed[:, :C], torch.tanh(gates[:, 3 * C:]))
        hidden = squashed[:, 2 * C:] * torch.tanh(cell)
        self._g, self._cell, self._cprev = (self._store(b, v) for b, v in ((self._g, gates), (self._cell, cell),
                                                                          (self._cprev, c_prev)))
        self._cprev_zero = zero_state
        self._refill_hidden_carry(hidden)
        for i, mod in enumerate((self.sigmoid1, self.sigmoid2, self.sigmoid3, self.tanh1)):
            mod.in_res.reservoir = self._g[:, i * C:(i + 1) * C]
        self.tanh2.in_res.reservoir = self._cell
        return hidden, cell

    @staticmethod
    def _store(buf, x):
        x = x.detach()
        if buf is not None and buf.shape == x.shape and buf.device == x.device:
            buf.copy_(x)
            return buf
        return x.clone().contiguous(memory_format=torch.channels_last)


class RecurrentConvLayerIncr(nn.Module):
    """Strided convolution + activation, then a ConvLSTM (reference ``:169-186``)."""

    def __init__(self, in_channels, out_channels, kernel_size=3, stride=1, padding=0,
                 recurrent_block_type='convlstm', activation='relu', norm=None):
        super().__init__()
        self.conv = ConvLayerIncr(in_channels, out_channels, kernel_size, stride, padding, activation, norm)
        self.recurrent_block = ConvLSTMIncr(input_size=out_channels, hidden_size=out_channels, kernel_size=3)

    def _run(self, ops, x, prev_state):
        state = ops.lstm(self.recurrent_block, self.conv._run(ops, x), prev_state)
        return state[0], state

    def forward(self, x_incr, prev_state_incr):
        return self._run(INCR, x_incr, prev_state_incr)

    def forward_refresh_reservoirs(self, x: DenseT, prev_state):
        return self._run(DENSE, x, prev_state)


class ResidualBlockIncr(nn.Module):
    """conv3x3 - relu - conv3x3 - (+ residual) - relu (reference ``:189-240``); incrementally the residual sum and the
    second activation are fused into the second convolution's epilogue."""

    def __init__(self, in_channels, out_channels, stride=1, downsample=None, norm=None):
        super().__init__()
        if norm == 'IN':
            raise NotImplementedError
        self.conv1 = nnConvIncr(in_channels, out_channels, kernel_size=3, stride=stride, padding=1, bias=norm != 'BN')
        self.norm = norm
        if norm == 'BN':
            self.bn1, self.bn2 = nnBatchNorm2dIncr(out_channels), nnBatchNorm2dIncr(out_channels)
        self.relu1 = nnReluIncr()
        self.conv2 = nnConvIncr(out_channels, out_channels, kernel_size=3, stride=1, padding=1, bias=norm != 'BN')
        self.relu2 = nnReluIncr()
        self.downsample = downsample

    def _run(self, ops, x):
        bn = self.norm == 'BN'
        if bn and ops.incremental:
            raise NotImplementedError("batch-norm inside the incremental residual block has no fused kernel")
        residual = x
        if self.downsample:
            residual = self.downsample(x) if ops.incremental else self.downsample.forward_refresh_reservoirs(x)
        y = ops.conv(self.conv1, x, self.relu1, norm=self.bn1 if bn else None)
        return ops.conv(self.conv2, y, self.relu2, addend=residual, norm=self.bn2 if bn else None)

    def forward(self, x_incr: Masked) -> Masked:
        return self._run(INCR, x_incr)

    def forward_refresh_reservoirs(self, x):
        return self._run(DENSE, x)


class TransposedConvLayerIncr(nn.Module):
    """The reference's transposed-convolution decoder refers to an undefined class and cannot be
    constructed (``:248``); it cannot be here either."""

    def __init__(self, *args, **kwargs):
        super().__init__()
        raise NotImplementedError("TransposedConvLayerIncr: use use_upsample_conv=True (the reference's transposed "
                                  "path references an undefined nnConvTranspose2dIncr)")


class UpsampleConvLayerIncr(nn.Module):
    """x2 bilinear upsample (optionally of the sum with a skip), convolution, activation (reference ``:279-325``)."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, activation='relu', norm=None):
        super().__init__()
        _conv_block(self, in_channels, out_channels, kernel_size, stride, padding, activation, norm)
        self._scratch = Scratch()

    def _run(self, ops, x, skip=None):
        norm = self.norm_layer if (self.norm == 'BN' and not ops.incremental) else None
        return ops.conv(self.conv2d, ops.upsample2x(x, skip, self._scratch), self.activation, norm=norm)

    def forward(self, x_incr: Masked, skip_incr: Optional[Masked] = None) -> Masked:
        return self._run(INCR, x_incr, skip_incr)

    def forward_refresh_reservoirs(self, x):
        return self._run(DENSE, x)


class BaseUNetIncr(nn.Module):
    """Hyper-parameters shared by the UNets and the final activation (reference ``:328-379``)."""

    def __init__(self, num_input_channels, num_output_channels=1, skip_type='sum', activation='sigmoid',
                 num_encoders=4, base_num_channels=32, num_residual_blocks=2, norm=None, use_upsample_conv=True):
        super().__init__()
        if skip_type != 'sum':
            raise NotImplementedError("only skip_type='sum' is wired (the reference's lambda is a sum as well)")
        assert num_input_channels > 0 and num_output_channels > 0
        self.num_input_channels, self.num_output_channels = num_input_channels, num_output_channels
        self.skip_type, self.norm = skip_type, norm
        self.apply_skip_connection = torch.add          # dense tensors (the reference's lambda, ``:333``)
        self.UpsampleLayer = UpsampleConvLayerIncr if use_upsample_conv else TransposedConvLayerIncr
        self.num_encoders, self.base_num_channels = num_encoders, base_num_channels
        self.num_residual_blocks = num_residual_blocks
        widths = [base_num_channels * 2 ** i for i in range(num_encoders + 1)]
        self.encoder_input_sizes, self.encoder_output_sizes = widths[:-1], widths[1:]
        self.max_num_channels = widths[-1]
        self.activation = nnReservedActivation(getattr(torch, activation, 'relu'))


class UNetRecurrentIncr(BaseUNetIncr):
    """Recurrent UNet (reference ``:382-468``): head conv5x5, ``num_encoders`` strided conv + ConvLSTM encoders,
    residual blocks, upsampling decoders with summed skips, 1x1 prediction and a final activation."""

    def __init__(self, num_input_channels, num_output_channels=1, skip_type='sum',
                 recurrent_block_type='convlstm', activation='sigmoid', num_encoders=4, base_num_channels=32,
                 num_residual_blocks=2, norm=None, use_upsample_conv=True, compat: Optional[str] = None):
        super().__init__(num_input_channels, num_output_channels, skip_type, activation, num_encoders,
                         base_num_channels, num_residual_blocks, norm, use_upsample_conv)
        self.compat = compat
        top = self.max_num_channels
        self.head = ConvLayerIncr(num_input_channels, base_num_channels, kernel_size=5, stride=1, padding=2)
        self.encoders = nn.ModuleList(
            RecurrentConvLayerIncr(ci, co, kernel_size=5, stride=2, padding=2, recurrent_block_type=recurrent_block_type,
                                   norm=norm) for ci, co in zip(self.encoder_input_sizes, self.encoder_output_sizes))
        self.resblocks = nn.ModuleList(ResidualBlockIncr(top, top, norm=norm) for _ in range(num_residual_blocks))
        self.decoders = nn.ModuleList(self.UpsampleLayer(c, c // 2, kernel_size=5, padding=2, norm=norm)
                                      for c in reversed(self.encoder_output_sizes))
        self.pred = ConvLayerIncr(base_num_channels, num_output_channels, 1, activation=None, norm=norm)
        self._scratch = Scratch()

    def _run(self, ops, x, prev_states):
        # "reference" wiring of the incremental pass: the skips are lost (two lists concatenated, element 0 read)
        skips = not ops.incremental or _compat(self) == "exact"
        for enc in self.encoders:
            enc.recurrent_block.compat = _compat(self)
        prev_states = prev_states if prev_states is not None else [None] * self.num_encoders
        head = x = self.head._run(ops, x)
        blocks, states = [], []
        for enc, prev in zip(self.encoders, prev_states):
            x, state = enc._run(ops, x, prev)
            blocks.append(x)
            states.append(state)
        for block in self.resblocks:
            x = block._run(ops, x)
        for dec in self.decoders:
            skip = blocks.pop()
            if ops.pairs:
                x = dec._run(ops, x, skip if skips else None)      # the sum happens inside the upsample kernel
            else:
                x = dec._run(ops, x + skip)
        # 1x1 prediction and the final activation, with the head's skip added as the kernel reads its input (one launch
        # incrementally; the reference sums first, ``:430-434``)
        norm = self.pred.norm_layer if (self.norm == 'BN' and not ops.incremental) else None
        return ops.conv(self.pred.conv2d, x, self.activation, norm=norm, second=head if skips else None), states

    def forward(self, x_incr: Masked, prev_states_incr):
        return self._run(INCR, x_incr, prev_states_incr)

    def forward_refresh_reservoirs(self, x: DenseT, prev_states):
        ops = dense_ops(self, x)
        if ops is not NATIVE:
            return self._run(DENSE, x, prev_states)
        prev = None if prev_states is None else [None if s is None else (NATIVE.lift(s[0]), NATIVE.lift(s[1]))
                                                 for s in prev_states]
        pred, states = self._run(NATIVE, NATIVE.lift(x), prev)
        out = NATIVE.lower(pred), [(NATIVE.lower(h), NATIVE.lower(c)) for h, c in states]
        fl.reset_delta_state(self)       # the kernels left dense values where the next step expects zero deltas
        return out


class E2VIDRecurrentIncr(nn.Module):
    """Top-level model (reference ``:471-498``).  The reference derives from ``BaseE2VID`` of an un-vendored
    sub-project, which only turns these config keys into attributes; they are read from the dict directly:
    ``num_bins`` (required), ``skip_type``, ``num_encoders``, ``base_num_channels``, ``num_residual_blocks``,
    ``norm``, ``use_upsample_conv``, ``recurrent_block_type``; plus ``compat`` (this library's)."""

    DEFAULTS = dict(skip_type='sum', num_encoders=4, base_num_channels=32, num_residual_blocks=2, norm=None,
                    use_upsample_conv=True, recurrent_block_type='convlstm')

    def __init__(self, config):
        super().__init__()
        assert 'num_bins' in config
        self.num_bins = int(config['num_bins'])
        for key, default in self.DEFAULTS.items():
            value = config.get(key, default)
            setattr(self, key, value if default is None else type(default)(value))
        self.unetrecurrent = UNetRecurrentIncr(
            num_input_channels=self.num_bins, num_output_channels=1, skip_type=self.skip_type,
            recurrent_block_type=self.recurrent_block_type, activation='sigmoid', num_encoders=self.num_encoders,
            base_num_channels=self.base_num_channels, num_residual_blocks=self.num_residual_blocks, norm=self.norm,
            use_upsample_conv=self.use_upsample_conv, compat=config.get('compat', None))

    def forward(self, event_tensor: Masked, prev_states):
        return self.unetrecurrent.forward(event_tensor, prev_states)

    def forward_refresh_reservoirs(self, event_tensor: DenseT, prev_states):
        return self.unetrecurrent.forward_refresh_reservoirs(event_tensor, prev_states)
