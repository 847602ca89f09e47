"""Incremental E2Depth: recurrent UNet with ConvLSTM encoders (reference: ``incr_modules/e2depth_incr.py:1-500``).

Same classes, constructor arguments, ``state_dict`` keys and two-entry-point protocol as the reference.
The dense entry point (``forward_refresh_reservoirs``) is the reference's computation with library
calls; the incremental entry point runs the fused libmie kernels.

``compat`` ("reference" | "exact", default ``fields.config.compat``) selects how the incremental pass is
wired.  The reference sums two ``[delta, mask]`` lists with ``+`` where it means a tensor sum
(``:333`` used at ``:430``/``:434``, and ``:113``), which concatenates them: the decoder skips and the
head skip are lost and the LSTM cell delta is the product m1 alone.  "reference" reproduces that;
"exact" sums the deltas, which makes the accumulated output equal to a dense recompute.
"""
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _native as nat
from .. import fields as fl
from ..fields import Scratch, TileMask, config
from .masked_types import DenseT, Masked
from .mask_incr_modules import (IncrementReserve, KFencedMaskModule, PointwiseMultiplyIncr, nnBatchNorm2dIncr,
                                nnConvIncr, nnReluIncr, nnReservedActivation, nnReservedMultiplication,
                                nnSigmoidIncr, nnTanhIncr)
from .mask_incr_functional import interpolate_from_module
from .utils import print_sparsity  # noqa: F401  (imported by the reference too)


def _compat(module) -> str:
    c = getattr(module, "compat", None) or config.compat
    if c not in ("reference", "exact"):
        raise ValueError("compat must be 'reference' or 'exact'")
    return c


class ConvLayerIncr(nn.Module):
    """Convolution + optional eval-BN + incremental activation (reference ``:12-52``)."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, activation='relu', norm=None):
        super(ConvLayerIncr, self).__init__()
        bias = False if norm == 'BN' else True
        self.conv2d = nnConvIncr(in_channels, out_channels, kernel_size, stride, padding, bias=bias)
        if activation is not None:
            op = getattr(torch, activation, 'relu')
            self.activation = nnReservedActivation(op)
        else:
            self.activation = None
        self.norm = norm
        if norm == 'BN':
            self.norm_layer = nnBatchNorm2dIncr(out_channels)
        elif norm == 'IN':
            raise NotImplementedError

    def forward(self, x_incr: Masked, addend: Optional[Masked] = None) -> Masked:
        # The reference tests `self.norm == ['BN', 'IN']` here (``:35``), which is never true: the norm layer
        # is skipped in the incremental pass.  Kept.
        return self.conv2d.forward_fused(x_incr, self.activation, addend)

    def forward_refresh_reservoirs(self, x: DenseT):
        out = self.conv2d.forward_refresh_reservoirs(x)
        if self.norm in ['BN', 'IN']:
            out = self.norm_layer.forward_refresh_reservoirs(out)
        if self.activation is not None:
            out = self.activation.forward_refresh_reservoirs(out)
        return out


class ConvLSTMIncr(nn.Module):
    """ConvLSTM cell on deltas (reference ``:55-166``).

    The incremental pass is two launches after the gate convolution's tile dilation: the 3x3 gate
    convolution over the active tiles, and one point-wise kernel that folds the gate deltas into the
    pre-activation state and evaluates the five nonlinearities and three products of the reference.
    State kept between steps: gate pre-activations ``g`` [N,4C,H,W] (the reference's four activation
    reservoirs side by side), the accumulated cell ``cell`` and the accumulated previous-cell input ``cprev``.
    The reference's gate, product and activation sub-modules are created for attribute compatibility; the
    activation ones are given views of ``g`` as reservoirs."""

    def __init__(self, input_size: int, hidden_size: int, kernel_size: int, prev_c_res: IncrementReserve = None):
        super(ConvLSTMIncr, self).__init__()
        self.input_size = input_size
        self.hidden_size = hidden_size
        self.kernel_size = kernel_size
        pad = kernel_size // 2
        self.zero_tensors = {}
        self.zero_tensors_incr = {}
        self.Gates = nnConvIncr(input_size + hidden_size, 4 * hidden_size, kernel_size, padding=pad)
        self.m1 = nnReservedMultiplication()
        self.m2 = nnReservedMultiplication()
        self.m3 = nnReservedMultiplication()
        self.sigmoid1 = nnSigmoidIncr()
        self.sigmoid2 = nnSigmoidIncr()
        self.sigmoid3 = nnSigmoidIncr()
        self.tanh1 = nnTanhIncr()
        self.tanh2 = nnTanhIncr()
        self.compat = None
        self._scratch = Scratch()
        self._g = self._cell = self._cprev = None
        self._cprev_zero = True

    def forward(self, input_incr: Masked, prev_state_incr):
        if self._g is None:
            raise RuntimeError("forward_refresh_reservoirs must run before the first incremental step")
        sc = self._scratch
        x, mx = fl.resolve(input_incr, sc, "in")
        n, _, h, w = x.shape
        C = self.hidden_size
        dev = x.device
        dcp = mcp = None
        if prev_state_incr is None:
            # zero hidden delta: the gate convolution only sees the first input_size channels
            gates = self.Gates.forward_fused([x, mx], cin_limit=self.input_size)
        else:
            prev_h, prev_c = prev_state_incr
            dh_prev, mh = fl.resolve(prev_h, sc, "hprev")
            dcp, mcp = fl.resolve(prev_c, sc, "cprev")
            stacked = sc.get("stacked", (n, self.input_size + C, h, w), torch.float32, dev, channels_last=True)
            sbits = sc.get("stacked.bits", (fl.n_tiles(n, h, w),), torch.int64, dev)
            ms = fl.cat2(x, mx, dh_prev, mh, stacked, sbits)
            gates = self.Gates.forward_fused([stacked, ms])
            self._cprev_zero = False
        dg, mg = gates
        dh = sc.get("dh", (n, C, h, w), torch.float32, dev, channels_last=True)
        dc = sc.get("dc", (n, C, h, w), torch.float32, dev, channels_last=True)
        hb = sc.get("dh.bits", (fl.n_tiles(n, h, w),), torch.int64, dev)
        cb = sc.get("dc.bits", (fl.n_tiles(n, h, w),), torch.int64, dev)
        use_cprev = not self._cprev_zero
        nat.check(nat.lib.mie_convlstm_point(
            dg.data_ptr(), fl.pixel_stride(dg), mg.bits.data_ptr(), self._g.data_ptr(), fl.pixel_stride(self._g),
            nat.ptr(dcp), fl.pixel_stride(dcp) if dcp is not None else 0, mcp.bits.data_ptr() if mcp is not None else None,
            self._cprev.data_ptr() if use_cprev else None, fl.pixel_stride(self._cprev),
            self._cell.data_ptr(), fl.pixel_stride(self._cell), dh.data_ptr(), fl.pixel_stride(dh), hb.data_ptr(),
            dc.data_ptr(), fl.pixel_stride(dc), cb.data_ptr(), n, C, h, w, 1 if _compat(self) == "exact" else 0,
            0.0, nat.stream_ptr(dev)), "convlstm_point")
        hidden = [dh, TileMask(hb, n, h, w)]
        cell = [dc, TileMask(cb, n, h, w)]
        return hidden, cell

    def forward_refresh_reservoirs(self, input_, prev_state):
        batch_size = input_.data.size()[0]
        spatial_size = input_.data.size()[2:]
        given = prev_state is not None
        if prev_state is None:
            state_size = tuple([batch_size, self.hidden_size] + list(spatial_size))
            if state_size not in self.zero_tensors:
                self.zero_tensors[state_size] = (
                    torch.zeros(state_size, device=input_.device).to(memory_format=torch.channels_last),
                    torch.zeros(state_size, device=input_.device).to(memory_format=torch.channels_last))
            prev_state = self.zero_tensors[tuple(state_size)]
        prev_h, prev_c = prev_state
        stacked_inputs = torch.cat((input_, prev_h), 1)
        gates = self.Gates.forward_refresh_reservoirs(stacked_inputs)
        in_gate, remember_gate, out_gate, cell_gate = gates.chunk(4, 1)
        in_gate = torch.sigmoid(in_gate)
        remember_gate = torch.sigmoid(remember_gate)
        out_gate = torch.sigmoid(out_gate)
        cell_gate = torch.tanh(cell_gate)
        cell = in_gate * cell_gate + remember_gate * prev_c
        hidden = out_gate * torch.tanh(cell)
        # persistent state of the fused incremental kernel (stable addresses across refreshes)
        self._g = self._store(self._g, gates)
        self._cell = self._store(self._cell, cell)
        self._cprev = self._store(self._cprev, prev_c)
        self._cprev_zero = not given
        C = self.hidden_size
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

    def forward(self, x_incr, prev_state_incr):
        x_incr = self.conv(x_incr)
        state_incr = self.recurrent_block(x_incr, prev_state_incr)
        x_incr = state_incr[0]
        return x_incr, state_incr

    def forward_refresh_reservoirs(self, x: DenseT, prev_state):
        x = self.conv.forward_refresh_reservoirs(x)
        state = self.recurrent_block.forward_refresh_reservoirs(x, prev_state)
        x = state[0]
        return x, state


class ResidualBlockIncr(nn.Module):
    """conv3x3 - relu - conv3x3 - (+ residual) - relu (reference ``:189-240``); the residual sum and the
    second activation are fused into the second convolution's epilogue."""

    def __init__(self, in_channels, out_channels, stride=1, downsample=None, norm=None):
        super().__init__()
        bias = False if norm == 'BN' else True
        self.conv1 = nnConvIncr(in_channels, out_channels, kernel_size=3, stride=stride, padding=1, bias=bias)
        self.norm = norm
        if norm == 'BN':
            self.bn1 = nnBatchNorm2dIncr(out_channels)
            self.bn2 = nnBatchNorm2dIncr(out_channels)
        elif norm == 'IN':
            raise NotImplementedError
        self.relu1 = nnReluIncr()
        self.conv2 = nnConvIncr(out_channels, out_channels, kernel_size=3, stride=1, padding=1, bias=bias)
        self.relu2 = nnReluIncr()
        self.downsample = downsample

    def forward(self, x_incr: Masked) -> Masked:
        if self.norm in ['BN', 'IN']:
            raise NotImplementedError("batch-norm inside the incremental residual block has no fused kernel")
        residual_incr = x_incr
        if self.downsample:
            residual_incr = self.downsample(x_incr)
        out_incr = self.conv1.forward_fused(x_incr, self.relu1)
        return self.conv2.forward_fused(out_incr, self.relu2, addend=residual_incr)

    def forward_refresh_reservoirs(self, x):
        residual = x
        out = self.conv1.forward_refresh_reservoirs(x)
        if self.norm in ['BN', 'IN']:
            out = self.bn1(out)
        out = self.relu1.forward_refresh_reservoirs(out)
        out = self.conv2.forward_refresh_reservoirs(out)
        if self.norm in ['BN', 'IN']:
            out = self.bn2(out)
        if self.downsample:
            residual = self.downsample.forward_refresh_reservoirs(x)
        out = out + residual
        out = self.relu2.forward_refresh_reservoirs(out)
        return out


class TransposedConvLayerIncr(nn.Module):
    """The reference's transposed-convolution decoder refers to an undefined class and cannot be
    constructed (``:248``); it cannot be here either."""

    def __init__(self, *args, **kwargs):
        super().__init__()
        raise NotImplementedError("TransposedConvLayerIncr: use use_upsample_conv=True (the reference's transposed "
                                  "path references an undefined nnConvTranspose2dIncr)")


class UpsampleConvLayerIncr(nn.Module):
    """x2 bilinear upsample of the delta (optionally of the sum with a skip delta), convolution,
    incremental activation (reference ``:279-325``)."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, activation='relu', norm=None):
        super().__init__()
        bias = False if norm == 'BN' else True
        self.conv2d = nnConvIncr(in_channels, out_channels, kernel_size, stride, padding, bias=bias)
        if activation is not None:
            op = getattr(torch, activation, 'relu')
            self.activation = nnReservedActivation(op)
        else:
            self.activation = None
        self.norm = norm
        if norm == 'BN':
            self.norm_layer = nnBatchNorm2dIncr(out_channels)
        elif norm == 'IN':
            raise NotImplementedError
        self._scratch = Scratch()

    def forward(self, x_incr: Masked, skip_incr: Optional[Masked] = None) -> Masked:
        sc = self._scratch
        x, mx = fl.resolve(x_incr, sc, "in")
        n, c, h, w = x.shape
        s = ms = None
        if skip_incr is not None:
            s, ms = fl.resolve(skip_incr, sc, "skip")
        up = sc.get("up", (n, c, 2 * h, 2 * w), torch.float32, x.device, channels_last=True)
        ub = sc.get("up.bits", (fl.n_tiles(n, 2 * h, 2 * w),), torch.int64, x.device)
        mu = fl.upsample2x(x, mx, s, ms, up, ub, nat.UP_BILINEAR)
        return self.conv2d.forward_fused([up, mu], self.activation)

    def forward_refresh_reservoirs(self, x):
        x_upsampled = F.interpolate(x, scale_factor=2, mode='bilinear', align_corners=False)
        out = self.conv2d.forward_refresh_reservoirs(x_upsampled)
        if self.norm in ['BN', 'IN']:
            out = self.norm_layer.forward_refresh_reservoirs(out)
        if self.activation is not None:
            out = self.activation.forward_refresh_reservoirs(out)
        return out


class BaseUNetIncr(nn.Module):
    """Shared UNet scaffolding (reference ``:328-379``)."""

    def __init__(self, num_input_channels, num_output_channels=1, skip_type='sum', activation='sigmoid',
                 num_encoders=4, base_num_channels=32, num_residual_blocks=2, norm=None, use_upsample_conv=True):
        super().__init__()
        self.num_input_channels = num_input_channels
        self.num_output_channels = num_output_channels
        self.skip_type = skip_type
        self.apply_skip_connection = lambda x1, x2: x1 + x2   # dense tensors only (refresh path)
        self.norm = norm
        if skip_type != 'sum':
            raise NotImplementedError("only skip_type='sum' is wired (the reference's lambda is a sum as well)")
        self.UpsampleLayer = UpsampleConvLayerIncr if use_upsample_conv else TransposedConvLayerIncr
        self.num_encoders = num_encoders
        self.base_num_channels = base_num_channels
        self.num_residual_blocks = num_residual_blocks
        self.max_num_channels = self.base_num_channels * pow(2, self.num_encoders)
        assert (self.num_input_channels > 0)
        assert (self.num_output_channels > 0)
        self.encoder_input_sizes = [self.base_num_channels * pow(2, i) for i in range(self.num_encoders)]
        self.encoder_output_sizes = [self.base_num_channels * pow(2, i + 1) for i in range(self.num_encoders)]
        op = getattr(torch, activation, 'relu')
        self.activation = nnReservedActivation(op)

    def build_resblocks(self):
        self.resblocks = nn.ModuleList()
        for i in range(self.num_residual_blocks):
            self.resblocks.append(ResidualBlockIncr(self.max_num_channels, self.max_num_channels, norm=self.norm))

    def build_decoders(self):
        decoder_input_sizes = list(reversed([self.base_num_channels * pow(2, i + 1) for i in range(self.num_encoders)]))
        self.decoders = nn.ModuleList()
        for input_size in decoder_input_sizes:
            self.decoders.append(self.UpsampleLayer(input_size if self.skip_type == 'sum' else 2 * input_size,
                                                    input_size // 2, kernel_size=5, padding=2, norm=self.norm))

    def build_prediction_layer(self):
        self.pred = ConvLayerIncr(self.base_num_channels if self.skip_type == 'sum' else 2 * self.base_num_channels,
                                  self.num_output_channels, 1, activation=None, norm=self.norm)


class UNetRecurrentIncr(BaseUNetIncr):
    """Recurrent UNet (reference ``:382-468``): head conv5x5, ``num_encoders`` strided conv + ConvLSTM
    encoders, residual blocks, upsampling decoders, 1x1 prediction and a final activation."""

    def __init__(self, num_input_channels, num_output_channels=1, skip_type='sum',
                 recurrent_block_type='convlstm', activation='sigmoid', num_encoders=4, base_num_channels=32,
                 num_residual_blocks=2, norm=None, use_upsample_conv=True, compat: Optional[str] = None):
        super().__init__(num_input_channels, num_output_channels, skip_type, activation, num_encoders,
                         base_num_channels, num_residual_blocks, norm, use_upsample_conv)
        self.compat = compat
        self.head = ConvLayerIncr(self.num_input_channels, self.base_num_channels, kernel_size=5, stride=1, padding=2)
        self.encoders = nn.ModuleList()
        for input_size, output_size in zip(self.encoder_input_sizes, self.encoder_output_sizes):
            self.encoders.append(RecurrentConvLayerIncr(input_size, output_size, kernel_size=5, stride=2, padding=2,
                                                        recurrent_block_type=recurrent_block_type, norm=self.norm))
        self.build_resblocks()
        self.build_decoders()
        self.build_prediction_layer()
        self._scratch = Scratch()

    def forward(self, x_incr: Masked, prev_states_incr):
        exact = _compat(self) == "exact"
        for enc in self.encoders:
            enc.recurrent_block.compat = _compat(self)
        x_incr = self.head(x_incr)
        head = x_incr
        if prev_states_incr is None:
            prev_states_incr = [None] * self.num_encoders
        blocks = []
        states_incr = []
        for i, encoder in enumerate(self.encoders):
            x_incr, state_incr = encoder(x_incr, prev_states_incr[i])
            blocks.append(x_incr)
            states_incr.append(state_incr)
        for resblock in self.resblocks:
            x_incr = resblock(x_incr)
        for i, decoder in enumerate(self.decoders):
            # "reference": the skip is lost (two lists concatenated, then only element 0 is read)
            x_incr = decoder(x_incr, blocks[self.num_encoders - i - 1] if exact else None)
        if exact:
            x, mx = x_incr
            n, c, h, w = x.shape
            s = self._scratch.get("tail", (n, c, h, w), torch.float32, x.device, channels_last=True)
            sb = self._scratch.get("tail.bits", (fl.n_tiles(n, h, w),), torch.int64, x.device)
            x_incr = [s, fl.add(x, mx, head[0], head[1], s, sb)]
        # 1x1 prediction and the final activation in one launch
        pred_incr = self.pred.conv2d.forward_fused(x_incr, self.activation)
        return pred_incr, states_incr

    def forward_refresh_reservoirs(self, x: DenseT, prev_states):
        x = self.head.forward_refresh_reservoirs(x)
        head = x
        if prev_states is None:
            prev_states = [None] * self.num_encoders
        blocks = []
        states = []
        for i, encoder in enumerate(self.encoders):
            x, state = encoder.forward_refresh_reservoirs(x, prev_states[i])
            blocks.append(x)
            states.append(state)
        for resblock in self.resblocks:
            x = resblock.forward_refresh_reservoirs(x)
        for i, decoder in enumerate(self.decoders):
            x = decoder.forward_refresh_reservoirs(self.apply_skip_connection(x, blocks[self.num_encoders - i - 1]))
        pred = self.pred.forward_refresh_reservoirs(self.apply_skip_connection(x, head))
        pred = self.activation.forward_refresh_reservoirs(pred)
        return pred, states


class E2VIDRecurrentIncr(nn.Module):
    """Top-level model (reference ``:471-498``).  The reference derives from ``BaseE2VID`` of an un-vendored
    sub-project, which only turns these config keys into attributes; they are read from the dict directly:
    ``num_bins`` (required), ``skip_type``, ``num_encoders``, ``base_num_channels``, ``num_residual_blocks``,
    ``norm``, ``use_upsample_conv``, ``recurrent_block_type``; plus ``compat`` (this library's)."""

    def __init__(self, config):
        super().__init__()
        assert ('num_bins' in config)
        self.num_bins = int(config['num_bins'])
        self.skip_type = str(config.get('skip_type', 'sum'))
        self.num_encoders = int(config.get('num_encoders', 4))
        self.base_num_channels = int(config.get('base_num_channels', 32))
        self.num_residual_blocks = int(config.get('num_residual_blocks', 2))
        self.norm = config.get('norm', None)
        self.use_upsample_conv = bool(config.get('use_upsample_conv', True))
        try:
            self.recurrent_block_type = str(config['recurrent_block_type'])
        except KeyError:
            self.recurrent_block_type = 'convlstm'
        self.unetrecurrent = UNetRecurrentIncr(num_input_channels=self.num_bins, num_output_channels=1,
                                               skip_type=self.skip_type,
                                               recurrent_block_type=self.recurrent_block_type, activation='sigmoid',
                                               num_encoders=self.num_encoders,
                                               base_num_channels=self.base_num_channels,
                                               num_residual_blocks=self.num_residual_blocks, norm=self.norm,
                                               use_upsample_conv=self.use_upsample_conv,
                                               compat=config.get('compat', None))

    def forward(self, event_tensor: Masked, prev_states):
        img_pred, states = self.unetrecurrent.forward(event_tensor, prev_states)
        return img_pred, states

    def forward_refresh_reservoirs(self, event_tensor: DenseT, prev_states):
        img_pred, states = self.unetrecurrent.forward_refresh_reservoirs(event_tensor, prev_states)
        return img_pred, states
