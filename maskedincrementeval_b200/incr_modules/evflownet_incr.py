"""Incremental EV-FlowNet: multi-resolution recurrent UNet with ConvGRU encoders
(reference: ``incr_modules/evflownet_incr.py:1-497``).

Every class states its topology once (``_run``) and is evaluated by the dense or the incremental interpreter of
``_algebra``; class names, constructor arguments and ``state_dict`` keys are the reference's.

``compat="reference"`` reproduces the reference as written: inside a residual block one activation module (one
reservoir) serves both activations and the residual delta is lost because a list is extended with ``+=``
(``:221-226``, ``:261-263``).  ``compat="exact"`` gives the second activation its own reservoir and adds the residual,
which makes the accumulated incremental output equal to a dense recompute.
"""
from typing import Optional

import torch
import torch.nn as nn

from ..fields import Scratch, config
from ._algebra import DENSE, INCR, run_dense
from .mask_incr_modules import (nnBatchNorm2dIncr, nnConvIncr, nnReservedActivation, nnReservedMultiplication,
                                nnSigmoidIncr, nnTanhIncr)


def _compat(module) -> str:
    c = getattr(module, "compat", None) or config.compat
    if c not in ("reference", "exact"):
        raise ValueError("compat must be 'reference' or 'exact'")
    return c


def skip_concat(x1, x2):
    """Zero-pad x1 to x2's spatial size and concatenate along channels (reference ``:9-14``); dense tensors."""
    return DENSE.cat(x1, x2)


def skip_concat_incr(x1_incr, x2_incr, scratch: Scratch, key: str):
    """Channel concatenation of two delta fields of equal spatial size, masks OR-ed."""
    return INCR.cat(x1_incr, x2_incr, scratch, key)


def _activation(name):
    return nnReservedActivation(getattr(torch, name)) if name is not None and hasattr(torch, name) else None


class ConvGRUIncr(nn.Module):
    """ConvGRU on deltas (reference ``:18-94``).

    As written, the incremental pass ignores the reset gate and feeds cat(dx, dh_prev) to the out gate
    (``:58-61``); with the zero previous state the network always passes (``:451``) that equals the dense
    recurrence.  With ``prev_state=None`` the two gate convolutions only read the first ``input_size`` input
    channels."""

    def __init__(self, input_size, hidden_size, kernel_size, activation=None):
        super().__init__()
        assert activation is None, "ConvGRU activation cannot be set (just for compatibility)"
        self.input_size, self.hidden_size = input_size, hidden_size
        gates = ("reset_gate", "update_gate", "out_gate")
        for name in gates:          # built first, initialised afterwards: the order in which the reference draws
            setattr(self, name, nnConvIncr(input_size + hidden_size, hidden_size, kernel_size, padding=kernel_size // 2))
        for name in gates:
            nn.init.orthogonal_(getattr(self, name).weight)
        for name in gates:
            nn.init.constant_(getattr(self, name).bias, 0.0)
        self.sigmoid1, self.sigmoid2, self.tanh = nnSigmoidIncr(), nnSigmoidIncr(), nnTanhIncr()
        self.mult = nnReservedMultiplication()
        self._scratch = Scratch()

    def forward(self, input_incr, prev_state):
        if prev_state is None:
            update = INCR.conv(self.update_gate, input_incr, self.sigmoid1, cin_limit=self.input_size)
            candidate = INCR.conv(self.out_gate, input_incr, self.tanh, cin_limit=self.input_size)
            state = self.mult(candidate, update)
            return state, state
        stacked = INCR.cat(input_incr, prev_state, self._scratch, "stacked")
        update = INCR.conv(self.update_gate, stacked, self.sigmoid1)
        candidate = INCR.conv(self.out_gate, stacked, self.tanh)
        moved = self.mult([candidate[0] - prev_state[0], None], update)
        state = [prev_state[0] + moved[0], None]
        return state, state

    def refresh_native(self, x_pair, prev_state):
        """The dense GRU step from the zero state on the kernels: with h_prev = 0 the reset gate has no effect and the
        new state is tanh(out_gate(x)) * sigmoid(update_gate(x)); both gate convolutions read the first ``input_size``
        channels only.  (A carried state takes the library pass: see ``_algebra.dense_ops``.)"""
        from ._algebra import NATIVE
        if prev_state is not None:
            raise NotImplementedError("the dense ConvGRU step on the kernels starts from the zero state")
        update = NATIVE.conv(self.update_gate, x_pair, self.sigmoid1, cin_limit=self.input_size)
        candidate = NATIVE.conv(self.out_gate, x_pair, self.tanh, cin_limit=self.input_size)
        state = NATIVE.mul(self.mult, candidate, update)
        return state, state

    def forward_refresh_reservoirs(self, x, prev_state):
        if prev_state is None:
            prev_state = x.new_zeros((x.shape[0], self.hidden_size) + tuple(x.shape[2:])).contiguous(
                memory_format=torch.channels_last)
        stacked = torch.cat([x, prev_state], dim=1)
        update = DENSE.conv(self.update_gate, stacked, self.sigmoid1)
        reset = DENSE.conv(self.reset_gate, stacked, self.sigmoid2)
        candidate = DENSE.conv(self.out_gate, torch.cat([x, prev_state * reset], dim=1), self.tanh)
        state = prev_state + DENSE.mul(self.mult, candidate - prev_state, update)
        return state, state


class ConvLayerIncr(nn.Module):
    """Convolution + incremental activation (reference ``:97-153``)."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, activation="relu", norm=None,
                 BN_momentum=0.1, w_scale=None, padding=None):
        super().__init__()
        if norm == "IN":
            raise NotImplementedError
        padding = kernel_size // 2 if padding is None else padding
        self.conv2d = nnConvIncr(in_channels, out_channels, kernel_size, stride, padding, bias=norm != "BN")
        if w_scale is not None:
            nn.init.uniform_(self.conv2d.weight, -w_scale, w_scale)
            nn.init.zeros_(self.conv2d.bias)
        if activation is None:
            self.activation = None
        elif hasattr(torch, activation):      # an unknown name leaves the attribute unset, as in the reference (``:117-121``)
            self.activation = _activation(activation)
        self.norm = norm
        if norm == "BN":
            self.norm_layer = nnBatchNorm2dIncr(out_channels, momentum=BN_momentum)

    def _run(self, ops, x):
        return ops.conv(self.conv2d, x, self.activation, norm=self.norm_layer if self.norm == "BN" else None)

    def forward(self, x):
        return self._run(INCR, x)

    def forward_refresh_reservoirs(self, x):
        return self._run(DENSE, x)


class RecurrentConvLayerIncr(nn.Module):
    """Strided convolution + activation, then a ConvGRU (reference ``:157-192``)."""

    def __init__(self, in_channels, out_channels, kernel_size=3, stride=1, activation_ff="relu", activation_rec=None,
                 norm=None, BN_momentum=0.1):
        super().__init__()
        self.conv = ConvLayerIncr(in_channels, out_channels, kernel_size, stride, activation_ff, norm,
                                  BN_momentum=BN_momentum)
        self.recurrent_block = ConvGRUIncr(input_size=out_channels, hidden_size=out_channels, kernel_size=3,
                                           activation=activation_rec)

    def _run(self, ops, x, prev_state):
        x = self.conv._run(ops, x)
        return ops.gru(self.recurrent_block, x, prev_state)

    def forward(self, x, prev_state):
        return self._run(INCR, x, prev_state)

    def forward_refresh_reservoirs(self, x, prev_state):
        return self._run(DENSE, x, prev_state)


class ResidualBlockIncr(nn.Module):
    """conv3x3 - act - conv3x3 - (+ residual) - act, returning ``(out2, out1)`` (reference ``:195-292``)."""

    def __init__(self, in_channels, out_channels, stride=1, activation="relu", downsample=None, norm=None,
                 BN_momentum=0.1, compat: Optional[str] = None):
        super().__init__()
        if norm == "IN":
            raise NotImplementedError
        self.conv1 = nnConvIncr(in_channels, out_channels, kernel_size=3, stride=stride, padding=1, bias=norm != "BN")
        # the reference's one activation module, and a second reservoir that only compat == "exact" uses
        self.activation, self.activation2 = _activation(activation), _activation(activation)
        self.norm = norm
        if norm == "BN":
            self.bn1 = nnBatchNorm2dIncr(out_channels, momentum=BN_momentum)
            self.bn2 = nnBatchNorm2dIncr(out_channels, momentum=BN_momentum)
        self.conv2 = nnConvIncr(out_channels, out_channels, kernel_size=3, stride=1, padding=1, bias=norm != "BN")
        self.downsample = downsample
        self.compat = compat

    def _run(self, ops, x):
        bn = self.norm == "BN"
        if bn and ops.incremental:
            raise NotImplementedError("batch-norm inside the incremental residual block has no fused kernel")
        exact = _compat(self) == "exact"
        residual = x
        if self.downsample:
            residual = self.downsample(x) if ops.incremental else self.downsample.forward_refresh_reservoirs(x)
        out1 = ops.conv(self.conv1, x, self.activation, norm=self.bn1 if bn else None)
        # as written, the incremental pass loses the residual and re-uses the first activation's reservoir
        keep_residual = exact or not ops.incremental
        out2 = ops.conv(self.conv2, out1, self.activation2 if exact else self.activation,
                        addend=residual if keep_residual else None, norm=self.bn2 if bn else None)
        return out2, out1

    def forward(self, x):
        return self._run(INCR, x)

    def forward_refresh_reservoirs(self, x):
        return self._run(DENSE, x)


class UpsampleConvLayerIncr(nn.Module):
    """x2 bilinear upsample of the delta, convolution, incremental activation (reference ``:297-344``)."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, activation="relu", padding=None, norm=None):
        super().__init__()
        if norm == "IN":
            raise NotImplementedError
        padding = kernel_size // 2 if padding is None else padding
        self.conv2d = nnConvIncr(in_channels, out_channels, kernel_size, stride, padding, bias=norm != "BN")
        self.activation = None if activation is None else nnReservedActivation(getattr(torch, activation))
        self.norm = norm
        if norm == "BN":
            self.norm_layer = nnBatchNorm2dIncr(out_channels)
        self._scratch = Scratch()

    def _run(self, ops, x):
        up = ops.upsample2x(x, None, self._scratch, pad4=True)      # 2*C + 2 input channels: 16-byte pixel stride
        norm = self.norm_layer if (self.norm == "BN" and not ops.incremental) else None
        return ops.conv(self.conv2d, up, self.activation, norm=norm)

    def forward(self, x):
        return self._run(INCR, x)

    def forward_refresh_reservoirs(self, x):
        return self._run(DENSE, x)


class MultiResUNetRecurrentIncr(nn.Module):
    """EV-FlowNet (reference ``:347-495``): 4 recurrent encoders 64/128/256/512 (conv3x3 stride 2 + ConvGRU),
    2 residual blocks, 4 decoders with concatenated skips, a 1x1 tanh flow prediction after each decoder."""

    def __init__(self, compat: Optional[str] = None):
        super().__init__()
        # fixed hyper-parameters (reference ``:351-365``)
        self.final_activation, self.w_scale_pred = 'tanh', None
        self.num_encoders, self.num_residual_blocks = 4, 2
        self.ff_act, self.rec_act = 'relu', None
        self.skip_ftn = skip_concat
        self.kernel_size, self.num_bins, self.norm = 3, 2, None
        self.base_num_channels, self.channel_multiplier, self.num_output_channels = 32, 2, 2
        self.compat = compat
        widths = [int(self.base_num_channels * self.channel_multiplier ** i) for i in range(self.num_encoders + 1)]
        self.encoder_input_sizes, self.encoder_output_sizes = widths[:-1], widths[1:]
        self.max_num_channels = top = widths[-1]
        k, out_c = self.kernel_size, self.num_output_channels
        self.encoders = nn.ModuleList(
            RecurrentConvLayerIncr(self.num_bins if i == 0 else ci, co, kernel_size=k, stride=2, activation_ff=self.ff_act,
                                   activation_rec=self.rec_act, norm=self.norm)
            for i, (ci, co) in enumerate(zip(widths[:-1], widths[1:])))
        self.resblocks = nn.ModuleList(ResidualBlockIncr(top, top, activation=self.ff_act, norm=self.norm)
                                       for _ in range(self.num_residual_blocks))
        # decoder i reads the concatenation [previous prediction (from the second level on) | features | skip]
        self.decoders = nn.ModuleList(
            UpsampleConvLayerIncr(2 * ci + (out_c if i else 0), co, kernel_size=k, activation=self.ff_act, norm=self.norm)
            for i, (ci, co) in enumerate(zip(reversed(widths[1:]), reversed(widths[:-1]))))
        self.preds = nn.ModuleList(ConvLayerIncr(co, out_c, 1, activation=self.final_activation, norm=self.norm)
                                   for co in reversed(widths[:-1]))
        self.num_states = self.num_encoders
        self.states = [None] * self.num_states
        self._scratch = Scratch()

    def reset_states(self):
        """Forget the recurrent state the dense pass carries from call to call (reference ``:478-480``)."""
        self.states = [None] * self.num_states

    def _run(self, ops, x):
        for rb in self.resblocks:
            rb.compat = _compat(self)
        # the incremental pass starts every call from a zero state delta (``:451``); the dense pass carries its state
        states = [None] * self.num_states if ops.incremental else list(self.states)
        blocks = []
        for i, encoder in enumerate(self.encoders):
            x, states[i] = encoder._run(ops, x, states[i])
            blocks.append(x)
        for resblock in self.resblocks:
            x, _ = resblock._run(ops, x)
        predictions = []
        for i, (decoder, pred) in enumerate(zip(self.decoders, self.preds)):
            x = ops.cat(x, blocks.pop(), self._scratch, f"skip{i}")
            if predictions:
                x = ops.cat(predictions[-1], x, self._scratch, f"pskip{i}")
            x = decoder._run(ops, x)
            predictions.append(pred._run(ops, x))
        return predictions, states

    def forward(self, x_incr):
        return self._run(INCR, x_incr)[0]

    def forward_refresh_reservoirs(self, x):
        predictions, self.states = run_dense(self, x)
        return predictions
