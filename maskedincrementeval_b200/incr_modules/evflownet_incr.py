"""Incremental EV-FlowNet: multi-resolution recurrent UNet with ConvGRU encoders
(reference: ``incr_modules/evflownet_incr.py:1-497``).

``compat="reference"`` reproduces the reference as written: inside a residual block one activation module
(one reservoir) serves both activations and the residual delta is lost because a list is extended with
``+=`` (``:221-226``, ``:261-263``).  ``compat="exact"`` gives the second activation its own reservoir and adds the
residual, which makes the accumulated incremental output equal to a dense recompute.
"""
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _native as nat
from .. import fields as fl
from ..fields import Scratch, TileMask, config
from .mask_incr_modules import (nnBatchNorm2dIncr, nnConvIncr, nnReservedActivation, nnReservedMultiplication,
                                nnSigmoidIncr, nnTanhIncr)


def _compat(module) -> str:
    c = getattr(module, "compat", None) or config.compat
    if c not in ("reference", "exact"):
        raise ValueError("compat must be 'reference' or 'exact'")
    return c


def skip_concat(x1, x2):
    """Zero-pad x1 to x2's spatial size and concatenate along channels (reference ``:9-14``); dense tensors."""
    diffY = x2.size()[2] - x1.size()[2]
    diffX = x2.size()[3] - x1.size()[3]
    padding = nn.ZeroPad2d((diffX // 2, diffX - diffX // 2, diffY // 2, diffY - diffY // 2))
    x1 = padding(x1)
    return torch.cat([x1, x2], dim=1)


def skip_concat_incr(x1_incr, x2_incr, scratch: Scratch, key: str):
    """Channel concatenation of two delta fields of equal spatial size, masks OR-ed."""
    a, ma = fl.resolve(x1_incr, scratch, key + ".a")
    b, mb = fl.resolve(x2_incr, scratch, key + ".b")
    if a.shape[2:] != b.shape[2:]:
        raise NotImplementedError("incremental skip_concat needs equal spatial sizes (pad the input to a multiple of 16)")
    n, ca, h, w = a.shape
    c = ca + b.shape[1]
    # pixel stride rounded up to 4 floats (the decoders see 2·C + 2 channels): 16-byte pixel addresses are what the
    # convolution's vector loads and TMA need; the padding channels are never written and stay zero
    full = scratch.get(key, (n, (c + 3) // 4 * 4, h, w), torch.float32, a.device, channels_last=True)
    out = full[:, :c]
    bits = scratch.get(key + ".bits", (fl.n_tiles(n, h, w),), torch.int64, a.device)
    return [out, fl.cat2(a, ma, b, mb, out, bits)]


class ConvGRUIncr(nn.Module):
    """ConvGRU on deltas (reference ``:18-94``).

    As written, the incremental pass ignores the reset gate and feeds cat(dx, dh_prev) to the out gate
    (``:58-61``); with the zero previous state the network always passes (``:451``) that equals the dense
    recurrence.  With ``prev_state=None`` the two gate convolutions only read the first ``input_size`` input
    channels."""

    def __init__(self, input_size, hidden_size, kernel_size, activation=None):
        super().__init__()
        padding = kernel_size // 2
        self.input_size = input_size
        self.hidden_size = hidden_size
        self.reset_gate = nnConvIncr(input_size + hidden_size, hidden_size, kernel_size, padding=padding)
        self.update_gate = nnConvIncr(input_size + hidden_size, hidden_size, kernel_size, padding=padding)
        self.out_gate = nnConvIncr(input_size + hidden_size, hidden_size, kernel_size, padding=padding)
        assert activation is None, "ConvGRU activation cannot be set (just for compatibility)"
        nn.init.orthogonal_(self.reset_gate.weight)
        nn.init.orthogonal_(self.update_gate.weight)
        nn.init.orthogonal_(self.out_gate.weight)
        nn.init.constant_(self.reset_gate.bias, 0.0)
        nn.init.constant_(self.update_gate.bias, 0.0)
        nn.init.constant_(self.out_gate.bias, 0.0)
        self.sigmoid1 = nnSigmoidIncr()
        self.sigmoid2 = nnSigmoidIncr()
        self.tanh = nnTanhIncr()
        self.mult = nnReservedMultiplication()
        self._scratch = Scratch()

    def forward(self, input_incr, prev_state):
        if prev_state is None:
            update = self.update_gate.forward_fused(input_incr, self.sigmoid1, cin_limit=self.input_size)
            out_inputs = self.out_gate.forward_fused(input_incr, self.tanh, cin_limit=self.input_size)
            new_state = self.mult(out_inputs, update)
            return new_state, new_state
        stacked = skip_concat_incr(input_incr, prev_state, self._scratch, "stacked")
        update = self.update_gate.forward_fused(stacked, self.sigmoid1)
        out_inputs = self.out_gate.forward_fused(stacked, self.tanh)
        diff = [out_inputs[0] - prev_state[0], None]
        new_state = [prev_state[0] + self.mult(diff, update)[0], None]
        return new_state, new_state

    def forward_refresh_reservoirs(self, x, prev_state):
        batch_size = x.data.size()[0]
        spatial_size = x.data.size()[2:]
        if prev_state is None:
            state_size = [batch_size, self.hidden_size] + list(spatial_size)
            prev_state = torch.zeros(state_size, dtype=x.dtype, device=x.device).to(memory_format=torch.channels_last)
        stacked_inputs = torch.cat([x, prev_state], dim=1)
        update = self.sigmoid1.forward_refresh_reservoirs(self.update_gate.forward_refresh_reservoirs(stacked_inputs))
        reset = self.sigmoid2.forward_refresh_reservoirs(self.reset_gate.forward_refresh_reservoirs(stacked_inputs))
        out_inputs = self.tanh.forward_refresh_reservoirs(
            self.out_gate.forward_refresh_reservoirs(torch.cat([x, prev_state * reset], dim=1)))
        new_state = prev_state + self.mult.forward_refresh_reservoirs(out_inputs - prev_state, update)
        return new_state, new_state


class ConvLayerIncr(nn.Module):
    """Convolution + incremental activation (reference ``:97-153``)."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, activation="relu", norm=None,
                 BN_momentum=0.1, w_scale=None, padding=None):
        super(ConvLayerIncr, self).__init__()
        bias = False if norm == "BN" else True
        if padding is None:
            padding = kernel_size // 2
        self.conv2d = nnConvIncr(in_channels, out_channels, kernel_size, stride, padding, bias=bias)
        if w_scale is not None:
            nn.init.uniform_(self.conv2d.weight, -w_scale, w_scale)
            nn.init.zeros_(self.conv2d.bias)
        if activation is not None:
            if hasattr(torch, activation):
                activation = getattr(torch, activation)
                self.activation = nnReservedActivation(activation)
        else:
            self.activation = None
        self.norm = norm
        if norm == "BN":
            self.norm_layer = nnBatchNorm2dIncr(out_channels, momentum=BN_momentum)
        elif norm == "IN":
            raise NotImplementedError

    def forward(self, x):
        if self.norm in ["BN", "IN"]:
            out = self.norm_layer(self.conv2d(x))
            return self.activation(out) if self.activation is not None else out
        return self.conv2d.forward_fused(x, self.activation)

    def forward_refresh_reservoirs(self, x):
        out = self.conv2d.forward_refresh_reservoirs(x)
        if self.norm in ["BN", "IN"]:
            out = self.norm_layer.forward_refresh_reservoirs(out)
        if self.activation is not None:
            out = self.activation.forward_refresh_reservoirs(out)
        return out


class RecurrentConvLayerIncr(nn.Module):
    """Strided convolution + activation, then a ConvGRU (reference ``:157-192``)."""

    def __init__(self, in_channels, out_channels, kernel_size=3, stride=1, activation_ff="relu", activation_rec=None,
                 norm=None, BN_momentum=0.1):
        super().__init__()
        self.conv = ConvLayerIncr(in_channels, out_channels, kernel_size, stride, activation_ff, norm,
                                  BN_momentum=BN_momentum)
        self.recurrent_block = ConvGRUIncr(input_size=out_channels, hidden_size=out_channels, kernel_size=3,
                                           activation=activation_rec)

    def forward(self, x, prev_state):
        x = self.conv(x)
        x, state = self.recurrent_block(x, prev_state)
        return x, state

    def forward_refresh_reservoirs(self, x, prev_state):
        x = self.conv.forward_refresh_reservoirs(x)
        x, state = self.recurrent_block.forward_refresh_reservoirs(x, prev_state)
        return x, state


class ResidualBlockIncr(nn.Module):
    """conv3x3 - act - conv3x3 - (+ residual) - act, returning ``(out2, out1)`` (reference ``:195-292``)."""

    def __init__(self, in_channels, out_channels, stride=1, activation="relu", downsample=None, norm=None,
                 BN_momentum=0.1, compat: Optional[str] = None):
        super(ResidualBlockIncr, self).__init__()
        bias = False if norm == "BN" else True
        self.conv1 = nnConvIncr(in_channels, out_channels, kernel_size=3, stride=stride, padding=1, bias=bias)
        if activation is not None:
            if hasattr(torch, activation):
                activation = getattr(torch, activation)
                self.activation = nnReservedActivation(activation)
                # second reservoir, used only when compat == "exact"
                self.activation2 = nnReservedActivation(activation)
        else:
            self.activation = None
            self.activation2 = None
        self.norm = norm
        if norm == "BN":
            self.bn1 = nnBatchNorm2dIncr(out_channels, momentum=BN_momentum)
            self.bn2 = nnBatchNorm2dIncr(out_channels, momentum=BN_momentum)
        elif norm == "IN":
            raise NotImplementedError
        self.conv2 = nnConvIncr(out_channels, out_channels, kernel_size=3, stride=1, padding=1, bias=bias)
        self.downsample = downsample
        self.compat = compat

    def forward(self, x):
        if self.norm in ["BN", "IN"]:
            raise NotImplementedError("batch-norm inside the incremental residual block has no fused kernel")
        exact = _compat(self) == "exact"
        residual = x
        if self.downsample:
            residual = self.downsample(x)
        out1 = self.conv1.forward_fused(x, self.activation)
        if exact:
            out2 = self.conv2.forward_fused(out1, self.activation2, addend=residual)
        else:
            out2 = self.conv2.forward_fused(out1, self.activation)
        return out2, out1

    def forward_refresh_reservoirs(self, x):
        exact = _compat(self) == "exact"
        residual = x
        out1 = self.conv1.forward_refresh_reservoirs(x)
        if self.norm in ["BN", "IN"]:
            out1 = self.bn1.forward_refresh_reservoirs(out1)
        if self.activation is not None:
            out1 = self.activation.forward_refresh_reservoirs(out1)
        out2 = self.conv2.forward_refresh_reservoirs(out1)
        if self.norm in ["BN", "IN"]:
            out2 = self.bn2.forward_refresh_reservoirs(out2)
        if self.downsample:
            residual = self.downsample.forward_refresh_reservoirs(x)
        out2 = out2 + residual
        if self.activation is not None:
            act2 = self.activation2 if exact else self.activation
            out2 = act2.forward_refresh_reservoirs(out2)
        return out2, out1


class UpsampleConvLayerIncr(nn.Module):
    """x2 bilinear upsample of the delta, convolution, incremental activation (reference ``:297-344``)."""

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, activation="relu", padding=None, norm=None):
        super(UpsampleConvLayerIncr, self).__init__()
        bias = False if norm == "BN" else True
        if padding is None:
            padding = kernel_size // 2
        self.conv2d = nnConvIncr(in_channels, out_channels, kernel_size, stride, padding, bias=bias)
        if activation is not None:
            activation = getattr(torch, activation)
            self.activation = nnReservedActivation(activation)
        else:
            self.activation = None
        self.norm = norm
        if norm == "BN":
            self.norm_layer = nnBatchNorm2dIncr(out_channels)
        elif norm == "IN":
            raise NotImplementedError
        self._scratch = Scratch()

    def forward(self, x):
        sc = self._scratch
        d, m = fl.resolve(x, sc, "in")
        n, c, h, w = d.shape
        # pixel stride rounded up to 4 floats (2·C + 2 input channels): see skip_concat_incr
        up = sc.get("up", (n, (c + 3) // 4 * 4, 2 * h, 2 * w), torch.float32, d.device, channels_last=True)[:, :c]
        ub = sc.get("up.bits", (fl.n_tiles(n, 2 * h, 2 * w),), torch.int64, d.device)
        mu = fl.upsample2x(d, m, None, None, up, ub, nat.UP_BILINEAR)
        return self.conv2d.forward_fused([up, mu], self.activation)

    def forward_refresh_reservoirs(self, x):
        x_upsampled = F.interpolate(x, scale_factor=2, mode="bilinear", align_corners=False)
        out = self.conv2d.forward_refresh_reservoirs(x_upsampled)
        if self.norm in ["BN", "IN"]:
            out = self.norm_layer.forward_refresh_reservoirs(out)
        if self.activation is not None:
            out = self.activation.forward_refresh_reservoirs(out)
        return out


class MultiResUNetRecurrentIncr(nn.Module):
    """EV-FlowNet (reference ``:347-495``): 4 recurrent encoders 64/128/256/512 (conv3x3 stride 2 + ConvGRU),
    2 residual blocks, 4 decoders with concatenated skips, a 1x1 tanh flow prediction after each decoder."""

    def __init__(self, compat: Optional[str] = None):
        super().__init__()
        self.final_activation = 'tanh'
        self.w_scale_pred = None
        self.num_encoders = 4
        self.num_residual_blocks = 2
        self.ff_act, self.rec_act = ['relu', None]
        self.skip_ftn = skip_concat
        self.kernel_size = 3
        self.num_bins = 2
        self.norm = None
        self.base_num_channels = 32
        self.channel_multiplier = 2
        self.num_output_channels = 2
        self.compat = compat
        self.encoder_input_sizes = [int(self.base_num_channels * pow(self.channel_multiplier, i))
                                    for i in range(self.num_encoders)]
        self.encoder_output_sizes = [int(self.base_num_channels * pow(self.channel_multiplier, i + 1))
                                     for i in range(self.num_encoders)]
        self.max_num_channels = self.encoder_output_sizes[-1]
        self.encoders = self.build_recurrent_encoders()
        self.resblocks = self.build_resblocks()
        self.decoders = self.build_multires_prediction_decoders()
        self.preds = self.build_multires_prediction_layer()
        self.num_states = self.num_encoders
        self.states = [None] * self.num_states
        self._scratch = Scratch()

    def build_recurrent_encoders(self):
        encoders = nn.ModuleList()
        for i, (input_size, output_size) in enumerate(zip(self.encoder_input_sizes, self.encoder_output_sizes)):
            if i == 0:
                input_size = self.num_bins
            encoders.append(RecurrentConvLayerIncr(input_size, output_size, kernel_size=self.kernel_size, stride=2,
                                                   activation_ff=self.ff_act, activation_rec=self.rec_act,
                                                   norm=self.norm))
        return encoders

    def build_resblocks(self):
        resblocks = nn.ModuleList()
        for i in range(self.num_residual_blocks):
            resblocks.append(ResidualBlockIncr(self.max_num_channels, self.max_num_channels, activation=self.ff_act,
                                               norm=self.norm))
        return resblocks

    def build_multires_prediction_layer(self):
        preds = nn.ModuleList()
        for output_size in reversed(self.encoder_input_sizes):
            preds.append(ConvLayerIncr(output_size, self.num_output_channels, 1, activation=self.final_activation,
                                       norm=self.norm))
        return preds

    def build_multires_prediction_decoders(self):
        decoder_input_sizes = reversed(self.encoder_output_sizes)
        decoder_output_sizes = reversed(self.encoder_input_sizes)
        decoders = nn.ModuleList()
        for i, (input_size, output_size) in enumerate(zip(decoder_input_sizes, decoder_output_sizes)):
            prediction_channels = 0 if i == 0 else self.num_output_channels
            decoders.append(UpsampleConvLayerIncr(2 * input_size + prediction_channels, output_size,
                                                  kernel_size=self.kernel_size, activation=self.ff_act, norm=self.norm))
        return decoders

    def reset_states(self):
        """Forget the recurrent state the dense pass carries from call to call (reference ``:478-480``)."""
        self.states = [None] * self.num_states

    def forward(self, x_incr):
        c = _compat(self)
        for rb in self.resblocks:
            rb.compat = c
        states_incr = [None] * self.num_states
        blocks = []
        for i, encoder in enumerate(self.encoders):
            x_incr, state = encoder(x_incr, states_incr[i])
            blocks.append(x_incr)
            states_incr[i] = state
        for resblock in self.resblocks:
            x_incr, _ = resblock(x_incr)
        predictions = []
        for i, (decoder, pred) in enumerate(zip(self.decoders, self.preds)):
            x_incr = skip_concat_incr(x_incr, blocks[self.num_encoders - i - 1], self._scratch, f"skip{i}")
            if i > 0:
                x_incr = skip_concat_incr(predictions[-1], x_incr, self._scratch, f"pskip{i}")
            x_incr = decoder(x_incr)
            predictions.append(pred(x_incr))
        return predictions

    def forward_refresh_reservoirs(self, x):
        c = _compat(self)
        for rb in self.resblocks:
            rb.compat = c
        blocks = []
        for i, encoder in enumerate(self.encoders):
            x, state = encoder.forward_refresh_reservoirs(x, self.states[i])
            blocks.append(x)
            self.states[i] = state
        for resblock in self.resblocks:
            x, _ = resblock.forward_refresh_reservoirs(x)
        predictions = []
        for i, (decoder, pred) in enumerate(zip(self.decoders, self.preds)):
            x = self.skip_ftn(x, blocks[self.num_encoders - i - 1])
            if i > 0:
                x = self.skip_ftn(predictions[-1], x)
            x = decoder.forward_refresh_reservoirs(x)
            predictions.append(pred.forward_refresh_reservoirs(x))
        return predictions
