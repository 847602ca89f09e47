"""Incremental "delayed prediction" EV-FlowNet: a feed-forward multi-resolution UNet whose per-level decoder
outputs and flow predictions are interpolated to the input resolution, concatenated and reduced by two 1x1 layers
(reference: ``incr_modules/delayedevflownet_incr.py:155-476``).

Differences from the reference, both deliberate: every returned flow is a ``[delta, TileMask]`` pair (the reference
returns bare tensors for the interpolated predictions and a pair for the delayed one, ``:262-276``), and the
interpolated fields are written straight into their channel slice of one concatenation buffer instead of being
concatenated afterwards.  ``compat`` selects the residual-block wiring as in ``evflownet_incr``.
"""
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _native as nat
from .. import fields as fl
from ..fields import Scratch, TileMask
from .mask_incr_modules import set_precision
from .evflownet_incr import ConvLayerIncr, ResidualBlockIncr, UpsampleConvLayerIncr, skip_concat, skip_concat_incr


class DelayedMultiResUNetIncr(nn.Module):
    """Reference ``DelayedMultiResUNetIncr`` (``:155-383``) with its ``BaseUNet`` (``:59-152``)."""

    def __init__(self, unet_kwargs, compat: Optional[str] = None):
        super().__init__()
        kw = dict(unet_kwargs)
        self.final_activation = kw.pop("final_activation", "none")
        self.base_num_channels = kw["base_num_channels"]
        self.num_encoders = kw["num_encoders"]
        self.num_residual_blocks = kw["num_residual_blocks"]
        self.num_output_channels = kw["num_output_channels"]
        self.kernel_size = kw.get("kernel_size", 5)
        self.norm = kw.get("norm")
        self.num_bins = kw["num_bins"]
        self.channel_multiplier = kw.get("channel_multiplier", 2)
        self.skip_type = "concat"
        if not kw.get("use_upsample_conv", True):
            raise NotImplementedError("transposed-convolution decoders have no incremental form in the reference either")
        assert self.num_output_channels > 0
        m, b, ne = self.channel_multiplier, self.base_num_channels, self.num_encoders
        self.encoder_input_sizes = [int(b * pow(m, i)) for i in range(ne)]
        self.encoder_output_sizes = [int(b * pow(m, i + 1)) for i in range(ne)]
        self.max_num_channels = self.encoder_output_sizes[-1]
        k = self.kernel_size

        self.encoders = nn.ModuleList(
            ConvLayerIncr(self.num_bins if i == 0 else ci, co, kernel_size=k, stride=2, padding=k // 2, norm=self.norm)
            for i, (ci, co) in enumerate(zip(self.encoder_input_sizes, self.encoder_output_sizes)))
        self.resblocks = nn.ModuleList(
            ResidualBlockIncr(self.max_num_channels, self.max_num_channels, norm=self.norm, compat=compat)
            for _ in range(self.num_residual_blocks))
        self.decoders = nn.ModuleList(
            UpsampleConvLayerIncr((2 if i == 0 else 1) * ci, co, kernel_size=k, padding=k // 2, norm=self.norm)
            for i, (ci, co) in enumerate(zip(reversed(self.encoder_output_sizes), reversed(self.encoder_input_sizes))))
        self.preds = nn.ModuleList(
            ConvLayerIncr(co, self.num_output_channels, 1, activation=self.final_activation, norm=self.norm)
            for co in reversed(self.encoder_input_sizes))
        delayed_in = sum(self.encoder_input_sizes[:-1]) + 2 * ne
        self.delayed_pred_layer_list = nn.ModuleList([
            ConvLayerIncr(delayed_in, b, 1, activation="relu", norm=self.norm),
            ConvLayerIncr(b + 2 * ne, 2, 1, activation=self.final_activation, norm=self.norm)])
        self._scratch = Scratch()

    # -- incremental ---------------------------------------------------------------------------------
    def forward(self, x):
        sc = self._scratch
        d0, m0 = fl.resolve(x, sc, "in")
        x = [d0, m0]
        n, _, H, W = d0.shape
        ne = self.num_encoders
        blocks = []
        for enc in self.encoders:
            x = enc(x)
            blocks.append(x)
        for rb in self.resblocks:
            x, _ = rb(x)

        # one buffer holds the concatenation [decoder outputs 1..ne-1 | predictions 0..ne-1] at full resolution;
        # every interpolation writes its own channel slice
        c_dec = sum(self.encoder_input_sizes[:-1])
        c_tot = c_dec + 2 * ne
        cat = sc.get("delayed.in", (n, (c_tot + 3) // 4 * 4, H, W), torch.float32, d0.device, channels_last=True)
        nt = fl.n_tiles(n, H, W)
        off_dec, off_pred = 0, c_dec
        masks, preds = [], []
        for i, (dec, pred) in enumerate(zip(self.decoders, self.preds)):
            d_in = skip_concat_incr(x, blocks[ne - 1], sc, "skip0") if i == 0 else blocks[ne - i - 1]
            d_out = dec(d_in)
            dd, dm = fl.resolve(d_out, sc, f"dec{i}")
            scale = H // dd.shape[2]
            if scale * dd.shape[2] != H or scale * dd.shape[3] != W:
                raise NotImplementedError("the input size must be a multiple of 2**num_encoders")
            if i != 0:
                c = dd.shape[1]
                bits = sc.get(f"delayed.dec{i}.bits", (nt,), torch.int64, d0.device)
                masks.append(fl.upsample(dd, dm, cat[:, off_dec:off_dec + c], bits, scale))
                off_dec += c
            p = pred(d_out)
            pd, pm = fl.resolve(p, sc, f"pred{i}")
            bits = sc.get(f"delayed.pred{i}.bits", (nt,), torch.int64, d0.device)
            sl = cat[:, off_pred:off_pred + 2]
            pmask = fl.upsample(pd, pm, sl, bits, scale)
            masks.append(pmask)
            preds.append([sl, pmask])
            off_pred += 2
        union = sc.get("delayed.union", (nt,), torch.int64, d0.device)
        torch.bitwise_or(masks[0].bits, masks[1].bits, out=union)
        for m in masks[2:]:
            union.bitwise_or_(m.bits)
        um = TileMask(union, n, H, W)
        mid = self.delayed_pred_layer_list[0]([cat[:, :c_tot], um])
        tail = skip_concat_incr(mid, [cat[:, c_tot - 2 * ne:c_tot], um], sc, "delayed.tail")
        out = self.delayed_pred_layer_list[1](tail)
        return preds, out

    # -- dense refresh -------------------------------------------------------------------------------
    def forward_refresh_reservoirs(self, x):
        size = x.shape[-2:]
        ne = self.num_encoders
        blocks = []
        for enc in self.encoders:
            x = enc.forward_refresh_reservoirs(x)
            blocks.append(x)
        for rb in self.resblocks:
            x, _ = rb.forward_refresh_reservoirs(x)
        outs, preds = [], []
        for i, (dec, pred) in enumerate(zip(self.decoders, self.preds)):
            d_in = skip_concat(x, blocks[ne - 1]) if i == 0 else blocks[ne - i - 1]
            d_out = dec.forward_refresh_reservoirs(d_in)
            if i != 0:
                outs.append(F.interpolate(d_out, size=size, mode="bilinear", align_corners=False))
            preds.append(F.interpolate(pred.forward_refresh_reservoirs(d_out), size=size, mode="bilinear",
                                       align_corners=False))
        din = torch.cat(outs + preds, dim=1)
        mid = self.delayed_pred_layer_list[0].forward_refresh_reservoirs(din)
        out = self.delayed_pred_layer_list[1].forward_refresh_reservoirs(torch.cat([mid, din[:, -2 * ne:]], dim=1))
        return preds, out


class DelayedEVFlowNetIncr(nn.Module):
    """Reference ``DelayedEVFlowNetIncr`` (``:387-476``): fixed hyper-parameters around the UNet above."""

    def __init__(self, unet_kwargs, num_bins, compat: Optional[str] = None, precision: Optional[str] = "split"):
        super().__init__()
        self.crop = None
        kw = dict(unet_kwargs)
        self.mask = kw["mask_output"]
        kw.update({"base_num_channels": kw["base_num_channels"], "num_encoders": 4, "num_residual_blocks": 2,
                   "num_output_channels": 2, "skip_type": "concat", "norm": None, "num_bins": num_bins,
                   "use_upsample_conv": True, "kernel_size": kw["kernel_size"], "channel_multiplier": 2,
                   "final_activation": "tanh"})
        self.num_encoders = 4
        for k in ("name", "eval", "encoding", "mask_output", "mask_smoothing", "flow_scaling"):
            kw.pop(k, None)
        self.multires_unet = DelayedMultiResUNetIncr(kw, compat=compat)
        # An un-normalised ReLU stack fed by raw event counts: a TF32 input's 2^-11 relative error is about 2e-3 of the
        # flow range after a few dozen steps, so the tensor-core layers run in split precision by default.
        set_precision(self, precision)

    def reset_states(self):
        pass

    def forward(self, x_incr):
        if self.crop is not None:
            raise NotImplementedError("cropping is not part of the incremental path")
        flows, delayed = self.multires_unet(x_incr)
        return {"flow": flows + [delayed]}

    def forward_refresh_reservoirs(self, x):
        if self.crop is not None:
            raise NotImplementedError("cropping is not part of the incremental path")
        flows, delayed = self.multires_unet.forward_refresh_reservoirs(x)
        return {"flow": flows + [delayed]}
