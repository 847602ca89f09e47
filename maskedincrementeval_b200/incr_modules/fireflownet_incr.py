"""Incremental FireFlowNet (reference: ``incr_modules/fireflownet_incr.py:1-74``): E1, E2, R1, E3, R2 at
``base_num_channels`` channels and a 1x1 tanh flow prediction."""
from typing import Optional

import torch
import torch.nn as nn

from .evflownet_incr import ConvLayerIncr, ResidualBlockIncr
from .mask_incr_modules import nnConvIncr, set_precision  # noqa: F401  (nnConvIncr is imported by the reference too)


class FireFlowNetIncr(nn.Module):
    def __init__(self, unet_kwargs, num_bins, compat: Optional[str] = None, precision: Optional[str] = "split"):
        super().__init__()
        base_num_channels = unet_kwargs["base_num_channels"]
        kernel_size = unet_kwargs["kernel_size"]
        self.mask = unet_kwargs["mask_output"]
        self.compat = compat
        padding = kernel_size // 2
        self.E1 = ConvLayerIncr(num_bins, base_num_channels, kernel_size, padding=padding)
        self.E2 = ConvLayerIncr(base_num_channels, base_num_channels, kernel_size, padding=padding)
        self.R1 = ResidualBlockIncr(base_num_channels, base_num_channels)
        self.E3 = ConvLayerIncr(base_num_channels, base_num_channels, kernel_size, padding=padding)
        self.R2 = ResidualBlockIncr(base_num_channels, base_num_channels)
        self.pred = ConvLayerIncr(base_num_channels, out_channels=2, kernel_size=1, activation="tanh")
        # Eight un-normalised ReLU layers fed by raw event counts, nothing recurrent to damp an error: with plain TF32
        # inputs (2^-11 relative, truncated or rounded alike) the output is 1e-3 of its range off after one step and
        # over 2e-3 within 16.  The tensor-core layers therefore run in split precision unless asked otherwise.
        set_precision(self, precision)

    def _sync_compat(self):
        if self.compat is not None:
            self.R1.compat = self.R2.compat = self.compat

    def forward_refresh_reservoirs(self, x):
        """x: N x num_bins x H x W dense input.  Returns {"flow": [N x 2 x H x W]}."""
        self._sync_compat()
        x = self.E1.forward_refresh_reservoirs(x)
        x = self.E2.forward_refresh_reservoirs(x)
        x, _ = self.R1.forward_refresh_reservoirs(x)
        x = self.E3.forward_refresh_reservoirs(x)
        x, _ = self.R2.forward_refresh_reservoirs(x)
        flow = self.pred.forward_refresh_reservoirs(x)
        return {"flow": [flow]}

    def forward(self, x_incr):
        """x_incr: [delta, mask].  Returns {"flow": [[delta_flow, mask]]}."""
        self._sync_compat()
        x_incr = self.E1(x_incr)
        x_incr = self.E2(x_incr)
        x_incr, _ = self.R1(x_incr)
        x_incr = self.E3(x_incr)
        x_incr, _ = self.R2(x_incr)
        flow = self.pred(x_incr)
        return {"flow": [flow]}
