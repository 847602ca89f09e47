"""Incremental FireFlowNet (reference: ``incr_modules/fireflownet_incr.py:1-74``): E1, E2, R1, E3, R2 at
``base_num_channels`` channels and a 1x1 tanh flow prediction; and its recurrent variant, in which the two plain
convolutions E2 and E3 are ConvGRU layers (``RecurrentFireFlowNetIncr``; the reference ships the ConvGRU,
``incr_modules/evflownet_incr.py:18-94``, but no network file that places it in FireFlowNet)."""
from typing import Optional

import torch
import torch.nn as nn

from ._algebra import INCR, run_dense
from .evflownet_incr import ConvGRUIncr, ConvLayerIncr, ResidualBlockIncr
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

    def _run(self, ops, x):
        self._sync_compat()
        x = self.E2._run(ops, self.E1._run(ops, x))
        x, _ = self.R1._run(ops, x)
        x = self.E3._run(ops, x)
        x, _ = self.R2._run(ops, x)
        return {"flow": [self.pred._run(ops, x)]}

    def forward_refresh_reservoirs(self, x):
        """x: N x num_bins x H x W dense input.  Returns {"flow": [N x 2 x H x W]}."""
        return run_dense(self, x)

    def forward(self, x_incr):
        """x_incr: [delta, mask].  Returns {"flow": [[delta_flow, mask]]}."""
        return self._run(INCR, x_incr)


class RecurrentFireFlowNetIncr(nn.Module):
    """FireFlowNet with two ConvGRU-style recurrent layers: E1, G1, R1, G2, R2 and the 1x1 tanh prediction, all 3x3
    convolutions at ``base_num_channels`` channels and stride 1.  An incremental step runs nine of them: E1, the update
    and output gates of each ConvGRU (the reset gate only takes part in the dense pass, as in the reference's ConvGRU,
    ``evflownet_incr.py:58-61``) and two per residual block.  Same constructor arguments, return convention and
    ``compat`` switch as ``FireFlowNetIncr``; ``state_dict`` keys ``G1.*`` / ``G2.*`` take the place of ``E2.*`` / ``E3.*``.

    The recurrent state follows the protocol of the reference's recurrent flow network (``evflownet_incr.py:449-480``):
    the dense pass carries its state from call to call until ``reset_states()``, the incremental pass starts every
    call from a zero state delta."""

    def __init__(self, unet_kwargs, num_bins, compat: Optional[str] = None, precision: Optional[str] = "split"):
        super().__init__()
        c = unet_kwargs["base_num_channels"]
        k = unet_kwargs["kernel_size"]
        self.mask = unet_kwargs["mask_output"]
        self.compat = compat
        self.E1 = ConvLayerIncr(num_bins, c, k, padding=k // 2)
        self.G1 = ConvGRUIncr(c, c, k)
        self.R1 = ResidualBlockIncr(c, c)
        self.G2 = ConvGRUIncr(c, c, k)
        self.R2 = ResidualBlockIncr(c, c)
        self.pred = ConvLayerIncr(c, out_channels=2, kernel_size=1, activation="tanh")
        self.num_states = 2
        self.states = [None, None]
        set_precision(self, precision)

    def reset_states(self):
        self.states = [None] * self.num_states

    def _sync_compat(self):
        if self.compat is not None:
            self.R1.compat = self.R2.compat = self.compat

    def _run(self, ops, x):
        self._sync_compat()
        states = [None, None] if ops.incremental else list(self.states)
        x = self.E1._run(ops, x)
        x, states[0] = ops.gru(self.G1, x, states[0])
        x, _ = self.R1._run(ops, x)
        x, states[1] = ops.gru(self.G2, x, states[1])
        x, _ = self.R2._run(ops, x)
        return {"flow": [self.pred._run(ops, x)]}, states

    def forward_refresh_reservoirs(self, x):
        out, self.states = run_dense(self, x)
        return out

    def forward(self, x_incr):
        return self._run(INCR, x_incr)[0]
