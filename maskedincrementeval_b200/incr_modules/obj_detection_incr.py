"""Incremental dense object detector (reference: ``incr_modules/obj_detection_incr.py:5-77``).

Topology: five blocks of [conv3x3 - BN - ReLU] x 2 with 16/32/64/128/256 channels, a 3x3 stride-2 max-pool after the
first four, then conv3x3 stride 2 to 512 channels - BN - ReLU, flatten, FC 1024 - ReLU - FC to a 5x7 (or 6x8) grid of
``nr_classes + 5 * nr_box`` values.  Parameter names follow the reference so that its checkpoints load.

Everything is assembled from the operator classes of ``mask_incr_modules``: convolutions and activations run on the
library's kernels, batch-norm, max-pool and the linear layers are that module's tensor-op classes.
"""
import torch
import torch.nn as nn

from .mask_incr_modules import (nnBatchNorm2dIncr, nnConvIncr, nnLinearIncr, nnMaxPool2dIncr, nnReluIncr,
                                nnSequentialIncr)

# (input channels are filled in from the previous row) output channels, max-pool after the block
_BLOCKS = ((16, True), (32, True), (64, True), (128, True), (256, False))


class DenseObjectDetIncr(nn.Module):
    def __init__(self, nr_classes, in_c=2, nr_box=2, small_out_map=True):
        super().__init__()
        self.nr_classes, self.nr_box, self.kernel_size = nr_classes, nr_box, 3
        stack, c_prev = [], in_c
        for c_out, pool in _BLOCKS:
            stack.append(self.conv_block(c_prev, c_out, max_pool=pool))
            c_prev = c_out
        stack += [nnConvIncr(in_channels=c_prev, out_channels=512, kernel_size=self.kernel_size, stride=2, bias=False),
                  nnBatchNorm2dIncr(512), nnReluIncr()]
        self.conv_layers = nnSequentialIncr(*stack)
        self.relu1 = nnReluIncr()
        self.cnn_spatial_output_size = [5, 7] if small_out_map else [6, 8]
        cells = self.cnn_spatial_output_size[0] * self.cnn_spatial_output_size[1]
        self.linear_input_features = cells * 512
        self.linear_1 = nnLinearIncr(self.linear_input_features, 1024)
        self.linear_2 = nnLinearIncr(1024, cells * self._per_cell())

    def _per_cell(self) -> int:
        return self.nr_classes + 5 * self.nr_box

    def conv_block(self, in_c, out_c, max_pool=True):
        def unit(ci):
            return [nnConvIncr(ci, out_c, kernel_size=self.kernel_size, padding=(1, 1), bias=False),
                    nnBatchNorm2dIncr(out_c), nnReluIncr()]
        tail = [nnMaxPool2dIncr(kernel_size=self.kernel_size, stride=2)] if max_pool else []
        return nnSequentialIncr(*(unit(in_c) + unit(out_c) + tail))

    def _grid(self, flat: torch.Tensor) -> torch.Tensor:
        return flat.view([-1] + self.cnn_spatial_output_size + [self._per_cell()])

    def forward(self, x_incr):
        feat = self.conv_layers(x_incr)
        head = self.linear_2(self.relu1(self.linear_1([torch.flatten(feat[0], 1), None])))
        return self._grid(head[0]), head[1]

    def forward_refresh_reservoirs(self, x):
        flat = torch.flatten(self.conv_layers.forward_refresh_reservoirs(x), 1)
        hidden = self.relu1.forward_refresh_reservoirs(self.linear_1.forward_refresh_reservoirs(flat))
        return self._grid(self.linear_2.forward_refresh_reservoirs(hidden))
