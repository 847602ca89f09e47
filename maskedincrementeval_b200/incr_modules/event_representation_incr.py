"""Incremental ResNet-34 classifier body (reference: ``incr_modules/event_representation_incr.py:10-143``).

Stem conv7x7/2 - BN - ReLU - max-pool3x3/2, four stages of basic blocks (3, 4, 6, 3 blocks of 64, 128, 256, 512
channels; the first block of stages 2-4 halves the resolution and has a 1x1/2 projection), global average pool, FC.
The ReLUs difference against reservoirs that the block itself advances after the activation has been evaluated, as
the reference orders it.  Parameter names follow the reference so that its checkpoints load.

The reference's ``ClassifierIncrEval`` additionally owns a learned quantisation layer from the un-vendored
``rpg_event_representation_learning`` project; here it takes the already quantised voxel tensor.
"""
import torch
import torch.nn as nn

from .mask_incr_functional import IncrementReserve
from .mask_incr_modules import (NonlinearPointOpIncr, nnAdaptiveAvgPool2dIncr, nnBatchNorm2dIncr, nnConvIncr,
                                nnLinearIncr, nnMaxPool2dIncr, nnSequentialIncr)


def _bn(c):
    return nnBatchNorm2dIncr(c, eps=1e-5, momentum=0.1, affine=True, track_running_stats=True)


class BasicBlockIncr(nn.Module):
    """conv3x3 - BN - ReLU - conv3x3 - BN, plus identity (or its 1x1/2 projection), ReLU."""

    def __init__(self, sz, downsample=False):
        nn.Module.__init__(self)
        c_in, stride = (sz // 2, 2) if downsample else (sz, 1)
        self.conv1 = nnConvIncr(c_in, sz, 3, stride=stride, padding=1, bias=False)
        self.bn1 = _bn(sz)
        self.res_in = IncrementReserve()
        self.relu = NonlinearPointOpIncr(self.res_in, op=torch.relu)
        self.conv2 = nnConvIncr(sz, sz, 3, stride=1, padding=1, bias=False)
        self.bn2 = _bn(sz)
        self.downsample = nnSequentialIncr(nnConvIncr(c_in, sz, 1, stride=2, bias=False), _bn(sz)) if downsample else None
        self.res_in2 = IncrementReserve()
        self.relu2 = NonlinearPointOpIncr(self.res_in2, op=torch.relu)

    def forward(self, x_incr):
        pre1 = self.bn1(self.conv1(x_incr))
        branch = self.bn2(self.conv2(self.relu(pre1)))
        shortcut = self.downsample(x_incr) if self.downsample is not None else x_incr
        pre2 = (branch[0] + shortcut[0], None)
        out = self.relu2(pre2)
        # the reservoirs move only now: both activations above differenced against the previous state
        self.res_in.accumulate(pre1)
        self.res_in2.accumulate(pre2)
        return out

    def forward_refresh_reservoirs(self, x):
        pre1 = self.bn1.forward_refresh_reservoirs(self.conv1.forward_refresh_reservoirs(x))
        branch = self.conv2.forward_refresh_reservoirs(self.relu.forward_refresh_reservoirs(pre1))
        branch = self.bn2.forward_refresh_reservoirs(branch)
        shortcut = self.downsample.forward_refresh_reservoirs(x) if self.downsample is not None else x
        pre2 = branch + shortcut
        self.res_in.update_reservoir(pre1)
        self.res_in2.update_reservoir(pre2)
        return self.relu2.forward_refresh_reservoirs(pre2)


def _stage(width, n_blocks, first_downsamples):
    return nnSequentialIncr(*[BasicBlockIncr(width, downsample=(first_downsamples and i == 0)) for i in range(n_blocks)])


class ResnetIncr(nn.Module):
    def __init__(self):
        nn.Module.__init__(self)
        self.conv1 = nnConvIncr(3, 64, 7, 2, 3, bias=False)
        self.bn1 = _bn(64)
        self.in_res = IncrementReserve()
        self.relu = NonlinearPointOpIncr(self.in_res, torch.relu)
        self.maxpool = nnMaxPool2dIncr(kernel_size=3, stride=2, padding=1)
        self.layer1 = _stage(64, 3, False)
        self.layer2 = _stage(128, 4, True)
        self.layer3 = _stage(256, 6, True)
        self.layer4 = _stage(512, 3, True)
        self.avgpool = nnAdaptiveAvgPool2dIncr(output_size=(1, 1))
        self.fc = nnLinearIncr(512, 1000, bias=True)

    def _stages(self):
        return (self.layer1, self.layer2, self.layer3, self.layer4)

    def forward(self, x_incr):
        pre = self.bn1(self.conv1(x_incr))
        out = self.maxpool(self.relu(pre))
        for stage in self._stages():
            out = stage(out)
        pooled = self.avgpool(out)
        logits = self.fc((torch.flatten(pooled[0], 1, -1), None))
        self.in_res.accumulate(pre)
        return logits

    def forward_refresh_reservoirs(self, x):
        pre = self.bn1.forward_refresh_reservoirs(self.conv1.forward_refresh_reservoirs(x))
        out = self.maxpool.forward_refresh_reservoirs(self.relu.forward_refresh_reservoirs(pre))
        for stage in self._stages():
            out = stage.forward_refresh_reservoirs(out)
        out = torch.flatten(self.avgpool.forward_refresh_reservoirs(out), 1, -1)
        self.in_res.update_reservoir(pre)
        return self.fc.forward_refresh_reservoirs(out)


class ClassifierIncrEval(nn.Module):
    """``ResnetIncr`` with its first convolution and last layer resized for ``2 * voxel_dimension[0]`` input channels and
    ``num_classes`` outputs (reference ``:146-190``, without the quantisation layer)."""

    def __init__(self, voxel_dimension=(9, 180, 240), crop_dimension=(224, 224), num_classes=101):
        nn.Module.__init__(self)
        self.crop_dimension = crop_dimension
        self.classifier = ResnetIncr()
        self.classifier.conv1 = nnConvIncr(2 * voxel_dimension[0], 64, kernel_size=7, stride=2, padding=3, bias=False)
        self.classifier.fc = nnLinearIncr(self.classifier.fc.in_features, num_classes)

    def forward(self, x_incr):
        return self.classifier(x_incr)

    def forward_refresh_reservoir(self, x):
        return self.classifier.forward_refresh_reservoirs(x)
