"""Type aliases of the masked incremental path (reference: ``incr_modules/masked_types.py:1-14``).

A ``Masked`` value is, as in the reference, a 2-item list or tuple ``[delta, mask]``.  ``delta`` is a dense
NCHW-logical, channels-last fp32 CUDA tensor that is exactly zero wherever ``mask`` is clear.  ``mask`` is
``None`` (not known yet), a bool/uint8/int32 tensor, or a ``TileMask`` (one 64-bit word per 8x8 tile).
"""
from typing import Union

import torch

from ..fields import TileMask  # noqa: F401

_device = 'cuda'

Sp = torch.Tensor          # the reference aliases a sparse tensor type here and never uses it
DenseT = torch.Tensor
SpOrDense = Union[Sp, DenseT]
Masked = torch.Tensor      # in practice [delta, mask]; kept as the reference spells it
