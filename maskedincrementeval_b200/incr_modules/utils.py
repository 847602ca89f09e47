"""Helpers next to the hot path (reference: ``incr_modules/utils.py:1-25``)."""
import torch
import torch.nn.functional as F

from ..fields import TileMask

total_ops = 0


def field_channel_sparsity(x: torch.Tensor, field_size: int, threshold: float = 0.000001):
    """Fraction of field_size x field_size fields whose max |x| <= threshold
    (reference: ``metrics/structural_sparsity.py:8-14``)."""
    mask = F.max_pool2d(torch.abs(x), field_size, stride=(1, 1), padding=((field_size - 1) // 2)).le(threshold).int()
    return mask.sum() / mask.numel()


def print_sparsity(x, prefix: str = ""):
    """Prints the 3x3-field sparsity of a Masked value.  The reference's version raises on a list
    (``incr_modules/utils.py:10``); this one accepts what the networks hand it."""
    d = x[0] if isinstance(x, (list, tuple)) else x
    print(prefix, float(torch.linalg.norm(d) / torch.numel(d)))
    print(prefix, float(field_channel_sparsity(d, field_size=3, threshold=0.1)))


def count_ops(x, ksize):
    global total_ops
    total_ops += int(x[0].count_nonzero()) * ksize
    return total_ops


def compute_mask(x: torch.Tensor, field_size=5, threshold=0.0001):
    """True where the field_size neighbourhood is INACTIVE (reference: ``incr_modules/utils.py:22-25``)."""
    return F.max_pool2d(torch.abs(x), field_size, stride=(1, 1), padding=((field_size - 1) // 2)).le(threshold)


def activity(x) -> dict:
    """Active pixel and tile fractions of a Masked value whose mask is a TileMask.  Synchronises."""
    m = x[1]
    if not isinstance(m, TileMask):
        raise RuntimeError("activity() needs a TileMask")
    px = m.active_pixels()
    tl = int((m.bits != 0).sum().item())
    return {"pixels": px / (m.n * m.h * m.w), "tiles": tl / m.bits.numel()}
