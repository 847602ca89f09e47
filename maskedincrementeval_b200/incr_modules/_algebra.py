"""Two interpreters for one network description.

Every network of this package states its topology once, as a ``_run(ops, ...)`` method written against the small
operator vocabulary below, and is evaluated by one of two interpreters:

``DENSE``  values are dense tensors; each operator computes the full result with bias and refills the persistent state
           of the module it is given (the reference's ``forward_refresh_reservoirs`` protocol,
           ``incr_modules/mask_incr_modules.py:182-196, 253-256, 77-81``);
``INCR``   values are ``[delta, TileMask]`` pairs; each operator is one fused libmie launch over the active tiles
           (the reference's ``forward`` protocol, ``mask_incr_modules.py:164-179, 248-251, 71-75``);
``NATIVE`` the dense pass again, but on this library's kernels: values are ``[dense tensor, full mask]`` pairs, every
           tile is listed, convolutions run in dense-evaluation mode (bias added, state set instead of advanced, full
           fp32).  No cuDNN on the path; a network's refresh then costs a few incremental steps instead of sixty.

The reference writes every network twice (a dense and an incremental method per class, kept consistent by hand, which
is where its skip-connection and residual quirks come from); here the two passes cannot drift apart, and a quirk the
``compat="reference"`` mode must reproduce is an explicit argument of the operator instead of an accident of list
arithmetic.
"""
from typing import Optional

import torch
import torch.nn.functional as F

from .. import _native as nat
from .. import fields as fl
from ..fields import Scratch


def _zero_pad_to(x: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    """Zero-pad ``x`` symmetrically to the spatial size of ``like`` (odd differences go right / bottom)."""
    dy, dx = like.shape[2] - x.shape[2], like.shape[3] - x.shape[3]
    if dy == 0 and dx == 0:
        return x
    return F.pad(x, (dx // 2, dx - dx // 2, dy // 2, dy - dy // 2))


class DenseOps:
    """Dense interpreter: tensors in, tensors out, state refilled."""
    incremental = False     # the pass is an incremental step
    pairs = False           # values are [tensor, mask] pairs

    def lift(self, x):
        return x

    def lower(self, v):
        return v

    def lstm(self, cell, x, prev_state):
        return cell.forward_refresh_reservoirs(x, prev_state)

    def gru(self, cell, x, prev_state):
        return cell.forward_refresh_reservoirs(x, prev_state)

    def conv(self, conv, x, act=None, addend=None, norm=None, cin_limit: Optional[int] = None, second=None):
        y = conv.forward_refresh_reservoirs(x if second is None else x + second)
        if norm is not None:
            y = norm.forward_refresh_reservoirs(y)
        if addend is not None:
            y = y + addend
        return y if act is None else act.forward_refresh_reservoirs(y)

    def act(self, act, x):
        return act.forward_refresh_reservoirs(x)

    def mul(self, mult, a, b):
        return mult.forward_refresh_reservoirs(a, b)

    def add(self, a, b, scratch: Scratch = None, key: str = ""):
        return a + b

    def cat(self, a, b, scratch: Scratch = None, key: str = ""):
        return torch.cat([_zero_pad_to(a, b), b], dim=1)

    def upsample2x(self, x, skip=None, scratch: Scratch = None, pad4: bool = False):
        if skip is not None:
            x = x + skip
        return F.interpolate(x, scale_factor=2, mode="bilinear", align_corners=False)


class IncrOps:
    """Incremental interpreter: ``[delta, TileMask]`` pairs in and out, one fused launch per operator."""
    incremental = True
    pairs = True

    def lift(self, x):
        return x

    def lower(self, v):
        return v

    def lstm(self, cell, x, prev_state):
        return cell(x, prev_state)

    def gru(self, cell, x, prev_state):
        return cell(x, prev_state)

    def conv(self, conv, x, act=None, addend=None, norm=None, cin_limit: Optional[int] = None, second=None):
        if second is not None and not (norm is None and addend is None and cin_limit is None and conv.takes_second_input()
                                       and not fl.config.kfenced_step and x[0].shape == second[0].shape):
            x, second = self.add(x, second, conv._scratch, "second.sum"), None      # no fused form: add first
        if norm is not None:      # batch-norm between convolution and activation: not fused
            y = norm(conv.forward_fused(x, None, addend, cin_limit=cin_limit))
            return y if act is None else act(y)
        return conv.forward_fused(x, act, addend, cin_limit=cin_limit, second=second)

    def act(self, act, x):
        return act(x)

    def mul(self, mult, a, b):
        return mult(a, b)

    def add(self, a, b, scratch: Scratch, key: str):
        x, mx = fl.resolve(a, scratch, key + ".a")
        y, my = fl.resolve(b, scratch, key + ".b")
        n, c, h, w = x.shape
        out = scratch.get(key, (n, c, h, w), torch.float32, x.device, channels_last=True)
        bits = scratch.get(key + ".bits", (fl.n_tiles(n, h, w),), torch.int64, x.device)
        return [out, fl.add(x, mx, y, my, out, bits)]

    def cat(self, a, b, scratch: Scratch, key: str):
        x, mx = fl.resolve(a, scratch, key + ".a")
        y, my = fl.resolve(b, scratch, key + ".b")
        if x.shape[2:] != y.shape[2:]:
            raise NotImplementedError("incremental concatenation needs equal spatial sizes (pad the input to a multiple of 16)")
        n, ca, h, w = x.shape
        c = ca + y.shape[1]
        # pixel stride rounded up to 4 floats (the flow decoders see 2*C + 2 channels): 16-byte pixel addresses are what
        # the convolution's vector loads and TMA need; the padding channels are never written and stay zero
        out = scratch.get(key, (n, (c + 3) // 4 * 4, h, w), torch.float32, x.device, channels_last=True)[:, :c]
        bits = scratch.get(key + ".bits", (fl.n_tiles(n, h, w),), torch.int64, x.device)
        return [out, fl.cat2(x, mx, y, my, out, bits)]

    def upsample2x(self, x, skip=None, scratch: Scratch = None, pad4: bool = False):
        d, m = fl.resolve(x, scratch, "in")
        n, c, h, w = d.shape
        s = ms = None
        if skip is not None:
            s, ms = fl.resolve(skip, scratch, "skip")
        cp = (c + 3) // 4 * 4 if pad4 else c
        up = scratch.get("up", (n, cp, 2 * h, 2 * w), torch.float32, d.device, channels_last=True)[:, :c]
        ub = scratch.get("up.bits", (fl.n_tiles(n, 2 * h, 2 * w),), torch.int64, d.device)
        return [up, fl.upsample2x(d, m, s, ms, up, ub, nat.UP_BILINEAR)]


class NativeDenseOps(IncrOps):
    """Dense interpreter on the library's own kernels: the point operators of ``IncrOps`` with every pixel active,
    convolutions in dense-evaluation mode.  Values are ``[dense tensor, full mask]`` pairs; ``lift`` / ``lower`` convert
    at the network's boundary.  The buffers the operators write are the modules' persistent delta buffers, so the caller
    clones what it keeps (``lower``) and zeroes them afterwards (``fields.reset_delta_state``)."""
    incremental = False
    pairs = True

    def lift(self, x):
        if x is None or isinstance(x, (list, tuple)):
            return x
        x = fl.as_channels_last(x)
        n, _, h, w = x.shape
        return [x, fl.full_mask(n, h, w, x.device)]

    def lower(self, v):
        return v[0].clone()

    def conv(self, conv, x, act=None, addend=None, norm=None, cin_limit: Optional[int] = None, second=None):
        if norm is not None:
            raise NotImplementedError("batch-norm layers take the library dense pass (config.refresh = 'library')")
        if second is not None and not (addend is None and cin_limit is None and conv.takes_second_input()
                                       and x[0].shape == second[0].shape):
            x, second = self.add(x, second, conv._scratch, "second.sum"), None
        return conv.forward_fused(x, act, addend, cin_limit=cin_limit, refresh=True, second=second)

    def act(self, act, x):
        return [act.forward_refresh_reservoirs(x[0]), x[1]]

    def mul(self, mult, a, b):
        return [mult.forward_refresh_reservoirs(a[0], b[0]), a[1]]

    def lstm(self, cell, x, prev_state):
        return cell.refresh_native(x, prev_state)

    def gru(self, cell, x, prev_state):
        return cell.refresh_native(x, prev_state)


DENSE, INCR, NATIVE = DenseOps(), IncrOps(), NativeDenseOps()


def dense_ops(module, x) -> DenseOps:
    """The interpreter a network's dense pass uses: the kernels when ``config.refresh == "native"``, the input lives on
    a CUDA device and the network has no normalisation layers; PyTorch's dense operators otherwise."""
    carried = any(s is not None for s in getattr(module, "states", None) or ())   # a ConvGRU state kept from the last call
    if fl.config.refresh == "native" and x.is_cuda and getattr(module, "norm", None) is None and not carried:
        return NATIVE
    if fl.config.refresh not in ("native", "library"):
        raise ValueError("config.refresh must be 'native' or 'library'")
    return DENSE



def run_dense(network, x, *extra):
    """A network's dense pass: ``network._run`` under the interpreter ``dense_ops`` picks; with the native one the
    input is lifted to a pair, every tensor of the result is cloned out of the modules' buffers, and those buffers
    are zeroed for the incremental steps that follow."""
    ops = dense_ops(network, x)
    if ops is not NATIVE:
        return network._run(DENSE, x, *extra)

    def lower(v):
        if isinstance(v, dict):
            return {k: lower(u) for k, u in v.items()}
        if isinstance(v, (list, tuple)) and len(v) == 2 and torch.is_tensor(v[0]) and isinstance(v[1], fl.TileMask):
            return NATIVE.lower(v)
        if isinstance(v, (list, tuple)):
            return type(v)(lower(u) for u in v)
        return v

    out = lower(network._run(NATIVE, NATIVE.lift(x), *extra))
    fl.reset_delta_state(network)
    return out
