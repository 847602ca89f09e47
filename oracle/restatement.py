"""CPU restatement of the reference's masked incremental path.  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline / ``--impl reference``
legs may import this file; the product package never does.

Pinning status
--------------
* Operator arithmetic (incremental activation, product, delta convolution, quantiser, BN-on-delta,
  bilinear upsample, max-pool) and the three networks as written at the reference's HEAD
  (``compat="reference"``) are pinned: ``tests/golden/*.npz`` were produced by running the reference's
  own modules (``tests/golden/make_golden.py``) and ``tests/test_oracle.py`` checks this file against
  them, and against the live reference when a checkout is present.
* Pixel masks, tile lists and the dilated output-tile sets are **parity unpinned**: the reference
  returns ``None`` for every mask (``incr_modules/mask_incr_modules.py:178``) and its only mask
  expression next to the path is ``compute_mask`` (``incr_modules/utils.py:22-25``).  The
  definitions below are this library's own and are what the CUDA kernels must match bit for bit.

Everything is plain ``torch`` on CPU tensors in NCHW, fp32.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

Tensor = torch.Tensor
TILE = 8

_OPS = {"relu": torch.relu, "sigmoid": torch.sigmoid, "tanh": torch.tanh, "none": lambda x: x}


# ------------------------------------------------------------------------------------------
# masks and tile lists  (this library's definitions; parity unpinned in the reference)
# ------------------------------------------------------------------------------------------
def pixel_mask(delta: Tensor, thr: float = 0.0) -> Tensor:
    """m[n,0,h,w] = any_c(|delta[n,c,h,w]| > thr), strict.  uint8.

    Modelled on the reference's ``compute_mask`` (``incr_modules/utils.py:22-25``) with a 1x1 field and
    the opposite polarity (True = active)."""
    return (delta.abs() > thr).any(dim=1, keepdim=True).to(torch.uint8)


def tile_bits(mask: Tensor) -> Tensor:
    """[N, TH, TW] int64: bit (py*8+px) of word (n,ty,tx) is the mask at pixel (ty*8+py, tx*8+px)."""
    n, _, h, w = mask.shape
    th, tw = -(-h // TILE), -(-w // TILE)
    m = F.pad(mask.to(torch.uint8), (0, tw * TILE - w, 0, th * TILE - h))
    m = m.view(n, th, TILE, tw, TILE).permute(0, 1, 3, 2, 4).reshape(n, th, tw, 64).numpy().astype(np.uint64)
    words = (m << np.arange(64, dtype=np.uint64)).sum(-1, dtype=np.uint64)
    return torch.from_numpy(words.view(np.int64).copy())


def tile_list(mask: Tensor) -> Tensor:
    """Ascending linear indices (n*TH + ty)*TW + tx of 8x8 tiles holding any active pixel.  int32."""
    t = F.max_pool2d(mask.float(), TILE, TILE, ceil_mode=True)
    return t.flatten().nonzero().flatten().to(torch.int32)


def conv_out_mask(mask: Tensor, k: int, stride: int, pad: int) -> Tensor:
    """Pixel mask of a k x k / stride / pad convolution's output: active where the receptive field
    holds an active input pixel."""
    return (F.max_pool2d(mask.float(), k, stride, pad) > 0).to(torch.uint8)


def bilinear_up2_mask(mask: Tensor) -> Tensor:
    """Pixel mask after a x2 bilinear (align_corners=False) upsample: an output pixel is active when
    one of the (up to four) source pixels it blends is."""
    up = F.interpolate(mask.float(), scale_factor=2, mode="bilinear", align_corners=False)
    return (up > 0).to(torch.uint8)


# ------------------------------------------------------------------------------------------
# operator arithmetic  (pinned against the reference)
# ------------------------------------------------------------------------------------------
def act_incr(res: Tensor, dx: Tensor, op: str) -> Tuple[Tensor, Tensor]:
    """Incremental point nonlinearity: dy = f(res + dx) - f(res); res' = res + dx.
    ``NonlinearPointOpIncr._nonlin`` + ``nnReservedActivation.forward``
    (``incr_modules/mask_incr_modules.py:101-103``, ``:248-251``)."""
    f = _OPS[op]
    dy = f(res + dx) - f(res)
    return dy, res + dx


THRESHOLD_GROUP = 16   # channels per send decision of a thresholded layer (MIE_THR_GROUP in include/mie.h)


def act_incr_thresholded(res: Tensor, emitted: Tensor, dx: Tensor, op: str, thr: float, touched: Tensor = None
                         ) -> Tuple[Tensor, Tensor, Tensor, Tensor]:
    """Thresholded incremental nonlinearity with residual carry (this library's extension; at
    thr = 0 it equals ``act_incr``).

    ``emitted`` is the sum of all output deltas sent downstream so far.  dy = f(res+dx) - emitted.  The decision unit
    is a pixel's group of ``THRESHOLD_GROUP`` consecutive channels: a group is sent when one of its channels has
    |dy| > thr, otherwise its dy is withheld (zero) and stays in the carry; a pixel is active when one of its groups is
    sent.  Only pixels whose input changed (``touched``, default: any channel of dx non-zero) are evaluated.
    Returns dy, pixel mask, res', emitted'."""
    f = _OPS[op]
    new = res + dx
    dy = f(new) - emitted
    if touched is None:
        touched = (dx != 0).any(dim=1, keepdim=True)
    n, c, h, w = dy.shape
    pad = (-c) % THRESHOLD_GROUP
    over = torch.nn.functional.pad(dy.abs() > thr, (0, 0, 0, 0, 0, pad))
    group_send = over.view(n, -1, THRESHOLD_GROUP, h, w).any(dim=2, keepdim=True)          # [n, groups, 1, h, w]
    send = group_send.expand(-1, -1, THRESHOLD_GROUP, -1, -1).reshape(n, c + pad, h, w)[:, :c] & touched
    dy = torch.where(send, dy, torch.zeros_like(dy))
    return dy, send.any(dim=1, keepdim=True).to(torch.uint8), new, emitted + dy


def mul_incr(x1: Tensor, dx1: Tensor, x2: Tensor, dx2: Tensor) -> Tuple[Tensor, Tensor, Tensor]:
    """d(x1*x2) = (dx2 + x2)*dx1 + x1*dx2, then both operands are accumulated.
    ``IncrPointwiseMultiply`` (``incr_modules/mask_incr_functional.py:52-54``) +
    ``nnReservedMultiplication.forward`` (``incr_modules/mask_incr_modules.py:71-75``)."""
    d = (dx2 + x2) * dx1 + x1 * dx2
    return d, x1 + dx1, x2 + dx2


def conv_delta(dx: Tensor, weight: Tensor, stride: int, pad: int) -> Tensor:
    """Convolution of a delta: no bias.  ``nnConvIncr.forward`` (``incr_modules/mask_incr_modules.py:175-178``)."""
    return F.conv2d(dx, weight, None, stride, pad)


# -- what the tensor-core path computes (this library's definition; the reference has no such path) -----------
def tf32_truncate(x: Tensor) -> Tensor:
    """fp32 -> TF32 by dropping the 13 low mantissa bits: what tcgen05.mma kind::tf32 does to an fp32 operand."""
    return (x.contiguous().view(torch.int32) & ~0x1FFF).view(torch.float32)


def tf32_round(x: Tensor) -> Tensor:
    """fp32 -> TF32, round to nearest (ties away from zero): how the library pre-rounds the filter."""
    return ((x.contiguous().view(torch.int32) + 0x1000) & ~0x1FFF).view(torch.float32)


def tc_eligible(cin: int, cout: int, k: int, stride: int, h: int, w: int) -> bool:
    """Host-side rule that sends a convolution to the tensor cores (given 16-byte aligned channel strides)."""
    halo_shape = stride == 1 and k in (3, 5, 7)     # the halo-resident kernel also takes channel counts off 4
    return (cin * k * k >= 256 and (cin % 4 == 0 or halo_shape) and cout % 4 == 0
            and stride in (1, 2) and (stride == 1 or (h % 2 == 0 and w % 2 == 0)))


def conv_delta_tf32(dx: Tensor, weight: Tensor, stride: int, pad: int) -> Tensor:
    """Tensor-core convolution of a delta: TF32-truncated inputs x TF32-rounded filter, fp32 accumulation.
    Truncating the inputs is not linear (trunc(a) + trunc(b) != trunc(a + b)), so on this path the accumulated
    incremental output of a network differs from a dense pass by the rounding of every step's deltas."""
    return F.conv2d(tf32_truncate(dx), tf32_round(weight), None, stride, pad)


def conv_dense(x: Tensor, weight: Tensor, bias: Optional[Tensor], stride: int, pad: int) -> Tensor:
    """Dense refresh convolution with bias.  ``nnConvIncr.forward_refresh_reservoirs`` (``:182-196``)."""
    return F.conv2d(x, weight, bias, stride, pad)


def up2(x: Tensor) -> Tensor:
    """x2 bilinear, align_corners=False.  ``interpolate_from_module`` (``incr_modules/mask_incr_functional.py:76-78``)."""
    return F.interpolate(x, scale_factor=2, mode="bilinear", align_corners=False)


def kfenced(carry: Tensor, dx: Tensor, k: float) -> Tuple[Tensor, Tensor]:
    """Sigma-delta quantiser: T = carry + dx; q = k*floor(0.5 + T/k); carry' = T - q.
    ``KFencedMaskModule.forward`` (``incr_modules/mask_incr_modules.py:31-41``)."""
    t = carry + dx
    q = k * torch.floor(0.5 + t / k)
    return q, t - q


def bn_delta(dx: Tensor, running_var: Tensor, weight: Tensor, eps: float) -> Tensor:
    """Eval batch-norm of a delta: mean forced to 0, bias omitted -> dx * gamma / sqrt(var + eps).
    ``bn2d_from_module`` (``incr_modules/mask_incr_functional.py:69-73``)."""
    return F.batch_norm(dx, torch.zeros_like(running_var), running_var, weight, None, False, 0.1, eps)


def maxpool_incr(res: Tensor, dx: Tensor, k: int, stride: int, pad: int) -> Tuple[Tensor, Tensor]:
    """``nnMaxPool2dIncr.forward`` (``incr_modules/mask_incr_modules.py:217-220``)."""
    out = F.max_pool2d(res + dx, k, stride, pad) - F.max_pool2d(res, k, stride, pad)
    return out, res + dx


class ConvLSTMOracle:
    """``ConvLSTMIncr`` (``incr_modules/e2depth_incr.py:55-166``): one 3x3 convolution producing the four
    gate pre-activations, five incremental nonlinearities and three incremental products.

    At HEAD ``m1(...) + m2(...)`` concatenates two lists (``:113``), so the cell delta that reaches
    ``tanh2`` is m1's alone; ``compat="exact"`` adds the two deltas."""

    def __init__(self, weight: Tensor, bias: Optional[Tensor], compat: str = "reference"):
        self.w, self.b, self.compat = weight, bias, compat
        self.res: Dict[str, Tensor] = {}

    def _act_d(self, x, key, op):
        self.res[key] = x.clone()
        return _OPS[op](x)

    def _act_i(self, dx, key, op):
        dy, self.res[key] = act_incr(self.res[key], dx, op)
        return dy

    def _mul_d(self, a, b, key):
        self.res[key + ".x1"], self.res[key + ".x2"] = a.clone(), b.clone()
        return a * b

    def _mul_i(self, da, db, key):
        d, self.res[key + ".x1"], self.res[key + ".x2"] = mul_incr(self.res[key + ".x1"], da, self.res[key + ".x2"], db)
        return d

    def refresh(self, x: Tensor, state=None):
        if state is None:
            state = (torch.zeros_like(x), torch.zeros_like(x))
        h_prev, c_prev = state
        g = conv_dense(torch.cat((x, h_prev), 1), self.w, self.b, 1, self.w.shape[-1] // 2)
        gi, gf, go, gc = g.chunk(4, 1)
        gi = self._act_d(gi, "sig1", "sigmoid")
        gf = self._act_d(gf, "sig2", "sigmoid")
        go = self._act_d(go, "sig3", "sigmoid")
        gc = self._act_d(gc, "tanh1", "tanh")
        cell = self._mul_d(gi, gc, "m1") + self._mul_d(gf, c_prev, "m2")
        hidden = self._mul_d(go, self._act_d(cell, "tanh2", "tanh"), "m3")
        return hidden, cell

    def step(self, dx: Tensor, state_incr=None):
        if state_incr is None:
            state_incr = (torch.zeros_like(dx), torch.zeros_like(dx))
        dh_prev, dc_prev = state_incr
        g = conv_delta(torch.cat((dx, dh_prev), 1), self.w, 1, self.w.shape[-1] // 2)
        gi, gf, go, gc = g.chunk(4, 1)
        gi = self._act_i(gi, "sig1", "sigmoid")
        gf = self._act_i(gf, "sig2", "sigmoid")
        go = self._act_i(go, "sig3", "sigmoid")
        gc = self._act_i(gc, "tanh1", "tanh")
        m1 = self._mul_i(gi, gc, "m1")
        m2 = self._mul_i(gf, dc_prev, "m2")
        cell = m1 + m2 if self.compat == "exact" else m1
        hidden = self._mul_i(go, self._act_i(cell, "tanh2", "tanh"), "m3")
        return hidden, cell


# ------------------------------------------------------------------------------------------
# E2Depth  (incr_modules/e2depth_incr.py)
# ------------------------------------------------------------------------------------------
class E2DepthOracle:
    """Functional restatement of ``E2VIDRecurrentIncr`` / ``UNetRecurrentIncr``
    (``incr_modules/e2depth_incr.py:382-498``) over a plain state dict.

    ``compat="reference"`` reproduces HEAD as written: skip connections are dropped in the
    incremental pass because two [delta, mask] lists are concatenated with ``+`` (``:333`` used at
    ``:430``, ``:434``) and the LSTM cell delta is the product m1 only (``:113``, ``:116``).
    ``compat="exact"`` sums the tensors instead, which makes the accumulated incremental output equal
    to a dense recompute.
    """

    def __init__(self, sd: Dict[str, Tensor], num_encoders: int = 3, num_residual_blocks: int = 2,
                 compat: str = "reference", prefix: str = "unetrecurrent."):
        assert compat in ("reference", "exact")
        self.sd = {k: v.detach().float().cpu() for k, v in sd.items()}
        self.ne, self.nr, self.compat, self.p = num_encoders, num_residual_blocks, compat, prefix
        self.res: Dict[str, Tensor] = {}
        self.lstm = [ConvLSTMOracle(*self._w(f"encoders.{i}.recurrent_block.Gates"), compat=compat)
                     for i in range(num_encoders)]

    # -- helpers ---------------------------------------------------------------------------
    def _w(self, name: str) -> Tuple[Tensor, Optional[Tensor]]:
        return self.sd[self.p + name + ".weight"], self.sd.get(self.p + name + ".bias")

    def _conv_d(self, x, name, stride, pad):
        w, b = self._w(name)
        return conv_dense(x, w, b, stride, pad)

    def _conv_i(self, dx, name, stride, pad):
        return conv_delta(dx, self._w(name)[0], stride, pad)

    def _act_d(self, x, key, op):
        self.res[key] = x.clone()
        return _OPS[op](x)

    def _act_i(self, dx, key, op):
        dy, self.res[key] = act_incr(self.res[key], dx, op)
        return dy

    def _mul_d(self, a, b, key):
        self.res[key + ".x1"], self.res[key + ".x2"] = a.clone(), b.clone()
        return a * b

    def _mul_i(self, da, db, key):
        d, self.res[key + ".x1"], self.res[key + ".x2"] = mul_incr(self.res[key + ".x1"], da, self.res[key + ".x2"], db)
        return d

    # -- dense refresh (e2depth_incr.py:442-468) ---------------------------------------------
    def refresh(self, x: Tensor, prev_states=None):
        x = self._act_d(self._conv_d(x, "head.conv2d", 1, 2), "head", "relu")
        head = x
        prev_states = prev_states or [None] * self.ne
        blocks, states = [], []
        for i in range(self.ne):
            e = f"encoders.{i}"
            x = self._act_d(self._conv_d(x, e + ".conv.conv2d", 2, 2), e + ".conv", "relu")
            hidden, cell = self.lstm[i].refresh(x, prev_states[i])
            x = hidden
            blocks.append(x)
            states.append((hidden, cell))
        for i in range(self.nr):
            rb = f"resblocks.{i}"
            out = self._act_d(self._conv_d(x, rb + ".conv1", 1, 1), rb + ".relu1", "relu")
            out = self._conv_d(out, rb + ".conv2", 1, 1) + x
            x = self._act_d(out, rb + ".relu2", "relu")
        for i in range(self.ne):
            d = f"decoders.{i}"
            x = x + blocks[self.ne - i - 1]
            x = self._act_d(self._conv_d(up2(x), d + ".conv2d", 1, 2), d, "relu")
        pred = self._conv_d(x + head, "pred.conv2d", 1, 0)
        pred = self._act_d(pred, "final", "sigmoid")
        return pred, states

    # -- incremental step (e2depth_incr.py:402-439) ------------------------------------------
    def step(self, dx: Tensor, prev_states_incr=None):
        exact = self.compat == "exact"
        x = self._act_i(self._conv_i(dx, "head.conv2d", 1, 2), "head", "relu")
        head = x
        prev_states_incr = prev_states_incr or [None] * self.ne
        blocks, states = [], []
        for i in range(self.ne):
            e = f"encoders.{i}"
            x = self._act_i(self._conv_i(x, e + ".conv.conv2d", 2, 2), e + ".conv", "relu")
            hidden, cell = self.lstm[i].step(x, prev_states_incr[i])
            x = hidden
            blocks.append(x)
            states.append((hidden, cell))
        for i in range(self.nr):
            rb = f"resblocks.{i}"
            out = self._act_i(self._conv_i(x, rb + ".conv1", 1, 1), rb + ".relu1", "relu")
            out = self._conv_i(out, rb + ".conv2", 1, 1) + x
            x = self._act_i(out, rb + ".relu2", "relu")
        for i in range(self.ne):
            d = f"decoders.{i}"
            if exact:
                x = x + blocks[self.ne - i - 1]
            x = self._act_i(self._conv_i(up2(x), d + ".conv2d", 1, 2), d, "relu")
        if exact:
            x = x + head
        pred = self._act_i(self._conv_i(x, "pred.conv2d", 1, 0), "final", "sigmoid")
        return pred, states


# ------------------------------------------------------------------------------------------
# flow networks  (incr_modules/evflownet_incr.py, fireflownet_incr.py)
# ------------------------------------------------------------------------------------------
def interp_to(x: Tensor, size) -> Tensor:
    """``F.interpolate(x, size=size, mode="bilinear", align_corners=False)``; linear, so exact on deltas."""
    return F.interpolate(x, size=tuple(size), mode="bilinear", align_corners=False)


def skip_concat(x1: Tensor, x2: Tensor) -> Tensor:
    """``skip_concat`` (``incr_modules/evflownet_incr.py:9-14``): zero-pad x1 to x2's size, concatenate."""
    dy, dxx = x2.shape[2] - x1.shape[2], x2.shape[3] - x1.shape[3]
    x1 = F.pad(x1, (dxx // 2, dxx - dxx // 2, dy // 2, dy - dy // 2))
    return torch.cat([x1, x2], 1)


class _FlowBase:
    def __init__(self, sd: Dict[str, Tensor], compat: str, tensor_cores: bool = False):
        assert compat in ("reference", "exact")
        self.sd = {k: v.detach().float().cpu() for k, v in sd.items()}
        self.compat = compat
        self.tensor_cores = tensor_cores   # emulate the TF32 path on the layers the library would send there
        self.res: Dict[str, Tensor] = {}

    def _conv_d(self, x, name, stride, pad):
        return conv_dense(x, self.sd[name + ".weight"], self.sd.get(name + ".bias"), stride, pad)

    def _conv_i(self, dx, name, stride, pad):
        w = self.sd[name + ".weight"]
        if self.tensor_cores and tc_eligible(dx.shape[1], w.shape[0], w.shape[2], stride, dx.shape[2], dx.shape[3]):
            return conv_delta_tf32(dx, w, stride, pad)
        return conv_delta(dx, w, stride, pad)

    def _act_d(self, x, key, op):
        self.res[key] = x.clone()
        return _OPS[op](x)

    def _act_i(self, dx, key, op):
        dy, self.res[key] = act_incr(self.res[key], dx, op)
        return dy

    # ConvLayerIncr (evflownet_incr.py:97-153)
    def _layer_d(self, x, name, stride, pad, op):
        y = self._conv_d(x, name + ".conv2d", stride, pad)
        return self._act_d(y, name, op) if op else y

    def _layer_i(self, dx, name, stride, pad, op):
        y = self._conv_i(dx, name + ".conv2d", stride, pad)
        return self._act_i(y, name, op) if op else y

    # ResidualBlockIncr (evflownet_incr.py:195-292).  At HEAD one activation module (one reservoir)
    # serves both activations and the residual add is lost in the incremental pass.
    def _resblock_d(self, x, name):
        k1 = name + ".act" if self.compat == "reference" else name + ".act1"
        k2 = name + ".act" if self.compat == "reference" else name + ".act2"
        out1 = self._act_d(self._conv_d(x, name + ".conv1", 1, 1), k1, "relu")
        out2 = self._conv_d(out1, name + ".conv2", 1, 1) + x
        return self._act_d(out2, k2, "relu")

    def _resblock_i(self, dx, name):
        ref = self.compat == "reference"
        k1 = name + ".act" if ref else name + ".act1"
        k2 = name + ".act" if ref else name + ".act2"
        out1 = self._act_i(self._conv_i(dx, name + ".conv1", 1, 1), k1, "relu")
        out2 = self._conv_i(out1, name + ".conv2", 1, 1)
        if not ref:
            out2 = out2 + dx
        return self._act_i(out2, k2, "relu")


class FireFlowNetOracle(_FlowBase):
    """``FireFlowNetIncr`` (``incr_modules/fireflownet_incr.py:6-72``)."""

    def __init__(self, sd, kernel_size: int = 3, compat: str = "reference", tensor_cores: bool = False):
        super().__init__(sd, compat, tensor_cores)
        self.k = kernel_size

    def refresh(self, x):
        p = self.k // 2
        x = self._layer_d(x, "E1", 1, p, "relu")
        x = self._layer_d(x, "E2", 1, p, "relu")
        x = self._resblock_d(x, "R1")
        x = self._layer_d(x, "E3", 1, p, "relu")
        x = self._resblock_d(x, "R2")
        return self._layer_d(x, "pred", 1, 0, "tanh")

    def step(self, dx):
        p = self.k // 2
        x = self._layer_i(dx, "E1", 1, p, "relu")
        x = self._layer_i(x, "E2", 1, p, "relu")
        x = self._resblock_i(x, "R1")
        x = self._layer_i(x, "E3", 1, p, "relu")
        x = self._resblock_i(x, "R2")
        return self._layer_i(x, "pred", 1, 0, "tanh")


class EVFlowNetOracle(_FlowBase):
    """``MultiResUNetRecurrentIncr`` (``incr_modules/evflownet_incr.py:347-495``): 4 recurrent encoders
    (conv3x3 s2 + ConvGRU), 2 residual blocks, 4 decoders with concatenated skips and multi-resolution
    tanh predictions."""

    def __init__(self, sd, compat: str = "reference", num_encoders: int = 4, num_residual_blocks: int = 2):
        super().__init__(sd, compat)
        self.ne, self.nr = num_encoders, num_residual_blocks
        self.states: List[Optional[Tensor]] = [None] * self.ne

    def reset_states(self):
        self.states = [None] * self.ne

    # ConvGRUIncr (evflownet_incr.py:18-94)
    def _gru_d(self, x, prev, name):
        if prev is None:
            prev = torch.zeros_like(x)
        st = torch.cat([x, prev], 1)
        update = self._act_d(self._conv_d(st, name + ".update_gate", 1, 1), name + ".sig1", "sigmoid")
        reset = self._act_d(self._conv_d(st, name + ".reset_gate", 1, 1), name + ".sig2", "sigmoid")
        out = self._act_d(self._conv_d(torch.cat([x, prev * reset], 1), name + ".out_gate", 1, 1), name + ".tanh", "tanh")
        a = out - prev
        self.res[name + ".mult.x1"], self.res[name + ".mult.x2"] = a.clone(), update.clone()
        return prev + a * update

    def _gru_i(self, dx, name):
        prev = torch.zeros_like(dx)  # incremental states are reset on every call (evflownet_incr.py:451)
        st = torch.cat([dx, prev], 1)
        update = self._act_i(self._conv_i(st, name + ".update_gate", 1, 1), name + ".sig1", "sigmoid")
        out = self._act_i(self._conv_i(st, name + ".out_gate", 1, 1), name + ".tanh", "tanh")
        d, self.res[name + ".mult.x1"], self.res[name + ".mult.x2"] = mul_incr(
            self.res[name + ".mult.x1"], out - prev, self.res[name + ".mult.x2"], update)
        return prev + d

    def refresh(self, x):
        blocks = []
        for i in range(self.ne):
            e = f"encoders.{i}"
            x = self._layer_d(x, e + ".conv", 2, 1, "relu")
            x = self._gru_d(x, self.states[i], e + ".recurrent_block")
            self.states[i] = x
            blocks.append(x)
        for i in range(self.nr):
            x = self._resblock_d(x, f"resblocks.{i}")
        preds = []
        for i in range(self.ne):
            x = skip_concat(x, blocks[self.ne - i - 1])
            if i > 0:
                x = skip_concat(preds[-1], x)
            x = self._act_d(self._conv_d(up2(x), f"decoders.{i}.conv2d", 1, 1), f"decoders.{i}", "relu")
            preds.append(self._layer_d(x, f"preds.{i}", 1, 0, "tanh"))
        return preds

    def step(self, dx):
        x = dx
        blocks = []
        for i in range(self.ne):
            e = f"encoders.{i}"
            x = self._layer_i(x, e + ".conv", 2, 1, "relu")
            x = self._gru_i(x, e + ".recurrent_block")
            blocks.append(x)
        for i in range(self.nr):
            x = self._resblock_i(x, f"resblocks.{i}")
        preds = []
        for i in range(self.ne):
            x = skip_concat(x, blocks[self.ne - i - 1])
            if i > 0:
                x = skip_concat(preds[-1], x)
            x = self._act_i(self._conv_i(up2(x), f"decoders.{i}.conv2d", 1, 1), f"decoders.{i}", "relu")
            preds.append(self._layer_i(x, f"preds.{i}", 1, 0, "tanh"))
        return preds


class DelayedEVFlowNetOracle(_FlowBase):
    """``DelayedMultiResUNetIncr`` (``incr_modules/delayedevflownet_incr.py:155-383``): feed-forward multi-resolution
    UNet -- stride-2 encoders, residual blocks, one decoder per level fed by the encoder output of that level (the
    lowest one by concat(resblock output, encoder output)), tanh predictions per level; decoder outputs (all but the
    lowest) and predictions are interpolated to the input resolution, concatenated and reduced by two 1x1 layers
    ("delayed" prediction).  Returns the interpolated predictions followed by the delayed prediction."""

    def __init__(self, sd, compat: str = "reference", num_encoders: int = 4, num_residual_blocks: int = 2,
                 kernel_size: int = 3):
        super().__init__(sd, compat)
        self.ne, self.nr, self.k = num_encoders, num_residual_blocks, kernel_size

    def _run(self, x, dense: bool):
        layer = self._layer_d if dense else self._layer_i
        conv = self._conv_d if dense else self._conv_i
        act = self._act_d if dense else self._act_i
        res = self._resblock_d if dense else self._resblock_i
        size = x.shape[-2:]
        pad = self.k // 2
        blocks = []
        for i in range(self.ne):
            x = layer(x, f"encoders.{i}", 2, pad, "relu")
            blocks.append(x)
        for i in range(self.nr):
            x = res(x, f"resblocks.{i}")
        outs, preds = [], []
        for i in range(self.ne):
            b = blocks[self.ne - i - 1]
            d_in = skip_concat(x, b) if i == 0 else b
            d = act(conv(up2(d_in), f"decoders.{i}.conv2d", 1, pad), f"decoders.{i}", "relu")
            if i != 0:
                outs.append(interp_to(d, size))
            preds.append(interp_to(layer(d, f"preds.{i}", 1, 0, "tanh"), size))
        din = torch.cat(outs + preds, 1)
        mid = layer(din, "delayed_pred_layer_list.0", 1, 0, "relu")
        last = layer(torch.cat([mid, din[:, -2 * self.ne:]], 1), "delayed_pred_layer_list.1", 1, 0, "tanh")
        return preds + [last]

    def refresh(self, x):
        return self._run(x, True)

    def step(self, dx):
        return self._run(dx, False)


class _BNNet:
    """Shared pieces of the two batch-normalised networks: bias-free convolutions, eval batch-norm (dense: the full
    affine map; on a delta: the scale only, ``bn2d_from_module``), ReLU and max-pool reservoirs."""

    def __init__(self, sd: Dict[str, Tensor]):
        self.sd = {k: v.detach().cpu() for k, v in sd.items()}
        self.res: Dict[str, Tensor] = {}

    def _conv(self, x, name, stride, pad, dense):
        w = self.sd[name + ".weight"].float()
        return conv_dense(x, w, None, stride, pad) if dense else conv_delta(x, w, stride, pad)

    def _bn(self, x, name, dense, eps=1e-5):
        var, w = self.sd[name + ".running_var"].float(), self.sd[name + ".weight"].float()
        if dense:
            return F.batch_norm(x, self.sd[name + ".running_mean"].float(), var, w, self.sd[name + ".bias"].float(),
                                False, 0.1, eps)
        return bn_delta(x, var, w, eps)

    def _relu(self, x, key, dense):
        if dense:
            self.res[key] = x.clone()
            return torch.relu(x)
        dy, self.res[key] = act_incr(self.res[key], x, "relu")
        return dy

    def _pool(self, x, key, k, stride, pad, dense):
        if dense:
            self.res[key] = x.clone()
            return F.max_pool2d(x, k, stride, pad)
        dy, self.res[key] = maxpool_incr(self.res[key], x, k, stride, pad)
        return dy

    def _fc(self, x, name, dense):
        return F.linear(x, self.sd[name + ".weight"].float(), self.sd[name + ".bias"].float() if dense else None)


class DenseObjectDetOracle(_BNNet):
    """``DenseObjectDetIncr`` (``incr_modules/obj_detection_incr.py:5-77``)."""

    def __init__(self, sd, nr_classes: int, nr_box: int = 2, small_out_map: bool = True):
        super().__init__(sd)
        self.grid = [5, 7] if small_out_map else [6, 8]
        self.per_cell = nr_classes + 5 * nr_box

    def _run(self, x, dense):
        for b in range(5):
            p = f"conv_layers.{b}"
            for j in (0, 3):
                x = self._conv(x, f"{p}.{j}", 1, 1, dense)
                x = self._bn(x, f"{p}.{j + 1}", dense)
                x = self._relu(x, f"{p}.{j + 2}", dense)
            if b < 4:
                x = self._pool(x, f"{p}.6", 3, 2, 0, dense)
        x = self._relu(self._bn(self._conv(x, "conv_layers.5", 2, 0, dense), "conv_layers.6", dense), "conv_layers.7", dense)
        x = self._relu(self._fc(torch.flatten(x, 1), "linear_1", dense), "relu1", dense)
        return self._fc(x, "linear_2", dense).view([-1] + self.grid + [self.per_cell])

    def refresh(self, x):
        return self._run(x, True)

    def step(self, dx):
        return self._run(dx, False)


class ResnetOracle(_BNNet):
    """``ResnetIncr`` / ``BasicBlockIncr`` (``incr_modules/event_representation_incr.py:10-143``): ResNet-34 body."""

    STAGES = ((64, 3, False), (128, 4, True), (256, 6, True), (512, 3, True))

    def _block(self, x, p, down, dense):
        stride = 2 if down else 1
        out = self._relu(self._bn(self._conv(x, p + ".conv1", stride, 1, dense), p + ".bn1", dense), p + ".relu", dense)
        out = self._bn(self._conv(out, p + ".conv2", 1, 1, dense), p + ".bn2", dense)
        if down:
            x = self._bn(self._conv(x, p + ".downsample.0", 2, 0, dense), p + ".downsample.1", dense)
        return self._relu(out + x, p + ".relu2", dense)

    def _run(self, x, dense):
        x = self._relu(self._bn(self._conv(x, "conv1", 2, 3, dense), "bn1", dense), "relu", dense)
        x = self._pool(x, "maxpool", 3, 2, 1, dense)
        for si, (_, n_blocks, down) in enumerate(self.STAGES, 1):
            for bi in range(n_blocks):
                x = self._block(x, f"layer{si}.{bi}", down and bi == 0, dense)
        x = torch.flatten(F.adaptive_avg_pool2d(x, (1, 1)), 1, -1)
        return self._fc(x, "fc", dense)

    def refresh(self, x):
        return self._run(x, True)

    def step(self, dx):
        return self._run(dx, False)
