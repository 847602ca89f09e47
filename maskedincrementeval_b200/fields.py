"""Delta fields on the device: a channels-last fp32 tensor plus one 64-bit activity word per 8x8 tile.

This is the host-side plumbing between the reference-shaped modules in ``incr_modules`` and the C ABI
of libmie.  A ``Masked`` value in the reference is a 2-item list ``[delta, mask_or_None]``
(``incr_modules/masked_types.py:14``); here the second item is ``None`` (unknown: the mask is derived
from the delta on first use), a bool/uint8/int32 tensor, or a ``TileMask``.
"""
from __future__ import annotations

import ctypes as C
import weakref
from typing import Dict, Optional, Tuple

import torch

from . import _native as nat

TILE = 8


def n_tiles(n: int, h: int, w: int) -> int:
    return n * (-(-h // TILE)) * (-(-w // TILE))


def conv_out_hw(h: int, w: int, k: int, stride: int, pad: int) -> Tuple[int, int]:
    return (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1


class IncrConfig:
    """Library-wide defaults; a module reads them when it runs, so they can be changed between steps.

    threshold        a pixel's group of 16 consecutive output channels is withheld while every |dy| in it is <= threshold
                     (0 = lossless; layers of up to 16 channels decide per pixel)
    carry            keep what was withheld and send it once it grows past the threshold (bounded error)
    input_threshold  threshold used when a mask has to be derived from a bare delta tensor
    tensor_cores     "auto" runs convolutions whose reduction depth Cin*k*k is at least 256 on the tensor cores
                     (TF32 inputs, FP32 accumulation; values then agree with FP32 to about 1e-3 of the range,
                     E2Depth's accumulated output to about 1e-5); "off" keeps every convolution on the FP32 path
    compat           "reference": networks wired as the reference is written; "exact": as intended, which
                     makes the accumulated incremental output equal to a dense recompute
    kfenced_step     None (default): the quantiser every convolution owns stays unused, as in the reference
                     (``mask_incr_modules.py:157`` builds it, ``:166`` has its call commented out).  A positive value
                     switches it on where the reference meant it to sit: each convolution's input delta passes through
                     T = carry + dx; q = k*floor(0.5 + T/k); carry = T - q with this quantisation step k, and the
                     convolution sees q (one more kernel per convolution; what is rounded away stays pending)
    refresh          "native" (default): the networks' dense pass (forward_refresh_reservoirs) runs on this library's
                     FP32 kernels in dense-evaluation mode -- every tile listed, bias added, state set instead of
                     advanced; "library": it runs on PyTorch's dense operators (cuDNN), as the reference's does
    tail_dilation    True: a convolution's tile dilation rides in the tail of the kernel that produces its input mask
                     (one launch less per convolution; measured slower than the separate launch when launches overlap
                     through programmatic dependent launch, so it is off by default); False: separate launch
    head_dilation    largest number of output tiles (at most 2048, the library's limit; default 0: never) up to which a
                     convolution's tile dilation runs inside the convolution kernel itself -- its first thread block
                     makes the lists while the others wait -- instead of as a launch of its own (28 launches per E2Depth
                     step instead of 37, measured slower: the hand-over costs more than the launch it saves)
    own_tiles        True (default): in a lossless run (threshold 0, no quantiser) a tensor-core convolution needs no tile
                     list from a launch before it -- its thread blocks share out the output tiles statically and each
                     tests its own against the input words (one launch per convolution instead of two, no hand-over
                     between blocks; E2Depth step 37 -> 23 launches).  False, and in thresholded runs: the separate
                     dilation launch, whose global list spreads sparse activity evenly over the blocks.  "always": in
                     thresholded runs too
    fuse_accumulate  True (default): IncrementalRunner lets a 1x1 prediction head add its output into the accumulated
                     prediction inside its own kernel instead of launching mie_accumulate afterwards
    tc_thresholded   True (default): thresholded convolutions (threshold > 0, with or without carry) use the tensor
                     cores like lossless ones; False routes them to the FP32 kernel
    """
    threshold: float = 0.0
    carry: bool = True
    input_threshold: float = 0.0
    compat: str = "reference"
    tensor_cores: str = "auto"   # "auto": tcgen05/TF32 for convolutions with Cin*k*k >= 256; "off": FP32 everywhere
    tc_thresholded: bool = True
    tail_dilation: bool = False
    head_dilation: int = 0
    own_tiles: object = True     # True, False or "always"
    fuse_accumulate: bool = True
    kfenced_step: Optional[float] = None
    refresh: str = "native"


config = IncrConfig()


def pixel_stride(x: torch.Tensor) -> int:
    """Pixel stride (floats) of a [N,C,H,W] tensor stored channels-last, possibly a channel slice."""
    if x.dim() != 4:
        raise RuntimeError("expected a 4-D NCHW tensor")
    n, c, h, w = x.shape
    ps = x.stride(3)
    ok = (c == 1 or x.stride(1) == 1) and ps >= c and (h == 1 or x.stride(2) == w * ps) and \
        (n == 1 or x.stride(0) == h * w * ps)
    if w == 1:
        ps = x.stride(2) if h > 1 else (x.stride(0) if n > 1 else c)
        ok = (c == 1 or x.stride(1) == 1) and ps >= c
    if not ok:
        raise RuntimeError("tensor must be channels_last (NHWC in memory); got strides %s for shape %s"
                           % (tuple(x.stride()), tuple(x.shape)))
    return ps


def as_channels_last(x: torch.Tensor) -> torch.Tensor:
    nat.require_cuda(x, "tensor")
    try:
        pixel_stride(x)
        return x
    except RuntimeError:
        return x.contiguous(memory_format=torch.channels_last)


def new_field(n: int, c: int, h: int, w: int, device) -> torch.Tensor:
    return torch.zeros((n, c, h, w), dtype=torch.float32, device=device).contiguous(memory_format=torch.channels_last)


def new_bits(n: int, h: int, w: int, device) -> torch.Tensor:
    return torch.zeros(n_tiles(n, h, w), dtype=torch.int64, device=device)


class TileMask:
    """Per-pixel activity of a delta field, stored as one int64 word per 8x8 tile (bit py*8+px)."""
    __slots__ = ("bits", "n", "h", "w")

    def __init__(self, bits: torch.Tensor, n: int, h: int, w: int):
        self.bits, self.n, self.h, self.w = bits, n, h, w

    @property
    def shape(self):
        return (self.n, 1, self.h, self.w)

    def pixel_mask(self) -> torch.Tensor:
        """[N,1,H,W] uint8, 1 where the pixel is active."""
        out = torch.empty((self.n, 1, self.h, self.w), dtype=torch.uint8, device=self.bits.device)
        nat.check(nat.lib.mie_mask_expand(self.bits.data_ptr(), self.n, self.h, self.w, out.data_ptr(),
                                          nat.stream_ptr(self.bits.device)), "mask_expand")
        return out

    def tile_list(self) -> torch.Tensor:
        """Ascending indices (n*TH+ty)*TW+tx of the active tiles (int32).  Synchronises."""
        nt = self.bits.numel()
        lst = torch.empty(nt, dtype=torch.int32, device=self.bits.device)
        cnt = torch.zeros(4, dtype=torch.int32, device=self.bits.device)
        nat.check(nat.lib.mie_tiles_compact(self.bits.data_ptr(), nt, lst.data_ptr(), cnt.data_ptr(),
                                            nat.stream_ptr(self.bits.device)), "tiles_compact")
        return lst[: int(cnt[0].item())]

    def active_pixels(self) -> int:
        return int(self.pixel_mask().sum().item())


# ---------------------------------------------------------------------------------------------------------------
# Tail jobs: a convolution's tile dilation, carried by the kernel that produces the convolution's input mask
# (``mie_tail_job`` in include/mie.h).  The consumer builds the job and runs the dilation itself the first time; it
# then *offers* the job under the address of its input's tile words.  From the next step on, the wrapper of whatever
# launch writes those words *takes* the job and passes it to the entry point, and the consumer, finding the job
# *carried*, leaves its own launch out.  Every step of a network runs the same launches in the same order, so after
# one step the pairing is stable (and it is what a captured CUDA graph replays).
# ---------------------------------------------------------------------------------------------------------------
class TailJob:
    """One offered dilation: the C structure, the plan it fills (weakly: when the plan dies the offer is withdrawn, so
    that no kernel writes into its released buffers), the input tensors it reads (strongly: their addresses cannot be
    reused while the offer stands), and whether a producer carried it since the consumer last looked."""
    __slots__ = ("c", "key", "plan", "carried", "keep", "__weakref__")

    def __init__(self, plan, in_bits: torch.Tensor, union_bits: Optional[torch.Tensor], n, hin, win, k, s, p):
        self.c = nat.TailJob(in_bits.data_ptr(), n, hin, win, plan.hout, plan.wout, k, s, p,
                             union_bits.data_ptr() if union_bits is not None else None, plan.out_bits.data_ptr(),
                             plan.list.data_ptr(), plan.stale.data_ptr(), plan.counts.data_ptr(), plan.flags.data_ptr())
        self.key, self.plan, self.carried = in_bits.data_ptr(), weakref.ref(plan), False
        self.keep = (in_bits, union_bits)

    def matches(self, in_bits: torch.Tensor, union_bits: Optional[torch.Tensor]) -> bool:
        return self.c.in_bits == in_bits.data_ptr() and \
            (self.c.union_bits or 0) == (union_bits.data_ptr() if union_bits is not None else 0)


_tail_jobs: Dict[int, TailJob] = {}
_produced_at: Dict[int, int] = {}       # tile-word address -> launch counter of the launch that last wrote it
_launch_counter = [0]


def take_tail(out_bits: torch.Tensor):
    """Called by the wrapper of every launch that writes ``out_bits`` and can carry a tail job: the job offered for
    these words as a pointer for the entry point's ``tail`` argument, or None."""
    key = out_bits.data_ptr()
    _launch_counter[0] += 1
    _produced_at[key] = _launch_counter[0]
    job = _tail_jobs.get(key)
    if job is None or not config.tail_dilation:
        return None
    if job.carried:
        # the consumer did not run since the job was last carried: its lists were rebuilt and never read.  Stop
        # pairing; the consumer starts from a cleared output when it runs again.
        job.carried = False
        plan = job.plan()
        if plan is not None:
            plan.needs_clear = True
        del _tail_jobs[key]
        return None
    job.carried = True
    return C.addressof(job.c)


def tail_carried(job: Optional[TailJob]) -> bool:
    """Consumer side: True when a producer's kernel ran this job since the last call (then the lists are ready)."""
    if job is not None and job.carried:
        job.carried = False
        return True
    return False


def offer_tail(job: TailJob) -> None:
    """Consumer side, after running the dilation itself: offer the job to the producer of its input words, unless
    another consumer holds that slot, the union mask is not known to be written before the input's producer runs, or
    the field is too large for one block."""
    if not config.tail_dilation or job.key in _tail_jobs:
        return
    if job.c.N * ((job.c.Hout + 7) // 8) * ((job.c.Wout + 7) // 8) > nat.TAIL_MAX_TILES:
        return
    at = _produced_at.get(job.key)
    if at is None:
        return                                  # words written by something that cannot carry a job
    if job.c.union_bits:
        u = _produced_at.get(job.c.union_bits)
        if u is None or u > at:
            return
    plan = job.plan()
    if plan is None:
        return
    _tail_jobs[job.key] = job
    weakref.finalize(plan, _withdraw, job.key, weakref.ref(job))


def _withdraw(key: int, job_ref) -> None:
    if _tail_jobs.get(key) is job_ref():
        _tail_jobs.pop(key, None)


def withdraw_tail(job: Optional[TailJob]) -> None:
    """Consumer side: the job is no longer the one its plan uses (the input or the union mask changed)."""
    if job is not None and _tail_jobs.get(job.key) is job:
        del _tail_jobs[job.key]


def forget_tails() -> None:
    """Drop every offered job and split request (the buffers they point to are about to be released)."""
    _tail_jobs.clear()
    _produced_at.clear()
    _split_requests.clear()


def mask_from_delta(x: torch.Tensor, thr: float = 0.0, bits: Optional[torch.Tensor] = None) -> TileMask:
    n, c, h, w = x.shape
    ps = pixel_stride(x)
    if bits is None:
        bits = torch.empty(n_tiles(n, h, w), dtype=torch.int64, device=x.device)
    nat.check(nat.lib.mie_mask_from_delta(x.data_ptr(), ps, n, c, h, w, float(thr), bits.data_ptr(),
                                          nat.stream_ptr(x.device)), "mask_from_delta")
    return TileMask(bits, n, h, w)


def mask_from_tensor(m: torch.Tensor, bits: Optional[torch.Tensor] = None) -> TileMask:
    """Tile words from an explicit [N,1,H,W] or [N,C,H,W] mask tensor (bool, uint8 or int32)."""
    if not m.is_cuda:
        raise RuntimeError("mask must be a CUDA tensor")
    if m.dtype == torch.bool:
        m = m.view(torch.uint8) if m.is_contiguous() or m.is_contiguous(memory_format=torch.channels_last) else m.to(torch.uint8)
    if m.dtype not in (torch.uint8, torch.int32):
        m = (m != 0).to(torch.uint8)
    n, c, h, w = m.shape
    try:
        ps = pixel_stride(m)
    except RuntimeError:
        m = m.contiguous(memory_format=torch.channels_last)
        ps = pixel_stride(m)
    if bits is None:
        bits = torch.empty(n_tiles(n, h, w), dtype=torch.int64, device=m.device)
    nat.check(nat.lib.mie_mask_from_mask(m.data_ptr(), m.element_size(), ps, c, n, h, w, bits.data_ptr(),
                                         nat.stream_ptr(m.device)), "mask_from_mask")
    return TileMask(bits, n, h, w)


_full_masks: Dict[Tuple, "TileMask"] = {}


def full_mask(n: int, h: int, w: int, device) -> "TileMask":
    """The mask with every pixel of an [n, *, h, w] field set (ragged edge tiles: only the pixels that exist).  Cached per
    geometry; what a dense tensor carries when it is fed to the kernels as if it were a delta."""
    key = (n, h, w, str(device))
    m = _full_masks.get(key)
    if m is None:
        th, tw = -(-h // TILE), -(-w // TILE)
        rows = torch.tensor([min(TILE, h - ty * TILE) for ty in range(th)])
        cols = torch.tensor([min(TILE, w - tx * TILE) for tx in range(tw)])
        rowbits = (1 << cols) - 1                                    # one byte per row of the tile
        words = torch.zeros(th, tw, dtype=torch.int64)
        for r in range(TILE):
            words |= torch.where(rows.view(-1, 1) > r, rowbits.view(1, -1), torch.zeros(1, 1, dtype=torch.int64)) << (8 * r)
        bits = words.view(1, th, tw).expand(n, th, tw).contiguous().view(-1).to(device)
        m = _full_masks[key] = TileMask(bits, n, h, w)
    return m


def reset_delta_state(model) -> None:
    """Zero every persistent delta buffer and tile-word array of ``model`` (the module-owned ``Scratch`` buffers and
    the convolution plans).  Called after a dense pass that ran through the kernels: it leaves dense values where the
    incremental steps expect deltas that are exactly zero."""
    for m in model.modules():
        sc = m.__dict__.get("_scratch")
        if isinstance(sc, Scratch):
            for t in sc._b.values():
                t.zero_()
        for plan in getattr(m, "_plans", {}).values() if hasattr(m, "_plans") else ():
            plan.out.zero_()
            plan.out_bits.zero_()
            plan.counts[:3].zero_()
            plan.own_scratch.zero_()


class Scratch:
    """Named persistent device buffers owned by a module, so that steady-state steps allocate nothing
    (a requirement for replaying a step as a CUDA graph)."""

    def __init__(self):
        self._b: Dict[Tuple, torch.Tensor] = {}

    def get(self, key, shape, dtype, device, zero: bool = True, channels_last: bool = False) -> torch.Tensor:
        k = (key, tuple(shape), dtype, str(device))
        t = self._b.get(k)
        if t is None:
            t = torch.zeros(shape, dtype=dtype, device=device) if zero else torch.empty(shape, dtype=dtype, device=device)
            if channels_last:
                t = t.contiguous(memory_format=torch.channels_last)
            self._b[k] = t
        return t

    def clear(self):
        self._b.clear()


def resolve(x_incr, scratch: Scratch, key: str = "in") -> Tuple[torch.Tensor, TileMask]:
    """Return (delta as channels-last CUDA tensor, TileMask) for a reference-style ``Masked`` value."""
    d, m = x_incr[0], x_incr[1]
    d = as_channels_last(d)
    n, c, h, w = d.shape
    if isinstance(m, TileMask):
        if (m.n, m.h, m.w) != (n, h, w):
            raise RuntimeError("mask geometry does not match the delta tensor")
        return d, m
    bits = scratch.get(key + ".bits", (n_tiles(n, h, w),), torch.int64, d.device)
    if m is None:
        return d, mask_from_delta(d, config.input_threshold, bits)
    return d, mask_from_tensor(m, bits)


# ------------------------------------------------------------------------------------------------
# thin wrappers over the point-wise entry points
# ------------------------------------------------------------------------------------------------
ACT_CODES = {"none": nat.ACT_NONE, "relu": nat.ACT_RELU, "sigmoid": nat.ACT_SIGMOID, "tanh": nat.ACT_TANH}


def act_code(op) -> int:
    """MIE_ACT_* for a torch unary function or a name."""
    if isinstance(op, str):
        name = op
    else:
        name = getattr(op, "__name__", str(op))
    if name not in ACT_CODES:
        raise NotImplementedError(f"incremental activation '{name}' has no kernel (relu, sigmoid, tanh do)")
    return ACT_CODES[name]


def act_incr(d, m: TileMask, res, emitted, out, out_bits, op_code: int, thr: float, accumulate: bool = True) -> TileMask:
    n, c, h, w = d.shape
    nat.check(nat.lib.mie_act_incr(d.data_ptr(), pixel_stride(d), m.bits.data_ptr(), res.data_ptr(), pixel_stride(res),
                                   nat.ptr(emitted), pixel_stride(emitted) if emitted is not None else 0,
                                   out.data_ptr(), pixel_stride(out), out_bits.data_ptr(), n, c, h, w, op_code,
                                   float(thr), 1 if accumulate else 0, nat.stream_ptr(d.device)), "act_incr")
    return TileMask(out_bits, n, h, w)


def mul_incr(d1, m1, x1, d2, m2, x2, out, out_bits, thr: float = 0.0, accumulate: bool = True) -> TileMask:
    n, c, h, w = x1.shape
    nat.check(nat.lib.mie_mul_incr(
        nat.ptr(d1), pixel_stride(d1) if d1 is not None else 0, m1.bits.data_ptr() if m1 is not None else None,
        x1.data_ptr(), pixel_stride(x1),
        nat.ptr(d2), pixel_stride(d2) if d2 is not None else 0, m2.bits.data_ptr() if m2 is not None else None,
        x2.data_ptr(), pixel_stride(x2), out.data_ptr(), pixel_stride(out), out_bits.data_ptr(), n, c, h, w,
        float(thr), 1 if accumulate else 0, nat.stream_ptr(x1.device)), "mul_incr")
    return TileMask(out_bits, n, h, w)


def upsample2x(a, ma: TileMask, b, mb: Optional[TileMask], out, out_bits, mode: int = nat.UP_BILINEAR) -> TileMask:
    n, c, h, w = a.shape
    nat.check(nat.lib.mie_upsample2x(a.data_ptr(), pixel_stride(a), ma.bits.data_ptr(), nat.ptr(b),
                                     pixel_stride(b) if b is not None else 0,
                                     mb.bits.data_ptr() if mb is not None else None, out.data_ptr(), pixel_stride(out),
                                     out_bits.data_ptr(), n, c, h, w, mode, take_tail(out_bits),
                                     nat.stream_ptr(a.device)), "upsample2x")
    return TileMask(out_bits, n, 2 * h, 2 * w)


def upsample(a, ma: TileMask, out, out_bits, scale: int, mode: int = nat.UP_BILINEAR) -> TileMask:
    """out[N,C,scale*H,scale*W] = interpolate(a) for scale in {2,4,8,16}."""
    n, c, h, w = a.shape
    nat.check(nat.lib.mie_upsample(a.data_ptr(), pixel_stride(a), ma.bits.data_ptr(), None, 0, None, out.data_ptr(),
                                   pixel_stride(out), out_bits.data_ptr(), n, c, h, w, scale, mode, take_tail(out_bits),
                                   nat.stream_ptr(a.device)), "upsample")
    return TileMask(out_bits, n, scale * h, scale * w)


def add(a, ma: TileMask, b, mb: TileMask, out, out_bits) -> TileMask:
    n, c, h, w = a.shape
    nat.check(nat.lib.mie_add(a.data_ptr(), pixel_stride(a), ma.bits.data_ptr(), b.data_ptr(), pixel_stride(b),
                              mb.bits.data_ptr(), out.data_ptr(), pixel_stride(out), out_bits.data_ptr(), n, c, h, w,
                              take_tail(out_bits), nat.stream_ptr(a.device)), "add")
    return TileMask(out_bits, n, h, w)


def cat2(a, ma: TileMask, b, mb: TileMask, out, out_bits) -> TileMask:
    n, ca, h, w = a.shape
    cb = b.shape[1]
    nat.check(nat.lib.mie_cat2(a.data_ptr(), pixel_stride(a), ma.bits.data_ptr(), ca, b.data_ptr(), pixel_stride(b),
                               mb.bits.data_ptr(), cb, out.data_ptr(), pixel_stride(out), out_bits.data_ptr(), n, h, w,
                               take_tail(out_bits), nat.stream_ptr(a.device)), "cat2")
    return TileMask(out_bits, n, h, w)


def accumulate(y, d, m: TileMask) -> None:
    n, c, h, w = d.shape
    nat.check(nat.lib.mie_accumulate(y.data_ptr(), pixel_stride(y), d.data_ptr(), pixel_stride(d), m.bits.data_ptr(),
                                     n, c, h, w, nat.stream_ptr(d.device)), "accumulate")


def pack_conv_weights(weight: torch.Tensor) -> Tuple[torch.Tensor, int, int]:
    """[Cout,Cin,k,k] -> device buffer laid out [k*k][cin_pad][cout_pad]; returns (buffer, cin_pad, cout_pad)."""
    cout, cin, k, k2 = weight.shape
    assert k == k2
    cp, op, nf = C.c_int(), C.c_int(), C.c_int64()
    nat.check(nat.lib.mie_conv_pack_dims(cin, cout, k, C.byref(cp), C.byref(op), C.byref(nf)), "pack_dims")
    w = weight.detach().contiguous()
    buf = torch.empty(nf.value, dtype=torch.float32, device=weight.device)
    nat.check(nat.lib.mie_pack_conv_weights(w.data_ptr(), cout, cin, k, buf.data_ptr(), nat.stream_ptr(weight.device)),
              "pack_conv_weights")
    return buf, cp.value, op.value


def pack_conv_weights_tc(weight: torch.Tensor) -> torch.Tensor:
    """[Cout,Cin,k,k] -> device buffer [k*k][cout_pad][cin_pad32], rounded to TF32, for the tensor-core path."""
    cout, cin, k, k2 = weight.shape
    assert k == k2
    cp, op, nf = C.c_int(), C.c_int(), C.c_int64()
    nat.check(nat.lib.mie_conv_pack_dims_tc(cin, cout, k, C.byref(cp), C.byref(op), C.byref(nf)), "pack_dims_tc")
    w = weight.detach().contiguous()
    buf = torch.empty(nf.value, dtype=torch.float32, device=weight.device)
    nat.check(nat.lib.mie_pack_conv_weights_tc(w.data_ptr(), cout, cin, k, buf.data_ptr(),
                                               nat.stream_ptr(weight.device)), "pack_conv_weights_tc")
    return buf


# A first layer that runs in split precision asks the producer of its input delta for the split copy: the request is
# filed under the delta's address after the layer made the copy itself once; `delta_mask` honours it from then on.
_split_requests: Dict[int, list] = {}     # delta address -> [copy tensor, copy tile words, made-by-producer flag]


def request_split(d: torch.Tensor, copy: torch.Tensor, copy_bits: torch.Tensor) -> None:
    _split_requests[d.data_ptr()] = [copy, copy_bits, False]


def split_made(d: torch.Tensor, copy: torch.Tensor) -> bool:
    """Consumer side: True when the producer of ``d`` wrote ``copy`` since the last call."""
    r = _split_requests.get(d.data_ptr())
    if r is not None and r[0] is copy and r[2]:
        r[2] = False
        return True
    return False


def delta_mask(x: torch.Tensor, x_prev: torch.Tensor, dx: torch.Tensor, bits: torch.Tensor, thr: float = 0.0) -> TileMask:
    """dx = x - x_prev, x_prev = x and the mask of dx in one kernel (pixels with every |dx| <= thr are deferred);
    also the split-precision copy of dx when the layer that consumes it has asked for one."""
    n, c, h, w = x.shape
    r = _split_requests.get(dx.data_ptr())
    sp = sps = sb = None
    if r is not None:
        if r[2] or r[0].shape[0] != n or r[0].shape[2:] != (h, w):      # the consumer did not pick the last copy up
            del _split_requests[dx.data_ptr()]
        else:
            sp, sps, sb, r[2] = r[0].data_ptr(), pixel_stride(r[0]), r[1].data_ptr(), True
    nat.check(nat.lib.mie_delta_mask(x.data_ptr(), pixel_stride(x), x_prev.data_ptr(), pixel_stride(x_prev), dx.data_ptr(),
                                     pixel_stride(dx), bits.data_ptr(), n, c, h, w, float(thr), sp, sps or 0, sb,
                                     take_tail(bits), nat.stream_ptr(x.device)), "delta_mask")
    return TileMask(bits, n, h, w)


def events_to_voxel(events: torch.Tensor, num_bins: int, sensor_hw, out: torch.Tensor, pad_left: int = 0, pad_top: int = 0):
    """Bin one window of events ([n,4] float32 on the device: t in [0,1), x, y, polarity) into ``out``
    ([1,num_bins,H,W] channels-last), as the reference's ``events_to_voxel_grid_absT`` does on the host."""
    if events.dtype != torch.float32 or not events.is_cuda or not events.is_contiguous():
        raise RuntimeError("events must be a contiguous float32 CUDA tensor [n, 4]")
    _, c, h, w = out.shape
    nat.check(nat.lib.mie_events_to_voxel(events.data_ptr(), events.shape[0], num_bins, sensor_hw[0], sensor_hw[1],
                                          out.data_ptr(), pixel_stride(out), h, w, pad_left, pad_top,
                                          nat.stream_ptr(out.device)), "events_to_voxel")
    return out


def events_to_count_image(events: torch.Tensor, sensor_hw, out: torch.Tensor, pad_left: int = 0, pad_top: int = 0):
    """Count one window of events ([n,4] float32 on the device: t, x, y, polarity) into ``out`` ([1,2,H,W]
    channels-last: negative counts, positive counts), as the reference's ``event_histogram`` does on the host."""
    if events.dtype != torch.float32 or not events.is_cuda or not events.is_contiguous():
        raise RuntimeError("events must be a contiguous float32 CUDA tensor [n, 4]")
    n, c, h, w = out.shape
    if n != 1 or c != 2:
        raise RuntimeError("the count image is [1, 2, H, W]")
    nat.check(nat.lib.mie_events_to_count_image(events.data_ptr(), events.shape[0], sensor_hw[0], sensor_hw[1],
                                                out.data_ptr(), pixel_stride(out), h, w, pad_left, pad_top,
                                                nat.stream_ptr(out.device)), "events_to_count_image")
    return out


def maxpool_incr(d, m: TileMask, res, out, out_bits, k: int, stride: int, pad: int) -> TileMask:
    """out = maxpool(res + d) - maxpool(res); the reservoir is left as it is (advance it with ``accumulate``)."""
    n, c, h, w = d.shape
    nat.check(nat.lib.mie_maxpool_incr(d.data_ptr(), pixel_stride(d), m.bits.data_ptr(), res.data_ptr(), pixel_stride(res),
                                       out.data_ptr(), pixel_stride(out), out_bits.data_ptr(), n, c, h, w, k, stride, pad,
                                       nat.stream_ptr(d.device)), "maxpool_incr")
    return TileMask(out_bits, n, out.shape[2], out.shape[3])


def reflect_border(field: torch.Tensor, sensor_hw, pad_left: int, pad_top: int):
    """Reflection-fill the border of a [1,C,H,W] field around the sensor image placed at (pad_top, pad_left)."""
    n, c, h, w = field.shape
    if n != 1:
        raise RuntimeError("reflect_border takes one stream at a time")
    nat.check(nat.lib.mie_reflect_border(field.data_ptr(), pixel_stride(field), c, h, w, sensor_hw[0], sensor_hw[1], pad_left,
                                         pad_top, nat.stream_ptr(field.device)), "reflect_border")


def split_tf32(d: torch.Tensor, m: TileMask, out: torch.Tensor, out_bits: torch.Tensor) -> TileMask:
    """out[:, :C] = d, out[:, half:half+C] = d - tf32_trunc(d), out[:, 2*half:2*half+C] = d (half = C rounded up to 8)
    on the active tiles."""
    n, c, h, w = d.shape
    nat.check(nat.lib.mie_split_tf32(d.data_ptr(), pixel_stride(d), m.bits.data_ptr(), c, out.data_ptr(), pixel_stride(out),
                                     out_bits.data_ptr(), n, h, w, take_tail(out_bits), nat.stream_ptr(d.device)),
              "split_tf32")
    return TileMask(out_bits, n, h, w)


def kfenced(dx: torch.Tensor, carry: torch.Tensor, k: float, q: torch.Tensor, bits: torch.Tensor) -> TileMask:
    n, c, h, w = dx.shape
    nat.check(nat.lib.mie_kfenced(dx.data_ptr(), pixel_stride(dx), carry.data_ptr(), pixel_stride(carry), float(k),
                                  q.data_ptr(), pixel_stride(q), bits.data_ptr(), n, c, h, w, nat.stream_ptr(dx.device)),
              "kfenced")
    return TileMask(bits, n, h, w)
