"""Module wrappers of the masked incremental path (reference: ``incr_modules/mask_incr_modules.py:1-271``).

Every class keeps the reference's name, constructor and two entry points --
``forward(Masked) -> Masked`` (incremental) and ``forward_refresh_reservoirs(DenseT) -> DenseT`` (dense
pass that refills the persistent state) -- but the incremental entry points run libmie kernels over the
active 8x8 tiles and return ``[delta, TileMask]`` instead of ``[delta, None]``.
"""
from typing import OrderedDict, Optional, Tuple

import ctypes as C

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _native as nat
from .. import fields as fl
from ..fields import Scratch, TileMask, config
from .masked_types import DenseT, Masked
from .mask_incr_functional import IncrementReserve, IncrPointwiseMultiply, bn2d_from_module, conv2d_from_module


class IncrementMaskModule(nn.Module):
    """Interface of an incremental module (reference ``:13-17``)."""

    def forward_refresh_reservoirs(self, x: DenseT) -> DenseT:
        return x


class KFencedMaskModule(IncrementMaskModule):
    """Sigma-delta quantiser with residual carry (reference ``:21-47``): T = carry + dx;
    q = k*floor(0.5 + T/k); carry = T - q.  The reference builds one into every convolution and never
    applies it in ``forward``; it is kept for the same reason and runs on one kernel (``mie_kfenced``)."""

    def __init__(self, tp: float = .1):
        super().__init__()
        self.delta = IncrementReserve()
        self.tp = tp
        self.k = tp

    def floor_by_k(self, T):
        return self.k * torch.floor(0.5 + T / self.k)

    def forward(self, incr: Masked) -> Masked:
        d = incr[0]
        nat.require_cuda(d, "incr")
        if d.dim() != 4:
            raise RuntimeError("KFencedMaskModule takes a [N,C,H,W] delta")
        if self.delta.reservoir is None:
            raise RuntimeError("forward_refresh_reservoirs must run before the first incremental step")
        # one kernel: quantise, update the carry, emit the mask of the quantised delta
        sc = self.__dict__.setdefault("_scratch", Scratch())
        d = fl.as_channels_last(d)
        n, c, h, w = d.shape
        q = sc.get("q", (n, c, h, w), torch.float32, d.device, channels_last=True)
        bits = sc.get("q.bits", (fl.n_tiles(n, h, w),), torch.int64, d.device)
        k = self._k_host if getattr(self, "_k_host", None) is not None else float(self.k)
        return q, fl.kfenced(d, self.delta.reservoir, k, q, bits)

    def forward_refresh_reservoirs(self, x: DenseT) -> DenseT:
        self.k = self.tp * torch.norm(x)
        self._k_host = float(self.k)   # one host read per refresh, none per step
        self.delta.update_reservoir(torch.zeros_like(x))
        return x


class PointwiseMultiplyIncr(IncrementMaskModule):
    """Incremental product that leaves its reservoirs alone (reference ``:51-64``)."""

    def __init__(self, x1res_module: IncrementReserve, x2res_module: IncrementReserve):
        super().__init__()
        self.x1_res: IncrementReserve = x1res_module
        self.x2_res: IncrementReserve = x2res_module

    def forward(self, x1_incr: Masked, x2_incr: Masked) -> Masked:
        return IncrPointwiseMultiply(x1_incr, self.x1_res, x2_incr, self.x2_res)

    def forward_refresh_reservoirs(self, x1: DenseT, x2: DenseT) -> DenseT:
        return x1 * x2


class nnReservedMultiplication(PointwiseMultiplyIncr):
    """Incremental product that accumulates both operands (reference ``:67-81``), one fused kernel."""

    def __init__(self):
        super().__init__(IncrementReserve(), IncrementReserve())
        self._scratch = Scratch()

    def forward(self, x1_incr: Masked, x2_incr: Masked) -> Masked:
        d1, m1 = fl.resolve(x1_incr, self._scratch, "in1")
        d2, m2 = fl.resolve(x2_incr, self._scratch, "in2")
        n, c, h, w = d1.shape
        out = self._scratch.get("out", (n, c, h, w), torch.float32, d1.device, channels_last=True)
        bits = self._scratch.get("out.bits", (fl.n_tiles(n, h, w),), torch.int64, d1.device)
        m = fl.mul_incr(d1, m1, self.x1_res.reservoir, d2, m2, self.x2_res.reservoir, out, bits)
        return [out, m]

    def forward_refresh_reservoirs(self, x1: DenseT, x2: DenseT) -> DenseT:
        out = x1 * x2
        self.x1_res.update_reservoir(x1)
        self.x2_res.update_reservoir(x2)
        return out


class NonlinearPointOpIncr(IncrementMaskModule):
    """dy = op(res + dx) - op(res) against an external reservoir, which it does not update
    (reference ``:86-103``)."""

    def __init__(self, res_in: IncrementReserve, op=torch.tanh):
        super().__init__()
        self.reservoir_in = res_in
        self.op = op

    def forward(self, x_incr: Masked) -> Masked:
        return self._nonlin(x_incr)

    def forward_refresh_reservoirs(self, x: DenseT):
        return self.op(x)

    def _nonlin(self, x_incr: Masked):
        return nnReservedActivation._run(self, x_incr, self.reservoir_in, accumulate=False)


class nnReservedActivation(NonlinearPointOpIncr):
    """Incremental activation with its own reservoir (reference ``:243-256``):
    dy = op(res + dx) - op(res); res += dx -- one kernel, evaluated on active pixels only.

    ``threshold`` (default: ``fields.config.threshold``) withholds pixels whose output change is at most
    the threshold in every channel; with ``fields.config.carry`` what is withheld stays pending in a second
    buffer and is sent once it grows, so the error downstream is bounded by the threshold."""

    def __init__(self, op=torch.relu, threshold: Optional[float] = None):
        self.in_res = IncrementReserve()
        NonlinearPointOpIncr.__init__(self, self.in_res, op)
        self.threshold = threshold
        self.emitted: Optional[torch.Tensor] = None
        self._scratch = Scratch()

    # -- shared by the stand-alone path and NonlinearPointOpIncr ---------------------------------
    def thr(self) -> float:
        t = getattr(self, "threshold", None)
        return float(config.threshold if t is None else t)

    def carry_buffer(self, thr: float) -> Optional[torch.Tensor]:
        """The buffer of what has been sent so far; created from the reservoir when first needed."""
        if not config.carry:
            self.emitted = None      # a step without the carry does not advance it: it must not survive into a later one
            return None
        if thr <= 0.0 and self.emitted is None:
            return None              # never thresholded since the last refresh: nothing is pending
        # Once a thresholded step has run, the buffer stays in use until the next refresh, also while the threshold
        # is 0: those steps send what is pending at the pixels they touch (dy = f(x + dx) - sent, every non-zero
        # change is sent) and keep the buffer current, so a later thresholded step starts from the truth.  A buffer
        # that was left behind instead would inject everything that happened in between as one spurious delta.
        r = self.in_res.reservoir
        if self.emitted is None or self.emitted.shape != r.shape or self.emitted.device != r.device:
            self.emitted = self.op(r).contiguous(memory_format=torch.channels_last)
        return self.emitted

    @staticmethod
    def _run(self, x_incr: Masked, reserve: IncrementReserve, accumulate: bool = True):
        d = x_incr[0]
        nat.require_cuda(d, "x_incr")
        code = fl.act_code(self.op)
        res = reserve.reservoir
        if res is None:
            raise RuntimeError("forward_refresh_reservoirs must run before the first incremental step")
        if d.dim() != 4:
            # any-shape dense form, as the reference's native entry point takes it (ops.cpp:8-23)
            if not (d.is_contiguous() and res.is_contiguous()):
                raise RuntimeError("x_incr must be contiguous")  # CHECK_CONTIGUOUS, include/checks.h:7
            out = torch.empty_like(d)
            if not accumulate:
                res = res.clone()    # the dense any-shape entry point always advances what it is given
            nat.check(nat.lib.mie_activation_increment(res.data_ptr(), d.data_ptr(), out.data_ptr(), d.numel(), code,
                                                       nat.stream_ptr(d.device)), "activation_increment")
            return [out, x_incr[1]]
        sc = getattr(self, "_scratch", None)
        if sc is None:
            sc = self._scratch = Scratch()
        d, m = fl.resolve(x_incr, sc, "in")
        n, c, h, w = d.shape
        out = sc.get("out", (n, c, h, w), torch.float32, d.device, channels_last=True)
        bits = sc.get("out.bits", (fl.n_tiles(n, h, w),), torch.int64, d.device)
        thr = self.thr() if isinstance(self, nnReservedActivation) else 0.0
        em = self.carry_buffer(thr) if isinstance(self, nnReservedActivation) else None
        mo = fl.act_incr(d, m, res, em, out, bits, code, thr, accumulate)
        return [out, mo]

    def forward(self, x_incr: Masked):
        return nnReservedActivation._run(self, x_incr, self.in_res)

    def forward_refresh_reservoirs(self, x: DenseT):
        out = self.op(x)
        self.in_res.update_reservoir(x)
        if self.emitted is not None:
            if self.emitted.shape == out.shape and self.thr() > 0.0 and config.carry:
                self.emitted.copy_(out)
            else:
                self.emitted = None      # nothing is pending after a refresh: a lossless layer needs no carry
        return out


class nnReluIncr(nnReservedActivation):
    def __init__(self):
        nnReservedActivation.__init__(self, torch.relu)


class nnSigmoidIncr(nnReservedActivation):
    def __init__(self):
        nnReservedActivation.__init__(self, torch.sigmoid)


class nnTanhIncr(nnReservedActivation):
    def __init__(self):
        nnReservedActivation.__init__(self, torch.tanh)


class nnLinearIncr(nn.Linear):
    """Fully connected layer on a delta: no bias (reference ``:106-116``)."""

    def forward(self, x_incr: Masked) -> Masked:
        return F.linear(x_incr[0], self.weight, bias=None), None

    def forward_refresh_reservoirs(self, x: DenseT) -> DenseT:
        return super().forward(x)


def _square(v) -> int:
    if isinstance(v, (tuple, list)):
        if len(v) != 2 or v[0] != v[1]:
            raise NotImplementedError("only square kernels / equal strides and paddings have a kernel")
        return int(v[0])
    return int(v)


class _ConvPlan:
    """Device buffers and the argument block of one convolution at one input geometry."""

    def __init__(self, conv: "nnConvIncr", n: int, hin: int, win: int, device):
        k, s, p = conv._k, conv._s, conv._p
        self.hout, self.wout = fl.conv_out_hw(hin, win, k, s, p)
        if self.hout <= 0 or self.wout <= 0:
            raise RuntimeError("convolution output would be empty")
        nt = fl.n_tiles(n, self.hout, self.wout)
        self.ntiles = nt
        self.out = fl.new_field(n, conv.out_channels, self.hout, self.wout, device)
        self.out_bits = torch.zeros(nt, dtype=torch.int64, device=device)
        self.list = torch.zeros(nt, dtype=torch.int32, device=device)
        self.stale = torch.zeros(nt, dtype=torch.int32, device=device)
        self.counts = torch.zeros(4, dtype=torch.int32, device=device)
        self.flags = torch.zeros(nt, dtype=torch.uint8, device=device)
        # own-tiles mode: per tile a 64-bit word under construction, then a 32-bit ticket (zero between launches)
        self.own_scratch = torch.zeros(3 * nt, dtype=torch.int32, device=device)
        self.geometry = (n, hin, win)
        a = nat.ConvArgs()
        a.hin, a.win, a.n, a.hout, a.wout = hin, win, n, self.hout, self.wout
        a.k, a.stride, a.pad = k, s, p
        a.list, a.stale, a.counts, a.max_tiles = self.list.data_ptr(), self.stale.data_ptr(), self.counts.data_ptr(), nt
        a.out, a.out_ps, a.out_bits = self.out.data_ptr(), fl.pixel_stride(self.out), self.out_bits.data_ptr()
        self.args = a
        self.mask = TileMask(self.out_bits, n, self.hout, self.wout)
        self.tail = None            # fields.TailJob: this convolution's dilation, offered to its input's producer
        self.needs_clear = False    # a carried dilation was never consumed: start from a cleared output
        self.accum_target = None    # set by a driver for the duration of one call: the kernel adds its output in
        self.accumulated = False    # ... and reports here that it did


class nnConvIncr(nn.Conv2d):
    """Convolution of a masked delta (reference ``:146-196``).

    incremental: out = conv(dx, W) without bias over the output tiles the active input pixels reach,
                 optionally with the following incremental activation and a residual delta fused in;
    refresh:     dense convolution with bias (a library call; it refills nothing by itself)."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, bias=True):
        nn.Conv2d.__init__(self, in_channels, out_channels, kernel_size, stride, padding, bias=bias)
        self.kf = KFencedMaskModule(0.3)
        self._k, self._s, self._p = _square(self.kernel_size), _square(self.stride), _square(self.padding)
        self.precision = None   # None: TF32 on the tensor cores; "split": split precision there (see _split_input)
        self._packed = {}   # cin_limit -> (version, device, buffer, cin_pad, cout_pad)
        self._plans = {}
        self._cw = None
        self._scratch = Scratch()

    # The reference keeps a [Cin,kH,kW,Cout] copy of the filter in this attribute (``:156``).
    @property
    def conv2d_weights(self):
        v = (self.weight._version, self.weight.device)
        if self._cw is None or self._cw[0] != v:
            self._cw = (v, torch.permute(self.weight.detach(), (1, 2, 3, 0)).contiguous())
        return self._cw[1]

    def load_state_dict(self, state_dict: 'OrderedDict[str, torch.Tensor]', strict: bool = True):
        r = nn.Conv2d.load_state_dict(self, state_dict, strict=strict)
        self._packed.clear()
        self._cw = None
        return r

    def _split_input(self, cin: int) -> bool:
        """Whether this layer runs on the tensor cores in split precision: input [d, d - tf32(d), d] against the
        filter blocks [W, W, W - tf32(W)] (three times the channels), which is the fp32 convolution up to the dropped
        lo*lo term.  Taken by
          * narrow-input layers (the 5-bin voxel head): the raw O(1) input delta must not be truncated to TF32 (it
            random-walks in the first reservoir) and neither may the filter be rounded (the input changes by its full
            scale between frames);
          * every tensor-core layer of a network built with ``precision = "split"`` (the un-normalised ReLU stacks
            fed by raw event counts, FireFlowNet and the delayed EV-FlowNet): there the 2^-11 relative error of a
            TF32 input is already 2e-3 of the output range after one step, whatever the rounding mode."""
        if config.tensor_cores != "auto" or self.out_channels % 4:
            return False
        if self._s == 1 and self._k in (3, 5, 7) and cin <= 8 and cin * self._k * self._k >= 100:
            return True
        return (getattr(self, "precision", None) == "split" and cin * self._k * self._k >= 256
                and self._k in (1, 3, 5, 7) and self._s in (1, 2))

    def _weights(self, cin_limit: Optional[int] = None, split: bool = False, bn: "Optional[nn.BatchNorm2d]" = None):
        """Packed filter for the kernels, repacked whenever the parameter changed or moved.  ``bn``: an eval
        batch-norm that follows the convolution; on a delta it is a per-channel scale (``bn2d_from_module``), which
        is folded into the packed filter."""
        key = cin_limit or self.in_channels
        ver = (self.weight._version, self.weight.device, self.weight.data_ptr())
        if bn is not None:
            ver = ver + (id(bn), bn.running_var._version, bn.running_var.data_ptr(), bn.eps,
                         None if bn.weight is None else (bn.weight._version, bn.weight.data_ptr()))
            key = ("bn", id(bn), key)
        if split:
            key = ("split", key)
        hit = self._packed.get(key)
        if hit is None or hit[0] != ver:
            w = self.weight.detach()
            if bn is not None:
                scale = (bn.weight.detach() if bn.weight is not None else 1.0) / torch.sqrt(bn.running_var + bn.eps)
                w = w * scale.view(-1, 1, 1, 1)
            if cin_limit and cin_limit != self.in_channels:
                w = w[:, :cin_limit].contiguous()
            if split:
                c = cin_limit or self.in_channels
                wf = w[:, :c].float()
                w_hi = (wf.view(torch.int32) + 0x1000 & ~0x1FFF).view(torch.float32)   # TF32 rounding, as the packing does
                half = (c + 7) // 8 * 8
                w3 = torch.zeros((w.shape[0], 3 * half, self._k, self._k), dtype=torch.float32, device=w.device)
                w3[:, :c] = wf
                w3[:, half:half + c] = wf
                w3[:, 2 * half:2 * half + c] = wf - w_hi
                w = w3
                key_depth = 3 * half
            else:
                key_depth = cin_limit or self.in_channels
            buf, cp, op = fl.pack_conv_weights(w.float())
            tc = None
            # the library decides per call whether the tensor-core copy is used; it never is below this depth
            if key_depth * self._k * self._k >= 256 and self.out_channels % 4 == 0:
                tc = fl.pack_conv_weights_tc(w.float())
            hit = (ver, buf, cp, op, tc)
            self._packed[key] = hit
        return hit[1], hit[2], hit[3], hit[4]

    def _plan(self, n, hin, win, device) -> _ConvPlan:
        if self.dilation != (1, 1) or self.groups != 1 or self.padding_mode != "zeros":
            raise NotImplementedError("dilated / grouped / non-zero-padded convolutions have no kernel")
        key = (n, hin, win, str(device))
        p = self._plans.get(key)
        if p is None:
            p = self._plans[key] = _ConvPlan(self, n, hin, win, device)
        return p

    def takes_second_input(self) -> bool:
        """True for the 1x1 prediction heads whose kernel can add a second input field as it reads the first."""
        return self._k == 1 and self._s == 1 and self._p == 0 and self.out_channels <= 4 and self.in_channels <= 2048

    def forward_fused(self, x_incr: Masked, activation: "Optional[nnReservedActivation]" = None,
                      addend: Optional[Masked] = None, cin_limit: Optional[int] = None,
                      bn: "Optional[nn.BatchNorm2d]" = None, refresh: bool = False,
                      second: Optional[Masked] = None) -> Masked:
        """conv(dx) [* batch-norm scale] [+ addend] [-> incremental activation], one dilation launch and one
        convolution launch.

        ``refresh=True`` is the dense evaluation of the same layer on the same kernels: the input pair carries a dense
        tensor, the bias is added, the activation's reservoir is set to conv + bias (+ addend) and the output is
        f(reservoir) -- in full fp32, whatever ``config.tensor_cores`` says."""
        sc = self._scratch
        if refresh and bn is not None:
            raise NotImplementedError("dense evaluation with a folded batch-norm")
        if config.kfenced_step and not refresh:
            x_incr = self._quantise_input(x_incr)
        d, m = fl.resolve(x_incr, sc, "in")
        n, cin, hin, win = d.shape
        cin_eff = cin_limit or self.in_channels
        if cin != cin_eff:
            raise RuntimeError(f"expected {cin_eff} input channels, got {cin}")
        plan = self._plan(n, hin, win, d.device)
        # Split precision is only meaningful on the tensor cores, which truncate the three channel blocks as the scheme
        # assumes; a thresholded layer that is routed to the FP32 kernel must see the plain input and filter.
        thresholded = activation is not None and (activation.thr() > 0.0 or
                                                  (config.carry and activation.emitted is not None))
        split = self._split_input(cin) and (config.tc_thresholded or not thresholded) and not refresh
        wbuf, cp, op, wtc = self._weights(cin_limit, split, bn)
        if split:
            c3 = 3 * ((cin + 7) // 8 * 8)
            d3 = sc.get("split", (n, c3, hin, win), torch.float32, d.device, channels_last=True)
            sb = sc.get("split.bits", (fl.n_tiles(n, hin, win),), torch.int64, d.device)
            # the producer of the delta (the driver's input-delta kernel) writes the copy itself once asked to
            if not fl.split_made(d, d3):
                fl.split_tf32(d, m, d3, sb)
                if x_incr[1] is m and cin_limit is None:
                    fl.request_split(d, d3, sb)
            d, cin = d3, c3
        a = plan.args
        union = None
        a.in2, a.in2_ps = None, 0
        if second is not None:
            # the sum x + second is formed as the 1x1 head kernel reads its input; the second mask joins the tile set
            # as the dilation's union mask (output geometry = input geometry for a 1x1 convolution)
            if not self.takes_second_input() or addend is not None or split or (config.kfenced_step and not refresh):
                raise RuntimeError("a second input needs a plain 1x1 prediction head")
            d2, m2 = fl.resolve(second, sc, "in2")
            if d2.shape != d.shape:
                raise RuntimeError("the second input must have the first one's shape")
            union = m2.bits
            a.in2, a.in2_ps = d2.data_ptr(), fl.pixel_stride(d2)
        if addend is not None:
            ad, am = fl.resolve(addend, sc, "addend")
            if ad.shape != plan.out.shape:
                raise RuntimeError("residual delta must have the convolution's output shape")
            union = am.bits
            a.addend, a.addend_ps = ad.data_ptr(), fl.pixel_stride(ad)
        else:
            a.addend, a.addend_ps = None, 0
        st = nat.stream_ptr(d.device)
        # The tile dilation: carried by the kernel that wrote the input mask when that pairing has been established
        # (fields.TailJob), else launched here and offered to that kernel for the steps to come.
        job = plan.tail
        if job is None or not job.matches(m.bits, union):
            fl.withdraw_tail(job)
            job = plan.tail = fl.TailJob(plan, m.bits, union, n, hin, win, self._k, self._s, self._p)
        if plan.needs_clear:
            plan.out.zero_(), plan.out_bits.zero_(), plan.counts[:3].zero_(), plan.own_scratch.zero_()
            plan.needs_clear = False
        a.head, a.own_tiles, a.own_scratch = None, 0, None
        if config.head_dilation and plan.ntiles <= min(config.head_dilation, nat.TAIL_MAX_TILES) and not config.tail_dilation:
            a.head = C.addressof(job.c)     # the convolution kernel's first block makes the lists itself
        elif (config.own_tiles and not refresh and not config.tail_dilation and not config.head_dilation
              and (config.own_tiles == "always" or (config.threshold == 0.0 and not config.kfenced_step))):
            # Every thread block of the convolution kernel finds its own tiles (the library falls back to the separate
            # launch for the FP32 kernels and for fields too large for that).  Lossless runs only: their fields are
            # densely active after the first layers, where the static deal of tiles to blocks loses nothing; a
            # thresholded run keeps the global list, which spreads few active tiles evenly (measured +3 % otherwise).
            a.head, a.own_tiles, a.own_scratch = C.addressof(job.c), 1, plan.own_scratch.data_ptr()
        elif not fl.tail_carried(job):
            nat.check(nat.lib.mie_tiles_dilate(m.bits.data_ptr(), n, hin, win, plan.hout, plan.wout, self._k, self._s,
                                               self._p, union.data_ptr() if union is not None else None,
                                               plan.out_bits.data_ptr(), plan.list.data_ptr(), plan.stale.data_ptr(),
                                               plan.counts.data_ptr(), plan.flags.data_ptr(), st), "tiles_dilate")
            fl.offer_tail(job)
        a.in_, a.in_ps, a.cin = d.data_ptr(), fl.pixel_stride(d), cin
        a.wpacked, a.cin_pad, a.cout, a.cout_pad = wbuf.data_ptr(), cp, self.out_channels, op
        a.wpacked_tc = wtc.data_ptr() if (wtc is not None and config.tensor_cores == "auto" and not refresh) else None
        a.refresh = 1 if refresh else 0
        a.bias = self.bias.data_ptr() if (refresh and self.bias is not None) else None
        if activation is not None:
            res = activation.in_res.reservoir
            if refresh and (res is None or res.shape != plan.out.shape or res.device != plan.out.device):
                activation.in_res.update_reservoir(plan.out)       # allocates; the kernel overwrites it
                res = activation.in_res.reservoir
            if res is None:
                raise RuntimeError("forward_refresh_reservoirs must run before the first incremental step")
            if res.shape != plan.out.shape:
                raise RuntimeError("activation reservoir does not match the convolution output")
            thr = 0.0 if refresh else activation.thr()
            em = None if refresh else activation.carry_buffer(thr)
            a.act, a.thr = fl.act_code(activation.op), thr
            a.res, a.res_ps = res.data_ptr(), fl.pixel_stride(res)
            a.emitted, a.emitted_ps = (em.data_ptr(), fl.pixel_stride(em)) if em is not None else (None, 0)
        else:
            a.act, a.thr, a.res, a.res_ps, a.emitted, a.emitted_ps = nat.ACT_NONE, 0.0, None, 0, None, 0
        if a.thr > 0.0 or a.emitted:
            nat.set_option(nat.OPT_TC_THRESHOLDED, 1 if config.tc_thresholded else 0)
        self.last_used_tensor_cores = bool(nat.lib.mie_conv_uses_tensor_cores(C.byref(a)))
        self.last_cluster_size = int(nat.lib.mie_conv_cluster_size(C.byref(a)))
        if split and not self.last_used_tensor_cores:
            raise RuntimeError("a split-precision convolution did not qualify for the tensor cores (its three channel "
                               "blocks only add up to the fp32 result there); set precision=None on this layer")
        a.tail = fl.take_tail(plan.out_bits)
        a.accum, a.accum_ps, plan.accumulated = None, 0, False
        tgt = plan.accum_target
        if tgt is not None and not refresh and self.takes_second_input() and tgt.shape == plan.out.shape:
            a.accum, a.accum_ps, plan.accumulated = tgt.data_ptr(), fl.pixel_stride(tgt), True
        nat.check(nat.lib.mie_conv_tiles(C.byref(a), st), "conv_tiles")
        if refresh and activation is not None and activation.emitted is not None:
            if activation.emitted.shape == plan.out.shape and activation.thr() > 0.0 and config.carry:
                activation.emitted.copy_(plan.out)      # what has been sent so far = f(reservoir)
            else:
                activation.emitted = None
        return [plan.out, plan.mask]

    def forward(self, x_incr):
        return self.forward_fused(x_incr)

    def _quantise_input(self, x_incr: Masked) -> Masked:
        """The reference's k-fenced quantiser in front of the convolution (``:157``, ``:166``), with the absolute
        step ``config.kfenced_step``; its carry starts at zero after a refresh."""
        kf, d = self.kf, x_incr[0]
        r = kf.delta.reservoir
        if r is None or r.shape != d.shape or r.device != d.device:
            kf.delta.update_reservoir(torch.zeros_like(d, memory_format=torch.channels_last))
        kf._k_host = float(config.kfenced_step)
        return kf(x_incr)

    def error_words(self):
        """``[(geometry, counts tensor)]`` of every plan: word 3 of ``counts`` holds the MIE_ERR_* bits the kernels
        raised since it was last cleared (see ``check_device_errors``)."""
        return [(p.geometry, p.counts) for p in self._plans.values()]

    def clear_errors(self):
        """Clear the error word of every plan, and the tile-word scratch of the own-tiles mode, which an aborted
        launch may have left half-filled."""
        for p in self._plans.values():
            p.counts[3] = 0
            p.own_scratch.zero_()

    def forward_refresh_reservoirs(self, x):
        # The reference also resets its (never applied) quantiser here, which costs a norm and a
        # zero tensor of the input's size per convolution (``:193``); nothing reads either.  When the quantiser is
        # switched on (config.kfenced_step) its carry is cleared instead.
        if config.kfenced_step and self.kf.delta.reservoir is not None:
            self.kf.delta.reservoir.zero_()
        return nn.Conv2d.forward(self, x)


def check_device_errors(model: nn.Module, clear: bool = True) -> None:
    """Read the device-side error word of every convolution of ``model`` (one small copy to the host, which
    synchronises) and raise ``MieError`` naming the layers whose kernels reported a skipped tile-list entry or an
    expired wait.  The kernels themselves never stop the device; without this call such a step would return wrong data
    silently.  The reference exits the process on any CUDA error instead (``include/checks.h:12-21``)."""
    named = [(name, geo, cnt) for name, m in model.named_modules() if isinstance(m, nnConvIncr)
             for geo, cnt in m.error_words()]
    if not named:
        return
    words = torch.stack([cnt[3] for _, _, cnt in named]).cpu().tolist()
    bad = [(name, geo, w) for (name, geo, _), w in zip(named, words) if w]
    if not bad:
        return
    if clear:
        for m in model.modules():
            if isinstance(m, nnConvIncr):
                m.clear_errors()
    raise nat.MieError("; ".join(f"{name or '<conv>'} (batch {g[0]}, input {g[1]}x{g[2]}): {nat.describe_error_word(w)}"
                                 for name, g, w in bad))


def set_precision(model: nn.Module, precision: Optional[str]) -> None:
    """Set ``precision`` (None or "split") on every convolution of ``model``."""
    if precision not in (None, "split"):
        raise ValueError("precision must be None or 'split'")
    for m in model.modules():
        if isinstance(m, nnConvIncr):
            m.precision = precision


class nnConvIncrBase(nnConvIncr):
    """The reference's variant that always routes through ``conv2d_from_module`` (``:122-142``)."""

    def forward(self, x_incr):
        return conv2d_from_module(x_incr, self.conv2d_weights, stride=self.stride, padding=self.padding)


class nnBatchNorm2dIncr(nn.BatchNorm2d):
    """Eval batch-norm: a per-channel scale on a delta (reference ``:200-207``)."""

    def forward(self, x_incr):
        return bn2d_from_module(x_incr, self)

    def forward_refresh_reservoirs(self, x):
        return super().forward(x)


class nnMaxPool2dIncr(nn.MaxPool2d):
    """mp(res + dx) - mp(res); res += dx (reference ``:210-225``).  One kernel evaluates the windows that touch an
    active input pixel against the reservoir, a second one advances the reservoir (windows overlap, so it may only
    move once every window has been read)."""

    def __init__(self, kernel_size, stride=None, padding=0):
        nn.MaxPool2d.__init__(self, kernel_size=kernel_size, stride=stride, padding=padding)
        self.functional = lambda x: F.max_pool2d(x, kernel_size=self.kernel_size, stride=self.stride, padding=self.padding)
        self.mp_res = IncrementReserve()
        self._scratch = Scratch()

    def forward(self, x_incr: Masked) -> Masked:
        res = self.mp_res.reservoir
        if res is None:
            raise RuntimeError("forward_refresh_reservoirs must run before the first incremental step")
        k, s, p = _square(self.kernel_size), _square(self.stride), _square(self.padding)
        if self.dilation != 1 or self.ceil_mode or self.return_indices or not (1 <= k <= 7 and 1 <= s <= 4 and 2 * p <= k):
            out = self.functional(res + x_incr[0]) - self.functional(res)     # shapes the kernel does not take
            self.mp_res.accumulate(x_incr)
            return out, None
        sc = self._scratch
        d, m = fl.resolve(x_incr, sc, "in")
        n, c, h, w = d.shape
        ho, wo = fl.conv_out_hw(h, w, k, s, p)
        out = sc.get("out", (n, c, ho, wo), torch.float32, d.device, channels_last=True)
        bits = sc.get("out.bits", (fl.n_tiles(n, ho, wo),), torch.int64, d.device)
        mo = fl.maxpool_incr(d, m, res, out, bits, k, s, p)
        fl.accumulate(res, d, m)
        return [out, mo]

    def forward_refresh_reservoirs(self, x: DenseT) -> DenseT:
        self.mp_res.update_reservoir(x)
        return super().forward(x)


class nnAdaptiveAvgPool2dIncr(nn.AdaptiveAvgPool2d):
    """Linear, so applied to the delta as is (reference ``:228-233``)."""

    def forward(self, x_incr):
        return nn.AdaptiveAvgPool2d.forward(self, x_incr[0]), None

    def forward_refresh_reservoirs(self, x):
        return super().forward(x)


class nnSequentialIncr(nn.Sequential):
    """Chains ``forward_refresh_reservoirs`` (reference ``:236-240``).  The incremental pass runs a convolution, the
    eval batch-norm behind it (a per-channel scale on a delta) and the activation behind that as one fused launch."""

    def forward(self, x_incr):
        mods = list(self)
        i = 0
        while i < len(mods):
            m = mods[i]
            if type(m) is nnConvIncr:
                j, bn, act = i + 1, None, None
                if j < len(mods) and type(mods[j]) is nnBatchNorm2dIncr and not mods[j].training and mods[j].track_running_stats:
                    bn, j = mods[j], j + 1
                if j < len(mods) and isinstance(mods[j], nnReservedActivation) and mods[j].in_res.reservoir is not None \
                        and mods[j].in_res.reservoir.dim() == 4:
                    act, j = mods[j], j + 1
                if bn is not None or act is not None:
                    x_incr = m.forward_fused(x_incr, act, bn=bn)
                    i = j
                    continue
            x_incr = m(x_incr)
            i += 1
        return x_incr

    def forward_refresh_reservoirs(self, x):
        for module in self:
            x = module.forward_refresh_reservoirs(x)
        return x
