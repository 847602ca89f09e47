"""The reference's driver protocol as a small runtime.

Every driver of the reference runs the same loop (``run_e2depth_continuous_dataset.py:55-74``,
``run_fireflownet.py:85-109``, ``run_evflownet.py:91-115``):

    frame 0, N, 2N, ...:  y = model.forward_refresh_reservoirs(x)            # dense pass, refills the state
    other frames:         dy = model((x - x_prev, None)[, None]); y += dy[0]   # incremental pass

``IncrementalRunner`` does exactly that with static device buffers, and replays the incremental step
(input delta, every kernel of the network, output accumulation) as one CUDA graph: the kernels read their
tile counts from device memory and run on fixed grids, so one captured graph serves every step whatever
the activity is.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from . import fields as fl
from .fields import TileMask


def _deltas_of(out) -> List:
    """The list of ``[delta, mask]`` outputs in whatever structure the network returns."""
    if isinstance(out, dict):
        return list(out["flow"])
    if isinstance(out, tuple) and len(out) == 2 and isinstance(out[1], list) and not torch.is_tensor(out[0]):
        # E2Depth: (pred_incr, states_incr)
        return [out[0]]
    if isinstance(out, (list, tuple)) and len(out) and isinstance(out[0], (list, tuple)):
        return list(out)
    if isinstance(out, (list, tuple)) and len(out) == 2 and torch.is_tensor(out[0]) and not torch.is_tensor(out[1]):
        return [out]                      # a single ``[delta, mask]`` pair (classifier / detector heads)
    raise TypeError("unrecognised network output")


def _dense_of(out) -> List[torch.Tensor]:
    if isinstance(out, dict):
        return list(out["flow"])
    if isinstance(out, tuple) and len(out) == 2 and isinstance(out[1], list):
        return [out[0]]
    if isinstance(out, (list, tuple)):
        return list(out)
    return [out]


class IncrementalRunner:
    """Runs one batch of independent event streams through a network with the refresh / delta protocol.

    model          E2VIDRecurrentIncr, FireFlowNetIncr or MultiResUNetRecurrentIncr (takes ``prev_states`` iff
                   it is the first)
    use_graph      replay the incremental step as a CUDA graph (captured on the second incremental step)
    refresh_every  dense refresh period in frames (None: only when ``refresh`` is called)
    feedback       feed the recurrent state back (E2Depth only).  The reference's drivers pass ``prev_states=None``
                   to every incremental step (``run_e2depth_continuous_dataset.py:70``), so as driven the network
                   computes f(x_t, zero state) - f(x_{t-1}, zero state).  With ``feedback=True`` the runner implements
                   the protocol ``UNetRecurrentIncr.forward`` is written for (``e2depth_incr.py:410-419``): the
                   reservoirs a refresh leaves behind are evaluated at (x_0, s_prev), so the first incremental step
                   is given the state delta ``s_0 - s_prev`` (the dense states themselves after a refresh from the
                   zero state), every later step the state deltas the step before returned; the accumulated output then
                   follows the dense recurrent trajectory ``y_t, s_t = refresh(x_t, s_{t-1})``.  The accumulated dense
                   states are kept too, so a scheduled refresh continues the trajectory instead of restarting it.
                   Meaningful with ``compat="exact"`` only (as written, the reference's cell delta is a list of four).
    """

    def __init__(self, model, use_graph: bool = True, refresh_every: Optional[int] = None, feedback: bool = False):
        self.model = model
        self.use_graph = use_graph
        self.refresh_every = refresh_every
        self.takes_states = hasattr(model, "unetrecurrent") or hasattr(model, "encoders") and hasattr(model, "head")
        if feedback and not self.takes_states:
            raise ValueError("feedback=True needs a network that takes recurrent states (E2Depth)")
        self.feedback = feedback
        self._heads, self._head_of, self._heads_known = [], {}, False   # prediction heads that accumulate in their kernel
        self._states = None        # accumulated dense (h, c) per encoder
        self._prev_incr = None     # state deltas handed to the next incremental step: [(dh, mask_h, dc, mask_c)]
        self._x_prev = self._x_in = self._dx = None
        self._y: List[torch.Tensor] = []
        self._graph = None
        self._pipe = None
        self._eager_steps = 0
        self._frame = 0
        self.graph_replays = 0

    # -- device-side error status ----------------------------------------------------------------
    def check(self) -> None:
        """Raise ``MieError`` if a kernel of an earlier step skipped a bad tile-list entry or gave up a bounded wait
        (the kernels record that in device memory and carry on).  Synchronises; ``refresh`` calls it, a caller
        that wants the status per step calls it after ``step``."""
        from .incr_modules.mask_incr_modules import check_device_errors
        check_device_errors(self.model)

    # -- dense pass ------------------------------------------------------------------------------
    def refresh(self, x: torch.Tensor, reset_states: bool = True):
        """Dense pass on frame ``x``.  ``reset_states=False`` (feedback mode) continues from the accumulated recurrent
        state instead of the zero state."""
        self.check()
        x = fl.as_channels_last(x)
        if hasattr(self.model, "reset_states"):
            self.model.reset_states()
        prev = None
        if self.feedback and not reset_states and self._states is not None:
            prev = [(h.clone(), c.clone()) for h, c in self._states]
        with torch.no_grad():
            out = self.model.forward_refresh_reservoirs(x, prev) if self.takes_states else \
                self.model.forward_refresh_reservoirs(x)
        if self.feedback:
            self._set_states(out[1], prev)
        ys = _dense_of(out)
        if self._x_prev is None or self._x_prev.shape != x.shape:
            self._x_prev = x.clone(memory_format=torch.channels_last)
            self._x_in = torch.empty_like(self._x_prev)
            n, c, h, w = x.shape
            cpad = (c + 3) // 4 * 4
            # pixel stride padded to a multiple of 4 floats so that the first convolution can stage the input
            # delta with 16-byte copies (5 voxel bins -> stride 8); the padding channels stay zero
            full = torch.zeros((n, cpad, h, w), dtype=x.dtype, device=x.device).contiguous(memory_format=torch.channels_last)
            self._dx = full[:, :c]
            self._dx_bits = fl.new_bits(n, h, w, x.device)
            self._y = [y.detach().clone().contiguous(memory_format=torch.channels_last) for y in ys]
            self._graph = None
            self._pipe = None
            self._eager_steps = 0
            self._heads, self._head_of, self._heads_known = [], {}, False
        else:
            self._x_prev.copy_(x)
            for dst, src in zip(self._y, ys):
                dst.copy_(src)
        self._frame = 1
        return self._y[0] if len(self._y) == 1 else self._y

    # -- recurrent-state feedback ------------------------------------------------------------------
    def _set_states(self, states, prev) -> None:
        """After a refresh that returned the dense ``states`` from the dense ``prev`` (None: zero state): keep the
        states, and make ``states - prev`` the state delta of the next incremental step."""
        new_shape = self._states is None or any(a[0].shape != b[0].shape for a, b in zip(self._states, states))
        if new_shape:
            self._states = [(fl.as_channels_last(h.detach().clone()), fl.as_channels_last(c.detach().clone()))
                            for h, c in states]
            self._prev_incr = []
            for h, c in self._states:
                n, _, hh, ww = h.shape
                self._prev_incr.append((torch.zeros_like(h), fl.new_bits(n, hh, ww, h.device),
                                        torch.zeros_like(c), fl.new_bits(n, hh, ww, h.device)))
            self._graph = None
        else:
            for (h, c), (hn, cn) in zip(self._states, states):
                h.copy_(hn)
                c.copy_(cn)
        for i, ((h, c), (dh, bh, dc, bc)) in enumerate(zip(self._states, self._prev_incr)):
            dh.copy_(h if prev is None else h - prev[i][0])
            dc.copy_(c if prev is None else c - prev[i][1])
            fl.mask_from_delta(dh, 0.0, bh)
            fl.mask_from_delta(dc, 0.0, bc)

    def _feed_back(self, states_incr) -> None:
        """After an incremental step: accumulate its state deltas and keep a copy for the next step (the network's own
        buffers are overwritten by that step while it still reads them)."""
        for (h, c), (dh, bh, dc, bc), ((sh, mh), (sc, mc)) in zip(self._states, self._prev_incr, states_incr):
            fl.accumulate(h, sh, mh)
            fl.accumulate(c, sc, mc)
            dh.copy_(sh)
            bh.copy_(mh.bits)
            dc.copy_(sc)
            bc.copy_(mc.bits)

    # -- incremental pass ------------------------------------------------------------------------
    def _step_body(self):
        # input delta, previous-frame update and input mask in one kernel
        m_in = fl.delta_mask(self._x_in, self._x_prev, self._dx, self._dx_bits, fl.config.input_threshold)
        x_incr = (self._dx, m_in)
        # A prediction head whose kernel can add its output into the accumulated prediction does so (one launch less);
        # which convolution writes which output buffer is learnt from the first step.  The target is lent for the
        # duration of this call only: the model behaves as usual when it is run outside the runner.
        for plan, y in self._heads:
            plan.accum_target = y
        try:
            if self.feedback:
                prev = [([dh, TileMask(bh, *dh.shape[:1], *dh.shape[2:])], [dc, TileMask(bc, *dc.shape[:1], *dc.shape[2:])])
                        for dh, bh, dc, bc in self._prev_incr]
                out = self.model(x_incr, prev)
                self._feed_back(out[1])
            else:
                out = self.model(x_incr, None) if self.takes_states else self.model(x_incr)
        finally:
            for plan, _ in self._heads:
                plan.accum_target = None
        deltas = list(_deltas_of(out))
        for y, d in zip(self._y, deltas):
            m = d[1]
            plan = self._head_of.get(d[0].data_ptr())
            if plan is not None and plan.accumulated:
                plan.accumulated = False          # the head's kernel has added this delta already
            elif isinstance(m, TileMask):
                fl.accumulate(y, d[0], m)
            else:
                y.add_(d[0])
        if not self._heads_known:
            self._learn_heads(deltas)

    def _learn_heads(self, deltas) -> None:
        """Find, for every output delta, the 1x1 prediction head whose plan owns that buffer."""
        from .incr_modules.mask_incr_modules import nnConvIncr
        self._heads_known = True
        plans = {p.out.data_ptr(): p for m in self.model.modules() if isinstance(m, nnConvIncr) and m.takes_second_input()
                 for p in m._plans.values()}
        self._heads, self._head_of = [], {}
        for y, d in zip(self._y, deltas):
            plan = plans.get(d[0].data_ptr())
            if plan is not None and plan.out.shape == y.shape and fl.config.fuse_accumulate:
                self._heads.append((plan, y))
                self._head_of[d[0].data_ptr()] = plan

    def step(self, x: torch.Tensor):
        if self._x_prev is None:
            raise RuntimeError("call refresh() on the first frame")
        if self.refresh_every and self._frame % self.refresh_every == 0:
            return self.refresh(x, reset_states=not self.feedback)
        self._x_in.copy_(x, non_blocking=True)
        return self._advance()

    def _advance(self):
        """One incremental step on the frame that sits in the input buffer."""
        with torch.no_grad():
            if self._graph is not None:
                self._graph.replay()
                self.graph_replays += 1
            elif self.use_graph and self._eager_steps >= 1:
                # every persistent buffer exists after one eager step; capture from now on
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._step_body()
                self._graph = g
                g.replay()
                self.graph_replays += 1
            else:
                self._step_body()
                self._eager_steps += 1
        self._frame += 1
        return self._y[0] if len(self._y) == 1 else self._y

    # -- raw events in ------------------------------------------------------------------------------
    def step_events(self, events, sensor_hw, num_bins: Optional[int] = None, representation: str = "voxel"):
        """One incremental step fed with the raw events of a window instead of a voxel grid
        (``representation="counts"``: instead of a two-channel signed count image, the flow networks' input,
        binned as the reference's ``event_histogram`` does).

        ``events``: one device tensor [n_events, 4] (t in [0,1), x, y, polarity) per stream.  The events are binned
        on the device straight into the network's input buffer (temporal-bilinear, spatial-nearest, as the
        reference's ``events_to_voxel_grid_absT`` does on the host with numpy), the border up to the padded size is
        filled by reflection as the reference's driver pads, and the step runs.  Per window this moves 16 bytes
        per event to the device instead of a dense grid."""
        if self._x_prev is None:
            raise RuntimeError("call refresh() on the first frame")
        n, c, h, w = self._x_in.shape
        if torch.is_tensor(events):
            events = [events]
        if len(events) != n:
            raise RuntimeError(f"expected the events of {n} streams, got {len(events)}")
        sh, sw = sensor_hw
        pl, pt = (w - sw) // 2, (h - sh) // 2
        for s, ev in enumerate(events):
            grid = self._x_in[s:s + 1]
            if representation == "counts":
                fl.events_to_count_image(ev, (sh, sw), grid, pl, pt)
            elif representation == "voxel":
                fl.events_to_voxel(ev, num_bins or c, (sh, sw), grid, pl, pt)
            else:
                raise ValueError("representation must be 'voxel' or 'counts'")
            if (h, w) != (sh, sw):
                fl.reflect_border(grid, (sh, sw), pl, pt)
        return self._advance()

    # -- pipelined host interface -----------------------------------------------------------------
    def step_host(self, x_host: torch.Tensor, out_host: Optional[torch.Tensor] = None, timing: bool = False):
        """``step()`` for a frame in pinned host memory, without a host wait.

        The upload runs on a copy stream into one of two device staging buffers, the download of the (first)
        accumulated output into ``out_host`` (pinned) on another stream from one of two staging copies.  A host loop
        that calls this back to back runs ahead of the device, so the upload of frame t+1 and the download of result
        t-1 overlap the kernels of frame t.  Returns the event that marks ``out_host`` valid (or the end of the step
        when ``out_host`` is None); everything is ordered for the caller's current stream afterwards as with step().
        """
        if self._x_prev is None:
            raise RuntimeError("call refresh() on the first frame")
        if not x_host.is_pinned() or (out_host is not None and not out_host.is_pinned()):
            raise RuntimeError("step_host needs pinned host tensors (torch.Tensor.pin_memory)")
        dev = self._x_prev.device
        cs = torch.cuda.current_stream(dev)
        if self._pipe is None:
            y0 = self._y[0]
            self._pipe = dict(
                s_in=torch.cuda.Stream(dev), s_out=torch.cuda.Stream(dev), n=0,
                stage_in=[torch.empty_like(self._x_in) for _ in range(2)],
                stage_out=[torch.empty_like(y0) for _ in range(2)],
                in_ready=[torch.cuda.Event() for _ in range(2)], in_free=[None, None], out_done=[None, None])
        P = self._pipe
        b = P["n"] & 1
        P["n"] += 1
        with torch.cuda.stream(P["s_in"]):
            if P["in_free"][b] is not None:
                P["s_in"].wait_event(P["in_free"][b])      # the step that last read this staging buffer has consumed it
            P["stage_in"][b].copy_(x_host, non_blocking=True)
            P["in_ready"][b].record(P["s_in"])
        cs.wait_event(P["in_ready"][b])
        y = self.step(P["stage_in"][b])
        free = torch.cuda.Event()
        free.record(cs)
        P["in_free"][b] = free
        if out_host is None:
            return free
        y0 = y[0] if isinstance(y, (list, tuple)) else y
        if P["out_done"][b] is not None:
            cs.wait_event(P["out_done"][b])                # the previous download from this staging copy has finished
        P["stage_out"][b].copy_(y0, non_blocking=True)
        ready = torch.cuda.Event()
        ready.record(cs)
        done = torch.cuda.Event(enable_timing=timing)
        with torch.cuda.stream(P["s_out"]):
            P["s_out"].wait_event(ready)
            out_host.copy_(P["stage_out"][b], non_blocking=True)
            done.record(P["s_out"])
        P["out_done"][b] = done
        return done

    @property
    def output(self):
        return self._y[0] if len(self._y) == 1 else self._y
