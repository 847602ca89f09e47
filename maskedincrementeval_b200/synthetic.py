"""Seeded synthetic inputs that stand in for the event-camera recordings the reference is driven with.

The reference's drivers read DAVIS 346x260 event recordings from absolute paths
(``run_e2depth_continuous_dataset.py:20-52``) and turn each time window into a
5-bin voxel grid (``data_fetchers/utils/util.py:78-110``) or a 2-channel count
image (``data_fetchers/utils/util.py:62-75``).  None of those recordings ship
with the code, so every benchmark and test here draws from the generators
below, which keep the shapes (346x260, 5 bins, 2 count channels) and the
binning arithmetic but synthesise the events.

Everything is driven by ``numpy.random.Generator(PCG64(seed))`` so that the
same seed gives the same bytes on every machine.
"""
from __future__ import annotations

import math
from typing import Dict, Iterator, List, Tuple

import numpy as np
import torch


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


# ----------------------------------------------------------------------------------------------
# weights
# ----------------------------------------------------------------------------------------------
def seeded_state_dict(shapes: Dict[str, Tuple[int, ...]], seed: int, init: str = "default",
                      gain: float = 1.0) -> Dict[str, torch.Tensor]:
    """Deterministic random weights for a ``{name: shape}`` map (use ``{k: v.shape for k, v in
    model.state_dict().items()}``).

    ``init="default"`` draws U(-1/sqrt(fan_in), 1/sqrt(fan_in)) for weights and biases, which is
    what ``nn.Conv2d`` does by default and therefore what the reference's random-init networks use.
    ``init="kaiming_normal"`` draws N(0, 2/fan_in) weights and zero biases.
    """
    rng = _rng(seed)
    out: Dict[str, torch.Tensor] = {}
    fan_in_of: Dict[str, int] = {}
    for name, shape in shapes.items():
        if name.endswith("weight") and len(shape) >= 2:
            fan_in_of[name[: -len("weight")]] = int(np.prod(shape[1:]))
    for name, shape in shapes.items():
        shape = tuple(int(s) for s in shape)
        prefix = name[: -len("weight")] if name.endswith("weight") else name[: -len("bias")]
        fan_in = fan_in_of.get(prefix, max(1, int(np.prod(shape[1:])) if len(shape) > 1 else 1))
        if name.endswith("weight"):
            if init == "kaiming_normal":
                w = rng.standard_normal(shape, dtype=np.float32) * np.float32(gain * math.sqrt(2.0 / fan_in))
            else:
                b = gain / math.sqrt(fan_in)
                w = rng.uniform(-b, b, size=shape).astype(np.float32)
            out[name] = torch.from_numpy(w)
        elif name.endswith("bias"):
            if init == "kaiming_normal":
                out[name] = torch.zeros(shape, dtype=torch.float32)
            else:
                b = 1.0 / math.sqrt(fan_in)
                out[name] = torch.from_numpy(rng.uniform(-b, b, size=shape).astype(np.float32))
        else:
            out[name] = torch.zeros(shape, dtype=torch.float32)
    return out


def seeded_bn_stats(sd: Dict[str, torch.Tensor], seed: int) -> Dict[str, torch.Tensor]:
    """Gives every batch-norm layer of a state dict (found by its ``running_var`` entry) plausible eval statistics:
    gamma and running_var in [0.5, 1.5), beta and running_mean ~ 0.1 * N(0,1).  In place; returns ``sd``."""
    rng = _rng(seed)
    for name in [k for k in sd if k.endswith("running_var")]:
        pre = name[: -len("running_var")]
        n = sd[name].numel()
        sd[pre + "running_var"] = torch.from_numpy(rng.uniform(0.5, 1.5, size=n).astype(np.float32))
        sd[pre + "running_mean"] = torch.from_numpy((0.1 * rng.standard_normal(n)).astype(np.float32))
        if pre + "weight" in sd:
            sd[pre + "weight"] = torch.from_numpy(rng.uniform(0.5, 1.5, size=n).astype(np.float32))
        if pre + "bias" in sd:
            sd[pre + "bias"] = torch.from_numpy((0.1 * rng.standard_normal(n)).astype(np.float32))
        if pre + "num_batches_tracked" in sd:
            sd[pre + "num_batches_tracked"] = torch.zeros((), dtype=torch.int64)
    return sd


# ----------------------------------------------------------------------------------------------
# drifting-blob deltas (single-layer and layer-chain workloads)
# ----------------------------------------------------------------------------------------------
def blob_delta_sequence(n: int, c: int, h: int, w: int, steps: int, active_frac: float, seed: int,
                        n_blobs: int = 8, sigma: float = 12.0, drift: float = 3.0,
                        delta_std: float = 0.5) -> Iterator[torch.Tensor]:
    """Yield ``steps`` deltas of shape [n, c, h, w] (channels_last) with about ``active_frac`` active pixels.

    Activity density per image is a mixture of ``n_blobs`` isotropic Gaussians (``sigma`` px) whose
    centres start uniform in the image and move ``drift`` px per step along a fixed random heading
    (wrapping around).  A pixel is active with probability proportional to the density, scaled so
    that the expected active fraction is ``active_frac``; active pixels carry N(0, delta_std) on all
    channels, every other pixel is exactly 0.
    """
    rng = _rng(seed)
    cx = rng.uniform(0, w, size=(n, n_blobs))
    cy = rng.uniform(0, h, size=(n, n_blobs))
    heading = rng.uniform(0, 2 * math.pi, size=(n, n_blobs))
    ys = np.arange(h, dtype=np.float32)[:, None]
    xs = np.arange(w, dtype=np.float32)[None, :]
    for _ in range(steps):
        out = np.zeros((n, h, w, c), dtype=np.float32)
        for i in range(n):
            dens = np.zeros((h, w), dtype=np.float32)
            for b in range(n_blobs):
                dens += np.exp(-((ys - cy[i, b]) ** 2 + (xs - cx[i, b]) ** 2) / (2 * sigma * sigma))
            p = dens * (active_frac * h * w / max(float(dens.sum()), 1e-12))
            # clipping at 1 loses a little mass at high fractions; rescale once
            p = np.minimum(p, 1.0)
            p = np.minimum(p * (active_frac * h * w / max(float(p.sum()), 1e-12)), 1.0)
            act = rng.uniform(size=(h, w)) < p
            k = int(act.sum())
            vals = rng.standard_normal((k, c), dtype=np.float32) * np.float32(delta_std)
            out[i][act] = vals
        cx = (cx + drift * np.cos(heading)) % w
        cy = (cy + drift * np.sin(heading)) % h
        t = torch.from_numpy(out).permute(0, 3, 1, 2)  # NCHW view of NHWC memory == channels_last
        yield t


# ----------------------------------------------------------------------------------------------
# synthetic event streams
# ----------------------------------------------------------------------------------------------
class EdgeEventStream:
    """Events sampled from drifting line segments plus uniform noise.

    ``n_segments`` segments have end points uniform in the image; every window each end point
    moves by an independent N(0, ``drift``) px step.  ``noise_frac`` of the events are uniform over
    the image.  Polarity is +1 or -1 with equal probability, time stamps are uniform in the window.
    """

    def __init__(self, h: int, w: int, n_events: int, n_segments: int, seed: int,
                 noise_frac: float = 0.05, drift: float = 2.0, jitter: float = 0.7):
        self.h, self.w, self.n_events, self.n_segments = h, w, n_events, n_segments
        self.noise_frac, self.drift, self.jitter = noise_frac, drift, jitter
        self.rng = _rng(seed)
        self.p0 = np.stack([self.rng.uniform(0, w, n_segments), self.rng.uniform(0, h, n_segments)], -1)
        self.p1 = np.stack([self.rng.uniform(0, w, n_segments), self.rng.uniform(0, h, n_segments)], -1)

    def window(self) -> np.ndarray:
        """One window of events as an [n_events, 4] float array with columns t in [0,1), x, y, p."""
        rng = self.rng
        n_noise = int(round(self.n_events * self.noise_frac))
        n_edge = self.n_events - n_noise
        seg = rng.integers(0, self.n_segments, n_edge)
        a = rng.uniform(0, 1, n_edge)[:, None]
        pts = self.p0[seg] * (1 - a) + self.p1[seg] * a + rng.standard_normal((n_edge, 2)) * self.jitter
        noise = np.stack([rng.uniform(0, self.w, n_noise), rng.uniform(0, self.h, n_noise)], -1)
        xy = np.concatenate([pts, noise], 0)
        x = np.clip(np.floor(xy[:, 0]), 0, self.w - 1)
        y = np.clip(np.floor(xy[:, 1]), 0, self.h - 1)
        t = rng.uniform(0, 1, self.n_events)
        p = rng.integers(0, 2, self.n_events) * 2.0 - 1.0
        self.p0 = self.p0 + rng.standard_normal(self.p0.shape) * self.drift
        self.p1 = self.p1 + rng.standard_normal(self.p1.shape) * self.drift
        return np.stack([t, x, y, p], -1)


def events_to_voxel_grid(events: np.ndarray, num_bins: int, h: int, w: int) -> np.ndarray:
    """Temporal-bilinear, spatial-nearest binning of events with t already normalised to [0, 1).

    Same arithmetic as the reference's ``events_to_voxel_grid_absT``
    (``data_fetchers/utils/util.py:78-110``): t is scaled to [0, num_bins-1], each event adds
    p*(1-dt) to bin floor(t) and p*dt to the next bin when it exists.
    """
    vox = np.zeros(num_bins * h * w, dtype=np.float32)
    if events.shape[0] == 0:
        return vox.reshape(num_bins, h, w)
    ts = (num_bins - 1) * events[:, 0]
    xs = events[:, 1].astype(np.int64)
    ys = events[:, 2].astype(np.int64)
    pols = events[:, 3].copy()
    pols[pols == 0] = -1
    tis = ts.astype(np.int64)
    dts = ts - tis
    left = pols * (1.0 - dts)
    right = pols * dts
    ok = tis < num_bins
    np.add.at(vox, xs[ok] + ys[ok] * w + tis[ok] * w * h, left[ok])
    ok = (tis + 1) < num_bins
    np.add.at(vox, xs[ok] + ys[ok] * w + (tis[ok] + 1) * w * h, right[ok])
    return vox.reshape(num_bins, h, w)


def events_to_count_image(events: np.ndarray, h: int, w: int) -> np.ndarray:
    """[2, h, w] image of negative / positive event counts, as the reference's ``event_histogram``
    (``data_fetchers/utils/util.py:62-75``) but channel-first."""
    x = events[:, 1].astype(np.int64)
    y = events[:, 2].astype(np.int64)
    p = events[:, 3]
    pos = np.zeros(h * w, dtype=np.float32)
    neg = np.zeros(h * w, dtype=np.float32)
    np.add.at(pos, x[p == 1] + w * y[p == 1], 1)
    np.add.at(neg, x[p == -1] + w * y[p == -1], 1)
    return np.stack([neg, pos], 0).reshape(2, h, w)


def reflection_pad_hw(h: int, w: int, multiple: int = 8) -> Tuple[int, int, int, int]:
    """(left, right, top, bottom) padding that brings h, w up to a multiple, split as the reference
    does for 260x346 -> 264x352: ``ReflectionPad2d((3, 3, 2, 2))`` (``run_e2depth_continuous_dataset.py:49``)."""
    ph = (-h) % multiple
    pw = (-w) % multiple
    return pw // 2, pw - pw // 2, ph // 2, ph - ph // 2


def voxel_sequence(n_streams: int, h: int, w: int, steps: int, n_events: int, n_segments: int, seed: int,
                   num_bins: int = 5, pad_to: int = 8) -> List[torch.Tensor]:
    """``steps`` voxel grids [n_streams, num_bins, H', W'] (channels_last), reflection-padded to a multiple of
    ``pad_to`` the way the reference pads before its network."""
    streams = [EdgeEventStream(h, w, n_events, n_segments, seed * 1000 + s) for s in range(n_streams)]
    l, r, t, b = reflection_pad_hw(h, w, pad_to)
    out = []
    for _ in range(steps):
        grids = np.stack([events_to_voxel_grid(s.window(), num_bins, h, w) for s in streams], 0)
        g = torch.from_numpy(grids)
        if l or r or t or b:
            g = torch.nn.functional.pad(g, (l, r, t, b), mode="reflect")
        out.append(g.contiguous(memory_format=torch.channels_last))
    return out


def count_image_sequence(n_streams: int, h: int, w: int, steps: int, n_events: int, n_segments: int,
                         seed: int) -> List[torch.Tensor]:
    """``steps`` 2-channel signed-count images [n_streams, 2, h, w] (channels_last)."""
    streams = [EdgeEventStream(h, w, n_events, n_segments, seed * 1000 + s) for s in range(n_streams)]
    out = []
    for _ in range(steps):
        imgs = np.stack([events_to_count_image(s.window(), h, w) for s in streams], 0)
        out.append(torch.from_numpy(imgs).contiguous(memory_format=torch.channels_last))
    return out
