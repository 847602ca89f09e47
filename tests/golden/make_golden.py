"""Generate ``tests/golden/*.npz`` by running the reference's own modules on seeded inputs.

Run from the repository root on a machine that has a checkout of the reference:

    python tests/golden/make_golden.py [/path/to/reference]

Each file stores the inputs, the seed the weights were drawn from
(``maskedincrementeval_b200.synthetic.seeded_state_dict``) and the outputs the reference produced,
so the restatement in ``oracle/restatement.py`` and the CUDA path can be checked on machines where
the reference is absent.
"""
from __future__ import annotations

import contextlib
import io
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from maskedincrementeval_b200.synthetic import seeded_state_dict  # noqa: E402
from oracle.reference_loader import DEFAULT_ROOT, E2DEPTH_CONFIG, load_reference  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def _np(t):
    return t.detach().cpu().contiguous().numpy()


def _shapes(m):
    return {k: tuple(v.shape) for k, v in m.state_dict().items()}


def _quiet(fn, *a, **k):
    with contextlib.redirect_stdout(io.StringIO()):
        return fn(*a, **k)


def _sparse_delta(g: torch.Generator, shape, frac=0.15, std=0.5):
    n, c, h, w = shape
    act = (torch.rand(n, 1, h, w, generator=g) < frac).float()
    return (torch.randn(shape, generator=g) * std * act).contiguous(memory_format=torch.channels_last)


def main(ref_root: str = DEFAULT_ROOT):
    ref = load_reference(ref_root)
    M = ref.modules
    torch.set_grad_enabled(False)
    g = torch.Generator().manual_seed(1234)

    # ---- activations: the reference's own test shape (tests/test_pointops.py:12) and a 4-D one ----
    out = {}
    for name, op in (("relu", torch.relu), ("sigmoid", torch.sigmoid), ("tanh", torch.tanh)):
        for tag, shape in (("3d", (1, 40, 80)), ("4d", (2, 6, 19, 23))):
            x = torch.randn(shape, generator=g)
            a = M.nnReservedActivation(op)
            y0 = a.forward_refresh_reservoirs(x)
            d1, d2 = torch.randn(shape, generator=g), torch.randn(shape, generator=g) * 0.1
            o1 = a.forward([d1, None])[0].clone()
            r1 = a.in_res.reservoir.clone()
            o2 = a.forward([d2, None])[0].clone()
            r2 = a.in_res.reservoir.clone()
            for k, v in dict(x=x, y0=y0, d1=d1, d2=d2, o1=o1, r1=r1, o2=o2, r2=r2).items():
                out[f"{name}_{tag}_{k}"] = _np(v)
    np.savez_compressed(os.path.join(OUT, "activation.npz"), **out)

    # ---- product ----
    out = {}
    x1, x2 = torch.randn(2, 5, 17, 21, generator=g), torch.randn(2, 5, 17, 21, generator=g)
    m = M.nnReservedMultiplication()
    out["y0"] = _np(m.forward_refresh_reservoirs(x1, x2))
    out["x1"], out["x2"] = _np(x1), _np(x2)
    for s in (1, 2):
        da, db = _sparse_delta(g, x1.shape), _sparse_delta(g, x1.shape)
        o = m.forward([da, None], [db, None])[0]
        out[f"da{s}"], out[f"db{s}"], out[f"o{s}"] = _np(da), _np(db), _np(o)
        out[f"r1_{s}"], out[f"r2_{s}"] = _np(m.x1_res.reservoir), _np(m.x2_res.reservoir)
    np.savez_compressed(os.path.join(OUT, "product.npz"), **out)

    # ---- convolution of a delta (tests/test_pointops.py:25-35 shape first) ----
    out = {}
    for tag, (cin, cout, k, s, p, h, w, n) in dict(
            ref_test=(3, 5, 3, 1, 1, 25, 25, 1), k5s2=(4, 6, 5, 2, 2, 22, 30, 2), k1=(8, 2, 1, 1, 0, 9, 13, 1),
            k3s2=(6, 8, 3, 2, 1, 21, 19, 1), k5s1=(5, 7, 5, 1, 2, 20, 27, 1)).items():
        c = M.nnConvIncr(cin, cout, k, s, p, bias=True).eval()
        sd = seeded_state_dict(_shapes(c), seed=len(tag) * 7 + k, init="kaiming_normal")
        sd["bias"] = torch.linspace(-0.5, 0.5, cout)
        c.load_state_dict(sd)
        x = torch.randn(n, cin, h, w, generator=g).contiguous(memory_format=torch.channels_last)
        dx = _sparse_delta(g, (n, cin, h, w))
        out[f"{tag}_cfg"] = np.array([cin, cout, k, s, p, h, w, n])
        out[f"{tag}_w"], out[f"{tag}_b"] = _np(c.weight), _np(c.bias)
        out[f"{tag}_x"], out[f"{tag}_dx"] = _np(x), _np(dx)
        out[f"{tag}_dense"] = _np(c.forward_refresh_reservoirs(x))
        out[f"{tag}_incr"] = _np(c([dx, None])[0])
    np.savez_compressed(os.path.join(OUT, "conv.npz"), **out)

    # ---- quantiser, BN on a delta, bilinear x2, max-pool ----
    out = {}
    kf = M.KFencedMaskModule(0.3)
    x = torch.randn(1, 4, 12, 14, generator=g)
    kf.forward_refresh_reservoirs(x)
    out["kf_x"], out["kf_k"] = _np(x), np.array(float(kf.k))
    for s in (1, 2, 3):
        d = torch.randn(1, 4, 12, 14, generator=g) * 2.0
        q = kf.forward([d, None])[0]
        out[f"kf_d{s}"], out[f"kf_q{s}"], out[f"kf_c{s}"] = _np(d), _np(q), _np(kf.delta.reservoir)
    bn = M.nnBatchNorm2dIncr(6).eval()
    bn.running_var.copy_(torch.rand(6, generator=g) + 0.5)
    bn.running_mean.copy_(torch.randn(6, generator=g))
    bn.weight.copy_(torch.randn(6, generator=g))
    bn.bias.copy_(torch.randn(6, generator=g))
    d = torch.randn(2, 6, 9, 11, generator=g)
    out["bn_var"], out["bn_w"], out["bn_eps"] = _np(bn.running_var), _np(bn.weight), np.array(bn.eps)
    out["bn_d"], out["bn_o"] = _np(d), _np(bn([d, None])[0])
    d = _sparse_delta(g, (2, 5, 11, 13), frac=0.1)
    out["up_d"], out["up_o"] = _np(d), _np(ref.functional.interpolate_from_module([d, None])[0])
    mp = M.nnMaxPool2dIncr(3, 2, 1)
    x = torch.randn(1, 4, 16, 18, generator=g)
    out["mp_x"], out["mp_y0"] = _np(x), _np(mp.forward_refresh_reservoirs(x))
    d = _sparse_delta(g, x.shape)
    out["mp_d"], out["mp_o"] = _np(d), _np(mp([d, None])[0])
    np.savez_compressed(os.path.join(OUT, "misc_ops.npz"), **out)

    # ---- ConvLSTM cell ----
    out = {}
    cell = ref.e2depth.ConvLSTMIncr(6, 6, 3).eval()
    cell.load_state_dict(seeded_state_dict(_shapes(cell), seed=11, init="kaiming_normal"))
    x = torch.randn(2, 6, 14, 18, generator=g).contiguous(memory_format=torch.channels_last)
    h0, c0 = cell.forward_refresh_reservoirs(x, None)
    out["x"], out["h0"], out["c0"], out["seed"] = _np(x), _np(h0), _np(c0), np.array(11)
    for s in (1, 2):
        d = _sparse_delta(g, x.shape, frac=0.2)
        hid, cl = cell([d, None], None)
        out[f"d{s}"], out[f"dh{s}"], out[f"dc{s}"] = _np(d), _np(hid[0]), _np(cl[0])
    np.savez_compressed(os.path.join(OUT, "convlstm.npz"), **out)

    # ---- E2Depth, small (base 4 channels, 64x96), reference as written ----
    out = {}
    cfg = dict(E2DEPTH_CONFIG)
    cfg["base_num_channels"] = 4
    net = _quiet(ref.e2depth.E2VIDRecurrentIncr, cfg).eval()
    net.load_state_dict(seeded_state_dict(_shapes(net), seed=21, init="kaiming_normal"))
    x = torch.randn(1, 5, 64, 96, generator=g).contiguous(memory_format=torch.channels_last)
    y0, st0 = net.forward_refresh_reservoirs(x, None)
    out["seed"], out["base"], out["x"], out["y0"] = np.array(21), np.array(4), _np(x), _np(y0)
    out["h0_0"], out["c0_0"] = _np(st0[0][0]), _np(st0[0][1])
    for s in (1, 2, 3):
        d = _sparse_delta(g, x.shape, frac=0.08)
        dy, st = net([d, None], None)
        out[f"d{s}"], out[f"dy{s}"] = _np(d), _np(dy[0])
        out[f"dh{s}_2"] = _np(st[2][0][0])
    np.savez_compressed(os.path.join(OUT, "e2depth_small.npz"), **out)

    # ---- FireFlowNet (8 base channels, 32x48) ----
    out = {}
    net = ref.fireflownet.FireFlowNetIncr(dict(base_num_channels=8, kernel_size=3, mask_output=False), 2).eval()
    net.load_state_dict(seeded_state_dict(_shapes(net), seed=31, init="kaiming_normal"))
    x = torch.randn(2, 2, 32, 48, generator=g).contiguous(memory_format=torch.channels_last)
    out["seed"], out["x"] = np.array(31), _np(x)
    out["y0"] = _np(net.forward_refresh_reservoirs(x)["flow"][0])
    for s in (1, 2, 3):
        d = _sparse_delta(g, x.shape, frac=0.1)
        out[f"d{s}"], out[f"dy{s}"] = _np(d), _np(net([d, None])["flow"][0][0])
    np.savez_compressed(os.path.join(OUT, "fireflownet_small.npz"), **out)

    # ---- EVFlowNet (fixed architecture), 32x32 ----
    out = {}
    net = ref.evflownet.MultiResUNetRecurrentIncr().eval()
    net.load_state_dict(seeded_state_dict(_shapes(net), seed=41, init="kaiming_normal"))
    x = torch.randn(1, 2, 32, 32, generator=g).contiguous(memory_format=torch.channels_last)
    out["seed"], out["x"] = np.array(41), _np(x)
    for i, p in enumerate(net.forward_refresh_reservoirs(x)):
        out[f"y0_{i}"] = _np(p)
    for s in (1, 2):
        d = _sparse_delta(g, x.shape, frac=0.1)
        out[f"d{s}"] = _np(d)
        for i, p in enumerate(net([d, None])):
            out[f"dy{s}_{i}"] = _np(p[0])
    np.savez_compressed(os.path.join(OUT, "evflownet_small.npz"), **out)
    # ---- delayed-prediction EVFlowNet (8 base channels, 32x48) ----
    import importlib
    delayed = importlib.import_module("incr_modules.delayedevflownet_incr")
    out = {}
    net = delayed.DelayedEVFlowNetIncr(dict(base_num_channels=8, kernel_size=3, mask_output=False), 2).eval()
    net.load_state_dict(seeded_state_dict(_shapes(net), seed=51, init="kaiming_normal"))
    x = torch.randn(1, 2, 32, 48, generator=g).contiguous(memory_format=torch.channels_last)
    out["seed"], out["x"] = np.array(51), _np(x)
    for i, p in enumerate(net.forward_refresh_reservoirs(x)["flow"]):
        out[f"y0_{i}"] = _np(p)
    for s in (1, 2, 3):
        d = _sparse_delta(g, x.shape, frac=0.1)
        out[f"d{s}"] = _np(d)
        for i, p in enumerate(net([d, None])["flow"]):
            out[f"dy{s}_{i}"] = _np(p if torch.is_tensor(p) else p[0])
    np.savez_compressed(os.path.join(OUT, "delayedevflownet_small.npz"), **out)
    # ---- ResNet-34 body (64x64) and dense object detector (191x255 -> 5x7 grid), batch-norm statistics seeded ----
    from maskedincrementeval_b200.synthetic import seeded_bn_stats
    for tag, net, shape, frac in (("resnet_small", ref.event_representation.ResnetIncr().eval(), (1, 3, 64, 64), 0.1),
                                  ("objdet_small", ref.obj_detection.DenseObjectDetIncr(2).eval(), (1, 2, 191, 255), 0.05)):
        out = {}
        net.load_state_dict(seeded_bn_stats(seeded_state_dict(_shapes(net), seed=61, init="kaiming_normal"), 62))
        x = (torch.randn(*shape, generator=g) * 4).round() / 4      # quarter steps: the fixture compresses
        x = x.contiguous(memory_format=torch.channels_last)
        out["seed"], out["bn_seed"], out["x"] = np.array(61), np.array(62), _np(x)
        out["y0"] = _np(net.forward_refresh_reservoirs(x))
        for s in (1, 2):
            d = _sparse_delta(g, x.shape, frac=frac)
            out[f"d{s}"], out[f"dy{s}"] = _np(d), _np(net([d, None])[0])
        np.savez_compressed(os.path.join(OUT, tag + ".npz"), **out)
    binning_golden(ref_root)
    print("wrote", sorted(f for f in os.listdir(OUT) if f.endswith(".npz")))


def binning_golden(ref_root: str):
    """Event binning of the reference's data fetchers (``data_fetchers/utils/util.py:62-110``): the voxel grid of
    ``events_to_voxel_grid_absT`` and the count image of ``event_histogram`` on seeded event windows, including
    polarity 0 (counted as -1 by the voxel grid, dropped by the histogram), a time stamp in the last bin and an empty
    window.  The module is loaded by path; ``np.int`` (removed from numpy 2, used at ``util.py:64-65``) is aliased to
    ``int`` for the call."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("ref_data_util", os.path.join(ref_root, "data_fetchers", "utils", "util.py"))
    util = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(util)
    if not hasattr(np, "int"):
        np.int = int
    from maskedincrementeval_b200.synthetic import EdgeEventStream
    out = {}
    h, w, bins = 40, 56, 5
    stream = EdgeEventStream(h, w, 3000, 6, seed=71)
    for i in range(3):
        ev = stream.window()                           # [n, 4]: t in [0, 1), x, y, p in {-1, +1}
        if i == 1:
            ev[:7, 3] = 0.0                            # polarity 0
            ev[7, 0] = 0.999999                        # lands in the last bin with almost all its weight
            ev[8, 0] = 0.0
        if i == 2:
            ev = ev[:0]                                # empty window
        out[f"ev{i}"] = ev.copy()
        ns = ev.copy()
        ns[:, 0] = ns[:, 0] * 1e9                      # the reference takes nanoseconds, a start time and a window length
        out[f"vox{i}"] = np.asarray(util.events_to_voxel_grid_absT(ns, bins, h, w, 1.0, 0.0), dtype=np.float32).copy()
        hist = util.event_histogram(ev.copy(), w, h) if ev.shape[0] else np.zeros((h, w, 2), np.float32)
        out[f"hist{i}"] = np.asarray(hist, dtype=np.float32)       # [H, W, 2] = (negative, positive)
    out["hwb"] = np.array([h, w, bins])
    np.savez_compressed(os.path.join(OUT, "binning.npz"), **out)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_ROOT)
