"""The benchmark configurations at their full sizes.  Where the CPU oracle would take minutes, the check is
the size-independent property of the path: the accumulated incremental output equals a dense recompute of
the same network on the same input (compat="exact"), and the delta buffers keep their zero invariant."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

from maskedincrementeval_b200.synthetic import (blob_delta_sequence, count_image_sequence, seeded_state_dict,  # noqa: E402
                                                voxel_sequence)
from oracle import restatement as R  # noqa: E402
from test_oracle import e2depth_shapes, flow_shapes_ev, flow_shapes_fire  # noqa: E402


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    return torch.device("cuda:0")


@pytest.fixture(autouse=True, params=["off", "auto"])
def tc_mode(request):
    from maskedincrementeval_b200 import fields as fl
    old = fl.config.tensor_cores
    fl.config.tensor_cores = request.param
    yield request.param
    fl.config.tensor_cores = old


def tol():
    from maskedincrementeval_b200 import fields as fl
    return 1e-4 if fl.config.tensor_cores == "off" else 2e-3


def rel_err(a, b):
    rng = max(float(b.max() - b.min()), 1e-6)
    return float((a - b).abs().max()) / rng


class Chain(torch.nn.Module):
    """Layer chain: conv3x3 32->64 stride 2, sigmoid, conv3x3 64->64, tanh, x2 nearest upsample, skip-add."""

    def __init__(self):
        super().__init__()
        from maskedincrementeval_b200.incr_modules.e2depth_incr import ConvLayerIncr
        from maskedincrementeval_b200.fields import Scratch
        self.c1 = ConvLayerIncr(32, 64, 3, 2, 1, activation="sigmoid")
        self.c2 = ConvLayerIncr(64, 64, 3, 1, 1, activation="tanh")
        self.sc = Scratch()

    def refresh(self, x, skip):
        y = self.c2.forward_refresh_reservoirs(self.c1.forward_refresh_reservoirs(x))
        return F.interpolate(y, scale_factor=2, mode="nearest") + skip

    def step(self, dx, dskip):
        from maskedincrementeval_b200 import _native as nat, fields as fl
        y, m = self.c2(self.c1([dx, None]))
        n, c, h, w = y.shape
        up = self.sc.get("up", (n, c, 2 * h, 2 * w), torch.float32, y.device, channels_last=True)
        ub = self.sc.get("up.bits", (fl.n_tiles(n, 2 * h, 2 * w),), torch.int64, y.device)
        mu = fl.upsample2x(y, m, None, None, up, ub, nat.UP_NEAREST)
        ds, ms = fl.resolve([dskip, None], self.sc, "skip")
        out = self.sc.get("out", (n, c, 2 * h, 2 * w), torch.float32, y.device, channels_last=True)
        ob = self.sc.get("out.bits", (fl.n_tiles(n, 2 * h, 2 * w),), torch.int64, y.device)
        return out, fl.add(up, mu, ds, ms, out, ob)


@pytest.mark.parametrize("frac", [0.01, 0.05, 0.20])
def test_config2_layer_chain_vs_oracle(dev, frac):
    """Batch 4, 260x346, drifting-blob deltas at 1 / 5 / 20 % active pixels, against the CPU oracle."""
    torch.manual_seed(0)
    net = Chain().to(dev).eval()
    sd = seeded_state_dict({k: tuple(v.shape) for k, v in net.state_dict().items()}, 3, "kaiming_normal")
    net.load_state_dict(sd)
    w1, b1, w2, b2 = sd["c1.conv2d.weight"], sd["c1.conv2d.bias"], sd["c2.conv2d.weight"], sd["c2.conv2d.bias"]
    g = torch.Generator().manual_seed(1)
    x = torch.randn(4, 32, 260, 346, generator=g)
    skip = torch.randn(4, 64, 260, 346, generator=g)
    cl = lambda t: t.to(dev).contiguous(memory_format=torch.channels_last)
    with torch.no_grad():
        y = net.refresh(cl(x), cl(skip)).clone()
        r1 = R.conv_dense(x, w1, b1, 2, 1)
        r2 = R.conv_dense(torch.sigmoid(r1), w2, b2, 1, 1)
        yo = F.interpolate(torch.tanh(r2), scale_factor=2, mode="nearest") + skip
        assert rel_err(y.cpu(), yo) <= tol()
        dxs = blob_delta_sequence(4, 32, 260, 346, 4, frac, seed=7)
        dss = blob_delta_sequence(4, 64, 260, 346, 4, frac, seed=8)
        for dx, ds in zip(dxs, dss):
            out, m = net.step(cl(dx), cl(ds))
            d1, r1 = R.act_incr(r1, R.conv_delta(dx.contiguous(), w1, 2, 1), "sigmoid")
            d2, r2 = R.act_incr(r2, R.conv_delta(d1, w2, 1, 1), "tanh")
            want = F.interpolate(d2, scale_factor=2, mode="nearest") + ds.contiguous()
            assert float((out.cpu() - want).abs().max()) <= tol() * 2.0   # tanh output range is 2
            pm = m.pixel_mask().cpu()
            assert float((out.cpu() * (1 - pm.float())).abs().max()) == 0.0
            # keep the oracle on the device's trajectory (sigmoid/tanh are smooth, this only stops TF32 drift compounding)
            r1 = net.c1.activation.in_res.reservoir.cpu().contiguous()
            r2 = net.c2.activation.in_res.reservoir.cpu().contiguous()


def _e2depth(dev, compat="exact"):
    from maskedincrementeval_b200.incr_modules.e2depth_incr import E2VIDRecurrentIncr
    net = E2VIDRecurrentIncr(dict(num_bins=5, num_encoders=3, base_num_channels=32, num_residual_blocks=2,
                                  skip_type="sum", norm=None, use_upsample_conv=True, compat=compat)).to(dev).eval()
    net.load_state_dict(seeded_state_dict(e2depth_shapes(32), 0, "default"))
    return net


@pytest.mark.parametrize("hw,streams,events,segs", [((260, 346), 1, 30000, 10), ((480, 640), 2, 80000, 15),
                                                     ((260, 346), 8, 30000, 10)])   # 8 streams: several work items per block
def test_config3_config4_e2depth_tracks_dense(dev, hw, streams, events, segs):
    """E2Depth at 260x346 (padded to 264x352) and 480x640, synthetic event voxel grids, graph-replayed steps."""
    from maskedincrementeval_b200.runtime import IncrementalRunner
    frames = [f.to(dev) for f in voxel_sequence(streams, hw[0], hw[1], 10, events, segs, seed=5)]
    net, dense = _e2depth(dev), _e2depth(dev)
    run = IncrementalRunner(net, use_graph=True)
    with torch.no_grad():
        run.refresh(frames[0])
        for f in frames[1:]:
            y = run.step(f)
        yd, _ = dense.forward_refresh_reservoirs(frames[-1], None)
    assert rel_err(y, yd) <= tol()
    assert run.graph_replays >= 7


def test_config5_flow_nets_track_dense(dev):
    """FireFlowNet (batch 2) and EVFlowNet (batch 1) at 256x336 on 2-channel event-count images, PyTorch's default
    convolution init (what the reference's random-init networks have).  With a unit-gain init (Kaiming normal) these
    un-normalised ReLU stacks amplify a 1e-3 relative perturbation of one layer to several per cent of the output, so
    the TF32 path cannot meet 2e-3 there whatever the kernel does (the FP32 path still meets 1e-4); the operator-level
    tests pin the TF32 arithmetic bit for bit instead."""
    from maskedincrementeval_b200.incr_modules.evflownet_incr import MultiResUNetRecurrentIncr
    from maskedincrementeval_b200.incr_modules.fireflownet_incr import FireFlowNetIncr
    from maskedincrementeval_b200.runtime import IncrementalRunner
    kw = dict(base_num_channels=32, kernel_size=3, mask_output=False)
    sd = seeded_state_dict(flow_shapes_fire(32), 2, "default")
    frames = [f.to(dev) for f in count_image_sequence(2, 256, 336, 8, 20000, 10, seed=9)]
    net, dense = FireFlowNetIncr(kw, 2, compat="exact").to(dev).eval(), FireFlowNetIncr(kw, 2, compat="exact").to(dev).eval()
    net.load_state_dict(sd), dense.load_state_dict(sd)
    run = IncrementalRunner(net, use_graph=True)
    with torch.no_grad():
        run.refresh(frames[0])
        for f in frames[1:]:
            y = run.step(f)
        yd = dense.forward_refresh_reservoirs(frames[-1])["flow"][0]
    assert rel_err(y, yd) <= tol()

    sd = seeded_state_dict(flow_shapes_ev(), 4, "default")
    frames = [f.to(dev) for f in count_image_sequence(1, 256, 336, 6, 20000, 10, seed=10)]
    net, dense = MultiResUNetRecurrentIncr(compat="exact").to(dev).eval(), MultiResUNetRecurrentIncr(compat="exact").to(dev).eval()
    net.load_state_dict(sd), dense.load_state_dict(sd)
    run = IncrementalRunner(net, use_graph=True)
    with torch.no_grad():
        run.refresh(frames[0])
        for f in frames[1:]:
            ys = run.step(f)
        dense.reset_states()
        yds = dense.forward_refresh_reservoirs(frames[-1])
    for y, yd in zip(ys, yds):
        assert rel_err(y, yd) <= tol()


def test_native_refresh_matches_library_refresh_full_size(dev):
    """The dense pass on the library's own kernels (dense-evaluation mode, every tile listed) against the same pass on
    PyTorch's dense operators, E2Depth at 264x352, from the zero state and from a given recurrent state: the
    prediction, the returned states and every layer's persistent state within 1e-5 of their range; afterwards every
    delta buffer is zero again, so the next incremental step starts clean."""
    from maskedincrementeval_b200 import fields as fl
    from maskedincrementeval_b200.incr_modules.mask_incr_modules import nnConvIncr
    from test_gpu_drift import layer_states
    frames = [f.to(dev) for f in voxel_sequence(1, 260, 346, 2, 30000, 10, seed=31)]
    nets = {}
    old = fl.config.refresh
    try:
        for how in ("native", "library"):
            fl.config.refresh = how
            net = _e2depth(dev)
            with torch.no_grad():
                y0, s0 = net.forward_refresh_reservoirs(frames[0], None)
                y1, s1 = net.forward_refresh_reservoirs(frames[1], [(h.clone(), c.clone()) for h, c in s0])
            nets[how] = (net, y0.clone(), y1.clone(), s1)
    finally:
        fl.config.refresh = old
    (na, ya0, ya1, sa), (nb, yb0, yb1, sb) = nets["native"], nets["library"]
    assert rel_err(ya0, yb0) <= 1e-5 and rel_err(ya1, yb1) <= 1e-5
    for (ha, ca), (hb, cb) in zip(sa, sb):
        assert rel_err(ha, hb) <= 1e-5 and rel_err(ca, cb) <= 1e-5
    la, lb = layer_states(na), layer_states(nb)
    assert la.keys() == lb.keys()
    for k in la:
        assert rel_err(la[k], lb[k]) <= 1e-5, k
    for m in na.modules():
        if isinstance(m, nnConvIncr):
            for plan in m._plans.values():
                assert float(plan.out.abs().max()) == 0.0 and int(plan.out_bits.abs().max()) == 0
