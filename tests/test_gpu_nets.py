"""Network-level parity on the GPU: ConvLSTM cell and the three incremental networks against the golden
vectors the reference produced (compat="reference") and against a dense recompute (compat="exact")."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from maskedincrementeval_b200.synthetic import seeded_state_dict  # noqa: E402
from oracle import restatement as R  # noqa: E402
from test_oracle import e2depth_shapes, flow_shapes_ev, flow_shapes_fire  # noqa: E402

T = torch.from_numpy


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.backends.cudnn.allow_tf32 = False   # dense refresh in full fp32, as eval_e2depth_continuous_inputs.py:3-4
    torch.backends.cuda.matmul.allow_tf32 = False
    return torch.device("cuda:0")


@pytest.fixture(autouse=True, params=["off", "auto"])
def tc_mode(request):
    """Every network test runs twice: FP32 kernels only (bar 1e-4 of the range) and with the tensor-core
    path enabled for the layers that qualify (bar 2e-3 of the range, TF32 inputs)."""
    from maskedincrementeval_b200 import fields as fl
    old = fl.config.tensor_cores
    fl.config.tensor_cores = request.param
    yield request.param
    fl.config.tensor_cores = old


def TOL():
    from maskedincrementeval_b200 import fields as fl
    return 1e-4 if fl.config.tensor_cores == "off" else 2e-3


def cl(t, dev):
    return t.to(dev).contiguous(memory_format=torch.channels_last)


def close(a, b, tol=1e-4, rng=None):
    a, b = a.detach().float().cpu(), b.detach().float().cpu()
    assert a.shape == b.shape, (a.shape, b.shape)
    rng = rng or max(float(b.max() - b.min()), 1e-6)
    err = float((a - b).abs().max())
    assert err <= tol * rng, (err, rng)


def sparse_delta(g, shape, frac, std=0.5):
    n, c, h, w = shape
    act = (torch.rand(n, 1, h, w, generator=g) < frac).float()
    return torch.randn(shape, generator=g) * std * act


def test_convlstm_golden(dev, golden):
    from maskedincrementeval_b200.incr_modules.e2depth_incr import ConvLSTMIncr
    g = golden("convlstm")
    cell = ConvLSTMIncr(6, 6, 3).to(dev).eval()
    cell.load_state_dict(seeded_state_dict({k: tuple(v.shape) for k, v in cell.state_dict().items()}, int(g["seed"]),
                                           "kaiming_normal"))
    with torch.no_grad():
        h0, c0 = cell.forward_refresh_reservoirs(cl(T(g["x"]), dev), None)
        close(h0, T(g["h0"]), 1e-5)
        close(c0, T(g["c0"]), 1e-5)
        for s in (1, 2):
            hid, cel = cell([cl(T(g[f"d{s}"]), dev), None], None)
            close(hid[0], T(g[f"dh{s}"]), TOL(), rng=float(T(g["h0"]).max() - T(g["h0"]).min()))
            close(cel[0], T(g[f"dc{s}"]), TOL(), rng=float(T(g["c0"]).max() - T(g["c0"]).min()))


def test_convlstm_state_feedback_exact(dev):
    """Feeding the returned state deltas back (no reference driver does) tracks the dense recurrence."""
    from maskedincrementeval_b200.incr_modules.e2depth_incr import ConvLSTMIncr
    g = torch.Generator().manual_seed(2)
    cell = ConvLSTMIncr(8, 8, 3).to(dev).eval()
    cell.compat = "exact"
    sd = seeded_state_dict({k: tuple(v.shape) for k, v in cell.state_dict().items()}, 5, "kaiming_normal")
    cell.load_state_dict(sd)
    orc = R.ConvLSTMOracle(sd["Gates.weight"], sd["Gates.bias"], "exact")
    x = torch.randn(1, 8, 24, 32, generator=g)
    with torch.no_grad():
        h, c = cell.forward_refresh_reservoirs(cl(x, dev), None)
        orc.refresh(x)
        st = ([h.clone(), None], [c.clone(), None])      # first step: delta against the zero state
        ost = (h.cpu().clone(), c.cpu().clone())
        for step in range(4):
            dx = sparse_delta(g, x.shape, 0.1)
            hid, cel = cell([cl(dx, dev), None], st)
            oh, oc = orc.step(dx, ost)
            close(hid[0], oh, TOL(), rng=2.0)
            close(cel[0], oc, TOL(), rng=2.0)
            st = ([hid[0].clone(), hid[1]], [cel[0].clone(), cel[1]])
            ost = (oh, oc)


def _e2depth(dev, base, seed, compat):
    from maskedincrementeval_b200.incr_modules.e2depth_incr import E2VIDRecurrentIncr
    net = E2VIDRecurrentIncr(dict(num_bins=5, num_encoders=3, base_num_channels=base, num_residual_blocks=2,
                                  skip_type="sum", norm=None, use_upsample_conv=True, compat=compat)).to(dev).eval()
    sd = seeded_state_dict(e2depth_shapes(base), seed, "kaiming_normal")
    net.load_state_dict(sd)
    return net, sd


def test_e2depth_golden_reference_compat(dev, golden):
    g = golden("e2depth_small")
    net, _ = _e2depth(dev, int(g["base"]), int(g["seed"]), "reference")
    with torch.no_grad():
        y0, st = net.forward_refresh_reservoirs(cl(T(g["x"]), dev), None)
        close(y0, T(g["y0"]), 1e-5)
        close(st[0][0], T(g["h0_0"]), 1e-5)
        rng = float(T(g["y0"]).max() - T(g["y0"]).min())
        for s in (1, 2, 3):
            dy, sti = net([cl(T(g[f"d{s}"]), dev), None], None)
            close(dy[0], T(g[f"dy{s}"]), TOL(), rng=rng)
            close(sti[2][0][0], T(g[f"dh{s}_2"]), TOL(), rng=1.0)


def test_e2depth_exact_drift_vs_dense_64_steps(dev):
    """compat="exact": accumulated incremental output vs dense recompute over 64 steps, 1e-4 of the range."""
    net, sd = _e2depth(dev, 8, 77, "exact")
    dense, _ = _e2depth(dev, 8, 77, "exact")
    g = torch.Generator().manual_seed(1)
    x = torch.randn(1, 5, 64, 96, generator=g)
    with torch.no_grad():
        y, _ = net.forward_refresh_reservoirs(cl(x, dev), None)
        y = y.clone()
        worst = 0.0
        for step in range(64):
            dx = sparse_delta(g, x.shape, 0.05)
            x = x + dx
            dy, _ = net([cl(dx, dev), None], None)
            y += dy[0]
            if step % 8 == 7 or step < 2:
                yd, _ = dense.forward_refresh_reservoirs(cl(x, dev), None)
                rng = float(yd.max() - yd.min())
                worst = max(worst, float((y - yd).abs().max()) / rng)
        assert worst <= TOL(), worst


def test_e2depth_batch_and_oracle_exact(dev):
    """Batch of 2 streams, odd-ish size (48x72), against the CPU oracle in exact mode."""
    net, sd = _e2depth(dev, 4, 13, "exact")
    orc = R.E2DepthOracle(sd, compat="exact")
    g = torch.Generator().manual_seed(4)
    x = torch.randn(2, 5, 48, 72, generator=g)
    with torch.no_grad():
        y, _ = net.forward_refresh_reservoirs(cl(x, dev), None)
        yo, _ = orc.refresh(x)
        close(y, yo, 1e-5)
        rng = float(yo.max() - yo.min())
        for step in range(3):
            dx = sparse_delta(g, x.shape, 0.05)
            dx[1] = 0  # one stream of the batch is idle
            dy, _ = net([cl(dx, dev), None], None)
            do, _ = orc.step(dx)
            close(dy[0], do, TOL(), rng=rng)
            assert float(dy[0][1].abs().max()) == 0.0


def test_fireflownet_golden_and_exact(dev, golden):
    from maskedincrementeval_b200.incr_modules.fireflownet_incr import FireFlowNetIncr
    g = golden("fireflownet_small")
    kw = dict(base_num_channels=8, kernel_size=3, mask_output=False)
    sd = seeded_state_dict(flow_shapes_fire(8), int(g["seed"]), "kaiming_normal")
    net = FireFlowNetIncr(kw, 2, compat="reference").to(dev).eval()
    net.load_state_dict(sd)
    with torch.no_grad():
        y0 = net.forward_refresh_reservoirs(cl(T(g["x"]), dev))["flow"][0]
        close(y0, T(g["y0"]), 1e-5)
        for s in (1, 2, 3):
            dy = net([cl(T(g[f"d{s}"]), dev), None])["flow"][0]
            close(dy[0], T(g[f"dy{s}"]), TOL(), rng=2.0)
        # exact wiring tracks a dense recompute
        ex = FireFlowNetIncr(kw, 2, compat="exact").to(dev).eval()
        de = FireFlowNetIncr(kw, 2, compat="exact").to(dev).eval()
        ex.load_state_dict(sd), de.load_state_dict(sd)
        x = T(g["x"])
        y = ex.forward_refresh_reservoirs(cl(x, dev))["flow"][0].clone()
        for s in (1, 2, 3):
            x = x + T(g[f"d{s}"])
            y += ex([cl(T(g[f"d{s}"]), dev), None])["flow"][0][0]
            close(y, de.forward_refresh_reservoirs(cl(x, dev))["flow"][0], TOL(), rng=2.0)


def test_recurrent_fireflownet_tracks_dense(dev):
    """FireFlowNet with two ConvGRU layers (the recurrent variant of the flow benchmark): accumulated incremental
    output against a dense recompute from the zero state, graph-replayed steps."""
    from maskedincrementeval_b200.incr_modules.fireflownet_incr import RecurrentFireFlowNetIncr
    from maskedincrementeval_b200.runtime import IncrementalRunner
    kw = dict(base_num_channels=32, kernel_size=3, mask_output=False)
    make = lambda: RecurrentFireFlowNetIncr(kw, 2, compat="exact").to(dev).eval()
    net, dense = make(), make()
    sd = seeded_state_dict({k: tuple(v.shape) for k, v in net.state_dict().items()}, 31, "default")
    net.load_state_dict(sd), dense.load_state_dict(sd)
    assert {"G1.update_gate.weight", "G2.out_gate.bias", "E1.conv2d.weight", "pred.conv2d.weight"} <= set(sd)
    g = torch.Generator().manual_seed(6)
    x = torch.randn(2, 2, 64, 88, generator=g).round()
    run = IncrementalRunner(net, use_graph=True)
    with torch.no_grad():
        run.refresh(cl(x, dev))
        for _ in range(8):
            x = x + sparse_delta(g, x.shape, 0.1, std=1.0).round()
            y = run.step(cl(x, dev))
        dense.reset_states()
        yd = dense.forward_refresh_reservoirs(cl(x, dev))["flow"][0]
    close(y, yd, TOL(), rng=2.0)
    assert run.graph_replays >= 6


def test_evflownet_golden(dev, golden):
    from maskedincrementeval_b200.incr_modules.evflownet_incr import MultiResUNetRecurrentIncr
    g = golden("evflownet_small")
    net = MultiResUNetRecurrentIncr(compat="reference").to(dev).eval()
    net.load_state_dict(seeded_state_dict(flow_shapes_ev(), int(g["seed"]), "kaiming_normal"))
    with torch.no_grad():
        for i, p in enumerate(net.forward_refresh_reservoirs(cl(T(g["x"]), dev))):
            close(p, T(g[f"y0_{i}"]), 1e-5, rng=2.0)
        for s in (1, 2):
            for i, p in enumerate(net([cl(T(g[f"d{s}"]), dev), None])):
                close(p[0], T(g[f"dy{s}_{i}"]), TOL(), rng=2.0)


def test_driver_protocol_with_graph_replay(dev):
    """The reference's driver loop (run_e2depth_continuous_dataset.py:55-74): refresh, then delta steps
    accumulated by the caller -- here with the step replayed as a CUDA graph."""
    from maskedincrementeval_b200.runtime import IncrementalRunner
    net, sd = _e2depth(dev, 8, 3, "exact")
    eager, _ = _e2depth(dev, 8, 3, "exact")
    g = torch.Generator().manual_seed(8)
    x = torch.randn(1, 5, 64, 96, generator=g)
    run = IncrementalRunner(net, use_graph=True)
    with torch.no_grad():
        y = run.refresh(cl(x, dev)).clone()
        ye, _ = eager.forward_refresh_reservoirs(cl(x, dev), None)
        ye = ye.clone()
        for step in range(5):
            x = x + sparse_delta(g, x.shape, 0.05)
            y = run.step(cl(x, dev))
            pass
        yd, _ = eager.forward_refresh_reservoirs(cl(x, dev), None)
        close(y, yd, TOL())
    assert run.graph_replays >= 3


def test_runner_state_feedback_tracks_dense_recurrence(dev):
    """IncrementalRunner(feedback=True): the state deltas of every step are fed to the next one (after a refresh, the
    dense states themselves), so the accumulated output follows the dense recurrent trajectory
    y_t, s_t = refresh(x_t, s_{t-1}) -- the protocol UNetRecurrentIncr.forward takes its prev_states_incr for
    (e2depth_incr.py:410-419), which none of the reference's drivers exercises.  Weights at twice the Kaiming scale so
    that the recurrent layers carry signal; a scheduled refresh in the middle continues the trajectory."""
    from maskedincrementeval_b200.incr_modules.e2depth_incr import E2VIDRecurrentIncr
    from maskedincrementeval_b200.runtime import IncrementalRunner
    cfg = dict(num_bins=5, num_encoders=3, base_num_channels=8, num_residual_blocks=2, skip_type="sum", norm=None,
               use_upsample_conv=True, compat="exact")
    sd = seeded_state_dict(e2depth_shapes(8), 9, "kaiming_normal", gain=2.0)
    net, dense = E2VIDRecurrentIncr(cfg).to(dev).eval(), E2VIDRecurrentIncr(cfg).to(dev).eval()
    net.load_state_dict(sd), dense.load_state_dict(sd)
    if TOL() > 1e-4:
        # signals of order one in every layer: plain TF32 inputs alone cost 2e-3 of the state range here
        from maskedincrementeval_b200.incr_modules.mask_incr_modules import set_precision
        set_precision(net, "split")
    g = torch.Generator().manual_seed(12)
    x = torch.randn(1, 5, 64, 96, generator=g)
    run = IncrementalRunner(net, use_graph=True, feedback=True, refresh_every=6)
    with torch.no_grad():
        y = run.refresh(cl(x, dev))
        yd, s = dense.forward_refresh_reservoirs(cl(x, dev), None)
        close(y, yd, 1e-6)
        worst, moved = 0.0, 0.0
        for step in range(10):
            x = x + sparse_delta(g, x.shape, 0.1)
            y = run.step(cl(x, dev))
            s_prev = [(h.clone(), c.clone()) for h, c in s]
            yd, s = dense.forward_refresh_reservoirs(cl(x, dev), s_prev)
            y0, _ = dense.forward_refresh_reservoirs(cl(x, dev), None)     # what the feedback-free protocol tracks
            rng = float(yd.max() - yd.min())
            worst = max(worst, float((y - yd).abs().max()) / rng)
            moved = max(moved, float((y0 - yd).abs().max()) / rng)
            for (h, c), (hr, cr) in zip(s, run._states):
                close(hr, h, TOL(), rng=2.0)
        assert worst <= TOL(), worst
        assert moved > max(10 * worst, 1e-3)   # the recurrent state matters here: without feedback the output differs
    assert run.graph_replays >= 4


def test_runner_step_host_matches_step(dev):
    """The pipelined host interface (uploads and downloads on side streams, no host wait) produces the outputs of
    the plain step() loop, and every step's prediction arrives in its pinned buffer."""
    from maskedincrementeval_b200.runtime import IncrementalRunner
    from maskedincrementeval_b200.synthetic import voxel_sequence
    frames = voxel_sequence(1, 64, 96, 7, 4000, 6, seed=3)
    net_a, net_b = _e2depth(dev, 8, 5, "exact")[0], _e2depth(dev, 8, 5, "exact")[0]
    ra, rb = IncrementalRunner(net_a, use_graph=True), IncrementalRunner(net_b, use_graph=True)
    pinned = [f.pin_memory() for f in frames]
    outs = [torch.empty(1, 1, 64, 96).pin_memory() for _ in frames]
    with torch.no_grad():
        ra.refresh(frames[0].to(dev))
        rb.refresh(frames[0].to(dev))
        want = []
        for f in frames[1:]:
            want.append(ra.step(f.to(dev)).clone())
        for i, f in enumerate(pinned[1:], 1):
            rb.step_host(f, outs[i])
        torch.cuda.synchronize()
    for i, w in enumerate(want, 1):
        assert torch.equal(outs[i], w.cpu())
    with pytest.raises(RuntimeError):
        rb.step_host(frames[1])   # not pinned


def test_runner_step_events_matches_host_binning(dev):
    """Feeding raw events (binned and reflection-padded on the device) gives the steps that host-binned voxel
    grids give; only the summation order of the binning differs."""
    import numpy as np
    import torch.nn.functional as F
    from maskedincrementeval_b200.runtime import IncrementalRunner
    from maskedincrementeval_b200.synthetic import EdgeEventStream, events_to_voxel_grid, reflection_pad_hw
    sh, sw, n_streams = 60, 90, 2
    l, r, t, b = reflection_pad_hw(sh, sw, 8)
    streams = [EdgeEventStream(sh, sw, 3000, 6, 40 + s) for s in range(n_streams)]
    net_a, net_b = _e2depth(dev, 8, 5, "exact")[0], _e2depth(dev, 8, 5, "exact")[0]
    ra, rb = IncrementalRunner(net_a, use_graph=True), IncrementalRunner(net_b, use_graph=True)

    def grid_of(evs):
        g = torch.from_numpy(np.stack([events_to_voxel_grid(e.copy(), 5, sh, sw) for e in evs], 0))
        return F.pad(g, (l, r, t, b), mode="reflect").contiguous(memory_format=torch.channels_last)

    with torch.no_grad():
        first = [s.window() for s in streams]
        ra.refresh(grid_of(first).to(dev))
        rb.refresh(grid_of(first).to(dev))
        for _ in range(5):
            evs = [s.window() for s in streams]
            ya = ra.step(grid_of(evs).to(dev))
            yb = rb.step_events([torch.from_numpy(e.astype("float32")).to(dev) for e in evs], (sh, sw))
            rng = float(ya.max() - ya.min())
            # FP32 path: only the order of the atomic adds differs; tensor-core path: those last-bit differences of
            # the input pass through the TF32 truncation of the layers
            bar = 1e-5 if TOL() <= 1e-4 else TOL()
            assert float((ya - yb).abs().max()) <= bar * max(rng, 1e-6)
    assert rb.graph_replays >= 3


def test_delayedevflownet_golden_and_dense(dev, golden):
    """The delayed-prediction EV-FlowNet: reference wiring against the golden vectors of the real reference,
    intended wiring against a dense recompute through the graph-replaying runner."""
    from maskedincrementeval_b200.incr_modules.delayedevflownet_incr import DelayedEVFlowNetIncr
    from maskedincrementeval_b200.runtime import IncrementalRunner
    from test_oracle import flow_shapes_delayed
    g = golden("delayedevflownet_small")
    kw = dict(base_num_channels=8, kernel_size=3, mask_output=False)
    sd = seeded_state_dict(flow_shapes_delayed(8), int(g["seed"]), "kaiming_normal")
    net = DelayedEVFlowNetIncr(kw, 2, compat="reference").to(dev).eval()
    net.load_state_dict(sd)
    with torch.no_grad():
        for i, p in enumerate(net.forward_refresh_reservoirs(cl(T(g["x"]), dev))["flow"]):
            close(p, T(g[f"y0_{i}"]), 1e-5)
        for s in (1, 2, 3):
            flows = net([cl(T(g[f"d{s}"]), dev), None])["flow"]
            for i, p in enumerate(flows):
                close(p[0], T(g[f"dy{s}_{i}"]), TOL(), rng=2.0)
                pm = p[1].pixel_mask().cpu()
                assert float((p[0].cpu() * (1 - pm.float())).abs().max()) == 0.0

    inc, dense = DelayedEVFlowNetIncr(kw, 2, compat="exact").to(dev).eval(), DelayedEVFlowNetIncr(kw, 2, compat="exact").to(dev).eval()
    inc.load_state_dict(sd), dense.load_state_dict(sd)
    run = IncrementalRunner(inc, use_graph=True)
    x = T(g["x"]).clone()
    gen = torch.Generator().manual_seed(3)
    with torch.no_grad():
        run.refresh(cl(x, dev))
        for _ in range(6):
            x = x + torch.randn(x.shape, generator=gen) * (torch.rand(1, 1, *x.shape[2:], generator=gen) < 0.1)
            ys = run.step(cl(x, dev))
        yds = dense.forward_refresh_reservoirs(cl(x, dev))["flow"]
    for y, yd in zip(ys, yds):
        close(y, yd, TOL(), rng=2.0)
    assert run.graph_replays >= 4


@pytest.mark.parametrize("tag", ["resnet_small", "objdet_small"])
def test_bn_networks_golden_and_dense(dev, golden, tag):
    """ResNet-34 body and the dense object detector (compositions of the operator classes; convolutions and
    activations on the kernels): golden vectors of the real reference, then accumulated output vs dense recompute."""
    from test_oracle import bn_net_state, objdet_shapes, resnet_shapes
    g = golden(tag)
    if tag == "resnet_small":
        from maskedincrementeval_b200.incr_modules.event_representation_incr import ResnetIncr
        make, sd = (lambda: ResnetIncr()), bn_net_state(resnet_shapes(), g)
    else:
        from maskedincrementeval_b200.incr_modules.obj_detection_incr import DenseObjectDetIncr
        make, sd = (lambda: DenseObjectDetIncr(2)), bn_net_state(objdet_shapes(), g)
    net, dense = make().to(dev).eval(), make().to(dev).eval()
    net.load_state_dict(sd), dense.load_state_dict(sd)
    # FP32 kernels: the project-wide 1e-4 bar.  Tensor cores: every one of the 11 / 36 convolutions in sequence truncates
    # its input delta to TF32 (1e-3 each, un-damped by any recurrence), so the network-level bar is 1e-2 here; the
    # operator-level tests pin the TF32 arithmetic itself.
    tol = 1e-4 if TOL() <= 1e-4 else 1e-2

    def rel(a, b, t):
        scale = max(float(b.abs().max()), 1e-6)
        assert float((a.cpu() - b.cpu()).abs().max()) <= t * scale, (float((a.cpu() - b.cpu()).abs().max()), scale)

    x = T(g["x"]).clone()
    with torch.no_grad():
        y = net.forward_refresh_reservoirs(cl(x, dev)).clone()
        rel(y, T(g["y0"]), 2e-5)       # dense refresh: cuDNN / cuBLAS in full fp32 against the CPU fixture
        for s in (1, 2):
            d = T(g[f"d{s}"])
            dy = net([cl(d, dev), None])[0]
            rel(dy, T(g[f"dy{s}"]), tol)
            x, y = x + d, y + dy
        rel(y, dense.forward_refresh_reservoirs(cl(x, dev)), tol)
