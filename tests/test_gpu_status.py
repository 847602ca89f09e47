"""Device-side error status, thresholded layers and split precision of the convolution kernels.

None of these tests faults, traps or hangs the device: a bad tile-list entry is written from the host and must be
skipped; the bounded barrier wait is made to run out by a launch option that withholds the loads it waits for, with a
limit of a few hundred polls, after which the kernel returns by itself and the next launch must work.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import restatement as R  # noqa: E402


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def restore_config():
    from maskedincrementeval_b200 import _native as nat
    from maskedincrementeval_b200 import fields as fl
    saved = {k: getattr(fl.config, k) for k in ("threshold", "carry", "tensor_cores", "tc_thresholded", "compat", "own_tiles")}
    fl.config.own_tiles = False     # the hand-made tile lists of these tests are only read in list mode
    yield
    for k, v in saved.items():
        setattr(fl.config, k, v)
    nat.set_option(nat.OPT_TC_SPIN_LIMIT, 0)
    nat.set_option(nat.OPT_TC_WITHHOLD_LOADS, 0)
    nat.set_option(nat.OPT_TC_THRESHOLDED, 1)


def cl(t, dev):
    return t.to(dev).contiguous(memory_format=torch.channels_last)


def sparse_delta(g, shape, frac, std=0.5):
    n, c, h, w = shape
    act = (torch.rand(n, 1, h, w, generator=g) < frac).float()
    return torch.randn(shape, generator=g) * std * act


def _layer(dev, cin, cout, k, s, act, seed=0):
    from maskedincrementeval_b200.incr_modules.e2depth_incr import ConvLayerIncr
    torch.manual_seed(seed)
    return ConvLayerIncr(cin, cout, k, s, k // 2, activation=act).to(dev).eval()


# ------------------------------------------------------------------------------------------------
# counts[3]: a bad tile-list entry is skipped and reported; an expired wait is reported; the host raises
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("cfg", [("off", 16, 32, 3, 1), ("auto", 32, 32, 3, 1), ("auto", 64, 64, 3, 1), ("auto", 32, 64, 5, 2)])
def test_bad_tile_entry_is_skipped_and_reported(dev, cfg):
    """The second entry of a hand-made tile list is out of range: its slot is skipped (nothing is written for it), the
    tiles either side of it are computed as usual, counts[3] carries MIE_ERR_BAD_TILE, and check_device_errors raises."""
    from maskedincrementeval_b200 import _native as nat
    from maskedincrementeval_b200 import fields as fl
    from maskedincrementeval_b200.incr_modules.mask_incr_modules import check_device_errors
    mode, cin, cout, k, s = cfg
    fl.config.tensor_cores = mode
    n, h, w = 1, 48, 64
    layer = _layer(dev, cin, cout, k, s, "relu")
    conv = layer.conv2d
    g = torch.Generator().manual_seed(11)
    x0 = torch.randn(n, cin, h, w, generator=g)
    dx = sparse_delta(g, (n, cin, h, w), 1.0)
    with torch.no_grad():
        layer.forward_refresh_reservoirs(cl(x0, dev))
        dxd = cl(dx, dev)                                  # kept alive: the raw call below reads it again
        dy, m = layer([dxd, None])                         # a regular step: builds the plan, full activity
        assert conv.last_used_tensor_cores == (mode == "auto")
        want = dy.clone()
        plan = conv._plan(n, h, w, dev)
        ho, wo = plan.hout, plan.wout
        tw = -(-wo // 8)
        # same step again from the same state, through the C ABI, with a corrupted list
        layer.forward_refresh_reservoirs(cl(x0, dev))
        good = [0, 1, 2, tw + 1, 3]
        lst = torch.tensor([good[0], 10 ** 6, good[1], -7, good[2], good[3], 10 ** 6 + 1, good[4]], dtype=torch.int32, device=dev)
        plan.list[: lst.numel()] = lst
        plan.counts.copy_(torch.tensor([lst.numel(), 0, 0, 0], dtype=torch.int32))
        plan.out.zero_()
        plan.out_bits.zero_()
        a = plan.args
        nat.check(nat.lib.mie_conv_tiles(C.byref(a), nat.stream_ptr(dev)), "conv_tiles")
        torch.cuda.synchronize()
        assert int(plan.counts[3]) & nat.ERR_BAD_TILE
        assert not int(plan.counts[3]) & nat.ERR_WAIT_EXPIRED
        got = plan.out
        tol = 2e-3 if mode == "auto" else 1e-5
        covered = torch.zeros(1, 1, ho, wo, dtype=torch.bool)
        for t in good:
            ty, tx = divmod(t, tw)
            covered[:, :, ty * 8:ty * 8 + 8, tx * 8:tx * 8 + 8] = True
            a_, b_ = got[:, :, ty * 8:ty * 8 + 8, tx * 8:tx * 8 + 8], want[:, :, ty * 8:ty * 8 + 8, tx * 8:tx * 8 + 8]
            assert float((a_ - b_).abs().max()) <= tol * max(float(want.abs().max()), 1.0)
        assert float((got.cpu() * (~covered).float()).abs().max()) == 0.0      # nothing outside the five good tiles
        with pytest.raises(nat.MieError, match="outside the field"):
            check_device_errors(layer)
        assert int(plan.counts[3]) == 0                                         # cleared by the check
        check_device_errors(layer)                                              # and quiet afterwards


@pytest.mark.parametrize("own", [False, True], ids=["list", "own-tiles"])
@pytest.mark.parametrize("cfg", [(32, 32, 3, 1), (64, 64, 3, 1), (32, 64, 5, 2), (256, 256, 3, 1)])
def test_bounded_wait_expires_cleanly(dev, cfg, own):
    """With the loads withheld and a limit of 300 polls every tensor-core block with work gives up its first wait:
    the kernel returns, counts[3] carries MIE_ERR_WAIT_EXPIRED, the tensor memory is free again (the next launch of the
    same kernel runs and is correct), and the runner-level check raises."""
    from maskedincrementeval_b200 import _native as nat
    from maskedincrementeval_b200 import fields as fl
    from maskedincrementeval_b200.incr_modules.mask_incr_modules import check_device_errors
    cin, cout, k, s = cfg
    fl.config.tensor_cores, fl.config.own_tiles = "auto", own
    n, h, w = 1, 40, 56
    layer = _layer(dev, cin, cout, k, s, "relu")
    wt, b = layer.conv2d.weight.detach().cpu(), layer.conv2d.bias.detach().cpu()
    g = torch.Generator().manual_seed(5)
    x0 = torch.randn(n, cin, h, w, generator=g)
    with torch.no_grad():
        layer.forward_refresh_reservoirs(cl(x0, dev))
        res = R.conv_dense(x0, wt, b, s, k // 2)
        dx = sparse_delta(g, (n, cin, h, w), 0.3)
        nat.set_option(nat.OPT_TC_SPIN_LIMIT, 300)
        nat.set_option(nat.OPT_TC_WITHHOLD_LOADS, 1)
        layer([cl(dx, dev), None])
        assert layer.conv2d.last_used_tensor_cores
        torch.cuda.synchronize()                         # returns: nothing waits forever
        plan = layer.conv2d._plan(n, h, w, dev)
        assert int(plan.counts[3]) & nat.ERR_WAIT_EXPIRED
        with pytest.raises(nat.MieError, match="wait ran out"):
            check_device_errors(layer)
        nat.set_option(nat.OPT_TC_SPIN_LIMIT, 0)
        nat.set_option(nat.OPT_TC_WITHHOLD_LOADS, 0)
        # the aborted launch wrote no output and did not touch the reservoir: the same step now runs normally
        dy, m = layer([cl(dx, dev), None])
        torch.cuda.synchronize()
        want, _ = R.act_incr(res, R.conv_delta_tf32(dx, wt, s, k // 2), "relu")
        assert float((dy.cpu() - want).abs().max()) <= 2e-5 * max(float(want.abs().max()), 1.0)
        assert int(plan.counts[3]) == 0
        check_device_errors(layer)


def test_runner_check_names_the_layer(dev):
    from maskedincrementeval_b200 import _native as nat
    from maskedincrementeval_b200.incr_modules.fireflownet_incr import FireFlowNetIncr
    from maskedincrementeval_b200.runtime import IncrementalRunner
    net = FireFlowNetIncr(dict(base_num_channels=16, kernel_size=3, mask_output=False), 2, compat="exact").to(dev).eval()
    run = IncrementalRunner(net, use_graph=False)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(1, 2, 32, 40, generator=g)
    run.refresh(cl(x, dev))
    run.step(cl(x + sparse_delta(g, x.shape, 0.2), dev))
    run.check()
    plan = next(iter(net.E2.conv2d._plans.values()))
    plan.counts[3] = nat.ERR_BAD_TILE
    with pytest.raises(nat.MieError, match="E2.conv2d"):
        run.check()
    run.check()


# ------------------------------------------------------------------------------------------------
# thresholded layers: FP32 kernel by default, the deep-layer shapes of E2Depth
# ------------------------------------------------------------------------------------------------
DEEP = [
    # cin, cout, k, s, h, w, addend
    (256, 256, 3, 1, 33, 44, True),     # residual block convolution (with the residual sum)
    (256, 128, 5, 1, 66, 88, False),    # decoder 0 behind its upsample
    (128, 256, 5, 2, 66, 88, False),    # encoder 2
    (64, 128, 5, 2, 132, 176, False),   # encoder 1
]


def _thresholded_run(dev, cfg, tc_thresholded, steps=5, thr=0.02):
    """One thresholded layer with carry over a few partially active steps; returns per-step (delta, mask, total sent)."""
    from maskedincrementeval_b200 import fields as fl
    cin, cout, k, s, h, w, with_addend = cfg
    fl.config.threshold, fl.config.carry, fl.config.tc_thresholded = thr, True, tc_thresholded
    layer = _layer(dev, cin, cout, k, s, "relu", seed=3)
    g = torch.Generator().manual_seed(cin + cout + k + s)
    x0 = torch.randn(1, cin, h, w, generator=g) * 0.5
    out = []
    with torch.no_grad():
        pre = layer.conv2d.forward_refresh_reservoirs(cl(x0, dev))
        ho, wo = pre.shape[2:]
        r0 = torch.randn(1, cout, ho, wo, generator=g) * 0.3 if with_addend else None
        if with_addend:
            pre = pre + cl(r0, dev)
        layer.activation.forward_refresh_reservoirs(pre)
        sent = torch.relu(pre).clone()
        for step, frac in enumerate([0.05, 0.3, 0.0, 0.02, 1.0][:steps]):
            dx = sparse_delta(g, (1, cin, h, w), frac, std=0.1)
            addend = None
            if with_addend:
                addend = [cl(sparse_delta(g, (1, cout, ho, wo), frac * 0.5, std=0.05), dev), None]
            dy, m = layer(([cl(dx, dev), None]), addend)
            sent += dy
            out.append((dy.clone(), m.pixel_mask().clone(), sent.clone(), layer.conv2d.last_used_tensor_cores))
        truth = torch.relu(layer.activation.in_res.reservoir).clone()
        from maskedincrementeval_b200.incr_modules.mask_incr_modules import check_device_errors
        check_device_errors(layer)
    return out, truth


@pytest.mark.parametrize("cfg", DEEP)
def test_thresholded_deep_layers_fp32_routed(dev, cfg):
    """Default routing: a thresholded layer never takes the tensor-core kernels, even when the filter has a
    tensor-core copy; the FP32 kernel keeps the carry invariant (total sent within the threshold of the true output),
    withheld pixels are exact zeros and the mask is exactly the set of non-zero pixels."""
    from maskedincrementeval_b200 import fields as fl
    fl.config.tensor_cores = "auto"
    steps, truth = _thresholded_run(dev, cfg, tc_thresholded=False)
    for dy, pm, sent, used_tc in steps:
        assert not used_tc
        assert torch.equal(pm, (dy != 0).any(1, keepdim=True).to(torch.uint8))
    assert float((steps[-1][2] - truth).abs().max()) <= 0.02 + 1e-5


def test_thresholded_narrow_input_layer_on_fp32_kernel_is_plain_fp32(dev):
    """The 5-channel 5x5 head takes split precision on the tensor cores; with a threshold it is routed to the FP32
    kernel, which must then see the plain input and filter (the three channel blocks of the split only add up to the
    fp32 result under the tensor cores' truncation): identical output to the run with the tensor cores switched off."""
    from maskedincrementeval_b200 import fields as fl
    outs = []
    for mode in ("auto", "off"):
        fl.config.tensor_cores = mode
        steps, _ = _thresholded_run(dev, (5, 32, 5, 1, 40, 56, False), tc_thresholded=False, steps=4, thr=1e-3)
        assert not any(s[3] for s in steps)
        outs.append(steps)
    for a, b in zip(*outs):
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_thresholded_channel_count_off_a_power_of_two(dev):
    """96 output channels with a threshold: six groups of 16 channels, each decided on its own, on the FP32 kernel
    (three blocks of 32 channels) and on the tensor cores (blocks of 32): the carry invariant holds on both."""
    from maskedincrementeval_b200 import fields as fl
    fl.config.tensor_cores = "auto"
    for flag in (False, True):
        steps, truth = _thresholded_run(dev, (64, 96, 3, 1, 24, 40, False), tc_thresholded=flag, steps=4)
        assert all(s[3] == flag for s in steps)
        assert float((steps[-1][2] - truth).abs().max()) <= 0.02 + (2e-3 if flag else 1e-5)
        for dy, pm, _, _ in steps:
            assert torch.equal(pm, (dy != 0).any(1, keepdim=True).to(torch.uint8))


@pytest.mark.parametrize("channels", [72, 70, 8, 160])
@pytest.mark.parametrize("op", ["relu", "tanh"])
def test_thresholded_groups_match_oracle(dev, channels, op):
    """The send decision of a thresholded activation is per pixel and per group of 16 consecutive channels: values,
    pixel mask, reservoir and carry against the CPU restatement, on the float4 kernel (channel counts that are
    multiples of 4) and on the scalar one (70)."""
    from maskedincrementeval_b200 import fields as fl
    from maskedincrementeval_b200.incr_modules.mask_incr_modules import nnReservedActivation
    fl.config.carry = True
    thr = 0.05
    g = torch.Generator().manual_seed(channels)
    x = torch.randn(2, channels, 19, 27, generator=g)
    act = nnReservedActivation(getattr(torch, op), threshold=thr)
    with torch.no_grad():
        act.forward_refresh_reservoirs(cl(x, dev))
        res, em = x.clone(), R._OPS[op](x)
        groups_differ = False
        for step in range(8):
            dx = sparse_delta(g, x.shape, 0.3, std=0.04)
            dy, m = act([cl(dx, dev), None])
            want, wm, res, em = R.act_incr_thresholded(res, em, dx, op, thr)
            assert torch.equal(m.pixel_mask().cpu(), wm)
            assert float((dy.cpu() - want).abs().max()) <= 1e-5
            assert float((act.emitted.cpu() - em).abs().max()) <= 1e-5
            if channels > 16:
                g0, g1 = (want[:, :16] != 0).any(1), (want[:, 16:32] != 0).any(1)
                groups_differ |= bool((g0 != g1).any())
        assert channels <= 16 or groups_differ      # the groups of a pixel really are decided independently


@pytest.mark.parametrize("cfg", DEEP)
def test_thresholded_tensor_core_layers_against_fp32_kernel(dev, cfg):
    """Thresholded layers on the tensor cores (opt-in) at the deep-layer shapes of E2Depth, partially active, with carry
    and residual addend: same carry invariant as the FP32 kernel, pixel masks that differ only where a change sits within
    the TF32 error of the threshold, and a clean error word."""
    from maskedincrementeval_b200 import fields as fl
    fl.config.tensor_cores = "auto"
    a, ta = _thresholded_run(dev, cfg, tc_thresholded=True)
    b, tb = _thresholded_run(dev, cfg, tc_thresholded=False)
    assert all(s[3] for s in a) and not any(s[3] for s in b)
    assert float((a[-1][2] - ta).abs().max()) <= 0.02 + 2e-3
    differing = sum(int((x[1] != y[1]).sum()) for x, y in zip(a, b))
    total = sum(x[1].numel() for x in a)
    assert differing <= 0.01 * total, (differing, total)


@pytest.mark.parametrize("hidden", [16, 64])
def test_thresholded_convlstm_hidden_output(dev, hidden):
    """A thresholded ConvLSTM sends its hidden delta against what it has sent so far, in groups of 16 channels: the total
    sent stays within the threshold of the true hidden state (recomputed from the cell's own state), withheld groups
    are exact zeros, the hidden mask is the set of pixels with a sent group, and the cell state itself is not
    thresholded -- it follows the lossless cell exactly."""
    from maskedincrementeval_b200 import fields as fl
    from maskedincrementeval_b200.incr_modules.e2depth_incr import ConvLSTMIncr
    from maskedincrementeval_b200.synthetic import seeded_state_dict
    thr = 0.01
    fl.config.tensor_cores = "off"
    g = torch.Generator().manual_seed(hidden)
    cells = []
    for _ in range(2):
        cell = ConvLSTMIncr(hidden, hidden, 3).to(dev).eval()
        cell.compat = "exact"
        cell.load_state_dict(seeded_state_dict({k: tuple(v.shape) for k, v in cell.state_dict().items()}, 5, "kaiming_normal"))
        cells.append(cell)
    lossy, exact = cells
    x = torch.randn(2, hidden, 27, 35, generator=g)
    with torch.no_grad():
        h0, _ = lossy.forward_refresh_reservoirs(cl(x, dev), None)
        exact.forward_refresh_reservoirs(cl(x, dev), None)
        sent = h0.clone()
        withheld_some = False
        for step in range(8):
            dx = cl(sparse_delta(g, x.shape, 0.2, std=0.05), dev)
            fl.config.threshold, fl.config.carry = thr, True
            (dh, mh), (dc, mc) = lossy([dx, None], None)
            fl.config.threshold = 0.0
            (dh_e, _), (dc_e, _) = exact([dx, None], None)
            sent += dh
            C = hidden
            truth = torch.sigmoid(lossy._g[:, 2 * C:3 * C]) * torch.tanh(lossy._cell)
            assert float((sent - truth).abs().max()) <= thr + 1e-5
            assert float((dc - dc_e).abs().max()) <= 1e-6 and float((lossy._cell - exact._cell).abs().max()) <= 1e-6
            pm = mh.pixel_mask()
            assert torch.equal(pm, (dh != 0).any(1, keepdim=True).to(torch.uint8))
            withheld_some |= bool(((dh == 0).all(1, keepdim=True) & (dh_e != 0).any(1, keepdim=True)).any())
        assert withheld_some


def test_carry_survives_threshold_toggle(dev):
    """threshold 0.05 -> 0 -> 0.05: once a thresholded step has run, the carry buffer stays in use while the threshold
    is 0 (those steps send what is pending where they touch), so the total sent stays within the threshold of the true
    output throughout; a refresh under threshold 0 drops the buffer."""
    from maskedincrementeval_b200 import fields as fl
    fl.config.tensor_cores = "off"
    layer = _layer(dev, 16, 32, 3, 1, "tanh")
    g = torch.Generator().manual_seed(2)
    x0 = torch.randn(1, 16, 24, 32, generator=g)
    with torch.no_grad():
        sent = layer.forward_refresh_reservoirs(cl(x0, dev)).clone()
        for thr in (0.05, 0.05, 0.0, 0.0, 0.05, 0.05):
            fl.config.threshold = thr
            dy, _ = layer([cl(sparse_delta(g, x0.shape, 0.2, std=0.1), dev), None])
            sent += dy
            truth = torch.tanh(layer.activation.in_res.reservoir)
            assert float((sent - truth).abs().max()) <= 0.05 + 1e-5
            assert layer.activation.emitted is not None
        fl.config.threshold = 0.0
        layer.forward_refresh_reservoirs(cl(x0, dev))
        assert layer.activation.emitted is None
        fl.config.carry = False
        fl.config.threshold = 0.05
        layer([cl(sparse_delta(g, x0.shape, 0.2, std=0.1), dev), None])
        assert layer.activation.emitted is None


# ------------------------------------------------------------------------------------------------
# split precision on wide layers
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("cfg", [(32, 32, 3, 1, 40, 56), (64, 32, 3, 2, 32, 48), (130, 32, 3, 1, 24, 40), (32, 64, 5, 1, 24, 32)])
def test_split_precision_matches_fp32(dev, cfg):
    """precision="split": the tensor-core result is the fp32 convolution (2e-5 of the range), not the TF32 one."""
    from maskedincrementeval_b200 import fields as fl
    cin, cout, k, s, h, w = cfg
    fl.config.tensor_cores = "auto"
    layer = _layer(dev, cin, cout, k, s, "relu", seed=4)
    layer.conv2d.precision = "split"
    wt, b = layer.conv2d.weight.detach().cpu(), layer.conv2d.bias.detach().cpu()
    g = torch.Generator().manual_seed(7)
    x0 = torch.randn(1, cin, h, w, generator=g)
    with torch.no_grad():
        layer.forward_refresh_reservoirs(cl(x0, dev))
        res = R.conv_dense(x0, wt, b, s, k // 2)
        for frac in (0.1, 1.0, 0.0, 0.03):
            dx = sparse_delta(g, (1, cin, h, w), frac) * 4.0
            dy, m = layer([cl(dx, dev), None])
            assert layer.conv2d.last_used_tensor_cores
            want, _ = R.act_incr(res, R.conv_delta(dx, wt, s, k // 2), "relu")
            scale = max(float(want.abs().max()), 1.0)
            assert float((dy.cpu() - want).abs().max()) <= 2e-5 * scale, float((dy.cpu() - want).abs().max()) / scale
            res = layer.activation.in_res.reservoir.cpu().contiguous()
            pm = m.pixel_mask().cpu()
            assert float((dy.cpu() * (1 - pm.float())).abs().max()) == 0.0
