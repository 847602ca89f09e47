"""The CPU restatement against the golden vectors produced by the reference's own modules, and
against the live reference when a checkout is present (it is not on the GPU box)."""
import contextlib
import io

import numpy as np
import pytest
import torch

from maskedincrementeval_b200.synthetic import seeded_state_dict
from oracle import restatement as R
from oracle.reference_loader import E2DEPTH_CONFIG, load_reference, reference_available

T = torch.from_numpy


def close(a, b, tol=1e-6):
    a = T(a) if isinstance(a, np.ndarray) else a
    b = T(b) if isinstance(b, np.ndarray) else b
    scale = max(1.0, float(b.abs().max()))
    assert a.shape == b.shape
    assert float((a - b).abs().max()) <= tol * scale, float((a - b).abs().max())


@pytest.mark.parametrize("op", ["relu", "sigmoid", "tanh"])
@pytest.mark.parametrize("tag", ["3d", "4d"])
def test_activation_golden(golden, op, tag):
    g = golden("activation")
    k = lambda s: T(g[f"{op}_{tag}_{s}"])
    o1, r1 = R.act_incr(k("x"), k("d1"), op)
    # the reference's own test pins this identity exactly (tests/test_pointops.py:11-22)
    # (exact for relu and the reservoir; the CPU sigmoid/tanh take a vector or a scalar path depending on memory layout
    # and on how the threads partition the tensor, a difference of up to two ulp per call: 5e-7 covers both calls)
    o2, r2 = R.act_incr(r1, k("d2"), op)
    assert torch.equal(r1, k("r1")) and torch.equal(r2, k("r2"))
    if op == "relu":
        assert torch.equal(o1, k("o1")) and torch.equal(o2, k("o2"))
    else:
        close(o1, k("o1"), 5e-7)
        close(o2, k("o2"), 5e-7)


def test_product_golden(golden):
    g = golden("product")
    x1, x2 = T(g["x1"]), T(g["x2"])
    close(x1 * x2, g["y0"], 0)
    for s in (1, 2):
        o, x1, x2 = R.mul_incr(x1, T(g[f"da{s}"]), x2, T(g[f"db{s}"]))
        assert torch.equal(o, T(g[f"o{s}"]))
        assert torch.equal(x1, T(g[f"r1_{s}"])) and torch.equal(x2, T(g[f"r2_{s}"]))


@pytest.mark.parametrize("tag", ["ref_test", "k5s2", "k1", "k3s2", "k5s1"])
def test_conv_golden(golden, tag):
    g = golden("conv")
    cin, cout, k, s, p, h, w, n = (int(v) for v in g[f"{tag}_cfg"])
    wt, b = T(g[f"{tag}_w"]), T(g[f"{tag}_b"])
    close(R.conv_dense(T(g[f"{tag}_x"]), wt, b, s, p), g[f"{tag}_dense"], 1e-6)
    close(R.conv_delta(T(g[f"{tag}_dx"]), wt, s, p), g[f"{tag}_incr"], 1e-6)
    # delta conv == dense bias-free conv of the same tensor (tests/test_pointops.py:25-35)
    close(R.conv_delta(T(g[f"{tag}_x"]), wt, s, p), T(g[f"{tag}_dense"]) - b.view(1, -1, 1, 1), 1e-6)


def test_misc_ops_golden(golden):
    g = golden("misc_ops")
    carry = torch.zeros_like(T(g["kf_x"]))
    k = float(g["kf_k"])
    assert abs(k - 0.3 * float(torch.norm(T(g["kf_x"])))) < 1e-5
    for s in (1, 2, 3):
        q, carry = R.kfenced(carry, T(g[f"kf_d{s}"]), k)
        close(q, g[f"kf_q{s}"], 1e-6)
        close(carry, g[f"kf_c{s}"], 1e-5)
    close(R.bn_delta(T(g["bn_d"]), T(g["bn_var"]), T(g["bn_w"]), float(g["bn_eps"])), g["bn_o"], 1e-6)
    close(R.up2(T(g["up_d"])), g["up_o"], 1e-6)
    o, _ = R.maxpool_incr(T(g["mp_x"]), T(g["mp_d"]), 3, 2, 1)
    close(o, g["mp_o"], 1e-6)


def test_convlstm_golden(golden):
    g = golden("convlstm")
    shapes = {"Gates.weight": (24, 12, 3, 3), "Gates.bias": (24,)}
    sd = seeded_state_dict(shapes, seed=int(g["seed"]), init="kaiming_normal")
    cell = R.ConvLSTMOracle(sd["Gates.weight"], sd["Gates.bias"], "reference")
    h0, c0 = cell.refresh(T(g["x"]))
    close(h0, g["h0"], 1e-6)
    close(c0, g["c0"], 1e-6)
    for s in (1, 2):
        dh, dc = cell.step(T(g[f"d{s}"]))
        close(dh, g[f"dh{s}"], 2e-6)
        close(dc, g[f"dc{s}"], 2e-6)


def e2depth_shapes(base, bins=5, ne=3, nr=2):
    s = {}
    p = "unetrecurrent."

    def conv(name, co, ci, k):
        s[p + name + ".weight"] = (co, ci, k, k)
        s[p + name + ".bias"] = (co,)

    conv("head.conv2d", base, bins, 5)
    for i in range(ne):
        ci, co = base * 2 ** i, base * 2 ** (i + 1)
        conv(f"encoders.{i}.conv.conv2d", co, ci, 5)
        conv(f"encoders.{i}.recurrent_block.Gates", 4 * co, 2 * co, 3)
    cm = base * 2 ** ne
    for i in range(nr):
        conv(f"resblocks.{i}.conv1", cm, cm, 3)
        conv(f"resblocks.{i}.conv2", cm, cm, 3)
    for i in range(ne):
        ci = base * 2 ** (ne - i)
        conv(f"decoders.{i}.conv2d", ci // 2, ci, 5)
    conv("pred.conv2d", 1, base, 1)
    return s


def test_e2depth_golden(golden):
    g = golden("e2depth_small")
    sd = seeded_state_dict(e2depth_shapes(int(g["base"])), seed=int(g["seed"]), init="kaiming_normal")
    net = R.E2DepthOracle(sd, compat="reference")
    y0, st = net.refresh(T(g["x"]))
    close(y0, g["y0"], 1e-6)
    close(st[0][0], g["h0_0"], 1e-6)
    close(st[0][1], g["c0_0"], 1e-6)
    for s in (1, 2, 3):
        dy, sti = net.step(T(g[f"d{s}"]))
        close(dy, g[f"dy{s}"], 2e-6)
        close(sti[2][0], g[f"dh{s}_2"], 2e-6)


def test_e2depth_exact_tracks_dense(golden):
    """compat="exact": the accumulated incremental output equals a dense recompute."""
    g = golden("e2depth_small")
    sd = seeded_state_dict(e2depth_shapes(4), seed=21, init="kaiming_normal")
    net, dense = R.E2DepthOracle(sd, compat="exact"), R.E2DepthOracle(sd, compat="exact")
    x = T(g["x"])
    y, _ = net.refresh(x)
    for s in (1, 2, 3):
        x = x + T(g[f"d{s}"])
        y = y + net.step(T(g[f"d{s}"]))[0]
        yd, _ = dense.refresh(x)
        close(y, yd, 5e-6)


def flow_shapes_fire(base, bins=2, k=3):
    s = {}

    def conv(name, co, ci, kk):
        s[name + ".weight"] = (co, ci, kk, kk)
        s[name + ".bias"] = (co,)

    conv("E1.conv2d", base, bins, k)
    conv("E2.conv2d", base, base, k)
    conv("R1.conv1", base, base, 3)
    conv("R1.conv2", base, base, 3)
    conv("E3.conv2d", base, base, k)
    conv("R2.conv1", base, base, 3)
    conv("R2.conv2", base, base, 3)
    conv("pred.conv2d", 2, base, 1)
    return s


def flow_shapes_ev():
    s = {}

    def conv(name, co, ci, kk):
        s[name + ".weight"] = (co, ci, kk, kk)
        s[name + ".bias"] = (co,)

    enc_in, enc_out = [32, 64, 128, 256], [64, 128, 256, 512]
    for i in range(4):
        ci = 2 if i == 0 else enc_in[i]
        conv(f"encoders.{i}.conv.conv2d", enc_out[i], ci, 3)
        for gname in ("reset_gate", "update_gate", "out_gate"):
            conv(f"encoders.{i}.recurrent_block.{gname}", enc_out[i], 2 * enc_out[i], 3)
    for i in range(2):
        conv(f"resblocks.{i}.conv1", 512, 512, 3)
        conv(f"resblocks.{i}.conv2", 512, 512, 3)
    for i, (ci, co) in enumerate(zip(reversed(enc_out), reversed(enc_in))):
        conv(f"decoders.{i}.conv2d", co, 2 * ci + (0 if i == 0 else 2), 3)
    for i, co in enumerate(reversed(enc_in)):
        conv(f"preds.{i}.conv2d", 2, co, 1)
    return s


def flow_shapes_delayed(base=8, k=3, bins=2):
    s = {}

    def conv(name, co, ci, kk):
        s["multires_unet." + name + ".weight"] = (co, ci, kk, kk)
        s["multires_unet." + name + ".bias"] = (co,)

    enc_in = [base * 2 ** i for i in range(4)]
    enc_out = [base * 2 ** (i + 1) for i in range(4)]
    for i in range(4):
        conv(f"encoders.{i}.conv2d", enc_out[i], bins if i == 0 else enc_in[i], k)
    for i in range(2):
        conv(f"resblocks.{i}.conv1", enc_out[-1], enc_out[-1], 3)
        conv(f"resblocks.{i}.conv2", enc_out[-1], enc_out[-1], 3)
    for i, (ci, co) in enumerate(zip(reversed(enc_out), reversed(enc_in))):
        conv(f"decoders.{i}.conv2d", co, (2 if i == 0 else 1) * ci, k)
    for i, co in enumerate(reversed(enc_in)):
        conv(f"preds.{i}.conv2d", 2, co, 1)
    conv("delayed_pred_layer_list.0.conv2d", base, sum(enc_in[:-1]) + 8, 1)
    conv("delayed_pred_layer_list.1.conv2d", 2, base + 8, 1)
    return s


def _delayed_oracle(sd, compat):
    return R.DelayedEVFlowNetOracle({k.replace("multires_unet.", ""): v for k, v in sd.items()}, compat=compat)


def test_delayedevflownet_golden(golden):
    g = golden("delayedevflownet_small")
    sd = seeded_state_dict(flow_shapes_delayed(8), seed=int(g["seed"]), init="kaiming_normal")
    net = _delayed_oracle(sd, "reference")
    for i, p in enumerate(net.refresh(T(g["x"]))):
        close(p, g[f"y0_{i}"], 2e-6)
    for s in (1, 2, 3):
        for i, p in enumerate(net.step(T(g[f"d{s}"]))):
            close(p, g[f"dy{s}_{i}"], 5e-6)


def test_delayedevflownet_exact_tracks_dense(golden):
    g = golden("delayedevflownet_small")
    sd = seeded_state_dict(flow_shapes_delayed(8), seed=51, init="kaiming_normal")
    net, dense = _delayed_oracle(sd, "exact"), _delayed_oracle(sd, "exact")
    x = T(g["x"])
    ys = net.refresh(x)
    for s in (1, 2, 3):
        x = x + T(g[f"d{s}"])
        ys = [y + d for y, d in zip(ys, net.step(T(g[f"d{s}"])))]
        for y, yd in zip(ys, dense.refresh(x)):
            close(y, yd, 2e-5)


def bn_net_state(net_cls_or_shapes, g):
    """Seeded weights and batch-norm statistics of the ResNet / detector fixtures."""
    from maskedincrementeval_b200.synthetic import seeded_bn_stats
    return seeded_bn_stats(seeded_state_dict(net_cls_or_shapes, seed=int(g["seed"]), init="kaiming_normal"), int(g["bn_seed"]))


def resnet_shapes():
    s = {}

    def bn(p, c):
        s.update({p + ".weight": (c,), p + ".bias": (c,), p + ".running_mean": (c,), p + ".running_var": (c,),
                  p + ".num_batches_tracked": ()})

    s["conv1.weight"] = (64, 3, 7, 7)
    bn("bn1", 64)
    for si, (c, n, down) in enumerate(R.ResnetOracle.STAGES, 1):
        for bi in range(n):
            p = f"layer{si}.{bi}"
            first = down and bi == 0
            s[p + ".conv1.weight"] = (c, c // 2 if first else c, 3, 3)
            bn(p + ".bn1", c)
            s[p + ".conv2.weight"] = (c, c, 3, 3)
            bn(p + ".bn2", c)
            if first:
                s[p + ".downsample.0.weight"] = (c, c // 2, 1, 1)
                bn(p + ".downsample.1", c)
    s["fc.weight"], s["fc.bias"] = (1000, 512), (1000,)
    return s


def objdet_shapes(nr_classes=2, in_c=2, nr_box=2):
    s = {}

    def bn(p, c):
        s.update({p + ".weight": (c,), p + ".bias": (c,), p + ".running_mean": (c,), p + ".running_var": (c,),
                  p + ".num_batches_tracked": ()})

    ci = in_c
    for b, co in enumerate((16, 32, 64, 128, 256)):
        p = f"conv_layers.{b}"
        s[p + ".0.weight"] = (co, ci, 3, 3)
        bn(p + ".1", co)
        s[p + ".3.weight"] = (co, co, 3, 3)
        bn(p + ".4", co)
        ci = co
    s["conv_layers.5.weight"] = (512, 256, 3, 3)
    bn("conv_layers.6", 512)
    s["linear_1.weight"], s["linear_1.bias"] = (1024, 35 * 512), (1024,)
    per = 35 * (nr_classes + 5 * nr_box)
    s["linear_2.weight"], s["linear_2.bias"] = (per, 1024), (per,)
    return s


def rel_close(a, b, tol):
    a, b = torch.as_tensor(a), torch.as_tensor(b)
    scale = max(float(b.abs().max()), 1e-6)
    assert float((a - b).abs().max()) <= tol * scale, (float((a - b).abs().max()), scale)


@pytest.mark.parametrize("tag", ["resnet_small", "objdet_small"])
def test_bn_networks_golden(golden, tag):
    g = golden(tag)
    if tag == "resnet_small":
        net = R.ResnetOracle(bn_net_state(resnet_shapes(), g))
    else:
        net = R.DenseObjectDetOracle(bn_net_state(objdet_shapes(), g), nr_classes=2)
    # the fixture was computed on channels-last tensors, this runs contiguous ones: a different convolution algorithm of
    # the same CPU library, i.e. another summation order through up to 36 layers and a 17920-wide linear layer
    rel_close(net.refresh(T(g["x"])), g["y0"], 2e-5)
    for s in (1, 2):
        rel_close(net.step(T(g[f"d{s}"])), g[f"dy{s}"], 1e-4)


def test_fireflownet_golden(golden):
    g = golden("fireflownet_small")
    sd = seeded_state_dict(flow_shapes_fire(8), seed=int(g["seed"]), init="kaiming_normal")
    net = R.FireFlowNetOracle(sd, compat="reference")
    close(net.refresh(T(g["x"])), g["y0"], 1e-6)
    for s in (1, 2, 3):
        close(net.step(T(g[f"d{s}"])), g[f"dy{s}"], 2e-6)


def test_evflownet_golden(golden):
    g = golden("evflownet_small")
    sd = seeded_state_dict(flow_shapes_ev(), seed=int(g["seed"]), init="kaiming_normal")
    net = R.EVFlowNetOracle(sd, compat="reference")
    for i, p in enumerate(net.refresh(T(g["x"]))):
        close(p, g[f"y0_{i}"], 2e-6)
    for s in (1, 2):
        for i, p in enumerate(net.step(T(g[f"d{s}"]))):
            close(p, g[f"dy{s}_{i}"], 5e-6)


def test_flow_exact_tracks_dense(golden):
    g = golden("fireflownet_small")
    sd = seeded_state_dict(flow_shapes_fire(8), seed=31, init="kaiming_normal")
    net, dense = R.FireFlowNetOracle(sd, compat="exact"), R.FireFlowNetOracle(sd, compat="exact")
    x = T(g["x"])
    y = net.refresh(x)
    for s in (1, 2, 3):
        x = x + T(g[f"d{s}"])
        y = y + net.step(T(g[f"d{s}"]))
        close(y, dense.refresh(x), 2e-5)


def test_mask_definitions():
    d = torch.zeros(2, 3, 12, 20)
    d[0, 1, 0, 0] = 2e-3
    d[0, 2, 7, 8] = -5e-4
    d[1, 0, 11, 19] = 1.0
    m = R.pixel_mask(d, 1e-3)
    assert m.sum() == 2 and m[0, 0, 0, 0] == 1 and m[1, 0, 11, 19] == 1
    assert R.tile_list(m).tolist() == [0, 11]
    assert R.tile_list(R.pixel_mask(d, 0.0)).tolist() == [0, 1, 11]
    bits = R.tile_bits(m)
    assert bits[0, 0, 0] == 1 and bits[1, 1, 2] == 1 << (3 * 8 + 3)
    # a 3x3 convolution spreads an active corner pixel of a tile into the three neighbouring tiles
    c = torch.zeros(1, 1, 24, 24, dtype=torch.uint8)
    c[0, 0, 8, 8] = 1
    assert R.tile_list(R.conv_out_mask(c, 3, 1, 1)).tolist() == [0, 1, 3, 4]
    c[0, 0, 8, 8], c[0, 0, 12, 12] = 0, 1
    assert R.tile_list(R.conv_out_mask(c, 3, 1, 1)).tolist() == [4]


@pytest.mark.skipif(not reference_available(), reason="no reference checkout on this machine")
def test_live_reference_e2depth_and_flow():
    """Fresh seeds, not the committed vectors: the restatement against the reference run here."""
    ref = load_reference()
    torch.manual_seed(7)
    cfg = dict(E2DEPTH_CONFIG, base_num_channels=8)
    with contextlib.redirect_stdout(io.StringIO()):
        net = ref.e2depth.E2VIDRecurrentIncr(cfg).eval()
    sd = seeded_state_dict({k: tuple(v.shape) for k, v in net.state_dict().items()}, 99, "kaiming_normal")
    net.load_state_dict(sd)
    assert set(sd) == set(e2depth_shapes(8))
    orc = R.E2DepthOracle(sd, compat="reference")
    x = torch.randn(2, 5, 40, 56)
    with torch.no_grad():
        close(orc.refresh(x)[0], net.forward_refresh_reservoirs(x, None)[0], 1e-6)
        for _ in range(3):
            d = torch.randn_like(x) * (torch.rand(2, 1, 40, 56) < 0.1)
            close(orc.step(d)[0], net([d, None], None)[0][0], 2e-6)
        ev = ref.evflownet.MultiResUNetRecurrentIncr().eval()
        assert {k: tuple(v.shape) for k, v in ev.state_dict().items()} == flow_shapes_ev()


def test_host_binning_matches_reference_golden(golden):
    """``synthetic.events_to_voxel_grid`` / ``events_to_count_image`` against vectors the reference's own
    ``events_to_voxel_grid_absT`` / ``event_histogram`` (``data_fetchers/utils/util.py:62-110``) produced:
    bit for bit, including polarity 0, the last-bin time stamp and the empty window."""
    from maskedincrementeval_b200.synthetic import events_to_count_image, events_to_voxel_grid
    g = golden("binning")
    h, w, bins = (int(v) for v in g["hwb"])
    for i in range(3):
        ev = g[f"ev{i}"]
        assert np.array_equal(events_to_voxel_grid(ev.copy(), bins, h, w), g[f"vox{i}"])
        assert np.array_equal(events_to_count_image(ev.copy(), h, w), g[f"hist{i}"].transpose(2, 0, 1))
