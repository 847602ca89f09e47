"""The 1x1 prediction head's extras: a second input added as the kernel reads the first (the skip sum in front of the
prediction layer) and the accumulated prediction advanced inside the same kernel (the driver's ``c += c_incr``)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def restore_config():
    from maskedincrementeval_b200 import fields as fl
    saved = {k: getattr(fl.config, k) for k in ("threshold", "carry", "tensor_cores", "fuse_accumulate", "compat", "refresh")}
    yield
    for k, v in saved.items():
        setattr(fl.config, k, v)


def cl(t, dev):
    return t.to(dev).contiguous(memory_format=torch.channels_last)


def sparse(g, shape, frac):
    n, c, h, w = shape
    return torch.randn(shape, generator=g) * (torch.rand(n, 1, h, w, generator=g) < frac).float()


@pytest.mark.parametrize("cin,cout,act", [(32, 1, "sigmoid"), (30, 2, None), (64, 4, "tanh")])
def test_second_input_equals_the_sum(dev, cin, cout, act):
    """conv1x1(a, second=b) == conv1x1(a + b): values, mask, reservoir; also where only b is active."""
    from maskedincrementeval_b200 import fields as fl
    from maskedincrementeval_b200.incr_modules._algebra import INCR
    from maskedincrementeval_b200.incr_modules.e2depth_incr import ConvLayerIncr
    from maskedincrementeval_b200.fields import Scratch
    g = torch.Generator().manual_seed(cin)
    n, h, w = 2, 37, 52
    outs = []
    for fused in (True, False):
        torch.manual_seed(1)
        layer = ConvLayerIncr(cin, cout, 1, 1, 0, activation=act).to(dev).eval()
        gg = torch.Generator().manual_seed(5)
        x0 = cl(torch.randn(n, cin, h, w, generator=gg), dev)
        sc = Scratch()
        res = []
        with torch.no_grad():
            layer.forward_refresh_reservoirs(x0)
            for step in range(4):
                a = cl(sparse(gg, (n, cin, h, w), 0.03 if step != 1 else 0.0), dev)
                b = cl(sparse(gg, (n, cin, h, w), 0.03 if step != 2 else 0.0), dev)
                if fused:
                    y = INCR.conv(layer.conv2d, [a, None], layer.activation, second=[b, None])
                else:
                    y = INCR.conv(layer.conv2d, INCR.add([a, None], [b, None], sc, "sum"), layer.activation)
                r = layer.activation.in_res.reservoir.clone() if act else torch.zeros(1)
                res.append((y[0].clone(), y[1].pixel_mask().clone(), r))
        outs.append(res)
    for (ya, ma, ra), (yb, mb, rb) in zip(*outs):
        assert torch.equal(ma, mb)
        assert torch.equal(ya, yb) and torch.equal(ra, rb)
        assert float((ya * (1 - ma.float())).abs().max()) == 0.0


def test_runner_accumulates_in_the_head_kernel(dev):
    """E2Depth through IncrementalRunner with and without the head's extras: accumulated predictions equal to the
    bit, one launch fewer per step (the separate accumulation)."""
    from maskedincrementeval_b200 import _native as nat, fields as fl
    from maskedincrementeval_b200.incr_modules.e2depth_incr import E2VIDRecurrentIncr
    from maskedincrementeval_b200.runtime import IncrementalRunner
    from maskedincrementeval_b200.synthetic import seeded_state_dict, voxel_sequence
    cfg = {"num_bins": 5, "skip_type": "sum", "recurrent_block_type": "convlstm", "num_encoders": 3, "base_num_channels": 32,
           "num_residual_blocks": 2, "use_upsample_conv": True, "norm": "none"}
    frames = [f.to(dev) for f in voxel_sequence(1, 128, 160, 9, 4000, 6, seed=3)]
    fl.config.compat = "exact"
    results, launches = [], []
    for fuse in (True, False):
        fl.config.fuse_accumulate = fuse
        net = E2VIDRecurrentIncr(dict(cfg)).to(dev).eval()
        shapes = {k_: tuple(v.shape) for k_, v in net.state_dict().items()}
        net.load_state_dict(seeded_state_dict(shapes, seed=1))
        run = IncrementalRunner(net, use_graph=True, refresh_every=6)
        with torch.no_grad():
            run.refresh(frames[0])
            run.step(frames[1])
            nat.reset_launch_count()
            run.step(frames[2])          # the captured step
            launches.append(nat.launch_count())
            ys = [run.step(f).clone() for f in frames[3:]]     # includes a scheduled refresh
            run.check()
        results.append(ys)
    for a, b in zip(*results):
        assert torch.equal(a, b)
    assert launches[0] == launches[1] - 1, launches      # the separate accumulation launch is gone


def test_input_delta_kernel_writes_the_split_copy(dev):
    """mie_delta_mask with a split target == mie_delta_mask followed by mie_split_tf32, over steps in which tiles come
    and go (the copy must return to zero where the delta does)."""
    from maskedincrementeval_b200 import _native as nat, fields as fl
    g = torch.Generator().manual_seed(2)
    n, c, h, w = 1, 5, 45, 70
    half = 8
    st = nat.stream_ptr(dev)
    x = cl(torch.randn(n, c, h, w, generator=g), dev)
    prev = [x.clone(), x.clone()]
    dxs = [torch.zeros_like(x), torch.zeros_like(x)]
    bits = [fl.new_bits(n, h, w, dev), fl.new_bits(n, h, w, dev)]
    copies = [fl.new_field(n, 3 * half, h, w, dev), fl.new_field(n, 3 * half, h, w, dev)]
    cbits = [fl.new_bits(n, h, w, dev), fl.new_bits(n, h, w, dev)]
    for step in range(5):
        x = x + cl(sparse(g, (n, c, h, w), [0.02, 0.0, 0.3, 0.01, 0.0][step]), dev)
        # fused
        nat.check(nat.lib.mie_delta_mask(x.data_ptr(), fl.pixel_stride(x), prev[0].data_ptr(), fl.pixel_stride(prev[0]),
                                         dxs[0].data_ptr(), fl.pixel_stride(dxs[0]), bits[0].data_ptr(), n, c, h, w, 0.0,
                                         copies[0].data_ptr(), 3 * half, cbits[0].data_ptr(), None, st), "delta_mask")
        # two launches
        m = fl.delta_mask(x, prev[1], dxs[1], bits[1])
        fl.split_tf32(dxs[1], m, copies[1], cbits[1])
        assert torch.equal(dxs[0], dxs[1]) and torch.equal(bits[0], bits[1])
        assert torch.equal(copies[0], copies[1]) and torch.equal(cbits[0], cbits[1])
    assert float(copies[0].abs().max()) == 0.0     # the last step had no change anywhere


def test_quantiser_in_front_of_the_head_falls_back_to_the_sum(dev):
    """With the k-fenced quantiser switched on the prediction head takes the explicit sum (the quantiser acts on one
    input delta), the dense pass on the kernels still adds the second input on the fly; the network runs and tracks."""
    from maskedincrementeval_b200 import fields as fl
    from maskedincrementeval_b200.incr_modules.e2depth_incr import E2VIDRecurrentIncr
    from maskedincrementeval_b200.runtime import IncrementalRunner
    from maskedincrementeval_b200.synthetic import seeded_state_dict, voxel_sequence
    cfg = {"num_bins": 5, "skip_type": "sum", "recurrent_block_type": "convlstm", "num_encoders": 3, "base_num_channels": 8,
           "num_residual_blocks": 2, "use_upsample_conv": True, "norm": "none"}
    frames = [f.to(dev) for f in voxel_sequence(1, 64, 96, 5, 2000, 4, seed=3)]
    fl.config.compat = "exact"
    old = fl.config.kfenced_step
    fl.config.kfenced_step = 1e-4
    try:
        net = E2VIDRecurrentIncr(dict(cfg)).to(dev).eval()
        shapes = {k_: tuple(v.shape) for k_, v in net.state_dict().items()}
        net.load_state_dict(seeded_state_dict(shapes, seed=1))
        run = IncrementalRunner(net, use_graph=False)
        with torch.no_grad():
            run.refresh(frames[0])
            for f in frames[1:]:
                y = run.step(f)
            fl.config.kfenced_step = None
            yd = net.forward_refresh_reservoirs(frames[-1], None)[0]
        rng = float(yd.max() - yd.min())
        assert float((y - yd).abs().max()) <= 2e-2 * rng
    finally:
        fl.config.kfenced_step = old
