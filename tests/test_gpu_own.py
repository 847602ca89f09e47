"""Own-tiles mode of the tensor-core convolutions (``mie_conv_args.own_tiles``, ``config.own_tiles``): no tile list is
made by a launch in front of the convolution; every thread block tests the output tiles it owns against the input
words itself.  Outputs, tile words and reservoirs must equal the separate-dilation path to the bit over steps in which
tiles appear, go stale and come back, for every kernel variant; the scratch words must be zero again after every call."""
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
    from maskedincrementeval_b200 import _native as nat, fields as fl
    keys = ("threshold", "carry", "tensor_cores", "compat", "own_tiles", "head_dilation", "tail_dilation")
    saved = {k: getattr(fl.config, k) for k in keys}
    own_kernels = nat.get_option(nat.OPT_TC_OWN_KERNELS)
    nat.set_option(nat.OPT_TC_OWN_KERNELS, 15)      # every kernel variant, also the one the default leaves out
    yield
    for k, v in saved.items():
        setattr(fl.config, k, v)
    nat.set_option(nat.OPT_TC_OWN_KERNELS, own_kernels)
    fl.forget_tails()


def cl(t, dev):
    return t.to(dev).contiguous(memory_format=torch.channels_last)


def sparse(g, shape, frac, std=0.3):
    n, c, h, w = shape
    # activity in blobs, so that whole tiles switch on and off
    coarse = (torch.rand(n, 1, (h + 7) // 8, (w + 7) // 8, generator=g) < frac).float()
    act = torch.nn.functional.interpolate(coarse, size=(h, w), mode="nearest") * (torch.rand(n, 1, h, w, generator=g) < 0.5).float()
    return torch.randn(shape, generator=g) * std * act


# mode, cin, cout, k, stride, n, h, w, threshold, addend, launches in own mode, what it exercises
CASES = [
    ("auto", 32, 32, 3, 1, 1, 34, 44, 0.0, False, 1, "per-tap kernel, coalesced epilogue, one block per tile"),
    ("auto", 32, 32, 3, 1, 2, 130, 170, 0.0, False, 1, "the same with several work items per block"),
    ("auto", 64, 64, 3, 1, 1, 34, 44, 0.0, False, 1, "halo kernel, two issuers"),
    ("auto", 64, 32, 5, 1, 1, 264, 352, 0.0, False, 1, "halo kernel, five work items per block (decoder 2)"),
    ("auto", 32, 64, 5, 2, 1, 68, 88, 0.0, False, 1, "per-tap kernel, stride 2, direct epilogue"),
    ("auto", 128, 256, 3, 1, 1, 132, 176, 0.0, False, 1, "per-tap kernel with 256-channel blocks (gates 0)"),
    ("auto", 128, 512, 3, 1, 1, 66, 88, 0.0, False, 1, "two column blocks finish every tile: the word goes through the scratch"),
    ("auto", 256, 256, 3, 1, 1, 33, 44, 0.0, False, 1, "halo kernel as clusters of four, two column blocks"),
    ("auto", 256, 256, 3, 1, 1, 33, 44, 0.0, True, 1, "... with a residual addend (union mask)"),
    ("auto", 256, 256, 3, 1, 1, 17, 22, 0.02, False, 1, "... thresholded, with carry"),
    ("auto", 128, 256, 5, 2, 1, 66, 88, 0.0, False, 1, "per-tap kernel as clusters (encoder 2)"),
    ("auto", 64, 128, 5, 2, 1, 132, 176, 0.0, False, 1, "per-tap kernel as clusters of two (encoder 1)"),
    ("auto", 64, 64, 3, 1, 1, 34, 44, 0.02, False, 1, "halo kernel, thresholded"),
    ("off", 16, 32, 3, 1, 1, 34, 44, 0.0, False, 2, "FP32 kernel: the entry point enqueues the separate dilation"),
    ("off", 32, 1, 1, 1, 1, 34, 44, 0.0, False, 2, "1x1 head kernel: the same"),
]


def _run(dev, case, own):
    from maskedincrementeval_b200 import _native as nat, fields as fl
    from maskedincrementeval_b200.incr_modules.e2depth_incr import ConvLayerIncr
    from maskedincrementeval_b200.incr_modules.mask_incr_modules import check_device_errors
    mode, cin, cout, k, s, n, h, w, thr, with_addend, _, _ = case
    fl.config.tensor_cores, fl.config.threshold, fl.config.carry, fl.config.own_tiles = mode, thr, True, "always" if own else False
    torch.manual_seed(0)
    layer = ConvLayerIncr(cin, cout, k, s, k // 2, activation="relu").to(dev).eval()
    gg = torch.Generator().manual_seed(5)
    x0 = cl(torch.randn(n, cin, h, w, generator=gg), dev)
    res, counts = [], []
    with torch.no_grad():
        layer.forward_refresh_reservoirs(x0)
        ho, wo = fl.conv_out_hw(h, w, k, s, k // 2)
        for frac in (0.05, 0.5, 0.0, 0.02, 1.0, 0.1):
            d = cl(sparse(gg, (n, cin, h, w), frac), dev)
            m = fl.mask_from_delta(d)
            addend = None
            if with_addend:
                ad = cl(sparse(gg, (n, cout, ho, wo), frac * 0.5, std=0.05), dev)
                addend = [ad, fl.mask_from_delta(ad)]
            nat.reset_launch_count()
            y = layer([d, m], addend) if with_addend else layer([d, m])
            counts.append(nat.launch_count())
            plan = next(iter(layer.conv2d._plans.values()))
            res.append((y[0].clone(), y[1].bits.clone(), layer.activation.in_res.reservoir.clone(), plan.own_scratch.clone()))
        check_device_errors(layer)
    return res, counts, layer


@pytest.mark.parametrize("case", CASES, ids=[c[-1] for c in CASES])
def test_own_tiles_equals_the_separate_dilation(dev, case):
    own, own_counts, layer = _run(dev, case, True)
    sep, sep_counts, _ = _run(dev, case, False)
    for step, ((ya, ba, ra, sa), (yb, bb, rb, _)) in enumerate(zip(own, sep)):
        assert torch.equal(ba, bb), f"tile words differ at step {step}"
        assert torch.equal(ya, yb), f"output differs at step {step}"
        assert torch.equal(ra, rb), f"reservoir differs at step {step}"
        assert int(sa.abs().max()) == 0, f"scratch not returned to zero at step {step}"
    assert sep_counts == [2] * len(sep_counts), sep_counts
    assert own_counts == [case[10]] * len(own_counts), own_counts


def test_share_too_large_for_a_block_falls_back(dev):
    """8 x 480x640 on the halo kernel: 148 blocks would own 260 tiles each, more than a block's list holds -- the library
    enqueues the separate dilation itself; same bits."""
    case = ("auto", 64, 32, 3, 1, 8, 480, 640, 0.0, False, 2, "")
    own, own_counts, _ = _run(dev, case, True)
    sep, _, _ = _run(dev, case, False)
    for (ya, ba, ra, _), (yb, bb, rb, _) in zip(own, sep):
        assert torch.equal(ba, bb) and torch.equal(ya, yb) and torch.equal(ra, rb)
    assert own_counts == [2] * len(own_counts), own_counts


def test_own_tiles_needs_its_arguments(dev):
    """own_tiles without a job or without scratch is refused before anything is launched."""
    import ctypes as C
    from maskedincrementeval_b200 import _native as nat, fields as fl
    from maskedincrementeval_b200.incr_modules.e2depth_incr import ConvLayerIncr
    fl.config.tensor_cores, fl.config.own_tiles = "auto", True
    torch.manual_seed(0)
    layer = ConvLayerIncr(64, 64, 3, 1, 1, activation=None).to(dev).eval()
    g = torch.Generator().manual_seed(1)
    d = cl(sparse(g, (1, 64, 24, 32), 0.3), dev)
    with torch.no_grad():
        layer.forward_refresh_reservoirs(cl(torch.randn(1, 64, 24, 32, generator=g), dev))
        layer([d, None])
    plan = next(iter(layer.conv2d._plans.values()))
    a = plan.args
    assert a.own_tiles == 1
    keep = a.own_scratch
    a.own_scratch = None
    assert nat.lib.mie_conv_tiles(C.byref(a), nat.stream_ptr(dev)) == nat.EINVAL
    a.own_scratch = keep + 4                      # not 8-byte aligned
    assert nat.lib.mie_conv_tiles(C.byref(a), nat.stream_ptr(dev)) == nat.EINVAL
    a.own_scratch, head = keep, a.head
    a.head = None
    assert nat.lib.mie_conv_tiles(C.byref(a), nat.stream_ptr(dev)) == nat.EINVAL
    a.head = head
    torch.cuda.synchronize()


def test_network_step_without_dilation_launches(dev):
    """E2Depth at 128x160 through the runner (graph replay, recurrent state fed back): the same accumulated output to the
    bit over ten steps and a refresh, and one launch fewer per tensor-core convolution."""
    from maskedincrementeval_b200 import _native as nat, fields as fl
    from maskedincrementeval_b200.incr_modules.e2depth_incr import E2VIDRecurrentIncr
    from maskedincrementeval_b200.runtime import IncrementalRunner
    from maskedincrementeval_b200.synthetic import seeded_state_dict, voxel_sequence
    cfg = {"num_bins": 5, "skip_type": "sum", "recurrent_block_type": "convlstm", "num_encoders": 3, "base_num_channels": 32,
           "num_residual_blocks": 2, "use_upsample_conv": True, "norm": "none"}
    frames = [f.to(dev) for f in voxel_sequence(1, 128, 160, 14, 4000, 6, seed=3)]
    fl.config.compat = "exact"
    results, launches = [], []
    for own in (True, False):
        fl.config.own_tiles = own
        net = E2VIDRecurrentIncr(dict(cfg)).to(dev).eval()
        shapes = {k_: tuple(v.shape) for k_, v in net.state_dict().items()}
        net.load_state_dict(seeded_state_dict(shapes, seed=1))
        run = IncrementalRunner(net, use_graph=True, refresh_every=7)
        with torch.no_grad():
            run.refresh(frames[0])
            run.step(frames[1])
            nat.reset_launch_count()
            run.step(frames[2])
            launches.append(nat.launch_count())
            ys = [run.step(f).clone() for f in frames[3:]]
            run.check()
        results.append(ys)
    for a, b in zip(*results):
        assert torch.equal(a, b)
    assert launches[0] == launches[1] - 14, launches      # every convolution but the 1x1 prediction head


def test_default_leaves_the_clustered_halo_kernel_on_the_list(dev):
    """MIE_OPT_TC_OWN_KERNELS defaults to 7: the halo kernel as clusters keeps its dilation launch (it measured slower
    without), the other variants drop it; the option rejects values outside the mask."""
    from maskedincrementeval_b200 import _native as nat
    nat.set_option(nat.OPT_TC_OWN_KERNELS, 7)
    halo_cluster = ("auto", 256, 256, 3, 1, 1, 33, 44, 0.0, False, 2, "")
    halo = ("auto", 64, 64, 3, 1, 1, 34, 44, 0.0, False, 1, "")
    for case in (halo_cluster, halo):
        _, counts, layer = _run(dev, case, True)
        assert counts == [case[10]] * len(counts), counts
    assert layer.conv2d.last_cluster_size == 1
    with pytest.raises(Exception):
        nat.set_option(nat.OPT_TC_OWN_KERNELS, 16)
    assert nat.get_option(nat.OPT_TC_OWN_KERNELS) == 7


def test_random_shapes_equal_the_separate_dilation(dev):
    """Forty seeded random layers (kernel size, stride, widths, field size, batch, threshold, activation): whatever kernel
    the library picks for each, own-tiles mode gives the bits of the list path at every step."""
    import random
    rnd = random.Random(11)
    checked = 0
    for it in range(40):
        k = rnd.choice([3, 3, 5, 7, 1])
        s = rnd.choice([1, 1, 2])
        cin = rnd.choice([32, 48, 64, 96, 128, 256, 320])
        cout = rnd.choice([16, 32, 48, 64, 96, 128, 256, 512])
        h = rnd.choice([16, 24, 33, 34, 40, 66, 70, 96])
        w = rnd.choice([16, 22, 44, 48, 56, 88, 90, 120])
        if s == 2:
            h, w = h + (h & 1), w + (w & 1)
        n = rnd.choice([1, 1, 2, 3])
        thr = rnd.choice([0.0, 0.0, 0.0, 0.02])
        case = ("auto", cin, cout, k, s, n, h, w, thr, False, 0, "")
        own, _, layer = _run(dev, case, True)
        sep, _, _ = _run(dev, case, False)
        checked += bool(layer.conv2d.last_used_tensor_cores)
        for step, ((ya, ba, ra, sa), (yb, bb, rb, _)) in enumerate(zip(own, sep)):
            assert torch.equal(ba, bb) and torch.equal(ya, yb) and torch.equal(ra, rb), (case, step)
            assert int(sa.abs().max()) == 0, (case, step)
    assert checked >= 25      # most of them run on the tensor cores, where the mode exists
