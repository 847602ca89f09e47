"""Tile dilations carried in the tail of the producing kernel (``mie_tail_job``).

A producer launched with a tail job must leave exactly what the producer followed by a separate ``mie_tiles_dilate``
launch leaves -- ordered tile list, stale list, counts, cleared output words, ticket back at zero -- and the tile lists
are checked against the CPU restatement as well.  At network level the pairing of producers and consumers must not
change a single bit of the output, only the number of launches.
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
    from maskedincrementeval_b200 import fields as fl
    saved = {k: getattr(fl.config, k) for k in ("threshold", "carry", "tensor_cores", "tail_dilation", "head_dilation", "compat",
                                                "own_tiles")}
    fl.config.own_tiles = False     # these tests compare with the separate dilation launch
    yield
    for k, v in saved.items():
        setattr(fl.config, k, v)


def cl(t, dev):
    return t.to(dev).contiguous(memory_format=torch.channels_last)


def sparse(g, shape, frac):
    n, c, h, w = shape
    return torch.randn(shape, generator=g) * (torch.rand(n, 1, h, w, generator=g) < frac).float()


class _Job:
    """Buffers of one dilation (as a convolution plan holds them) and the C structure that points at them."""

    def __init__(self, dev, in_bits, n, hin, win, k, s, p, union=None):
        from maskedincrementeval_b200 import _native as nat, fields as fl
        self.hout, self.wout = fl.conv_out_hw(hin, win, k, s, p)
        nt = fl.n_tiles(n, self.hout, self.wout)
        self.nt = nt
        self.list = torch.full((nt,), -1, dtype=torch.int32, device=dev)
        self.stale = torch.full((nt,), -1, dtype=torch.int32, device=dev)
        self.counts = torch.zeros(4, dtype=torch.int32, device=dev)
        self.flags = torch.zeros(nt, dtype=torch.uint8, device=dev)
        self.out_bits = torch.zeros(nt, dtype=torch.int64, device=dev)
        self.out_bits[::3] = 5          # every third output tile holds data from "last step"
        self.geo = (n, hin, win, self.hout, self.wout, k, s, p)
        self.in_bits, self.union = in_bits, union
        self.c = nat.TailJob(in_bits.data_ptr(), n, hin, win, self.hout, self.wout, k, s, p,
                             union.data_ptr() if union is not None else None, self.out_bits.data_ptr(),
                             self.list.data_ptr(), self.stale.data_ptr(), self.counts.data_ptr(), self.flags.data_ptr())

    def ptr(self):
        return C.addressof(self.c)

    def separate(self, dev):
        from maskedincrementeval_b200 import _native as nat
        n, hin, win, ho, wo, k, s, p = self.geo
        nat.check(nat.lib.mie_tiles_dilate(self.in_bits.data_ptr(), n, hin, win, ho, wo, k, s, p,
                                           self.union.data_ptr() if self.union is not None else None,
                                           self.out_bits.data_ptr(), self.list.data_ptr(), self.stale.data_ptr(),
                                           self.counts.data_ptr(), self.flags.data_ptr(), nat.stream_ptr(dev)), "dilate")

    def result(self):
        c = self.counts.cpu().tolist()
        return c, self.list[: c[0]].cpu().tolist(), self.stale[: c[1]].cpu().tolist(), self.out_bits.cpu().tolist()


def _same(a: _Job, b: _Job):
    ca, la, sa, oa = a.result()
    cb, lb, sb, ob = b.result()
    assert ca == cb and ca[2] == 0 and ca[3] == 0
    assert la == lb and sa == sb and oa == ob
    assert len(la) + len(sa) > 0


GEOS = [(3, 1, 1), (5, 2, 2), (5, 1, 2), (1, 1, 0)]


@pytest.mark.parametrize("k,s,p", GEOS)
def test_point_kernels_carry_the_dilation(dev, k, s, p):
    """add, concat, x2 upsample, input delta + mask, TF32 split (both variants): tail job == separate launch, and the
    tile list equals the restatement's."""
    from maskedincrementeval_b200 import _native as nat, fields as fl
    g = torch.Generator().manual_seed(7 * k + s)
    n, c, h, w = 2, 8, 45, 70
    st = nat.stream_ptr(dev)
    a, b = cl(sparse(g, (n, c, h, w), 0.01), dev), cl(sparse(g, (n, c, h, w), 0.01), dev)
    ma, mb = fl.mask_from_delta(a), fl.mask_from_delta(b)

    def run(launch, out_hw):
        """``launch(out_bits, tail_ptr)`` enqueues the producer; returns the two jobs (tail / separate)."""
        jobs = []
        for carried in (True, False):
            bits = fl.new_bits(n, out_hw[0], out_hw[1], dev)
            job = _Job(dev, bits, n, out_hw[0], out_hw[1], k, s, p)
            launch(bits, job.ptr() if carried else None)
            if not carried:
                job.separate(dev)
            jobs.append(job)
        _same(*jobs)
        return jobs[0]

    out = fl.new_field(n, c, h, w, dev)
    j = run(lambda bits, t: nat.check(nat.lib.mie_add(a.data_ptr(), c, ma.bits.data_ptr(), b.data_ptr(), c, mb.bits.data_ptr(),
                                                      out.data_ptr(), c, bits.data_ptr(), n, c, h, w, t, st), "add"), (h, w))
    act = ((a != 0).any(1, keepdim=True) | (b != 0).any(1, keepdim=True)).cpu().to(torch.uint8)
    assert j.result()[1] == R.tile_list(R.conv_out_mask(act, k, s, p)).tolist()

    out2 = fl.new_field(n, 2 * c, h, w, dev)
    run(lambda bits, t: nat.check(nat.lib.mie_cat2(a.data_ptr(), c, ma.bits.data_ptr(), c, b.data_ptr(), c, mb.bits.data_ptr(), c,
                                                   out2.data_ptr(), 2 * c, bits.data_ptr(), n, h, w, t, st), "cat2"), (h, w))
    up = fl.new_field(n, c, 2 * h, 2 * w, dev)
    run(lambda bits, t: nat.check(nat.lib.mie_upsample2x(a.data_ptr(), c, ma.bits.data_ptr(), b.data_ptr(), c, mb.bits.data_ptr(),
                                                         up.data_ptr(), c, bits.data_ptr(), n, c, h, w, nat.UP_BILINEAR, t, st),
                                  "upsample2x"), (2 * h, 2 * w))
    for cc in (8, 5):   # float4 and scalar variants of the split kernel
        x = cl(sparse(g, (n, cc, h, w), 0.02), dev)
        mx = fl.mask_from_delta(x)
        half = (cc + 7) // 8 * 8
        o3 = fl.new_field(n, 3 * half, h, w, dev)
        run(lambda bits, t: nat.check(nat.lib.mie_split_tf32(x.data_ptr(), fl.pixel_stride(x), mx.bits.data_ptr(), cc, o3.data_ptr(),
                                                             3 * half, bits.data_ptr(), n, h, w, t, st), "split"), (h, w))
    x0 = cl(torch.randn(n, 5, h, w, generator=g), dev)
    x1 = x0 + cl(sparse(g, (n, 5, h, w), 0.02), dev)
    jobs = []
    for carried in (True, False):
        prev, dx = x0.clone(), torch.zeros_like(x0)
        bits = fl.new_bits(n, h, w, dev)
        job = _Job(dev, bits, n, h, w, k, s, p)
        nat.check(nat.lib.mie_delta_mask(x1.data_ptr(), fl.pixel_stride(x1), prev.data_ptr(), fl.pixel_stride(prev),
                                         dx.data_ptr(), fl.pixel_stride(dx), bits.data_ptr(), n, 5, h, w, 0.0, None, 0, None,
                                         job.ptr() if carried else None, st), "delta_mask")
        if not carried:
            job.separate(dev)
        jobs.append(job)
    _same(*jobs)


def test_tail_job_with_union_mask_and_rejections(dev):
    """A union mask (the residual addend's) is honoured; a job that does not read the words the call writes is refused;
    a job too large for one block is run as a separate launch by the entry point itself."""
    from maskedincrementeval_b200 import _native as nat, fields as fl
    g = torch.Generator().manual_seed(3)
    n, c, h, w = 1, 8, 40, 56
    st = nat.stream_ptr(dev)
    a, b = cl(sparse(g, (n, c, h, w), 0.01), dev), cl(sparse(g, (n, c, h, w), 0.01), dev)
    ma, mb = fl.mask_from_delta(a), fl.mask_from_delta(b)
    u = fl.mask_from_delta(cl(sparse(g, (n, c, h, w), 0.01), dev))
    out = fl.new_field(n, c, h, w, dev)
    jobs = []
    for carried in (True, False):
        bits = fl.new_bits(n, h, w, dev)
        job = _Job(dev, bits, n, h, w, 3, 1, 1, union=u.bits)
        nat.check(nat.lib.mie_add(a.data_ptr(), c, ma.bits.data_ptr(), b.data_ptr(), c, mb.bits.data_ptr(), out.data_ptr(), c,
                                  bits.data_ptr(), n, c, h, w, job.ptr() if carried else None, st), "add")
        if not carried:
            job.separate(dev)
        jobs.append(job)
    _same(*jobs)
    # wrong words
    other = fl.new_bits(n, h, w, dev)
    bad = _Job(dev, other, n, h, w, 3, 1, 1)
    bits = fl.new_bits(n, h, w, dev)
    assert nat.lib.mie_add(a.data_ptr(), c, ma.bits.data_ptr(), b.data_ptr(), c, mb.bits.data_ptr(), out.data_ptr(), c,
                           bits.data_ptr(), n, c, h, w, bad.ptr(), st) == nat.EINVAL
    # more output tiles than one block takes: same result through the entry point's own separate launch
    n2, h2, w2 = 2, 264, 352
    a2, b2 = cl(sparse(g, (n2, 4, h2, w2), 0.001), dev), cl(sparse(g, (n2, 4, h2, w2), 0.001), dev)
    m2a, m2b = fl.mask_from_delta(a2), fl.mask_from_delta(b2)
    o2 = fl.new_field(n2, 4, h2, w2, dev)
    assert fl.n_tiles(n2, h2, w2) > nat.TAIL_MAX_TILES
    jobs = []
    for carried in (True, False):
        bits = fl.new_bits(n2, h2, w2, dev)
        job = _Job(dev, bits, n2, h2, w2, 5, 1, 2)
        nat.reset_launch_count()
        nat.check(nat.lib.mie_add(a2.data_ptr(), 4, m2a.bits.data_ptr(), b2.data_ptr(), 4, m2b.bits.data_ptr(), o2.data_ptr(), 4,
                                  bits.data_ptr(), n2, 4, h2, w2, job.ptr() if carried else None, st), "add")
        assert nat.launch_count() == (2 if carried else 1)
        if not carried:
            job.separate(dev)
        jobs.append(job)
    _same(*jobs)


@pytest.mark.parametrize("cfg", [("off", 16, 32, 3, 1), ("auto", 32, 32, 3, 1), ("auto", 64, 64, 3, 1), ("auto", 32, 64, 5, 2),
                                 ("off", 32, 1, 1, 1)])
def test_convolution_kernels_carry_the_dilation(dev, cfg):
    """FP32 kernel, 1x1 kernel, per-tap and halo tensor-core kernels as producers: two chained layers give the same
    bits with and without the pairing, and the second layer's launch disappears from the count."""
    from maskedincrementeval_b200 import _native as nat, fields as fl
    from maskedincrementeval_b200.incr_modules.e2depth_incr import ConvLayerIncr
    mode, cin, cout, k, s = cfg
    fl.config.tensor_cores = mode
    g = torch.Generator().manual_seed(11)
    n, h, w = 1, 48, 72
    outs, counts = [], []
    fl.config.head_dilation = 0          # compare with the separate launch, not with the in-kernel dilation
    for tails in (True, False):
        fl.config.tail_dilation = tails
        torch.manual_seed(0)
        l1 = ConvLayerIncr(cin, cout, k, s, k // 2, activation="relu").to(dev).eval()
        l2 = ConvLayerIncr(cout, 32, 3, 1, 1, activation="relu").to(dev).eval()
        gg = torch.Generator().manual_seed(5)
        x0 = cl(torch.randn(n, cin, h, w, generator=gg), dev)
        with torch.no_grad():
            l2.forward_refresh_reservoirs(l1.forward_refresh_reservoirs(x0))
            res = []
            for step in range(4):
                d = cl(sparse(gg, (n, cin, h, w), 0.02 if step != 2 else 0.0), dev)
                nat.reset_launch_count()
                y = l2(l1([d, None]))
                counts.append(nat.launch_count())
                res.append((y[0].clone(), y[1].bits.clone()))
        outs.append(res)
    for (ya, ba), (yb, bb) in zip(*outs):
        assert torch.equal(ya, yb) and torch.equal(ba, bb)
    with_tails, without = counts[:4], counts[4:]
    assert with_tails[0] == without[0]                      # first step: the consumer dilates and offers the job
    assert all(a == b - 1 for a, b in zip(with_tails[1:], without[1:]))


def test_network_step_is_bit_identical_and_shorter(dev):
    """E2Depth at 128x160: same accumulated output to the bit with carried dilations, a third fewer launches."""
    from maskedincrementeval_b200 import _native as nat, fields as fl
    from maskedincrementeval_b200.incr_modules.e2depth_incr import E2VIDRecurrentIncr
    from maskedincrementeval_b200.runtime import IncrementalRunner
    from maskedincrementeval_b200.synthetic import seeded_state_dict, voxel_sequence
    cfg = {"num_bins": 5, "skip_type": "sum", "recurrent_block_type": "convlstm", "num_encoders": 3, "base_num_channels": 32,
           "num_residual_blocks": 2, "use_upsample_conv": True, "norm": "none"}
    frames = [f.to(dev) for f in voxel_sequence(1, 128, 160, 8, 4000, 6, seed=3)]
    fl.config.compat = "exact"
    fl.config.head_dilation = 0
    results, launches = [], []
    for tails in (True, False):
        fl.config.tail_dilation = tails
        net = E2VIDRecurrentIncr(dict(cfg)).to(dev).eval()
        shapes = {k_: tuple(v.shape) for k_, v in net.state_dict().items()}
        net.load_state_dict(seeded_state_dict(shapes, seed=1))
        run = IncrementalRunner(net, use_graph=True)
        with torch.no_grad():
            run.refresh(frames[0])
            run.step(frames[1])
            nat.reset_launch_count()
            run.step(frames[2])          # the captured step
            launches.append(nat.launch_count())
            for f in frames[3:]:
                run.step(f)
            run.check()
            results.append(run.output.clone())
    assert torch.equal(results[0], results[1])
    assert launches[0] <= launches[1] - 12, launches


def test_consumer_that_skips_a_step_starts_clean(dev):
    """The producer runs twice before its consumer runs again: the pairing is dissolved and the consumer's output
    still obeys the zero invariant and equals the unpaired result."""
    from maskedincrementeval_b200 import fields as fl
    from maskedincrementeval_b200.incr_modules.e2depth_incr import ConvLayerIncr
    fl.config.tensor_cores = "off"
    n, cin, h, w = 1, 16, 40, 56
    outs = []
    for tails in (True, False):
        fl.config.tail_dilation = tails
        torch.manual_seed(0)
        l1 = ConvLayerIncr(cin, 32, 3, 1, 1, activation="relu").to(dev).eval()
        l2 = ConvLayerIncr(32, 32, 3, 1, 1, activation=None).to(dev).eval()
        gg = torch.Generator().manual_seed(9)
        x0 = cl(torch.randn(n, cin, h, w, generator=gg), dev)
        ds = [cl(sparse(gg, (n, cin, h, w), 0.03), dev) for _ in range(5)]
        with torch.no_grad():
            l2.forward_refresh_reservoirs(l1.forward_refresh_reservoirs(x0))
            l2(l1([ds[0], None]))
            l2(l1([ds[1], None]))
            l1([ds[2], None])                 # the consumer sits this step out ...
            y_late = l1([ds[3], None])        # ... and the producer runs again before it returns
            y = l2(y_late)
            outs.append((y[0].clone(), y[1].pixel_mask().clone()))
    (ya, pa), (yb, pb) = outs
    assert torch.equal(pa, pb) and torch.equal(ya, yb)
    assert float((ya * (1 - pa.float())).abs().max()) == 0.0


def test_feedback_runner_with_changing_inputs_is_bit_identical(dev):
    """With recurrent-state feedback the gate convolution reads the encoder output on the first step and the
    concatenation [encoder output, previous hidden delta] afterwards: the job offered under the first input is withdrawn
    when the plan changes to the second, and the trajectory equals the unpaired one to the bit."""
    from maskedincrementeval_b200 import fields as fl
    from maskedincrementeval_b200.incr_modules.e2depth_incr import E2VIDRecurrentIncr
    from maskedincrementeval_b200.runtime import IncrementalRunner
    from maskedincrementeval_b200.synthetic import seeded_state_dict
    cfg = dict(num_bins=5, num_encoders=3, base_num_channels=8, num_residual_blocks=2, skip_type="sum", norm=None,
               use_upsample_conv=True, compat="exact")
    fl.config.tensor_cores = "off"
    outs = []
    for tails in (True, False):
        fl.config.tail_dilation = tails
        net = E2VIDRecurrentIncr(dict(cfg)).to(dev).eval()
        shapes = {k_: tuple(v.shape) for k_, v in net.state_dict().items()}
        net.load_state_dict(seeded_state_dict(shapes, 9, "kaiming_normal", gain=2.0))
        g = torch.Generator().manual_seed(12)
        x = torch.randn(1, 5, 64, 96, generator=g)
        run = IncrementalRunner(net, use_graph=True, feedback=True, refresh_every=6)
        ys = []
        with torch.no_grad():
            run.refresh(cl(x, dev))
            for step in range(10):
                x = x + sparse(g, x.shape, 0.1)
                ys.append(run.step(cl(x, dev)).clone())
        outs.append(ys)
    for a, b in zip(*outs):
        assert torch.equal(a, b)


# ------------------------------------------------------------------------------------------------
# head jobs: the convolution kernel's first block runs the convolution's own dilation
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("cfg", [("off", 16, 32, 3, 1), ("auto", 32, 32, 3, 1), ("auto", 64, 64, 3, 1), ("auto", 32, 64, 5, 2),
                                 ("off", 32, 1, 1, 1), ("auto", 256, 256, 3, 1), ("auto", 128, 256, 5, 2)])
def test_convolution_kernels_run_their_own_dilation(dev, cfg):
    """FP32, 1x1, per-tap, halo and both cluster kernels: identical output bits with the dilation inside the kernel and
    as a launch of its own, over steps in which tiles go stale; one launch less per layer."""
    from maskedincrementeval_b200 import _native as nat, fields as fl
    from maskedincrementeval_b200.incr_modules.e2depth_incr import ConvLayerIncr
    from maskedincrementeval_b200.incr_modules.mask_incr_modules import check_device_errors
    mode, cin, cout, k, s = cfg
    fl.config.tensor_cores = mode
    n, h, w = 1, 34, 44
    outs, counts = [], []
    for head in (2048, 0):
        fl.config.head_dilation = head
        torch.manual_seed(0)
        layer = ConvLayerIncr(cin, cout, k, s, k // 2, activation="relu").to(dev).eval()
        gg = torch.Generator().manual_seed(5)
        x0 = cl(torch.randn(n, cin, h, w, generator=gg), dev)
        res = []
        with torch.no_grad():
            layer.forward_refresh_reservoirs(x0)
            for step in range(5):
                d = cl(sparse(gg, (n, cin, h, w), [0.02, 0.3, 0.0, 0.01, 1.0][step]), dev)
                m = fl.mask_from_delta(d)
                nat.reset_launch_count()
                y = layer([d, m])
                counts.append(nat.launch_count())
                res.append((y[0].clone(), y[1].bits.clone()))
            check_device_errors(layer)
        outs.append(res)
    for (ya, ba), (yb, bb) in zip(*outs):
        assert torch.equal(ya, yb) and torch.equal(ba, bb)
    # the cluster variants keep the separate launch (the entry point enqueues it itself): two launches either way
    clustered = layer.conv2d.last_cluster_size > 1
    assert counts[:5] == [2 if clustered else 1] * 5 and counts[5:] == [2] * 5, counts


def test_head_job_must_describe_the_call(dev):
    """A head job whose lists or geometry are not the convolution's own is refused before anything is launched."""
    import ctypes as C
    from maskedincrementeval_b200 import _native as nat, fields as fl
    from maskedincrementeval_b200.incr_modules.e2depth_incr import ConvLayerIncr
    fl.config.tensor_cores = "off"
    torch.manual_seed(0)
    layer = ConvLayerIncr(16, 32, 3, 1, 1, activation=None).to(dev).eval()
    g = torch.Generator().manual_seed(1)
    d = cl(sparse(g, (1, 16, 24, 32), 0.05), dev)
    with torch.no_grad():
        layer.forward_refresh_reservoirs(cl(torch.randn(1, 16, 24, 32, generator=g), dev))
        layer([d, None])
    plan = next(iter(layer.conv2d._plans.values()))
    a = plan.args
    other = torch.zeros_like(plan.list)
    bad = nat.TailJob(plan.tail.c.in_bits, 1, 24, 32, 24, 32, 3, 1, 1, None, plan.out_bits.data_ptr(), other.data_ptr(),
                      plan.stale.data_ptr(), plan.counts.data_ptr(), plan.flags.data_ptr())
    a.head = C.addressof(bad)
    assert nat.lib.mie_conv_tiles(C.byref(a), nat.stream_ptr(dev)) == nat.EINVAL
    a.head = None
    torch.cuda.synchronize()


def test_network_step_with_in_kernel_dilation(dev):
    """E2Depth at 128x160 through the runner: the same accumulated output to the bit, a launch fewer per convolution
    that does not run as clusters."""
    from maskedincrementeval_b200 import _native as nat, fields as fl
    from maskedincrementeval_b200.incr_modules.e2depth_incr import E2VIDRecurrentIncr
    from maskedincrementeval_b200.runtime import IncrementalRunner
    from maskedincrementeval_b200.synthetic import seeded_state_dict, voxel_sequence
    cfg = {"num_bins": 5, "skip_type": "sum", "recurrent_block_type": "convlstm", "num_encoders": 3, "base_num_channels": 32,
           "num_residual_blocks": 2, "use_upsample_conv": True, "norm": "none"}
    frames = [f.to(dev) for f in voxel_sequence(1, 128, 160, 10, 4000, 6, seed=3)]
    fl.config.compat = "exact"
    results, launches = [], []
    for head in (2048, 0):
        fl.config.head_dilation = head
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
    assert launches[0] <= launches[1] - 6, launches      # every convolution that is not a cluster launch (7 of 15 here)
