"""The cluster variant of the stride-1 tensor-core convolution: the thread blocks of a cluster split a work item's
input channels and exchange partial sums through distributed shared memory.  It must give what the one-block kernel
gives (up to fp32 summation order) and what the CPU restatement gives, with identical masks, in lossless and in
thresholded mode, with a residual addend, and when only part of the field is active."""
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
    saved = {k: getattr(fl.config, k) for k in ("threshold", "carry", "tensor_cores", "tc_thresholded", "compat")}
    yield
    for k, v in saved.items():
        setattr(fl.config, k, v)
    nat.set_option(nat.OPT_TC_KSPLIT, 1)


def cl(t, dev):
    return t.to(dev).contiguous(memory_format=torch.channels_last)


def sparse_delta(g, shape, frac, std=0.5):
    n, c, h, w = shape
    act = (torch.rand(n, 1, h, w, generator=g) < frac).float()
    return torch.randn(shape, generator=g) * std * act


# cin, cout, k, stride, h, w, activation, addend, threshold, expected cluster size
CASES = [
    (256, 256, 3, 1, 33, 44, "relu", False, 0.0, 4),     # E2Depth residual convolutions
    (256, 256, 3, 1, 33, 44, "relu", True, 0.0, 4),      # ... the second one of a block, with the skip added
    (256, 128, 5, 1, 66, 88, "relu", False, 0.0, 1),     # decoder 0: the 5x5 halo leaves no room for the partial sums
    (256, 128, 3, 1, 66, 88, "relu", False, 0.0, 2),     # 50 tile pairs: clusters of two
    (256, 64, 3, 1, 16, 24, None, False, 0.0, 4),        # slices of a single 16-channel group
    (512, 128, 3, 1, 17, 22, "relu", False, 0.0, 4),     # four channel chunks per thread block
    (256, 256, 3, 1, 17, 22, "relu", False, 0.02, 4),    # thresholded, with carry
    (512, 512, 3, 1, 16, 21, "relu", False, 0.0, 4),     # EV-FlowNet's deepest level
    (128, 256, 5, 2, 66, 88, "relu", False, 0.0, 4),     # encoder 2 (stride 2: the per-tap kernel), one chunk per block
    (64, 128, 5, 2, 132, 176, "relu", False, 0.0, 2),    # encoder 1
    (128, 256, 5, 2, 66, 88, "relu", False, 0.02, 4),    # encoder 2, thresholded
]


def _run(dev, case, ksplit):
    from maskedincrementeval_b200 import _native as nat, fields as fl
    from maskedincrementeval_b200.incr_modules.e2depth_incr import ConvLayerIncr
    from maskedincrementeval_b200.incr_modules.mask_incr_modules import check_device_errors
    cin, cout, k, stride, h, w, act, with_addend, thr, _ = case
    nat.set_option(nat.OPT_TC_KSPLIT, ksplit)
    fl.config.tensor_cores, fl.config.threshold, fl.config.carry = "auto", thr, True
    torch.manual_seed(3)
    layer = ConvLayerIncr(cin, cout, k, stride, k // 2, activation=act).to(dev).eval()
    g = torch.Generator().manual_seed(cin + cout + k)
    x0 = torch.randn(1, cin, h, w, generator=g) * 0.5
    out = []
    with torch.no_grad():
        pre = layer.conv2d.forward_refresh_reservoirs(cl(x0, dev))
        if act is not None:
            layer.activation.forward_refresh_reservoirs(pre)
        for frac in (0.05, 1.0, 0.0, 0.3):
            dx = sparse_delta(g, (1, cin, h, w), frac, std=0.1)
            ho, wo = pre.shape[2:]
            addend = [cl(sparse_delta(g, (1, cout, ho, wo), frac * 0.5, std=0.05), dev), None] if with_addend else None
            dy, m = layer([cl(dx, dev), None], addend)
            out.append((dy.clone(), m.pixel_mask().clone(), dx, addend[0].cpu() if with_addend else None,
                        layer.conv2d.last_cluster_size))
        check_device_errors(layer)
    return out, layer


@pytest.mark.parametrize("case", CASES)
def test_cluster_variant_matches_one_block_kernel(dev, case):
    with_cluster, layer = _run(dev, case, 1)
    plain, _ = _run(dev, case, 0)
    assert all(o[4] == case[9] for o in with_cluster), [o[4] for o in with_cluster]
    assert all(o[4] == 1 for o in plain)
    for (ya, ma, _, _, _), (yb, mb, _, _, _) in zip(with_cluster, plain):
        rng = max(float(yb.abs().max()), 1e-6)
        if case[8] == 0.0:
            assert torch.equal(ma, mb)
            assert float((ya - yb).abs().max()) <= 2e-5 * rng
        else:
            # a thresholded group whose change sits within rounding of the threshold may be decided differently
            assert float((ma != mb).float().mean()) < 1e-3
            assert float((ya - yb).abs().max()) <= case[8] * 1.01 + 2e-5 * rng
        assert float((ya * (1 - ma.float())).abs().max()) == 0.0      # zero outside the mask


def test_cluster_variant_against_the_restatement(dev):
    """Lossless 3x3 256 -> 256 at 33x44 without activation: the delta convolution itself, TF32 arithmetic restated on the CPU."""
    case = (256, 256, 3, 1, 33, 44, None, False, 0.0, 4)
    steps, layer = _run(dev, case, 1)
    wgt = layer.conv2d.weight.detach().cpu()
    for dy, m, dx, _, ks in steps:
        assert ks == 4
        want = R.conv_delta_tf32(dx, wgt, 1, 1)
        rng = max(float(want.abs().max()), 1e-6)
        assert float((dy.cpu() - want).abs().max()) <= 5e-5 * rng
