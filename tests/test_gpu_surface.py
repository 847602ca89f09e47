"""The stand-alone pieces of the operator surface that no network exercises: ``IncrPointwiseMultiply`` and
``NonlinearPointOpIncr`` (reservoirs only read), ``nnConvIncrBase`` (always through the native convolution entry
point), the benchmark wrappers ``Conv{1x1,3x3,5x5}Incr`` / ``ActivationIncr`` and the 7x7 native entry point."""
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
def fp32_path():
    from maskedincrementeval_b200 import fields as fl
    old = fl.config.tensor_cores
    fl.config.tensor_cores = "off"
    yield
    fl.config.tensor_cores = old


def cl(t, dev):
    return t.to(dev).contiguous(memory_format=torch.channels_last)


def sparse_delta(g, shape, frac, std=0.5):
    n, c, h, w = shape
    act = (torch.rand(n, 1, h, w, generator=g) < frac).float()
    return torch.randn(shape, generator=g) * std * act


def test_incr_pointwise_multiply_reads_only(dev):
    """d(x1*x2) = (dx2 + x2)*dx1 + x1*dx2 (mask_incr_functional.py:52-54); neither reservoir moves."""
    from maskedincrementeval_b200.incr_modules.mask_incr_functional import IncrementReserve, IncrPointwiseMultiply
    from maskedincrementeval_b200.incr_modules.mask_incr_modules import PointwiseMultiplyIncr
    g = torch.Generator().manual_seed(3)
    shape = (2, 12, 21, 27)
    x1, x2 = torch.randn(shape, generator=g), torch.randn(shape, generator=g)
    r1, r2 = IncrementReserve(cl(x1, dev)), IncrementReserve(cl(x2, dev))
    mod = PointwiseMultiplyIncr(r1, r2)
    for frac in (0.2, 0.0, 1.0):
        d1, d2 = sparse_delta(g, shape, frac), sparse_delta(g, shape, frac * 0.5)
        want = (d2 + x2) * d1 + x1 * d2
        for out, m in (IncrPointwiseMultiply([cl(d1, dev), None], r1, [cl(d2, dev), None], r2),
                       mod([cl(d1, dev), None], [cl(d2, dev), None])):
            assert float((out.cpu() - want).abs().max()) <= 1e-6 * max(float(want.abs().max()), 1.0)
            pm = m.pixel_mask().cpu()
            assert float((out.cpu() * (1 - pm.float())).abs().max()) == 0.0
        assert torch.equal(r1.reservoir.cpu(), x1) and torch.equal(r2.reservoir.cpu(), x2)


@pytest.mark.parametrize("op", ["relu", "sigmoid", "tanh"])
def test_nonlinear_point_op_leaves_reservoir(dev, op):
    """dy = op(res + dx) - op(res) against a reservoir another module owns (mask_incr_modules.py:86-103)."""
    from maskedincrementeval_b200.incr_modules.mask_incr_functional import IncrementReserve
    from maskedincrementeval_b200.incr_modules.mask_incr_modules import NonlinearPointOpIncr
    g = torch.Generator().manual_seed(4)
    shape = (1, 8, 19, 23)
    x = torch.randn(shape, generator=g)
    res = IncrementReserve(cl(x, dev))
    mod = NonlinearPointOpIncr(res, getattr(torch, op))
    for frac in (0.3, 1.0):
        dx = sparse_delta(g, shape, frac)
        dy, _ = mod([cl(dx, dev), None])
        want = R._OPS[op](x + dx) - R._OPS[op](x)
        assert float((dy.cpu() - want).abs().max()) <= 1e-6
        assert torch.equal(res.reservoir.cpu(), x)
    assert float((mod.forward_refresh_reservoirs(cl(x, dev)).cpu() - R._OPS[op](x)).abs().max()) <= 1e-6


@pytest.mark.parametrize("k,s", [(1, 1), (3, 1), (3, 2), (5, 1), (5, 2), (7, 1)])
def test_conv_increment_ext_all_kernel_sizes(dev, k, s):
    """conv{1,3,5,7}x*_increment_ext (ops.cpp:51-114) through the reference-shaped entry points: output = delta
    convolution without bias, every element of the uninitialised output written."""
    from maskedincrementeval_b200.ext.pointops import pointops_functional as pf
    g = torch.Generator().manual_seed(10 * k + s)
    cin, cout, h, w = 6, 10, 29, 35
    wt = torch.randn(cout, cin, k, k, generator=g) * 0.2
    dx = sparse_delta(g, (2, cin, h, w), 0.1)
    ho, wo = (h + 2 * (k // 2) - k) // s + 1, (w + 2 * (k // 2) - k) // s + 1
    out = torch.full((2, cout, ho, wo), float("nan"), device=dev).contiguous(memory_format=torch.channels_last)
    fn = getattr(pf, f"conv{k}x{k}_increment_ext")
    fn(cl(dx, dev), None, pf.convert_filter_out_channels_last(wt.to(dev)), out, s)
    want = R.conv_delta(dx, wt, s, k // 2)
    assert not bool(torch.isnan(out).any())
    assert float((out.cpu() - want).abs().max()) <= 1e-5 * max(float(want.abs().max()), 1.0)


def test_conv_incr_base_routes_through_native_entry_point(dev):
    """nnConvIncrBase.forward = conv2d_from_module on the [Cin,kH,kW,Cout] copy of the filter
    (mask_incr_modules.py:122-142); refresh is the dense convolution with bias."""
    from maskedincrementeval_b200.incr_modules.mask_incr_modules import nnConvIncrBase
    g = torch.Generator().manual_seed(6)
    conv = nnConvIncrBase(6, 12, 3, 1, 1).to(dev).eval()
    wt, b = conv.weight.detach().cpu(), conv.bias.detach().cpu()
    x = torch.randn(1, 6, 26, 30, generator=g)
    with torch.no_grad():
        y0 = conv.forward_refresh_reservoirs(cl(x, dev))
        assert float((y0.cpu() - R.conv_dense(x, wt, b, 1, 1)).abs().max()) <= 1e-5
        dx = sparse_delta(g, x.shape, 0.15)
        out, mask = conv([cl(dx, dev), None])
        assert mask is None
        want = R.conv_delta(dx, wt, 1, 1)
        assert float((out.cpu() - want).abs().max()) <= 1e-5 * max(float(want.abs().max()), 1.0)
        assert tuple(conv.conv2d_weights.shape) == (6, 3, 3, 12)


@pytest.mark.parametrize("name,k", [("Conv1x1Incr", 1), ("Conv3x3Incr", 3), ("Conv5x5Incr", 5)])
def test_benchmark_conv_wrappers(dev, name, k):
    """Conv{1x1,3x3,5x5}Incr (ext/pointops/pointops_modules.py:43-63): a delta that lives on the module's mask gives the
    plain delta convolution; tiles the mask does not reach are exactly zero."""
    from maskedincrementeval_b200.ext.pointops import pointops_modules as pm
    g = torch.Generator().manual_seed(20 + k)
    cin, cout, h, w = 8, 16, 40, 48
    wt = (torch.randn(cout, cin, k, k, generator=g) * 0.2).to(dev)
    mod = getattr(pm, name)((1, cin, h, w), cin, cout, wt, stride=1, device=dev)
    assert tuple(mod.weight_t.shape) == (cin, k, k, cout) and mod.mask.dtype == torch.bool
    mod.mask[:, :, 24:, :] = False                       # the lower part of the image is outside the mask
    dx = torch.randn(1, cin, h, w, generator=g).to(dev) * mod.mask.any(1, keepdim=True)
    out = mod(dx.contiguous(memory_format=torch.channels_last))
    want = R.conv_delta(dx.cpu().contiguous(), wt.cpu(), 1, k // 2)
    assert out.is_contiguous(memory_format=torch.channels_last)
    assert float((out.cpu() - want).abs().max()) <= 1e-5 * max(float(want.abs().max()), 1.0)
    assert float(out[:, :, 32:].abs().max()) == 0.0
    dense = mod.forward_refresh_reservoir(dx)
    assert float((dense.cpu() - want).abs().max()) <= 1e-4 * max(float(want.abs().max()), 1.0)


def test_benchmark_activation_wrapper(dev):
    """ActivationIncr (ext/pointops/pointops_modules.py:8-19): relu(res + d) - relu(res), reservoir advanced in place."""
    from maskedincrementeval_b200.ext.pointops.pointops_modules import ActivationIncr
    g = torch.Generator().manual_seed(8)
    shape = (1, 40, 80)                                   # the reference's own test shape (tests/test_pointops.py:12)
    x = torch.randn(shape, generator=g)
    mod = ActivationIncr(shape, device=dev)
    assert float(mod.reservoir.abs().max()) == 0.0
    y0 = mod.forward_refresh_reservoir(x.to(dev))
    assert torch.equal(y0.cpu(), torch.relu(x))
    d = torch.randn(shape, generator=g)
    out = mod([d.to(dev), None])
    assert torch.equal(out.cpu(), torch.relu(x + d) - torch.relu(x))
    assert torch.equal(mod.reservoir.cpu(), x + d)
