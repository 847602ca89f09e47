"""Python face of the native boundary (reference: ``ext/pointops/pointops_functional.py:1-44``).

Same five native names, same three functions, same argument meaning; underneath, ctypes calls into
libmie instead of a pybind11 torch extension."""
import torch

from ... import _native as nat


def _stream(t):
    return nat.stream_ptr(t.device)


# --- the five functions the reference's extension module exports (ops.cpp:117-123) -----------------
def activation_increment(X, in_incr, out_incr):
    """out = relu(X + in) - relu(X); X += in (in place).  All three contiguous CUDA tensors."""
    for name, t in (("X", X), ("in_incr", in_incr), ("out_incr", out_incr)):
        nat.require_cuda(t, name)
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
    if not (X.numel() == in_incr.numel() == out_incr.numel()):
        raise RuntimeError("X, in_incr and out_incr must have the same number of elements")
    nat.check(nat.lib.mie_activation_increment(X.data_ptr(), in_incr.data_ptr(), out_incr.data_ptr(), X.numel(),
                                               nat.ACT_RELU, _stream(X)), "activation_increment")


_ws_cache = {}


def _conv_increment(k, x_incr, mask, filter, out_incr, stride):
    nat.require_cuda(x_incr, "x_incr")
    nat.require_cuda(filter, "filter")
    nat.require_cuda(out_incr, "out_incr")
    if not filter.is_contiguous():
        raise RuntimeError("filter must be contiguous")  # CHECK_INPUT(filter), ops.cpp:37
    if filter.dim() != 4 or filter.shape[1] != k or filter.shape[2] != k:
        raise RuntimeError(f"filter must be [Cin,{k},{k},Cout]")
    n, cin, h, w = x_incr.shape
    cout = filter.shape[3]
    if filter.shape[0] != cin:
        raise RuntimeError("filter and x_incr disagree on the input channels")
    cl = torch.channels_last
    if not x_incr.is_contiguous(memory_format=cl) or not out_incr.is_contiguous(memory_format=cl):
        raise RuntimeError("x_incr and out_incr must be channels_last")
    stride = int(stride)
    pad = k // 2
    ho, wo = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
    if tuple(out_incr.shape) != (n, cout, ho, wo):
        raise RuntimeError(f"out_incr must be {(n, cout, ho, wo)}")
    mptr, msz = None, 0
    if mask is not None:
        if not mask.is_cuda:
            raise RuntimeError("mask must be a CUDA tensor")  # CHECK_CUDA(mask), ops.cpp:36
        if tuple(mask.shape) != tuple(x_incr.shape):
            raise RuntimeError("mask must have the shape of x_incr")
        if mask.dtype == torch.bool:
            mask = mask.to(torch.uint8)
        if mask.dtype not in (torch.uint8, torch.int32):
            mask = mask.to(torch.int32)
        mask = mask.contiguous(memory_format=cl)
        mptr, msz = mask.data_ptr(), mask.element_size()
    need = nat.lib.mie_conv_increment_workspace_bytes(n, cin, h, w, cout, k, stride)
    if need < 0:
        nat.check(int(need), "conv_increment_workspace_bytes")
    key = (str(x_incr.device), torch.cuda.current_stream(x_incr.device).cuda_stream)
    ws = _ws_cache.get(key)
    if ws is None or ws.numel() < need:
        ws = _ws_cache[key] = torch.empty(int(need) + 256, dtype=torch.uint8, device=x_incr.device)
    base = ws.data_ptr()
    off = (-base) % 256
    nat.check(nat.lib.mie_conv_increment_ext(x_incr.data_ptr(), mptr, msz, filter.data_ptr(), out_incr.data_ptr(),
                                             n, cin, h, w, cout, k, stride, base + off, ws.numel() - off,
                                             _stream(x_incr)), f"conv{k}x{k}_increment_ext")


def conv1x1_increment_ext(x_incr, mask, filter, out_incr, stride):
    _conv_increment(1, x_incr, mask, filter, out_incr, stride)


def conv3x3_increment_ext(x_incr, mask, filter, out_incr, stride):
    _conv_increment(3, x_incr, mask, filter, out_incr, stride)


def conv5x5_increment_ext(x_incr, mask, filter, out_incr, stride):
    _conv_increment(5, x_incr, mask, filter, out_incr, stride)


def conv7x7_increment_ext(x_incr, mask, filter, out_incr, stride):
    _conv_increment(7, x_incr, mask, filter, out_incr, stride)


# --- the reference's Python-level functions ----------------------------------------------------------
def activation_incr(x, input_incr):
    """Returns relu(x + input_incr) - relu(x) and updates x in place (reference ``:7-10``)."""
    output_ = torch.empty(x.shape, dtype=torch.float, device=x.device)
    activation_increment(x, input_incr, output_)
    return output_


def convert_filter_out_channels_last(conv_weights):
    """[Cout,Cin,kH,kW] -> [Cin,kH,kW,Cout] (reference ``:13-14``)."""
    return torch.permute(conv_weights, (1, 2, 3, 0)).contiguous().clone()


def functional_conv_module(x_incr, conv_weights, mask=None, stride=(1, 1), padding=(1, 1)):
    """Masked delta convolution with a [Cin,kH,kW,Cout] filter; returns ``[out, None]`` (reference ``:18-42``).

    The reference overwrites the caller's mask with all-ones (``:22``); here a given mask is honoured and a
    missing one is derived from ``x_incr != 0``.  Only padding == k // 2 is supported, as in the reference's
    kernels."""
    k = conv_weights.shape[1]
    if k not in (1, 3, 5, 7):
        raise NotImplementedError("not Implemented convolution for these dimensions!")
    pad = padding[0] if isinstance(padding, (tuple, list)) else int(padding)
    if pad != k // 2:
        raise NotImplementedError("only padding == kernel_size // 2 is supported")
    s = stride[0] if isinstance(stride, (tuple, list)) else int(stride)
    x_incr = x_incr.contiguous(memory_format=torch.channels_last)
    out_H = int((x_incr.shape[2] + 2 * pad - k) // s + 1)
    out_W = int((x_incr.shape[3] + 2 * pad - k) // s + 1)
    out_C = conv_weights.shape[3]
    output_ = torch.empty((x_incr.shape[0], out_C, out_H, out_W), dtype=torch.float, device=x_incr.device,
                          memory_format=torch.channels_last)
    if isinstance(mask, (list, tuple)) or (mask is not None and not torch.is_tensor(mask)):
        mask = mask.pixel_mask().expand(-1, x_incr.shape[1], -1, -1) if hasattr(mask, "pixel_mask") else None
    _conv_increment(k, x_incr, mask, conv_weights.contiguous(), output_, s)
    return [output_, None]
