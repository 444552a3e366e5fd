"""A framework caller for the library: the role upstream's Caffe layer plays
(external/caffe/src/caffe/layers/xnor_nn_conv_layer.cpp), written for PyTorch tensors that
already live on the GPU.

`XnorConv2d` follows that layer step by step:

* forward (xnor_nn_conv_layer.cpp:25-67): the convolution object is created on first use from
  the shape of the input (bcast algorithm, NCHW / OIHW / NCHW), the weights are re-binarised
  only after they changed, and the whole minibatch goes through one `forward` call. Here the
  call gets device pointers and PyTorch's current stream, so nothing is copied or waited for.
  A bias, if the layer has one, is added afterwards like any Caffe convolution layer does.
* backward (xnor_nn_conv_layer.cpp:88-125): a plain float convolution backward. The gradient
  of the weights uses the real input and the output gradient; the gradient of the input uses
  `binarize_weights_float(weight)` = sign(w) * mean(w) in place of the weights; afterwards the
  weights count as changed. The float gradients are library calls (`torch.nn.grad`), as they
  are GEMM calls upstream; the binary forward pass is the part this library accelerates.

torch is imported here only; the rest of the package does not need it.
"""
import torch

import xnor_nn_b200 as xb


class _XnorConvFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, layer):
        y = layer._forward_device(x)
        if bias is not None:
            y += bias.view(1, -1, 1, 1)
        ctx.layer = layer
        ctx.has_bias = bias is not None
        ctx.save_for_backward(x, weight)
        return y

    @staticmethod
    def backward(ctx, grad_y):
        x, weight = ctx.saved_tensors
        layer = ctx.layer
        grad_y = grad_y.contiguous()
        grad_x = grad_w = grad_b = None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            grad_b = grad_y.sum(dim=(0, 2, 3))
        if ctx.needs_input_grad[1]:
            grad_w = torch.nn.grad.conv2d_weight(x, weight.shape, grad_y, stride=layer.stride,
                                                 padding=layer.padding)
            layer._weights_changed = True
        if ctx.needs_input_grad[0]:
            bweight = torch.empty_like(weight)
            layer._conv_for(x).binarize_weights_float(
                weight.detach(), bweight, stream=torch.cuda.current_stream().cuda_stream)
            grad_x = torch.nn.grad.conv2d_input(x.shape, bweight, grad_y, stride=layer.stride,
                                                padding=layer.padding)
        return grad_x, grad_w, grad_b, None


class XnorConv2d(torch.nn.Module):
    """Binary convolution layer over `xnor_nn_b200.Convolution`.

    Arguments mirror the Caffe layer's convolution parameters: `in_channels` (IC),
    `out_channels` (OC), `kernel_size` (KH, KW), `stride` (SH, SW), `padding` (PH, PW).
    Inputs are float32 CUDA tensors in NCHW; the result is a new float32 NCHW tensor whose
    spatial size is the library's (`oh`/`ow` of the descriptor, which uses the width padding
    for both, as upstream does: src/common_convolution.cpp:40-41).
    """

    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, bias=False,
                 kernel=None):
        super().__init__()
        pair = lambda v: (v, v) if isinstance(v, int) else tuple(v)
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.padding = pair(kernel_size), pair(stride), pair(padding)
        self.kernel = kernel
        self.weight = torch.nn.Parameter(torch.empty(out_channels, in_channels, *self.kernel_size))
        self.bias = torch.nn.Parameter(torch.zeros(out_channels)) if bias else None
        torch.nn.init.normal_(self.weight, std=0.05)
        self._convs = {}           # (device index, mb, ih, iw) -> Convolution
        self._weights_seen = {}    # same key -> (data_ptr, version) last binarised
        self._weights_changed = True

    def mark_weights_changed(self):
        """What the Caffe layer's `changeWeights` flag records; in-place updates of `weight`
        (an optimiser step, `copy_`) are noticed without it through the tensor's version."""
        self._weights_changed = True

    def _key(self, x):
        return (x.device.index, x.shape[0], x.shape[2], x.shape[3])

    def _conv_for(self, x):
        key = self._key(x)
        conv = self._convs.get(key)
        if conv is None:
            mb, ic, ih, iw = x.shape
            with torch.cuda.device(x.device):
                conv = xb.Convolution(xb.ALGORITHM_BCAST, xb.NCHW, xb.OIHW, xb.NCHW, mb,
                                      self.out_channels, ic, ih, iw, *self.kernel_size,
                                      *self.stride, *self.padding, kernel=self.kernel)
            self._convs[key] = conv
        return conv

    def _forward_device(self, x):
        if not x.is_cuda or x.dtype != torch.float32 or x.dim() != 4:
            raise ValueError("XnorConv2d takes a float32 CUDA tensor of shape (mb, ic, ih, iw); "
                             "there is no CPU path")
        if x.shape[1] != self.in_channels:
            raise ValueError("expected %d input channels, got %d" % (self.in_channels, x.shape[1]))
        if self.weight.device != x.device:
            raise ValueError("weights are on %s, input on %s" % (self.weight.device, x.device))
        x = x.contiguous()
        conv = self._conv_for(x)
        key = self._key(x)
        with torch.cuda.device(x.device):
            conv.set_stream(torch.cuda.current_stream().cuda_stream)
            w = self.weight.detach()
            stamp = (w.data_ptr(), w._version)
            if self._weights_changed or self._weights_seen.get(key) != stamp:
                if self._weights_changed:
                    self._weights_seen.clear()
                    self._weights_changed = False
                conv.change_weights(w.contiguous())
                self._weights_seen[key] = stamp
            y = torch.empty(conv.out_shape, dtype=torch.float32, device=x.device)
            conv.forward(x, y)
        return y

    def forward(self, x):
        return _XnorConvFunction.apply(x, self.weight, self.bias, self)

    def extra_repr(self):
        return "%d, %d, kernel_size=%s, stride=%s, padding=%s, bias=%s" % (
            self.in_channels, self.out_channels, self.kernel_size, self.stride, self.padding,
            self.bias is not None)
