"""LayerNorm of the hidden activations, optionally with the ReLU before it folded in, on the
library's row-normalisation kernels (csrc/layer_norm.cu).  The reference applies activation and
torch.nn.LayerNorm between its graph convolutions (models/model.py:117-121)."""
import torch
import torch.nn.functional as F
from torch.autograd import Function

from ..core import _native
from ..core import _DT, _ptr, _scratch, _stream

MAX_WIDTH = 1024


class _ActNormFunction(Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, relu):
        lib = _native.lib()
        x = x.contiguous()
        rows, C = x.shape
        y = torch.empty_like(x)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        weight, bias = weight.contiguous(), bias.contiguous()
        _native.check(lib.grws_layer_norm_fwd(_ptr(x), _ptr(weight), _ptr(bias), y.data_ptr(), mean.data_ptr(),
                                              rstd.data_ptr(), rows, C, _DT[x.dtype], 1 if relu else 0, float(eps),
                                              _stream(x.device)))
        ctx.save_for_backward(x, weight, mean, rstd)
        ctx.relu = relu
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _native.lib()
        x, weight, mean, rstd = ctx.saved_tensors
        rows, C = x.shape
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        dgamma = torch.empty(C, dtype=torch.float32, device=x.device)
        dbeta = torch.empty(C, dtype=torch.float32, device=x.device)
        scratch = _scratch(lib.grws_layer_norm_scratch_bytes(C), x.device)
        _native.check(lib.grws_layer_norm_bwd(_ptr(x), _ptr(weight), _ptr(dy), mean.data_ptr(), rstd.data_ptr(),
                                              dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), rows, C, _DT[x.dtype],
                                              1 if ctx.relu else 0, scratch.data_ptr(), scratch.numel(),
                                              _stream(x.device)))
        return dx, dgamma.to(weight.dtype), dbeta.to(weight.dtype), None, None


def act_layer_norm(x: torch.Tensor, norm: torch.nn.LayerNorm, relu: bool) -> torch.Tensor:
    """``norm(relu(x))`` (or ``norm(x)``) for a 2-D CUDA activation.  Shapes and dtypes the kernels do
    not cover (width no multiple of 8 or above 1,024, parameters in another dtype than the
    activations, no affine parameters) go through torch's own operators."""
    C = x.shape[-1]
    fits = (x.is_cuda and x.dim() == 2 and x.dtype in _DT and C % 8 == 0 and C <= MAX_WIDTH
            and norm.weight is not None and norm.bias is not None and norm.weight.dtype == x.dtype
            and tuple(norm.normalized_shape) == (C,) and not torch.is_autocast_enabled())
    if not fits:
        return norm(F.relu(x) if relu else x)
    return _ActNormFunction.apply(x, norm.weight, norm.bias, norm.eps, relu)
