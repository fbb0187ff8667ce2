"""The elementwise layers in front of the first Mellin layer, on B200.

Same names, arguments, parameter names and error text as the reference's
``layers.py`` (``dilation_lift`` ``:8-21``, ``DilationLift`` ``:41-77``,
``LogCompression`` ``:80-101``), so that a checkpoint's ``lift.log_tau`` and
``log_compression.log_eps`` load unchanged.  Underneath, each is ONE CUDA pass
(``csrc/prologue.cu``) instead of a chain of torch kernels, and
:class:`LogCompressionLift` runs the pair the model applies back to back
(``models.py:413-417``: compression, then the lift) as a single pass with a
single-pass backward.  The parameter gradients are summed in a fixed order:
two runs give the same bits.

There is no CPU path: the functions raise on tensors that are not on a CUDA
device.  ``ScaledGaussianNoise`` (``layers.py:104-137`` there; imported by the
reference's ``running.py:19``) is training-time noise outside the accelerated
path: it is kept, on stock torch operators, only so that this module can stand
in for the reference's file.
"""
from typing import Optional

import torch

import capi

__all__ = ["dilation_lift", "log_compression", "lift_compress", "DilationLift", "LogCompression", "LogCompressionLift",
           "ScaledGaussianNoise"]


def _scalar_for(param: Optional[torch.Tensor], like: torch.Tensor) -> Optional[torch.Tensor]:
    if param is None:
        return None
    if param.numel() != 1:
        raise RuntimeError("expected a scalar parameter, got shape %s" % (tuple(param.shape),))
    return param.reshape(()).to(device=like.device, dtype=like.dtype)


class _LiftCompress(torch.autograd.Function):
    """``y = (t + 1)^tau * log(eps + |x|)`` along ``dim``; either parameter may be None."""

    @staticmethod
    def forward(ctx, x, tau, eps, dim, log_domain):
        x = x.contiguous()
        shape = x.shape
        outer = 1
        for extent in shape[:dim]:
            outer *= extent
        length = shape[dim] if tau is not None else 1
        inner = x.numel() // max(outer * length, 1) if x.numel() else 0
        if x.numel() == 0:
            outer, length, inner = 0, max(length, 1), 1
        tau_c = None if tau is None else tau.contiguous()
        eps_c = None if eps is None else eps.contiguous()
        y = torch.empty_like(x)
        capi.lift_compress(x, tau_c, eps_c, log_domain, outer, length, inner, y)
        ctx.save_for_backward(x, tau_c, eps_c)
        ctx.geometry = (outer, length, inner, log_domain)
        return y

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_y):
        x, tau, eps = ctx.saved_tensors
        outer, length, inner, log_domain = ctx.geometry
        grad_y = grad_y.contiguous()
        grad_x = torch.empty_like(x)
        grad_tau = None if tau is None else torch.empty_like(tau)
        grad_eps = None if eps is None else torch.empty_like(eps)
        capi.lift_compress_backward(x, grad_y, tau, eps, log_domain, outer, length, inner, grad_x, grad_tau, grad_eps)
        return grad_x, grad_tau, grad_eps, None, None


def _run(x, tau, eps, dim, log_domain):
    if not x.is_cuda:
        raise RuntimeError("layers: expected a CUDA tensor (there is no CPU implementation)")
    if x.dtype in (torch.float16, torch.bfloat16):  # computed in float32, returned in the input's type
        return _run(x.float(), tau, eps, dim, log_domain).to(x.dtype)
    if x.dtype not in (torch.float32, torch.float64):
        raise TypeError("layers: unsupported dtype %s" % x.dtype)
    return _LiftCompress.apply(x, _scalar_for(tau, x), _scalar_for(eps, x), dim, log_domain)


def _checked_dim(x: torch.Tensor, dim: int) -> int:
    dim_ = dim + x.dim() if dim < 0 else dim
    if dim_ >= x.dim() or dim_ < 0:
        raise RuntimeError(f"{dim} not a valid dimension for a tensor if dimension {x.dim()}")
    return dim_


def dilation_lift(input: torch.Tensor, tau: torch.Tensor, dim: int) -> torch.Tensor:
    """``output[t - 1] = t ** tau * input[t - 1]`` along ``dim`` (reference ``layers.py:8-21``)."""
    return _run(input, tau, None, _checked_dim(input, dim), False)


def log_compression(input: torch.Tensor, eps: torch.Tensor) -> torch.Tensor:
    """``out[i] = log(eps + abs(input[i]))`` (reference ``layers.py:100-101`` with ``eps = exp(log_eps)``)."""
    return _run(input, None, eps, 0, False)


def lift_compress(input: torch.Tensor, log_tau: Optional[torch.Tensor], log_eps: Optional[torch.Tensor],
                  dim: int) -> torch.Tensor:
    """Log compression followed by the lift along ``dim``, from the modules' own parameters (logarithms)."""
    return _run(input, log_tau, log_eps, _checked_dim(input, dim), True)


class DilationLift(torch.nn.Module):
    r"""``output[t - 1] = t^\tau input[t - 1]`` along ``dim``, with learnable ``log_tau`` (reference ``layers.py:41-77``)."""

    __constants__ = ["dim"]

    def __init__(self, dim: int = 2):
        super().__init__()
        self.log_tau = torch.nn.Parameter(torch.tensor(0.0))
        self.dim = dim
        self.reset_parameters()

    def extra_repr(self) -> str:
        return f"dim={self.dim}"

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return lift_compress(input, self.log_tau, None, self.dim)

    def reset_parameters(self) -> None:
        torch.nn.init.normal_(self.log_tau)


class LogCompression(torch.nn.Module):
    """``out[i] = log(eps + abs(input[i]))`` with learnable ``log_eps`` (reference ``layers.py:80-101``)."""

    def __init__(self):
        super().__init__()
        self.log_eps = torch.nn.Parameter(torch.tensor(0.0))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        torch.nn.init.normal_(self.log_eps)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return _run(input, None, self.log_eps, 0, True)


class LogCompressionLift(torch.nn.Module):
    """The model's ``log_compression`` then ``lift`` (``models.py:413-417``) as one pass.

    Holds the two reference modules under the reference's attribute names, so that the state dict keys are
    ``log_compression.log_eps`` and ``lift.log_tau``; either can be switched off as the model's
    ``use_log_compression`` / ``use_lift`` do.
    """

    def __init__(self, use_log_compression: bool = True, use_lift: bool = True, dim: int = 2):
        super().__init__()
        self.log_compression = LogCompression() if use_log_compression else None
        self.lift = DilationLift(dim) if use_lift else None

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        if self.log_compression is None and self.lift is None:
            return input
        log_tau = None if self.lift is None else self.lift.log_tau
        log_eps = None if self.log_compression is None else self.log_compression.log_eps
        return lift_compress(input, log_tau, log_eps, self.lift.dim if self.lift is not None else 0)


class ScaledGaussianNoise(torch.nn.Module):
    """Training only: adds zero-mean Gaussian noise whose deviation is ``eps`` times the largest magnitude along
    ``dim``; the identity in evaluation mode (reference ``layers.py:24-38,104-137``).  Stock torch operators."""

    __constants__ = ["dim", "eps"]

    def __init__(self, dim: int = 1, eps: float = 1e-3):
        super().__init__()
        self.dim, self.eps = dim, eps

    def extra_repr(self) -> str:
        return f"dim={self.dim}, eps={self.eps}"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        dim = _checked_dim(x, self.dim)
        if not self.training:
            return x
        peak = x.abs().amax(dim, keepdim=True)
        return x + (peak * self.eps) * torch.randn_like(x)
