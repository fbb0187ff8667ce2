"""CPU checker for the elementwise layers in front of the first Mellin layer -- TEST INFRASTRUCTURE ONLY.

Nothing in the product imports this module.  numpy restatement, in the dtype of the input, of

* the reference's ``dilation_lift`` (``layers.py:8-21``): ``out[t] = (t + 1) ** tau * in[t]`` along ``dim``, with the
  same check (and message) for a bad ``dim``;
* ``LogCompression.forward`` (``layers.py:100-101``): ``out = log(abs(in) + exp(log_eps))``;
* the two applied in the model's order (``models.py:413-417``: compression first, then the lift), and the
  derivatives of that composition written out by hand (the reference leaves them to autograd).

Pinned by ``tests/golden/prologue_cases.npz``, recorded from the reference's own ``layers.py`` (forward values and
autograd gradients), in ``tests/test_oracle.py``.
"""
import numpy as np


def _dim(x, dim):
    dim_ = dim + x.ndim if dim < 0 else dim
    if dim_ >= x.ndim or dim_ < 0:
        raise RuntimeError(f"{dim} not a valid dimension for a tensor if dimension {x.ndim}")
    return dim_


def _weights(x, tau, dim):
    """(t + 1) ** tau shaped to broadcast along ``dim`` (layers.py:17-20)."""
    shape = [1] * x.ndim
    shape[dim] = x.shape[dim]
    steps = np.arange(1, x.shape[dim] + 1, dtype=x.dtype)
    return (steps ** x.dtype.type(tau)).reshape(shape), np.log(steps).reshape(shape)


def dilation_lift(x, tau, dim):
    dim = _dim(x, dim)
    return x * _weights(x, tau, dim)[0]


def log_compression(x, log_eps):
    return np.log(np.abs(x) + x.dtype.type(np.exp(log_eps)))


def lift_compress(x, log_tau, log_eps, dim):
    """Compression (if ``log_eps`` is not None) then lift (if ``log_tau`` is not None)."""
    out = x if log_eps is None else log_compression(x, log_eps)
    return out if log_tau is None else dilation_lift(out, np.exp(log_tau), dim)


def lift_compress_backward(x, grad_y, log_tau, log_eps, dim, with_scales=False):
    """(grad_x, grad_log_tau, grad_log_eps) of ``lift_compress``; sums in float64.

    ``with_scales`` appends the sums of the ABSOLUTE values of the terms of the two parameter gradients: what a
    tolerance on those sums has to be relative to when the terms cancel."""
    dim = _dim(x, dim) if log_tau is not None else 0
    g = grad_y.astype(np.float64)
    xd = x.astype(np.float64)
    grad_log_tau = grad_log_eps = None
    scale_tau = scale_eps = 0.0
    c = xd
    if log_tau is not None:
        tau = float(np.exp(log_tau))
        w, log_steps = _weights(xd, tau, dim)
    else:
        w, log_steps = 1.0, 0.0
    gc = g * w
    gx = gc
    if log_eps is not None:
        eps = float(np.exp(log_eps))
        c = np.log(np.abs(xd) + eps)
        inv = 1.0 / (np.abs(xd) + eps)
        grad_log_eps = float((gc * inv).sum() * eps)   # d/d log_eps = eps d/d eps
        scale_eps = float(np.abs(gc * inv).sum() * eps)
        gx = gc * inv * np.sign(xd)                    # torch: abs'(0) = 0
    if log_tau is not None:
        grad_log_tau = float((gc * c * log_steps).sum() * tau)  # d (t+1)^tau / d log_tau = tau log(t+1) (t+1)^tau
        scale_tau = float(np.abs(gc * c * log_steps).sum() * tau)
    if with_scales:
        return gx.astype(x.dtype), grad_log_tau, grad_log_eps, scale_tau, scale_eps
    return gx.astype(x.dtype), grad_log_tau, grad_log_eps
