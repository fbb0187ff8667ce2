"""float16 entry points of the C ABI against the oracle.

The reference dispatches Half tensors into its kernels with a float32 accumulator
(ext/torch_cuda.cu:62, mconv_cuda.cuh:135-139) and rounds once at the end.  The
oracle is therefore the reference's float32 CPU kernel run on the float16-rounded
operands; results must agree to one float16 unit (2^-10 of the tensor's largest
value).  Wide layers run on the tensor cores with one MMA per product (every
float16 value is exact in TF32), narrow ones on the CUDA-core kernels.
"""
import numpy as np
import pytest
import torch

import capi
import helpers
from oracle.oracle import Oracle

pytestmark = pytest.mark.gpu

HALF_ULP = 2.0 ** -10
S, P, U = (1, 1), (0, 1), (1, 1)


@pytest.mark.parametrize("shape", [
    (2, 24, 40, (12, 128), (4, 3), (2, 1)),   # wide: tensor cores
    (3, 3, 64, (12, 256), (4, 3), (1, 1)),    # first layer
    (2, 5, 6, (9, 44), (3, 2), (1, 1)),       # small: CUDA-core kernels
    (4, 32, 48, (96, 1), (6, 1), (2, 1)),     # wide 1-D Mellin layer (batch plays the linear axis)
], ids=["wide", "first_layer", "small", "mellin_1d"])
def test_half_layer_matches_the_oracle_on_the_rounded_operands(shape):
    n, ci, co, ng, nf, d = shape
    oracle = Oracle("reference") if Oracle.reference_available() else Oracle("port")
    p = P if ng[1] > 1 else (0, 0)
    rng = np.random.default_rng(7)
    x = torch.from_numpy(rng.standard_normal((n, ci) + ng).astype(np.float32)).cuda().half()
    w = torch.from_numpy((rng.standard_normal((co, ci) + nf) / np.sqrt(ci * nf[0] * nf[1])).astype(np.float32)).cuda().half()
    b = torch.from_numpy(rng.standard_normal(co).astype(np.float32)).cuda().half()
    r = (ng[0] - oracle.mcorr_valid_size(nf[0], ng[0], 1, d[0]), 1 if ng[1] > 1 else 0)
    x_h, w_h, b_h = (t.float().cpu().numpy() for t in (x, w, b))
    y_exp = oracle.mcorrlcorr(x_h, w_h, b_h, S, d, p, U, r)
    y = torch.full(y_exp.shape, float("nan"), device="cuda", dtype=torch.half)
    capi.forward_f16(x, w, b, y, S, d, p, U)
    go = torch.from_numpy(rng.standard_normal(y_exp.shape).astype(np.float32)).cuda().half()
    gx = torch.full_like(x, float("nan"))
    capi.grad_input_f16(w, go, gx, S, d, p, U)
    gw = torch.full_like(w, float("nan"))
    gb = torch.full_like(b, float("nan"))
    capi.grad_weight_f16(x, go, gw, gb, S, d, p, U)
    torch.cuda.synchronize()
    gx_exp, gw_exp, gb_exp = oracle.mcorrlcorr_backward(x_h, w_h, go.float().cpu().numpy(), S, d, p, U)
    assert helpers.rel_err(y.float().cpu().numpy(), y_exp) <= HALF_ULP
    assert helpers.rel_err(gx.float().cpu().numpy(), gx_exp) <= HALF_ULP
    assert helpers.rel_err(gw.float().cpu().numpy(), gw_exp) <= HALF_ULP
    assert helpers.rel_err(gb.float().cpu().numpy(), gb_exp) <= HALF_ULP
    assert capi.device_status() == 0


def test_half_entry_points_reject_a_short_workspace():
    x = torch.zeros((1, 16, 8, 64), device="cuda", dtype=torch.half)
    w = torch.zeros((32, 16, 2, 3), device="cuda", dtype=torch.half)
    y = torch.zeros((1, 32, 8, 64), device="cuda", dtype=torch.half)
    geom = capi._geometry(x.shape, w.shape, y.shape, S, (1, 1), P, U)
    ws = torch.empty(256, dtype=torch.uint8, device="cuda")
    rc = capi.lib().mellin_mcorrlcorr_forward_f16(capi._p(x), capi._p(w), capi._p(None), *geom, capi._p(y), capi._p(ws),
                                                  __import__("ctypes").c_size_t(256), capi._stream())
    assert rc == 3 and b"workspace" in capi.lib().mellin_last_error()
