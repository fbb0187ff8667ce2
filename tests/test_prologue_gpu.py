"""The elementwise layers in front of the first Mellin layer (``layers.py`` -> ``csrc/prologue.cu``).

Checked against values and autograd gradients recorded from the reference's own ``layers.py``
(``tests/golden/prologue_cases.npz``), against the numpy restatement at the benchmark layer's input size, over the
kernel's code paths (16-byte and scalar accesses, weights from the shared-memory table and computed per element, 32-
and 64-bit... element counts are kept small: the 64-bit index path is the same code with another integer type), for
run-to-run bit identity, and for the reference's error behaviour.
"""
import os

import numpy as np
import pytest
import torch

import capi
import helpers
import layers
from oracle import prologue_oracle as po

pytestmark = pytest.mark.gpu

GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "prologue_cases.npz"))
TAGS = sorted({k.rsplit("_", 1)[0] for k in GOLDEN.files if k.endswith("_meta")})
TOL = {np.dtype(np.float32): 1e-5, np.dtype(np.float64): 1e-12}


def _module(dim, use_lc, use_lift, log_tau, log_eps, dtype):
    m = layers.LogCompressionLift(use_lc, use_lift, dim).cuda().to(dtype)
    with torch.no_grad():
        if use_lift:
            m.lift.log_tau.fill_(log_tau)
        if use_lc:
            m.log_compression.log_eps.fill_(log_eps)
    return m


def _close_sum(got, want, scale, tol):
    return abs(got - want) <= tol * max(scale, 1e-30)


@pytest.mark.parametrize("tag", TAGS)
def test_against_the_reference_layers(tag):
    dim, use_lc, use_lift = (int(v) for v in GOLDEN[tag + "_meta"])
    log_tau, log_eps = (float(v) for v in GOLDEN[tag + "_params"])
    x_h, gy_h = GOLDEN[tag + "_x"], GOLDEN[tag + "_grad_y"]
    tol = TOL[x_h.dtype]
    m = _module(dim, use_lc, use_lift, log_tau, log_eps, torch.from_numpy(x_h).dtype)
    x = torch.from_numpy(x_h).cuda().requires_grad_(True)
    before = capi.launch_count()
    y = m(x)
    assert capi.launch_count() - before == 1, "the pair is one pass"
    y.backward(torch.from_numpy(gy_h).cuda())
    assert capi.launch_count() - before == 3, "backward: one pass and the sum of the block sums"
    assert helpers.rel_err(y.detach().cpu().numpy(), GOLDEN[tag + "_y"]) <= tol
    assert helpers.rel_err(x.grad.cpu().numpy(), GOLDEN[tag + "_grad_x"]) <= tol
    _, _, _, scale_tau, scale_eps = po.lift_compress_backward(
        x_h, gy_h, log_tau if use_lift else None, log_eps if use_lc else None, dim, with_scales=True)
    ref_tau, ref_eps = GOLDEN[tag + "_grad_params"]
    ptol = 1e-5 if x_h.dtype == np.float32 else 1e-11  # the reference sums in the tensor's own precision
    if use_lift:
        assert _close_sum(float(m.lift.log_tau.grad), ref_tau, scale_tau, ptol)
    if use_lc:
        assert _close_sum(float(m.log_compression.log_eps.grad), ref_eps, scale_eps, ptol)


def test_separate_modules_match_the_pair():
    """``LogCompression`` then ``DilationLift`` as two modules (the reference's own sequence) = the fused pair."""
    gen = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(6, 9, 44, device="cuda", generator=gen)
    pair = _module(2, True, True, 0.3, -0.7, torch.float32)
    lc, lift = layers.LogCompression().cuda(), layers.DilationLift(2).cuda()
    with torch.no_grad():
        lc.log_eps.fill_(-0.7)
        lift.log_tau.fill_(0.3)
    two = lift(lc(x))
    assert float((two - pair(x)).abs().max() / two.abs().max()) <= 1e-6
    assert set(pair.state_dict()) == {"log_compression.log_eps", "lift.log_tau"}


# (shape, dim): the benchmark layer's input; a lifted axis longer than the shared-memory table (weights computed per
# element); the lift over the contiguous axis (scalar accesses); an odd inner extent
SHAPES = [((32, 3, 41, 800), 2), ((2, 20000, 4), 1), ((8, 3, 1000), -1), ((5, 300, 7), 1)]


@pytest.mark.parametrize("shape,dim", SHAPES, ids=[str(i) for i in range(len(SHAPES))])
def test_against_the_restatement_and_twice_the_same(shape, dim):
    rng = np.random.default_rng(sum(shape))
    x_h = rng.standard_normal(shape).astype(np.float32)
    x_h.flat[::13] = 0.0
    gy_h = rng.standard_normal(shape).astype(np.float32)
    log_tau, log_eps = -0.4, -1.1
    y_exp = po.lift_compress(x_h.astype(np.float64), log_tau, log_eps, dim)
    gx_exp, gt_exp, ge_exp, scale_tau, scale_eps = po.lift_compress_backward(
        x_h.astype(np.float64), gy_h.astype(np.float64), log_tau, log_eps, dim, with_scales=True)
    m = _module(dim, True, True, log_tau, log_eps, torch.float32)
    runs = []
    for _ in range(3):
        m.zero_grad()
        x = torch.from_numpy(x_h).cuda().requires_grad_(True)
        y = m(x)
        y.backward(torch.from_numpy(gy_h).cuda())
        runs.append((y.detach(), x.grad, m.lift.log_tau.grad.clone(), m.log_compression.log_eps.grad.clone()))
    y, gx, gt, ge = runs[0]
    assert helpers.rel_err(y.cpu().numpy(), y_exp) <= 1e-5
    assert helpers.rel_err(gx.cpu().numpy(), gx_exp) <= 1e-5
    assert _close_sum(float(gt), gt_exp, scale_tau, 1e-5) and _close_sum(float(ge), ge_exp, scale_eps, 1e-5)
    for other in runs[1:]:
        assert all(torch.equal(a, b) for a, b in zip(runs[0], other)), "two runs differ"


def test_function_with_tau_itself_and_a_pointer_off_the_16_byte_grid():
    """``dilation_lift(input, tau, dim)`` takes tau, not its logarithm; a view that starts 4 bytes into a buffer."""
    gen = torch.Generator(device="cuda").manual_seed(9)
    base = torch.randn(4 * 6 * 8 + 1, device="cuda", generator=gen)
    x = base[1:].view(4, 6, 8).requires_grad_(True)
    assert x.data_ptr() % 16 != 0
    tau = torch.tensor(1.3, device="cuda", requires_grad=True)
    gy = torch.randn(4, 6, 8, device="cuda", generator=gen)
    y = layers.dilation_lift(x, tau, 1)
    y.backward(gy)
    x_h, gy_h = x.detach().cpu().numpy().astype(np.float64), gy.cpu().numpy().astype(np.float64)
    assert helpers.rel_err(y.detach().cpu().numpy(), po.dilation_lift(x_h, 1.3, 1)) <= 1e-5
    gx_exp, g_log_tau, _ = po.lift_compress_backward(x_h, gy_h, float(np.log(1.3)), None, 1)
    assert helpers.rel_err(x.grad.cpu().numpy(), gx_exp) <= 1e-5
    assert abs(float(tau.grad) - g_log_tau / 1.3) <= 1e-4 * max(1.0, abs(g_log_tau / 1.3))


def test_gradcheck_in_float64():
    gen = torch.Generator(device="cuda").manual_seed(2)
    x = (torch.rand(3, 5, 4, device="cuda", dtype=torch.float64, generator=gen) + 0.1).requires_grad_(True)
    log_tau = torch.tensor(0.2, device="cuda", dtype=torch.float64, requires_grad=True)
    log_eps = torch.tensor(-0.5, device="cuda", dtype=torch.float64, requires_grad=True)
    assert torch.autograd.gradcheck(lambda a, b, c: layers.lift_compress(a, b, c, 1), (x, log_tau, log_eps))
    assert torch.autograd.gradcheck(lambda a, b: layers.lift_compress(a, b, None, -1), (x, log_tau))
    assert torch.autograd.gradcheck(lambda a, c: layers.lift_compress(a, None, c, 0), (x, log_eps))


def test_half_input_is_computed_in_float32():
    gen = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(3, 9, 16, device="cuda", generator=gen)
    m = _module(1, True, True, 0.1, -0.3, torch.float32)
    y16 = m(x.half())
    assert y16.dtype == torch.float16
    assert float((y16.float() - m(x.half().float())).abs().max()) <= 2e-3 * float(m(x).abs().max())


def test_errors_and_empty_input():
    m = layers.DilationLift(3).cuda()
    with pytest.raises(RuntimeError, match="3 not a valid dimension for a tensor if dimension 3"):
        m(torch.zeros(2, 3, 4, device="cuda"))
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        layers.LogCompression()(torch.zeros(2, 3))
    x = torch.zeros(0, 5, 4, device="cuda", requires_grad=True)
    pair = layers.LogCompressionLift(dim=1).cuda()
    y = pair(x)
    assert y.shape == (0, 5, 4)
    y.sum().backward()
    assert float(pair.lift.log_tau.grad) == 0.0 and float(pair.log_compression.log_eps.grad) == 0.0
    # a workspace below the library's answer is refused
    x = torch.ones(2, 3, 4, device="cuda")
    with pytest.raises(capi.MellinError) as err:
        capi.lift_compress_backward(x, x, None, None, False, 2, 3, 4, torch.empty_like(x), None, None,
                                    workspace=torch.empty(64, dtype=torch.uint8, device="cuda"))
    assert err.value.code == 3
    assert capi.device_status() == 0
