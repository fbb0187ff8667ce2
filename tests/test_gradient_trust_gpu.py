"""The gradient kernels must give the same, right answer on every launch.

The reference's kernels are atomics-free and repeatable (its own suite checks
that an operator gives the CPU's answer 1, 2 and 10 times in a row,
tests/test_mconv.py:894-919).  These tests hold the first-layer kernels (the
row-streaming weight gradient and grad-input, the tensor-core forward) to
that, in the two regimes where a race once hid:

* the first launch over freshly written tensors of a geometry seen for the
  first time (a warp could read a tile's tap mask before the issuing thread
  had published it -- only when the copies completed unusually fast);
* many launches at the full benchmark shape.

Every result is compared with a float64 sum taken from the definition, not
only with another launch.  The last test is the bounded-wait self-test: a
launch that waits on a barrier nothing arms must come back and raise the
device status word.
"""
import numpy as np
import pytest
import torch

import capi
import helpers
from oracle.oracle import Oracle

pytestmark = pytest.mark.gpu

S, P, U = (1, 1), (0, 1), (1, 1)
F32_TOL = 1e-5


def _grad_w_definition(x, go, nf, d):
    """float64 weight gradient from the definition, on the device: for every Mellin tap the
    output rows ox with (ox + 1)(kx + d) - 1 inside the input, times the three linear taps."""
    ngx, ngy = x.shape[2:]
    xp = torch.nn.functional.pad(x.double(), (1, 1))
    god = go.double()
    gw = torch.zeros((go.shape[1], x.shape[1]) + tuple(nf), dtype=torch.float64, device=x.device)
    for kx in range(nf[0]):
        oxs = [ox for ox in range(ngx) if (ox + 1) * (kx + d[0]) - 1 < ngx]
        if not oxs:
            continue
        ixs = [(ox + 1) * (kx + d[0]) - 1 for ox in oxs]
        g = god[:, :, oxs, :]
        for ky in range(nf[1]):
            gw[:, :, kx, ky] = torch.einsum("naoy,nboy->ab", g, xp[:, :, ixs, ky * d[1]:ky * d[1] + ngy])
    return gw


def _rel(a, b):
    return float((a.double() - b.double()).abs().max() / b.double().abs().max())


def test_first_launch_over_fresh_tensors_is_right():
    """60 geometries, each new to the library, each over tensors written just before the launch."""
    gen = torch.Generator(device="cuda").manual_seed(5)
    n, ci, co, nf, d = 4, 3, 64, (8, 3), (1, 1)
    worst = 0.0
    for trial in range(60):
        ngx = 20 + trial % 40
        ngy = 4 * (32 + (trial * 7) % 40)
        x = torch.randn((n, ci, ngx, ngy), device="cuda", generator=gen)
        go = torch.randn((n, co, ngx, ngy), device="cuda", generator=gen)
        for _ in range(2):
            gw = torch.full((co, ci) + nf, float("nan"), device="cuda")
            gb = torch.full((co,), float("nan"), device="cuda")
            capi.grad_weight(x, go, gw, gb, S, d, P, U)
            exact_w = _grad_w_definition(x, go, nf, d)
            exact_b = go.double().sum(dim=(0, 2, 3))
            worst = max(worst, _rel(gw, exact_w), _rel(gb, exact_b))
            assert _rel(gw, exact_w) <= F32_TOL, (trial, ngx, ngy)
            assert _rel(gb, exact_b) <= F32_TOL, (trial, ngx, ngy)
    assert capi.device_status() == 0


def test_benchmark_layer_is_bit_repeatable_and_right_30_times():
    """Forward, grad-input and weight gradient of the 3 -> 64 layer at batch 32, 41 x 800."""
    n, ci, co, ng, nf, d = 32, 3, 64, (41, 800), (8, 3), (1, 1)
    gen = torch.Generator(device="cuda").manual_seed(77)
    x = torch.randn((n, ci) + ng, device="cuda", generator=gen)
    w = torch.randn((co, ci) + nf, device="cuda", generator=gen) / float(np.sqrt(ci * nf[0] * nf[1]))
    bias = torch.randn(co, device="cuda", generator=gen)
    go = torch.randn((n, co) + ng, device="cuda", generator=gen)
    exact_w = _grad_w_definition(x, go, nf, d)
    exact_b = go.double().sum(dim=(0, 2, 3))
    # float64 forward / grad-input from the same definition through autograd on a float64 copy
    first = None
    for rep in range(30):
        y = torch.full_like(go, float("nan"))
        gx = torch.full_like(x, float("nan"))
        gw = torch.full_like(w, float("nan"))
        gb = torch.full_like(bias, float("nan"))
        capi.forward(x, w, bias, y, S, d, P, U)
        capi.grad_input(w, go, gx, S, d, P, U)
        capi.grad_weight(x, go, gw, gb, S, d, P, U)
        if first is None:
            first = (y, gx, gw, gb)
            assert _rel(gw, exact_w) <= F32_TOL and _rel(gb, exact_b) <= F32_TOL
            # the three kernels are one bilinear form: <go, y - bias> = <gx, x> = <gw, w>
            form = float(((y - bias.view(1, -1, 1, 1)).double() * go.double()).sum())
            scale = float(go.double().norm() * y.double().norm())
            assert abs(float((gx.double() * x.double()).sum()) - form) <= F32_TOL * scale
            assert abs(float((exact_w * w.double()).sum()) - form) <= F32_TOL * scale
        else:
            for got, ref, name in zip((y, gx, gw, gb), first, ("y", "grad_x", "grad_w", "grad_b")):
                assert torch.equal(got, ref), "%s differs on launch %d" % (name, rep)
    assert capi.device_status() == 0


@pytest.mark.parametrize("shape", [
    # (batch, c_in, c_out, (ngx, ngy), (nfx, nfy), d)
    (4, 3, 64, (41, 200), (8, 3), (1, 1)),
    (3, 2, 96, (24, 132), (6, 3), (2, 1)),
    (2, 24, 40, (12, 96), (4, 3), (2, 1)),
], ids=["first_layer", "two_channels", "wide_layer"])
def test_regular_and_no_alloc_entry_points_alternate_against_the_oracle(shape):
    n, ci, co, ng, nf, d = shape
    oracle = Oracle("reference") if Oracle.reference_available() else Oracle("port")
    rng = np.random.default_rng(11)
    for rep in range(20):
        x_h = rng.standard_normal((n, ci) + ng).astype(np.float32)
        go_h = rng.standard_normal((n, co) + ng).astype(np.float32)
        w_h = np.zeros((co, ci) + nf, dtype=np.float32)
        # float64 oracle: the float32 CPU sum is itself ~1e-5 off for long reductions
        _, gw_exp, gb_exp = oracle.mcorrlcorr_backward(x_h.astype(np.float64), w_h.astype(np.float64),
                                                       go_h.astype(np.float64), S, d, P, U)
        x, go = torch.from_numpy(x_h).cuda(), torch.from_numpy(go_h).cuda()
        for which in (capi.grad_weight, capi.grad_weight_noalloc):
            gw = torch.full((co, ci) + nf, float("nan"), device="cuda")
            gb = torch.full((co,), float("nan"), device="cuda")
            which(x, go, gw, gb, S, d, P, U)
            assert helpers.rel_err(gw.cpu().numpy(), gw_exp) <= F32_TOL, (rep, which.__name__)
            assert helpers.rel_err(gb.cpu().numpy(), gb_exp) <= F32_TOL, (rep, which.__name__)
    assert capi.device_status() == 0


def test_a_wait_nobody_answers_gives_up_and_raises_the_status_word():
    assert capi.device_status() == 0
    capi.selftest_unarmed_wait()
    assert capi.device_status() == 202  # 200 + code 2: the self-test's barrier
    assert capi.device_status() == 0    # reading clears it
    # the context is still usable
    x = torch.randn((2, 3, 20, 64), device="cuda")
    go = torch.randn((2, 8, 20, 64), device="cuda")
    gw = torch.empty((8, 3, 4, 3), device="cuda")
    capi.grad_weight(x, go, gw, None, S, (1, 1), P, U)
    assert _rel(gw, _grad_w_definition(x, go, (4, 3), (1, 1))) <= F32_TOL
