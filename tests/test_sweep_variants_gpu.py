"""Stride / dilation variants of the wide 1-D operators (the large-shape sweep's cells).

* Linear stride / dilation 2 are computed as stride-1, dilation-1 operators on
  de-interleaved tensors (polyphase forms); small batches of the 1-D Mellin
  operator are padded to the 16 positions the tensor-core kernels need.  Both
  rewrites are checked here against the CPU oracle on whole tensors at sizes it
  finishes in seconds, for forward, grad-input and grad-weight.
* At the sweep's full size (batch 64, 256 -> 256 channels, 16384 samples,
  64 taps) every (stride, dilation) cell is checked on sampled outputs against
  float64 sums taken from the definition.
"""
import numpy as np
import pytest
import torch

import capi
import helpers
from oracle.oracle import Oracle

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5


@pytest.fixture(scope="module")
def oracle():
    return Oracle("reference") if Oracle.reference_available() else Oracle("port")


def _run_layer(x_h, w_h, b_h, go_shape, s, d, p, rng):
    x, w, b = (torch.from_numpy(a).cuda() for a in (x_h, w_h, b_h))
    y = torch.full(go_shape, float("nan"), device="cuda")
    capi.forward(x, w, b, y, s, d, p, (1, 1))
    go_h = rng.standard_normal(go_shape).astype(np.float32)
    go = torch.from_numpy(go_h).cuda()
    gx = torch.full_like(x, float("nan"))
    capi.grad_input(w, go, gx, s, d, p, (1, 1))
    gw = torch.full_like(w, float("nan"))
    gb = torch.full_like(b, float("nan"))
    capi.grad_weight(x, go, gw, gb, s, d, p, (1, 1))
    torch.cuda.synchronize()
    return y.cpu().numpy(), go_h, gx.cpu().numpy(), gw.cpu().numpy(), gb.cpu().numpy()


@pytest.mark.parametrize("sd", [(1, 2), (2, 1), (2, 2)], ids=lambda v: "s%d_d%d" % v)
@pytest.mark.parametrize("shape", [
    # (batch, c_in, c_out, Mellin extent, linear extent, Mellin taps, linear taps)
    (3, 16, 32, 1, 203, 1, 9),     # 1-D linear operator, odd lengths
    (2, 24, 40, 5, 128, 2, 4),     # 2-D layer with a strided / dilated linear axis
], ids=["linear_1d", "layer_2d"])
def test_linear_stride_and_dilation_two_match_the_oracle(oracle, shape, sd):
    n, ci, co, ngx, ngy, nfx, nfy = shape
    s, d, p = (1, sd[0]), (1, sd[1]), (0, 0)
    rng = np.random.default_rng(5 + sd[0] * 2 + sd[1])
    x_h = rng.standard_normal((n, ci, ngx, ngy)).astype(np.float32)
    w_h = (rng.standard_normal((co, ci, nfx, nfy)) / np.sqrt(ci * nfx * nfy)).astype(np.float32)
    b_h = rng.standard_normal(co).astype(np.float32)
    r = (ngx - oracle.mcorr_valid_size(nfx, ngx), 0)
    y_exp = oracle.mcorrlcorr(x_h, w_h, b_h, s, d, p, (1, 1), r)
    y, go_h, gx, gw, gb = _run_layer(x_h, w_h, b_h, y_exp.shape, s, d, p, rng)
    gx_exp, gw_exp, gb_exp = oracle.mcorrlcorr_backward(x_h.astype(np.float64), w_h.astype(np.float64),
                                                        go_h.astype(np.float64), s, d, p, (1, 1))
    assert helpers.rel_err(y, y_exp) <= F32_TOL
    assert helpers.rel_err(gx, gx_exp) <= F32_TOL
    assert helpers.rel_err(gw, gw_exp) <= F32_TOL
    assert helpers.rel_err(gb, gb_exp) <= F32_TOL
    assert capi.device_status() == 0


@pytest.mark.parametrize("batch", [2, 5, 8, 12, 20])
def test_wide_1d_mellin_with_small_batches_matches_the_oracle(oracle, batch):
    ci, co, length, taps = 32, 48, 96, 6
    rng = np.random.default_rng(batch)
    x_h = rng.standard_normal((batch, ci, length, 1)).astype(np.float32)
    w_h = (rng.standard_normal((co, ci, taps, 1)) / np.sqrt(ci * taps)).astype(np.float32)
    b_h = rng.standard_normal(co).astype(np.float32)
    s, d, p = (1, 1), (2, 1), (0, 0)
    r = (length - oracle.mcorr_valid_size(taps, length, 1, 2), 0)  # same-size output
    y_exp = oracle.mcorrlcorr(x_h, w_h, b_h, s, d, p, (1, 1), r)
    y, go_h, gx, gw, gb = _run_layer(x_h, w_h, b_h, y_exp.shape, s, d, p, rng)
    gx_exp, gw_exp, gb_exp = oracle.mcorrlcorr_backward(x_h.astype(np.float64), w_h.astype(np.float64),
                                                        go_h.astype(np.float64), s, d, p, (1, 1))
    assert helpers.rel_err(y, y_exp) <= F32_TOL
    assert helpers.rel_err(gx, gx_exp) <= F32_TOL
    assert helpers.rel_err(gw, gw_exp) <= F32_TOL
    assert helpers.rel_err(gb, gb_exp) <= F32_TOL


# ---- the sweep's full size: sampled outputs against the definition in float64 ----------------------------
N, C, L, K = 64, 256, 16384, 64


def _sample_forward(x, w, y, kind, s, d, rng, count=12):
    """y[n, a, t] against sum_{b, k} w[a, b, k] x[n, b, index(t, k)] in float64 for `count` random (n, a, t)."""
    worst = 0.0
    scale = float(y.abs().max())
    xd, wd = x.double(), w.double()
    nh = y.shape[2] if kind == "mellin" else y.shape[3]
    for _ in range(count):
        n, a, t = int(rng.integers(N)), int(rng.integers(C)), int(rng.integers(nh))
        total = 0.0
        ks = torch.arange(K, device="cuda")
        if kind == "mellin":
            idx = (t + s) * (ks + d) - 1
            ok = idx < L
            total = float((wd[a, :, ks[ok], 0] * xd[n, :, idx[ok], 0]).sum())
            got = float(y[n, a, t, 0])
        else:
            idx = s * t + d * ks
            ok = idx < L
            total = float((wd[a, :, 0, ks[ok]] * xd[n, :, 0, idx[ok]]).sum())
            got = float(y[n, a, 0, t])
        worst = max(worst, abs(got - total) / scale)
    return worst


@pytest.mark.parametrize("sd", [(1, 2), (2, 1)], ids=lambda v: "s%d_d%d" % v)
@pytest.mark.parametrize("kind", ["mellin", "linear"])
def test_full_size_sweep_cells_match_the_definition(kind, sd):
    s, d = sd
    gen = torch.Generator(device="cuda").manual_seed(17 + 2 * s + d)
    rng = np.random.default_rng(3)
    I = __import__("ctypes").c_int64
    if kind == "mellin":
        xs, ws = (N, C, L, 1), (C, C, K, 1)
        S, D, P = (s, 1), (d, 1), (0, 0)
        ys = (N, C, L, 1)  # same-size output
    else:
        nh = int(capi.lib().mellin_lcorr_valid_size(I(K), I(L), I(s), I(d), I(0), I(1)))
        xs, ws, ys = (N, C, 1, L), (C, C, 1, K), (N, C, 1, nh)
        S, D, P = (1, s), (1, d), (0, 0)
    x = torch.randn(xs, device="cuda", generator=gen)
    w = torch.randn(ws, device="cuda", generator=gen) / float(np.sqrt(C * K))
    y = torch.empty(ys, device="cuda")
    capi.forward(x, w, None, y, S, D, P, (1, 1))
    assert _sample_forward(x, w, y, kind, s, d, rng) <= F32_TOL
    # the three kernels are one bilinear form: <go, y> = <gx, x> = <gw, w>
    go = torch.randn(ys, device="cuda", generator=gen)
    gx = torch.empty_like(x)
    capi.grad_input(w, go, gx, S, D, P, (1, 1))
    gw = torch.empty_like(w)
    capi.grad_weight(x, go, gw, None, S, D, P, (1, 1))
    form = float((go.double() * y.double()).sum())
    scale = float(go.double().norm() * y.double().norm())
    assert abs(float((gx.double() * x.double()).sum()) - form) <= F32_TOL * scale
    assert abs(float((gw.double() * w.double()).sum()) - form) <= F32_TOL * scale
    assert capi.device_status() == 0


# ---- operator-level entry points (accumulate into h, transposition flags, no workspace) on wide layers ----
@pytest.mark.parametrize("flags", [(0, 0, 0), (1, 0, 0), (0, 1, 0), (0, 0, 1), (1, 1, 1)], ids=lambda f: "t%d%d%d" % f)
@pytest.mark.parametrize("kind", ["corr", "conv"])
def test_operator_level_calls_on_wide_layers_match_the_oracle(oracle, kind, flags):
    """These reach the tensor-core kernels through library-owned scratch; the oracle is the reference's own
    operator with the same flags, accumulating into the same pre-filled output."""
    tf, tg, th = flags
    n, ci, co, ng, nf = 3, 24, 40, (12, 96), (4, 3)
    s, d, p, u = (1, 1), (2, 1), (0, 1), (1, 1)
    rng = np.random.default_rng(41)
    f_h = (rng.standard_normal(((ci, co) if tf else (co, ci)) + nf) / np.sqrt(ci * 12)).astype(np.float32)
    g_h = rng.standard_normal(((ci, n) if tg else (n, ci)) + ng).astype(np.float32)
    if kind == "corr":
        nh = (ng[0], oracle.lcorr_valid_size(nf[1], ng[1], s[1], d[1], p[1], u[1]) + 1)
    else:
        nh = (oracle.mconv_support_size(nf[0], ng[0], s[0], d[0], p[0], u[0]),
              oracle.lconv_valid_size(nf[1], ng[1], s[1], d[1], p[1], u[1]) + 2)
    h0 = rng.standard_normal(((co, n) if th else (n, co)) + nh).astype(np.float32)
    h_exp = oracle.op2d(kind, f_h, g_h, h0.copy(), co, ci, n, s, d, p, u, bool(tf), bool(tg), bool(th))
    f, g, h = (torch.from_numpy(a).cuda() for a in (f_h, g_h, h0))
    capi.op2d("mcorrlcorr" if kind == "corr" else "mconvlconv", f, g, h, co, ci, n, s, d, p, u, bool(tf), bool(tg), bool(th))
    torch.cuda.synchronize()
    assert helpers.rel_err(h.cpu().numpy(), h_exp) <= F32_TOL
    assert capi.device_status() == 0


@pytest.mark.parametrize("sd", [(1, 1), (2, 1), (1, 2), (2, 2)], ids=lambda v: "s%d_d%d" % v)
def test_operator_level_linear_1d_variants_match_the_oracle(oracle, sd):
    n, ci, co, length, taps = 2, 16, 32, 200, 8
    s, d = (1, sd[0]), (1, sd[1])
    rng = np.random.default_rng(43)
    f_h = (rng.standard_normal((co, ci, 1, taps)) / np.sqrt(ci * taps)).astype(np.float32)
    g_h = rng.standard_normal((n, ci, 1, length)).astype(np.float32)
    nh = (1, oracle.lcorr_valid_size(taps, length, sd[0], sd[1], 0, 1))
    h0 = rng.standard_normal((n, co) + nh).astype(np.float32)
    h_exp = oracle.op2d("corr", f_h, g_h, h0.copy(), co, ci, n, s, d, (0, 0), (1, 1))
    f, g, h = (torch.from_numpy(a).cuda() for a in (f_h, g_h, h0))
    capi.op2d("mcorrlcorr", f, g, h, co, ci, n, s, d, (0, 0), (1, 1))
    torch.cuda.synchronize()
    assert helpers.rel_err(h.cpu().numpy(), h_exp) <= F32_TOL


def test_operator_level_1d_mellin_reaches_the_fast_kernels(oracle):
    """mellin_mcorr1d_f32 / mellin_mconv1d_f32 at the sweep's channel counts (reduced length and batch): parity with
    the oracle, and a time that is the tensor-core path's, not the per-output kernel's."""
    n, c, length, taps = 8, 256, 2048, 64
    rng = np.random.default_rng(47)
    f_h = (rng.standard_normal((c, c, taps)) / np.sqrt(c * taps)).astype(np.float32)
    g_h = rng.standard_normal((n, c, length)).astype(np.float32)
    f, g = torch.from_numpy(f_h).cuda(), torch.from_numpy(g_h).cuda()
    for kind, name in (("corr", "mcorr1d"), ("conv", "mconv1d")):
        nh = length if kind == "corr" else oracle.mconv_support_size(taps, length, 1, 1, 0, 1) // 4
        h = torch.zeros((n, c, nh), device="cuda")
        capi.op1d(name, f, g, h, c, c, n, 1, 1, 0, 1)  # warm-up: tables, scratch
        h.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        capi.op1d(name, f, g, h, c, c, n, 1, 1, 0, 1)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        # sampled outputs in float64 from the definition
        worst, scale = 0.0, float(h.abs().max())
        fd, gd = f.double(), g.double()
        ks = torch.arange(taps, device="cuda")
        for _ in range(10):
            b, a, t = int(rng.integers(n)), int(rng.integers(c)), int(rng.integers(nh))
            if kind == "corr":
                idx = (t + 1) * (ks + 1) - 1
                ok = idx < length
            else:
                ok = ((t + 1) % (ks + 1)) == 0
                idx = torch.div(t + 1, ks + 1, rounding_mode="floor") - 1
                ok = ok & (idx >= 0) & (idx < length)
            total = float((fd[a][:, ks[ok]] * gd[b][:, idx[ok]]).sum())
            worst = max(worst, abs(float(h[b, a, t]) - total) / scale)
        assert worst <= F32_TOL, (name, worst)
        flop = 2.0 * n * c * c * (77701 / 16384.0 * nh if kind == "corr" else nh * 4)  # rough: pairs per output
        assert ms < 20.0, "%s took %.1f ms: the per-output kernel, not the tensor-core path" % (name, ms)
