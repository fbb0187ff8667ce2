"""Parity of the CUDA kernels with the CPU oracle, called through the C ABI
(raw device pointers via ctypes), on a B200."""
import itertools

import numpy as np
import pytest
import torch

import capi
import helpers
from oracle.oracle import Oracle

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5  # max|a-b| / max|b| per tensor, the tolerance the parity target states for FP32
F64_TOL = 1e-12


@pytest.fixture(scope="module")
def oracle():
    return Oracle("reference") if Oracle.reference_available() else Oracle("port")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


def _conv_ids():
    return [(op, i) for op in helpers.KAT_CONV_OPS for i in range(len(helpers.kat()[op]))]


def _col_ids():
    return [(op, i) for op in helpers.KAT_COL_OPS for i in range(len(helpers.kat()[op]))]


@pytest.mark.parametrize("op,idx", _conv_ids(), ids=lambda v: str(v))
@pytest.mark.parametrize("dtype,tol", [(np.float64, 1e-10), (np.float32, 2e-5)])
def test_known_answers_conv(op, idx, dtype, tol):
    """All 63 convolution/correlation known-answer cases, every transposition
    flag, batch 1 and 3, outputs shorter / equal / longer than the support."""
    prob = helpers.kat_conv_problem(op, idx, dtype)
    f, g = prob["f"], prob["g"]
    co, ci = f.shape[:2]
    name = "mcorrlcorr" if prob["kind"] == "corr" else "mconvlconv"
    for extra, batch, tf, tg, th in itertools.product((-1, 0, 3), (1, 3), (False, True), (False, True), (False, True)):
        gb = np.repeat(g, batch, axis=0)
        exp = np.repeat(helpers.pad_or_crop(prob["h"], extra), batch, axis=0)
        fa = f.transpose(1, 0, 2, 3) if tf else f
        ga = gb.transpose(1, 0, 2, 3) if tg else gb
        shape = exp.shape if not th else (exp.shape[1], exp.shape[0]) + exp.shape[2:]
        h = torch.full(shape, 0.75, dtype=torch.from_numpy(np.zeros(1, dtype)).dtype, device="cuda")
        capi.op2d(name, dev(fa), dev(ga), h, co, ci, batch, prob["s"], prob["d"], prob["p"], prob["u"], tf, tg, th)
        got = host(h)
        got = got.transpose(1, 0, 2, 3) if th else got
        np.testing.assert_allclose(got, exp + 0.75, rtol=0, atol=tol * max(1.0, np.abs(exp).max(initial=0.0)))


@pytest.mark.parametrize("op,idx", [(o, i) for o, i in _conv_ids() if o in ("mcorr1d", "mconv1d")], ids=lambda v: str(v))
def test_known_answers_1d_entry_points(op, idx):
    prob = helpers.kat_conv_problem(op, idx, np.float64)
    f, g, exp = prob["f"][..., 0], prob["g"][..., 0], prob["h"][..., 0]
    h = torch.zeros(exp.shape, dtype=torch.float64, device="cuda")
    capi.op1d(op, dev(f), dev(g), h, f.shape[0], f.shape[1], 1, prob["s"][0], prob["d"][0], prob["p"][0], prob["u"][0])
    np.testing.assert_allclose(host(h), exp, rtol=0, atol=1e-10)


@pytest.mark.parametrize("op,idx", _col_ids(), ids=lambda v: str(v))
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_known_answers_col(op, idx, dtype):
    prob = helpers.kat_col_problem(op, idx, dtype)
    for batch, tg, tgg in itertools.product((1, 2), (False, True), (False, True)):
        g = np.repeat(prob["g"], batch, axis=0)
        gg = np.repeat(prob["gg"], batch, axis=0)
        ga = np.swapaxes(g, 0, 1) if tg else g
        gga = np.swapaxes(gg, 0, 1) if tgg else gg
        ci = g.shape[1]
        if prob["direction"] == "gather":
            out = torch.full(gga.shape, -12345.0, dtype=dev(gga).dtype, device="cuda")
            capi.col2d("spec2col", dev(ga), out, ci, batch, prob["nf"], g.shape[2:], gg.shape[4:],
                       prob["s"], prob["d"], prob["p"], prob["u"], tg, tgg)
            np.testing.assert_allclose(host(out), gga, rtol=0, atol=1e-6)
        else:
            out = torch.full(ga.shape, -12345.0, dtype=dev(ga).dtype, device="cuda")
            capi.col2d("col2spec", dev(gga), out, ci, batch, prob["nf"], g.shape[2:], gg.shape[4:],
                       prob["s"], prob["d"], prob["p"], prob["u"], tg, tgg)
            np.testing.assert_allclose(host(out), ga, rtol=0, atol=1e-5)


def test_col_1d_entry_points():
    arrays, meta = helpers.ext_cases()
    m = meta["snd2col"]
    x, gg_exp = arrays["snd2col.x"], arrays["snd2col.gg"]
    gg = torch.full(gg_exp.shape, -12345.0, device="cuda")
    capi.col1d("snd2col", dev(x), gg, x.shape[1], x.shape[0], m["kernel_width"], x.shape[2], gg_exp.shape[3],
               m["s"], m["d"], m["p"], m["u"])
    np.testing.assert_array_equal(host(gg), gg_exp)
    back = torch.full(x.shape, -12345.0, device="cuda")
    capi.col1d("col2snd", dev(arrays["snd2col.cot"]), back, x.shape[1], x.shape[0], m["kernel_width"], x.shape[2],
               gg_exp.shape[3], m["s"], m["d"], m["p"], m["u"])
    assert helpers.rel_err(host(back), arrays["snd2col.back"]) <= 1e-6
    m = meta["spec2col"]
    x, gg_exp = arrays["spec2col.x"], arrays["spec2col.gg"]
    gg = torch.full(gg_exp.shape, -12345.0, device="cuda")
    capi.col2d("spec2col", dev(x), gg, x.shape[1], x.shape[0], m["kernel_size"], x.shape[2:], gg_exp.shape[4:],
               m["s"], m["d"], m["p"], m["u"])
    np.testing.assert_array_equal(host(gg), gg_exp)
    back = torch.full(x.shape, -12345.0, device="cuda")
    capi.col2d("col2spec", dev(arrays["spec2col.cot"]), back, x.shape[1], x.shape[0], m["kernel_size"], x.shape[2:],
               gg_exp.shape[4:], m["s"], m["d"], m["p"], m["u"])
    assert helpers.rel_err(host(back), arrays["spec2col.back"]) <= 1e-6


@pytest.fixture(params=["tensor_cores", "cuda_cores"])
def engine(request):
    """Run a test once on the tcgen05 kernels and once on the CUDA-core kernels;
    afterwards the tensor-core kernels' timeout flag must still be clear."""
    previous = capi.set_tensor_cores(request.param == "tensor_cores")
    yield request.param
    capi.set_tensor_cores(previous)
    assert capi.device_status() == 0


def layer_all(x, w, b, go, s, d, p, u):
    """forward, grad_input, grad_weight (+bias) through the layer-level entry points."""
    xt, wt, got = dev(x), dev(w), dev(go)
    bt = None if b is None else dev(b)
    y = torch.full(go.shape, float("nan"), dtype=got.dtype, device="cuda")
    capi.forward(xt, wt, bt, y, s, d, p, u)
    gx = torch.full(x.shape, float("nan"), dtype=got.dtype, device="cuda")
    capi.grad_input(wt, got, gx, s, d, p, u)
    gw = torch.full(w.shape, float("nan"), dtype=got.dtype, device="cuda")
    gb = torch.full((w.shape[0],), float("nan"), dtype=got.dtype, device="cuda")
    capi.grad_weight(xt, got, gw, gb, s, d, p, u)
    return host(y), host(gx), host(gw), host(gb)


def _ext_names():
    _, meta = helpers.ext_cases()
    return [k for k, v in meta.items() if v.get("kind") in ("1d", "2d")]


@pytest.mark.parametrize("name", _ext_names())
@pytest.mark.parametrize("tag,dtype,tol", [("f32", np.float32, F32_TOL), ("f64", np.float64, F64_TOL)])
def test_layer_against_reference_extension(engine, name, tag, dtype, tol):
    """Outputs and all gradients vs what the reference's CPU torch extension
    produced for the same inputs (recorded in tests/golden/)."""
    arrays, meta = helpers.ext_cases()
    m = meta[name]
    x, w, go = (arrays["%s.%s" % (name, k)].astype(dtype) for k in ("x", "w", "go"))
    b = arrays[name + ".b"].astype(dtype) if m["bias"] else None
    s, d, p, u = m["s"], m["d"], m["p"], m["u"]
    if m["kind"] == "1d":
        x, w, go = x[..., None], w[..., None], go[..., None]
        s, d, p, u = (s, 1), (d, 1), (p, 0), (u, 1)
    y, gx, gw, gb = layer_all(x, w, b, go, s, d, p, u)
    exp = {k: arrays["%s.%s.%s" % (name, k, tag)] for k in ("y", "gx", "gw")}
    if m["kind"] == "1d":
        y, gx, gw = y[..., 0], gx[..., 0], gw[..., 0]
    assert helpers.rel_err(y, exp["y"]) <= tol
    assert helpers.rel_err(gx, exp["gx"]) <= tol
    assert helpers.rel_err(gw, exp["gw"]) <= tol
    if m["bias"]:
        assert helpers.rel_err(gb, arrays["%s.gb.%s" % (name, tag)]) <= tol


# (batch, c_in, c_out, (ngx, ngy), (nfx, nfy), s, d, p, u, r): shapes chosen to
# reach every tile-kernel variant (channel counts above/below the register
# tiles, ragged linear extents, 1..5 linear taps, dilated Mellin axis)
RANDOM_CASES = [
    (2, 3, 64, (41, 100), (8, 3), (1, 1), (1, 1), (0, 1), (1, 1), ("same", 1)),
    (2, 3, 64, (41, 97), (8, 3), (1, 1), (1, 1), (0, 1), (1, 1), (0, 1)),
    (1, 64, 128, (41, 50), (6, 3), (1, 1), (2, 1), (0, 1), (1, 1), ("same", 1)),
    (2, 7, 5, (12, 33), (4, 2), (1, 1), (1, 1), (0, 0), (1, 1), (3, 0)),
    (2, 9, 20, (10, 45), (3, 5), (2, 1), (1, 1), (1, 2), (1, 1), (2, 2)),
    (1, 4, 70, (9, 130), (3, 1), (1, 1), (1, 1), (0, 0), (1, 1), ("same", 0)),
    (2, 5, 6, (7, 40), (2, 3), (1, 2), (1, 2), (0, 2), (1, 1), (1, 1)),   # strided, dilated linear axis
    (2, 4, 4, (6, 24), (3, 7), (1, 1), (1, 1), (0, 3), (1, 1), (2, 3)),   # 7 linear taps: run-time tap path
    (3, 2, 3, (8, 20), (3, 3), (1, 1), (1, 1), (2, 1), (2, 3), (2, 1)),   # u != 1: divisor on the linear axis
    (2, 6, 9, (1, 200), (1, 5), (1, 1), (1, 1), (0, 2), (1, 1), (0, 2)),  # linear correlation only
    (4, 5, 7, (300, 1), (16, 1), (1, 1), (1, 1), (0, 0), (1, 1), (100, 0)),  # 1-D Mellin
    # wide layers whose linear extent is a multiple of 4: tensor-core weight gradient
    (2, 64, 128, (41, 48), (6, 3), (1, 1), (2, 1), (0, 1), (1, 1), ("same", 1)),
    (3, 20, 40, (12, 36), (3, 2), (1, 1), (1, 1), (0, 0), (1, 1), (2, 1)),       # partial channel tiles
    (2, 70, 130, (10, 52), (4, 3), (1, 1), (1, 2), (0, 2), (1, 1), (1, 2)),      # two tiles each way, dilated taps
    (1, 16, 32, (30, 200), (5, 1), (1, 1), (1, 1), (0, 0), (1, 1), ("same", 0)),  # one linear tap, long reduction
    # wide 1-D Mellin operators with a batch of >= 32: the batch stands in for the linear axis
    (32, 16, 32, (300, 1), (16, 1), (1, 1), (1, 1), (0, 0), (1, 1), ("same", 0)),
    (36, 20, 40, (200, 1), (12, 1), (2, 1), (2, 1), (1, 0), (1, 1), (50, 0)),     # s, d, p on the Mellin axis; ragged tiles
    (64, 32, 48, (700, 1), (64, 1), (1, 1), (1, 1), (0, 0), (1, 1), (0, 0)),      # table too long for shared memory
    (16, 16, 32, (120, 1), (7, 1), (1, 1), (1, 1), (0, 0), (1, 1), ("same", 0)),   # smallest batch that takes this path
    # wide linear 1-D operators (singleton Mellin axis): weight gradient in slices of three taps
    (2, 16, 32, (1, 400), (1, 8), (1, 1), (1, 1), (0, 0), (1, 1), (0, 0)),
    (3, 24, 40, (1, 240), (1, 7), (1, 1), (1, 2), (0, 3), (1, 1), (0, 5)),          # dilated taps, padding both sides
]


@pytest.mark.parametrize("case", RANDOM_CASES, ids=lambda c: "n%d_ci%d_co%d_g%s_f%s_s%s_d%s_p%s_u%s" % c[:9])
def test_layer_random_against_oracle(engine, oracle, case):
    n, ci, co, ng, nf, s, d, p, u, r = case
    rng = np.random.default_rng(abs(hash(case[:9])) % (2 ** 31))
    x = rng.standard_normal((n, ci) + ng).astype(np.float32)
    w = (rng.standard_normal((co, ci) + nf) / np.sqrt(ci * nf[0] * nf[1])).astype(np.float32)
    b = rng.standard_normal(co).astype(np.float32)
    if r[0] == "same":
        r = (ng[0] - oracle.mcorr_valid_size(nf[0], ng[0], s[0], d[0], p[0], u[0]), r[1])
    y_exp = oracle.mcorrlcorr(x, w, b, s, d, p, u, r)
    go = rng.standard_normal(y_exp.shape).astype(np.float32)
    gx_exp, gw_exp, gb_exp = oracle.mcorrlcorr_backward(x, w, go, s, d, p, u)
    # float64 referee: the FP32 CPU sum is itself only ~1e-6..1e-5 accurate
    o64 = oracle.mcorrlcorr_backward(x.astype(np.float64), w.astype(np.float64), go.astype(np.float64), s, d, p, u)
    y, gx, gw, gb = layer_all(x, w, b, go, s, d, p, u)
    assert helpers.rel_err(y, y_exp) <= F32_TOL
    assert helpers.rel_err(gx, gx_exp) <= F32_TOL
    assert helpers.rel_err(gw, o64[1]) <= max(F32_TOL, helpers.rel_err(gw_exp, o64[1]))
    assert helpers.rel_err(gb, o64[2]) <= max(F32_TOL, helpers.rel_err(gb_exp, o64[2]))
    # determinism: a second run is bit-identical (no atomics anywhere)
    y2, gx2, gw2, gb2 = layer_all(x, w, b, go, s, d, p, u)
    assert np.array_equal(y, y2) and np.array_equal(gx, gx2) and np.array_equal(gw, gw2) and np.array_equal(gb, gb2)


def test_batching_consistency():
    """A batch-N result equals N batch-1 results (the reference's
    c/tests/test_batching.cc property), through the operator-level entry point."""
    rng = np.random.default_rng(7)
    x = rng.standard_normal((5, 3, 20, 37)).astype(np.float32)
    w = rng.standard_normal((6, 3, 4, 3)).astype(np.float32)
    s, d, p, u = (1, 1), (1, 1), (0, 1), (1, 1)
    h = torch.zeros((5, 6, 20, 37), device="cuda")
    capi.op2d("mcorrlcorr", dev(w), dev(x), h, 6, 3, 5, s, d, p, u)
    full = host(h)
    for n in range(5):
        h1 = torch.zeros((1, 6, 20, 37), device="cuda")
        capi.op2d("mcorrlcorr", dev(w), dev(x[n:n + 1]), h1, 6, 3, 1, s, d, p, u)
        np.testing.assert_array_equal(host(h1)[0], full[n])


def test_empty_and_degenerate_inputs():
    z = torch.zeros((0, 3, 5, 8), device="cuda")
    w = torch.ones((4, 3, 2, 3), device="cuda")
    y = torch.zeros((0, 4, 2, 8), device="cuda")
    capi.forward(z, w, None, y, 1, 1, (0, 1), 1)  # empty batch: no launch, no error
    # output longer than the support on both axes: the tail holds the bias only
    x = torch.ones((1, 1, 3, 4), device="cuda")
    w = torch.ones((1, 1, 1, 1), device="cuda")
    b = torch.full((1,), 2.0, device="cuda")
    y = torch.full((1, 1, 6, 7), float("nan"), device="cuda")
    capi.forward(x, w, b, y, 1, 1, 0, 1)
    exp = np.full((6, 7), 2.0, dtype=np.float32)
    exp[:3, :4] += 1.0
    np.testing.assert_array_equal(host(y)[0, 0], exp)


def test_bad_arguments_are_reported():
    x = torch.ones((1, 1, 3, 4), device="cuda")
    w = torch.ones((1, 1, 1, 1), device="cuda")
    y = torch.zeros((1, 1, 3, 4), device="cuda")
    with pytest.raises(capi.MellinError) as e:
        capi.forward(x, w, None, y, 1, 1, (-1, 0), 1)  # Mellin p < 0
    assert e.value.code == 1
    with pytest.raises(capi.MellinError) as e:
        capi.forward(x, w, None, y, 1, 1, 0, (1, 0))  # zero divisor on the linear axis
    assert e.value.code == 1
    gw = torch.zeros((64, 3, 8, 3), device="cuda")
    xx = torch.zeros((2, 3, 41, 64), device="cuda")
    gy = torch.zeros((2, 64, 41, 64), device="cuda")
    with pytest.raises(capi.MellinError) as e:
        capi.grad_weight(xx, gy, gw, None, 1, 1, (0, 1), 1, workspace=torch.empty(16, dtype=torch.uint8, device="cuda"))
    assert e.value.code == 3
    torch.cuda.synchronize()  # the context is still healthy


MASKED_CASES = [
    # n, ci, co, (bins, frames), kernel, d, lens
    (5, 3, 64, (41, 300), (8, 3), (1, 1), [300, 257, 128, 40, 0]),      # narrow layer: resident weights
    (4, 64, 128, (41, 272), (6, 3), (2, 1), [272, 129, 127, 1]),         # wide layer: streamed weights
    (3, 5, 6, (9, 40), (3, 2), (1, 1), [40, 17, 3]),                     # CUDA-core kernels + the separate pass
]


@pytest.mark.parametrize("relu", [True, False])
@pytest.mark.parametrize("case", MASKED_CASES, ids=lambda c: "n%d_ci%d_co%d" % c[:3])
def test_fused_mask_and_relu_equal_the_separate_steps(engine, case, relu):
    """forward_masked = mask * act(forward): bit-identical to the plain forward followed
    by the mask and the activation (the fused epilogue touches no arithmetic)."""
    n, ci, co, ng, nf, d, lens = case
    rng = np.random.default_rng(n * 100 + ci)
    x = dev(rng.standard_normal((n, ci) + ng).astype(np.float32))
    w = dev((rng.standard_normal((co, ci) + nf) / np.sqrt(ci * nf[0] * nf[1])).astype(np.float32))
    b = dev(rng.standard_normal(co).astype(np.float32))
    lens_t = torch.tensor(lens, dtype=torch.int32, device="cuda")
    s, p, u = (1, 1), (0, 1), (1, 1)
    nhy = ng[1] + 2 - nf[1] + 1
    shape = (n, co, ng[0], nhy)
    plain = torch.empty(shape, device="cuda")
    capi.forward(x, w, b, plain, s, d, p, u)
    expected = plain.relu() if relu else plain.clone()
    mask = torch.arange(nhy, device="cuda")[None, :] < lens_t[:, None]
    expected = expected * mask[:, None, None, :]
    got = torch.full(shape, float("nan"), device="cuda")
    capi.forward_masked(x, w, b, lens_t, relu, got, s, d, p, u)
    assert torch.equal(got, expected)
    if ci == 5:  # float64 goes through the generic kernel and the separate pass
        got64 = torch.full(shape, float("nan"), device="cuda", dtype=torch.float64)
        capi.forward_masked(x.double(), w.double(), b.double(), lens_t, relu, got64, s, d, p, u)
        assert helpers.rel_err(got64.cpu().numpy(), expected.double().cpu().numpy()) <= F32_TOL


@pytest.mark.parametrize("case", MASKED_CASES[:2] + [(4, 128, 64, (41, 272), (6, 3), (2, 1), [272, 130, 128, 0])],
                         ids=lambda c: "n%d_ci%d_co%d" % c[:3])
def test_masked_grad_input_equals_the_plain_one_on_masked_gradients(engine, case):
    """grad_input_masked skips tiles that can only hold zeros: same bits as grad_input."""
    n, ci, co, ng, nf, d, lens = case
    rng = np.random.default_rng(n * 7 + co)
    w = dev((rng.standard_normal((co, ci) + nf) / np.sqrt(ci * nf[0] * nf[1])).astype(np.float32))
    lens_t = torch.tensor(lens, dtype=torch.int32, device="cuda")
    s, p, u = (1, 1), (0, 1), (1, 1)
    nhy = ng[1] + 2 - nf[1] + 1
    go = dev(rng.standard_normal((n, co, ng[0], nhy)).astype(np.float32))
    go = go * (torch.arange(nhy, device="cuda")[None, :] < lens_t[:, None])[:, None, None, :]
    plain = torch.empty((n, ci) + ng, device="cuda")
    capi.grad_input(w, go, plain, s, d, p, u)
    got = torch.full((n, ci) + ng, float("nan"), device="cuda")
    capi.grad_input_masked(w, go, lens_t, got, s, d, p, u)
    assert torch.equal(got, plain)


@pytest.mark.parametrize("case", [MASKED_CASES[1], (4, 128, 64, (41, 272), (6, 3), (2, 1), [272, 130, 16, 0]),
                                  (3, 20, 40, (12, 50), (3, 2), (1, 1), [49, 17, 30])],
                         ids=lambda c: "n%d_ci%d_co%d" % c[:3])
def test_masked_grad_weight_equals_the_plain_one_on_masked_gradients(engine, case):
    """The masked weight gradient stops each utterance's reduction at its length: the terms it
    leaves out are exact zeros, so it agrees with grad_weight to rounding of a different
    summation split (the slices' work is divided differently)."""
    n, ci, co, ng, nf, d, lens = case
    rng = np.random.default_rng(n * 11 + co)
    x = dev(rng.standard_normal((n, ci) + ng).astype(np.float32))
    lens_t = torch.tensor(lens, dtype=torch.int32, device="cuda")
    s, p, u = (1, 1), (0, 1), (1, 1)
    nhy = ng[1] + 2 - nf[1] + 1
    go = dev(rng.standard_normal((n, co, ng[0], nhy)).astype(np.float32))
    go = go * (torch.arange(nhy, device="cuda")[None, :] < lens_t[:, None])[:, None, None, :]
    gw0, gb0 = torch.empty((co, ci) + nf, device="cuda"), torch.empty(co, device="cuda")
    capi.grad_weight(x, go, gw0, gb0, s, d, p, u)
    gw1, gb1 = torch.full_like(gw0, float("nan")), torch.full_like(gb0, float("nan"))
    capi.grad_weight(x, go, gw1, gb1, s, d, p, u, lens=lens_t)
    assert helpers.rel_err(gw1.cpu().numpy(), gw0.cpu().numpy()) <= 2e-6
    assert helpers.rel_err(gb1.cpu().numpy(), gb0.cpu().numpy()) <= 2e-6
