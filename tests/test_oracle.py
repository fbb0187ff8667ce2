"""Pin the CPU oracle: the plain-C restatement (and, where it has been built,
the reference's own CPU kernels behind the shim) against every known-answer
case of the reference and against recorded outputs of the reference's CPU
torch extension."""
import itertools

import numpy as np
import pytest

import helpers
from oracle.oracle import Oracle

BACKENDS = ["port"] + (["reference"] if Oracle.reference_available() else [])


@pytest.fixture(scope="module", params=BACKENDS)
def oracle(request):
    return Oracle(request.param)


def _conv_ids():
    return [(op, i) for op in helpers.KAT_CONV_OPS for i in range(len(helpers.kat()[op]))]


def _col_ids():
    return [(op, i) for op in helpers.KAT_COL_OPS for i in range(len(helpers.kat()[op]))]


def test_fixture_counts():
    # 83 known-answer cases, as counted from the reference's kNumTests constants
    counts = {op: len(v) for op, v in helpers.kat().items()}
    assert counts == {"mconv1d": 13, "mcorr1d": 15, "lconv1d": 10, "lcorr1d": 8, "mconvlconv": 3,
                      "mcorrlcorr": 4, "snd2col": 7, "col2snd": 7, "lin2col": 7, "col2lin": 7,
                      "spec2col": 1, "col2spec": 1}


@pytest.mark.parametrize("op,idx", _conv_ids(), ids=lambda v: str(v))
@pytest.mark.parametrize("extra", [-1, 0, 3])
def test_conv_known_answers(oracle, op, idx, extra):
    prob = helpers.kat_conv_problem(op, idx)
    f, g = prob["f"], prob["g"]
    co, ci = f.shape[:2]
    for batch, tf, tg, th in itertools.product((1, 3), (False, True), (False, True), (False, True)):
        gb = np.ascontiguousarray(np.repeat(g, batch, axis=0))
        exp = np.repeat(helpers.pad_or_crop(prob["h"], extra), batch, axis=0)
        fa = np.ascontiguousarray(f.transpose(1, 0, 2, 3)) if tf else f
        ga = np.ascontiguousarray(gb.transpose(1, 0, 2, 3)) if tg else gb
        h = np.zeros(exp.shape if not th else (exp.shape[1], exp.shape[0]) + exp.shape[2:])
        oracle.op2d(prob["kind"], fa, ga, h, co, ci, batch, prob["s"], prob["d"], prob["p"], prob["u"], tf, tg, th)
        got = h.transpose(1, 0, 2, 3) if th else h
        np.testing.assert_allclose(got, exp, rtol=0, atol=1e-10)


@pytest.mark.parametrize("op,idx", _conv_ids(), ids=lambda v: str(v))
def test_conv_known_answers_float32_and_accumulate(oracle, op, idx):
    # float32 path, and "+=" semantics: a pre-filled output keeps its contents
    prob = helpers.kat_conv_problem(op, idx, np.float32)
    co, ci = prob["f"].shape[:2]
    h = np.full(prob["h"].shape, 2.5, dtype=np.float32)
    oracle.op2d(prob["kind"], prob["f"], prob["g"], h, co, ci, 1, prob["s"], prob["d"], prob["p"], prob["u"])
    np.testing.assert_allclose(h, prob["h"] + 2.5, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("op,idx", _col_ids(), ids=lambda v: str(v))
def test_col_known_answers(oracle, op, idx):
    prob = helpers.kat_col_problem(op, idx)
    for batch, tg, tgg in itertools.product((1, 2), (False, True), (False, True)):
        g = np.ascontiguousarray(np.repeat(prob["g"], batch, axis=0))
        gg = np.ascontiguousarray(np.repeat(prob["gg"], batch, axis=0))
        ga = np.ascontiguousarray(np.swapaxes(g, 0, 1)) if tg else g
        gga = np.ascontiguousarray(np.swapaxes(gg, 0, 1)) if tgg else gg
        if prob["direction"] == "gather":
            out = np.full(gga.shape, -12345.0)
            oracle.spec2col_raw(ga, out, prob["nf"], prob["s"], prob["d"], prob["p"], prob["u"], tg, tgg)
            np.testing.assert_allclose(out, gga, rtol=0, atol=1e-10)
        else:
            out = np.full(ga.shape, -12345.0)
            oracle.col2spec_raw(gga, out, prob["s"], prob["d"], prob["p"], prob["u"], tg, tgg)
            np.testing.assert_allclose(out, ga, rtol=0, atol=1e-10)


def test_sizes_against_closed_forms(oracle):
    # closed forms of mconv.py:73-118 over a parameter sweep
    for nf, ng, s, d, p, u in itertools.product((1, 3, 8), (1, 5, 41), (1, 2, 3), (1, 2, 5), (0, 1, 3), (1, 2)):
        assert oracle.lconv_support_size(nf, ng, s, d, p, u) == max((u * (ng - 1) + d * (nf - 1) - p) // s + 1, 0)
        assert oracle.lconv_valid_size(nf, ng, s, d, p, u) == max((u * (ng - 1) - p) // s + 1, 0)
        assert oracle.lcorr_support_size(nf, ng, s, d, p, u) == max((u * (ng - 1) + p) // s + 1, 0)
        assert oracle.lcorr_valid_size(nf, ng, s, d, p, u) == max((u * (ng - 1) - d * (nf - 1) + p) // s + 1, 0)
        assert oracle.mconv_support_size(nf, ng, s, d, p, u) == max(((nf + d - 1) * (ng + u - 1)) // (p + 1) - s + 1, 0)
        assert oracle.mconv_valid_size(nf, ng, s, d, p, u) == max((d * (ng + u - 1)) // (p + 1) - s + 1, 0)
        assert oracle.mcorr_support_size(nf, ng, s, d, p, u) == max(((ng + u - 1) * (p + 1)) // d - s + 1, 0)
        assert oracle.mcorr_valid_size(nf, ng, s, d, p, u) == max(((ng + u - 1) * (p + 1)) // (nf + d - 1) - s + 1, 0)


def _ext_names(kind):
    _, meta = helpers.ext_cases()
    return [k for k, v in meta.items() if v.get("kind") == kind]


@pytest.mark.parametrize("name", _ext_names("2d") + _ext_names("1d"))
@pytest.mark.parametrize("tag,dtype,tol", [("f32", np.float32, 2e-6), ("f64", np.float64, 1e-12)])
def test_against_reference_extension(oracle, name, tag, dtype, tol):
    """Forward and all three gradients against what the reference's CPU torch
    extension produced on the same inputs (tests/golden/make_golden.py)."""
    arrays, meta = helpers.ext_cases()
    m = meta[name]
    x, w, go = (arrays["%s.%s" % (name, k)].astype(dtype) for k in ("x", "w", "go"))
    b = arrays[name + ".b"].astype(dtype) if m["bias"] else None
    if m["kind"] == "2d":
        y = oracle.mcorrlcorr(x, w, b, m["s"], m["d"], m["p"], m["u"], m["r"])
        gx, gw, gb = oracle.mcorrlcorr_backward(x, w, go, m["s"], m["d"], m["p"], m["u"])
    else:
        y = oracle.mcorr1d(x, w, b, m["s"], m["d"], m["p"], m["u"], m["r"])
        gx, gw, gb = oracle.mcorr1d_backward(x, w, go, m["s"], m["d"], m["p"], m["u"])
    assert helpers.rel_err(y, arrays["%s.y.%s" % (name, tag)]) <= tol
    assert helpers.rel_err(gx, arrays["%s.gx.%s" % (name, tag)]) <= tol
    assert helpers.rel_err(gw, arrays["%s.gw.%s" % (name, tag)]) <= tol
    if m["bias"]:
        assert helpers.rel_err(gb, arrays["%s.gb.%s" % (name, tag)]) <= 10 * tol


def test_column_ops_against_reference_extension(oracle):
    arrays, meta = helpers.ext_cases()
    m = meta["spec2col"]
    gg = oracle.spec2col(arrays["spec2col.x"], m["kernel_size"], m["s"], m["d"], m["p"], m["u"], m["r"])
    np.testing.assert_array_equal(gg, arrays["spec2col.gg"])
    back = oracle.col2spec(arrays["spec2col.cot"], arrays["spec2col.x"].shape[2:], m["s"], m["d"], m["p"], m["u"])
    assert helpers.rel_err(back, arrays["spec2col.back"]) <= 1e-6
    m = meta["snd2col"]
    gg = oracle.snd2col(arrays["snd2col.x"], m["kernel_width"], m["s"], m["d"], m["p"], m["u"], m["r"])
    np.testing.assert_array_equal(gg, arrays["snd2col.gg"])
    back = oracle.col2snd(arrays["snd2col.cot"], arrays["snd2col.x"].shape[2], m["s"], m["d"], m["p"], m["u"])
    assert helpers.rel_err(back, arrays["snd2col.back"]) <= 1e-6


# ---- the elementwise layers in front of the first Mellin layer ------------------------------------------------


def _prologue_cases():
    import os

    data = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "prologue_cases.npz"))
    tags = sorted({k.rsplit("_", 1)[0] for k in data.files if k.endswith("_meta")})
    return data, tags


def test_prologue_restatement_against_the_reference_layers():
    """``oracle/prologue_oracle.py`` against values and autograd gradients recorded from the reference's ``layers.py``."""
    from oracle import prologue_oracle as po

    data, tags = _prologue_cases()
    assert len(tags) == 18
    for tag in tags:
        dim, use_lc, use_lift = (int(v) for v in data[tag + "_meta"])
        log_tau, log_eps = (float(v) for v in data[tag + "_params"])
        lt, le = (log_tau if use_lift else None), (log_eps if use_lc else None)
        x, gy = data[tag + "_x"], data[tag + "_grad_y"]
        tol = 2e-6 if x.dtype == np.float32 else 1e-13
        y = po.lift_compress(x, lt, le, dim)
        assert y.dtype == x.dtype
        assert helpers.rel_err(y, data[tag + "_y"]) <= tol, tag
        gx, g_tau, g_eps = po.lift_compress_backward(x, gy, lt, le, dim)
        assert helpers.rel_err(gx, data[tag + "_grad_x"]) <= tol, tag
        ref_tau, ref_eps = data[tag + "_grad_params"]
        ptol = 2e-5 if x.dtype == np.float32 else 1e-11  # the reference sums in the tensor's own precision
        if use_lift:
            assert abs(g_tau - ref_tau) <= ptol * max(1.0, abs(ref_tau)), (tag, g_tau, ref_tau)
        if use_lc:
            assert abs(g_eps - ref_eps) <= ptol * max(1.0, abs(ref_eps)), (tag, g_eps, ref_eps)


def test_prologue_restatement_rejects_a_bad_dim():
    from oracle import prologue_oracle as po

    with pytest.raises(RuntimeError, match="3 not a valid dimension for a tensor if dimension 3"):
        po.dilation_lift(np.zeros((2, 3, 4), np.float32), 1.0, 3)
    with pytest.raises(RuntimeError, match="-4 not a valid dimension"):
        po.dilation_lift(np.zeros((2, 3, 4), np.float32), 1.0, -4)
