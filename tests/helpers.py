"""Shared test helpers: golden-fixture loading and the parity metric."""
import json
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

_KAT = None
_EXT = None


def kat():
    global _KAT
    if _KAT is None:
        with open(os.path.join(GOLDEN, "kat_fixtures.json")) as fp:
            _KAT = json.load(fp)
    return _KAT


def ext_cases():
    """(arrays, meta) of tests/golden/ref_ext_cases.npz."""
    global _EXT
    if _EXT is None:
        z = np.load(os.path.join(GOLDEN, "ref_ext_cases.npz"))
        meta = json.loads(bytes(z["meta"]).decode())
        _EXT = ({k: z[k] for k in z.files if k != "meta"}, meta)
    return _EXT


# which family each known-answer header belongs to, and how its 1-D cases
# embed into the 2-D operators (the reference folds them the same way:
# c/tests/test_mcorrlcorr.cc:34-72, tests/test_mconv.py:374-437)
KAT_CONV_OPS = {
    "mcorr1d": ("corr", "x"), "lcorr1d": ("corr", "y"), "mcorrlcorr": ("corr", "xy"),
    "mconv1d": ("conv", "x"), "lconv1d": ("conv", "y"), "mconvlconv": ("conv", "xy"),
}
KAT_COL_OPS = {
    "snd2col": ("gather", "x"), "lin2col": ("gather", "y"), "spec2col": ("gather", "xy"),
    "col2snd": ("scatter", "x"), "col2lin": ("scatter", "y"), "col2spec": ("scatter", "xy"),
}


def _as_2d_params(case, axis):
    if axis == "xy":
        return tuple(tuple(case[k]) for k in ("nf", "ng", "s", "d", "p", "u"))
    # neutral parameters of the missing axis: size 1, s=d=u=1, p=0
    neutral = {"nf": 1, "ng": 1, "s": 1, "d": 1, "p": 0, "u": 1}
    out = []
    for k in ("nf", "ng", "s", "d", "p", "u"):
        out.append((case[k], neutral[k]) if axis == "x" else (neutral[k], case[k]))
    return tuple(out)


def support_sizes(kind, nf, ng, s, d, p, u):
    """Support size per axis, the extent the expected arrays are stored with
    (c/tests/test_mcorr1d.cc:29, test_mconv1d.cc:29, test_mcorrlcorr.cc:74-75)."""
    def fl(a, b):
        return a // b  # Python floors

    if kind == "corr":
        nx = max(fl((ng[0] + u[0] - 1) * (p[0] + 1), d[0]) - s[0] + 1, 0)
        ny = max(fl(u[1] * (ng[1] - 1) + p[1], s[1]) + 1, 0)
    else:
        nx = max(fl((nf[0] + d[0] - 1) * (ng[0] + u[0] - 1), p[0] + 1) - s[0] + 1, 0)
        ny = max(fl(u[1] * (ng[1] - 1) + d[1] * (nf[1] - 1) - p[1], s[1]) + 1, 0)
    return nx, ny


def kat_conv_problem(op, idx, dtype=np.float64):
    """Known-answer case as 4-D arrays: returns dict(kind, f, g, h, s, d, p, u)
    with f (c_out,c_in,nfx,nfy), g (1,c_in,ngx,ngy), h (1,c_out,nhx,nhy) where
    (nhx, nhy) are the support sizes."""
    kind, axis = KAT_CONV_OPS[op]
    case = kat()[op][idx]
    nf, ng, s, d, p, u = _as_2d_params(case, axis)
    ci, co = case["c_in"], case["c_out"]
    nh = support_sizes(kind, nf, ng, s, d, p, u)
    f = np.array(case["F"][: co * ci * nf[0] * nf[1]], dtype=dtype).reshape((co, ci) + nf)
    g = np.array(case["G"][: ci * ng[0] * ng[1]], dtype=dtype).reshape((1, ci) + ng)
    flat_h = case["H"]
    need = co * nh[0] * nh[1]
    assert len(flat_h) >= need, (op, idx, len(flat_h), need)
    h = np.array(flat_h[:need], dtype=dtype).reshape((1, co) + nh)
    return dict(kind=kind, f=f, g=g, h=h, s=s, d=d, p=p, u=u)


def kat_col_problem(op, idx, dtype=np.float64):
    """Known-answer column case: dict(direction, g (1,c_in,ngx,ngy),
    gg (1,c_in,nfx,nfy,nggx,nggy), nf, s, d, p, u); column extents are the
    correlation support sizes (c/tests/test_col2snd.cc:31)."""
    direction, axis = KAT_COL_OPS[op]
    case = kat()[op][idx]
    nf, ng, s, d, p, u = _as_2d_params(case, axis)
    ci = case["c_in"]
    ngg = support_sizes("corr", nf, ng, s, d, p, u)
    g = np.array(case["G"][: ci * ng[0] * ng[1]], dtype=dtype).reshape((1, ci) + ng)
    need = ci * nf[0] * nf[1] * ngg[0] * ngg[1]
    assert len(case["H"]) >= need, (op, idx, len(case["H"]), need)
    gg = np.array(case["H"][:need], dtype=dtype).reshape((1, ci) + nf + ngg)
    return dict(direction=direction, g=g, gg=gg, nf=nf, s=s, d=d, p=p, u=u)


def pad_or_crop(h, extra):
    """Expected array when the output is allocated `extra` samples longer
    (zeros) or shorter (cropped) than the support size on every non-singleton
    trailing axis (c/tests/test_utils_cpu.h:29-90)."""
    out = h
    for ax in (2, 3):
        if ax >= out.ndim:
            continue
        n = out.shape[ax]
        if extra < 0:
            out = np.take(out, range(max(n + extra, 0)), axis=ax)
        elif extra > 0:
            pad = [(0, 0)] * out.ndim
            pad[ax] = (0, extra)
            out = np.pad(out, pad)
    return np.ascontiguousarray(out)


def rel_err(a, b):
    """max|a-b| / max|b|: the per-tensor parity metric (tolerance 1e-5 in FP32)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    assert a.shape == b.shape, (a.shape, b.shape)
    denom = np.abs(b).max() if b.size else 0.0
    if denom == 0.0:
        return float(np.abs(a).max()) if a.size else 0.0
    return float(np.abs(a - b).max() / denom)
