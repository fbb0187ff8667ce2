"""Regenerate the golden fixtures under tests/golden/ from a checkout of the
reference (sdrobert/cnn-mellin).

Run where the reference is checked out; ``MELLIN_REFERENCE`` names the
checkout when it is not at the default location coded below::

    python tests/golden/make_golden.py

It writes three files next to itself, all committed (``--stack-only`` rewrites
only the last):

``kat_fixtures.json``
    Every known-answer case of the reference's ``c/tests/test_*_buffers.h``
    (83 cases over 12 operators), read as text from those headers: operand
    values (exact rationals evaluated in double), sizes and the
    ``s, d, p, u`` parameters, plus the expected result.  These are the same
    cases the reference's ``c/tests/*.cc`` and ``tests/test_mconv.py:604-647``
    consume.

``ref_ext_cases.npz``
    Inputs, outputs and gradients of the reference's *own CPU torch
    extension* (``torch.ops.mellin.*``, built unmodified from the reference's
    ``ext/``) on seeded random inputs, in float32 and float64: the first
    BASELINE configuration in full (1-D Mellin correlation, batch 8, 4->8
    channels, length 256, kernel 16) and reduced-size versions of the 2-D
    layer configurations, with strides / dilations / paddings / ``u`` that
    the reference's gradcheck tests sweep.

Neither the tests nor the benchmark ever read the reference checkout; they
read only these two files.

``ref_stack3.npz``
    Three stacked same-size layers (3 -> 8 -> 12 -> 16 channels, kernel 6x3,
    Mellin dilation 1, 2, 2) with ReLU and per-utterance length masks before
    every layer, forward and every gradient through the reference's extension
    in float32 and float64: the reference's three-layer benchmark stack at
    reduced width.
"""
import json
import os
import re
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE = os.environ.get("MELLIN_REFERENCE", "/root/reference")

HEADERS = [
    "mconv1d", "mcorr1d", "lconv1d", "lcorr1d", "mconvlconv", "mcorrlcorr",
    "snd2col", "col2snd", "lin2col", "col2lin", "spec2col", "col2spec",
]


def parse_header(path):
    """Return {array_name: nested list} for every ``const T kName[...] = {...};``."""
    text = open(path).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    out = {}
    for m in re.finditer(r"const\s+(?:double|int)\s+(k\w+)\s*((?:\[[^\]]*\])+)\s*=\s*(\{.*?\})\s*;", text, flags=re.S):
        name, body = m.group(1), m.group(3)
        body = body.replace("{", "[").replace("}", "]")
        body = re.sub(r"(\d)\.(?!\d)", r"\1.0", body)  # "5." -> "5.0"
        assert re.fullmatch(r"[\d\s\.\,\[\]\-\+/eE]*", body), (path, name)
        out[name] = eval(body, {"__builtins__": {}})  # numeric literals, '/', ',' and brackets only
    return out


def kat_fixtures():
    cases = {}
    for op in HEADERS:
        arrays = parse_header(os.path.join(REFERENCE, "c", "tests", "test_%s_buffers.h" % op))
        n = len(arrays["kG"])
        two_d = "kNFX" in arrays
        op_cases = []
        for i in range(n):
            c = {"c_in": int(arrays["kCIn"][i])}
            if "kCOut" in arrays:
                c["c_out"] = int(arrays["kCOut"][i])
            if two_d:
                for key, name in (("nf", "kNF"), ("ng", "kNG"), ("s", "kS"), ("d", "kD"), ("p", "kP"), ("u", "kU")):
                    c[key] = [int(arrays[name + "X"][i]), int(arrays[name + "Y"][i])]
            else:
                for key, name in (("nf", "kNF"), ("ng", "kNG"), ("s", "kS"), ("d", "kD"), ("p", "kP"), ("u", "kU")):
                    c[key] = int(arrays[name][i])
            if "kF" in arrays:
                c["F"] = [float(v) for v in arrays["kF"][i]]
            c["G"] = [float(v) for v in arrays["kG"][i]]
            c["H"] = [float(v) for v in arrays["kH"][i]]
            op_cases.append(c)
        cases[op] = op_cases
    return cases


# ---------------------------------------------------------------------------
# outputs of the reference's own CPU extension

EXT_CASES_2D = [
    # name, batch, c_in, c_out, (ngx, ngy), (nfx, nfy), s, d, p, u, r, bias
    ("layer2d_same", 2, 3, 8, (41, 48), (8, 3), (1, 1), (1, 1), (0, 1), (1, 1), ("same", 1), True),
    ("layer2d_valid", 2, 3, 8, (41, 48), (8, 3), (1, 1), (1, 1), (0, 1), (1, 1), (0, 1), False),
    ("layer2d_dil2", 2, 5, 6, (41, 40), (6, 3), (1, 1), (2, 1), (0, 1), (1, 1), ("same", 1), True),
    ("layer2d_wide", 1, 16, 24, (20, 36), (6, 3), (1, 1), (1, 1), (0, 1), (1, 1), ("same", 1), True),
    ("layer2d_s2d2", 2, 2, 3, (12, 17), (3, 4), (2, 2), (2, 2), (3, 4), (1, 1), (4, 3), True),
    ("layer2d_mixed", 3, 2, 2, (9, 13), (4, 2), (1, 2), (2, 1), (3, 3), (2, 2), (2, 1), False),
    ("layer2d_u2", 2, 3, 2, (8, 8), (3, 3), (2, 1), (1, 2), (4, 3), (2, 2), (3, 4), True),
    ("linear_only", 2, 4, 5, (1, 64), (1, 7), (1, 2), (1, 2), (0, 3), (1, 1), (0, 2), True),
]

EXT_CASES_1D = [
    # name, batch, c_in, c_out, ng, nf, s, d, p, u, r, bias
    ("config1_valid", 8, 4, 8, 256, 16, 1, 1, 0, 1, 0, False),
    ("config1_same", 8, 4, 8, 256, 16, 1, 1, 0, 1, 240, False),
    ("mellin1d_s2d2p1", 3, 5, 4, 100, 12, 2, 2, 1, 1, 30, True),
    ("mellin1d_u2p3", 2, 3, 3, 40, 5, 1, 2, 3, 2, 20, True),
]


def ext_cases():
    os.environ.setdefault("TORCH_EXTENSIONS_DIR", os.path.join(HERE, "..", "..", "_work", "torch_ext"))
    sys.path.insert(0, REFERENCE)
    if not hasattr(np, "product"):
        np.product = np.prod  # the reference predates numpy 2
    import torch
    import mconv  # the reference's module; JIT-builds its CPU extension

    assert mconv._ext_mcorrlcorr is not None, "reference extension failed to build"
    out = {}
    meta = {}

    def run(name, op, x, w, b, args, grad_seed):
        for dt, tag in ((torch.float32, "f32"), (torch.float64, "f64")):
            xt = torch.from_numpy(x).to(dt).requires_grad_(True)
            wt = torch.from_numpy(w).to(dt).requires_grad_(True)
            bt = None if b is None else torch.from_numpy(b).to(dt).requires_grad_(True)
            y = op(xt, wt, bt, *args)
            go = np.random.default_rng(grad_seed).standard_normal(tuple(y.shape)).astype(np.float32)
            grads = torch.autograd.grad(y, [xt, wt] + ([] if bt is None else [bt]), torch.from_numpy(go).to(dt))
            if tag == "f32":
                out[name + ".x"], out[name + ".w"], out[name + ".go"] = x, w, go
                if b is not None:
                    out[name + ".b"] = b
            out["%s.y.%s" % (name, tag)] = y.detach().numpy()
            out["%s.gx.%s" % (name, tag)] = grads[0].numpy()
            out["%s.gw.%s" % (name, tag)] = grads[1].numpy()
            if bt is not None:
                out["%s.gb.%s" % (name, tag)] = grads[2].numpy()

    for i, (name, n, ci, co, ng, nf, s, d, p, u, r, bias) in enumerate(EXT_CASES_2D):
        rng = np.random.default_rng(1000 + i)
        x = rng.standard_normal((n, ci) + ng).astype(np.float32)
        w = (rng.standard_normal((co, ci) + nf) * (2.0 / (ci * nf[0] * nf[1])) ** 0.5).astype(np.float32)
        b = rng.standard_normal(co).astype(np.float32) if bias else None
        if r[0] == "same":
            r = (ng[0] - mconv.mcorr_valid_size(nf[0], ng[0], s[0], d[0], p[0], u[0]), r[1])
        meta[name] = dict(kind="2d", s=s, d=d, p=p, u=u, r=r, bias=bias)
        run(name, mconv._ext_mcorrlcorr, x, w, b, (s, d, p, u, r), 2000 + i)

    for i, (name, n, ci, co, ng, nf, s, d, p, u, r, bias) in enumerate(EXT_CASES_1D):
        rng = np.random.default_rng(3000 + i)
        x = rng.standard_normal((n, ci, ng)).astype(np.float32)
        w = (rng.standard_normal((co, ci, nf)) / (ci * nf) ** 0.5).astype(np.float32)
        b = rng.standard_normal(co).astype(np.float32) if bias else None
        meta[name] = dict(kind="1d", s=s, d=d, p=p, u=u, r=r, bias=bias)
        run(name, mconv._ext_mcorr1d, x, w, b, (s, d, p, u, r), 4000 + i)

    # column operators (forward and adjoint), float32 only: pure data movement
    rng = np.random.default_rng(5000)
    x = rng.standard_normal((2, 3, 9, 11)).astype(np.float32)
    args = ((3, 2), (1, 2), (2, 1), (1, 3), (1, 1), (2, 1))
    gg = mconv._ext_spec2col(torch.from_numpy(x), *args)
    cot = rng.standard_normal(tuple(gg.shape)).astype(np.float32)
    back = torch.ops.mellin.col2spec(torch.from_numpy(cot), [9, 11], *args[1:5])
    out["spec2col.x"], out["spec2col.gg"], out["spec2col.cot"], out["spec2col.back"] = x, gg.numpy(), cot, back.numpy()
    meta["spec2col"] = dict(kernel_size=args[0], s=args[1], d=args[2], p=args[3], u=args[4], r=args[5])
    x = rng.standard_normal((3, 2, 30)).astype(np.float32)
    args = (4, 2, 1, 1, 1, 5)
    gg = mconv._ext_snd2col(torch.from_numpy(x), *args)
    cot = rng.standard_normal(tuple(gg.shape)).astype(np.float32)
    back = torch.ops.mellin.col2snd(torch.from_numpy(cot), 30, *args[1:5])
    out["snd2col.x"], out["snd2col.gg"], out["snd2col.cot"], out["snd2col.back"] = x, gg.numpy(), cot, back.numpy()
    meta["snd2col"] = dict(kernel_width=args[0], s=args[1], d=args[2], p=args[3], u=args[4], r=args[5])

    out["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    return out


# three stacked layers with ReLU and length masks, the shape of the reference's
# three-layer benchmark stack at reduced width: channels, kernel, Mellin dilation
STACK = dict(batch=4, bins=41, frames=48, channels=(3, 8, 12, 16), kernel=(6, 3), dilation=((1, 1), (2, 1), (2, 1)),
             lens=(48, 37, 29, 20))


def stack_forward(mcorrlcorr, valid_size, x, weights, biases, mask):
    """y = mask * relu(layer3(mask * relu(layer2(mask * relu(layer1(mask * x)))))), every layer same-size."""
    h = x
    for w, b, d in zip(weights, biases, STACK["dilation"]):
        r = (STACK["bins"] - valid_size(STACK["kernel"][0], STACK["bins"], 1, d[0], 0, 1), 1)
        h = mcorrlcorr(h * mask, w, b, (1, 1), d, (0, 1), (1, 1), r).relu()
    return h * mask


def stack_case():
    sys.path.insert(0, REFERENCE)
    if not hasattr(np, "product"):
        np.product = np.prod
    import torch
    import mconv

    rng = np.random.default_rng(7000)
    ch, k = STACK["channels"], STACK["kernel"]
    x = rng.standard_normal((STACK["batch"], ch[0], STACK["bins"], STACK["frames"])).astype(np.float32)
    ws = [(rng.standard_normal((ch[i + 1], ch[i]) + k) * (2.0 / (ch[i] * k[0] * k[1])) ** 0.5).astype(np.float32)
          for i in range(3)]
    bs = [(0.1 * rng.standard_normal(ch[i + 1])).astype(np.float32) for i in range(3)]
    mask = (np.arange(STACK["frames"])[None, :] < np.asarray(STACK["lens"])[:, None]).astype(np.float32)
    mask = mask[:, None, None, :]
    go = rng.standard_normal((STACK["batch"], ch[3], STACK["bins"], STACK["frames"])).astype(np.float32)
    out = {"x": x, "go": go, "mask": mask}
    for i in range(3):
        out["w%d" % i], out["b%d" % i] = ws[i], bs[i]
    for dt, tag in ((torch.float32, "f32"), (torch.float64, "f64")):
        leaves = [torch.from_numpy(a).to(dt).requires_grad_(True) for a in [x] + ws + bs]
        y = stack_forward(mconv._ext_mcorrlcorr, mconv.mcorr_valid_size, leaves[0], leaves[1:4], leaves[4:7],
                          torch.from_numpy(mask).to(dt))
        grads = torch.autograd.grad(y, leaves, torch.from_numpy(go).to(dt))
        out["y." + tag] = y.detach().numpy()
        for name, g in zip(["gx", "gw0", "gw1", "gw2", "gb0", "gb1", "gb2"], grads):
            out["%s.%s" % (name, tag)] = g.numpy()
    return out


def main():
    if "--stack-only" not in sys.argv:
        with open(os.path.join(HERE, "kat_fixtures.json"), "w") as fp:
            json.dump(kat_fixtures(), fp, indent=0, separators=(",", ":"))
        np.savez_compressed(os.path.join(HERE, "ref_ext_cases.npz"), **ext_cases())
    os.environ.setdefault("TORCH_EXTENSIONS_DIR", os.path.join(HERE, "..", "..", "_work", "torch_ext"))
    np.savez_compressed(os.path.join(HERE, "ref_stack3.npz"), **stack_case())


if __name__ == "__main__":
    main()
