"""Acceptance tests of the PyTorch surface (``mconv.py`` + ``torch.ops.mellin``)
on a B200.  They follow the reference's ``tests/test_mconv.py``: known-answer
values with and without bias and with the ``r`` argument (:575-647), float64
``gradcheck`` over the (s, d, p, u) sweep (:663-773), direct-vs-mm equivalence
(:632-660), training smoke tests (:776-811) and repeatability (:894-919)."""
import numpy as np
import pytest
import torch

import helpers

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mconv():
    import mconv as module  # cnn-mellin_b200/mconv.py (conftest puts it on sys.path)

    return module


def _conv_ids(kind):
    return [(op, i) for op, (k, _) in helpers.KAT_CONV_OPS.items() if k == kind for i in range(len(helpers.kat()[op]))]


def _with_r(op, g, f_or_size, lead_args, h_exp):
    """Call once with r = 0 to learn the valid size, then with the r that yields
    the expected (support-sized) output, as the reference's _test_values does."""
    nd = h_exp.dim() - 2 if h_exp.dim() <= 4 else 2
    h0 = op(g, f_or_size, *lead_args)
    r = [h_exp.size(h_exp.dim() - nd + i) - h0.size(h0.dim() - nd + i) for i in range(nd)]
    return op(g, f_or_size, *lead_args, r if nd == 2 else r[0])


@pytest.mark.parametrize("op,idx", _conv_ids("corr"), ids=lambda v: str(v))
@pytest.mark.parametrize("bias", [True, False])
def test_mcorrlcorr_values(mconv, op, idx, bias):
    prob = helpers.kat_conv_problem(op, idx, np.float32)
    f, g, h = (torch.from_numpy(prob[k]).cuda() for k in ("f", "g", "h"))
    b = torch.rand(f.size(0), device="cuda") if bias else None
    if bias:
        h = h + b.view(1, -1, 1, 1)
    got = _with_r(mconv._ext_mcorrlcorr, g, f, (b, prob["s"], prob["d"], prob["p"], prob["u"]), h)
    assert got.shape == h.shape
    assert torch.allclose(h, got)


@pytest.mark.parametrize("idx", range(len(helpers.kat()["mcorr1d"])))
@pytest.mark.parametrize("bias", [True, False])
def test_mcorr1d_values(mconv, idx, bias):
    prob = helpers.kat_conv_problem("mcorr1d", idx, np.float32)
    f, g, h = (torch.from_numpy(prob[k][..., 0]).cuda() for k in ("f", "g", "h"))
    b = torch.rand(f.size(0), device="cuda") if bias else None
    if bias:
        h = h + b.view(1, -1, 1)
    got = _with_r(mconv._ext_mcorr1d, g, f, (b, prob["s"][0], prob["d"][0], prob["p"][0], prob["u"][0]), h)
    assert got.shape == h.shape
    assert torch.allclose(h, got)


@pytest.mark.parametrize("op,idx", _conv_ids("conv"), ids=lambda v: str(v))
def test_mconvlconv_values(mconv, op, idx):
    prob = helpers.kat_conv_problem(op, idx, np.float32)
    f, g, h = (torch.from_numpy(prob[k]).cuda() for k in ("f", "g", "h"))
    got = _with_r(torch.ops.mellin.mconvlconv, g, f, (None, prob["s"], prob["d"], prob["p"], prob["u"]), h)
    assert got.shape == h.shape
    assert torch.allclose(h, got)


def _col_ids(direction):
    return [(op, i) for op, (k, _) in helpers.KAT_COL_OPS.items() if k == direction
            for i in range(len(helpers.kat()[op]))]


@pytest.mark.parametrize("op,idx", _col_ids("gather"), ids=lambda v: str(v))
def test_spec2col_values(mconv, op, idx):
    prob = helpers.kat_col_problem(op, idx, np.float32)
    g, gg = torch.from_numpy(prob["g"]).cuda(), torch.from_numpy(prob["gg"]).cuda()
    got = _with_r(mconv._ext_spec2col, g, list(prob["nf"]), (prob["s"], prob["d"], prob["p"], prob["u"]), gg)
    assert got.shape == gg.shape
    assert torch.allclose(gg, got)


@pytest.mark.parametrize("op,idx", _col_ids("scatter"), ids=lambda v: str(v))
def test_col2spec_values(mconv, op, idx):
    prob = helpers.kat_col_problem(op, idx, np.float32)
    g, gg = torch.from_numpy(prob["g"]).cuda(), torch.from_numpy(prob["gg"]).cuda()
    got = torch.ops.mellin.col2spec(gg, list(g.shape[2:]), prob["s"], prob["d"], prob["p"], prob["u"])
    assert torch.allclose(g, got)


def test_mcorr1d_impl(mconv):
    torch.manual_seed(10)
    batch, c_out, c_in, nf, ng, s, d, p, r = 128, 8, 16, 4, 12, 1, 2, 3, 4
    f = torch.rand((c_out, c_in, nf), device="cuda")
    g = torch.rand((batch, c_in, ng), device="cuda")
    b = torch.rand((c_out,), device="cuda")
    h_exp = mconv.mcorr1d(g, f, b, s, d, p, r, _impl="direct")
    h_act = mconv.mcorr1d(g, f, b, s, d, p, r, _impl="mm")
    assert h_exp.size() == h_act.size()
    assert torch.allclose(h_exp, h_act, atol=1e-5)


def test_mcorrlcorr_impl(mconv):
    torch.manual_seed(20)
    batch, c_out, c_in, nf, ng = 64, 16, 8, (32, 32), (8, 8)
    s, d, p, r = (1, 2), (2, 1), (3, 3), (1, 1)
    f = torch.rand((c_out, c_in) + nf, device="cuda")
    g = torch.rand((batch, c_in) + ng, device="cuda")
    b = torch.rand((c_out,), device="cuda")
    h_exp = mconv.mcorrlcorr(g, f, b, s, d, p, r, _impl="direct")
    h_act = mconv.mcorrlcorr(g, f, b, s, d, p, r, _impl="mm")
    assert h_exp.size() == h_act.size()
    assert torch.allclose(h_exp, h_act, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("s", [1, 2])
@pytest.mark.parametrize("d", [1, 2])
@pytest.mark.parametrize("p", [3, 4])
@pytest.mark.parametrize("u", [1, 2])
@pytest.mark.parametrize("bias", [True, False])
def test_mcorr1d_gradcheck(mconv, s, d, p, u, bias):
    c_out, c_in, batch, nf, ng, r = 3, 2, 2, 4, 6, p
    f = torch.rand((c_out, c_in, nf), dtype=torch.double, device="cuda", requires_grad=True)
    g = torch.rand((batch, c_in, ng), dtype=torch.double, device="cuda", requires_grad=True)
    b = torch.rand((c_out,), dtype=torch.double, device="cuda", requires_grad=True) if bias else None
    assert torch.autograd.gradcheck(mconv._ext_mcorr1d, (g, f, b, s, d, p, u, r))


@pytest.mark.parametrize("s", [1, 2])
@pytest.mark.parametrize("d", [(1, 1), (2, 2), (2, 1)])
@pytest.mark.parametrize("p", [3, 4])
@pytest.mark.parametrize("u", [1, 2])
@pytest.mark.parametrize("extra_layers", [True, False])
def test_mcorrlcorr_gradcheck(mconv, s, d, p, u, extra_layers):
    c_out, c_in, batch, nf, ng = 2, 3, 2, (3, 2), (4, 5)
    f = torch.rand((c_out, c_in) + nf, dtype=torch.double, device="cuda", requires_grad=True)
    g = torch.rand((batch, c_in) + ng, dtype=torch.double, device="cuda", requires_grad=True)
    b = torch.rand((c_out,), dtype=torch.double, device="cuda", requires_grad=True)
    args = ((s, s), d, (p, p), (u, u), (p, p))
    if extra_layers:
        m1 = torch.rand((ng[1], ng[1]), dtype=torch.double, device="cuda")

        def func(g_, f_, b_):
            y = mconv._ext_mcorrlcorr(torch.matmul(g_, m1), f_, b_, *args)
            return torch.tanh(y).sum(1)

        assert torch.autograd.gradcheck(func, (g, f, b))
    else:
        assert torch.autograd.gradcheck(mconv._ext_mcorrlcorr, (g, f, b) + args)


@pytest.mark.parametrize("s,d,p,u", [(1, 1, 3, 1), (2, 2, 4, 2), (1, 2, 3, 2)])
def test_col_gradcheck(mconv, s, d, p, u):
    g = torch.rand((2, 3, 6), dtype=torch.double, device="cuda", requires_grad=True)
    assert torch.autograd.gradcheck(mconv._ext_snd2col, (g, 4, s, d, p, u, p))
    g2 = torch.rand((2, 2, 4, 5), dtype=torch.double, device="cuda", requires_grad=True)
    assert torch.autograd.gradcheck(mconv._ext_spec2col, (g2, (3, 2), (s, s), (d, d), (p, p), (u, u), (p, p)))


def test_can_train_layers(mconv):
    torch.manual_seed(1)
    layer = mconv.MCorr1d(4, 5, 12, r=10).cuda()
    x = torch.rand(3, 4, 40, device="cuda")
    layer(x).sum().backward()
    assert layer.weight.grad.abs().sum() > 0 and layer.bias.grad.abs().sum() > 0
    layer2 = mconv.MCorrLCorr(3, 6, (6, 3), p=(0, 1), r=(35, 1)).cuda()
    x2 = torch.rand(2, 3, 41, 50, device="cuda", requires_grad=True)
    y2 = layer2(x2)
    assert y2.shape == (2, 6, 41, 50)
    y2.sum().backward()
    assert layer2.weight.grad.abs().sum() > 0 and layer2.bias.grad.abs().sum() > 0 and x2.grad.abs().sum() > 0
    assert set(dict(layer2.named_parameters())) == {"weight", "bias"}


def test_frozen_inputs_skip_gradients(mconv):
    w = torch.rand(4, 3, 3, 3, device="cuda", requires_grad=True)
    x = torch.rand(2, 3, 9, 20, device="cuda")  # no grad wanted for the input
    y = mconv.mcorrlcorr(x, w, None, 1, 1, (0, 1), (3, 1), _impl="direct")
    y.sum().backward()
    assert w.grad is not None and x.grad is None


@pytest.mark.parametrize("repeats", [1, 2, 10])
def test_results_are_repeatable(mconv, repeats):
    torch.manual_seed(3)
    layer = mconv.MCorrLCorr(3, 16, (5, 3), p=(0, 1), r=(10, 1)).cuda()
    x = torch.rand(4, 3, 20, 64, device="cuda", requires_grad=True)
    first = None
    for _ in range(repeats):
        layer.zero_grad()
        x.grad = None
        y = layer(x)
        y.square().sum().backward()
        now = (y.detach().clone(), x.grad.clone(), layer.weight.grad.clone(), layer.bias.grad.clone())
        if first is None:
            first = now
        else:
            for a, b in zip(first, now):
                assert torch.equal(a, b)


def test_transposed_operands_need_no_copy(mconv):
    # dim-0/1 transposes of dense tensors go through the transposition flags
    torch.manual_seed(5)
    x = torch.rand(3, 2, 10, 12, device="cuda")
    w = torch.rand(4, 3, 3, 2, device="cuda")
    ref = torch.ops.mellin.mcorrlcorr(x.transpose(0, 1).contiguous(), w, None, [1, 1], [1, 1], [0, 1], [1, 1], [2, 1])
    got = torch.ops.mellin.mcorrlcorr(x.transpose(0, 1), w, None, [1, 1], [1, 1], [0, 1], [1, 1], [2, 1])
    assert torch.equal(ref, got)
    wt = w.transpose(0, 1)  # (3, 4, ...) viewed as (c_out=3, c_in=4)
    x4 = torch.rand(2, 4, 10, 12, device="cuda")
    ref = torch.ops.mellin.mconvlconv(x4, wt.contiguous(), None, [1, 1], [1, 1], [0, 1], [1, 1], [2, 1])
    got = torch.ops.mellin.mconvlconv(x4, wt, None, [1, 1], [1, 1], [0, 1], [1, 1], [2, 1])
    assert torch.equal(ref, got)


def test_argument_errors(mconv):
    with pytest.raises(RuntimeError, match="Expected 3-dimensional"):
        mconv._ext_mcorr1d(torch.zeros(1, 1, 2, 2, device="cuda"), torch.zeros(1, 1, 2, device="cuda"))
    with pytest.raises(RuntimeError, match="Expected tensor to have size 3 at dimension 1"):
        mconv._ext_mcorr1d(torch.zeros(1, 2, 5, device="cuda"), torch.zeros(1, 3, 2, device="cuda"))
    with pytest.raises(RuntimeError, match="integer or a tuple of 2"):
        mconv.mcorrlcorr(torch.zeros(1, 1, 2, 2, device="cuda"), torch.zeros(1, 1, 2, 2, device="cuda"), s=(1, 2, 3))
    with pytest.raises(NotImplementedError):
        mconv.mcorr1d(torch.zeros(1, 1, 20), torch.zeros(1, 1, 12))  # CPU tensors: no such backend here


# ---- float16 / autocast (reference: tests/test_mconv.py:814-891) -------------------
def test_autocast_mcorrlcorr_func(mconv):
    """Under autocast the operator returns float16 and agrees with the float32
    result to float16 precision; inputs are exactly representable in float16."""
    n, c_in, c_out, t_in, f_in, t_kern, f_kern = 16, 24, 40, 48, 32, 6, 3
    x = torch.rand(n, c_in, t_in, f_in, device="cuda", dtype=torch.half).float()
    w = torch.rand(c_out, c_in, t_kern, f_kern, device="cuda", dtype=torch.half).float()
    b = torch.rand(c_out, device="cuda", dtype=torch.half).float()
    expected = mconv.mcorrlcorr(x, w, b).half()
    with torch.autocast("cuda"):
        got = mconv.mcorrlcorr(x, w, b)
    assert got.dtype == torch.half
    assert torch.allclose(expected, got, rtol=1e-2, atol=1e-2)
    # float32 accumulation: the float16 result is the rounded float32 one
    assert torch.equal(expected, got)


def test_autocast_mcorr1d_func(mconv):
    n, c_in, c_out, t_in, t_kern = 32, 16, 32, 128, 16
    x = torch.rand(n, c_in, t_in, device="cuda", dtype=torch.half).float()
    w = torch.rand(c_out, c_in, t_kern, device="cuda", dtype=torch.half).float()
    b = torch.rand(c_out, device="cuda", dtype=torch.half).float()
    expected = mconv.mcorr1d(x, w, b).half()
    with torch.autocast("cuda"):
        got = mconv.mcorr1d(x, w, b)
    assert got.dtype == torch.half
    assert torch.allclose(expected, got, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("kind", ["mcorr1d", "mcorrlcorr"])
def test_autocast_layers_train_with_a_grad_scaler(mconv, kind):
    torch.manual_seed(4)
    if kind == "mcorr1d":
        layer = mconv.MCorr1d(12, 8, 8).cuda()
        x = torch.randn(16, 12, 16, device="cuda")
    else:
        layer = mconv.MCorrLCorr(12, 8, (4, 2)).cuda()
        x = torch.randn(16, 12, 16, 8, device="cuda")
    before = layer.weight.detach().clone()
    optimizer = torch.optim.Adam(layer.parameters())
    scaler = torch.amp.GradScaler("cuda", init_scale=256.0)  # the default 65536 is not a float16 number
    optimizer.zero_grad()
    with torch.autocast("cuda"):
        out = layer(x)  # float16 from the fused operator; the narrow-kernel "mm" route adds a float32 bias
        assert out.dtype in (torch.half, torch.float32)
        loss = out.sum()
    scaler.scale(loss).backward()
    assert layer.weight.grad.dtype == torch.float32 and torch.isfinite(layer.weight.grad).all()
    scaler.step(optimizer)
    scaler.update()
    assert not torch.equal(before, layer.weight.detach())


def test_half_tensors_and_column_operators(mconv):
    x = torch.randn(3, 4, 20, 6, device="cuda").half()
    cols = mconv.spec2col(x, (3, 2))
    assert cols.dtype == torch.half
    assert torch.equal(cols, mconv.spec2col(x.float(), (3, 2)).half())
    w = torch.randn(5, 4, 3, 2, device="cuda").half()
    y = mconv.mcorrlcorr(x, w, _impl="direct")  # the fused operator: float32 arithmetic on widened operands
    assert y.dtype == torch.half
    assert torch.equal(y, mconv.mcorrlcorr(x.float(), w.float(), _impl="direct").half())


def test_half_operators_match_the_oracle_on_the_rounded_inputs(mconv):
    """The reference computes float16 tensors with a float32 accumulator (mconv_cuda.cuh:135-139) and rounds the
    result.  Oracle: its float32 CPU kernels on the float16-rounded operands; tolerance one float16 unit
    (2^-10 relative to the tensor's largest value) for outputs and gradients."""
    import numpy as np

    import helpers
    from oracle.oracle import Oracle

    oracle = Oracle("reference") if Oracle.reference_available() else Oracle("port")
    half_ulp = 2.0 ** -10
    torch.manual_seed(11)
    for n, ci, co, ng, nf, d in ((3, 3, 16, (12, 40), (4, 3), (1, 1)), (2, 24, 40, (12, 64), (4, 3), (2, 1))):
        s, p = (1, 1), (0, 1)
        r = (ng[0] - mconv.mcorr_valid_size(nf[0], ng[0], 1, d[0]), 1)
        x = torch.randn((n, ci) + ng, device="cuda").half().requires_grad_(True)
        w = (torch.randn((co, ci) + nf, device="cuda") / (ci * nf[0] * nf[1]) ** 0.5).half().requires_grad_(True)
        b = torch.randn(co, device="cuda").half().requires_grad_(True)
        y = mconv.mcorrlcorr(x, w, b, s, d, p, r, _impl="direct")
        assert y.dtype == torch.half
        go = torch.randn_like(y)
        y.backward(go)
        x_h, w_h, b_h, go_h = (t.detach().float().cpu().numpy() for t in (x, w, b, go))
        y_exp = oracle.mcorrlcorr(x_h, w_h, b_h, s, d, p, (1, 1), r)
        gx_exp, gw_exp, gb_exp = oracle.mcorrlcorr_backward(x_h, w_h, go_h, s, d, p, (1, 1))
        assert helpers.rel_err(y.detach().float().cpu().numpy(), y_exp) <= half_ulp
        assert x.grad.dtype == torch.half and w.grad.dtype == torch.half
        assert helpers.rel_err(x.grad.float().cpu().numpy(), gx_exp) <= half_ulp
        assert helpers.rel_err(w.grad.float().cpu().numpy(), gw_exp) <= half_ulp
        assert helpers.rel_err(b.grad.float().cpu().numpy(), gb_exp) <= half_ulp
    # autocast: float32 parameters and inputs, float16 arithmetic inputs and result
    x = torch.randn(4, 24, 12, 64, device="cuda")
    w = torch.randn(40, 24, 4, 3, device="cuda") / 17.0
    b = torch.randn(40, device="cuda")
    with torch.autocast("cuda"):
        got = mconv.mcorrlcorr(x, w, b, _impl="direct")
    assert got.dtype == torch.half
    exp = oracle.mcorrlcorr(x.half().float().cpu().numpy(), w.half().float().cpu().numpy(),
                            b.half().float().cpu().numpy(), 1, 1, 0, 1, 0)
    assert helpers.rel_err(got.float().cpu().numpy(), exp) <= half_ulp


# ---- three stacked layers with ReLU and length masks against the reference extension ----
def test_three_layer_stack_matches_the_reference_extension(mconv):
    """The reference's three-layer stack at reduced width (tests/golden/make_golden.py,
    ``stack_case``): output and every gradient within the float32 tolerance of the
    reference extension's float64 run, or no further from it than its float32 run."""
    import os

    data = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_stack3.npz"))
    dilation = ((1, 1), (2, 1), (2, 1))
    leaves = [torch.from_numpy(data[k]).cuda().requires_grad_(True) for k in ("x", "w0", "w1", "w2", "b0", "b1", "b2")]
    mask = torch.from_numpy(data["mask"]).cuda()
    h = leaves[0]
    for w, b, d in zip(leaves[1:4], leaves[4:7], dilation):
        r = (41 - mconv.mcorr_valid_size(6, 41, 1, d[0], 0, 1), 1)
        h = mconv.mcorrlcorr(h * mask, w, b, (1, 1), d, (0, 1), r, _impl="direct").relu()
    y = h * mask
    grads = torch.autograd.grad(y, leaves, torch.from_numpy(data["go"]).cuda())
    got = dict(zip(["gx", "gw0", "gw1", "gw2", "gb0", "gb1", "gb2"], grads), y=y.detach())
    for name, value in got.items():
        exact, ref32 = data[name + ".f64"], data[name + ".f32"]
        mine = helpers.rel_err(value.cpu().numpy(), exact)
        assert mine <= max(1e-5, helpers.rel_err(ref32, exact)), (name, mine)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_fused_masked_layers_reproduce_the_reference_stack(mconv, dtype):
    """The same three-layer stack through ``mcorrlcorr_masked`` (mask and ReLU
    fused into each layer's kernel): output and gradients against the reference
    extension's run of the unfused operators."""
    import os

    data = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_stack3.npz"))
    dilation = ((1, 1), (2, 1), (2, 1))
    names = ("x", "w0", "w1", "w2", "b0", "b1", "b2")
    leaves = [torch.from_numpy(data[k]).cuda().to(dtype).requires_grad_(True) for k in names]
    mask = torch.from_numpy(data["mask"]).cuda().to(dtype)
    lens = mask[:, 0, 0, :].sum(dim=1).to(torch.int32)
    h = leaves[0] * mask
    for w, b, d in zip(leaves[1:4], leaves[4:7], dilation):
        r = (41 - mconv.mcorr_valid_size(6, 41, 1, d[0], 0, 1), 1)
        h = mconv.mcorrlcorr_masked(h, w, b, lens, True, (1, 1), d, (0, 1), r)
    grads = torch.autograd.grad(h, leaves, torch.from_numpy(data["go"]).cuda().to(dtype))
    got = dict(zip(["gx", "gw0", "gw1", "gw2", "gb0", "gb1", "gb2"], grads), y=h.detach())
    for name, value in got.items():
        exact, ref32 = data[name + ".f64"], data[name + ".f32"]
        mine = helpers.rel_err(value.double().cpu().numpy(), exact)
        bound = 1e-12 if dtype == torch.float64 else max(1e-5, helpers.rel_err(ref32, exact))
        assert mine <= bound, (name, mine)


def test_fused_masked_layer_without_relu_and_half(mconv):
    x = torch.randn(3, 4, 9, 30, device="cuda", requires_grad=True)
    w = torch.randn(5, 4, 3, 2, device="cuda", requires_grad=True)
    b = torch.randn(5, device="cuda", requires_grad=True)
    lens = torch.tensor([30, 11, 0], dtype=torch.int32, device="cuda")
    y = mconv.mcorrlcorr_masked(x, w, b, lens, False)
    plain = mconv.mcorrlcorr(x, w, b, _impl="direct")
    mask = (torch.arange(plain.size(3), device="cuda")[None, :] < lens[:, None])[:, None, None, :]
    assert torch.equal(y, plain * mask)
    go = torch.randn_like(y)
    got = torch.autograd.grad(y, [x, w, b], go)
    exp = torch.autograd.grad(plain * mask, [x, w, b], go)
    for a_, e_ in zip(got, exp):
        assert helpers.rel_err(a_.cpu().numpy(), e_.cpu().numpy()) <= 1e-6
    yh = mconv.mcorrlcorr_masked(x.half(), w.half(), b.half(), lens, True)
    assert yh.dtype == torch.half and torch.equal(yh[2], torch.zeros_like(yh[2]))
