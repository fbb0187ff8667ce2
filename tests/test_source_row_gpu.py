"""Few-output-channel operators walked by SOURCE row on tensor cores (``csrc/tc_scatter.cu``).

The input gradient of a first layer (a handful of feature maps receive the
gradient of 16..128 channels) fetches every row of ``grad_y`` once, serves all
the Mellin table entries of the row with one tcgen05 GEMM, keeps one partial
plane per entry and sums the planes of every output row in table order.  Checked here against the CPU oracle (the reference's own
kernels where they were built, ``mconv.h:296-371``) over the template space of
the kernel -- 1..4 receiving channels, 1..3 linear taps, 1..8 Mellin taps,
Mellin stride / dilation / padding that give long, short and EMPTY table
rows, linear extents that are not multiples of the 128-position items,
channel counts that do not fill the last 8-channel box -- and for run-to-run
bit identity.  Each case also checks that the by-source-row kernels are the
ones that ran (three launches: B operands, partial planes, plane sum).
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


# (batch, c_in, c_out, (ngx, ngy), (nfx, nfy), s, d, p, u)
CASES = [
    (3, 3, 64, (41, 800), (8, 3), (1, 1), (1, 1), (0, 1), (1, 1)),     # the benchmark layer, small batch
    (2, 1, 16, (17, 132), (5, 3), (1, 1), (1, 1), (0, 1), (1, 1)),     # one receiving channel, 16 reduced
    (2, 2, 20, (23, 260), (3, 2), (1, 1), (2, 1), (1, 1), (1, 1)),     # 20 channels: last box half empty; 2 taps
    (2, 4, 24, (30, 128), (8, 1), (2, 1), (1, 1), (2, 0), (1, 1)),     # Mellin stride 2, padding 2, one linear tap
    (1, 3, 40, (64, 516), (6, 3), (1, 1), (3, 1), (0, 2), (1, 1)),     # Mellin dilation 3, linear padding 2
    (2, 3, 32, (12, 70), (8, 3), (1, 1), (1, 1), (0, 0), (1, 1)),      # no linear padding: valid output is shorter
    (2, 3, 16, (9, 200), (2, 3), (3, 1), (1, 1), (0, 1), (1, 1)),      # Mellin stride 3: most table rows empty
    (1, 4, 128, (20, 400), (4, 3), (1, 1), (1, 1), (1, 1), (1, 1)),    # 128 reduced channels
]


def _shapes(case, oracle):
    """Output extents: the valid size on the Mellin axis (the benchmark layer: same size), the valid size
    rounded up to a multiple of 4 on the linear axis (the layer's ``r``; rows are copied in 16-byte chunks)."""
    n, ci, co, ng, nf, s, d, p, u = case
    nhx = ng[0] if case is CASES[0] else oracle.mcorr_valid_size(nf[0], ng[0], s[0], d[0], p[0], u[0])
    nhy = (oracle.lcorr_valid_size(nf[1], ng[1], s[1], d[1], p[1], u[1]) + 3) // 4 * 4
    return (n, ci) + ng, (co, ci) + nf, (n, co, nhx, nhy)


@pytest.mark.parametrize("case", CASES, ids=[str(i) for i in range(len(CASES))])
def test_grad_input_by_source_row_matches_the_oracle(oracle, case):
    n, ci, co, ng, nf, s, d, p, u = case
    x_shape, w_shape, y_shape = _shapes(case, oracle)
    assert y_shape[2] >= 1 and y_shape[3] >= 1
    rng = np.random.default_rng(sum(ng) + co)
    w_h = rng.standard_normal(w_shape).astype(np.float32)
    go_h = rng.standard_normal(y_shape).astype(np.float32)
    x_h = rng.standard_normal(x_shape).astype(np.float32)
    gx_exp, _, _ = oracle.mcorrlcorr_backward(x_h, w_h, go_h, s, d, p, u)
    w, go = torch.from_numpy(w_h).cuda(), torch.from_numpy(go_h).cuda()
    results = []
    for _ in range(3):
        gx = torch.full(x_shape, float("nan"), device="cuda")
        before = capi.launch_count()
        capi.grad_input(w, go, gx, s, d, p, u)
        launches = capi.launch_count() - before
        results.append(gx)
    assert launches == 3, "the by-source-row kernels did not take this problem"
    assert helpers.rel_err(results[0].cpu().numpy(), gx_exp) <= F32_TOL
    assert torch.equal(results[0], results[1]) and torch.equal(results[0], results[2])
    assert capi.device_status() == 0


def test_forward_onto_few_channels_by_source_row(oracle):
    """A forward pass onto 2 channels takes the same kernels (bias added by the plane sum)."""
    n, ci, co, ng, nf, s, d, p, u = 2, 48, 2, (25, 300), (7, 3), (1, 1), (1, 1), (0, 1), (1, 1)
    rng = np.random.default_rng(3)
    x_h = rng.standard_normal((n, ci) + ng).astype(np.float32)
    w_h = rng.standard_normal((co, ci) + nf).astype(np.float32)
    b_h = rng.standard_normal(co).astype(np.float32)
    y_exp = oracle.mcorrlcorr(x_h, w_h, b_h, s, d, p, u, (2, 1))
    assert y_exp.shape[3] == 300
    y = torch.full(y_exp.shape, float("nan"), device="cuda")
    before = capi.launch_count()
    capi.forward(torch.from_numpy(x_h).cuda(), torch.from_numpy(w_h).cuda(), torch.from_numpy(b_h).cuda(), y, s, d, p, u)
    assert capi.launch_count() - before == 3
    assert helpers.rel_err(y.cpu().numpy(), y_exp) <= F32_TOL
    assert capi.device_status() == 0


def test_without_workspace_the_by_output_row_kernel_answers(oracle):
    """The partial planes live in the caller's workspace; a call that brings less gets the other kernel, same result."""
    case = CASES[0]
    n, ci, co, ng, nf, s, d, p, u = case
    x_shape, w_shape, y_shape = _shapes(case, oracle)
    gen = torch.Generator(device="cuda").manual_seed(11)
    w = torch.randn(w_shape, device="cuda", generator=gen)
    go = torch.randn(y_shape, device="cuda", generator=gen)
    full = torch.empty(x_shape, device="cuda")
    capi.grad_input(w, go, full, s, d, p, u)
    small = torch.empty(x_shape, device="cuda")
    capi.grad_input(w, go, small, s, d, p, u, workspace=torch.empty(65536, dtype=torch.uint8, device="cuda"))
    assert float((full - small).abs().max() / full.abs().max()) <= F32_TOL
