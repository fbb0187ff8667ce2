"""First-layer weight gradient on tensor cores (``csrc/tc_gradw_few_in.cu``): few input channels.

grad_y is read once; one GEMM per (output row, 128 positions) serves every
table entry of the row, with the positions as the reduction, two halves of 64
positions stacked along M, operand A (grad_y) in tensor memory and two-level
sums.  Checked here against the CPU oracle (the reference's own kernels where
they were built, ``mconv.h:373-460`` through the recipe of
``ext/torch.cpp:261-308``) over the template space of the kernel -- 1..4 input
channels, 1..3 linear taps, output channel counts that are not multiples of the
64-channel tile, Mellin stride / dilation / padding that leave rows of grad_y
that no tap reads (they count for the bias only), linear extents that are not
multiples of the 128-position items, with and without the bias gradient -- and
for run-to-run bit identity.  Each case also checks that this kernel is the one
that ran (two launches: partial sums, their reduction).
"""
import numpy as np
import pytest
import torch

import capi
import helpers
from oracle.oracle import Oracle

pytestmark = pytest.mark.gpu

F32_TOL = 2e-5


@pytest.fixture(scope="module")
def oracle():
    return Oracle("reference") if Oracle.reference_available() else Oracle("port")


# (batch, c_in, c_out, (ngx, ngy), (nfx, nfy), s, d, p, u, r, bias)
CASES = [
    (3, 3, 64, (41, 800), (8, 3), (1, 1), (1, 1), (0, 1), (1, 1), (36, 1), True),    # the benchmark layer, small batch
    (2, 1, 16, (17, 132), (5, 3), (1, 1), (1, 1), (0, 1), (1, 1), (0, 1), True),     # one input channel, 16 outputs
    (2, 2, 100, (23, 260), (3, 2), (1, 1), (2, 1), (1, 1), (1, 1), (3, 0), False),   # 100 channels: second tile partly empty
    (2, 4, 128, (30, 128), (6, 1), (2, 1), (1, 1), (2, 0), (1, 1), (0, 0), True),    # Mellin stride 2, one linear tap
    (1, 3, 200, (64, 516), (6, 3), (1, 1), (3, 1), (0, 2), (1, 1), (20, 0), True),   # 4 channel tiles, rows no tap reads
    (5, 4, 48, (9, 200), (2, 3), (3, 1), (1, 1), (0, 1), (1, 1), (5, 1), True),      # mostly rows no tap reads
]


@pytest.mark.parametrize("case", CASES, ids=[str(i) for i in range(len(CASES))])
def test_first_layer_weight_gradient_matches_the_oracle(oracle, case):
    n, ci, co, ng, nf, s, d, p, u, r, with_bias = case
    nhx = oracle.mcorr_valid_size(nf[0], ng[0], s[0], d[0], p[0], u[0]) + r[0]
    nhy = oracle.lcorr_valid_size(nf[1], ng[1], s[1], d[1], p[1], u[1]) + r[1]
    assert nhy % 4 == 0 and nhy >= 64
    rng = np.random.default_rng(sum(ng) + co)
    x_h = rng.standard_normal((n, ci) + ng).astype(np.float32)
    w_h = rng.standard_normal((co, ci) + nf).astype(np.float32)
    go_h = rng.standard_normal((n, co, nhx, nhy)).astype(np.float32)
    _, gw_exp, gb_exp = oracle.mcorrlcorr_backward(x_h, w_h, go_h, s, d, p, u)
    x, go = torch.from_numpy(x_h).cuda(), torch.from_numpy(go_h).cuda()
    results = []
    for _ in range(3):
        gw = torch.full((co, ci) + nf, float("nan"), device="cuda")
        gb = torch.full((co,), float("nan"), device="cuda") if with_bias else None
        before = capi.launch_count()
        capi.grad_weight(x, go, gw, gb, s, d, p, u)
        launches = capi.launch_count() - before
        results.append((gw, gb))
    assert launches == 2, "the first-layer tensor-core kernel did not take this problem"
    assert helpers.rel_err(results[0][0].cpu().numpy(), gw_exp) <= F32_TOL
    if with_bias:
        assert helpers.rel_err(results[0][1].cpu().numpy(), gb_exp) <= F32_TOL
    for gw, gb in results[1:]:
        assert torch.equal(gw, results[0][0])
        if with_bias:
            assert torch.equal(gb, results[0][1])
    assert capi.device_status() == 0
