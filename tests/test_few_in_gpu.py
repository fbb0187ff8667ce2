"""First-layer forward on tensor cores (``csrc/tc_few_in.cu``): few input channels, many output channels.

The kernel folds the linear taps into the reduction (operand A is built in
tensor memory from three reads one position apart), takes the weights of an
output row's table entries as one prepared operand and writes every 64 x 128
output tile with one TMA store.  Checked here against the CPU oracle (the
reference's own kernels where they were built, ``mconv.h:296-371``) over the
template space of the kernel -- 1..4 input channels, 1..3 linear taps, channel
counts that are not multiples of the 64-channel tile, Mellin stride / dilation
/ padding that leave output rows WITHOUT table entries (they receive the
bias), linear extents that are not multiples of the 128-position tile, no bias
-- and for run-to-run bit identity.  Each case also checks that this kernel is
the one that ran (two launches: operand preparation, the kernel).
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


# (batch, c_in, c_out, (ngx, ngy), (nfx, nfy), s, d, p, u, r, bias)
CASES = [
    (3, 3, 64, (41, 800), (8, 3), (1, 1), (1, 1), (0, 1), (1, 1), (36, 1), True),    # the benchmark layer, small batch
    (2, 1, 16, (17, 132), (5, 3), (1, 1), (1, 1), (0, 1), (1, 1), (0, 1), True),     # one input channel, 16 outputs
    (2, 2, 100, (23, 260), (3, 2), (1, 1), (2, 1), (1, 1), (1, 1), (3, 0), False),   # 100 channels: second tile partly empty
    (2, 4, 128, (30, 128), (8, 1), (2, 1), (1, 1), (2, 0), (1, 1), (0, 0), True),    # Mellin stride 2, one linear tap
    (1, 3, 200, (64, 516), (6, 3), (1, 1), (3, 1), (0, 2), (1, 1), (20, 0), True),   # 4 channel tiles, rows without entries
    (2, 3, 32, (12, 72), (8, 3), (1, 1), (1, 1), (0, 0), (1, 1), (0, 2), True),      # no linear padding on the left
    (2, 4, 48, (9, 200), (2, 3), (3, 1), (1, 1), (0, 1), (1, 1), (5, 1), True),      # mostly rows without entries
]


@pytest.mark.parametrize("case", CASES, ids=[str(i) for i in range(len(CASES))])
def test_first_layer_forward_matches_the_oracle(oracle, case):
    n, ci, co, ng, nf, s, d, p, u, r, with_bias = case
    rng = np.random.default_rng(sum(ng) + co)
    x_h = rng.standard_normal((n, ci) + ng).astype(np.float32)
    w_h = rng.standard_normal((co, ci) + nf).astype(np.float32)
    b_h = rng.standard_normal(co).astype(np.float32) if with_bias else None
    y_exp = oracle.mcorrlcorr(x_h, w_h, b_h, s, d, p, u, r)
    assert y_exp.shape[3] % 4 == 0 and y_exp.shape[3] >= 64, y_exp.shape
    x, w = torch.from_numpy(x_h).cuda(), torch.from_numpy(w_h).cuda()
    b = torch.from_numpy(b_h).cuda() if with_bias else None
    results = []
    for _ in range(3):
        y = torch.full(y_exp.shape, float("nan"), device="cuda")
        before = capi.launch_count()
        capi.forward(x, w, b, y, s, d, p, u)
        launches = capi.launch_count() - before
        results.append(y)
    assert launches == 2, "the first-layer tensor-core kernel did not take this problem"
    assert helpers.rel_err(results[0].cpu().numpy(), y_exp) <= F32_TOL
    assert torch.equal(results[0], results[1]) and torch.equal(results[0], results[2])
    assert capi.device_status() == 0


def test_tensor_cores_off_gives_the_same_layer(oracle):
    case = CASES[0]
    n, ci, co, ng, nf, s, d, p, u, r, _ = case
    gen = torch.Generator(device="cuda").manual_seed(13)
    x = torch.randn((n, ci) + ng, device="cuda", generator=gen)
    w = torch.randn((co, ci) + nf, device="cuda", generator=gen)
    b = torch.randn((co,), device="cuda", generator=gen)
    shape = (n, co, ng[0], ng[1])
    on = torch.empty(shape, device="cuda")
    capi.forward(x, w, b, on, s, d, p, u)
    previous = capi.set_tensor_cores(False)
    try:
        off = torch.empty(shape, device="cuda")
        capi.forward(x, w, b, off, s, d, p, u)
    finally:
        capi.set_tensor_cores(previous)
    assert float((on - off).abs().max() / off.abs().max()) <= F32_TOL
