"""The grad-weight entry point that brings its own scratch.

Hosts that cannot allocate device memory where they need the gradient (a runtime
plugin handed a fixed arena, a real-time loop whose memory is pinned down at
start-up, a backward pass whose framework forbids allocation) call
``mellin_mcorrlcorr_grad_weight_noalloc_f32``: partial sums and index tables
live in a fixed array inside the library.  The file is collected last, so that
a run stopping at the first failure has already exercised everything else; the
test also passes when run alone in a fresh process.
"""
import numpy as np
import pytest
import torch

import capi

pytestmark = pytest.mark.gpu

TOL = 1e-5  # the per-tensor max-norm tolerance of the other float32 parity tests


def _rel(a, b):
    return float((a - b).abs().max() / b.abs().max())


@pytest.mark.parametrize("shape", [
    # (batch, c_in, c_out, (ngx, ngy), (nfx, nfy), d): first-layer and wide-layer kernels
    (4, 3, 64, (41, 200), (8, 3), (1, 1)),
    (2, 24, 40, (12, 96), (4, 3), (2, 1)),
])
def test_noalloc_matches_regular_entry_point_twice(shape):
    n, ci, co, ng, nf, d = shape
    s, p, u = (1, 1), (0, 1), (1, 1)
    gen = torch.Generator(device="cpu").manual_seed(1234)
    x = torch.randn((n, ci) + ng, generator=gen).cuda()
    gy = torch.randn((n, co) + ng, generator=gen).cuda()
    ref_w = torch.empty((co, ci) + nf, device="cuda")
    ref_b = torch.empty(co, device="cuda")
    capi.grad_weight(x, gy, ref_w, ref_b, s, d, p, u)
    for call in range(2):  # the second call finds the first one's leftovers in the shared array
        got_w = torch.full_like(ref_w, float("nan"))
        got_b = torch.full_like(ref_b, float("nan"))
        capi.grad_weight_noalloc(x, gy, got_w, got_b, s, d, p, u)
        torch.cuda.synchronize()
        assert _rel(got_w, ref_w) <= TOL, "call %d" % call
        assert _rel(got_b, ref_b) <= TOL, "call %d" % call
        # different data on the next round, same geometry
        x = x * 0.5 + 0.25
        capi.grad_weight(x, gy, ref_w, ref_b, s, d, p, u)


def test_noalloc_rejects_oversized_geometry():
    # 512 x 512 channels, 6 x 3 kernel: one copy of the gradient alone is 18.9 MB, above the built-in 8 MiB
    x = torch.zeros((1, 512, 8, 64), device="cuda")
    gy = torch.zeros((1, 512, 8, 64), device="cuda")
    gw = torch.zeros((512, 512, 6, 3), device="cuda")
    with pytest.raises(capi.MellinError) as e:
        capi.grad_weight_noalloc(x, gy, gw, None, (1, 1), (1, 1), (0, 1), (1, 1))
    assert e.value.code == 3 and "built-in scratch" in str(e.value)
    torch.cuda.synchronize()
