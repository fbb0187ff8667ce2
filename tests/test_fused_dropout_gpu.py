"""Dropout fused into the layer's epilogue (conv -> ReLU -> length mask -> dropout in one kernel).

The reference's acoustic model applies these as separate operators
(models.py:424-434).  Checked here: the fused output equals the unfused layer
output times a 0 / (1 / (1 - p)) mask; the mask depends on the seed and the
element's position only -- not on which kernel wrote the tensor (tensor cores,
CUDA-core row kernel, extra pass, float64); the drop rate is p; backward equals
autograd through the unfused formulation with the same mask.
"""
import numpy as np
import pytest
import torch

import capi

pytestmark = pytest.mark.gpu

S, P, U = (1, 1), (0, 1), (1, 1)


@pytest.fixture(scope="module")
def mconv():
    import mconv as module

    return module


def _layer(n, ci, co, ng, nf, seed=0):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn((n, ci) + ng, device="cuda", generator=gen)
    w = torch.randn((co, ci) + nf, device="cuda", generator=gen) / float(np.sqrt(ci * nf[0] * nf[1]))
    b = torch.randn(co, device="cuda", generator=gen)
    lens = torch.randint(ng[1] // 3, ng[1] + 1, (n,), device="cuda", generator=gen, dtype=torch.int32)
    return x, w, b, lens


@pytest.mark.parametrize("shape", [
    (3, 3, 64, (12, 256), (4, 3)),     # first layer: tensor cores, or the row kernel when they are off
    (2, 24, 40, (12, 128), (4, 3)),    # wide layer
    (2, 5, 6, (9, 44), (3, 2)),        # covered by neither: plain operator + one more pass
], ids=["first_layer", "wide_layer", "odd_layer"])
def test_mask_is_a_function_of_seed_and_position_only(shape):
    n, ci, co, ng, nf = shape
    x, w, b, lens = _layer(n, ci, co, ng, nf)
    ys = (n, co) + ng
    p_drop, seed = 0.25, 12345
    base = torch.empty(ys, device="cuda")
    capi.forward_masked(x, w, b, lens, True, base, S, (1, 1), P, U)
    results = []
    for engine in (True, False):
        previous = capi.set_tensor_cores(engine)
        y = torch.full(ys, float("nan"), device="cuda")
        capi.forward_fused(x, w, b, lens, True, p_drop, seed, y, S, (1, 1), P, U)
        capi.set_tensor_cores(previous)
        results.append(y)
    y64 = torch.full(ys, float("nan"), device="cuda", dtype=torch.float64)
    capi.forward_fused(x.double(), w.double(), b.double(), lens, True, p_drop, seed, y64, S, (1, 1), P, U)
    kept = results[0] != 0
    # same mask whichever kernel wrote it (compare where the unfused output is clearly positive)
    live = base > 1e-3
    for other in (results[1], y64):
        assert torch.equal((other != 0) & live, kept & live)
    # kept elements are the unfused output scaled by 1 / (1 - p); dropped ones are zero
    scale = 1.0 / (1.0 - p_drop)
    assert torch.allclose(results[0][kept], base[kept] * scale, rtol=1e-5, atol=1e-6)
    assert float(results[0][~kept].abs().max()) == 0.0
    rate = 1.0 - float((kept & live).sum()) / float(live.sum())
    assert abs(rate - p_drop) < 0.02
    # another seed, another mask
    y2 = torch.empty(ys, device="cuda")
    capi.forward_fused(x, w, b, lens, True, p_drop, seed + 1, y2, S, (1, 1), P, U)
    assert float(((y2 != 0) != kept)[live].float().mean()) > 0.2  # two independent masks differ on 2 p (1 - p) = 37 % of the elements
    assert capi.device_status() == 0


def test_backward_matches_autograd_through_the_unfused_layer(mconv):
    n, ci, co, ng, nf = 2, 24, 40, (12, 128), (4, 3)
    x, w, b, lens = _layer(n, ci, co, ng, nf, seed=3)
    r = (ng[0] - mconv.mcorr_valid_size(nf[0], ng[0]), 1)
    p_drop, seed = 0.1, 777
    xa, wa, ba = (t.clone().requires_grad_(True) for t in (x, w, b))
    y = mconv.mcorrlcorr_masked(xa, wa, ba, lens, True, 1, 1, (0, 1), r, dropout_p=p_drop, seed=seed)
    go = torch.randn_like(y)
    y.backward(go)
    # unfused: the same mask (read off the fused output) applied by hand
    keep = (y.detach() != 0).float() / (1.0 - p_drop)
    xb, wb, bb = (t.clone().requires_grad_(True) for t in (x, w, b))
    base = mconv.mcorrlcorr_masked(xb, wb, bb, lens, True, 1, 1, (0, 1), r)
    (base * keep).backward(go)
    for got, ref in ((xa.grad, xb.grad), (wa.grad, wb.grad), (ba.grad, bb.grad)):
        assert float((got - ref).abs().max()) <= 1e-5 * float(ref.abs().max())
    # evaluation mode and p = 0 are the plain masked layer
    y_eval = mconv.mcorrlcorr_masked(x, w, b, lens, True, 1, 1, (0, 1), r, dropout_p=p_drop, training=False)
    assert torch.equal(y_eval, base.detach())
    # torch.manual_seed governs the mask when no seed is given
    torch.manual_seed(5)
    y1 = mconv.mcorrlcorr_masked(x, w, b, lens, True, 1, 1, (0, 1), r, dropout_p=p_drop)
    torch.manual_seed(5)
    y2 = mconv.mcorrlcorr_masked(x, w, b, lens, True, 1, 1, (0, 1), r, dropout_p=p_drop)
    assert torch.equal(y1, y2)
    with pytest.raises(RuntimeError):
        mconv.mcorrlcorr_masked(x, w, b, lens, False, 1, 1, (0, 1), r, dropout_p=p_drop)
