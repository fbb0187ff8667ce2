"""The conv stack of the reference's acoustic model, at its shapes, against the oracle.

The reference's ``models.AcousticModel`` (models.py:261-340, 395-434) cuts every
utterance into overlapping windows and feeds ALL windows of ALL utterances as one
big batch of small images to its conv stack: inputs ``(N', 1, window, freq)`` with
the Mellin axis on the window (2-9 samples) and the linear axis on frequency
(41 or 81 bins), 3x3 kernels, Mellin padding ``p = (kx - 1) // 2``, frequency
stride 1 or 2, Mellin dilation ``(decim - 1) kx + 1`` on the "on" layers, and
``r`` chosen so that the output has ``window // decim`` samples (it can be
negative).  With 9 taps the functional interface picks the gather + matrix
product implementation (``_impl="mm"``, mconv.py:975-986 there), a regime no
benchmark configuration touches.  The model itself needs the ``param`` package,
which is not installed here, so its layers are rebuilt from their constructor
arithmetic and compared, forward and backward, with the CPU oracle; both
implementations (``mm`` and ``direct``) are held to it.
"""
import numpy as np
import pytest
import torch

import helpers
from oracle.oracle import Oracle

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5


@pytest.fixture(scope="module")
def mconv():
    import mconv as module

    return module


@pytest.fixture(scope="module")
def oracle():
    return Oracle("reference") if Oracle.reference_available() else Oracle("port")


def _stack(window, freq, layers, initial_channels, channel_factor, time_factor, freq_factor, schedule, kx=3, ky=3):
    """Constructor arithmetic of the reference's Mellin branch (models.py:281-327): list of
    (c_in, c_out, (kx, ky), s, d, p, r) and the (window, freq) extents each layer sees."""
    def mcorr_valid(nf, ng, s, d, p):
        return max((ng * (p + 1)) // (nf + d - 1) - s + 1, 0)

    def lcorr_valid(nf, ng, s, d, p):
        return max((ng - 1 - d * (nf - 1) + p) // s + 1, 0)

    x, y, ci, co = window, freq, 1, initial_channels
    px, py = (kx - 1) // 2, (ky - 1) // 2
    on_dx = (time_factor - 1) * kx + 1
    out = []
    for layer_no in range(1, layers + 1):
        if layer_no % schedule:
            dx, sx, sy, big_dx, big_dy = 1, 1, 1, 1, 1
        else:
            dx, sx, sy, co, big_dx, big_dy = on_dx, 1, freq_factor, channel_factor * co, time_factor, freq_factor
        new_x = mcorr_valid(kx, x, sx, dx, px)
        rx = max(x // big_dx, 1) - new_x
        new_y = lcorr_valid(ky, y, sy, 1, py)
        ry = max(y // big_dy, 1) - new_y
        out.append(dict(ci=ci, co=co, nf=(kx, ky), s=(sx, sy), d=(dx, 1), p=(px, py), r=(rx, ry), size=(x, y)))
        x, y, ci = new_x + rx, new_y + ry, co
    return out


STACKS = {
    # window, freq, layers, initial channels, channel factor, time (window) factor, freq factor, schedule
    "window9_freq41": (9, 41, 4, 8, 2, 2, 2, 2),
    "window5_freq81": (5, 81, 3, 4, 2, 2, 3, 2),
    "window2_freq41": (2, 41, 2, 8, 1, 1, 2, 1),
}


@pytest.mark.parametrize("impl", ["mm", "direct", None])
@pytest.mark.parametrize("name", sorted(STACKS))
def test_conv_stack_layers_match_the_oracle(mconv, oracle, name, impl):
    rng = np.random.default_rng(len(name) * 7 + STACKS[name][0])
    frames = 37  # N': windows of all utterances packed into one batch
    for layer in _stack(*STACKS[name]):
        ci, co, nf, s, d, p, r, size = (layer[k] for k in ("ci", "co", "nf", "s", "d", "p", "r", "size"))
        x_h = rng.standard_normal((frames, ci) + size).astype(np.float32)
        w_h = (rng.standard_normal((co, ci) + nf) / np.sqrt(ci * nf[0] * nf[1])).astype(np.float32)
        b_h = rng.standard_normal(co).astype(np.float32)
        y_exp = oracle.mcorrlcorr(x_h, w_h, b_h, s, d, p, (1, 1), r)
        assert y_exp.shape[2] >= 1 and y_exp.shape[3] >= 1, layer
        go_h = rng.standard_normal(y_exp.shape).astype(np.float32)
        gx_exp, gw_exp, gb_exp = oracle.mcorrlcorr_backward(x_h, w_h, go_h, s, d, p, (1, 1))
        x = torch.from_numpy(x_h).cuda().requires_grad_(True)
        w = torch.from_numpy(w_h).cuda().requires_grad_(True)
        b = torch.from_numpy(b_h).cuda().requires_grad_(True)
        y = mconv.mcorrlcorr(x, w, b, s, d, p, r, _impl=impl)
        y.backward(torch.from_numpy(go_h).cuda())
        assert y.shape == y_exp.shape, layer
        assert helpers.rel_err(y.detach().cpu().numpy(), y_exp) <= F32_TOL, layer
        assert helpers.rel_err(x.grad.cpu().numpy(), gx_exp) <= F32_TOL, layer
        assert helpers.rel_err(w.grad.cpu().numpy(), gw_exp) <= 2 * F32_TOL, layer
        assert helpers.rel_err(b.grad.cpu().numpy(), gb_exp) <= F32_TOL, layer


def test_raw_audio_branch_uses_the_1d_layer(mconv, oracle):
    """freq_dim == 1 in the reference's model (models.py:279, 305-306): MCorr1d over the window axis."""
    rng = np.random.default_rng(8)
    frames, window, kx = 64, 9, 3
    for ci, co, d, r in ((1, 8, 1, 0), (8, 16, 4, 3)):
        p = (kx - 1) // 2
        x_h = rng.standard_normal((frames, ci, window)).astype(np.float32)
        w_h = (rng.standard_normal((co, ci, kx)) / np.sqrt(ci * kx)).astype(np.float32)
        b_h = rng.standard_normal(co).astype(np.float32)
        y_exp = oracle.mcorr1d(x_h, w_h, b_h, 1, d, p, 1, r)
        go_h = rng.standard_normal(y_exp.shape).astype(np.float32)
        gx_exp, gw_exp, gb_exp = oracle.mcorr1d_backward(x_h, w_h, go_h, 1, d, p, 1)
        layer = mconv.MCorr1d(ci, co, kx, 1, d, p, r).cuda()
        with torch.no_grad():
            layer.weight.copy_(torch.from_numpy(w_h))
            layer.bias.copy_(torch.from_numpy(b_h))
        x = torch.from_numpy(x_h).cuda().requires_grad_(True)
        y = layer(x)
        y.backward(torch.from_numpy(go_h).cuda())
        assert helpers.rel_err(y.detach().cpu().numpy(), y_exp) <= F32_TOL
        assert helpers.rel_err(x.grad.cpu().numpy(), gx_exp) <= F32_TOL
        assert helpers.rel_err(layer.weight.grad.cpu().numpy(), gw_exp) <= 2 * F32_TOL
        assert helpers.rel_err(layer.bias.grad.cpu().numpy(), gb_exp) <= F32_TOL
