"""Regenerate ``tests/golden/prologue_cases.npz`` from a checkout of the reference (sdrobert/cnn-mellin).

    python tests/golden/make_prologue_golden.py

imports the reference's own ``layers.py`` (stock torch operators, CPU) and records, on seeded inputs in float32 and
float64, what the model's prologue computes (``models.py:413-417``: ``LogCompression`` then ``DilationLift``) and
what autograd returns for it: the output, the gradient of the input and of ``log_tau`` / ``log_eps``, for the pair and
for each layer alone, over several ``dim`` (negative ones too), shapes with a lifted axis of 1, inner extents that
are and are not multiples of 4, and an input holding exact zeros.  ``MELLIN_REFERENCE`` names the checkout when it
is not at the default location.  Neither the tests nor the benchmark read the checkout; they read the file.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE = os.environ.get("MELLIN_REFERENCE", "/root/reference")

# (shape, dim, use_log_compression, use_lift)
CASES = [
    ((5, 9, 41), 2, True, True),       # the model's call: packed windows (N', w, F), lift over dim 2
    ((2, 3, 41, 20), 2, True, True),   # a layer-shaped batch, lift over the Mellin axis
    ((2, 3, 41, 20), -1, True, True),  # lift over the last (contiguous) axis
    ((6, 7, 5), 1, True, True),        # inner extent not a multiple of 4
    ((3, 1, 8), 1, True, True),        # lifted axis of length 1
    ((2, 3, 16, 12), 0, False, True),  # the lift alone, over the first axis
    ((2, 3, 16, 12), -2, False, True),
    ((7, 33), 1, True, False),         # compression alone
    ((64, 20), 0, True, True),
]


def main():
    sys.path.insert(0, REFERENCE)
    import torch

    import layers  # the reference's

    out = {}
    rng = np.random.default_rng(20240611)
    for idx, (shape, dim, use_lc, use_lift) in enumerate(CASES):
        for dtype in (np.float32, np.float64):
            tag = "c%d_%s" % (idx, np.dtype(dtype).name)
            x_h = rng.standard_normal(shape).astype(dtype)
            x_h.flat[:: 11] = 0.0  # exact zeros: abs is not differentiable there, torch takes 0
            g_h = rng.standard_normal(shape).astype(dtype)
            log_tau, log_eps = float(rng.normal() * 0.5), float(rng.normal())
            x = torch.from_numpy(x_h.copy()).requires_grad_(True)
            lc, lift = layers.LogCompression(), layers.DilationLift(dim)
            if dtype == np.float64:  # parameters in the input's precision, so that exp() is taken in it too
                lc, lift = lc.double(), lift.double()
            with torch.no_grad():
                lc.log_eps.fill_(log_eps)
                lift.log_tau.fill_(log_tau)
            y = x
            if use_lc:
                y = lc(y)
            if use_lift:
                y = lift(y)
            y.backward(torch.from_numpy(g_h))
            out[tag + "_x"], out[tag + "_grad_y"], out[tag + "_y"] = x_h, g_h, y.detach().numpy()
            out[tag + "_grad_x"] = x.grad.numpy()
            out[tag + "_meta"] = np.array([dim, int(use_lc), int(use_lift)], dtype=np.int64)
            out[tag + "_params"] = np.array([float(lift.log_tau.detach()), float(lc.log_eps.detach())], dtype=np.float64)
            out[tag + "_grad_params"] = np.array(
                [float(lift.log_tau.grad) if use_lift else np.nan, float(lc.log_eps.grad) if use_lc else np.nan])
    np.savez_compressed(os.path.join(HERE, "prologue_cases.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
