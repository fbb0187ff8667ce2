"""CPU-only checks: the C-ABI library loads and exports everything the header
declares, its size functions match the oracle, and the host-built Mellin index
maps contain exactly the index triples the defining relations allow."""
import itertools
import os
import re

import numpy as np
import pytest

import capi
from oracle.oracle import Oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OWNER, ONLY, MASK = 1 << 29, 1 << 30, (1 << 29) - 1


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "mellin_b200.h")).read()
    # plain prototypes "name(" and macro-declared families "DECL(name, T, ...)"
    declared = set(re.findall(r"\b(mellin_[a-z0-9_]+)\s*[\(,]", header))
    assert declared == set(capi.exported_symbols()), declared ^ set(capi.exported_symbols())
    lib = capi.lib()
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.mellin_abi_version() == 100


def test_size_functions_match_oracle():
    o = Oracle("port")
    lib = capi.lib()
    for nf, ng, s, d, p, u in itertools.product((1, 3, 8, 16), (1, 5, 41, 256), (1, 2, 3), (1, 2, 5), (0, 1, 3), (1, 2)):
        assert lib.mellin_mconv_valid_size(ng, s, d, p, u) == o.mconv_valid_size(nf, ng, s, d, p, u)
        assert lib.mellin_mconv_support_size(nf, ng, s, d, p, u) == o.mconv_support_size(nf, ng, s, d, p, u)
        assert lib.mellin_mcorr_valid_size(nf, ng, s, d, p, u) == o.mcorr_valid_size(nf, ng, s, d, p, u)
        assert lib.mellin_mcorr_support_size(ng, s, d, p, u) == o.mcorr_support_size(nf, ng, s, d, p, u)
        assert lib.mellin_lconv_valid_size(ng, s, p, u) == o.lconv_valid_size(nf, ng, s, d, p, u)
        assert lib.mellin_lconv_support_size(nf, ng, s, d, p, u) == o.lconv_support_size(nf, ng, s, d, p, u)
        assert lib.mellin_lcorr_valid_size(nf, ng, s, d, p, u) == o.lcorr_valid_size(nf, ng, s, d, p, u)
        assert lib.mellin_lcorr_support_size(ng, s, p, u) == o.lcorr_support_size(nf, ng, s, d, p, u)


def brute_triples(relation, nf, ng, nh, s, d, p, u):
    P = p + 1
    out = set()
    for h in range(nh):
        for f in range(nf):
            num, den = ((h + s) * (f + d), P) if relation == "corr" else (P * (h + s), f + d)
            if den == 0 or num % den:
                continue
            g = num // den - u
            if 0 <= g < ng:
                out.add((h, f, g))
    return out


@pytest.mark.parametrize("relation", ["corr", "conv"])
@pytest.mark.parametrize("nf,ng,nh,s,d,p,u", [
    (8, 41, 41, 1, 1, 0, 1), (6, 41, 41, 1, 2, 0, 1), (16, 256, 256, 1, 1, 0, 1), (4, 12, 20, 2, 2, 3, 1),
    (3, 4, 9, 2, 3, 3, 5), (5, 7, 3, 1, 1, 1, 2), (1, 1, 1, 1, 1, 0, 1), (3, 10, 0, 1, 1, 0, 1), (0, 5, 5, 1, 1, 0, 1),
])
def test_index_maps_hold_exactly_the_valid_triples(relation, nf, ng, nh, s, d, p, u):
    want = brute_triples(relation, nf, ng, nh, s, d, p, u)
    # rows = hx
    rp, en = capi.index_map(relation, "h", nf, ng, nh, s, d, p, u)
    got = {(h, int(a), int(b)) for h in range(nh) for a, b in en[rp[h]:rp[h + 1]]}
    assert got == want and len(en) == len(want)
    # rows = gx
    rp, en = capi.index_map(relation, "g", nf, ng, nh, s, d, p, u)
    got = {(int(b), int(a), g) for g in range(ng) for a, b in en[rp[g]:rp[g + 1]]}
    assert got == want and len(en) == len(want)
    # rows = fx, with the bias bookkeeping: every hx row is owned exactly once
    rp, en = capi.index_map(relation, "f", nf, ng, nh, s, d, p, u)
    got, owners = set(), []
    for f in range(nf):
        for a, b in en[rp[f]:rp[f + 1]]:
            a, b = int(a), int(b)
            if a & OWNER:
                owners.append(a & MASK)
            if a & ONLY:
                assert f == 0 and (a & OWNER)
            else:
                got.add((a & MASK, f, b))
    assert got == want
    if nf > 0:
        assert sorted(owners) == list(range(nh))


def test_pair_counts_of_the_baseline_configurations():
    # number of (hx, fx) index pairs per configuration: these drive the
    # algorithmic flop counts quoted for the benchmark
    def pairs(nf, ng, nh, d=1):
        return len(capi.index_map("corr", "h", nf, ng, nh, 1, d, 0, 1)[1])

    assert pairs(16, 256, 16) == 256 and pairs(16, 256, 256) == 861      # 1-D, valid / same size
    assert pairs(8, 41, 41) == 108 and pairs(8, 41, 5) == 40              # 2-D layer, kernel 8 x 3
    assert pairs(6, 41, 41) == 98 and pairs(6, 41, 41, d=2) == 62         # stacked layers, kernel 6 x 3
    assert pairs(64, 16384, 256) == 16384 and pairs(64, 16384, 16384) == 77701


def test_bad_index_map_arguments():
    with pytest.raises(capi.MellinError):
        capi.index_map("corr", "h", 3, 5, 5, 1, 1, -1, 1)


def test_prologue_layers_keep_the_reference_names_and_refuse_the_cpu():
    """``layers.py``: parameter names of the reference (``lift.log_tau``, ``log_compression.log_eps``), its error for a
    bad ``dim``, and no CPU path."""
    import pytest
    import torch

    import layers

    pair = layers.LogCompressionLift()
    assert set(pair.state_dict()) == {"log_compression.log_eps", "lift.log_tau"}
    assert pair.lift.dim == 2 and pair.lift.log_tau.shape == () and pair.log_compression.log_eps.shape == ()
    assert set(layers.LogCompressionLift(use_lift=False).state_dict()) == {"log_compression.log_eps"}
    assert "dim=2" in repr(layers.DilationLift())
    with pytest.raises(RuntimeError, match="-4 not a valid dimension for a tensor if dimension 3"):
        layers.dilation_lift(torch.zeros(2, 3, 4), torch.tensor(1.0), -4)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        pair(torch.zeros(2, 3, 4))
    x = torch.zeros(2, 3)
    assert layers.LogCompressionLift(False, False)(x) is x
    # the noise layer the reference's training loop imports from the same file: identity in evaluation mode,
    # deviation eps * max|x| along dim when training
    noise = layers.ScaledGaussianNoise(1, 0.5)
    x = torch.ones(4, 20000)
    assert noise.eval()(x) is x
    torch.manual_seed(1)
    y = noise.train()(x)
    assert abs(float((y - x).std()) - 0.5) < 0.02 and abs(float((y - x).mean())) < 0.02


def test_prologue_entry_points_validate_before_touching_the_device():
    """Argument checks of ``mellin_lift_compress_*`` answer on a host without a GPU: nothing is launched for them."""
    import ctypes

    lib = capi.lib()
    i64, null = ctypes.c_int64, ctypes.c_void_p(0)
    fwd = lib.mellin_lift_compress_f32
    assert fwd(null, null, null, 1, i64(-1), i64(4), i64(4), null, null) == 1  # negative extent
    assert b"negative extent" in lib.mellin_last_error()
    assert fwd(null, null, null, 1, i64(2), i64(4), i64(4), null, null) == 1   # null tensors, 32 elements
    assert b"null pointer" in lib.mellin_last_error()
    assert fwd(null, null, null, 1, i64(0), i64(4), i64(4), null, null) == 0   # nothing to do
    assert fwd(null, null, null, 1, i64(2 ** 40), i64(2 ** 20), i64(2 ** 20), null, null) == 4  # beyond 2^63 elements
    bwd = lib.mellin_lift_compress_backward_f64
    assert bwd(null, null, null, null, 0, i64(0), i64(4), i64(4), null, null, null, null, ctypes.c_size_t(0), null) == 3
    assert b"workspace" in lib.mellin_last_error()
    assert capi.lift_compress_workspace_bytes() == 4096 * 2 * 8
