"""CPU checkers for the Mellin operators -- TEST INFRASTRUCTURE ONLY.

Nothing in the product imports this module.  It is used by the test-suite,
by the smoke check and by the CPU-baseline leg of the benchmark.

Two interchangeable backends share one interface (:class:`Oracle`):

``Oracle("port")``
    the plain-C restatement in ``mellin_oracle.c`` (always available);
``Oracle("reference")``
    the reference's own header-only CPU kernels behind ``ref_shim.cpp``
    (available where ``oracle/_ref/libmellin_ref.so`` has been built).

All arrays are C-contiguous numpy arrays of float32 or float64.  The low-level
methods mirror the reference's L0 entry points
(``ext/include/cdrobert/mellin/mconv.h:52-425``): raw buffers, explicit sizes,
transposition flags, accumulate-into-``h`` semantics.  The ``forward`` /
``backward`` helpers on top restate what the reference's torch binding does
around them (``ext/torch_cpu.cpp:29-145``, ``ext/torch.cpp:176-308``).
"""
import ctypes
import os

import numpy as np

from . import build_oracle

_I64 = ctypes.c_int64
_INT = ctypes.c_int


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _sfx(dtype):
    if dtype == np.float32:
        return "f32"
    if dtype == np.float64:
        return "f64"
    raise TypeError("oracle supports float32 and float64, got %s" % dtype)


def _pair(v):
    if isinstance(v, (int, np.integer)):
        return (int(v), int(v))
    v = tuple(int(x) for x in v)
    assert len(v) == 2
    return v


class Oracle:
    def __init__(self, kind="port"):
        self.kind = kind
        if kind == "port":
            path = build_oracle.build_port()
            self._prefix = "oracle_"
        elif kind == "reference":
            path = build_oracle.build_reference()
            if path is None:
                raise FileNotFoundError(
                    "oracle/_ref/libmellin_ref.so is not built and no reference checkout is reachable"
                )
            self._prefix = "ref_"
        else:
            raise ValueError(kind)
        self._lib = ctypes.CDLL(path)
        for name, nargs in (
            ("mconv_valid_size", 5),
            ("mconv_support_size", 6),
            ("mcorr_valid_size", 6),
            ("mcorr_support_size", 5),
            ("lconv_valid_size", 4),
            ("lconv_support_size", 6),
            ("lcorr_valid_size", 6),
            ("lcorr_support_size", 4),
        ):
            fn = getattr(self._lib, self._prefix + name)
            fn.restype = _I64
            fn.argtypes = [_I64] * nargs

    @staticmethod
    def reference_available():
        return build_oracle.build_reference() is not None

    # ---- sizes (uniform Python signature of mconv.py:73-118) ----------------
    def mconv_valid_size(self, nf, ng, s=1, d=1, p=0, u=1):
        return self._lib.__getattr__(self._prefix + "mconv_valid_size")(ng, s, d, p, u)

    def mconv_support_size(self, nf, ng, s=1, d=1, p=0, u=1):
        return self._lib.__getattr__(self._prefix + "mconv_support_size")(nf, ng, s, d, p, u)

    def mcorr_valid_size(self, nf, ng, s=1, d=1, p=0, u=1):
        return self._lib.__getattr__(self._prefix + "mcorr_valid_size")(nf, ng, s, d, p, u)

    def mcorr_support_size(self, nf, ng, s=1, d=1, p=0, u=1):
        return self._lib.__getattr__(self._prefix + "mcorr_support_size")(ng, s, d, p, u)

    def lconv_valid_size(self, nf, ng, s=1, d=1, p=0, u=1):
        return self._lib.__getattr__(self._prefix + "lconv_valid_size")(ng, s, p, u)

    def lconv_support_size(self, nf, ng, s=1, d=1, p=0, u=1):
        return self._lib.__getattr__(self._prefix + "lconv_support_size")(nf, ng, s, d, p, u)

    def lcorr_valid_size(self, nf, ng, s=1, d=1, p=0, u=1):
        return self._lib.__getattr__(self._prefix + "lcorr_valid_size")(nf, ng, s, d, p, u)

    def lcorr_support_size(self, nf, ng, s=1, d=1, p=0, u=1):
        return self._lib.__getattr__(self._prefix + "lcorr_support_size")(ng, s, p, u)

    # ---- raw operators --------------------------------------------------------
    def op2d(self, kind, f, g, h, c_out, c_in, batch, s, d, p, u, tf=False, tg=False, th=False):
        """Accumulate the 2-D operator into ``h`` in place.

        ``kind``: "corr" (Mellin corr x linear corr) or "conv".  ``f``/``g``/``h``
        are 4-D; when a ``t*`` flag is set the array's two leading extents are
        (channels, batch) / (c_in, c_out) instead of the usual order.
        """
        (sx, sy), (dx, dy), (px, py), (ux, uy) = _pair(s), _pair(d), _pair(p), _pair(u)
        assert f.dtype == g.dtype == h.dtype
        for a in (f, g, h):
            assert a.flags["C_CONTIGUOUS"] and a.ndim == 4
        nfx, nfy = f.shape[2:]
        ngx, ngy = g.shape[2:]
        nhx, nhy = h.shape[2:]
        sfx = _sfx(f.dtype)
        common = [_I64(c_out), _I64(c_in), _I64(batch), _I64(nfx), _I64(nfy), _I64(ngx), _I64(ngy),
                  _I64(nhx), _I64(nhy), _I64(sx), _I64(sy), _I64(dx), _I64(dy), _I64(px), _I64(py),
                  _I64(ux), _I64(uy), _INT(tf), _INT(tg), _INT(th), _ptr(h)]
        if self.kind == "port":
            fn = getattr(self._lib, "oracle_op2d_" + sfx)
            fn.restype = None
            fn(_INT(0 if kind == "corr" else 1), _ptr(f), _ptr(g), *common)
        else:
            fn = getattr(self._lib, ("ref_mcorrlcorr_" if kind == "corr" else "ref_mconvlconv_") + sfx)
            fn.restype = None
            fn(_ptr(f), _ptr(g), *common)
        return h

    def op1d(self, kind, f, g, h, c_out, c_in, batch, s, d, p, u, tf=False, tg=False, th=False):
        """1-D Mellin operator, accumulated into ``h`` (3-D arrays)."""
        if self.kind == "reference":
            # the reference has dedicated 1-D entry points; use them so that
            # they are exercised too
            sfx = _sfx(f.dtype)
            fn = getattr(self._lib, ("ref_mcorr1d_" if kind == "corr" else "ref_mconv1d_") + sfx)
            fn.restype = None
            fn(_ptr(f), _ptr(g), _I64(c_out), _I64(c_in), _I64(batch), _I64(f.shape[2]),
               _I64(g.shape[2]), _I64(h.shape[2]), _I64(s), _I64(d), _I64(p), _I64(u),
               _INT(tf), _INT(tg), _INT(th), _ptr(h))
            return h
        self.op2d(kind, f[..., None], g[..., None], h[..., None], c_out, c_in, batch,
                  (s, 1), (d, 1), (p, 0), (u, 1), tf, tg, th)
        return h

    def _col(self, name, src, dst, c_in, batch, nf, ng, ngg, s, d, p, u, tg, tgg):
        (sx, sy), (dx, dy), (px, py), (ux, uy) = _pair(s), _pair(d), _pair(p), _pair(u)
        sfx = _sfx(src.dtype)
        assert src.dtype == dst.dtype and src.flags["C_CONTIGUOUS"] and dst.flags["C_CONTIGUOUS"]
        fn = getattr(self._lib, self._prefix + name + "_" + sfx)
        fn.restype = None
        fn(_ptr(src), _I64(c_in), _I64(batch), _I64(nf[0]), _I64(nf[1]), _I64(ng[0]), _I64(ng[1]),
           _I64(ngg[0]), _I64(ngg[1]), _I64(sx), _I64(sy), _I64(dx), _I64(dy), _I64(px), _I64(py),
           _I64(ux), _I64(uy), _INT(tg), _INT(tgg), _ptr(dst))
        return dst

    def spec2col_raw(self, g, gg, nf, s, d, p, u, tg=False, tgg=False):
        batch, c_in = (g.shape[1], g.shape[0]) if tg else g.shape[:2]
        return self._col("spec2col", g, gg, c_in, batch, _pair(nf), g.shape[2:], gg.shape[4:], s, d, p, u, tg, tgg)

    def col2spec_raw(self, gg, g, s, d, p, u, tg=False, tgg=False):
        batch, c_in = (g.shape[1], g.shape[0]) if tg else g.shape[:2]
        return self._col("col2spec", gg, g, c_in, batch, gg.shape[2:4], g.shape[2:], gg.shape[4:], s, d, p, u, tg, tgg)

    # ---- what the torch binding does around the raw operators -----------------
    @staticmethod
    def _init_out(shape, dtype, bias):
        # output starts as the broadcast bias or zero (ext/torch.cpp:88-101)
        h = np.zeros(shape, dtype=dtype)
        if bias is not None:
            h += bias.reshape((1, -1) + (1,) * (len(shape) - 2)).astype(dtype)
        return h

    def mcorrlcorr(self, x, w, bias=None, s=1, d=1, p=0, u=1, r=0):
        s, d, p, u, r = map(_pair, (s, d, p, u, r))
        nhx = self.mcorr_valid_size(w.shape[2], x.shape[2], s[0], d[0], p[0], u[0]) + r[0]
        nhy = self.lcorr_valid_size(w.shape[3], x.shape[3], s[1], d[1], p[1], u[1]) + r[1]
        h = self._init_out((x.shape[0], w.shape[0], nhx, nhy), w.dtype, bias)
        return self.op2d("corr", w, x, h, w.shape[0], w.shape[1], x.shape[0], s, d, p, u)

    def mconvlconv(self, x, w, bias=None, s=1, d=1, p=0, u=1, r=0):
        s, d, p, u, r = map(_pair, (s, d, p, u, r))
        nhx = self.mconv_valid_size(w.shape[2], x.shape[2], s[0], d[0], p[0], u[0]) + r[0]
        nhy = self.lconv_valid_size(w.shape[3], x.shape[3], s[1], d[1], p[1], u[1]) + r[1]
        h = self._init_out((x.shape[0], w.shape[0], nhx, nhy), w.dtype, bias)
        return self.op2d("conv", w, x, h, w.shape[0], w.shape[1], x.shape[0], s, d, p, u)

    def mcorr1d(self, x, w, bias=None, s=1, d=1, p=0, u=1, r=0):
        nh = self.mcorr_valid_size(w.shape[2], x.shape[2], s, d, p, u) + r
        h = self._init_out((x.shape[0], w.shape[0], nh), w.dtype, bias)
        return self.op1d("corr", w, x, h, w.shape[0], w.shape[1], x.shape[0], s, d, p, u)

    def mconv1d(self, x, w, bias=None, s=1, d=1, p=0, u=1, r=0):
        nh = self.mconv_valid_size(w.shape[2], x.shape[2], s, d, p, u) + r
        h = self._init_out((x.shape[0], w.shape[0], nh), w.dtype, bias)
        return self.op1d("conv", w, x, h, w.shape[0], w.shape[1], x.shape[0], s, d, p, u)

    def mcorrlcorr_backward(self, x, w, grad_out, s=1, d=1, p=0, u=1):
        """(grad_x, grad_w, grad_b) by the reference's recipe (ext/torch.cpp:261-308):
        grad-input is a *convolution* of the transposed weight with grad_out
        playing the kernel, (s,d,p,u) <- (u,s,p,d); grad-weight is a correlation
        of the transposed input with the transposed grad_out playing the kernel,
        (s,d,p,u) <- (d,s,p,u).  The transposes are expressed with the L0
        transposition flags, as the reference does (ext/torch.cpp:40-53)."""
        s, d, p, u = map(_pair, (s, d, p, u))
        n, ci = x.shape[:2]
        co = w.shape[0]
        gi = np.zeros_like(x)
        # operands: "g" = w viewed (c_in, c_out, ...) i.e. batch'=c_in, c_in'=c_out with
        # transposed_g set; "f" = grad_out (c_out'=batch, c_in'=c_out); output transposed.
        self.op2d("conv", grad_out, w, gi, n, co, ci, u, s, p, d, tf=False, tg=True, th=True)
        gw = np.zeros_like(w)
        # operands: "g" = x viewed (c_in, batch, ...): batch'=c_in, c_in'=batch, transposed_g;
        # "f" = grad_out viewed (c_out, batch, ...): c_out'=c_out, c_in'=batch, transposed_f;
        # output (c_in, c_out, ...) transposed back.
        self.op2d("corr", grad_out, x, gw, co, n, ci, d, s, p, u, tf=True, tg=True, th=True)
        gb = grad_out.sum(axis=0).reshape(co, -1).sum(axis=1)
        return gi, gw, gb

    def mcorr1d_backward(self, x, w, grad_out, s=1, d=1, p=0, u=1):
        gi, gw, gb = self.mcorrlcorr_backward(
            x[..., None], w[..., None], grad_out[..., None], (s, 1), (d, 1), (p, 0), (u, 1))
        return gi[..., 0], gw[..., 0], gb

    def spec2col(self, x, kernel_size, s=1, d=1, p=0, u=1, r=0):
        nf = _pair(kernel_size)
        s, d, p, u, r = map(_pair, (s, d, p, u, r))
        nggx = self.mcorr_valid_size(nf[0], x.shape[2], s[0], d[0], p[0], u[0]) + r[0]
        nggy = self.lcorr_valid_size(nf[1], x.shape[3], s[1], d[1], p[1], u[1]) + r[1]
        gg = np.full(x.shape[:2] + nf + (nggx, nggy), -12345.0, dtype=x.dtype)
        return self.spec2col_raw(x, gg, nf, s, d, p, u)

    def col2spec(self, gg, spec_size, s=1, d=1, p=0, u=1):
        g = np.full(gg.shape[:2] + _pair(spec_size), -12345.0, dtype=gg.dtype)
        return self.col2spec_raw(gg, g, s, d, p, u)

    def snd2col(self, x, kernel_width, s=1, d=1, p=0, u=1, r=0):
        gg = self.spec2col(x[..., None], (kernel_width, 1), (s, 1), (d, 1), (p, 0), (u, 1), (r, 0))
        return gg[:, :, :, 0, :, 0]

    def col2snd(self, gg, snd_width, s=1, d=1, p=0, u=1):
        g = self.col2spec(np.ascontiguousarray(gg[:, :, :, None, :, None]), (snd_width, 1),
                          (s, 1), (d, 1), (p, 0), (u, 1))
        return g[..., 0]
