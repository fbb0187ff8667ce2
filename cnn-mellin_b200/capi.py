"""ctypes view of the C ABI declared in ``include/mellin_b200.h``.

Used by the tests and the benchmark to call the library exactly as a foreign
host would: raw device pointers, extents and a stream handle.  Tensors are
``torch`` CUDA tensors only because torch is how this repository owns device
memory; nothing here touches their contents.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libmellin_b200.so")

_I64 = ctypes.c_int64
_INT = ctypes.c_int
_PTR = ctypes.c_void_p

SIZE_FUNCTIONS = {
    "mellin_mconv_valid_size": 5, "mellin_mconv_support_size": 6, "mellin_mcorr_valid_size": 6,
    "mellin_mcorr_support_size": 5, "mellin_lconv_valid_size": 4, "mellin_lconv_support_size": 6,
    "mellin_lcorr_valid_size": 6, "mellin_lcorr_support_size": 4,
}
OP1D = ["mellin_mconv1d", "mellin_mcorr1d"]
OP2D = ["mellin_mconvlconv", "mellin_mcorrlcorr"]
COL1D = ["mellin_snd2col", "mellin_col2snd"]
COL2D = ["mellin_spec2col", "mellin_col2spec"]
LAYER = ["mellin_mcorrlcorr_forward", "mellin_mcorrlcorr_forward_masked", "mellin_mcorrlcorr_forward_fused",
         "mellin_relu_dropout_backward", "mellin_mcorrlcorr_grad_input",
         "mellin_mcorrlcorr_grad_input_masked",
         "mellin_mcorrlcorr_grad_weight", "mellin_mcorrlcorr_grad_weight_masked"]
MISC = ["mellin_abi_version", "mellin_last_error", "mellin_launch_count", "mellin_clear_tables",
        "mellin_set_tensor_cores", "mellin_set_dependent_launch", "mellin_device_status", "mellin_mcorrlcorr_forward_workspace_bytes",
        "mellin_mcorrlcorr_grad_input_workspace_bytes", "mellin_mcorrlcorr_grad_weight_noalloc_f32",
        "mellin_mcorrlcorr_grad_weight_workspace_bytes", "mellin_index_map_build",
        "mellin_selftest_unarmed_wait", "mellin_selftest_fma_rate",
        "mellin_mcorrlcorr_forward_f16", "mellin_mcorrlcorr_grad_input_f16", "mellin_mcorrlcorr_grad_weight_f16",
        "mellin_mcorrlcorr_forward_workspace_bytes_f16", "mellin_mcorrlcorr_grad_input_workspace_bytes_f16",
        "mellin_mcorrlcorr_grad_weight_workspace_bytes_f16", "mellin_lift_compress_workspace_bytes"]
PROLOGUE = ["mellin_lift_compress", "mellin_lift_compress_backward"]


def exported_symbols():
    """Every symbol the header declares."""
    names = list(SIZE_FUNCTIONS) + MISC
    for base in OP1D + OP2D + COL1D + COL2D + LAYER + PROLOGUE:
        names += [base + "_f32", base + "_f64"]
    return names


class MellinError(RuntimeError):
    def __init__(self, code, message):
        super().__init__("mellin_b200 error %d: %s" % (code, message))
        self.code = code


_lib = None


def lib():
    """Load the shared library; fails loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.isfile(LIB_PATH):
            raise FileNotFoundError(
                "%s is missing: run `python cnn-mellin_b200/build.py` (there is no CPU fallback)" % LIB_PATH)
        _lib = ctypes.CDLL(LIB_PATH)
        for name, nargs in SIZE_FUNCTIONS.items():
            fn = getattr(_lib, name)
            fn.restype, fn.argtypes = _I64, [_I64] * nargs
        _lib.mellin_last_error.restype = ctypes.c_char_p
        _lib.mellin_launch_count.restype = _I64
        for name in ("grad_weight", "forward", "grad_input"):
            for sfx in ("", "_f16"):
                fn = getattr(_lib, "mellin_mcorrlcorr_%s_workspace_bytes%s" % (name, sfx))
                fn.restype, fn.argtypes = ctypes.c_size_t, [_I64] * 17
        _lib.mellin_lift_compress_workspace_bytes.restype = ctypes.c_size_t
    return _lib


def _check(code):
    if code != 0:
        raise MellinError(code, lib().mellin_last_error().decode())


def _sfx(t):
    import torch

    if t.dtype == torch.float32:
        return "_f32"
    if t.dtype == torch.float64:
        return "_f64"
    raise TypeError("unsupported dtype %s" % t.dtype)


def _p(t):
    return _PTR(0 if t is None else t.data_ptr())


def _stream():
    import torch

    return _PTR(torch.cuda.current_stream().cuda_stream)


def _pair(v):
    return (int(v), int(v)) if isinstance(v, int) else (int(v[0]), int(v[1]))


def index_map(relation, order, nf, ng, nh, s, d, p, u):
    """Host-side index map as (row_ptr, entries) numpy arrays; needs no GPU."""
    import numpy as np

    fn = lib().mellin_index_map_build
    fn.restype = _I64
    rel = {"corr": 0, "conv": 1}[relation]
    srt = {"h": 0, "g": 1, "f": 2}[order]
    args = [_INT(rel), _INT(srt)] + [_I64(v) for v in (nf, ng, nh, s, d, p, u)]
    count = fn(*args, _PTR(0), _PTR(0), _I64(0))
    if count < 0:
        raise MellinError(1, lib().mellin_last_error().decode())
    rows = {0: nh, 1: ng, 2: nf}[srt]
    row_ptr = np.zeros(rows + 1, dtype=np.int32)
    entries = np.zeros((max(count, 1), 2), dtype=np.int32)
    fn(*args, row_ptr.ctypes.data_as(_PTR), entries.ctypes.data_as(_PTR), _I64(count))
    return row_ptr, entries[:count]


def launch_count():
    return int(lib().mellin_launch_count())


def op2d(name, f, g, h, c_out, c_in, batch, s, d, p, u, tf=False, tg=False, th=False):
    """``name`` in {"mcorrlcorr", "mconvlconv"}: accumulate into ``h``."""
    (sx, sy), (dx, dy), (px, py), (ux, uy) = map(_pair, (s, d, p, u))
    fn = getattr(lib(), "mellin_%s%s" % (name, _sfx(h)))
    _check(fn(_p(f), _p(g), _I64(c_out), _I64(c_in), _I64(batch), _I64(f.shape[2]), _I64(f.shape[3]),
              _I64(g.shape[2]), _I64(g.shape[3]), _I64(h.shape[2]), _I64(h.shape[3]), _I64(sx), _I64(sy),
              _I64(dx), _I64(dy), _I64(px), _I64(py), _I64(ux), _I64(uy), _INT(tf), _INT(tg), _INT(th),
              _p(h), _stream()))
    return h


def op1d(name, f, g, h, c_out, c_in, batch, s, d, p, u, tf=False, tg=False, th=False):
    """``name`` in {"mcorr1d", "mconv1d"}: accumulate into ``h``."""
    fn = getattr(lib(), "mellin_%s%s" % (name, _sfx(h)))
    _check(fn(_p(f), _p(g), _I64(c_out), _I64(c_in), _I64(batch), _I64(f.shape[2]), _I64(g.shape[2]),
              _I64(h.shape[2]), _I64(s), _I64(d), _I64(p), _I64(u), _INT(tf), _INT(tg), _INT(th), _p(h),
              _stream()))
    return h


def col2d(name, src, dst, c_in, batch, nf, ng, ngg, s, d, p, u, tg=False, tgg=False):
    """``name`` in {"spec2col", "col2spec"}."""
    (sx, sy), (dx, dy), (px, py), (ux, uy) = map(_pair, (s, d, p, u))
    fn = getattr(lib(), "mellin_%s%s" % (name, _sfx(dst)))
    _check(fn(_p(src), _I64(c_in), _I64(batch), _I64(nf[0]), _I64(nf[1]), _I64(ng[0]), _I64(ng[1]),
              _I64(ngg[0]), _I64(ngg[1]), _I64(sx), _I64(sy), _I64(dx), _I64(dy), _I64(px), _I64(py),
              _I64(ux), _I64(uy), _INT(tg), _INT(tgg), _p(dst), _stream()))
    return dst


def col1d(name, src, dst, c_in, batch, nf, ng, ngg, s, d, p, u, tg=False, tgg=False):
    """``name`` in {"snd2col", "col2snd"}."""
    fn = getattr(lib(), "mellin_%s%s" % (name, _sfx(dst)))
    _check(fn(_p(src), _I64(c_in), _I64(batch), _I64(nf), _I64(ng), _I64(ngg), _I64(s), _I64(d), _I64(p),
              _I64(u), _INT(tg), _INT(tgg), _p(dst), _stream()))
    return dst


def _geometry(x_shape, w_shape, y_shape, s, d, p, u):
    (sx, sy), (dx, dy), (px, py), (ux, uy) = map(_pair, (s, d, p, u))
    batch, c_in, ngx, ngy = x_shape
    c_out, _, nfx, nfy = w_shape
    nhx, nhy = y_shape[2:]
    return [_I64(v) for v in (batch, c_in, c_out, nfx, nfy, ngx, ngy, nhx, nhy, sx, sy, dx, dy, px, py, ux, uy)]


def set_dependent_launch(enable):
    """Switch the programmatic dependent launches of the first-layer operators on/off process-wide; returns the previous setting."""
    return int(lib().mellin_set_dependent_launch(_INT(1 if enable else 0)))


def set_tensor_cores(enable):
    """Switch the tcgen05 kernels on/off process-wide; returns the previous setting."""
    return int(lib().mellin_set_tensor_cores(_INT(1 if enable else 0)))


def selftest_unarmed_wait():
    """Launch the bounded-wait self-test: device_status() must report 202 afterwards."""
    _check(lib().mellin_selftest_unarmed_wait(_stream()))


def fma_rate(out, blocks, iters):
    """Launch the FMA-bound micro-kernel; returns the multiply-adds it performs (time it with events)."""
    fn = lib().mellin_selftest_fma_rate
    fn.restype = _I64
    n = fn(_p(out), _I64(blocks), _I64(iters), _stream())
    if n < 0:
        raise MellinError(1, lib().mellin_last_error().decode())
    return int(n)


def device_status():
    """Synchronise and return the kernels' timeout code (0 = healthy)."""
    code = _INT(0)
    _check(lib().mellin_device_status(ctypes.byref(code)))
    return code.value


def forward_workspace_bytes(x_shape, w_shape, y_shape, s, d, p, u):
    return int(lib().mellin_mcorrlcorr_forward_workspace_bytes(*_geometry(x_shape, w_shape, y_shape, s, d, p, u)))


def grad_input_workspace_bytes(x_shape, w_shape, y_shape, s, d, p, u):
    return int(lib().mellin_mcorrlcorr_grad_input_workspace_bytes(*_geometry(x_shape, w_shape, y_shape, s, d, p, u)))


def _scratch(need, like, workspace):
    import torch

    if workspace is None and need:
        workspace = torch.empty(need, dtype=torch.uint8, device=like.device)
    nbytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    return workspace, nbytes


def forward(x, w, bias, y, s, d, p, u, workspace=None):
    """y = bias + mcorrlcorr(x, w); 4-D tensors (use a singleton last axis for 1-D)."""
    import torch

    geom = _geometry(x.shape, w.shape, y.shape, s, d, p, u)
    need = int(lib().mellin_mcorrlcorr_forward_workspace_bytes(*geom)) if y.dtype == torch.float32 else 0
    workspace, nbytes = _scratch(need, y, workspace)
    fn = getattr(lib(), "mellin_mcorrlcorr_forward" + _sfx(y))
    _check(fn(_p(x), _p(w), _p(bias), *geom, _p(y), _p(workspace), ctypes.c_size_t(nbytes), _stream()))
    return y


def forward_masked(x, w, bias, lens, relu, y, s, d, p, u, workspace=None):
    """y = (position < lens[n]) * act(bias + mcorrlcorr(x, w)); lens: int32 device tensor or None."""
    import torch

    geom = _geometry(x.shape, w.shape, y.shape, s, d, p, u)
    need = int(lib().mellin_mcorrlcorr_forward_workspace_bytes(*geom)) if y.dtype == torch.float32 else 0
    workspace, nbytes = _scratch(need, y, workspace)
    fn = getattr(lib(), "mellin_mcorrlcorr_forward_masked" + _sfx(y))
    _check(fn(_p(x), _p(w), _p(bias), _p(lens), _INT(1 if relu else 0), *geom, _p(y), _p(workspace),
              ctypes.c_size_t(nbytes), _stream()))
    return y


def forward_fused(x, w, bias, lens, relu, dropout_p, seed, y, s, d, p, u, workspace=None):
    """y = dropout(mask * act(bias + mcorrlcorr(x, w))) with the mask a function of (seed, position)."""
    import torch

    geom = _geometry(x.shape, w.shape, y.shape, s, d, p, u)
    need = int(lib().mellin_mcorrlcorr_forward_workspace_bytes(*geom)) if y.dtype == torch.float32 else 0
    workspace, nbytes = _scratch(need, y, workspace)
    fn = getattr(lib(), "mellin_mcorrlcorr_forward_fused" + _sfx(y))
    _check(fn(_p(x), _p(w), _p(bias), _p(lens), _INT(1 if relu else 0), ctypes.c_double(dropout_p),
              ctypes.c_uint32(seed & 0xFFFFFFFF), *geom, _p(y), _p(workspace), ctypes.c_size_t(nbytes), _stream()))
    return y


def relu_dropout_backward(grad_y, y, scale, grad_pre):
    """grad_pre = y > 0 ? grad_y * scale : 0 (one pass)."""
    fn = getattr(lib(), "mellin_relu_dropout_backward" + _sfx(y))
    _check(fn(_p(grad_y), _p(y), ctypes.c_double(scale), _p(grad_pre), _I64(y.numel()), _stream()))
    return grad_pre


def lift_compress_workspace_bytes():
    return int(lib().mellin_lift_compress_workspace_bytes())


def lift_compress(x, tau, eps, log_domain, outer, length, inner, y):
    """y = (t + 1)^tau * log(eps + |x|) on x viewed as [outer][length][inner]; tau / eps: device scalars or None."""
    fn = getattr(lib(), "mellin_lift_compress" + _sfx(x))
    _check(fn(_p(x), _p(tau), _p(eps), _INT(1 if log_domain else 0), _I64(outer), _I64(length), _I64(inner), _p(y),
              _stream()))
    return y


def lift_compress_backward(x, grad_y, tau, eps, log_domain, outer, length, inner, grad_x, grad_tau, grad_eps,
                           workspace=None):
    import torch

    need = lift_compress_workspace_bytes()
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    fn = getattr(lib(), "mellin_lift_compress_backward" + _sfx(x))
    _check(fn(_p(x), _p(grad_y), _p(tau), _p(eps), _INT(1 if log_domain else 0), _I64(outer), _I64(length), _I64(inner),
              _p(grad_x), _p(grad_tau), _p(grad_eps), _p(workspace), ctypes.c_size_t(workspace.numel()), _stream()))
    return grad_x


def grad_input(w, grad_y, grad_x, s, d, p, u, workspace=None):
    import torch

    geom = _geometry(grad_x.shape, w.shape, grad_y.shape, s, d, p, u)
    need = int(lib().mellin_mcorrlcorr_grad_input_workspace_bytes(*geom)) if grad_x.dtype == torch.float32 else 0
    workspace, nbytes = _scratch(need, grad_x, workspace)
    fn = getattr(lib(), "mellin_mcorrlcorr_grad_input" + _sfx(grad_x))
    _check(fn(_p(w), _p(grad_y), *geom, _p(grad_x), _p(workspace), ctypes.c_size_t(nbytes), _stream()))
    return grad_x


def grad_input_masked(w, grad_y, lens, grad_x, s, d, p, u, workspace=None):
    """grad_input for a grad_y that is zero from position lens[n] on."""
    import torch

    geom = _geometry(grad_x.shape, w.shape, grad_y.shape, s, d, p, u)
    need = int(lib().mellin_mcorrlcorr_grad_input_workspace_bytes(*geom)) if grad_x.dtype == torch.float32 else 0
    workspace, nbytes = _scratch(need, grad_x, workspace)
    fn = getattr(lib(), "mellin_mcorrlcorr_grad_input_masked" + _sfx(grad_x))
    _check(fn(_p(w), _p(grad_y), _p(lens), *geom, _p(grad_x), _p(workspace), ctypes.c_size_t(nbytes), _stream()))
    return grad_x


def _half_workspace(name, geom, like):
    import torch

    need = int(getattr(lib(), "mellin_mcorrlcorr_%s_workspace_bytes_f16" % name)(*geom))
    return torch.empty(need + 256, dtype=torch.uint8, device=like.device), need


def forward_f16(x, w, bias, y, s, d, p, u):
    """float16 tensors in and out, float32 accumulation; the tensor cores run one MMA per product."""
    geom = _geometry(x.shape, w.shape, y.shape, s, d, p, u)
    ws, need = _half_workspace("forward", geom, y)
    _check(lib().mellin_mcorrlcorr_forward_f16(_p(x), _p(w), _p(bias), *geom, _p(y), _p(ws), ctypes.c_size_t(need), _stream()))
    return y


def grad_input_f16(w, grad_y, grad_x, s, d, p, u):
    geom = _geometry(grad_x.shape, w.shape, grad_y.shape, s, d, p, u)
    ws, need = _half_workspace("grad_input", geom, grad_x)
    _check(lib().mellin_mcorrlcorr_grad_input_f16(_p(w), _p(grad_y), *geom, _p(grad_x), _p(ws), ctypes.c_size_t(need), _stream()))
    return grad_x


def grad_weight_f16(x, grad_y, grad_w, grad_b, s, d, p, u):
    geom = _geometry(x.shape, grad_w.shape, grad_y.shape, s, d, p, u)
    ws, need = _half_workspace("grad_weight", geom, x)
    _check(lib().mellin_mcorrlcorr_grad_weight_f16(_p(x), _p(grad_y), *geom, _p(grad_w), _p(grad_b), _p(ws),
                                                   ctypes.c_size_t(need), _stream()))
    return grad_w, grad_b


def grad_weight_noalloc(x, grad_y, grad_w, grad_b, s, d, p, u):
    """grad_weight through the entry point that owns its scratch (float32 only)."""
    geom = _geometry(x.shape, grad_w.shape, grad_y.shape, s, d, p, u)
    fn = lib().mellin_mcorrlcorr_grad_weight_noalloc_f32
    _check(fn(_p(x), _p(grad_y), *geom, _p(grad_w), _p(grad_b), _stream()))
    return grad_w, grad_b


def grad_weight_workspace_bytes(x_shape, w_shape, y_shape, s, d, p, u):
    return int(lib().mellin_mcorrlcorr_grad_weight_workspace_bytes(*_geometry(x_shape, w_shape, y_shape, s, d, p, u)))


def grad_weight(x, grad_y, grad_w, grad_b, s, d, p, u, workspace=None, lens=None):
    """lens: int32 device tensor promising grad_y is zero from position lens[n] on (masked entry point)."""
    import torch

    geom = _geometry(x.shape, grad_w.shape, grad_y.shape, s, d, p, u)
    need = int(lib().mellin_mcorrlcorr_grad_weight_workspace_bytes(*geom)) if x.dtype == torch.float32 else 0
    if workspace is None and need:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    nbytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    if lens is not None:
        fn = getattr(lib(), "mellin_mcorrlcorr_grad_weight_masked" + _sfx(grad_w))
        _check(fn(_p(x), _p(grad_y), _p(lens), *geom, _p(grad_w), _p(grad_b), _p(workspace), ctypes.c_size_t(nbytes),
                  _stream()))
        return grad_w, grad_b
    fn = getattr(lib(), "mellin_mcorrlcorr_grad_weight" + _sfx(grad_w))
    _check(fn(_p(x), _p(grad_y), *geom, _p(grad_w), _p(grad_b), _p(workspace), ctypes.c_size_t(nbytes), _stream()))
    return grad_w, grad_b
