// Torch binding: registers the `mellin::` operator schemas of the reference
// (ext/torch.cpp:467-476) and implements them for CUDA tensors on top of the
// C ABI in include/mellin_b200.h.  It contains no kernels and no arithmetic;
// PyTorch is used for tensor allocation, the current stream and autograd
// bookkeeping only.
//
// Differences from the reference's binding, none of which change results:
//   * forward of mcorr1d / mcorrlcorr writes bias + correlation in one kernel
//     instead of filling the output and accumulating into it
//     (ext/torch.cpp:88-101);
//   * backward calls dedicated grad-input and grad-weight(+bias) kernels
//     instead of re-invoking the forward operators on transposed operands
//     (ext/torch.cpp:211-231, 282-300), and skips gradients autograd does not
//     ask for (the reference always computes all three);
//   * there is no CPU implementation: CPU tensors are rejected by the
//     dispatcher;
//   * float16 tensors (what the Autocast registrations below produce, as the
//     reference's do, ext/torch.cpp:403-450) are widened to float32 around the
//     float32 kernels and the result narrowed again: float16 storage, float32
//     arithmetic and accumulation, like the reference's Half kernels
//     (mconv_cuda.cuh:135-139), at the price of the conversion passes.
#include <ATen/autocast_mode.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/torch.h>

#include <array>
#include <string>
#include <vector>

#include "mellin_b200.h"

namespace {

using torch::Tensor;
using OptTensor = c10::optional<Tensor>;
using Pair = std::array<int64_t, 2>;

void check_status(int code, const char *op) {
  TORCH_CHECK(code == MELLIN_OK, "mellin_b200 error ", code, " in ", op, ": ", mellin_last_error());
}

void *current_stream(const Tensor &t) {
  return static_cast<void *>(at::cuda::getCurrentCUDAStream(t.device().index()).stream());
}

// ---- argument checking (messages follow torch::checkDim / checkSize, which
// the reference uses: ext/torch.cpp:20-39) -----------------------------------

void check_dim(const char *c, const Tensor &t, const char *name, int pos, int64_t dim) {
  TORCH_CHECK(t.dim() == dim, "Expected ", dim, "-dimensional tensor, but got ", t.dim(),
              "-dimensional tensor for argument #", pos, " '", name, "' (while checking arguments for ", c, ")");
}

void check_size(const char *c, const Tensor &t, const char *name, int pos, int64_t dim, int64_t size) {
  TORCH_CHECK(t.size(dim) == size, "Expected tensor to have size ", size, " at dimension ", dim,
              ", but got size ", t.size(dim), " for argument #", pos, " '", name,
              "' (while checking arguments for ", c, ")");
}

void check_cuda_float(const char *c, const Tensor &t, const char *name) {
  TORCH_CHECK(t.is_cuda(), c, ": '", name, "' must be a CUDA tensor (this build has no CPU path)");
  TORCH_CHECK(t.scalar_type() == at::kFloat || t.scalar_type() == at::kDouble || t.scalar_type() == at::kHalf, c,
              ": '", name, "' must be float16, float32 or float64, got ", t.scalar_type());
}

Pair pair_of(at::IntArrayRef v, const char *c, const char *name) {
  TORCH_CHECK(v.size() == 2, c, ": expected 2 integers for '", name, "'");
  return {v[0], v[1]};
}

// A tensor handed to the C ABI: dense, possibly with its two leading extents
// swapped in memory (the reference detects the same case to avoid a copy,
// ext/torch.cpp:40-53).
struct Operand {
  Tensor dense;     // contiguous storage
  bool transposed;  // storage order is (dim1, dim0, ...)
};

Operand as_operand(const Tensor &t) {
  if (t.is_contiguous()) return {t, false};
  if (t.dim() >= 2 && t.transpose(0, 1).is_contiguous()) return {t.transpose(0, 1), true};
  return {t.contiguous(), false};
}

struct ConvArgs {
  Operand f, g;
  int64_t c_out, c_in, batch, nfx, nfy, ngx, ngy;
};

ConvArgs check_conv(const char *c, int64_t dim, const Tensor &input, const Tensor &weight, const OptTensor &bias) {
  check_cuda_float(c, input, "input");
  check_cuda_float(c, weight, "weight");
  check_dim(c, weight, "weight", 2, dim);
  check_dim(c, input, "input", 1, dim);
  TORCH_CHECK(input.scalar_type() == weight.scalar_type(), c, ": input and weight must have the same dtype");
  TORCH_CHECK(input.device() == weight.device(), c, ": input and weight must be on the same device");
  ConvArgs a;
  a.c_out = weight.size(0), a.c_in = weight.size(1), a.batch = input.size(0);
  a.nfx = weight.size(2), a.ngx = input.size(2);
  a.nfy = dim == 4 ? weight.size(3) : 1;
  a.ngy = dim == 4 ? input.size(3) : 1;
  check_size(c, input, "input", 1, 1, a.c_in);
  if (bias) {
    check_cuda_float(c, *bias, "bias");
    check_dim(c, *bias, "bias", 3, 1);
    check_size(c, *bias, "bias", 3, 0, a.c_out);
    TORCH_CHECK(bias->scalar_type() == weight.scalar_type(), c, ": bias and weight must have the same dtype");
  }
  a.f = as_operand(weight);
  a.g = as_operand(input);
  return a;
}

// output pre-filled with the bias (or zero) for the accumulate-into-h entry
// points, as ext/torch.cpp:88-101 does
Tensor build_output(const Tensor &like, const OptTensor &bias, at::IntArrayRef size) {
  Tensor out = at::empty(size, like.options());
  if (bias) {
    std::vector<int64_t> view(size.size(), 1);
    view[1] = size[1];
    out.copy_(bias->view(view).expand(size));
  } else {
    out.zero_();
  }
  return out;
}

struct LayerGeometry {
  int64_t batch, c_in, c_out, nfx, nfy, ngx, ngy, nhx, nhy;
  Pair s, d, p, u;
};

#define LAYER_ARGS(q)                                                                                       \
  (q).batch, (q).c_in, (q).c_out, (q).nfx, (q).nfy, (q).ngx, (q).ngy, (q).nhx, (q).nhy, (q).s[0], (q).s[1],  \
      (q).d[0], (q).d[1], (q).p[0], (q).p[1], (q).u[0], (q).u[1]

// ---- the four correlation / convolution operators ------------------------------

enum class Op { Corr, Conv };

Tensor conv_like(const char *c, Op op, int64_t dim, const Tensor &input, const Tensor &weight, const OptTensor &bias,
                 Pair s, Pair d, Pair p, Pair u, Pair r, const Tensor *lens = nullptr, bool relu = false,
                 double dropout_p = 0.0, int64_t seed = 0) {
  c10::cuda::CUDAGuard guard(weight.device());
  if (weight.scalar_type() == at::kHalf && input.scalar_type() == at::kHalf &&
      (!bias || bias->scalar_type() == at::kHalf)) {
    if (op == Op::Corr && lens == nullptr && input.is_contiguous() && weight.is_contiguous()) {
      // the float16 entry point: widened in the library's scratch, one MMA per product on the tensor cores
      ConvArgs a = check_conv(c, dim, input, weight, bias);
      const int64_t nhx = mellin_mcorr_valid_size(a.nfx, a.ngx, s[0], d[0], p[0], u[0]) + r[0];
      const int64_t nhy = dim == 4 ? mellin_lcorr_valid_size(a.nfy, a.ngy, s[1], d[1], p[1], u[1]) + r[1] : 1;
      TORCH_CHECK(nhx >= 0 && nhy >= 0, c, ": r makes the output size negative");
      std::vector<int64_t> size = {a.batch, a.c_out, nhx};
      if (dim == 4) size.push_back(nhy);
      Tensor out = at::empty(size, weight.options());
      if (out.numel() == 0) return out;
      LayerGeometry q{a.batch, a.c_in, a.c_out, a.nfx, a.nfy, a.ngx, a.ngy, nhx, nhy, s, d, p, u};
      const size_t bytes = mellin_mcorrlcorr_forward_workspace_bytes_f16(LAYER_ARGS(q));
      Tensor ws = at::empty({static_cast<int64_t>(bytes)}, weight.options().dtype(at::kByte));
      Tensor b = bias ? bias->contiguous() : Tensor();
      check_status(mellin_mcorrlcorr_forward_f16(input.data_ptr(), weight.data_ptr(), bias ? b.data_ptr() : nullptr,
                                                 LAYER_ARGS(q), out.data_ptr(), ws.data_ptr(), bytes,
                                                 current_stream(weight)),
                   c);
      return out;
    }
    const OptTensor wide_bias = bias ? OptTensor(bias->to(at::kFloat)) : OptTensor();
    return conv_like(c, op, dim, input.to(at::kFloat), weight.to(at::kFloat), wide_bias, s, d, p, u, r, lens, relu,
                     dropout_p, seed)
        .to(at::kHalf);
  }
  ConvArgs a = check_conv(c, dim, input, weight, bias);
  int64_t nhx, nhy = 1;
  if (op == Op::Corr) {
    nhx = mellin_mcorr_valid_size(a.nfx, a.ngx, s[0], d[0], p[0], u[0]) + r[0];
    if (dim == 4) nhy = mellin_lcorr_valid_size(a.nfy, a.ngy, s[1], d[1], p[1], u[1]) + r[1];
  } else {
    nhx = mellin_mconv_valid_size(a.ngx, s[0], d[0], p[0], u[0]) + r[0];
    if (dim == 4) nhy = mellin_lconv_valid_size(a.ngy, s[1], p[1], u[1]) + r[1];
  }
  TORCH_CHECK(nhx >= 0 && nhy >= 0, c, ": r makes the output size negative");
  std::vector<int64_t> size = {a.batch, a.c_out, nhx};
  if (dim == 4) size.push_back(nhy);
  void *stream = current_stream(weight);
  const bool f64 = weight.scalar_type() == at::kDouble;

  if (op == Op::Corr && !a.f.transposed && !a.g.transposed) {
    // layer fast path: bias + correlation written in one pass
    Tensor out = at::empty(size, weight.options());
    LayerGeometry q{a.batch, a.c_in, a.c_out, a.nfx, a.nfy, a.ngx, a.ngy, nhx, nhy, s, d, p, u};
    Tensor b = bias ? bias->contiguous() : Tensor();
    int rc;
    if (lens != nullptr) {
      // fused length mask / ReLU epilogue
      TORCH_CHECK(lens->is_cuda() && lens->scalar_type() == at::kInt && lens->dim() == 1 && lens->size(0) == a.batch &&
                      lens->is_contiguous(),
                  c, ": 'lens' must be a contiguous int32 CUDA tensor with one length per utterance");
      const size_t bytes = f64 ? 0 : mellin_mcorrlcorr_forward_workspace_bytes(LAYER_ARGS(q));
      Tensor ws = at::empty({static_cast<int64_t>(bytes ? bytes : 16)}, weight.options().dtype(at::kByte));
      const uint32_t seed32 = static_cast<uint32_t>(static_cast<uint64_t>(seed) ^ (static_cast<uint64_t>(seed) >> 32));
      rc = f64 ? mellin_mcorrlcorr_forward_fused_f64(a.g.dense.data_ptr<double>(), a.f.dense.data_ptr<double>(),
                                                     bias ? b.data_ptr<double>() : nullptr, lens->data_ptr<int>(),
                                                     relu, dropout_p, seed32, LAYER_ARGS(q), out.data_ptr<double>(),
                                                     nullptr, 0, stream)
               : mellin_mcorrlcorr_forward_fused_f32(a.g.dense.data_ptr<float>(), a.f.dense.data_ptr<float>(),
                                                     bias ? b.data_ptr<float>() : nullptr, lens->data_ptr<int>(),
                                                     relu, dropout_p, seed32, LAYER_ARGS(q), out.data_ptr<float>(),
                                                     ws.data_ptr(), bytes, stream);
    } else if (f64) {
      rc = mellin_mcorrlcorr_forward_f64(a.g.dense.data_ptr<double>(), a.f.dense.data_ptr<double>(),
                                         bias ? b.data_ptr<double>() : nullptr, LAYER_ARGS(q), out.data_ptr<double>(),
                                         nullptr, 0, stream);
    } else {
      const size_t bytes = mellin_mcorrlcorr_forward_workspace_bytes(LAYER_ARGS(q));
      Tensor ws = at::empty({static_cast<int64_t>(bytes ? bytes : 16)}, weight.options().dtype(at::kByte));
      rc = mellin_mcorrlcorr_forward_f32(a.g.dense.data_ptr<float>(), a.f.dense.data_ptr<float>(),
                                         bias ? b.data_ptr<float>() : nullptr, LAYER_ARGS(q), out.data_ptr<float>(),
                                         ws.data_ptr(), bytes, stream);
    }
    check_status(rc, c);
    return out;
  }

  TORCH_CHECK(lens == nullptr, c, ": the masked operator takes contiguous, untransposed operands");
  Tensor out = build_output(weight, bias, size);
  int rc;
#define CALL_OP(fn, T)                                                                                      \
  fn(a.f.dense.data_ptr<T>(), a.g.dense.data_ptr<T>(), a.c_out, a.c_in, a.batch, a.nfx, a.nfy, a.ngx, a.ngy,  \
     nhx, nhy, s[0], s[1], d[0], d[1], p[0], p[1], u[0], u[1], a.f.transposed, a.g.transposed, 0,            \
     out.data_ptr<T>(), stream)
  if (op == Op::Corr)
    rc = f64 ? CALL_OP(mellin_mcorrlcorr_f64, double) : CALL_OP(mellin_mcorrlcorr_f32, float);
  else
    rc = f64 ? CALL_OP(mellin_mconvlconv_f64, double) : CALL_OP(mellin_mconvlconv_f32, float);
#undef CALL_OP
  check_status(rc, c);
  return out;
}

Tensor mcorr1d_cuda(const Tensor &input, const Tensor &weight, const OptTensor &bias, int64_t s, int64_t d,
                    int64_t p, int64_t u, int64_t r) {
  return conv_like("mcorr1d_cuda", Op::Corr, 3, input, weight, bias, {s, 1}, {d, 1}, {p, 0}, {u, 1}, {r, 0});
}
Tensor mconv1d_cuda(const Tensor &input, const Tensor &weight, const OptTensor &bias, int64_t s, int64_t d,
                    int64_t p, int64_t u, int64_t r) {
  return conv_like("mconv1d_cuda", Op::Conv, 3, input, weight, bias, {s, 1}, {d, 1}, {p, 0}, {u, 1}, {r, 0});
}
Tensor mcorrlcorr_cuda(const Tensor &input, const Tensor &weight, const OptTensor &bias, at::IntArrayRef s,
                       at::IntArrayRef d, at::IntArrayRef p, at::IntArrayRef u, at::IntArrayRef r) {
  const char *c = "mcorrlcorr_cuda";
  return conv_like(c, Op::Corr, 4, input, weight, bias, pair_of(s, c, "s"), pair_of(d, c, "d"), pair_of(p, c, "p"),
                   pair_of(u, c, "u"), pair_of(r, c, "r"));
}
Tensor mcorrlcorr_masked_cuda(const Tensor &input, const Tensor &weight, const OptTensor &bias, const Tensor &lens,
                             bool relu, at::IntArrayRef s, at::IntArrayRef d, at::IntArrayRef p, at::IntArrayRef u,
                             at::IntArrayRef r, double dropout_p, int64_t seed) {
  const char *c = "mcorrlcorr_masked_cuda";
  TORCH_CHECK(dropout_p >= 0.0 && dropout_p < 1.0, c, ": dropout_p must be in [0, 1)");
  TORCH_CHECK(dropout_p == 0.0 || relu, c, ": the fused dropout needs relu=True (its backward reads the mask off the output)");
  return conv_like(c, Op::Corr, 4, input.contiguous(), weight.contiguous(), bias, pair_of(s, c, "s"),
                   pair_of(d, c, "d"), pair_of(p, c, "p"), pair_of(u, c, "u"), pair_of(r, c, "r"), &lens, relu,
                   dropout_p, seed);
}

Tensor mconvlconv_cuda(const Tensor &input, const Tensor &weight, const OptTensor &bias, at::IntArrayRef s,
                       at::IntArrayRef d, at::IntArrayRef p, at::IntArrayRef u, at::IntArrayRef r) {
  const char *c = "mconvlconv_cuda";
  return conv_like(c, Op::Conv, 4, input, weight, bias, pair_of(s, c, "s"), pair_of(d, c, "d"), pair_of(p, c, "p"),
                   pair_of(u, c, "u"), pair_of(r, c, "r"));
}

// ---- column operators -----------------------------------------------------------

Tensor gather_cols(const char *c, int64_t dim, const Tensor &input, Pair nf, Pair s, Pair d, Pair p, Pair u, Pair r) {
  c10::cuda::CUDAGuard guard(input.device());
  check_cuda_float(c, input, "input");
  if (input.scalar_type() == at::kHalf)  // a pure gather: exact in any width
    return gather_cols(c, dim, input.to(at::kFloat), nf, s, d, p, u, r).to(at::kHalf);
  check_dim(c, input, "input", 1, dim);
  Operand g = as_operand(input);
  const int64_t batch = input.size(0), c_in = input.size(1), ngx = input.size(2), ngy = dim == 4 ? input.size(3) : 1;
  const int64_t nggx = mellin_mcorr_valid_size(nf[0], ngx, s[0], d[0], p[0], u[0]) + r[0];
  const int64_t nggy = dim == 4 ? mellin_lcorr_valid_size(nf[1], ngy, s[1], d[1], p[1], u[1]) + r[1] : 1;
  TORCH_CHECK(nggx >= 0 && nggy >= 0 && nf[0] >= 0 && nf[1] >= 0, c, ": negative output size");
  std::vector<int64_t> size = dim == 4 ? std::vector<int64_t>{batch, c_in, nf[0], nf[1], nggx, nggy}
                                       : std::vector<int64_t>{batch, c_in, nf[0], nggx};
  Tensor gg = at::empty(size, input.options());
  void *stream = current_stream(input);
  int rc;
  if (input.scalar_type() == at::kDouble)
    rc = mellin_spec2col_f64(g.dense.data_ptr<double>(), c_in, batch, nf[0], nf[1], ngx, ngy, nggx, nggy, s[0], s[1],
                             d[0], d[1], p[0], p[1], u[0], u[1], g.transposed, 0, gg.data_ptr<double>(), stream);
  else
    rc = mellin_spec2col_f32(g.dense.data_ptr<float>(), c_in, batch, nf[0], nf[1], ngx, ngy, nggx, nggy, s[0], s[1],
                             d[0], d[1], p[0], p[1], u[0], u[1], g.transposed, 0, gg.data_ptr<float>(), stream);
  check_status(rc, c);
  return gg;
}

Tensor scatter_cols(const char *c, int64_t dim, const Tensor &input, Pair ng, Pair s, Pair d, Pair p, Pair u) {
  c10::cuda::CUDAGuard guard(input.device());
  check_cuda_float(c, input, "input");
  if (input.scalar_type() == at::kHalf)
    return scatter_cols(c, dim, input.to(at::kFloat), ng, s, d, p, u).to(at::kHalf);
  check_dim(c, input, "input", 1, dim);
  Operand gg = as_operand(input);
  const int64_t batch = input.size(0), c_in = input.size(1), nfx = input.size(2);
  const int64_t nfy = dim == 6 ? input.size(3) : 1;
  const int64_t nggx = dim == 6 ? input.size(4) : input.size(3);
  const int64_t nggy = dim == 6 ? input.size(5) : 1;
  TORCH_CHECK(ng[0] >= 0 && ng[1] >= 0, c, ": negative output size");
  std::vector<int64_t> size = dim == 6 ? std::vector<int64_t>{batch, c_in, ng[0], ng[1]}
                                       : std::vector<int64_t>{batch, c_in, ng[0]};
  Tensor g = at::empty(size, input.options());
  void *stream = current_stream(input);
  int rc;
  if (input.scalar_type() == at::kDouble)
    rc = mellin_col2spec_f64(gg.dense.data_ptr<double>(), c_in, batch, nfx, nfy, ng[0], ng[1], nggx, nggy, s[0], s[1],
                             d[0], d[1], p[0], p[1], u[0], u[1], 0, gg.transposed, g.data_ptr<double>(), stream);
  else
    rc = mellin_col2spec_f32(gg.dense.data_ptr<float>(), c_in, batch, nfx, nfy, ng[0], ng[1], nggx, nggy, s[0], s[1],
                             d[0], d[1], p[0], p[1], u[0], u[1], 0, gg.transposed, g.data_ptr<float>(), stream);
  check_status(rc, c);
  return g;
}

Tensor snd2col_cuda(const Tensor &input, int64_t kernel_width, int64_t s, int64_t d, int64_t p, int64_t u, int64_t r) {
  return gather_cols("snd2col_cuda", 3, input, {kernel_width, 1}, {s, 1}, {d, 1}, {p, 0}, {u, 1}, {r, 0});
}
Tensor col2snd_cuda(const Tensor &input, int64_t snd_width, int64_t s, int64_t d, int64_t p, int64_t u) {
  return scatter_cols("col2snd_cuda", 4, input, {snd_width, 1}, {s, 1}, {d, 1}, {p, 0}, {u, 1});
}
Tensor spec2col_cuda(const Tensor &input, at::IntArrayRef kernel_size, at::IntArrayRef s, at::IntArrayRef d,
                     at::IntArrayRef p, at::IntArrayRef u, at::IntArrayRef r) {
  const char *c = "spec2col_cuda";
  return gather_cols(c, 4, input, pair_of(kernel_size, c, "kernel_size"), pair_of(s, c, "s"), pair_of(d, c, "d"),
                     pair_of(p, c, "p"), pair_of(u, c, "u"), pair_of(r, c, "r"));
}
Tensor col2spec_cuda(const Tensor &input, at::IntArrayRef spec_size, at::IntArrayRef s, at::IntArrayRef d,
                     at::IntArrayRef p, at::IntArrayRef u) {
  const char *c = "col2spec_cuda";
  return scatter_cols(c, 6, input, pair_of(spec_size, c, "spec_size"), pair_of(s, c, "s"), pair_of(d, c, "d"),
                      pair_of(p, c, "p"), pair_of(u, c, "u"));
}

// ---- dispatcher trampolines (used from autograd nodes) ----------------------------

template <typename Sig>
auto &typed_op(const char *name) {
  static auto op = c10::Dispatcher::singleton().findSchemaOrThrow(name, "").typed<Sig>();
  return op;
}

Tensor call_mcorr1d(const Tensor &i, const Tensor &w, const OptTensor &b, int64_t s, int64_t d, int64_t p, int64_t u,
                    int64_t r) {
  return typed_op<Tensor(const Tensor &, const Tensor &, const OptTensor &, int64_t, int64_t, int64_t, int64_t,
                         int64_t)>("mellin::mcorr1d")
      .call(i, w, b, s, d, p, u, r);
}
Tensor call_mcorrlcorr(const Tensor &i, const Tensor &w, const OptTensor &b, at::IntArrayRef s, at::IntArrayRef d,
                       at::IntArrayRef p, at::IntArrayRef u, at::IntArrayRef r) {
  return typed_op<Tensor(const Tensor &, const Tensor &, const OptTensor &, at::IntArrayRef, at::IntArrayRef,
                         at::IntArrayRef, at::IntArrayRef, at::IntArrayRef)>("mellin::mcorrlcorr")
      .call(i, w, b, s, d, p, u, r);
}
Tensor call_snd2col(const Tensor &i, int64_t k, int64_t s, int64_t d, int64_t p, int64_t u, int64_t r) {
  return typed_op<Tensor(const Tensor &, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t)>("mellin::snd2col")
      .call(i, k, s, d, p, u, r);
}
Tensor call_col2snd(const Tensor &i, int64_t k, int64_t s, int64_t d, int64_t p, int64_t u) {
  return typed_op<Tensor(const Tensor &, int64_t, int64_t, int64_t, int64_t, int64_t)>("mellin::col2snd")
      .call(i, k, s, d, p, u);
}
Tensor call_spec2col(const Tensor &i, at::IntArrayRef k, at::IntArrayRef s, at::IntArrayRef d, at::IntArrayRef p,
                     at::IntArrayRef u, at::IntArrayRef r) {
  return typed_op<Tensor(const Tensor &, at::IntArrayRef, at::IntArrayRef, at::IntArrayRef, at::IntArrayRef,
                         at::IntArrayRef, at::IntArrayRef)>("mellin::spec2col")
      .call(i, k, s, d, p, u, r);
}
Tensor call_col2spec(const Tensor &i, at::IntArrayRef k, at::IntArrayRef s, at::IntArrayRef d, at::IntArrayRef p,
                     at::IntArrayRef u) {
  return typed_op<Tensor(const Tensor &, at::IntArrayRef, at::IntArrayRef, at::IntArrayRef, at::IntArrayRef,
                         at::IntArrayRef)>("mellin::col2spec")
      .call(i, k, s, d, p, u);
}

// ---- autograd ---------------------------------------------------------------------

// Gradients of a correlation layer through the layer-level C entry points.
// 1-D tensors are viewed with a trailing singleton linear axis.
std::vector<Tensor> layer_backward(const Tensor &grad_out_in, const Tensor &input_in, const Tensor &weight_in,
                                   bool has_bias, Pair s, Pair d, Pair p, Pair u, bool need_input, bool need_weight,
                                   bool need_bias, const Tensor *lens = nullptr) {
  const bool one_d = input_in.dim() == 3;
  c10::cuda::CUDAGuard guard(weight_in.device());
  if (weight_in.scalar_type() == at::kHalf && lens == nullptr && grad_out_in.scalar_type() == at::kHalf &&
      input_in.scalar_type() == at::kHalf && grad_out_in.numel() > 0 && input_in.numel() > 0 && weight_in.numel() > 0) {
    // the float16 entry points (one MMA per product on the tensor cores)
    Tensor go = grad_out_in.contiguous(), x = input_in.contiguous(), w = weight_in.contiguous();
    LayerGeometry q{x.size(0), x.size(1), w.size(0), w.size(2), one_d ? 1 : w.size(3), x.size(2),
                    one_d ? 1 : x.size(3), go.size(2), one_d ? 1 : go.size(3), s, d, p, u};
    void *stream = current_stream(w);
    Tensor gi, gw, gb;
    if (need_input) {
      gi = at::empty_like(x);
      const size_t bytes = mellin_mcorrlcorr_grad_input_workspace_bytes_f16(LAYER_ARGS(q));
      Tensor ws = at::empty({static_cast<int64_t>(bytes)}, w.options().dtype(at::kByte));
      check_status(mellin_mcorrlcorr_grad_input_f16(w.data_ptr(), go.data_ptr(), LAYER_ARGS(q), gi.data_ptr(), ws.data_ptr(),
                                                    bytes, stream),
                   "mcorrlcorr_grad_input");
    }
    if (need_weight || (need_bias && has_bias)) {
      gw = at::empty_like(w);
      if (need_bias && has_bias) gb = at::empty({w.size(0)}, w.options());
      const size_t bytes = mellin_mcorrlcorr_grad_weight_workspace_bytes_f16(LAYER_ARGS(q));
      Tensor ws = at::empty({static_cast<int64_t>(bytes)}, w.options().dtype(at::kByte));
      check_status(mellin_mcorrlcorr_grad_weight_f16(x.data_ptr(), go.data_ptr(), LAYER_ARGS(q), gw.data_ptr(),
                                                     gb.defined() ? gb.data_ptr() : nullptr, ws.data_ptr(), bytes, stream),
                   "mcorrlcorr_grad_weight");
      if (!need_weight) gw = Tensor();
    }
    return {gi, gw, gb};
  }
  if (weight_in.scalar_type() == at::kHalf) {
    std::vector<Tensor> wide = layer_backward(grad_out_in.to(at::kFloat), input_in.to(at::kFloat),
                                              weight_in.to(at::kFloat), has_bias, s, d, p, u, need_input, need_weight,
                                              need_bias, lens);
    for (Tensor &t : wide)
      if (t.defined()) t = t.to(at::kHalf);
    return wide;
  }
  Tensor go = grad_out_in.contiguous(), x = input_in.contiguous(), w = weight_in.contiguous();
  LayerGeometry q{x.size(0), x.size(1), w.size(0), w.size(2), one_d ? 1 : w.size(3), x.size(2),
                  one_d ? 1 : x.size(3), go.size(2), one_d ? 1 : go.size(3), s, d, p, u};
  void *stream = current_stream(w);
  const bool f64 = w.scalar_type() == at::kDouble;
  Tensor gi, gw, gb;
  if (need_input) {
    gi = at::empty_like(x);
    const size_t gi_bytes = f64 ? 0 : mellin_mcorrlcorr_grad_input_workspace_bytes(LAYER_ARGS(q));
    Tensor gi_ws = at::empty({static_cast<int64_t>(gi_bytes ? gi_bytes : 16)}, w.options().dtype(at::kByte));
    int rc;
    if (lens != nullptr && !one_d) {
      // grad_out is zero past every utterance's length: tiles that can only hold zeros are skipped
      rc = f64 ? mellin_mcorrlcorr_grad_input_masked_f64(w.data_ptr<double>(), go.data_ptr<double>(),
                                                         lens->data_ptr<int>(), LAYER_ARGS(q), gi.data_ptr<double>(),
                                                         nullptr, 0, stream)
               : mellin_mcorrlcorr_grad_input_masked_f32(w.data_ptr<float>(), go.data_ptr<float>(),
                                                         lens->data_ptr<int>(), LAYER_ARGS(q), gi.data_ptr<float>(),
                                                         gi_ws.data_ptr(), gi_bytes, stream);
    } else {
      rc = f64 ? mellin_mcorrlcorr_grad_input_f64(w.data_ptr<double>(), go.data_ptr<double>(), LAYER_ARGS(q),
                                                   gi.data_ptr<double>(), nullptr, 0, stream)
               : mellin_mcorrlcorr_grad_input_f32(w.data_ptr<float>(), go.data_ptr<float>(), LAYER_ARGS(q),
                                                   gi.data_ptr<float>(), gi_ws.data_ptr(), gi_bytes, stream);
    }
    check_status(rc, "mcorrlcorr_grad_input");
  }
  if (need_weight || (need_bias && has_bias)) {
    gw = at::empty_like(w);
    if (need_bias && has_bias) gb = at::empty({w.size(0)}, w.options());
    const size_t bytes = f64 ? 0 : mellin_mcorrlcorr_grad_weight_workspace_bytes(LAYER_ARGS(q));
    Tensor ws;
    if (bytes) ws = at::empty({static_cast<int64_t>(bytes)}, w.options().dtype(at::kByte));
    int rc;
    if (lens != nullptr && !one_d && !f64) {
      // grad_out is zero past every utterance's length: each utterance's reduction stops there
      rc = mellin_mcorrlcorr_grad_weight_masked_f32(x.data_ptr<float>(), go.data_ptr<float>(), lens->data_ptr<int>(),
                                                    LAYER_ARGS(q), gw.data_ptr<float>(),
                                                    gb.defined() ? gb.data_ptr<float>() : nullptr,
                                                    bytes ? ws.data_ptr() : nullptr, bytes, stream);
    } else {
      rc = f64 ? mellin_mcorrlcorr_grad_weight_f64(x.data_ptr<double>(), go.data_ptr<double>(), LAYER_ARGS(q),
                                                        gw.data_ptr<double>(), gb.defined() ? gb.data_ptr<double>() : nullptr,
                                                        nullptr, 0, stream)
                   : mellin_mcorrlcorr_grad_weight_f32(x.data_ptr<float>(), go.data_ptr<float>(), LAYER_ARGS(q),
                                                        gw.data_ptr<float>(), gb.defined() ? gb.data_ptr<float>() : nullptr,
                                                        bytes ? ws.data_ptr() : nullptr, bytes, stream);
    }
    check_status(rc, "mcorrlcorr_grad_weight");
    if (!need_weight) gw = Tensor();
  }
  return {gi, gw, gb};
}

class MCorr1DFunction : public torch::autograd::Function<MCorr1DFunction> {
 public:
  static Tensor forward(torch::autograd::AutogradContext *ctx, const Tensor &input, const Tensor &weight,
                        const OptTensor &bias, int64_t s, int64_t d, int64_t p, int64_t u, int64_t r) {
    ctx->save_for_backward({input, weight});
    ctx->saved_data["has_bias"] = bias.has_value();
    ctx->saved_data["sdpu"] = std::vector<int64_t>{s, d, p, u};
    at::AutoDispatchBelowADInplaceOrView guard;
    return call_mcorr1d(input, weight, bias, s, d, p, u, r);
  }
  static torch::autograd::tensor_list backward(torch::autograd::AutogradContext *ctx,
                                               torch::autograd::tensor_list grads) {
    auto saved = ctx->get_saved_variables();
    auto v = ctx->saved_data["sdpu"].toIntVector();
    // gradient edges exist for tensor arguments only; an absent bias has none
    const bool has_bias = ctx->saved_data["has_bias"].toBool();
    auto out = layer_backward(grads[0], saved[0], saved[1], has_bias, {v[0], 1}, {v[1], 1}, {v[2], 0}, {v[3], 1},
                              ctx->needs_input_grad(0), ctx->needs_input_grad(1),
                              has_bias && ctx->needs_input_grad(2));
    return {out[0], out[1], out[2], Tensor(), Tensor(), Tensor(), Tensor(), Tensor()};
  }
};

class MCorrLCorrFunction : public torch::autograd::Function<MCorrLCorrFunction> {
 public:
  static Tensor forward(torch::autograd::AutogradContext *ctx, const Tensor &input, const Tensor &weight,
                        const OptTensor &bias, at::IntArrayRef s, at::IntArrayRef d, at::IntArrayRef p,
                        at::IntArrayRef u, at::IntArrayRef r) {
    ctx->save_for_backward({input, weight});
    ctx->saved_data["has_bias"] = bias.has_value();
    ctx->saved_data["s"] = s.vec(), ctx->saved_data["d"] = d.vec();
    ctx->saved_data["p"] = p.vec(), ctx->saved_data["u"] = u.vec();
    at::AutoDispatchBelowADInplaceOrView guard;
    return call_mcorrlcorr(input, weight, bias, s, d, p, u, r);
  }
  static torch::autograd::tensor_list backward(torch::autograd::AutogradContext *ctx,
                                               torch::autograd::tensor_list grads) {
    auto saved = ctx->get_saved_variables();
    const char *c = "mcorrlcorr backward";
    const bool has_bias = ctx->saved_data["has_bias"].toBool();
    auto out = layer_backward(grads[0], saved[0], saved[1], has_bias,
                              pair_of(ctx->saved_data["s"].toIntVector(), c, "s"),
                              pair_of(ctx->saved_data["d"].toIntVector(), c, "d"),
                              pair_of(ctx->saved_data["p"].toIntVector(), c, "p"),
                              pair_of(ctx->saved_data["u"].toIntVector(), c, "u"), ctx->needs_input_grad(0),
                              ctx->needs_input_grad(1), has_bias && ctx->needs_input_grad(2));
    return {out[0], out[1], out[2], Tensor(), Tensor(), Tensor(), Tensor(), Tensor()};
  }
};

Tensor call_mcorrlcorr_masked(const Tensor &i, const Tensor &w, const OptTensor &b, const Tensor &lens, bool relu,
                              at::IntArrayRef s, at::IntArrayRef d, at::IntArrayRef p, at::IntArrayRef u,
                              at::IntArrayRef r, double dropout_p, int64_t seed) {
  return typed_op<Tensor(const Tensor &, const Tensor &, const OptTensor &, const Tensor &, bool, at::IntArrayRef,
                         at::IntArrayRef, at::IntArrayRef, at::IntArrayRef, at::IntArrayRef, double, int64_t)>(
             "mellin::mcorrlcorr_masked")
      .call(i, w, b, lens, relu, s, d, p, u, r, dropout_p, seed);
}

// y = mask * act(layer(x)): dy/dz = mask * act'(z); for ReLU both factors are (y > 0)
class MCorrLCorrMaskedFunction : public torch::autograd::Function<MCorrLCorrMaskedFunction> {
 public:
  static Tensor forward(torch::autograd::AutogradContext *ctx, const Tensor &input, const Tensor &weight,
                        const OptTensor &bias, const Tensor &lens, bool relu, at::IntArrayRef s, at::IntArrayRef d,
                        at::IntArrayRef p, at::IntArrayRef u, at::IntArrayRef r, double dropout_p, int64_t seed) {
    ctx->saved_data["has_bias"] = bias.has_value();
    ctx->saved_data["relu"] = relu;
    ctx->saved_data["dropout_p"] = dropout_p;
    ctx->saved_data["s"] = s.vec(), ctx->saved_data["d"] = d.vec();
    ctx->saved_data["p"] = p.vec(), ctx->saved_data["u"] = u.vec();
    Tensor y;
    {
      at::AutoDispatchBelowADInplaceOrView guard;
      y = call_mcorrlcorr_masked(input, weight, bias, lens, relu, s, d, p, u, r, dropout_p, seed);
    }
    ctx->save_for_backward({input, weight, lens, y});
    return y;
  }
  static torch::autograd::tensor_list backward(torch::autograd::AutogradContext *ctx,
                                               torch::autograd::tensor_list grads) {
    auto saved = ctx->get_saved_variables();
    const char *c = "mcorrlcorr_masked backward";
    const bool has_bias = ctx->saved_data["has_bias"].toBool();
    const Tensor &lens = saved[2], &y = saved[3];
    Tensor go;
    const double dropout_p = ctx->saved_data["dropout_p"].toDouble();
    if (ctx->saved_data["relu"].toBool() && dropout_p > 0.0 && y.scalar_type() != at::kHalf) {
      // relu, mask and dropout in one pass over y: an element is positive exactly where it passed all three
      Tensor g = grads[0].contiguous();
      go = at::empty_like(y);
      c10::cuda::CUDAGuard guard(y.device());
      const int rc = y.scalar_type() == at::kDouble
                         ? mellin_relu_dropout_backward_f64(g.data_ptr<double>(), y.data_ptr<double>(), 1.0 / (1.0 - dropout_p),
                                                            go.data_ptr<double>(), y.numel(), current_stream(y))
                         : mellin_relu_dropout_backward_f32(g.data_ptr<float>(), y.data_ptr<float>(), 1.0 / (1.0 - dropout_p),
                                                            go.data_ptr<float>(), y.numel(), current_stream(y));
      check_status(rc, c);
    } else if (ctx->saved_data["relu"].toBool()) {
      go = at::threshold_backward(grads[0], y, 0);  // grad where y > 0, else 0: one pass
      if (dropout_p > 0.0) go.mul_(1.0 / (1.0 - dropout_p));
    } else {
      Tensor mask = at::arange(y.size(3), lens.options()).unsqueeze(0) < lens.unsqueeze(1);  // (N, positions)
      go = grads[0] * mask.unsqueeze(1).unsqueeze(1);
    }
    auto out = layer_backward(go, saved[0], saved[1], has_bias, pair_of(ctx->saved_data["s"].toIntVector(), c, "s"),
                              pair_of(ctx->saved_data["d"].toIntVector(), c, "d"),
                              pair_of(ctx->saved_data["p"].toIntVector(), c, "p"),
                              pair_of(ctx->saved_data["u"].toIntVector(), c, "u"), ctx->needs_input_grad(0),
                              ctx->needs_input_grad(1), has_bias && ctx->needs_input_grad(2), &lens);
    return {out[0], out[1], out[2], Tensor(), Tensor(), Tensor(), Tensor(), Tensor(), Tensor(), Tensor(), Tensor(), Tensor()};
  }
};

class Snd2ColFunction : public torch::autograd::Function<Snd2ColFunction> {
 public:
  static Tensor forward(torch::autograd::AutogradContext *ctx, const Tensor &input, int64_t kernel_width, int64_t s,
                        int64_t d, int64_t p, int64_t u, int64_t r) {
    ctx->saved_data["args"] = std::vector<int64_t>{input.size(2), s, d, p, u};
    at::AutoDispatchBelowADInplaceOrView guard;
    return call_snd2col(input, kernel_width, s, d, p, u, r);
  }
  static torch::autograd::tensor_list backward(torch::autograd::AutogradContext *ctx,
                                               torch::autograd::tensor_list grads) {
    auto v = ctx->saved_data["args"].toIntVector();
    return {call_col2snd(grads[0], v[0], v[1], v[2], v[3], v[4]), Tensor(), Tensor(), Tensor(), Tensor(), Tensor(),
            Tensor()};
  }
};

class Spec2ColFunction : public torch::autograd::Function<Spec2ColFunction> {
 public:
  static Tensor forward(torch::autograd::AutogradContext *ctx, const Tensor &input, at::IntArrayRef kernel_size,
                        at::IntArrayRef s, at::IntArrayRef d, at::IntArrayRef p, at::IntArrayRef u,
                        at::IntArrayRef r) {
    ctx->saved_data["size"] = std::vector<int64_t>{input.size(2), input.size(3)};
    ctx->saved_data["s"] = s.vec(), ctx->saved_data["d"] = d.vec();
    ctx->saved_data["p"] = p.vec(), ctx->saved_data["u"] = u.vec();
    at::AutoDispatchBelowADInplaceOrView guard;
    return call_spec2col(input, kernel_size, s, d, p, u, r);
  }
  static torch::autograd::tensor_list backward(torch::autograd::AutogradContext *ctx,
                                               torch::autograd::tensor_list grads) {
    return {call_col2spec(grads[0], ctx->saved_data["size"].toIntVector(), ctx->saved_data["s"].toIntVector(),
                          ctx->saved_data["d"].toIntVector(), ctx->saved_data["p"].toIntVector(),
                          ctx->saved_data["u"].toIntVector()),
            Tensor(), Tensor(), Tensor(), Tensor(), Tensor(), Tensor()};
  }
};

Tensor mcorr1d_autograd(const Tensor &input, const Tensor &weight, const OptTensor &bias, int64_t s, int64_t d,
                        int64_t p, int64_t u, int64_t r) {
  return MCorr1DFunction::apply(input, weight, bias, s, d, p, u, r);
}
Tensor mcorrlcorr_autograd(const Tensor &input, const Tensor &weight, const OptTensor &bias, at::IntArrayRef s,
                           at::IntArrayRef d, at::IntArrayRef p, at::IntArrayRef u, at::IntArrayRef r) {
  return MCorrLCorrFunction::apply(input, weight, bias, s, d, p, u, r);
}
Tensor mcorrlcorr_masked_autograd(const Tensor &input, const Tensor &weight, const OptTensor &bias, const Tensor &lens,
                                 bool relu, at::IntArrayRef s, at::IntArrayRef d, at::IntArrayRef p, at::IntArrayRef u,
                                 at::IntArrayRef r, double dropout_p, int64_t seed) {
  return MCorrLCorrMaskedFunction::apply(input, weight, bias, lens, relu, s, d, p, u, r, dropout_p, seed);
}
Tensor snd2col_autograd(const Tensor &input, int64_t kernel_width, int64_t s, int64_t d, int64_t p, int64_t u,
                        int64_t r) {
  return Snd2ColFunction::apply(input, kernel_width, s, d, p, u, r);
}
Tensor spec2col_autograd(const Tensor &input, at::IntArrayRef kernel_size, at::IntArrayRef s, at::IntArrayRef d,
                         at::IntArrayRef p, at::IntArrayRef u, at::IntArrayRef r) {
  return Spec2ColFunction::apply(input, kernel_size, s, d, p, u, r);
}

}  // namespace

// The schemas are the reference's, character for character in meaning
// (ext/torch.cpp:467-476), so that code written against torch.ops.mellin.*
// keeps working.
TORCH_LIBRARY(mellin, m) {
  m.def("mconv1d(Tensor input, Tensor weight, Tensor? bias=None, int s=1, int d=1, int p=0, int u=1, int r=0) -> Tensor");
  m.def("mcorr1d(Tensor input, Tensor weight, Tensor? bias=None, int s=1, int d=1, int p=0, int u=1, int r=0) -> Tensor");
  m.def("mcorrlcorr(Tensor input, Tensor weight, Tensor? bias=None, int[2] s=1, int[2] d=1, int[2] p=0, int[2] u=1, int[2] r=0) -> Tensor");
  m.def("mconvlconv(Tensor input, Tensor weight, Tensor? bias=None, int[2] s=1, int[2] d=1, int[2] p=0, int[2] u=1, int[2] r=0) -> Tensor");
  m.def("snd2col(Tensor input, int kernel_width, int s=1, int d=1, int p=0, int u=1, int r=0) -> Tensor");
  m.def("col2snd(Tensor input, int snd_width, int s=1, int d=1, int p=0, int u=1) -> Tensor");
  m.def("spec2col(Tensor input, int[2] kernel_size, int[2] s=1, int[2] d=1, int[2] p=0, int[2] u=1, int[2] r=0) -> Tensor");
  m.def("col2spec(Tensor input, int[2] spec_size, int[2] s=1, int[2] d=1, int[2] p=0, int[2] u=1) -> Tensor");
  // not in the reference: mcorrlcorr with the length mask and ReLU its models apply around a layer fused in
  m.def("mcorrlcorr_masked(Tensor input, Tensor weight, Tensor? bias, Tensor lens, bool relu=True, int[2] s=1, int[2] d=1, int[2] p=0, int[2] u=1, int[2] r=0, float dropout_p=0.0, int seed=0) -> Tensor");
}

TORCH_LIBRARY_IMPL(mellin, CUDA, m) {
  m.impl("mconv1d", mconv1d_cuda);
  m.impl("mcorr1d", mcorr1d_cuda);
  m.impl("mconvlconv", mconvlconv_cuda);
  m.impl("mcorrlcorr", mcorrlcorr_cuda);
  m.impl("mcorrlcorr_masked", mcorrlcorr_masked_cuda);
  m.impl("snd2col", snd2col_cuda);
  m.impl("col2snd", col2snd_cuda);
  m.impl("spec2col", spec2col_cuda);
  m.impl("col2spec", col2spec_cuda);
}

// Under torch.autocast the operators run in float16, like torch's own
// convolutions: cast the tensor arguments and call the operator again below
// the Autocast key.
Tensor to_half(const Tensor &t) { return at::autocast::cached_cast(at::kHalf, t); }
OptTensor to_half(const OptTensor &t) { return t ? OptTensor(to_half(*t)) : OptTensor(); }

Tensor mcorr1d_autocast(const Tensor &input, const Tensor &weight, const OptTensor &bias, int64_t s, int64_t d,
                        int64_t p, int64_t u, int64_t r) {
  c10::impl::ExcludeDispatchKeyGuard below(c10::DispatchKey::Autocast);
  return call_mcorr1d(to_half(input), to_half(weight), to_half(bias), s, d, p, u, r);
}
Tensor mconv1d_autocast(const Tensor &input, const Tensor &weight, const OptTensor &bias, int64_t s, int64_t d,
                        int64_t p, int64_t u, int64_t r) {
  c10::impl::ExcludeDispatchKeyGuard below(c10::DispatchKey::Autocast);
  return typed_op<Tensor(const Tensor &, const Tensor &, const OptTensor &, int64_t, int64_t, int64_t, int64_t,
                         int64_t)>("mellin::mconv1d")
      .call(to_half(input), to_half(weight), to_half(bias), s, d, p, u, r);
}
Tensor mcorrlcorr_autocast(const Tensor &input, const Tensor &weight, const OptTensor &bias, at::IntArrayRef s,
                           at::IntArrayRef d, at::IntArrayRef p, at::IntArrayRef u, at::IntArrayRef r) {
  c10::impl::ExcludeDispatchKeyGuard below(c10::DispatchKey::Autocast);
  return call_mcorrlcorr(to_half(input), to_half(weight), to_half(bias), s, d, p, u, r);
}
Tensor mconvlconv_autocast(const Tensor &input, const Tensor &weight, const OptTensor &bias, at::IntArrayRef s,
                           at::IntArrayRef d, at::IntArrayRef p, at::IntArrayRef u, at::IntArrayRef r) {
  c10::impl::ExcludeDispatchKeyGuard below(c10::DispatchKey::Autocast);
  return typed_op<Tensor(const Tensor &, const Tensor &, const OptTensor &, at::IntArrayRef, at::IntArrayRef,
                         at::IntArrayRef, at::IntArrayRef, at::IntArrayRef)>("mellin::mconvlconv")
      .call(to_half(input), to_half(weight), to_half(bias), s, d, p, u, r);
}
Tensor snd2col_autocast(const Tensor &input, int64_t kernel_width, int64_t s, int64_t d, int64_t p, int64_t u,
                        int64_t r) {
  c10::impl::ExcludeDispatchKeyGuard below(c10::DispatchKey::Autocast);
  return call_snd2col(to_half(input), kernel_width, s, d, p, u, r);
}
Tensor col2snd_autocast(const Tensor &input, int64_t snd_width, int64_t s, int64_t d, int64_t p, int64_t u) {
  c10::impl::ExcludeDispatchKeyGuard below(c10::DispatchKey::Autocast);
  return call_col2snd(to_half(input), snd_width, s, d, p, u);
}
Tensor spec2col_autocast(const Tensor &input, at::IntArrayRef kernel_size, at::IntArrayRef s, at::IntArrayRef d,
                         at::IntArrayRef p, at::IntArrayRef u, at::IntArrayRef r) {
  c10::impl::ExcludeDispatchKeyGuard below(c10::DispatchKey::Autocast);
  return call_spec2col(to_half(input), kernel_size, s, d, p, u, r);
}
Tensor col2spec_autocast(const Tensor &input, at::IntArrayRef spec_size, at::IntArrayRef s, at::IntArrayRef d,
                         at::IntArrayRef p, at::IntArrayRef u) {
  c10::impl::ExcludeDispatchKeyGuard below(c10::DispatchKey::Autocast);
  return call_col2spec(to_half(input), spec_size, s, d, p, u);
}

TORCH_LIBRARY_IMPL(mellin, Autocast, m) {
  m.impl("mconv1d", mconv1d_autocast);
  m.impl("mcorr1d", mcorr1d_autocast);
  m.impl("mconvlconv", mconvlconv_autocast);
  m.impl("mcorrlcorr", mcorrlcorr_autocast);
  m.impl("snd2col", snd2col_autocast);
  m.impl("col2snd", col2snd_autocast);
  m.impl("spec2col", spec2col_autocast);
  m.impl("col2spec", col2spec_autocast);
}

TORCH_LIBRARY_IMPL(mellin, Autograd, m) {
  m.impl("mcorr1d", mcorr1d_autograd);
  m.impl("mcorrlcorr", mcorrlcorr_autograd);
  m.impl("mcorrlcorr_masked", mcorrlcorr_masked_autograd);
  m.impl("snd2col", snd2col_autograd);
  m.impl("spec2col", spec2col_autograd);
}
