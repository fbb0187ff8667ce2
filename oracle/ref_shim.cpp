// C-ABI window onto the reference's own CPU kernels.
//
// TEST INFRASTRUCTURE.  This file contains no algorithm: it includes the
// reference's header-only library (ext/include/cdrobert/mellin/mconv.h) from
// the reference checkout where it lies (the include path is given on the
// compiler command line by build_oracle.py) and forwards plain-C calls to its
// templates.  The resulting library is written to oracle/_ref/ and is used to
// (1) validate the C restatement in mellin_oracle.c and (2) time the
// reference's CPU implementation as the benchmark's CPU baseline.  It is
// built with -O3 -fopenmp so that the reference's "#pragma omp parallel for"
// loops use all host cores (its CMake build links OpenMP the same way:
// c/cpu/CMakeLists.txt:64-66).
#include <cstdint>
#include <algorithm>
#include "cdrobert/mellin/mconv.h"

namespace cm = cdrobert::mellin;
typedef int64_t i64;

#define CONV1D_ARGS(T) \
  const T *f, const T *g, i64 c_out, i64 c_in, i64 batch, i64 nf, i64 ng, \
  i64 nh, i64 s, i64 d, i64 p, i64 u, int tf, int tg, int th, T *h
#define CONV1D_PASS \
  f, g, c_out, c_in, batch, nf, ng, nh, s, d, p, u, tf != 0, tg != 0, th != 0, h
#define CONV2D_ARGS(T) \
  const T *f, const T *g, i64 c_out, i64 c_in, i64 batch, i64 nfx, i64 nfy, \
  i64 ngx, i64 ngy, i64 nhx, i64 nhy, i64 sx, i64 sy, i64 dx, i64 dy, \
  i64 px, i64 py, i64 ux, i64 uy, int tf, int tg, int th, T *h
#define CONV2D_PASS \
  f, g, c_out, c_in, batch, nfx, nfy, ngx, ngy, nhx, nhy, sx, sy, dx, dy, \
  px, py, ux, uy, tf != 0, tg != 0, th != 0, h
#define COL1D_ARGS(T, in, out) \
  const T *in, i64 c_in, i64 batch, i64 nf, i64 ng, i64 ngg, i64 s, i64 d, \
  i64 p, i64 u, int tg, int tgg, T *out
#define COL1D_PASS(in, out) \
  in, c_in, batch, nf, ng, ngg, s, d, p, u, tg != 0, tgg != 0, out
#define COL2D_ARGS(T, in, out) \
  const T *in, i64 c_in, i64 batch, i64 nfx, i64 nfy, i64 ngx, i64 ngy, \
  i64 nggx, i64 nggy, i64 sx, i64 sy, i64 dx, i64 dy, i64 px, i64 py, \
  i64 ux, i64 uy, int tg, int tgg, T *out
#define COL2D_PASS(in, out) \
  in, c_in, batch, nfx, nfy, ngx, ngy, nggx, nggy, sx, sy, dx, dy, px, py, \
  ux, uy, tg != 0, tgg != 0, out

#define EXPORT_ALL(T, sfx) \
  void ref_mconv1d_##sfx(CONV1D_ARGS(T)) { cm::MConv1D<T>(CONV1D_PASS); } \
  void ref_mcorr1d_##sfx(CONV1D_ARGS(T)) { cm::MCorr1D<T>(CONV1D_PASS); } \
  void ref_mconvlconv_##sfx(CONV2D_ARGS(T)) { cm::MConvLConv<T>(CONV2D_PASS); } \
  void ref_mcorrlcorr_##sfx(CONV2D_ARGS(T)) { cm::MCorrLCorr<T>(CONV2D_PASS); } \
  void ref_snd2col_##sfx(COL1D_ARGS(T, g, gg)) { cm::Snd2Col<T>(COL1D_PASS(g, gg)); } \
  void ref_col2snd_##sfx(COL1D_ARGS(T, gg, g)) { cm::Col2Snd<T>(COL1D_PASS(gg, g)); } \
  void ref_spec2col_##sfx(COL2D_ARGS(T, g, gg)) { cm::Spec2Col<T>(COL2D_PASS(g, gg)); } \
  void ref_col2spec_##sfx(COL2D_ARGS(T, gg, g)) { cm::Col2Spec<T>(COL2D_PASS(gg, g)); }

extern "C" {

EXPORT_ALL(float, f32)
EXPORT_ALL(double, f64)

i64 ref_mconv_valid_size(i64 ng, i64 s, i64 d, i64 p, i64 u)
{ return cm::MConvValidSize(ng, s, d, p, u); }
i64 ref_mconv_support_size(i64 nf, i64 ng, i64 s, i64 d, i64 p, i64 u)
{ return cm::MConvSupportSize(nf, ng, s, d, p, u); }
i64 ref_mcorr_valid_size(i64 nf, i64 ng, i64 s, i64 d, i64 p, i64 u)
{ return cm::MCorrValidSize(nf, ng, s, d, p, u); }
i64 ref_mcorr_support_size(i64 ng, i64 s, i64 d, i64 p, i64 u)
{ return cm::MCorrSupportSize(ng, s, d, p, u); }
i64 ref_lconv_valid_size(i64 ng, i64 s, i64 p, i64 u)
{ return cm::LConvValidSize(ng, s, p, u); }
i64 ref_lconv_support_size(i64 nf, i64 ng, i64 s, i64 d, i64 p, i64 u)
{ return cm::LConvSupportSize(nf, ng, s, d, p, u); }
i64 ref_lcorr_valid_size(i64 nf, i64 ng, i64 s, i64 d, i64 p, i64 u)
{ return cm::LCorrValidSize(nf, ng, s, d, p, u); }
i64 ref_lcorr_support_size(i64 ng, i64 s, i64 p, i64 u)
{ return cm::LCorrSupportSize(ng, s, p, u); }

}  // extern "C"
