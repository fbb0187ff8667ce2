/* CPU restatement of the Mellin / linear correlation and convolution
 * operators of sdrobert/cnn-mellin.
 *
 * THIS IS TEST INFRASTRUCTURE.  It exists so that the CUDA kernels can be
 * checked against an independent, obviously-correct statement of the maths.
 * Only the test-suite, the smoke check and the CPU-baseline leg of the
 * benchmark may load it; the product library never does.
 *
 * Parity status: PINNED.  tests/test_oracle.py checks every routine here
 * against (a) all rational-valued known-answer cases of the reference's
 * c/tests/test_*_buffers.h and (b) outputs and gradients of the reference's own
 * CPU extension on seeded random inputs (tests/golden/).
 *
 * Everything is written from the defining relations, evaluated by brute
 * force for every (output, tap) combination; there are no bound
 * computations, tables or strides to get wrong.
 *
 * Axis relations (1-based Mellin positions; P = p + 1):
 *   Mellin correlation  (mconv.h:62-66):    (hx + s)(fx + d) = P (gx + u)
 *   Mellin convolution  (mconv.h:21-26):    P (hx + s)       = (fx + d)(gx + u)
 *   linear correlation  (mconv.h:166-172):  s hy + d fy - p  = u gy
 *   linear convolution  (mconv.h:106-112):  s hy - d fy + p  = u gy
 * A tap contributes only when the relation has an integer solution g with
 * 0 <= g < ng.
 */
#include <stdint.h>
#include <stddef.h>

typedef int64_t i64;

enum { KIND_CORR = 0, KIND_CONV = 1 };

static i64 imax(i64 a, i64 b) { return a > b ? a : b; }

/* floor(a / b) for b > 0 (C division truncates toward zero;
 * mconv.h:774-778 corrects it the same way) */
static i64 floordiv(i64 a, i64 b)
{
  i64 q = a / b;
  if ((a % b != 0) && ((a < 0) != (b < 0))) --q;
  return q;
}

/* ---- output sizes: mconv.h:452-672; Python twins mconv.py:73-118 ---------- */

i64 oracle_mconv_valid_size(i64 ng, i64 s, i64 d, i64 p, i64 u)
{ return imax(floordiv(d * (ng + u - 1), p + 1) - s + 1, 0); }

i64 oracle_mconv_support_size(i64 nf, i64 ng, i64 s, i64 d, i64 p, i64 u)
{ return imax(floordiv((nf + d - 1) * (ng + u - 1), p + 1) - s + 1, 0); }

i64 oracle_mcorr_valid_size(i64 nf, i64 ng, i64 s, i64 d, i64 p, i64 u)
{ return imax(floordiv((ng + u - 1) * (p + 1), nf + d - 1) - s + 1, 0); }

i64 oracle_mcorr_support_size(i64 ng, i64 s, i64 d, i64 p, i64 u)
{ return imax(floordiv((ng + u - 1) * (p + 1), d) - s + 1, 0); }

i64 oracle_lconv_valid_size(i64 ng, i64 s, i64 p, i64 u)
{ return imax(floordiv(u * (ng - 1) - p, s) + 1, 0); }

i64 oracle_lconv_support_size(i64 nf, i64 ng, i64 s, i64 d, i64 p, i64 u)
{ return imax(floordiv(u * (ng - 1) + d * (nf - 1) - p, s) + 1, 0); }

i64 oracle_lcorr_valid_size(i64 nf, i64 ng, i64 s, i64 d, i64 p, i64 u)
{ return imax(floordiv(u * (ng - 1) - d * (nf - 1) + p, s) + 1, 0); }

i64 oracle_lcorr_support_size(i64 ng, i64 s, i64 p, i64 u)
{ return imax(floordiv(u * (ng - 1) + p, s) + 1, 0); }

/* ---- axis relations ------------------------------------------------------- */

/* exact quotient num/den shifted by -off, or -1 when den does not divide num
 * or the result falls outside [0, n) */
static i64 exact_index(i64 num, i64 den, i64 off, i64 n)
{
  if (den == 0 || num % den != 0) return -1;
  const i64 q = num / den - off;
  return (q >= 0 && q < n) ? q : -1;
}

/* source position along the Mellin axis for output hx and tap fx */
static i64 mellin_source(int kind, i64 hx, i64 fx, i64 s, i64 d, i64 p, i64 u, i64 ng)
{
  const i64 P = p + 1;
  return kind == KIND_CORR ? exact_index((hx + s) * (fx + d), P, u, ng)
                           : exact_index(P * (hx + s), fx + d, u, ng);
}

/* source position along the linear axis for output hy and tap fy */
static i64 linear_source(int kind, i64 hy, i64 fy, i64 s, i64 d, i64 p, i64 u, i64 ng)
{
  return kind == KIND_CORR ? exact_index(s * hy + d * fy - p, u, 0, ng)
                           : exact_index(s * hy - d * fy + p, u, 0, ng);
}

/* column position ggx whose correlation source is gx, for tap fx:
 * (ggx + s)(fx + d) = P (gx + u)   (mconv.h:1292-1297) */
static i64 mellin_column(i64 gx, i64 fx, i64 s, i64 d, i64 p, i64 u, i64 ngg)
{ return exact_index((p + 1) * (gx + u), fx + d, s, ngg); }

/* column position ggy whose correlation source is gy, for tap fy:
 * s ggy + d fy - p = u gy   (mconv.h:1370-1373) */
static i64 linear_column(i64 gy, i64 fy, i64 s, i64 d, i64 p, i64 u, i64 ngg)
{ return exact_index(u * gy - d * fy + p, s, 0, ngg); }

/* ---- the operators, once per element type -------------------------------- */

#define REAL float
#define ACC float
#define SFX f32
#include "mellin_oracle_impl.inc"
#undef REAL
#undef ACC
#undef SFX

#define REAL double
#define ACC double
#define SFX f64
#include "mellin_oracle_impl.inc"
#undef REAL
#undef ACC
#undef SFX
