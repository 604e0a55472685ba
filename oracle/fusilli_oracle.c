/*
 * fusilli_oracle.c -- CPU restatement of the arithmetic the Fusilli graph ops
 * denote. TEST INFRASTRUCTURE ONLY: it is the checker for the CUDA path and the
 * timed CPU baseline; the product library never links or calls it.
 *
 * Where the algorithm comes from. The reference contains no arithmetic of its
 * own: each node is emitted as one torch-dialect op
 * (include/fusilli/support/asm_emitter.h) and executed by the IREE compiler +
 * runtime, pinned at iree 3.12.0rc20260515 (version.json:3), which is not part
 * of the reference tree. This file therefore restates the published ATen
 * semantics of the ops the emitter names, and is pinned by (a) the reference's
 * closed-form known-answer samples (samples/) and (b) PyTorch CPU outputs on
 * seeded inputs (tests/golden). Seeded-random bf16 results at the benchmark
 * shapes are not pinned by anything in the reference: "parity unpinned" there.
 *
 * All tensors arrive as dense float32 (or int64) arrays in LOGICAL order
 * (N,C,spatial.. / B..,M,K / B,H,S,D); the Python side converts dtypes and
 * applies stride permutations, and rounds results to each tensor's declared
 * dtype. Contractions, statistics and reductions accumulate in double and round
 * once at the end.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../include/fusilli_b200.h"


#define ORC_API __attribute__((visibility("default")))

#ifdef _OPENMP
#include <omp.h>
#endif

/* Threads the loops below use. A launcher may export OMP_NUM_THREADS=1 to every process it starts
 * (torchrun does); a caller that owns the host for the duration of a timing asks for the cores
 * here instead. Returns the count in force. */
ORC_API int orc_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

/* ---------------------------------------------------------------------- */
/* Convolution. Dims are always given for three spatial axes (leading axes of */
/* size 1 for 1-D/2-D). x[N,C,D,H,W], w[K,Cg,T,R,S], y[N,K,OD,OH,OW].         */
/* groups = C / Cg (asm_emitter.h:634-641); output extent formula            */
/* node/conv_node.h:50-54; cross-correlation, no flip (asm_emitter.h:667-731) */
/* ---------------------------------------------------------------------- */

typedef struct {
  int64_t N, C, D, H, W;
  int64_t K, Cg, T, R, S;
  int64_t OD, OH, OW;
  int64_t pd, ph, pw, sd, sh, sw, dd, dh, dw;
  int64_t groups, Kg;
} conv_geom;

static conv_geom make_geom(const int64_t *xd, const int64_t *wd,
                           const int64_t *yd, const int64_t *pad,
                           const int64_t *str, const int64_t *dil) {
  conv_geom g;
  g.N = xd[0]; g.C = xd[1]; g.D = xd[2]; g.H = xd[3]; g.W = xd[4];
  g.K = wd[0]; g.Cg = wd[1]; g.T = wd[2]; g.R = wd[3]; g.S = wd[4];
  g.OD = yd[2]; g.OH = yd[3]; g.OW = yd[4];
  g.pd = pad[0]; g.ph = pad[1]; g.pw = pad[2];
  g.sd = str[0]; g.sh = str[1]; g.sw = str[2];
  g.dd = dil[0]; g.dh = dil[1]; g.dw = dil[2];
  g.groups = g.C / g.Cg;
  g.Kg = g.K / g.groups;
  return g;
}

/* Range of ow for which iw = ow*sw - pw + s*dw lies in [0, W). */
static void valid_range(int64_t O, int64_t I, int64_t stride, int64_t pad,
                        int64_t tap_off, int64_t *lo, int64_t *hi) {
  /* smallest o with o*stride - pad + tap_off >= 0 */
  int64_t a = pad - tap_off;
  int64_t l = a <= 0 ? 0 : (a + stride - 1) / stride;
  /* largest o with o*stride - pad + tap_off <= I-1 */
  int64_t b = I - 1 + pad - tap_off;
  int64_t h = b < 0 ? -1 : b / stride;
  if (h > O - 1) h = O - 1;
  *lo = l;
  *hi = h + 1; /* exclusive */
}

/* Y = conv(X, W): aten.convolution, transposed=false (asm_emitter.h:667-731). */
ORC_API void orc_conv_fprop(const float *x, const float *w, float *y,
                            const int64_t *xd, const int64_t *wd,
                            const int64_t *yd, const int64_t *pad,
                            const int64_t *str, const int64_t *dil) {
  conv_geom g = make_geom(xd, wd, yd, pad, str, dil);
  int64_t plane = g.OD * g.OH * g.OW;
#pragma omp parallel
  {
    double *acc = (double *)malloc(sizeof(double) * (size_t)plane);
#pragma omp for collapse(2) schedule(dynamic)
    for (int64_t n = 0; n < g.N; ++n)
      for (int64_t k = 0; k < g.K; ++k) {
        memset(acc, 0, sizeof(double) * (size_t)plane);
        int64_t grp = k / g.Kg;
        for (int64_t cg = 0; cg < g.Cg; ++cg) {
          int64_t c = grp * g.Cg + cg;
          const float *xc = x + ((n * g.C + c) * g.D) * g.H * g.W;
          for (int64_t t = 0; t < g.T; ++t)
            for (int64_t r = 0; r < g.R; ++r)
              for (int64_t s = 0; s < g.S; ++s) {
                double wv = w[(((k * g.Cg + cg) * g.T + t) * g.R + r) * g.S + s];
                int64_t lo, hi;
                valid_range(g.OW, g.W, g.sw, g.pw, s * g.dw, &lo, &hi);
                for (int64_t od = 0; od < g.OD; ++od) {
                  int64_t id = od * g.sd - g.pd + t * g.dd;
                  if (id < 0 || id >= g.D) continue;
                  for (int64_t oh = 0; oh < g.OH; ++oh) {
                    int64_t ih = oh * g.sh - g.ph + r * g.dh;
                    if (ih < 0 || ih >= g.H) continue;
                    const float *xr = xc + (id * g.H + ih) * g.W - g.pw + s * g.dw;
                    double *ar = acc + (od * g.OH + oh) * g.OW;
                    if (g.sw == 1) {
                      for (int64_t ow = lo; ow < hi; ++ow) ar[ow] += wv * xr[ow];
                    } else {
                      for (int64_t ow = lo; ow < hi; ++ow)
                        ar[ow] += wv * xr[ow * g.sw];
                    }
                  }
                }
              }
        }
        float *yo = y + (n * g.K + k) * plane;
        for (int64_t i = 0; i < plane; ++i) yo[i] = (float)acc[i];
      }
    free(acc);
  }
}

/* dX = adjoint of fprop w.r.t. X: aten.convolution_backward, output_mask
 * [true,false,false] (asm_emitter.h:1018-1064). */
ORC_API void orc_conv_dgrad(const float *dy, const float *w, float *dx,
                            const int64_t *xd, const int64_t *wd,
                            const int64_t *yd, const int64_t *pad,
                            const int64_t *str, const int64_t *dil) {
  conv_geom g = make_geom(xd, wd, yd, pad, str, dil);
  int64_t plane = g.D * g.H * g.W;
#pragma omp parallel
  {
    double *acc = (double *)malloc(sizeof(double) * (size_t)plane);
#pragma omp for collapse(2) schedule(dynamic)
    for (int64_t n = 0; n < g.N; ++n)
      for (int64_t c = 0; c < g.C; ++c) {
        memset(acc, 0, sizeof(double) * (size_t)plane);
        int64_t grp = c / g.Cg, cg = c % g.Cg;
        for (int64_t kk = 0; kk < g.Kg; ++kk) {
          int64_t k = grp * g.Kg + kk;
          const float *dyk = dy + (n * g.K + k) * g.OD * g.OH * g.OW;
          for (int64_t t = 0; t < g.T; ++t)
            for (int64_t r = 0; r < g.R; ++r)
              for (int64_t s = 0; s < g.S; ++s) {
                double wv = w[(((k * g.Cg + cg) * g.T + t) * g.R + r) * g.S + s];
                int64_t lo, hi;
                valid_range(g.OW, g.W, g.sw, g.pw, s * g.dw, &lo, &hi);
                for (int64_t od = 0; od < g.OD; ++od) {
                  int64_t id = od * g.sd - g.pd + t * g.dd;
                  if (id < 0 || id >= g.D) continue;
                  for (int64_t oh = 0; oh < g.OH; ++oh) {
                    int64_t ih = oh * g.sh - g.ph + r * g.dh;
                    if (ih < 0 || ih >= g.H) continue;
                    double *ar = acc + (id * g.H + ih) * g.W - g.pw + s * g.dw;
                    const float *dr = dyk + (od * g.OH + oh) * g.OW;
                    if (g.sw == 1) {
                      for (int64_t ow = lo; ow < hi; ++ow) ar[ow] += wv * dr[ow];
                    } else {
                      for (int64_t ow = lo; ow < hi; ++ow)
                        ar[ow * g.sw] += wv * dr[ow];
                    }
                  }
                }
              }
        }
        float *o = dx + (n * g.C + c) * plane;
        for (int64_t i = 0; i < plane; ++i) o[i] = (float)acc[i];
      }
    free(acc);
  }
}

/* dW = adjoint of fprop w.r.t. W: aten.convolution_backward, output_mask
 * [false,true,false] (asm_emitter.h:856-903). */
ORC_API void orc_conv_wgrad(const float *dy, const float *x, float *dwt,
                            const int64_t *xd, const int64_t *wd,
                            const int64_t *yd, const int64_t *pad,
                            const int64_t *str, const int64_t *dil) {
  conv_geom g = make_geom(xd, wd, yd, pad, str, dil);
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int64_t k = 0; k < g.K; ++k)
    for (int64_t cg = 0; cg < g.Cg; ++cg) {
      int64_t grp = k / g.Kg;
      int64_t c = grp * g.Cg + cg;
      for (int64_t t = 0; t < g.T; ++t)
        for (int64_t r = 0; r < g.R; ++r)
          for (int64_t s = 0; s < g.S; ++s) {
            int64_t lo, hi;
            valid_range(g.OW, g.W, g.sw, g.pw, s * g.dw, &lo, &hi);
            double sum = 0.0;
            for (int64_t n = 0; n < g.N; ++n) {
              const float *xc = x + ((n * g.C + c) * g.D) * g.H * g.W;
              const float *dyk = dy + (n * g.K + k) * g.OD * g.OH * g.OW;
              for (int64_t od = 0; od < g.OD; ++od) {
                int64_t id = od * g.sd - g.pd + t * g.dd;
                if (id < 0 || id >= g.D) continue;
                for (int64_t oh = 0; oh < g.OH; ++oh) {
                  int64_t ih = oh * g.sh - g.ph + r * g.dh;
                  if (ih < 0 || ih >= g.H) continue;
                  const float *xr = xc + (id * g.H + ih) * g.W - g.pw + s * g.dw;
                  const float *dr = dyk + (od * g.OH + oh) * g.OW;
                  double part = 0.0;
                  for (int64_t ow = lo; ow < hi; ++ow)
                    part += (double)dr[ow] * (double)xr[ow * g.sw];
                  sum += part;
                }
              }
            }
            dwt[(((k * g.Cg + cg) * g.T + t) * g.R + r) * g.S + s] = (float)sum;
          }
    }
}

/* ---------------------------------------------------------------------- */
/* Matmul: aten.matmul with batch broadcast (asm_emitter.h:1669-1696,         */
/* node/matmul_node.h:40-66). a_off/b_off give, per output batch, the element */
/* offset of the A / B matrix used (broadcast = repeated offsets).            */
/* ---------------------------------------------------------------------- */
ORC_API void orc_matmul(const float *a, const float *b, float *c,
                        int64_t nbatch, const int64_t *a_off,
                        const int64_t *b_off, int64_t M, int64_t N, int64_t K) {
  /* Rows of A are taken eight at a time so that every row of B is streamed once per
   * eight output rows; each output element still adds its K products in ascending k,
   * in double, exactly as one row at a time would. */
  enum { RB = 8 };
  const int64_t mblocks = (M + RB - 1) / RB;
#pragma omp parallel
  {
    double *acc = (double *)malloc(sizeof(double) * (size_t)N * RB);
#pragma omp for collapse(2) schedule(static)
    for (int64_t bi = 0; bi < nbatch; ++bi)
      for (int64_t mb = 0; mb < mblocks; ++mb) {
        const int64_t m0 = mb * RB;
        const int64_t rows = (M - m0) < RB ? (M - m0) : RB;
        const float *am = a + a_off[bi] + m0 * K;
        const float *bm = b + b_off[bi];
        for (int64_t i = 0; i < rows * N; ++i) acc[i] = 0.0;
        for (int64_t k = 0; k < K; ++k) {
          const float *br = bm + k * N;
          for (int64_t r = 0; r < rows; ++r) {
            const double av = am[r * K + k];
            double *ar = acc + r * N;
            for (int64_t n = 0; n < N; ++n) ar[n] += av * br[n];
          }
        }
        for (int64_t r = 0; r < rows; ++r) {
          float *cm = c + (bi * M + m0 + r) * N;
          for (int64_t n = 0; n < N; ++n) cm[n] = (float)acc[r * N + n];
        }
      }
    free(acc);
  }
}

/* ---------------------------------------------------------------------- */
/* SDPA: aten.scaled_dot_product_attention (asm_emitter.h:2409-2468); scalar  */
/* statement in samples/sdpa_utils.cpp:49-102. q[B,Hq,Sq,D] k[B,Hk,Skv,D]      */
/* v[B,Hv,Skv,Dv]; kv head of query head h is h / (Hq/Hk) resp. h / (Hq/Hv).   */
/* mask: additive, dims md[4] each 1 or full (node/sdpa_node.h:145-175).      */
/* causal masks keys j > i (top-left aligned, sdpa_utils.cpp:75-77).          */
/* ---------------------------------------------------------------------- */
ORC_API void orc_sdpa(const float *q, const float *k, const float *v,
                      const float *mask, const int64_t *md, float *o, int64_t B,
                      int64_t Hq, int64_t Hk, int64_t Hv, int64_t Sq,
                      int64_t Skv, int64_t D, int64_t Dv, int32_t causal,
                      double scale) {
#pragma omp parallel
  {
    double *p = (double *)malloc(sizeof(double) * (size_t)Skv);
    double *acc = (double *)malloc(sizeof(double) * (size_t)Dv);
#pragma omp for collapse(3) schedule(dynamic)
    for (int64_t b = 0; b < B; ++b)
      for (int64_t h = 0; h < Hq; ++h)
        for (int64_t i = 0; i < Sq; ++i) {
          int64_t hk = h / (Hq / Hk), hv = h / (Hq / Hv);
          const float *qi = q + ((b * Hq + h) * Sq + i) * D;
          const float *kb = k + (b * Hk + hk) * Skv * D;
          const float *vb = v + (b * Hv + hv) * Skv * Dv;
          int64_t jend = causal ? (i + 1 < Skv ? i + 1 : Skv) : Skv;
          double mx = -INFINITY;
          for (int64_t j = 0; j < jend; ++j) {
            const float *kj = kb + j * D;
            double dot = 0.0;
            for (int64_t d = 0; d < D; ++d) dot += (double)qi[d] * (double)kj[d];
            dot *= scale;
            if (mask) {
              int64_t mb = md[0] == 1 ? 0 : b, mh = md[1] == 1 ? 0 : h;
              int64_t mi = md[2] == 1 ? 0 : i, mj = md[3] == 1 ? 0 : j;
              dot += mask[((mb * md[1] + mh) * md[2] + mi) * md[3] + mj];
            }
            p[j] = dot;
            if (dot > mx) mx = dot;
          }
          double sum = 0.0;
          for (int64_t j = 0; j < jend; ++j) {
            p[j] = exp(p[j] - mx);
            sum += p[j];
          }
          for (int64_t d = 0; d < Dv; ++d) acc[d] = 0.0;
          for (int64_t j = 0; j < jend; ++j) {
            double pj = p[j];
            const float *vj = vb + j * Dv;
            for (int64_t d = 0; d < Dv; ++d) acc[d] += pj * vj[d];
          }
          float *oi = o + ((b * Hq + h) * Sq + i) * Dv;
          for (int64_t d = 0; d < Dv; ++d) oi[d] = (float)(acc[d] / sum);
        }
    free(p);
    free(acc);
  }
}

/* ---------------------------------------------------------------------- */
/* LayerNorm over all non-batch dims: aten.layer_norm / native_layer_norm     */
/* (asm_emitter.h:1427-1503); biased variance; INV_VARIANCE = rsqrt(var+eps). */
/* x[B,R]; scale/bias [R] or NULL; mean/rstd [B] or NULL.                     */
/* ---------------------------------------------------------------------- */
ORC_API void orc_layernorm(const float *x, const float *scale,
                           const float *bias, double eps, float *y, float *mean,
                           float *rstd, int64_t B, int64_t R) {
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < B; ++b) {
    const float *xr = x + b * R;
    double s = 0.0;
    for (int64_t i = 0; i < R; ++i) s += xr[i];
    double mu = s / (double)R;
    double ss = 0.0;
    for (int64_t i = 0; i < R; ++i) {
      double d = xr[i] - mu;
      ss += d * d;
    }
    double rs = 1.0 / sqrt(ss / (double)R + eps);
    float *yr = y + b * R;
    for (int64_t i = 0; i < R; ++i) {
      double val = (xr[i] - mu) * rs;
      if (scale) val *= scale[i];
      if (bias) val += bias[i];
      yr[i] = (float)val;
    }
    if (mean) mean[b] = (float)mu;
    if (rstd) rstd[b] = (float)rs;
  }
}

/* RMSNorm: aten.rms_norm (asm_emitter.h:1592-1626): x*rsqrt(mean(x^2)+eps)*w */
ORC_API void orc_rmsnorm(const float *x, const float *scale, double eps,
                         float *y, int64_t B, int64_t R) {
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < B; ++b) {
    const float *xr = x + b * R;
    double ss = 0.0;
    for (int64_t i = 0; i < R; ++i) ss += (double)xr[i] * (double)xr[i];
    double rs = 1.0 / sqrt(ss / (double)R + eps);
    float *yr = y + b * R;
    for (int64_t i = 0; i < R; ++i) {
      double val = xr[i] * rs;
      if (scale) val *= scale[i];
      yr[i] = (float)val;
    }
  }
}

/* ---------------------------------------------------------------------- */
/* Reduction with keepdim over {i : yd[i]==1 && xd[i]>1}                      */
/* (node/reduction_node.h:47-57; op table asm_emitter.h:2282-2317).          */
/* ---------------------------------------------------------------------- */
static int64_t y_index(int64_t lin, int rank, const int64_t *xd,
                       const int64_t *yd) {
  int64_t idx[FB_MAX_RANK];
  for (int i = rank - 1; i >= 0; --i) {
    idx[i] = lin % xd[i];
    lin /= xd[i];
  }
  int64_t yi = 0;
  for (int i = 0; i < rank; ++i) yi = yi * yd[i] + (yd[i] == 1 ? 0 : idx[i]);
  return yi;
}

ORC_API void orc_reduce_f(int32_t mode, const float *x, float *y, int32_t rank,
                          const int64_t *xd, const int64_t *yd) {
  int64_t xn = 1, yn = 1;
  for (int i = 0; i < rank; ++i) {
    xn *= xd[i];
    yn *= yd[i];
  }
  double *acc = (double *)malloc(sizeof(double) * (size_t)yn);
  for (int64_t i = 0; i < yn; ++i) {
    switch (mode) {
    case FB_RED_MUL:
    case FB_RED_MUL_NO_ZEROS: acc[i] = 1.0; break;
    case FB_RED_MIN: acc[i] = INFINITY; break;
    case FB_RED_MAX: acc[i] = -INFINITY; break;
    default: acc[i] = 0.0; break;
    }
  }
  for (int64_t l = 0; l < xn; ++l) {
    double v = x[l];
    double *a = acc + y_index(l, rank, xd, yd);
    switch (mode) {
    case FB_RED_ADD:
    case FB_RED_SUM:
    case FB_RED_AVG: *a += v; break;
    case FB_RED_MUL: *a *= v; break;
    case FB_RED_MUL_NO_ZEROS: if (v != 0.0) *a *= v; break;
    case FB_RED_MIN: if (v < *a || isnan(v)) *a = v; break;
    case FB_RED_MAX: if (v > *a || isnan(v)) *a = v; break;
    case FB_RED_AMAX: if (fabs(v) > *a || isnan(v)) *a = fabs(v); break;
    case FB_RED_NORM1: *a += fabs(v); break;
    case FB_RED_NORM2: *a += v * v; break;
    default: break;
    }
  }
  double cnt = (double)(xn / yn);
  for (int64_t i = 0; i < yn; ++i) {
    double r = acc[i];
    if (mode == FB_RED_AVG) r /= cnt;
    if (mode == FB_RED_NORM2) r = sqrt(r);
    y[i] = (float)r;
  }
  free(acc);
}

/* Row-sum fast path for big row-major inputs (reduction over the last dim). */
ORC_API void orc_rowsum_f(const float *x, float *y, int64_t rows, int64_t cols) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float *xr = x + r * cols;
    double s = 0.0;
    for (int64_t i = 0; i < cols; ++i) s += xr[i];
    y[r] = (float)s;
  }
}

/* Integer reductions stay integer and are exact (the reference's samples compare
 * with ==, samples/reduction/reduction_ops.cpp:229-236). */
ORC_API void orc_reduce_i(int32_t mode, const int64_t *x, int64_t *y,
                          int32_t rank, const int64_t *xd, const int64_t *yd) {
  int64_t xn = 1, yn = 1;
  for (int i = 0; i < rank; ++i) {
    xn *= xd[i];
    yn *= yd[i];
  }
  for (int64_t i = 0; i < yn; ++i) {
    switch (mode) {
    case FB_RED_MUL:
    case FB_RED_MUL_NO_ZEROS: y[i] = 1; break;
    case FB_RED_MIN: y[i] = INT64_MAX; break;
    case FB_RED_MAX: y[i] = INT64_MIN; break;
    default: y[i] = 0; break;
    }
  }
  for (int64_t l = 0; l < xn; ++l) {
    int64_t v = x[l];
    int64_t *a = y + y_index(l, rank, xd, yd);
    int64_t av = v < 0 ? -v : v;
    switch (mode) {
    case FB_RED_ADD:
    case FB_RED_SUM: *a += v; break;
    case FB_RED_MUL: *a *= v; break;
    case FB_RED_MUL_NO_ZEROS: if (v != 0) *a *= v; break;
    case FB_RED_MIN: if (v < *a) *a = v; break;
    case FB_RED_MAX: if (v > *a) *a = v; break;
    case FB_RED_AMAX: if (av > *a) *a = av; break;
    case FB_RED_NORM1: *a += av; break;
    case FB_RED_NORM2: *a += v * v; break;
    default: break;
    }
  }
  if (mode == FB_RED_NORM2)
    for (int64_t i = 0; i < yn; ++i) y[i] = (int64_t)sqrt((double)y[i]);
}

/* ---------------------------------------------------------------------- */
/* Pointwise (asm_emitter.h:1959-2116). Inputs already broadcast to the output */
/* shape. prm = {elu_alpha, softplus_beta, softplus_threshold, swish_beta}.    */
/* Floating modes compute in double and return float; compare/logical modes    */
/* write 0/1 into out as floats (the caller narrows to one byte).              */
/* ---------------------------------------------------------------------- */
static double sigmoid_d(double x) { return 1.0 / (1.0 + exp(-x)); }

ORC_API void orc_pointwise_f(int32_t mode, int64_t n, const float *a,
                             const float *b, const float *c, float *out,
                             const double *prm) {
  const double kSqrt2OverPi = 0.79788456080286535588;
  const double kInvSqrt2 = 0.70710678118654752440;
  const double kInvSqrt2Pi = 0.39894228040143267794;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    double x = a[i];
    double y = b ? b[i] : 0.0;
    double r = 0.0;
    switch (mode) {
    case FB_PW_ABS: r = fabs(x); break;
    case FB_PW_ADD: r = x + y; break;
    case FB_PW_ADD_SQUARE: r = x + y * y; break;
    case FB_PW_BINARY_SELECT: r = (x != 0.0) ? y : (double)c[i]; break;
    case FB_PW_CEIL: r = ceil(x); break;
    case FB_PW_CMP_EQ: r = x == y; break;
    case FB_PW_CMP_GE: r = x >= y; break;
    case FB_PW_CMP_GT: r = x > y; break;
    case FB_PW_CMP_LE: r = x <= y; break;
    case FB_PW_CMP_LT: r = x < y; break;
    case FB_PW_CMP_NEQ: r = x != y; break;
    case FB_PW_DIV: r = x / y; break;
    case FB_PW_ELU_FWD: r = x > 0 ? x : prm[0] * expm1(x); break;
    case FB_PW_ERF: r = erf(x); break;
    case FB_PW_EXP: r = exp(x); break;
    case FB_PW_FLOOR: r = floor(x); break;
    case FB_PW_GELU_FWD: r = 0.5 * x * (1.0 + erf(x * kInvSqrt2)); break;
    case FB_PW_GELU_APPROX_TANH_FWD:
      r = 0.5 * x * (1.0 + tanh(kSqrt2OverPi * (x + 0.044715 * x * x * x)));
      break;
    case FB_PW_GELU_BWD: { /* (dy = a, x = b) */
      double cdf = 0.5 * (1.0 + erf(y * kInvSqrt2));
      double pdf = kInvSqrt2Pi * exp(-0.5 * y * y);
      r = x * (cdf + y * pdf);
    } break;
    case FB_PW_GELU_APPROX_TANH_BWD: {
      double u = kSqrt2OverPi * (y + 0.044715 * y * y * y);
      double t = tanh(u);
      double du = kSqrt2OverPi * (1.0 + 3.0 * 0.044715 * y * y);
      r = x * (0.5 * (1.0 + t) + 0.5 * y * (1.0 - t * t) * du);
    } break;
    case FB_PW_IDENTITY: r = x; break;
    case FB_PW_LOG: r = log(x); break;
    case FB_PW_LOGICAL_AND: r = (x != 0.0) && (y != 0.0); break;
    case FB_PW_LOGICAL_NOT: r = !(x != 0.0); break;
    case FB_PW_LOGICAL_OR: r = (x != 0.0) || (y != 0.0); break;
    case FB_PW_MAX_OP: r = (x > y || isnan(x)) ? x : y; break;
    case FB_PW_MIN_OP: r = (x < y || isnan(x)) ? x : y; break;
    case FB_PW_MUL: r = x * y; break;
    case FB_PW_NEG: r = -x; break;
    case FB_PW_RECIPROCAL: r = 1.0 / x; break;
    case FB_PW_RELU_BWD: r = y > 0.0 ? x : 0.0; break; /* threshold_backward */
    case FB_PW_RELU_FWD: r = x > 0.0 ? x : 0.0; break;
    case FB_PW_RSQRT: r = 1.0 / sqrt(x); break;
    case FB_PW_SIGMOID_FWD: r = sigmoid_d(x); break;
    case FB_PW_SIN: r = sin(x); break;
    case FB_PW_SOFTPLUS_FWD:
      r = (x * prm[1] > prm[2]) ? x : log1p(exp(x * prm[1])) / prm[1];
      break;
    case FB_PW_SQRT: r = sqrt(x); break;
    case FB_PW_SUB: r = x - y; break;
    case FB_PW_SWISH_FWD: r = x * sigmoid_d(prm[3] * x); break;
    case FB_PW_SWISH_BWD: { /* (dy = a, x = b) */
      double s = sigmoid_d(prm[3] * y);
      r = x * (s + prm[3] * y * s * (1.0 - s));
    } break;
    case FB_PW_TAN: r = tan(x); break;
    case FB_PW_TANH_BWD: { /* tanh_backward(dy, tanh(x)) */
      double t = tanh(y);
      r = x * (1.0 - t * t);
    } break;
    case FB_PW_TANH_FWD: r = tanh(x); break;
    default: r = NAN; break;
    }
    out[i] = (float)r;
  }
}

/* Integer pointwise: exact, C truncating division (the reference expects
 * -50/13 == -3, samples/pointwise/pointwise_binary_ops.cpp:129-131). Returns
 * -1 for modes that have no integer meaning. */
ORC_API int32_t orc_pointwise_i(int32_t mode, int64_t n, const int64_t *a,
                                const int64_t *b, const int64_t *c,
                                int64_t *out) {
  for (int64_t i = 0; i < n; ++i) {
    int64_t x = a[i], y = b ? b[i] : 0, r = 0;
    switch (mode) {
    case FB_PW_ABS: r = x < 0 ? -x : x; break;
    case FB_PW_ADD: r = x + y; break;
    case FB_PW_ADD_SQUARE: r = x + y * y; break;
    case FB_PW_BINARY_SELECT: r = x != 0 ? y : c[i]; break;
    case FB_PW_CMP_EQ: r = x == y; break;
    case FB_PW_CMP_GE: r = x >= y; break;
    case FB_PW_CMP_GT: r = x > y; break;
    case FB_PW_CMP_LE: r = x <= y; break;
    case FB_PW_CMP_LT: r = x < y; break;
    case FB_PW_CMP_NEQ: r = x != y; break;
    case FB_PW_DIV: r = y == 0 ? 0 : x / y; break;
    case FB_PW_IDENTITY:
    case FB_PW_CEIL:
    case FB_PW_FLOOR: r = x; break;
    case FB_PW_LOGICAL_AND: r = (x != 0) && (y != 0); break;
    case FB_PW_LOGICAL_NOT: r = !(x != 0); break;
    case FB_PW_LOGICAL_OR: r = (x != 0) || (y != 0); break;
    case FB_PW_MAX_OP: r = x > y ? x : y; break;
    case FB_PW_MIN_OP: r = x < y ? x : y; break;
    case FB_PW_MUL: r = x * y; break;
    case FB_PW_NEG: r = -x; break;
    case FB_PW_RELU_BWD: r = y > 0 ? x : 0; break;
    case FB_PW_RELU_FWD: r = x > 0 ? x : 0; break;
    case FB_PW_SUB: r = x - y; break;
    default: return -1;
    }
    out[i] = r;
  }
  return 0;
}
