/*
 * CPU oracle for the DCNv4 / FlashDeformAttn operator path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the GPU kernels are
 * compared against; it is never the thing measured or shipped.  Only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg may load it.
 *
 * It restates, in plain C, the arithmetic of the reference CUDA sources
 * (paths relative to the reference project root):
 *   DCNv4 forward            DCNv4_op/src/cuda/dcnv4_im2col_cuda.cuh:142-244
 *   DCNv4 backward           DCNv4_op/src/cuda/dcnv4_col2im_cuda.cuh:196-366
 *   FlashDeformAttn forward  DCNv4_op/src/cuda/flash_deform_im2col_cuda.cuh:129-209
 *   FlashDeformAttn backward DCNv4_op/src/cuda/flash_deform_col2im_cuda.cuh:171-318
 *   bilinear gather/scatter  DCNv4_op/src/cuda/common.h:41-212
 *   output-size rule         DCNv4_op/src/cuda/dcnv4_cuda.cu:48-52
 *
 * Numerics: sampling coordinates are computed in fp32 with exactly the
 * operation order the reference kernels compile to (so floor() picks the same
 * corner pixels bit for bit); everything downstream of the coordinates
 * (bilinear weights, products, sums, softmax) is carried in fp64 so the oracle
 * is the "exact" answer the fp32/fp16/bf16 kernels are measured against.
 *
 * Parity pin: the DCNv4 half is pinned against the reference's own
 * pure-PyTorch core (classification/ops_dcnv3/functions/dcnv3_func.py:172-220)
 * through committed golden vectors.  The reference has no CPU formula for
 * FlashDeformAttn; that half (and DCNv4 once more) is pinned against golden
 * vectors produced by the reference's own CUDA kernels, compiled unmodified and
 * run on a B200, and against an independent grid_sample + autograd formulation.
 *
 * Inputs are float32 arrays (fp16/bf16 test inputs are rounded to the storage
 * type first and then widened, so the oracle sees exactly the values the GPU
 * sees).  Outputs are float64.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_SKIPPED INT32_MIN

/* Bilinear footprint of one sampling point (common.h:47-58). */
typedef struct {
  int h_low, w_low;
  double w1, w2, w3, w4; /* weights of (h0,w0) (h0,w0+1) (h0+1,w0) (h0+1,w0+1) */
  double lh, lw, hh, hw;
} footprint_t;

static inline footprint_t footprint(float h, float w) {
  footprint_t f;
  f.h_low = (int)floorf(h);
  f.w_low = (int)floorf(w);
  /* h - h_low is exact in fp32, so carrying it in fp64 changes nothing. */
  f.lh = (double)h - (double)f.h_low;
  f.lw = (double)w - (double)f.w_low;
  f.hh = 1.0 - f.lh;
  f.hw = 1.0 - f.lw;
  f.w1 = f.hh * f.hw;
  f.w2 = f.hh * f.lw;
  f.w3 = f.lh * f.hw;
  f.w4 = f.lh * f.lw;
  return f;
}

/* Range test applied before a point is sampled at all
 * (dcnv4_im2col_cuda.cuh:227, flash_deform_im2col_cuda.cuh:190). */
static inline int in_range(float h, float w, int H, int W) {
  return h > -1.0f && w > -1.0f && h < (float)H && w < (float)W;
}

/* DCNv4 sampling coordinate of tap index t along one axis
 * (dcnv4_im2col_cuda.cuh:203-224).  base = p0 - c*s and the final
 * multiply-add are each a single fused multiply-add, which is what nvcc's
 * default contraction makes of the reference expressions. */
static inline float dcn_base(int p0, int c, float s) {
  return fmaf(-(float)c, s, (float)p0);
}
static inline float dcn_coord(float base, int tap_dil, float off, float s) {
  return fmaf((float)tap_dil + off, s, base);
}

/* FlashDeformAttn pixel coordinate loc*size - 0.5 (flash_deform_im2col_cuda.cuh:188-189).  The
 * reference binary evaluates it as ONE fused multiply-add: nvcc demotes the double literal's
 * subtraction to fp32 and contracts it with the product.  Checked against the reference
 * kernels run on a B200: at a sample whose product rounds to x.5 exactly, the two-rounding
 * form selects the next row (floor 16, lh 0) while the reference and the fused form select
 * floor 15 with lh just under 1 -- same value, different location gradient. */
static inline float fda_coord(float loc, int size) {
  return fmaf(loc, (float)size, -0.5f);
}

static void softmax_f64(const float *logits, int n, double *p) {
  double mx = -INFINITY, sum = 0.0;
  for (int i = 0; i < n; ++i)
    if ((double)logits[i] > mx) mx = (double)logits[i];
  for (int i = 0; i < n; ++i) {
    p[i] = exp((double)logits[i] - mx);
    sum += p[i];
  }
  for (int i = 0; i < n; ++i) p[i] /= sum;
}

int oracle_dcnv4_out_size(int in, int pad, int dil, int k, int stride) {
  return (in + 2 * pad - (dil * (k - 1) + 1)) / stride + 1;
}

/* Gather one point for all D channels of a group; returns nothing when the
 * corner is outside the map (zero padding by omission, common.h:74-90). */
static inline void gather_point(const float *img, int H, int W, int C, int D,
                                const footprint_t *f, double scale,
                                double *acc) {
  const int h0 = f->h_low, w0 = f->w_low, h1 = h0 + 1, w1 = w0 + 1;
  for (int c = 0; c < D; ++c) {
    double v = 0.0;
    if (h0 >= 0 && w0 >= 0) v += f->w1 * (double)img[((size_t)h0 * W + w0) * C + c];
    if (h0 >= 0 && w1 < W) v += f->w2 * (double)img[((size_t)h0 * W + w1) * C + c];
    if (h1 < H && w0 >= 0) v += f->w3 * (double)img[((size_t)h1 * W + w0) * C + c];
    if (h1 < H && w1 < W) v += f->w4 * (double)img[((size_t)h1 * W + w1) * C + c];
    acc[c] += scale * v;
  }
}

/* Scatter + partial derivatives of one point (common.h:100-212).
 * img / gimg point at channel 0 of the group in pixel (0,0).
 * gout: D upstream gradients.  Returns d/dw (x), d/dh (y) of the bilinear
 * value dotted with gout, and the bilinear value dotted with gout. */
static inline void scatter_point(const float *img, double *gimg, int H, int W,
                                 int C, int D, const footprint_t *f,
                                 double attn, const float *gout, double *d_w,
                                 double *d_h, double *d_val) {
  const int h0 = f->h_low, w0 = f->w_low, h1 = h0 + 1, w1 = w0 + 1;
  double sw = 0.0, sh = 0.0, sv = 0.0;
  for (int c = 0; c < D; ++c) {
    const double g = (double)gout[c];
    double v1 = 0, v2 = 0, v3 = 0, v4 = 0;
    if (h0 >= 0 && w0 >= 0) {
      size_t i = ((size_t)h0 * W + w0) * C + c;
      v1 = img[i];
      gimg[i] += g * attn * f->w1;
    }
    if (h0 >= 0 && w1 < W) {
      size_t i = ((size_t)h0 * W + w1) * C + c;
      v2 = img[i];
      gimg[i] += g * attn * f->w2;
    }
    if (h1 < H && w0 >= 0) {
      size_t i = ((size_t)h1 * W + w0) * C + c;
      v3 = img[i];
      gimg[i] += g * attn * f->w3;
    }
    if (h1 < H && w1 < W) {
      size_t i = ((size_t)h1 * W + w1) * C + c;
      v4 = img[i];
      gimg[i] += g * attn * f->w4;
    }
    sw += g * (-f->hh * v1 + f->hh * v2 - f->lh * v3 + f->lh * v4);
    sh += g * (-f->hw * v1 - f->lw * v2 + f->hw * v3 + f->lw * v4);
    sv += g * (f->w1 * v1 + f->w2 * v2 + f->w3 * v3 + f->w4 * v4);
  }
  *d_w = sw;
  *d_h = sh;
  *d_val = sv;
}

/* ------------------------------------------------------------------ DCNv4 */

typedef struct {
  int N, H, W, G, D, kh, kw, sh, sw, ph, pw, dh, dw;
  float offset_scale;
  int remove_center, padded_offset_dim, softmax;
} dcn_params_t;

static int dcn_points(const dcn_params_t *p) {
  return p->kh * p->kw - (p->remove_center ? 1 : 0);
}

/*
 * value       (N,H,W,G*D) float32
 * offset_mask (N,Ho,Wo,Ppad) float32, per group [x0,y0,...,x(K-1),y(K-1),m0..m(K-1)]
 * out         (N,Ho,Wo,G*D) float64
 * corners     optional (N,Ho,Wo,G,K,2) int32: (h_low,w_low) of every point, or
 *             ORACLE_SKIPPED for a point that failed the range test.
 */
int oracle_dcnv4_forward(const float *value, const float *offset_mask,
                         double *out, int32_t *corners, int N, int H, int W,
                         int G, int D, int kh, int kw, int sh, int sw, int ph,
                         int pw, int dh, int dw, float offset_scale,
                         int remove_center, int padded_offset_dim,
                         int softmax) {
  dcn_params_t P = {N, H, W, G, D, kh, kw, sh, sw, ph, pw, dh, dw,
                    offset_scale, remove_center, padded_offset_dim, softmax};
  const int K = dcn_points(&P);
  const int Ho = oracle_dcnv4_out_size(H, ph, dh, kh, sh);
  const int Wo = oracle_dcnv4_out_size(W, pw, dw, kw, sw);
  const int C = G * D;
  if (K <= 0 || Ho <= 0 || Wo <= 0 || padded_offset_dim < 3 * K * G) return -1;
  const int cw = (dw * (kw - 1)) >> 1, ch = (dh * (kh - 1)) >> 1;
  const int center_h = kh / 2, center_w = kw / 2;

#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < N; ++b) {
    for (int y = 0; y < Ho; ++y) {
      double *mk = (double *)malloc(sizeof(double) * (size_t)K);
      for (int x = 0; x < Wo; ++x) {
        const size_t q = ((size_t)b * Ho + y) * Wo + x;
        const float base_w = dcn_base(cw - pw + x * sw, cw, offset_scale);
        const float base_h = dcn_base(ch - ph + y * sh, ch, offset_scale);
        for (int g = 0; g < G; ++g) {
          const float *row = offset_mask + q * padded_offset_dim + (size_t)g * 3 * K;
          const float *img = value + (size_t)b * H * W * C + (size_t)g * D;
          double *o = out + q * C + (size_t)g * D;
          for (int c = 0; c < D; ++c) o[c] = 0.0;
          if (softmax) {
            softmax_f64(row + 2 * K, K, mk);
          } else {
            for (int k = 0; k < K; ++k) mk[k] = (double)row[2 * K + k];
          }
          int k = 0;
          for (int i = 0; i < kw; ++i) {
            for (int j = 0; j < kh; ++j) {
              if (remove_center && i == center_w && j == center_h) continue;
              const float w_im = dcn_coord(base_w, i * dw, row[2 * k], offset_scale);
              const float h_im = dcn_coord(base_h, j * dh, row[2 * k + 1], offset_scale);
              int32_t *cr = corners ? corners + ((q * G + g) * K + k) * 2 : NULL;
              if (in_range(h_im, w_im, H, W)) {
                footprint_t f = footprint(h_im, w_im);
                gather_point(img, H, W, C, D, &f, mk[k], o);
                if (cr) { cr[0] = f.h_low; cr[1] = f.w_low; }
              } else if (cr) {
                cr[0] = ORACLE_SKIPPED; cr[1] = ORACLE_SKIPPED;
              }
              ++k;
            }
          }
        }
      }
      free(mk);
    }
  }
  return 0;
}

/*
 * grad_out         (N,Ho,Wo,G*D) float32
 * grad_value       (N,H,W,G*D) float64   (overwritten)
 * grad_offset_mask (N,Ho,Wo,Ppad) float64 (overwritten; pad columns are 0)
 */
int oracle_dcnv4_backward(const float *value, const float *offset_mask,
                          const float *grad_out, double *grad_value,
                          double *grad_offset_mask, int N, int H, int W, int G,
                          int D, int kh, int kw, int sh, int sw, int ph, int pw,
                          int dh, int dw, float offset_scale, int remove_center,
                          int padded_offset_dim, int softmax) {
  dcn_params_t P = {N, H, W, G, D, kh, kw, sh, sw, ph, pw, dh, dw,
                    offset_scale, remove_center, padded_offset_dim, softmax};
  const int K = dcn_points(&P);
  const int Ho = oracle_dcnv4_out_size(H, ph, dh, kh, sh);
  const int Wo = oracle_dcnv4_out_size(W, pw, dw, kw, sw);
  const int C = G * D;
  if (K <= 0 || Ho <= 0 || Wo <= 0 || padded_offset_dim < 3 * K * G) return -1;
  const int cw = (dw * (kw - 1)) >> 1, ch = (dh * (kh - 1)) >> 1;
  const int center_h = kh / 2, center_w = kw / 2;
  memset(grad_value, 0, sizeof(double) * (size_t)N * H * W * C);
  memset(grad_offset_mask, 0, sizeof(double) * (size_t)N * Ho * Wo * padded_offset_dim);

  /* One thread per image: the scatter into grad_value never crosses images
   * (dcnv4_col2im_cuda.cuh:287), so no atomics are needed. */
#pragma omp parallel for schedule(dynamic)
  for (int b = 0; b < N; ++b) {
    double *mk = (double *)malloc(sizeof(double) * (size_t)K);
    double *tk = (double *)malloc(sizeof(double) * (size_t)K);
    for (int y = 0; y < Ho; ++y) {
      for (int x = 0; x < Wo; ++x) {
        const size_t q = ((size_t)b * Ho + y) * Wo + x;
        const float base_w = dcn_base(cw - pw + x * sw, cw, offset_scale);
        const float base_h = dcn_base(ch - ph + y * sh, ch, offset_scale);
        for (int g = 0; g < G; ++g) {
          const float *row = offset_mask + q * padded_offset_dim + (size_t)g * 3 * K;
          double *grow = grad_offset_mask + q * padded_offset_dim + (size_t)g * 3 * K;
          const float *img = value + (size_t)b * H * W * C + (size_t)g * D;
          double *gimg = grad_value + (size_t)b * H * W * C + (size_t)g * D;
          const float *go = grad_out + q * C + (size_t)g * D;
          if (softmax) {
            softmax_f64(row + 2 * K, K, mk);
          } else {
            for (int k = 0; k < K; ++k) mk[k] = (double)row[2 * K + k];
          }
          int k = 0;
          for (int i = 0; i < kw; ++i) {
            for (int j = 0; j < kh; ++j) {
              if (remove_center && i == center_w && j == center_h) continue;
              const float w_im = dcn_coord(base_w, i * dw, row[2 * k], offset_scale);
              const float h_im = dcn_coord(base_h, j * dh, row[2 * k + 1], offset_scale);
              double d_w = 0, d_h = 0, d_v = 0;
              if (in_range(h_im, w_im, H, W)) {
                footprint_t f = footprint(h_im, w_im);
                scatter_point(img, gimg, H, W, C, D, &f, mk[k], go, &d_w, &d_h, &d_v);
              }
              grow[2 * k] = (double)offset_scale * mk[k] * d_w;
              grow[2 * k + 1] = (double)offset_scale * mk[k] * d_h;
              tk[k] = d_v;
              ++k;
            }
          }
          if (softmax) { /* dcnv4_col2im_cuda.cuh:352-365 */
            double sum = 0.0;
            for (int t = 0; t < K; ++t) sum += tk[t] * mk[t];
            for (int t = 0; t < K; ++t) grow[2 * K + t] = tk[t] * mk[t] - mk[t] * sum;
          } else {
            for (int t = 0; t < K; ++t) grow[2 * K + t] = tk[t];
          }
        }
      }
    }
    free(mk);
    free(tk);
  }
  return 0;
}

/* -------------------------------------------------------- FlashDeformAttn */

/*
 * value             (B,Len_in,G,D) float32
 * spatial_shapes    (L,2) int64 (H_l,W_l); level_start (L) int64
 * sampling_loc_attn (B,Len_q,G,3*L*K) float32: [x,y] x (L*K) level-major, then L*K logits
 * out               (B,Len_q,G*D) float64
 * corners           optional (B,Len_q,G,L*K,2) int32
 */
int oracle_fda_forward(const float *value, const int64_t *spatial_shapes,
                       const int64_t *level_start, const float *sampling_loc_attn,
                       double *out, int32_t *corners, int B, int Len_in, int G,
                       int D, int L, int Len_q, int K) {
  const int LK = L * K, C = G * D;
  if (LK <= 0) return -1;
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < B; ++b) {
    for (int qi = 0; qi < Len_q; ++qi) {
      double *p = (double *)malloc(sizeof(double) * (size_t)LK);
      const size_t q = (size_t)b * Len_q + qi;
      for (int g = 0; g < G; ++g) {
        const float *row = sampling_loc_attn + (q * G + g) * (size_t)(3 * LK);
        double *o = out + q * C + (size_t)g * D;
        for (int c = 0; c < D; ++c) o[c] = 0.0;
        softmax_f64(row + 2 * LK, LK, p);
        for (int l = 0; l < L; ++l) {
          const int Hl = (int)spatial_shapes[2 * l], Wl = (int)spatial_shapes[2 * l + 1];
          const float *img = value + ((size_t)b * Len_in + (size_t)level_start[l]) * C + (size_t)g * D;
          for (int k = 0; k < K; ++k) {
            const int t = l * K + k;
            const float w_im = fda_coord(row[2 * t], Wl);
            const float h_im = fda_coord(row[2 * t + 1], Hl);
            int32_t *cr = corners ? corners + ((q * G + g) * LK + t) * 2 : NULL;
            if (in_range(h_im, w_im, Hl, Wl)) {
              footprint_t f = footprint(h_im, w_im);
              gather_point(img, Hl, Wl, C, D, &f, p[t], o);
              if (cr) { cr[0] = f.h_low; cr[1] = f.w_low; }
            } else if (cr) {
              cr[0] = ORACLE_SKIPPED; cr[1] = ORACLE_SKIPPED;
            }
          }
        }
      }
      free(p);
    }
  }
  return 0;
}

/*
 * grad_out  (B,Len_q,G*D) float32
 * grad_value (B,Len_in,G,D) float64; grad_sampling_loc_attn like sampling_loc_attn, float64.
 * Points that fail the range test contribute exactly zero to every gradient
 * (the reference reads an unwritten shared-memory slot for them,
 * flash_deform_col2im_cuda.cuh:272-316; zero is the mathematical value).
 */
int oracle_fda_backward(const float *value, const int64_t *spatial_shapes,
                        const int64_t *level_start, const float *sampling_loc_attn,
                        const float *grad_out, double *grad_value,
                        double *grad_sampling_loc_attn, int B, int Len_in, int G,
                        int D, int L, int Len_q, int K) {
  const int LK = L * K, C = G * D;
  if (LK <= 0) return -1;
  memset(grad_value, 0, sizeof(double) * (size_t)B * Len_in * C);
  memset(grad_sampling_loc_attn, 0, sizeof(double) * (size_t)B * Len_q * G * 3 * LK);
#pragma omp parallel for schedule(dynamic)
  for (int b = 0; b < B; ++b) {
    double *p = (double *)malloc(sizeof(double) * (size_t)LK);
    double *gv = (double *)malloc(sizeof(double) * (size_t)LK);
    for (int qi = 0; qi < Len_q; ++qi) {
      const size_t q = (size_t)b * Len_q + qi;
      for (int g = 0; g < G; ++g) {
        const float *row = sampling_loc_attn + (q * G + g) * (size_t)(3 * LK);
        double *grow = grad_sampling_loc_attn + (q * G + g) * (size_t)(3 * LK);
        const float *go = grad_out + q * C + (size_t)g * D;
        softmax_f64(row + 2 * LK, LK, p);
        for (int l = 0; l < L; ++l) {
          const int Hl = (int)spatial_shapes[2 * l], Wl = (int)spatial_shapes[2 * l + 1];
          const size_t base = ((size_t)b * Len_in + (size_t)level_start[l]) * C + (size_t)g * D;
          for (int k = 0; k < K; ++k) {
            const int t = l * K + k;
            const float w_im = fda_coord(row[2 * t], Wl);
            const float h_im = fda_coord(row[2 * t + 1], Hl);
            double d_w = 0, d_h = 0, d_v = 0;
            if (in_range(h_im, w_im, Hl, Wl)) {
              footprint_t f = footprint(h_im, w_im);
              scatter_point(value + base, grad_value + base, Hl, Wl, C, D, &f, p[t], go, &d_w, &d_h, &d_v);
            }
            grow[2 * t] = (double)Wl * p[t] * d_w;     /* flash_deform_col2im_cuda.cuh:273-276 */
            grow[2 * t + 1] = (double)Hl * p[t] * d_h;
            gv[t] = d_v;
          }
        }
        /* softmax Jacobian, flash_deform_col2im_cuda.cuh:301-316:
         * g_i p_i (1-p_i) - sum_{j!=i} g_j p_i p_j = p_i (g_i - sum_j g_j p_j) */
        double dot = 0.0;
        for (int t = 0; t < LK; ++t) dot += gv[t] * p[t];
        for (int t = 0; t < LK; ++t) grow[2 * LK + t] = p[t] * (gv[t] - dot);
      }
    }
    free(p);
    free(gv);
  }
  return 0;
}

int oracle_abi_version(void) { return 1; }
