/*
 * Independent double-precision restatement of the triangle multiplicative update forward pass.
 * TEST INFRASTRUCTURE ONLY: built into oracle/_build/libtrimul_ref.so by oracle/Makefile and used by
 * the CPU tests to cross-check oracle/trimul_oracle.py. PARITY UNPINNED: the reference module's source
 * (miniworld-engine 2.4.4, pyproject.toml:105 of the reference project) is not in the reference tree;
 * this follows docs/paper/supplement.tex:100-117 and
 * docs/archive/trimul-fusion/history/initial-triton.py:11-26,84-104 of that project:
 *
 *   x      = LayerNorm_in(z)                       over the channel dimension, biased variance
 *   left   = sigmoid(x Wlg^T) * (x Wl^T) * m_ik    (mask on left/right only)
 *   right  = sigmoid(x Wrg^T) * (x Wr^T) * m_ik
 *   tri_ij = sum_k left_ik * right_jk              (outgoing)   |   sum_k left_ki * right_kj  (incoming)
 *   out    = z + sigmoid(x Wg^T) * (LayerNorm_out(tri) Wo^T)    (gate unmasked, output unmasked)
 *
 * Plain loops, one sample at a time; meant for N <= 64.
 */
#include <math.h>
#include <stdlib.h>

static void layer_norm(const double* v, int n, const double* g, const double* b, double eps, double* out) {
  double mean = 0.0, var = 0.0;
  for (int i = 0; i < n; ++i) mean += v[i];
  mean /= n;
  for (int i = 0; i < n; ++i) var += (v[i] - mean) * (v[i] - mean);
  var /= n;
  const double rstd = 1.0 / sqrt(var + eps);
  for (int i = 0; i < n; ++i) out[i] = (v[i] - mean) * rstd * g[i] + b[i];
}

static double dot(const double* a, const double* b, int n) {
  double s = 0.0;
  for (int i = 0; i < n; ++i) s += a[i] * b[i];
  return s;
}

static double sigmoid(double x) { return 1.0 / (1.0 + exp(-x)); }

/*
 * z, out: [N, N, C]; pair_valid: [N, N] (1 = valid) or NULL; weights row-major [out_features, in_features];
 * returns 0 on success.
 */
int trimul_ref_forward(const double* z, const unsigned char* pair_valid, const double* ln_in_w, const double* ln_in_b,
                       const double* w_left, const double* w_left_gate, const double* w_right,
                       const double* w_right_gate, const double* ln_out_w, const double* ln_out_b,
                       const double* w_gate, const double* w_out, int N, int C, int H, int outgoing, double eps_in,
                       double eps_out, int residual, double* out) {
  const size_t cells = (size_t)N * N;
  double* x = (double*)malloc(cells * C * sizeof(double));
  double* left = (double*)malloc(cells * H * sizeof(double));
  double* right = (double*)malloc(cells * H * sizeof(double));
  double* tri = (double*)malloc(H * sizeof(double));
  double* tn = (double*)malloc(H * sizeof(double));
  if (!x || !left || !right || !tri || !tn) return -1;
  for (size_t p = 0; p < cells; ++p) {
    layer_norm(z + p * C, C, ln_in_w, ln_in_b, eps_in, x + p * C);
    const double m = (pair_valid == NULL || pair_valid[p]) ? 1.0 : 0.0;
    for (int h = 0; h < H; ++h) {
      left[p * H + h] = sigmoid(dot(x + p * C, w_left_gate + (size_t)h * C, C)) * dot(x + p * C, w_left + (size_t)h * C, C) * m;
      right[p * H + h] = sigmoid(dot(x + p * C, w_right_gate + (size_t)h * C, C)) * dot(x + p * C, w_right + (size_t)h * C, C) * m;
    }
  }
  for (int i = 0; i < N; ++i) {
    for (int j = 0; j < N; ++j) {
      for (int h = 0; h < H; ++h) {
        double s = 0.0;
        for (int k = 0; k < N; ++k) {
          if (outgoing)
            s += left[((size_t)i * N + k) * H + h] * right[((size_t)j * N + k) * H + h];
          else
            s += left[((size_t)k * N + i) * H + h] * right[((size_t)k * N + j) * H + h];
        }
        tri[h] = s;
      }
      layer_norm(tri, H, ln_out_w, ln_out_b, eps_out, tn);
      const size_t p = (size_t)i * N + j;
      for (int c = 0; c < C; ++c) {
        const double upd = sigmoid(dot(x + p * C, w_gate + (size_t)c * C, C)) * dot(tn, w_out + (size_t)c * H, H);
        out[p * C + c] = (residual ? z[p * C + c] : 0.0) + upd;
      }
    }
  }
  free(x);
  free(left);
  free(right);
  free(tri);
  free(tn);
  return 0;
}

/*
 * Bidirectional form (docs/paper/supplement.tex:125-136 of the reference project): one input LayerNorm, l and r of
 * width 2h from [2h, C] matrices; channels 0..h-1 contracted outgoing, h..2h-1 incoming; one LayerNorm over the 2h
 * contracted channels, w_out [C, 2h], one gate [C, C], residual. drop_scale: [N, C] (shared by all rows i) or NULL.
 */
int trimul_ref_bidir_forward(const double* z, const unsigned char* pair_valid, const double* ln_in_w,
                             const double* ln_in_b, const double* w_left, const double* w_left_gate,
                             const double* w_right, const double* w_right_gate, const double* ln_out_w,
                             const double* ln_out_b, const double* w_gate, const double* w_out,
                             const double* drop_scale, int N, int C, int h, double eps_in, double eps_out,
                             int residual, double* out) {
  const int H2 = 2 * h;
  const size_t cells = (size_t)N * N;
  double* x = (double*)malloc(cells * C * sizeof(double));
  double* left = (double*)malloc(cells * H2 * sizeof(double));
  double* right = (double*)malloc(cells * H2 * sizeof(double));
  double* tri = (double*)malloc(H2 * sizeof(double));
  double* tn = (double*)malloc(H2 * sizeof(double));
  if (!x || !left || !right || !tri || !tn) return -1;
  for (size_t p = 0; p < cells; ++p) {
    layer_norm(z + p * C, C, ln_in_w, ln_in_b, eps_in, x + p * C);
    const double m = (pair_valid == NULL || pair_valid[p]) ? 1.0 : 0.0;
    for (int c = 0; c < H2; ++c) {
      left[p * H2 + c] = sigmoid(dot(x + p * C, w_left_gate + (size_t)c * C, C)) * dot(x + p * C, w_left + (size_t)c * C, C) * m;
      right[p * H2 + c] = sigmoid(dot(x + p * C, w_right_gate + (size_t)c * C, C)) * dot(x + p * C, w_right + (size_t)c * C, C) * m;
    }
  }
  for (int i = 0; i < N; ++i) {
    for (int j = 0; j < N; ++j) {
      for (int c = 0; c < H2; ++c) {
        double s = 0.0;
        for (int k = 0; k < N; ++k) {
          if (c < h)
            s += left[((size_t)i * N + k) * H2 + c] * right[((size_t)j * N + k) * H2 + c];
          else
            s += left[((size_t)k * N + i) * H2 + c] * right[((size_t)k * N + j) * H2 + c];
        }
        tri[c] = s;
      }
      layer_norm(tri, H2, ln_out_w, ln_out_b, eps_out, tn);
      const size_t p = (size_t)i * N + j;
      for (int c = 0; c < C; ++c) {
        double upd = sigmoid(dot(x + p * C, w_gate + (size_t)c * C, C)) * dot(tn, w_out + (size_t)c * H2, H2);
        if (drop_scale != NULL) upd *= drop_scale[(size_t)j * C + c];
        out[p * C + c] = (residual ? z[p * C + c] : 0.0) + upd;
      }
    }
  }
  free(x);
  free(left);
  free(right);
  free(tri);
  free(tn);
  return 0;
}

/*
 * Pair Transition (src/miniworld/modules/mini_pairformer.py:81-84,108; parameter names
 * benchmarks/protenix_finetune/patch_engine.py:35-37 of the reference project):
 *   y = x + W_s ( SiLU(W_a LN(x)) * (W_b LN(x)) ),  W_a, W_b: [n*C, C], W_s: [C, n*C], no biases.
 * x, out: [rows, C].
 */
int transition_ref_forward(const double* x, const double* ln_w, const double* ln_b, const double* w_a,
                           const double* w_b, const double* w_s, long rows, int C, int hidden, double eps,
                           int residual, double* out) {
  double* xn = (double*)malloc((size_t)C * sizeof(double));
  double* hdn = (double*)malloc((size_t)hidden * sizeof(double));
  if (!xn || !hdn) return -1;
  for (long r = 0; r < rows; ++r) {
    layer_norm(x + (size_t)r * C, C, ln_w, ln_b, eps, xn);
    for (int k = 0; k < hidden; ++k) {
      const double a = dot(xn, w_a + (size_t)k * C, C);
      hdn[k] = a * sigmoid(a) * dot(xn, w_b + (size_t)k * C, C);
    }
    for (int c = 0; c < C; ++c)
      out[(size_t)r * C + c] = (residual ? x[(size_t)r * C + c] : 0.0) + dot(hdn, w_s + (size_t)c * hidden, hidden);
  }
  free(xn);
  free(hdn);
  return 0;
}
