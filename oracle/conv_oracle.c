/* TEST INFRASTRUCTURE — not part of the product.
 *
 * Plain-C restatement of the CPU algorithm of the reference's convolution hot path (type-1 lowering + three
 * GEMMs + inverse lowering + bias), written from the reference's behaviour; each function names the reference
 * location it follows (paths inside the reference project).  Parity status: PINNED — tests/test_oracle.py
 * checks this file against the reference's own golden files (tests/input, tests/output of the reference tree,
 * when that tree is mounted) and against outputs of the reference's compiled CPU code (oracle/_ref, and the
 * fixtures under tests/golden/ generated from it).
 *
 * Only tests, the smoke check and the CPU-baseline leg of the benchmark may load this library.
 *
 * All tensors are fp32, NCHW ("c fastest, then r, d, b": src/LogicalCube_impl.hxx:217-219).  `acc64` selects
 * double accumulators inside the GEMMs (a truth estimate used to put error bars on fp32 results); the reference
 * itself accumulates in fp32 inside its BLAS.
 */
#include <float.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

static int out_size(int n, int k, int s, int p) { return (n + 2 * p - k) / s + 1; } /* src/DeepNet.h:112-115 */

/* Type-1 lowering, eq. 4 of docs/lowering/type_1/type_1_lowering_pad_stride.tex:103-109 and the plain loop at
 * src/sched/DeviceDriver_CPU.cpp:263-299:
 *   Dhat[b*m*m + r*m + c][d*k*k + kr*k + kc] = X[b][d][r*s-p+kr][c*s-p+kc], zero outside the image. */
void oracle_lower_type1(const float* X, float* Dhat, int B, int D, int n, int k, int s, int p) {
  const int m = out_size(n, k, s, p);
  const size_t K = (size_t)k * k * D;
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < B; ++b)
    for (int r = 0; r < m; ++r)
      for (int c = 0; c < m; ++c) {
        float* row = Dhat + ((size_t)b * m * m + (size_t)r * m + c) * K;
        for (int d = 0; d < D; ++d)
          for (int kr = 0; kr < k; ++kr)
            for (int kc = 0; kc < k; ++kc) {
              const int y = r * s - p + kr, x = c * s - p + kc;
              const int inside = y >= 0 && y < n && x >= 0 && x < n;
              row[(size_t)d * k * k + kr * k + kc] = inside ? X[(((size_t)b * D + d) * n + y) * n + x] : 0.0f;
            }
      }
}

/* C[i][j] (row pitch ldc) = sum_l A(i,l) * B(l,j) with arbitrary element strides: A(i,l) = A[i*a_rs + l*a_cs],
 * B(l,j) = Bm[l*b_rs + j*b_cs].  Covers the three operand arrangements the reference's GEMM wrapper selects
 * (src/Kernel_impl.hxx:124-155) without a BLAS. */
void oracle_gemm(int M, int N, int K, const float* A, size_t a_rs, size_t a_cs, const float* Bm, size_t b_rs,
                 size_t b_cs, float* C, size_t ldc, int acc64) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < M; ++i) {
    for (int j = 0; j < N; ++j) {
      if (acc64) {
        double acc = 0.0;
        for (int l = 0; l < K; ++l) acc += (double)A[i * a_rs + l * a_cs] * (double)Bm[l * b_rs + j * b_cs];
        C[i * ldc + j] = (float)acc;
      } else {
        float acc = 0.0f;
        for (int l = 0; l < K; ++l) acc += A[i * a_rs + l * a_cs] * Bm[l * b_rs + j * b_cs];
        C[i * ldc + j] = acc;
      }
    }
  }
}

/* Plane permutation [outer][inner][plane] -> [inner][outer][plane], the effect of Connector::remap_output
 * (src/Connector_impl_Lowering_type1.hxx:92-128, src/kernels/lowering.hxx:241-258), done through a copy. */
void oracle_remap(float* T, int outer, int inner, int plane) {
  const size_t total = (size_t)outer * inner * plane;
  float* tmp = (float*)malloc(total * sizeof(float));
  memcpy(tmp, T, total * sizeof(float));
  for (int a = 0; a < outer; ++a)
    for (int b = 0; b < inner; ++b)
      memcpy(T + ((size_t)b * outer + a) * plane, tmp + ((size_t)a * inner + b) * plane, plane * sizeof(float));
  free(tmp);
}

/* Inverse lowering (col2im scatter-add), src/Connector_impl_Lowering_type1.hxx:156 (zero first) and
 * src/sched/DeviceDriver_CPU.cpp:322-345 (loop order d, b, kr, cr, kc, cc; fp32 "+=" in that order):
 *   dX[b][d][cr*s+kr-p][cc*s+kc-p] += G[d*k*k + kr*k + kc][b*m*m + cr*m + cc]. */
void oracle_inverse_lower(const float* G, float* dX, int B, int D, int n, int k, int s, int p) {
  const int m = out_size(n, k, s, p);
  const size_t cols = (size_t)m * m * B;
  memset(dX, 0, sizeof(float) * (size_t)B * D * n * n);
  for (int d = 0; d < D; ++d)
    for (int b = 0; b < B; ++b)
      for (int kr = 0; kr < k; ++kr)
        for (int cr = 0; cr < m; ++cr)
          for (int kc = 0; kc < k; ++kc)
            for (int cc = 0; cc < m; ++cc) {
              const int y = cr * s + kr - p, x = cc * s + kc - p;
              if (y >= 0 && y < n && x >= 0 && x < n)
                dX[(((size_t)b * D + d) * n + y) * n + x] +=
                    G[((size_t)d * k * k + kr * k + kc) * cols + (size_t)b * m * m + (size_t)cr * m + cc];
            }
}

/* One group-less convolution forward exactly as ConvolutionBridge<CPUDriver>::forward does it
 * (src/bridges/ConvolutionBridge_impl.hxx:294-373): lower, Y' = W * Dhat^T laid out [o][b][pix]
 * (src/Kernel_impl.hxx:132-139), remap to [b][o][pix], add bias per plane (src/kernels/conv.hxx:10-26). */
static void conv_forward_1g(const float* X, const float* W, const float* bias, float* Y, int B, int D, int n, int o,
                            int k, int s, int p, int acc64) {
  const int m = out_size(n, k, s, p);
  const size_t K = (size_t)k * k * D, P = (size_t)m * m * B;
  float* Dhat = (float*)malloc(P * K * sizeof(float));
  oracle_lower_type1(X, Dhat, B, D, n, k, s, p);
  oracle_gemm(o, (int)P, (int)K, W, K, 1, Dhat, 1, K, Y, P, acc64);
  oracle_remap(Y, o, B, m * m);
  if (bias)
    for (int b = 0; b < B; ++b)
      for (int f = 0; f < o; ++f) {
        float* plane = Y + ((size_t)b * o + f) * m * m;
        for (int i = 0; i < m * m; ++i) plane[i] += bias[f];
      }
  free(Dhat);
}

/* One group-less backward as ConvolutionBridge<CPUDriver>::backward (src/bridges/ConvolutionBridge_impl.hxx:551-628):
 * db from plane sums added in (b, o) memory order (src/kernels/conv.hxx:31-49), dY permuted to [o][b][pix] (:604),
 * G = W^T * dY' then inverse lowering (:610-613), dW = dY' * Dhat with beta = 0 (:619-621).  The caller's dY is
 * left untouched here (the reference permutes it in place). */
static void conv_backward_1g(const float* X, const float* W, const float* dY, float* dX, float* dW, float* db, int B,
                             int D, int n, int o, int k, int s, int p, int acc64) {
  const int m = out_size(n, k, s, p);
  const size_t K = (size_t)k * k * D, P = (size_t)m * m * B;
  if (db) {
    for (int f = 0; f < o; ++f) db[f] = 0.0f;
    for (int b = 0; b < B; ++b)
      for (int f = 0; f < o; ++f) {
        const float* plane = dY + ((size_t)b * o + f) * m * m;
        float sum = 0.0f;
        for (int i = 0; i < m * m; ++i) sum += plane[i];
        db[f] += sum;
      }
  }
  float* dYp = (float*)malloc(P * o * sizeof(float));
  memcpy(dYp, dY, P * o * sizeof(float));
  oracle_remap(dYp, B, o, m * m);
  if (dX) {
    float* G = (float*)malloc(K * P * sizeof(float));
    oracle_gemm((int)K, (int)P, o, W, 1, K, dYp, P, 1, G, P, acc64);
    oracle_inverse_lower(G, dX, B, D, n, k, s, p);
    free(G);
  }
  float* Dhat = (float*)malloc(P * K * sizeof(float));
  oracle_lower_type1(X, Dhat, B, D, n, k, s, p);
  oracle_gemm(o, (int)K, (int)P, dYp, P, 1, Dhat, K, 1, dW, K, acc64);
  free(Dhat);
  free(dYp);
}

/* Channel-slice helpers for grouped layers.  The reference bridge has no group concept (src/DeepNet.h:1075-1077
 * warns and ignores it); a grouped layer is the same bridge applied to each channel slice, which is what these do. */
static void take_channels(const float* T, float* S, int B, int C, int c0, int cn, size_t plane) {
  for (int b = 0; b < B; ++b)
    memcpy(S + (size_t)b * cn * plane, T + ((size_t)b * C + c0) * plane, (size_t)cn * plane * sizeof(float));
}
static void put_channels(float* T, const float* S, int B, int C, int c0, int cn, size_t plane) {
  for (int b = 0; b < B; ++b)
    memcpy(T + ((size_t)b * C + c0) * plane, S + (size_t)b * cn * plane, (size_t)cn * plane * sizeof(float));
}

void oracle_conv_forward(const float* X, const float* W, const float* bias, float* Y, int B, int D, int n, int o,
                         int k, int s, int p, int g, int acc64) {
  if (g == 1) { conv_forward_1g(X, W, bias, Y, B, D, n, o, k, s, p, acc64); return; }
  const int m = out_size(n, k, s, p), Dg = D / g, og = o / g;
  float* Xs = (float*)malloc(sizeof(float) * (size_t)B * Dg * n * n);
  float* Ys = (float*)malloc(sizeof(float) * (size_t)B * og * m * m);
  for (int gi = 0; gi < g; ++gi) {
    take_channels(X, Xs, B, D, gi * Dg, Dg, (size_t)n * n);
    conv_forward_1g(Xs, W + (size_t)gi * og * Dg * k * k, bias ? bias + gi * og : NULL, Ys, B, Dg, n, og, k, s, p, acc64);
    put_channels(Y, Ys, B, o, gi * og, og, (size_t)m * m);
  }
  free(Xs); free(Ys);
}

void oracle_conv_backward(const float* X, const float* W, const float* dY, float* dX, float* dW, float* db, int B,
                          int D, int n, int o, int k, int s, int p, int g, int acc64) {
  if (g == 1) { conv_backward_1g(X, W, dY, dX, dW, db, B, D, n, o, k, s, p, acc64); return; }
  const int m = out_size(n, k, s, p), Dg = D / g, og = o / g;
  float* Xs = (float*)malloc(sizeof(float) * (size_t)B * Dg * n * n);
  float* dXs = dX ? (float*)malloc(sizeof(float) * (size_t)B * Dg * n * n) : NULL;
  float* dYs = (float*)malloc(sizeof(float) * (size_t)B * og * m * m);
  for (int gi = 0; gi < g; ++gi) {
    take_channels(X, Xs, B, D, gi * Dg, Dg, (size_t)n * n);
    take_channels(dY, dYs, B, o, gi * og, og, (size_t)m * m);
    conv_backward_1g(Xs, W + (size_t)gi * og * Dg * k * k, dYs, dXs, dW + (size_t)gi * og * Dg * k * k,
                     db ? db + gi * og : NULL, B, Dg, n, og, k, s, p, acc64);
    if (dX) put_channels(dX, dXs, B, D, gi * Dg, Dg, (size_t)n * n);
  }
  free(Xs); free(dXs); free(dYs);
}

/* Max pooling forward, src/bridges/MaxPoolingBridge_impl.hxx:60-84 (output starts at -FLT_MAX, index cube at 0,
 * output size by floor) and src/sched/DeviceDriver_CPU.cpp:369-400: scan rows then columns, strict '>', so the
 * first maximum wins; windows are clipped at the bottom/right border, there is no padding.  idx is the int32
 * offset h*n+w inside the (n x n) input plane. */
void oracle_maxpool_forward(const float* X, float* Y, int* idx, int planes, int n, int k, int s) {
  const int m = (n - k) / s + 1;
#pragma omp parallel for schedule(static)
  for (int i = 0; i < planes; ++i) {
    const float* in = X + (size_t)i * n * n;
    float* out = Y + (size_t)i * m * m;
    int* ix = idx + (size_t)i * m * m;
    for (int ph = 0; ph < m; ++ph)
      for (int pw = 0; pw < m; ++pw) {
        float best = -FLT_MAX;
        int where = 0;
        const int he = ph * s + k < n ? ph * s + k : n, we = pw * s + k < n ? pw * s + k : n;
        for (int h = ph * s; h < he; ++h)
          for (int w = pw * s; w < we; ++w)
            if (in[h * n + w] > best) { best = in[h * n + w]; where = h * n + w; }
        out[ph * m + pw] = best;
        ix[ph * m + pw] = where;
      }
  }
}

/* Max pooling backward, src/bridges/MaxPoolingBridge_impl.hxx:118 (zero fill) and
 * src/sched/DeviceDriver_CPU.cpp:402-421: dX[plane][idx] += dY, windows visited in (ph, pw) order. */
void oracle_maxpool_backward(const float* dY, const int* idx, float* dX, int planes, int n, int m) {
  memset(dX, 0, sizeof(float) * (size_t)planes * n * n);
  for (int i = 0; i < planes; ++i)
    for (int j = 0; j < m * m; ++j) dX[(size_t)i * n * n + idx[(size_t)i * m * m + j]] += dY[(size_t)i * m * m + j];
}

/* ReLU, src/kernels/relu.hxx:17-43: y = max(x, 0); dx = dy * (x > 0). */
void oracle_relu_forward(const float* X, float* Y, size_t count) {
  for (size_t i = 0; i < count; ++i) Y[i] = X[i] > 0.0f ? X[i] : 0.0f;
}
void oracle_relu_backward(const float* X, const float* dY, float* dX, size_t count) {
  for (size_t i = 0; i < count; ++i) dX[i] = dY[i] * (float)(X[i] > 0.0f);
}

/* Learning-rate policies of src/util.h:76-100 (policy: 0 fixed, 1 step, 2 exp, 3 inv, 4 poly, 5 sigmoid).
 * The reference evaluates them with float arguments and a float result. */
float oracle_learning_rate(int policy, float base_lr, float gamma, float iter, float stepsize, float power,
                           float max_iter) {
  switch (policy) {
    case 0: return base_lr;
    case 1: return (float)(base_lr * pow(gamma, (double)(int)(iter / stepsize)));
    case 2: return (float)(base_lr * pow(gamma, iter));
    case 3: return (float)(base_lr * pow(1.0 + gamma * iter, -power));
    case 4: return (float)(base_lr * pow(1.0 - (iter / max_iter), power));
    case 5: return (float)(base_lr * (1.0 / (1.0 + exp(-gamma * (iter - stepsize)))));
    default: return NAN;
  }
}

/* SGD with momentum and L2 decay, src/algorithms/GradientUpdater.h:154-193, as three BLAS-1 steps in fp32:
 *   g += lambda * w   (only when lambda != 0; modifies the gradient buffer as the reference does)
 *   h  = lr * g + momentum * h
 *   w -= h */
void oracle_sgd_update(size_t count, float* w, float* g, float* h, float lr, float momentum, float lambda) {
  if (lambda != 0.0f)
    for (size_t i = 0; i < count; ++i) g[i] += lambda * w[i];
  for (size_t i = 0; i < count; ++i) h[i] = lr * g[i] + momentum * h[i];
  for (size_t i = 0; i < count; ++i) w[i] += -1.0f * h[i];
}
