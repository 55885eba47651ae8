/*
 * TEST INFRASTRUCTURE -- CPU restatement ("port") of the reference algorithms
 * on the hot path.  Nothing in the product library links or calls this file;
 * only tests/, the smoke check and the bench's CPU-baseline leg load it.
 *
 * Parity status: PINNED.  Every function here is checked bit-for-bit against
 * the reference's own exocc-generated C (compiled from the reference's golden
 * test outputs by oracle/build_ref.py) and against fixtures generated from it
 * (tests/golden/), see tests/test_oracle.py.  One sub-step is pinned by this
 * project's specification rather than by the reference: the rounding inside
 * ACC_SCALE (round-half-even), because that macro lives in a third-party
 * header (exo-lang/gemmini-rocc-tests @ exo-v3) that is not vendored in the
 * reference and whose own tests only use integral scales.
 *
 * Citations are paths inside the exo-lang/exo checkout.
 *
 * Build: gcc -O3 -fPIC -shared -fopenmp -mfma -mavx2 exo_oracle.c -o libexo_oracle.so -lm
 * (GNU mode; every multiply-add below is an explicit fmaf so the result does
 * not depend on -ffp-contract.)
 */
#include <math.h>
#include <stdbool.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static int g_threads = 1;

/* Number of OpenMP threads used by the row-parallel loops (default 1 so that
 * a timed "1 core" figure means one core). */
void oracle_set_threads(int n) { g_threads = n < 1 ? 1 : n; }
int oracle_get_threads(void) { return g_threads; }

/* ------------------------------------------------------------------ SGEMM
 * apps/x86/sgemm/sgemm.py:11-23:  C[i,j] += A[i,k] * B[k,j].
 * The generated microkernels (tests/golden/test_apps/test_x86_sgemm.txt:425-461)
 * use _mm512_fmadd_ps with k ascending and reload the fp32 partial between
 * k-blocks of 512 (:810), so each output element is ONE chain
 *     c = fmaf(A[i,k], B[k,j], c)   for k = 0 .. K-1, starting at the incoming C.
 * The loop nest below is blocked for cache but keeps that per-element order
 * (k-blocks ascending outside the row loop, k ascending inside). */
void oracle_sgemm(int64_t M, int64_t N, int64_t K, const float *A, const float *B, float *C) {
  const int64_t JB = 1024, KB = 128;
  for (int64_t j0 = 0; j0 < N; j0 += JB) {
    const int64_t j1 = j0 + JB < N ? j0 + JB : N;
    for (int64_t k0 = 0; k0 < K; k0 += KB) {
      const int64_t k1 = k0 + KB < K ? k0 + KB : K;
#pragma omp parallel for num_threads(g_threads) schedule(static)
      for (int64_t i = 0; i < M; i++) {
        float *c = C + i * N;
        for (int64_t k = k0; k < k1; k++) {
          const float a = A[i * K + k];
          const float *b = B + k * N;
          for (int64_t j = j0; j < j1; j++) c[j] = fmaf(a, b[j], c[j]);
        }
      }
    }
  }
}

/* Plain triple loop with the reduction innermost; the slow but obviously
 * correct statement of the same chain, used to check oracle_sgemm itself. */
void oracle_sgemm_naive(int64_t M, int64_t N, int64_t K, const float *A, const float *B, float *C) {
  for (int64_t i = 0; i < M; i++)
    for (int64_t j = 0; j < N; j++) {
      float c = C[i * N + j];
      for (int64_t k = 0; k < K; k++) c = fmaf(A[i * K + k], B[k * N + j], c);
      C[i * N + j] = c;
    }
}

/* ------------------------------------------------------------------ SSYRK
 * The reference holds no Exo procedure for SSYRK, only the comparison benchmark
 * apps/x86/ssyrk/bench_ssyrk.cpp:49-58: cblas_ssyrk(CblasRowMajor, CblasUpper,
 * CblasNoTrans, n, k, 1.0, a, k, 1.0, c, n), i.e.  C[i,j] += sum_k A[i,k] * A[j,k]
 * for j >= i; the strict lower triangle of C is not referenced.  The BLAS call does
 * not fix an accumulation order; this restatement (and the kernels checked against
 * it) use the order of the reference's SGEMM, one fmaf chain in increasing k that
 * starts from the incoming C -- parity for SSYRK is therefore pinned to
 * oracle_sgemm on (A, A^T), not to a reference kernel. */
void oracle_ssyrk(int64_t N, int64_t K, const float *A, float *C) {
#pragma omp parallel for num_threads(g_threads) schedule(dynamic, 8)
  for (int64_t i = 0; i < N; i++)
    for (int64_t j = i; j < N; j++) {
      float c = C[i * N + j];
      const float *a = A + i * K, *b = A + j * K;
      for (int64_t k = 0; k < K; k++) c = fmaf(a[k], b[k], c);
      C[i * N + j] = c;
    }
}

/* ------------------------------------------------------------------- conv
 * apps/x86/conv/conv.py:10-45: NHWC input, weights f32[Ci,Kh,Kw,Co], bias,
 * stride 1, no padding, ReLU via select(0, x, x, 0)  (= x > 0 ? x : 0).
 * Generated code (tests/golden/test_apps/test_x86_conv.txt:79-108): res starts
 * at bias, FMA chain in ky -> kx -> kc order, then _mm512_max_ps(res, 0).
 * Argument order follows conv.py:11-24. */
void oracle_conv(int64_t out_h, int64_t out_w, int64_t out_channel, int64_t in_h, int64_t in_w,
                 int64_t in_channel, int64_t kernel_dim, int64_t batch_size, const float *inp,
                 float *output, const float *weights, const float *bias) {
  (void)in_h;
#pragma omp parallel for num_threads(g_threads) collapse(2) schedule(static)
  for (int64_t n = 0; n < batch_size; n++)
    for (int64_t oy = 0; oy < out_h; oy++)
      for (int64_t ox = 0; ox < out_w; ox++) {
        float *o = output + ((n * out_h + oy) * out_w + ox) * out_channel;
        for (int64_t oc = 0; oc < out_channel; oc++) o[oc] = bias[oc];
        for (int64_t ky = 0; ky < kernel_dim; ky++)
          for (int64_t kx = 0; kx < kernel_dim; kx++)
            for (int64_t kc = 0; kc < in_channel; kc++) {
              const float x = inp[((n * in_h + oy + ky) * in_w + ox + kx) * in_channel + kc];
              const float *w = weights + ((kc * kernel_dim + ky) * kernel_dim + kx) * out_channel;
              for (int64_t oc = 0; oc < out_channel; oc++) o[oc] = fmaf(w[oc], x, o[oc]);
            }
        /* _mm512_max_ps(res, 0): returns the second operand (0) for NaN */
        for (int64_t oc = 0; oc < out_channel; oc++) o[oc] = o[oc] > 0.0f ? o[oc] : 0.0f;
      }
}

/* General NHWC convolution asked for by the conv configuration: weights in
 * Kh,Kw,Ci,Co order (the layout of apps/gemmini/src/exo/conv.py:17), square
 * kernel, stride 1, symmetric zero padding `pad`, optional ReLU.  The input is
 * treated as zero-extended: padded taps still go through fmaf(w, 0, acc), the
 * same arithmetic the reference performs when its caller pre-pads the input
 * (apps/gemmini/test/CMakeLists.txt:56-64 passes a 58x58 input for a 56x56
 * output).  Chain order ky -> kx -> ci as in conv.py:33-41. */
void oracle_conv_nhwc(int64_t batch, int64_t in_h, int64_t in_w, int64_t in_c, int64_t out_c,
                      int64_t kdim, int64_t pad, bool relu, const float *inp, float *output,
                      const float *weights, const float *bias) {
  const int64_t out_h = in_h + 2 * pad - kdim + 1, out_w = in_w + 2 * pad - kdim + 1;
#pragma omp parallel for num_threads(g_threads) collapse(2) schedule(static)
  for (int64_t n = 0; n < batch; n++)
    for (int64_t oy = 0; oy < out_h; oy++)
      for (int64_t ox = 0; ox < out_w; ox++) {
        float *o = output + ((n * out_h + oy) * out_w + ox) * out_c;
        for (int64_t oc = 0; oc < out_c; oc++) o[oc] = bias ? bias[oc] : 0.0f;
        for (int64_t ky = 0; ky < kdim; ky++)
          for (int64_t kx = 0; kx < kdim; kx++) {
            const int64_t iy = oy + ky - pad, ix = ox + kx - pad;
            const bool inside = iy >= 0 && iy < in_h && ix >= 0 && ix < in_w;
            for (int64_t ci = 0; ci < in_c; ci++) {
              const float x = inside ? inp[((n * in_h + iy) * in_w + ix) * in_c + ci] : 0.0f;
              const float *w = weights + ((ky * kdim + kx) * in_c + ci) * out_c;
              for (int64_t oc = 0; oc < out_c; oc++) o[oc] = fmaf(x, w[oc], o[oc]);
            }
          }
        if (relu)
          for (int64_t oc = 0; oc < out_c; oc++) o[oc] = o[oc] > 0.0f ? o[oc] : 0.0f;
      }
}

/* The same with a stride: out = (in + 2 pad - kdim) / stride + 1 per spatial dimension, the output
 * size of the reference's convolution harness (apps/x86/conv/conv_instance.hpp:44-45), whose layer
 * list holds two stride-2 layers (apps/x86/conv/bench_conv.cpp:47-49) that the Exo procedure itself
 * cannot run ("todo: add padding, stride", apps/x86/conv/conv.py:37).  Same chain as above. */
void oracle_conv_nhwc_strided(int64_t batch, int64_t in_h, int64_t in_w, int64_t in_c, int64_t out_c,
                              int64_t kdim, int64_t pad, int64_t stride, bool relu, const float *inp,
                              float *output, const float *weights, const float *bias) {
  const int64_t out_h = (in_h + 2 * pad - kdim) / stride + 1, out_w = (in_w + 2 * pad - kdim) / stride + 1;
#pragma omp parallel for num_threads(g_threads) collapse(2) schedule(static)
  for (int64_t n = 0; n < batch; n++)
    for (int64_t oy = 0; oy < out_h; oy++)
      for (int64_t ox = 0; ox < out_w; ox++) {
        float *o = output + ((n * out_h + oy) * out_w + ox) * out_c;
        for (int64_t oc = 0; oc < out_c; oc++) o[oc] = bias ? bias[oc] : 0.0f;
        for (int64_t ky = 0; ky < kdim; ky++)
          for (int64_t kx = 0; kx < kdim; kx++) {
            const int64_t iy = oy * stride + ky - pad, ix = ox * stride + kx - pad;
            const bool inside = iy >= 0 && iy < in_h && ix >= 0 && ix < in_w;
            for (int64_t ci = 0; ci < in_c; ci++) {
              const float x = inside ? inp[((n * in_h + iy) * in_w + ix) * in_c + ci] : 0.0f;
              const float *w = weights + ((ky * kdim + kx) * in_c + ci) * out_c;
              for (int64_t oc = 0; oc < out_c; oc++) o[oc] = fmaf(x, w[oc], o[oc]);
            }
          }
        if (relu)
          for (int64_t oc = 0; oc < out_c; oc++) o[oc] = o[oc] > 0.0f ? o[oc] : 0.0f;
      }
}

/* im2col marshalling stage of "im2col + SGEMM".  The reference only has a 1-D
 * schedule test of this decomposition (tests/test_im2col.py:41-62: y[c,r,i] =
 * x[c,i-r], then a matmul whose reduction runs over (c, r)); this is its 2-D
 * NHWC statement: col[(n,oy,ox), (ky,kx,ci)] = zero-extended inp[n, oy+ky-pad,
 * ox+kx-pad, ci].  With KhKwCiCo weights viewed as a (Kh*Kw*Ci) x Co matrix,
 * sgemm(col, W) into a bias-initialised C followed by ReLU equals
 * oracle_conv_nhwc bit-for-bit (same chain order). */
void oracle_im2col_nhwc(int64_t batch, int64_t in_h, int64_t in_w, int64_t in_c, int64_t kdim,
                        int64_t pad, const float *inp, float *col) {
  const int64_t out_h = in_h + 2 * pad - kdim + 1, out_w = in_w + 2 * pad - kdim + 1;
  const int64_t kk = kdim * kdim * in_c;
  for (int64_t n = 0; n < batch; n++)
    for (int64_t oy = 0; oy < out_h; oy++)
      for (int64_t ox = 0; ox < out_w; ox++) {
        float *row = col + ((n * out_h + oy) * out_w + ox) * kk;
        for (int64_t ky = 0; ky < kdim; ky++)
          for (int64_t kx = 0; kx < kdim; kx++) {
            const int64_t iy = oy + ky - pad, ix = ox + kx - pad;
            const bool inside = iy >= 0 && iy < in_h && ix >= 0 && ix < in_w;
            for (int64_t ci = 0; ci < in_c; ci++)
              row[(ky * kdim + kx) * in_c + ci] =
                  inside ? inp[((n * in_h + iy) * in_w + ix) * in_c + ci] : 0.0f;
          }
      }
}

/* ------------------------------------------------------- int8 epilogue
 * acc_scale (src/exo/platforms/gemmini.py:279-281) -> ACC_SCALE macro, here
 * round-half-even of the fp32 product (see header note);
 * clamp (gemmini.py:798-807; generated test_gemmini_matmul.txt:241-250):
 *   tmp = (127 < src) ? 127 : src;  tmp = (src < -128) ? -128 : tmp;  (int8_t)tmp
 * relu (src/exo/libs/externs.py:33-68): x > 0 ? x : 0, only if act. */
static inline int8_t i8_epilogue(int32_t acc, float scale, bool act) {
  const float src = nearbyintf((float)acc * scale);
  float tmp = (127.0f < src) ? 127.0f : src;
  tmp = (src < -128.0f) ? -128.0f : tmp;
  int8_t q = (int8_t)tmp;
  if (act) q = q > 0 ? q : 0;
  return q;
}

/* matmul_on_cpu, apps/gemmini/src/exo/matmul.py:7-43 (Exo names the rows N and
 * the columns M): acc = sum_k (i32)A[i,k] * (i32)B[k,j] from 0, then the
 * epilogue above.  Integer sums are order independent, so the loop order is
 * i-k-j for speed. */
void oracle_matmul_i8(int64_t N, int64_t M, int64_t K, const float *scale, bool act,
                      const int8_t *A, const int8_t *B, int8_t *C) {
  const float s = *scale;
#pragma omp parallel num_threads(g_threads)
  {
    int32_t *acc = (int32_t *)malloc(sizeof(int32_t) * (size_t)M);
#pragma omp for schedule(static)
    for (int64_t i = 0; i < N; i++) {
      memset(acc, 0, sizeof(int32_t) * (size_t)M);
      for (int64_t k = 0; k < K; k++) {
        const int32_t a = A[i * K + k];
        const int8_t *b = B + k * M;
        for (int64_t j = 0; j < M; j++) acc[j] += a * (int32_t)b[j];
      }
      for (int64_t j = 0; j < M; j++) C[i * M + j] = i8_epilogue(acc[j], s, act);
    }
    free(acc);
  }
}

/* conv_on_cpu_stride_1, apps/gemmini/src/exo/conv.py:6-55: NHWC int8, weights
 * i8[Kh,Kw,Ci,Co], bias i32[1,Co] as the accumulator's start value, square
 * input and kernel, no padding, same epilogue.  Argument order follows the
 * generated conv_*_cpu (tests/golden/test_apps/test_gemmini_conv.txt:146) after
 * the sizes. */
void oracle_conv_i8(int64_t batch_size, int64_t out_dim, int64_t out_channel, int64_t kernel_dim,
                    int64_t in_channel, int64_t in_dim, int8_t *output, const int32_t *bias,
                    const int8_t *inp, const int8_t *weights, bool act, const float *scale) {
  const float s = *scale;
#pragma omp parallel num_threads(g_threads)
  {
    int32_t *acc = (int32_t *)malloc(sizeof(int32_t) * (size_t)out_channel);
#pragma omp for collapse(2) schedule(static)
    for (int64_t b = 0; b < batch_size; b++)
      for (int64_t orow = 0; orow < out_dim; orow++)
        for (int64_t ocol = 0; ocol < out_dim; ocol++) {
          for (int64_t och = 0; och < out_channel; och++) acc[och] = bias[och];
          for (int64_t krow = 0; krow < kernel_dim; krow++)
            for (int64_t kcol = 0; kcol < kernel_dim; kcol++)
              for (int64_t kch = 0; kch < in_channel; kch++) {
                const int32_t x =
                    inp[((b * in_dim + orow + krow) * in_dim + ocol + kcol) * in_channel + kch];
                const int8_t *w =
                    weights + ((krow * kernel_dim + kcol) * in_channel + kch) * out_channel;
                for (int64_t och = 0; och < out_channel; och++) acc[och] += x * (int32_t)w[och];
              }
          int8_t *o = output + ((b * out_dim + orow) * out_dim + ocol) * out_channel;
          for (int64_t och = 0; och < out_channel; och++) o[och] = i8_epilogue(acc[och], s, act);
        }
    free(acc);
  }
}

/* ------------------------------------------------------------------- bf16
 * The reference has no bf16 type (src/exo/core/LoopIR.py:446-462); the large
 * bf16 GEMM is checked against the reference fp32 SGEMM run on the bf16 inputs
 * widened exactly to fp32.  Helpers for that comparison. */
static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* round-to-nearest-even fp32 -> bf16 bits; NaN stays a quiet NaN */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

void oracle_bf16_widen(int64_t n, const uint16_t *src, float *dst) {
  for (int64_t i = 0; i < n; i++) dst[i] = bf16_to_f32(src[i]);
}

void oracle_bf16_round(int64_t n, const float *src, uint16_t *dst) {
  for (int64_t i = 0; i < n; i++) dst[i] = f32_to_bf16(src[i]);
}

/* C(bf16, row-major MxN) = A(bf16, row-major MxK) * B(bf16, column-major KxN,
 * i.e. element (k,j) at B[j*K + k]) with the reference SGEMM chain in fp32 on
 * the widened inputs (C starts at 0) and one final RNE rounding to bf16. */
void oracle_gemm_bf16(int64_t M, int64_t N, int64_t K, const uint16_t *A, const uint16_t *B,
                      uint16_t *C) {
  float *Af = (float *)malloc(sizeof(float) * (size_t)(M * K));
  float *Bf = (float *)malloc(sizeof(float) * (size_t)(K * N));
  float *Cf = (float *)calloc((size_t)(M * N), sizeof(float));
  oracle_bf16_widen(M * K, A, Af);
  for (int64_t j = 0; j < N; j++)
    for (int64_t k = 0; k < K; k++) Bf[k * N + j] = bf16_to_f32(B[j * K + k]);
  oracle_sgemm(M, N, K, Af, Bf, Cf);
  oracle_bf16_round(M * N, Cf, C);
  free(Af);
  free(Bf);
  free(Cf);
}
