/* Drop-in check for the Gemmini library's "auto" entry points, as the reference's shim
 * overrides them (apps/gemmini/test/bare-metal/shims/gemmini.c:5-58, :60-141): an upstream
 * style caller hands tiled_matmul_auto / tiled_conv_auto plain int8 arrays and the full
 * upstream parameter list.  Checked here: a shape with a generated instance (512^3,
 * conv_3), a shape without one (generic kernels), and a call that asks for something the
 * kernels do not compute (refused, output untouched).  Expected values are spelled out in C
 * with the arithmetic of apps/gemmini/src/exo/matmul.py:18-43 / conv.py:6-55. */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "exo_b200.h"
#include "exo_b200_gemmini_shim.h"

static int8_t out_stage(int32_t acc, float scale, int act) {
  float t = nearbyintf((float)acc * scale);
  t = t > 127.0f ? 127.0f : (t < -128.0f ? -128.0f : t);
  int8_t q = (int8_t)t;
  if (act && q < 0) q = 0;
  return q;
}

static long check_matmul(size_t I, size_t J, size_t K, float scale, int act) {
  int8_t* A = malloc(I * K);
  int8_t* B = malloc(K * J);
  int8_t* C = malloc(I * J);
  for (size_t i = 0; i < I; i++)
    for (size_t k = 0; k < K; k++) A[i * K + k] = (int8_t)((i * 7 + k * 3) % 23 - 11);
  for (size_t k = 0; k < K; k++)
    for (size_t j = 0; j < J; j++) B[k * J + j] = (int8_t)((k * 5 + j * 11) % 19 - 9);
  memset(C, 0x55, I * J);
  tiled_matmul_auto(I, J, K, A, B, NULL, C, K, J, J, J, 1.0f, 1.0f, 1.0f, act, scale, 0.0f, false, false, false,
                    false, false, 3, 1);
  if (exo_b200_last_error() != EXO_B200_OK) {
    printf("tiled_matmul_auto failed: %s\n", exo_b200_last_error_string());
    return -1;
  }
  long bad = 0;
  for (size_t i = 0; i < I; i++)
    for (size_t j = 0; j < J; j++) {
      int32_t acc = 0;
      for (size_t k = 0; k < K; k++) acc += (int32_t)A[i * K + k] * (int32_t)B[k * J + j];
      if (C[i * J + j] != out_stage(acc, scale, act)) bad++;
    }
  free(A);
  free(B);
  free(C);
  return bad;
}

static long check_conv(int batch, int in_dim, int ci, int co, int kd, float scale, int act, int against_symbol) {
  const int od = in_dim - kd + 1;
  const size_t n_in = (size_t)batch * in_dim * in_dim * ci, n_w = (size_t)kd * kd * ci * co,
               n_out = (size_t)batch * od * od * co;
  int8_t* inp = malloc(n_in);
  int8_t* w = malloc(n_w);
  int32_t* bias = malloc(sizeof(int32_t) * co);
  int8_t* out = malloc(n_out);
  int8_t* want = malloc(n_out);
  for (size_t i = 0; i < n_in; i++) inp[i] = (int8_t)((i * 13) % 17 - 8);
  for (size_t i = 0; i < n_w; i++) w[i] = (int8_t)((i * 7) % 13 - 6);
  for (int c = 0; c < co; c++) bias[c] = 100 - 9 * c;
  memset(out, 0x55, n_out);
  tiled_conv_auto(batch, in_dim, in_dim, ci, co, od, od, 1, 1, 1, 0, kd, false, false, false, false, false, inp, w,
                  bias, out, act, scale, 1, 1, 0, 1);
  if (exo_b200_last_error() != EXO_B200_OK) {
    printf("tiled_conv_auto failed: %s\n", exo_b200_last_error_string());
    return -1;
  }
  if (against_symbol) {
    float s = scale;
    conv_3_cpu(NULL, want, bias, inp, w, act != 0, &s);
  } else {
    for (int b = 0; b < batch; b++)
      for (int oy = 0; oy < od; oy++)
        for (int ox = 0; ox < od; ox++)
          for (int c = 0; c < co; c++) {
            int32_t acc = bias[c];
            for (int ky = 0; ky < kd; ky++)
              for (int kx = 0; kx < kd; kx++)
                for (int k = 0; k < ci; k++)
                  acc += (int32_t)inp[(((size_t)b * in_dim + oy + ky) * in_dim + ox + kx) * ci + k] *
                         (int32_t)w[(((size_t)ky * kd + kx) * ci + k) * co + c];
            want[(((size_t)b * od + oy) * od + ox) * co + c] = out_stage(acc, scale, act);
          }
  }
  long bad = 0;
  for (size_t i = 0; i < n_out; i++) bad += out[i] != want[i];
  free(inp);
  free(w);
  free(bias);
  free(out);
  free(want);
  return bad;
}

int main(void) {
  long bad = 0, r;
  if ((r = check_matmul(512, 512, 512, 1.0f / 64, 0)) != 0) printf("matmul 512^3 (instance): %ld wrong\n", r), bad++;
  if ((r = check_matmul(96, 80, 48, 0.05f, 1)) != 0) printf("matmul 96x80x48 (generic): %ld wrong\n", r), bad++;
  if ((r = check_matmul(33, 17, 5, 0.5f, 0)) != 0) printf("matmul 33x17x5 (generic, SIMT): %ld wrong\n", r), bad++;
  if ((r = check_conv(2, 10, 16, 16, 3, 1.0f / 32, 1, 0)) != 0) printf("conv generic: %ld wrong\n", r), bad++;
  if ((r = check_conv(4, 58, 64, 64, 3, 1.0f / 128, 0, 1)) != 0) printf("conv_3 (instance): %ld wrong\n", r), bad++;

  /* a request the kernels do not compute: refused, output untouched */
  int8_t a[64], c[64];
  memset(a, 1, sizeof a);
  memset(c, 0x55, sizeof c);
  tiled_matmul_auto(8, 8, 8, a, a, NULL, c, 8, 8, 8, 8, 1.0f, 1.0f, 1.0f, 0, 1.0f, 0.0f, false, true, false, false,
                    false, 3, 1);
  if (exo_b200_last_error() != EXO_B200_ERR_UNSUPPORTED) printf("transpose_A was not refused\n"), bad++;
  for (int i = 0; i < 64; i++)
    if (c[i] != 0x55) {
      printf("refused call wrote its output\n");
      bad++;
      break;
    }
  tiled_conv_auto(1, 8, 8, 16, 16, 4, 4, 2, 1, 1, 0, 2, false, false, false, false, false, a, a, NULL, c, 0, 1.0f, 1,
                  1, 0, 1);
  if (exo_b200_last_error() != EXO_B200_ERR_UNSUPPORTED) printf("stride 2 was not refused\n"), bad++;

  if (bad == 0) {
    printf("Correct\n");
    return 0;
  }
  printf("Results Don't Match (%ld checks failed)\n", bad);
  return 1;
}
