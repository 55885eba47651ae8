/* Drop-in check for the Gemmini int8 symbols, shaped like the reference's runner
 * (apps/gemmini/test/run_matmul.c:26-63): x[i][j] = i + 2j, y[i][j] = 3j + i wrapped to
 * int8, scale 2.0, act false, an UNINITIALISED context pointer, the plain-C function
 * and the accelerator function called one after the other and compared for equality --
 * here both symbols come from libexo_b200.so, and the result is also compared with the
 * arithmetic spelled out in C.  Plain C on purpose: the reference's callers are C. */
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include "exo_b200.h"

#define NN 512
#define MM 512
#define KK 512

static float c_scale[1] = {2.0f};
static int8_t x[NN * KK];
static int8_t y[KK * MM];
static int8_t z_cpu[NN * MM];
static int8_t z_gemmini[NN * MM];

int main(void) {
  for (int i = 0; i < NN; i++)
    for (int j = 0; j < KK; j++) x[KK * i + j] = (int8_t)(i + j * 2);
  for (int i = 0; i < KK; i++)
    for (int j = 0; j < MM; j++) y[MM * i + j] = (int8_t)(j * 3 + i);

  void *ctxt = (void *)(size_t)0x1234560; /* never dereferenced by the callee */
  cpu_matmul_512x512x512(ctxt, c_scale, false, x, y, z_cpu);
  if (exo_b200_last_error() != EXO_B200_OK) {
    printf("cpu_matmul_512x512x512 failed: %s\n", exo_b200_last_error_string());
    return 1;
  }
  matmul_512x512x512(ctxt, c_scale, false, x, y, z_gemmini);

  long bad = 0;
  for (int i = 0; i < NN; i++)
    for (int j = 0; j < MM; j++) {
      int32_t acc = 0;
      for (int k = 0; k < KK; k++) acc += (int32_t)x[KK * i + k] * (int32_t)y[MM * k + j];
      float t = nearbyintf((float)acc * c_scale[0]);
      t = t > 127.0f ? 127.0f : (t < -128.0f ? -128.0f : t);
      if (z_cpu[MM * i + j] != (int8_t)t || z_gemmini[MM * i + j] != z_cpu[MM * i + j]) bad++;
    }
  if (bad == 0) {
    printf("Correct\n");
    return 0;
  }
  printf("Results Don't Match (%ld)\n", bad);
  return 1;
}
