// Drop-in check for the SGEMM symbol: a C++ caller written the way the reference's own
// checker is (apps/x86/sgemm/test.cpp:22-50 -- random A, B, C; call sgemm_exo(nullptr,
// n, n, n, a, b, c) through the generated header's prototype; compare with a trusted
// result, print mismatches), linked against libexo_b200.so instead of the exocc output.
// The trusted result here is the scalar fused-multiply-add chain the generated
// microkernels implement; the comparison is exact (the reference's own tolerance is 1e-3
// relative).  Usage: sgemm_check M N K
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>

#include "exo_b200.h"

static std::vector<float> gen_matrix(long m, long n, unsigned seed) {
  std::mt19937 rng{seed};
  std::uniform_real_distribution<float> rv{-1.0f, 1.0f};
  std::vector<float> mat(m * n);
  for (auto &x : mat) x = rv(rng);
  return mat;
}

int main(int argc, char *argv[]) {
  if (argc != 4) {
    printf("Usage: %s M N K\n", argv[0]);
    return 2;
  }
  const long m = atol(argv[1]), n = atol(argv[2]), k = atol(argv[3]);
  auto a = gen_matrix(m, k, 1), b = gen_matrix(k, n, 2), c = gen_matrix(m, n, 3);
  auto c2 = c;

  for (long i = 0; i < m; i++)
    for (long kk = 0; kk < k; kk++) {
      const float av = a[i * k + kk];
      for (long j = 0; j < n; j++) c[i * n + j] = std::fmaf(av, b[kk * n + j], c[i * n + j]);
    }

  sgemm_exo(nullptr, m, n, k, a.data(), b.data(), c2.data());
  if (exo_b200_last_error() != EXO_B200_OK) {
    printf("sgemm_exo failed: %s\n", exo_b200_last_error_string());
    return 1;
  }

  long bad = 0;
  for (long i = 0; i < m * n; i++) {
    if (std::memcmp(&c[i], &c2[i], sizeof(float)) != 0) {
      if (bad < 10) printf("%ld %.9g %.9g\n", i, c[i], c2[i]);
      bad++;
    }
  }
  printf("%ld mismatches out of %ld\n", bad, m * n);
  return bad == 0 ? 0 : 1;
}
