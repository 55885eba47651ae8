// Drop-in check for conv_specialized, following the reference's harness: the problem
// container's deterministic fill (apps/x86/conv/conv_instance.hpp:52-60: cos / sin /
// tanh of a float counter), the call shape of apps/x86/conv/exo_conv.cpp:16, and a
// direct-loop comparison like apps/x86/conv/test_conv.cpp:12-35 -- exact here, against
// the bias-initialised FMA chain in ky -> kx -> kc order that the generated code runs.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <vector>

#include "exo_b200.h"

int main() {
  const long N = 5, IH = 82, IW = 102, IC = 128, OC = 128, K = 3, OH = 80, OW = 100;
  std::vector<float> src(N * IH * IW * IC), w(IC * K * K * OC), bias(OC), dst(N * OH * OW * OC), ref(dst.size());
  {
    float i = 0.0f;
    for (auto &x : src) x = std::cos(i++ / 10.f);
    i = 0.0f;
    for (auto &x : w) x = std::sin(i++ * 2.f);
    i = 0.0f;
    for (auto &x : bias) x = std::tanh(i++);
  }
  conv_specialized(nullptr, src.data(), dst.data(), w.data(), bias.data());
  if (exo_b200_last_error() != EXO_B200_OK) {
    printf("conv_specialized failed: %s\n", exo_b200_last_error_string());
    return 1;
  }
  // every 7th output pixel is enough to catch an indexing or ordering error
  long bad = 0, checked = 0;
  for (long p = 0; p < N * OH * OW; p += 7) {
    const long n = p / (OH * OW), oy = (p / OW) % OH, ox = p % OW;
    for (long oc = 0; oc < OC; oc++) {
      float acc = bias[oc];
      for (long ky = 0; ky < K; ky++)
        for (long kx = 0; kx < K; kx++)
          for (long kc = 0; kc < IC; kc++)
            acc = std::fmaf(w[((kc * K + ky) * K + kx) * OC + oc], src[((n * IH + oy + ky) * IW + ox + kx) * IC + kc], acc);
      acc = acc > 0.0f ? acc : 0.0f;
      const float got = dst[p * OC + oc];
      if (std::memcmp(&acc, &got, sizeof(float)) != 0) bad++;
      checked++;
    }
  }
  printf("%ld mismatches out of %ld checked\n", bad, checked);
  return bad == 0 ? 0 : 1;
}
