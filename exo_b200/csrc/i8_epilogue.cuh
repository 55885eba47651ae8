// The Gemmini int8 output stage, shared by every int8 kernel so that all of
// them produce the same bits.  Reference statement:
//   acc_scale  src/exo/platforms/gemmini.py:279-281  (ACC_SCALE: round-half-even of
//              the fp32 product (f32)acc * scale; the int32 -> fp32 conversion
//              itself rounds to nearest even once |acc| > 2^24)
//   clamp      src/exo/platforms/gemmini.py:798-807, generated
//              tests/golden/test_apps/test_gemmini_matmul.txt:241-250: two selects
//              on the FLOAT value, then the cast
//   relu       src/exo/libs/externs.py:33-68, applied only when act is true
// Each step is a separate correctly rounded operation: no FMA contraction of
// the multiply with anything else, no conversion of an unclamped float to int.
#pragma once
#include <stdint.h>

namespace exob200 {

__device__ __forceinline__ int8_t i8_epilogue(int32_t acc, float scale, bool act) {
  const float src = rintf(__fmul_rn(__int2float_rn(acc), scale));
  float tmp = (127.0f < src) ? 127.0f : src;
  tmp = (src < -128.0f) ? -128.0f : tmp;
  int8_t q = (int8_t)(int)tmp;
  if (act) q = q > 0 ? q : (int8_t)0;
  return q;
}

}  // namespace exob200
