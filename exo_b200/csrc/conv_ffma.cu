// Exact-fp32 NHWC convolution as an implicit GEMM on the SIMT tile engine.
//
// Replaces conv / conv_specialized (apps/x86/conv/conv.py:10-45; generated code
// tests/golden/test_apps/test_x86_conv.txt:74-113):
//   out[n,oy,ox,co] = relu(bias[co] + sum_{ky,kx,ci} W(ky,kx,ci,co) * inp[n,oy+ky-pad,ox+kx-pad,ci])
// The generated code starts each accumulator at bias and runs one FMA chain in
// ky -> kx -> kc order, then max(x, 0) (golden :82, :85-95, :105).  Here the
// GEMM view is M = batch*out_h*out_w (output pixels; the NHWC output IS the
// row-major M x Co matrix), N = Co, K = kdim*kdim*Ci ordered (ky, kx, ci), so
// the tile engine's increasing-k chain is the reference's order and results
// are bit-identical.  The im2col matrix is never materialised: the A loader
// turns (pixel, k) into an input address, zero for padded taps (a padded tap
// still goes through fmaf(w, 0, acc), as it does when the reference's caller
// pre-pads the input).
//
// Weights may be in either layout the reference uses -- [Ci,Kh,Kw,Co]
// (apps/x86/conv/conv.py:22) or [Kh,Kw,Ci,Co] (apps/gemmini/src/exo/conv.py:17)
// -- expressed as element strides for (ky, kx, ci); co is contiguous.
#include "ffma_tile.cuh"
#include "kernels.cuh"

namespace exob200 {
namespace {

using ffma::ldg4;
using ffma::zero4;

template <bool VEC>  // VEC: in_c % 4 == 0, out_c % 4 == 0, 16-byte aligned bases
struct ConvPolicy {
  int M, N, K;
  ConvShape s;
  const float* __restrict__ inp;
  const float* __restrict__ w;
  const float* __restrict__ bias;
  float* __restrict__ out;

  static constexpr bool kTransposedB = false;
  static constexpr bool kUpperTriangle = false;

  struct RowCtx {
    int64_t base;  // element offset of inp[n, 0, 0, 0]
    int iy0, ix0;  // input coordinates of tap (0, 0)
    bool valid;
  };
  __device__ __forceinline__ RowCtx row_ctx(int m) const {
    RowCtx rc;
    rc.valid = m < M;
    const int mm = rc.valid ? m : 0;
    const int hw = s.out_h * s.out_w;
    const int n = mm / hw;
    const int r = mm - n * hw;
    const int oy = r / s.out_w;
    const int ox = r - oy * s.out_w;
    rc.base = (int64_t)n * s.in_h * s.in_w * s.in_c;
    rc.iy0 = oy * s.stride - s.pad;
    rc.ix0 = ox * s.stride - s.pad;
    return rc;
  }
  __device__ __forceinline__ void decode(int k, int& ky, int& kx, int& ci) const {
    const int tap = k / s.in_c;
    ci = k - tap * s.in_c;
    ky = tap / s.kdim;
    kx = tap - ky * s.kdim;
  }
  __device__ __forceinline__ float load_a1(const RowCtx& rc, int k) const {
    if (k >= K) return 0.f;
    int ky, kx, ci;
    decode(k, ky, kx, ci);
    const int iy = rc.iy0 + ky, ix = rc.ix0 + kx;
    if (iy < 0 || iy >= s.in_h || ix < 0 || ix >= s.in_w) return 0.f;
    return __ldg(inp + rc.base + ((int64_t)iy * s.in_w + ix) * s.in_c + ci);
  }
  __device__ __forceinline__ float4 load_a(const RowCtx& rc, int, int k) const {
    float4 v = zero4();
    if (!rc.valid) return v;
    if (VEC) {
      if (k >= K) return v;
      int ky, kx, ci;
      decode(k, ky, kx, ci);  // in_c % 4 == 0: the quad stays inside one tap
      const int iy = rc.iy0 + ky, ix = rc.ix0 + kx;
      if (iy < 0 || iy >= s.in_h || ix < 0 || ix >= s.in_w) return v;
      return ldg4(inp + rc.base + ((int64_t)iy * s.in_w + ix) * s.in_c + ci);
    }
    v.x = load_a1(rc, k + 0);
    v.y = load_a1(rc, k + 1);
    v.z = load_a1(rc, k + 2);
    v.w = load_a1(rc, k + 3);
    return v;
  }
  __device__ __forceinline__ void copy_b(float* smem, int k, int col) const {
    const bool kin = k < K;
    int ky, kx, ci;
    decode(kin ? k : 0, ky, kx, ci);
    const float* p = w + ky * s.w_stride_ky + kx * s.w_stride_kx + ci * s.w_stride_ci;
    if (VEC) {
      const bool ok = kin && col < N;
      ffma::cp_async16(smem, p + (ok ? col : 0), ok);
    } else {
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const bool ok = kin && col + j < N;
        ffma::cp_async4(smem + j, p + (ok ? col + j : 0), ok);
      }
    }
  }
  __device__ __forceinline__ float4 init(int, int col) const {
    float4 v = zero4();
    if (bias == nullptr) return v;
    if (col + 0 < N) v.x = __ldg(bias + col + 0);
    if (col + 1 < N) v.y = __ldg(bias + col + 1);
    if (col + 2 < N) v.z = __ldg(bias + col + 2);
    if (col + 3 < N) v.w = __ldg(bias + col + 3);
    return v;
  }
  // _mm512_max_ps(res, 0) (golden :105): NaN -> 0, -0 -> +0
  __device__ __forceinline__ float act(float x) const { return s.relu ? (x > 0.f ? x : 0.f) : x; }
  __device__ __forceinline__ void store(int row, int col, float4 v) const {
    if (row >= M) return;
    float* p = out + (int64_t)row * N + col;
    v.x = act(v.x);
    v.y = act(v.y);
    v.z = act(v.z);
    v.w = act(v.w);
    if (VEC) {
      if (col < N) *reinterpret_cast<float4*>(p) = v;
    } else {
      if (col + 0 < N) p[0] = v.x;
      if (col + 1 < N) p[1] = v.y;
      if (col + 2 < N) p[2] = v.z;
      if (col + 3 < N) p[3] = v.w;
    }
  }
};

}  // namespace

cudaError_t launch_conv_ffma(cudaStream_t stream, const ConvShape& s, const float* inp, float* out,
                             const float* weights, const float* bias) {
  const int64_t M = (int64_t)s.batch * s.out_h * s.out_w;
  const int64_t K = (int64_t)s.kdim * s.kdim * s.in_c;
  if (M > INT32_MAX || K > INT32_MAX) return cudaErrorInvalidValue;
  const bool vec = s.in_c % 4 == 0 && s.out_c % 4 == 0 && ffma::aligned16(inp) &&
                   ffma::aligned16(out) && ffma::aligned16(weights);
  if (vec)
    return ffma::launch_tiles(stream, ConvPolicy<true>{(int)M, s.out_c, (int)K, s, inp, weights, bias, out});
  return ffma::launch_tiles(stream, ConvPolicy<false>{(int)M, s.out_c, (int)K, s, inp, weights, bias, out});
}

}  // namespace exob200
