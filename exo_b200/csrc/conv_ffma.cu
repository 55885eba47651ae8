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
  int wsy, wsx, wsc;  // the weight tensor's element strides for (ky, kx, ci), checked to fit 32 bits

  static constexpr bool kTransposedB = false;
  static constexpr bool kUpperTriangle = false;

  struct RowCtx {
    int64_t base;  // element offset of inp[n, iy0, ix0, 0] (tap (0, 0) of this pixel; may lie in the padding)
    int iy0, ix0;  // input coordinates of tap (0, 0)
    bool valid;
  };
  // Cursor along K = (ky, kx, ci): decoded once with two divisions, then advanced by additions.
  struct KCtx {
    int k, ky, kx, ci;
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
    rc.iy0 = oy * s.stride - s.pad;
    rc.ix0 = ox * s.stride - s.pad;
    rc.base = ((int64_t)n * s.in_h * s.in_w + (int64_t)rc.iy0 * s.in_w + rc.ix0) * s.in_c;
    return rc;
  }
  __device__ __forceinline__ KCtx k_ctx(int k) const {
    KCtx c;
    c.k = k;
    const int tap = k / s.in_c;
    c.ci = k - tap * s.in_c;
    c.ky = tap / s.kdim;
    c.kx = tap - c.ky * s.kdim;
    return c;
  }
  __device__ __forceinline__ void k_advance(KCtx& c, int step) const {
    c.k += step;
    c.ci += step;
    while (c.ci >= s.in_c) {
      c.ci -= s.in_c;
      if (++c.kx == s.kdim) c.kx = 0, ++c.ky;
    }
  }
  __device__ __forceinline__ bool tap_inside(const RowCtx& rc, const KCtx& c) const {
    return (unsigned)(rc.iy0 + c.ky) < (unsigned)s.in_h && (unsigned)(rc.ix0 + c.kx) < (unsigned)s.in_w;
  }
  __device__ __forceinline__ const float* tap_ptr(const RowCtx& rc, const KCtx& c) const {
    return inp + rc.base + ((c.ky * s.in_w + c.kx) * s.in_c + c.ci);
  }
  __device__ __forceinline__ float4 load_a(const RowCtx& rc, int, const KCtx& c) const {
    float4 v = zero4();
    if (!rc.valid) return v;
    if (VEC) {  // in_c % 4 == 0: the quad stays inside one tap
      if (c.k < K && tap_inside(rc, c)) v = ldg4(tap_ptr(rc, c));
      return v;
    }
    KCtx e = c;
    float r[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      r[j] = (e.k < K && tap_inside(rc, e)) ? __ldg(tap_ptr(rc, e)) : 0.f;
      k_advance(e, 1);
    }
    return make_float4(r[0], r[1], r[2], r[3]);
  }
  __device__ __forceinline__ void copy_b(float* smem, const KCtx& c, int col) const {
    const bool kin = c.k < K;
    const float* p = w + (kin ? c.ky * wsy + c.kx * wsx + c.ci * wsc : 0);
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
  // 32-bit offsets inside one image and inside the weight tensor
  if ((int64_t)s.in_h * s.in_w * s.in_c > INT32_MAX || K * (int64_t)s.out_c > INT32_MAX) return cudaErrorInvalidValue;
  const int wsy = (int)s.w_stride_ky, wsx = (int)s.w_stride_kx, wsc = (int)s.w_stride_ci;
  const bool vec = s.in_c % 4 == 0 && s.out_c % 4 == 0 && ffma::aligned16(inp) &&
                   ffma::aligned16(out) && ffma::aligned16(weights);
  if (vec)
    return ffma::launch_tiles(stream, ConvPolicy<true>{(int)M, s.out_c, (int)K, s, inp, weights, bias, out, wsy, wsx, wsc});
  return ffma::launch_tiles(stream, ConvPolicy<false>{(int)M, s.out_c, (int)K, s, inp, weights, bias, out, wsy, wsx, wsc});
}

}  // namespace exob200
