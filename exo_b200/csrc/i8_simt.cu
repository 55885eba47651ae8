// Exact int8 SIMT kernels: the Gemmini-style matmul and NHWC convolution for
// shapes whose pitches the tensor-core path's TMA descriptors cannot express
// (row pitch not a multiple of 16 bytes, unaligned base) and for tiny problems.
//
// Arithmetic (apps/gemmini/src/exo/matmul.py:18-43, conv.py:22-53):
//   acc (int32) = start + sum_k (i32)a * (i32)b        exact, order independent
//   t = round_half_even((f32)acc * scale)              acc_scale, gemmini.py:279-281
//   q = (int8) (t > 127 ? 127 : t < -128 ? -128 : t)   clamp, gemmini.py:798-807
//   if (act) q = q > 0 ? q : 0                          relu, libs/externs.py:33-68
#include "i8_epilogue.cuh"
#include "kernels.cuh"

namespace exob200 {
namespace {

constexpr int TM = 64, TN = 64, TK = 32;

// Policy: int M, N, K;  int8_t a(m, k) (0 outside);  int8_t b(k, n) (0 outside);
//         int32_t start(n);  void store(m, n, int8_t)
template <class Policy>
__global__ void __launch_bounds__(256) i8_tile_kernel(const Policy P) {
  __shared__ int8_t As[TM][TK + 4];
  __shared__ int8_t Bs[TK][TN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.x * TM, n0 = blockIdx.y * TN;
  int32_t acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = P.start(n0 + tx * 4 + j);

  for (int k0 = 0; k0 < P.K; k0 += TK) {
    for (int e = tid; e < TM * TK; e += 256) {
      const int r = e / TK, k = e % TK;
      As[r][k] = P.a(m0 + r, k0 + k);
    }
    for (int e = tid; e < TK * TN; e += 256) {
      const int k = e / TN, c = e % TN;
      Bs[k][c] = P.b(k0 + k, n0 + c);
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < TK; kk++) {
      int32_t a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = As[ty * 4 + i][kk];
#pragma unroll
      for (int j = 0; j < 4; j++) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] += a[i] * b[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < P.M && n < P.N) P.store(m, n, i8_epilogue(acc[i][j], P.scale, P.act));
    }
}

struct MatmulPolicy {
  int M, N, K;  // GEMM view: rows, columns, reduction
  float scale;
  bool act;
  const int8_t* __restrict__ A;
  const int8_t* __restrict__ B;
  int8_t* __restrict__ C;
  __device__ __forceinline__ int8_t a(int m, int k) const {
    return (m < M && k < K) ? A[(int64_t)m * K + k] : (int8_t)0;
  }
  __device__ __forceinline__ int8_t b(int k, int n) const {
    return (k < K && n < N) ? B[(int64_t)k * N + n] : (int8_t)0;
  }
  __device__ __forceinline__ int32_t start(int) const { return 0; }
  __device__ __forceinline__ void store(int m, int n, int8_t q) const { C[(int64_t)m * N + n] = q; }
};

struct ConvI8Policy {
  int M, N, K;
  float scale;
  bool act;
  ConvShape s;
  const int8_t* __restrict__ inp;
  const int8_t* __restrict__ w;
  const int32_t* __restrict__ bias;
  int8_t* __restrict__ out;
  __device__ __forceinline__ int8_t a(int m, int k) const {
    if (m >= M || k >= K) return 0;
    const int hw = s.out_h * s.out_w;
    const int n = m / hw, r = m - n * hw;
    const int oy = r / s.out_w, ox = r - oy * s.out_w;
    const int tap = k / s.in_c, ci = k - tap * s.in_c;
    const int ky = tap / s.kdim, kx = tap - ky * s.kdim;
    const int iy = oy + ky - s.pad, ix = ox + kx - s.pad;
    if (iy < 0 || iy >= s.in_h || ix < 0 || ix >= s.in_w) return 0;
    return inp[(((int64_t)n * s.in_h + iy) * s.in_w + ix) * s.in_c + ci];
  }
  __device__ __forceinline__ int8_t b(int k, int n) const {
    if (k >= K || n >= N) return 0;
    const int tap = k / s.in_c, ci = k - tap * s.in_c;
    const int ky = tap / s.kdim, kx = tap - ky * s.kdim;
    return w[ky * s.w_stride_ky + kx * s.w_stride_kx + ci * s.w_stride_ci + n];
  }
  __device__ __forceinline__ int32_t start(int n) const {
    return (bias != nullptr && n < N) ? bias[n] : 0;
  }
  __device__ __forceinline__ void store(int m, int n, int8_t q) const { out[(int64_t)m * N + n] = q; }
};

}  // namespace

cudaError_t launch_matmul_i8_simt(cudaStream_t stream, int64_t N, int64_t M, int64_t K, float scale,
                                  bool act, const int8_t* A, const int8_t* B, int8_t* C) {
  // Exo's names: A is N x K, B is K x M, C is N x M.
  if (N > INT32_MAX || M > INT32_MAX || K > INT32_MAX) return cudaErrorInvalidValue;
  MatmulPolicy P{(int)N, (int)M, (int)K, scale, act, A, B, C};
  dim3 grid((unsigned)((N + TM - 1) / TM), (unsigned)((M + TN - 1) / TN));
  if (grid.y > 65535) return cudaErrorInvalidValue;
  i8_tile_kernel<MatmulPolicy><<<grid, 256, 0, stream>>>(P);
  return cudaGetLastError();
}

cudaError_t launch_conv_i8_simt(cudaStream_t stream, const ConvShape& s, float scale, bool act,
                                const int8_t* inp, int8_t* out, const int8_t* weights,
                                const int32_t* bias) {
  const int64_t M = (int64_t)s.batch * s.out_h * s.out_w;
  const int64_t K = (int64_t)s.kdim * s.kdim * s.in_c;
  if (M > INT32_MAX || K > INT32_MAX) return cudaErrorInvalidValue;
  ConvI8Policy P{(int)M, s.out_c, (int)K, scale, act, s, inp, weights, bias, out};
  dim3 grid((unsigned)((M + TM - 1) / TM), (unsigned)((s.out_c + TN - 1) / TN));
  if (grid.y > 65535) return cudaErrorInvalidValue;
  i8_tile_kernel<ConvI8Policy><<<grid, 256, 0, stream>>>(P);
  return cudaGetLastError();
}

}  // namespace exob200
