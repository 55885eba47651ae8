// Exact-fp32 SSYRK on the SIMT tile engine:  C += A * A^T on the upper triangle
// (j >= i), A : f32[N, K] row-major, C : f32[N, N] row-major.
//
// The reference has no Exo procedure for this; it only measures MKL's
// cblas_ssyrk(CblasRowMajor, CblasUpper, CblasNoTrans, n, k, 1, a, k, 1, c, n)
// (apps/x86/ssyrk/bench_ssyrk.cpp:49-58) over n = 64 .. 2048, k = 16 .. 2048
// (:60-65).  The arithmetic here is the reference SGEMM's: every output element
// is one chain  c = fmaf(A[i,k], A[j,k], c)  in increasing k starting from the
// incoming C[i,j] (tests/golden/test_apps/test_x86_sgemm.txt:437-454), so the
// result equals sgemm_exo(N, N, K, A, A^T, C) bit for bit on the upper triangle,
// while the strict lower triangle of C is neither read nor written.
//
// Both operands are rows of A (k contiguous), so the B tile takes the A tile's
// route: 128-bit global loads along k, transposed through registers into the
// k-major shared-memory layout.  The grid holds only the tiles that reach the
// diagonal or lie above it; tiles on the diagonal mask their loads of C and
// their stores.
#include "ffma_tile.cuh"
#include "kernels.cuh"

namespace exob200 {
namespace {

using ffma::ldg4;
using ffma::zero4;

template <bool VA, bool VC>  // VA: K % 4 == 0 and A 16-byte aligned; VC: N % 4 == 0 and C 16-byte aligned
struct SyrkPolicy {
  int M, N, K;  // M == N
  const float* __restrict__ A;
  float* __restrict__ C;
  static constexpr bool kTransposedB = true;
  static constexpr bool kUpperTriangle = true;
  struct RowCtx {};
  using KCtx = int;  // the k index itself
  __device__ __forceinline__ RowCtx row_ctx(int) const { return RowCtx(); }
  __device__ __forceinline__ KCtx k_ctx(int k) const { return k; }
  __device__ __forceinline__ void k_advance(KCtx& k, int step) const { k += step; }
  __device__ __forceinline__ float4 load_row(int row, int k) const {
    float4 v = zero4();
    if (row < N) {
      const float* p = A + (int64_t)row * K + k;
      if (VA) {
        if (k < K) v = ldg4(p);
      } else {
        if (k + 0 < K) v.x = __ldg(p + 0);
        if (k + 1 < K) v.y = __ldg(p + 1);
        if (k + 2 < K) v.z = __ldg(p + 2);
        if (k + 3 < K) v.w = __ldg(p + 3);
      }
    }
    return v;
  }
  __device__ __forceinline__ float4 load_a(const RowCtx&, int row, int k) const { return load_row(row, k); }
  __device__ __forceinline__ float4 load_bt(int n, int k) const { return load_row(n, k); }
  __device__ __forceinline__ void copy_b(float*, int, int) const {}
  __device__ __forceinline__ float4 init(int row, int col) const {
    float4 v = zero4();
    if (row >= N || col + 3 < row) return v;  // outside, or a quad entirely below the diagonal
    const float* p = C + (int64_t)row * N + col;
    if (VC && col >= row) {
      if (col < N) v = *reinterpret_cast<const float4*>(p);
    } else {
      if (col + 0 < N && col + 0 >= row) v.x = p[0];
      if (col + 1 < N && col + 1 >= row) v.y = p[1];
      if (col + 2 < N && col + 2 >= row) v.z = p[2];
      if (col + 3 < N && col + 3 >= row) v.w = p[3];
    }
    return v;
  }
  __device__ __forceinline__ void store(int row, int col, float4 v) const {
    if (row >= N || col + 3 < row) return;
    float* p = C + (int64_t)row * N + col;
    if (VC && col >= row) {
      if (col < N) *reinterpret_cast<float4*>(p) = v;
    } else {
      if (col + 0 < N && col + 0 >= row) p[0] = v.x;
      if (col + 1 < N && col + 1 >= row) p[1] = v.y;
      if (col + 2 < N && col + 2 >= row) p[2] = v.z;
      if (col + 3 < N && col + 3 >= row) p[3] = v.w;
    }
  }
};

}  // namespace

cudaError_t launch_ssyrk_ffma(exo_b200_Context* ctx, int64_t N, int64_t K, const float* A, float* C) {
  if (N > INT32_MAX || K > INT32_MAX) return cudaErrorInvalidValue;
  const bool va = (K % 4 == 0) && ffma::aligned16(A);
  const bool vc = (N % 4 == 0) && ffma::aligned16(C);
  const int sms = ctx->sm_count;
#define EXOB200_SYRK(VA_, VC_) \
  return ffma::launch_tiles(ctx->stream, SyrkPolicy<VA_, VC_>{(int)N, (int)N, (int)K, A, C}, sms)
  if (va && vc) EXOB200_SYRK(true, true);
  if (va) EXOB200_SYRK(true, false);
  if (vc) EXOB200_SYRK(false, true);
  EXOB200_SYRK(false, false);
#undef EXOB200_SYRK
}

}  // namespace exob200
