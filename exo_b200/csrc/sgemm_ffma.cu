// Exact-fp32 SIMT SGEMM:  C += A * B, all row-major, any M, N, K >= 1.
//
// Replaces sgemm_exo (apps/x86/sgemm/sgemm.py:11-23; generated code
// tests/golden/test_apps/test_x86_sgemm.txt:788-889).  The generated AVX-512
// microkernels compute every output element as ONE chain of fused
// multiply-adds in increasing k that starts from the incoming C value
// (_mm512_fmadd_ps, golden :437-454; k-blocking only round-trips the fp32
// partial).  The tile engine in ffma_tile.cuh keeps that chain, so results are
// bit-identical to the reference.  Global loads are 128-bit and coalesced when
// the row pitch allows it (K % 4 == 0 for A, N % 4 == 0 for B and C), scalar
// otherwise -- the ragged-shape path that stands in for the reference's masked
// right-panel / bottom-panel / corner kernels (golden :470-494, :543-737, :768-776).
#include "ffma_tile.cuh"
#include "kernels.cuh"

namespace exob200 {
namespace {

using ffma::ldg4;
using ffma::zero4;

template <bool VA, bool VB>
struct SgemmPolicy {
  int M, N, K;
  const float* __restrict__ A;
  const float* __restrict__ B;
  float* __restrict__ C;
  struct RowCtx {};
  __device__ __forceinline__ RowCtx row_ctx(int) const { return RowCtx(); }
  __device__ __forceinline__ float4 load_a(const RowCtx&, int row, int k) const {
    float4 v = zero4();
    if (row < M) {
      const float* p = A + (int64_t)row * K + k;
      if (VA) {
        if (k < K) v = ldg4(p);  // K % 4 == 0: a quad is entirely inside or outside
      } else {
        if (k + 0 < K) v.x = __ldg(p + 0);
        if (k + 1 < K) v.y = __ldg(p + 1);
        if (k + 2 < K) v.z = __ldg(p + 2);
        if (k + 3 < K) v.w = __ldg(p + 3);
      }
    }
    return v;
  }
  __device__ __forceinline__ void copy_b(float* smem, int k, int col) const {
    // Out-of-range sources are never dereferenced (src-size 0), but keep the
    // address inside the allocation anyway.
    const bool kin = k < K;
    const float* p = B + (kin ? (int64_t)k * N : 0);
    if (VB) {
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
  __device__ __forceinline__ float4 init(int row, int col) const {
    float4 v = zero4();
    if (row < M) {
      const float* p = C + (int64_t)row * N + col;
      if (VB) {
        if (col < N) v = *reinterpret_cast<const float4*>(p);
      } else {
        if (col + 0 < N) v.x = p[0];
        if (col + 1 < N) v.y = p[1];
        if (col + 2 < N) v.z = p[2];
        if (col + 3 < N) v.w = p[3];
      }
    }
    return v;
  }
  __device__ __forceinline__ void store(int row, int col, float4 v) const {
    if (row >= M) return;
    float* p = C + (int64_t)row * N + col;
    if (VB) {
      if (col < N) *reinterpret_cast<float4*>(p) = v;
    } else {
      if (col + 0 < N) p[0] = v.x;
      if (col + 1 < N) p[1] = v.y;
      if (col + 2 < N) p[2] = v.z;
      if (col + 3 < N) p[3] = v.w;
    }
  }
};

// --------------------------------------------------------------------------
// Skinny-M kernel (M <= 32): bandwidth bound, B is streamed exactly once.
// One thread owns `ROWS` x 4 outputs (4 adjacent columns, all rows of a 4- or
// 8-row slab) and walks K sequentially, so the chain order is unchanged.  A CTA
// covers 128 columns x up to 32 rows; A's slab rows for the current K chunk sit
// in shared memory and are read as broadcasts.  Loads of B for KU consecutive
// k are issued before the dependent FMAs so each thread keeps KU x 16 bytes in
// flight.
constexpr int SK_THREADS = 128;  // 32 column quads x 4 row slabs
constexpr int SK_KC = 64;        // K chunk staged in shared memory for A
constexpr int SK_KU = 8;         // B loads in flight per thread

template <bool VB>
__global__ void __launch_bounds__(SK_THREADS)
sgemm_skinny_kernel(int M, int N, int K, const float* __restrict__ A, const float* __restrict__ B,
                    float* __restrict__ C) {
  __shared__ float As[32][SK_KC + 1];
  const int tid = threadIdx.x;
  const int cq = tid & 31;           // column quad within the CTA
  const int slab = tid >> 5;         // 8-row slab (warp index): rows slab*8 .. +7
  const int col = blockIdx.x * 128 + cq * 4;
  const int r0 = blockIdx.y * 32 + slab * 8;
  const int row_base = blockIdx.y * 32;
  const bool slab_live = r0 < M;

  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int r = r0 + i, c = col + j;
      acc[i][j] = (r < M && c < N) ? C[(int64_t)r * N + c] : 0.f;
    }

  for (int k0 = 0; k0 < K; k0 += SK_KC) {
    const int kc = min(SK_KC, K - k0);
    __syncthreads();
    for (int e = tid; e < 32 * SK_KC; e += SK_THREADS) {
      const int r = e / SK_KC, k = e % SK_KC;
      As[r][k] = (row_base + r < M && k < kc) ? __ldg(A + (int64_t)(row_base + r) * K + k0 + k) : 0.f;
    }
    __syncthreads();
    if (!slab_live) continue;
    int k = 0;
    for (; k + SK_KU <= kc; k += SK_KU) {
      float4 b[SK_KU];
#pragma unroll
      for (int u = 0; u < SK_KU; u++) {
        const float* p = B + (int64_t)(k0 + k + u) * N + col;
        if (VB) {
          b[u] = col < N ? ldg4(p) : make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
          b[u].x = col + 0 < N ? __ldg(p + 0) : 0.f;
          b[u].y = col + 1 < N ? __ldg(p + 1) : 0.f;
          b[u].z = col + 2 < N ? __ldg(p + 2) : 0.f;
          b[u].w = col + 3 < N ? __ldg(p + 3) : 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < SK_KU; u++)
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const float a = As[slab * 8 + i][k + u];
          acc[i][0] = fmaf(a, b[u].x, acc[i][0]);
          acc[i][1] = fmaf(a, b[u].y, acc[i][1]);
          acc[i][2] = fmaf(a, b[u].z, acc[i][2]);
          acc[i][3] = fmaf(a, b[u].w, acc[i][3]);
        }
    }
    for (; k < kc; k++) {
      const float* p = B + (int64_t)(k0 + k) * N + col;
      float4 b;
      b.x = col + 0 < N ? __ldg(p + 0) : 0.f;
      b.y = col + 1 < N ? __ldg(p + 1) : 0.f;
      b.z = col + 2 < N ? __ldg(p + 2) : 0.f;
      b.w = col + 3 < N ? __ldg(p + 3) : 0.f;
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const float a = As[slab * 8 + i][k];
        acc[i][0] = fmaf(a, b.x, acc[i][0]);
        acc[i][1] = fmaf(a, b.y, acc[i][1]);
        acc[i][2] = fmaf(a, b.z, acc[i][2]);
        acc[i][3] = fmaf(a, b.w, acc[i][3]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int r = r0 + i, c = col + j;
      if (r < M && c < N) C[(int64_t)r * N + c] = acc[i][j];
    }
}

}  // namespace

cudaError_t launch_sgemm_ffma(cudaStream_t stream, int64_t M, int64_t N, int64_t K, const float* A,
                              const float* B, float* C) {
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return cudaErrorInvalidValue;
  const bool va = (K % 4 == 0) && ffma::aligned16(A);
  const bool vb = (N % 4 == 0) && ffma::aligned16(B) && ffma::aligned16(C);
  if (M <= 32) {
    dim3 grid((unsigned)((N + 127) / 128), (unsigned)((M + 31) / 32));
    if (vb)
      sgemm_skinny_kernel<true><<<grid, SK_THREADS, 0, stream>>>((int)M, (int)N, (int)K, A, B, C);
    else
      sgemm_skinny_kernel<false><<<grid, SK_THREADS, 0, stream>>>((int)M, (int)N, (int)K, A, B, C);
    return cudaGetLastError();
  }
#define EXOB200_LAUNCH(VA_, VB_) \
  return ffma::launch_tiles(stream, SgemmPolicy<VA_, VB_>{(int)M, (int)N, (int)K, A, B, C})
  if (va && vb) EXOB200_LAUNCH(true, true);
  if (va) EXOB200_LAUNCH(true, false);
  if (vb) EXOB200_LAUNCH(false, true);
  EXOB200_LAUNCH(false, false);
#undef EXOB200_LAUNCH
}

}  // namespace exob200
