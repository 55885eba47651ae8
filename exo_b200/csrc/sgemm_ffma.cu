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
// Skinny-M kernel (M <= 32): bandwidth bound -- B is streamed exactly once.
//
// A CTA owns a strip of 64 output columns (and up to 32 rows) for the whole K
// loop, so every output is still one thread's sequential-k FMA chain.  B (and
// the matching K chunk of A, stored k-major) flow through a deep ring of
// shared-memory stages filled by cp.async: with 9 stages of 32 K-rows a CTA
// keeps 64 KB of B loads in flight, and two CTAs fit per SM, which is what it
// takes to cover HBM latency when the only parallelism is across N.
// Thread (cq, rg): column quad cq (16 per strip) x row group rg (8 groups of 4
// rows): 16 accumulators, per k one 128-bit load of B, one of A, 16 FMAs.
constexpr int SK_W = 64;        // columns per CTA
constexpr int SK_KS = 32;       // K rows per stage
constexpr int SK_STAGES = 9;    // 108 KiB of shared memory: two CTAs per SM
constexpr int SK_THREADS = 128;
constexpr int SK_SMEM = SK_STAGES * (SK_KS * SK_W + SK_KS * 32) * (int)sizeof(float);  // 9 x 12 KiB

template <bool VB>
__global__ void __launch_bounds__(SK_THREADS)
sgemm_skinny_kernel(int M, int N, int K, const float* __restrict__ A, const float* __restrict__ B,
                    float* __restrict__ C) {
  extern __shared__ __align__(16) float sk_smem[];
  float(*Bs)[SK_KS][SK_W] = reinterpret_cast<float(*)[SK_KS][SK_W]>(sk_smem);
  float(*As)[SK_KS][32] = reinterpret_cast<float(*)[SK_KS][32]>(sk_smem + SK_STAGES * SK_KS * SK_W);

  const int tid = threadIdx.x;
  const int cq = tid & 15, rg = tid >> 4;
  const int n0 = blockIdx.x * SK_W, m0 = blockIdx.y * 32;
  const int col = n0 + cq * 4;
  const int rows_here = min(32, M - m0);
  const bool live = rg * 4 < rows_here;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int r = m0 + rg * 4 + i, c = col + j;
      acc[i][j] = (r < M && c < N) ? C[(int64_t)r * N + c] : 0.f;
    }

  const int nstages = (K + SK_KS - 1) / SK_KS;
  auto issue = [&](int st) {
    if (st < nstages) {
      const int buf = st % SK_STAGES, k0 = st * SK_KS;
      // B: 32 k-rows x 16 quads = 512 quads, 4 per thread
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int e = tid + i * SK_THREADS;
        const int kk = e >> 4, q = e & 15;
        const int k = k0 + kk, c = n0 + q * 4;
        const bool kin = k < K;
        const float* src = B + (kin ? (int64_t)k * N : 0);
        if (VB) {
          const bool ok = kin && c < N;
          ffma::cp_async16(&Bs[buf][kk][q * 4], src + (ok ? c : 0), ok);
        } else {
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const bool ok = kin && c + j < N;
            ffma::cp_async4(&Bs[buf][kk][q * 4 + j], src + (ok ? c + j : 0), ok);
          }
        }
      }
      // A chunk, stored k-major: As[kk][row]; consecutive threads walk k within a row
      for (int e = tid; e < rows_here * SK_KS; e += SK_THREADS) {
        const int r = e / SK_KS, kk = e - r * SK_KS;
        const bool ok = k0 + kk < K;
        ffma::cp_async4(&As[buf][kk][r], A + (int64_t)(m0 + r) * K + (ok ? k0 + kk : 0), ok);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  for (int st = 0; st < SK_STAGES - 1; st++) issue(st);
  for (int st = 0; st < nstages; st++) {
    asm volatile("cp.async.wait_group %0;" ::"n"(SK_STAGES - 2) : "memory");
    __syncthreads();               // stage st has landed for every thread; stage st-1 is free
    issue(st + SK_STAGES - 1);     // refill the buffer that stage st-1 used
    if (live) {
      const int buf = st % SK_STAGES;
      const int kmax = min(SK_KS, K - st * SK_KS);
      auto step = [&](int kk) {
        const float4 b = *reinterpret_cast<const float4*>(&Bs[buf][kk][cq * 4]);
        const float4 a = *reinterpret_cast<const float4*>(&As[buf][kk][rg * 4]);
        const float av[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
          acc[i][0] = fmaf(av[i], b.x, acc[i][0]);
          acc[i][1] = fmaf(av[i], b.y, acc[i][1]);
          acc[i][2] = fmaf(av[i], b.z, acc[i][2]);
          acc[i][3] = fmaf(av[i], b.w, acc[i][3]);
        }
      };
      if (kmax == SK_KS) {
#pragma unroll
        for (int kk = 0; kk < SK_KS; kk++) step(kk);
      } else {
        for (int kk = 0; kk < kmax; kk++) step(kk);  // ragged K tail: no padded steps
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int r = m0 + rg * 4 + i, c = col + j;
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
    dim3 grid((unsigned)((N + SK_W - 1) / SK_W), (unsigned)((M + 31) / 32));
    cudaError_t e;
    if (vb) {
      e = cudaFuncSetAttribute(sgemm_skinny_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SK_SMEM);
      if (e != cudaSuccess) return e;
      sgemm_skinny_kernel<true><<<grid, SK_THREADS, SK_SMEM, stream>>>((int)M, (int)N, (int)K, A, B, C);
    } else {
      e = cudaFuncSetAttribute(sgemm_skinny_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SK_SMEM);
      if (e != cudaSuccess) return e;
      sgemm_skinny_kernel<false><<<grid, SK_THREADS, SK_SMEM, stream>>>((int)M, (int)N, (int)K, A, B, C);
    }
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
