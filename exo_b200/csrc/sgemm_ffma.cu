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
#include "tc_common.cuh"
#include "umma.cuh"

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
  static constexpr bool kTransposedB = false;
  static constexpr bool kUpperTriangle = false;
  struct RowCtx {};
  using KCtx = int;  // the k index itself
  __device__ __forceinline__ RowCtx row_ctx(int) const { return RowCtx(); }
  __device__ __forceinline__ KCtx k_ctx(int k) const { return k; }
  __device__ __forceinline__ void k_advance(KCtx& k, int step) const { k += step; }
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

// RPT rows per thread: 4 (eight row groups: up to 32 rows), or 2 (up to 16 rows) for the at most 8 rows the
// default dispatch sends here -- with four rows per thread those keep one warp of the four busy.  Measured, us,
// 4 / 2 / 1 rows per thread: 8 x 8192 x 512 14.1 / 12.4 / 13.1; 8 x 8192 x 4096 101.8 / 83.7 / 87.7;
// 8 x 32768 x 512 31.1 / 31.4 / 39.9 (one row per thread needs a shared-memory load per four FMAs).
template <bool VB, int RPT>
__global__ void __launch_bounds__(SK_THREADS)
sgemm_skinny_kernel(int M, int N, int K, const float* __restrict__ A, const float* __restrict__ B,
                    float* __restrict__ C) {
  extern __shared__ __align__(16) float sk_smem[];
  float(*Bs)[SK_KS][SK_W] = reinterpret_cast<float(*)[SK_KS][SK_W]>(sk_smem);
  float(*As)[SK_KS][32] = reinterpret_cast<float(*)[SK_KS][32]>(sk_smem + SK_STAGES * SK_KS * SK_W);

  const int tid = threadIdx.x;
  const int cq = tid & 15, rg = tid >> 4;
  const int n0 = blockIdx.x * SK_W, m0 = blockIdx.y * (8 * RPT);
  const int col = n0 + cq * 4;
  const int rows_here = min(8 * RPT, M - m0);
  const bool live = rg * RPT < rows_here;

  float acc[RPT][4];
#pragma unroll
  for (int i = 0; i < RPT; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int r = m0 + rg * RPT + i, c = col + j;
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
        float av[4];
        if constexpr (RPT == 4) {
          const float4 a = *reinterpret_cast<const float4*>(&As[buf][kk][rg * 4]);
          av[0] = a.x, av[1] = a.y, av[2] = a.z, av[3] = a.w;
        } else {
          const float2 a = *reinterpret_cast<const float2*>(&As[buf][kk][rg * 2]);
          av[0] = a.x, av[1] = a.y;
        }
#pragma unroll
        for (int i = 0; i < RPT; i++) {
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
  for (int i = 0; i < RPT; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int r = m0 + rg * RPT + i, c = col + j;
      if (r < M && c < N) C[(int64_t)r * N + c] = acc[i][j];
    }
}

// --------------------------------------------------------------------------
// GEMV-like kernel (M <= 4): the same ring, narrower strips.  With so few rows
// the FMA work is negligible and the job is to keep HBM busy, so a CTA takes only
// 32 columns (N = 8192 gives 256 CTAs) and 16 stages of 32 K-rows; one warp walks
// K (thread = column, up to 4 rows, one chain each), all four warps feed the ring.
constexpr int GV_W = 32, GV_KS = 32, GV_STAGES = 16, GV_THREADS = 128;
constexpr int GV_SMEM = GV_STAGES * (GV_KS * GV_W + GV_KS * 4) * (int)sizeof(float);  // 72 KiB

template <bool VB>
__global__ void __launch_bounds__(GV_THREADS)
sgemm_gemv_kernel(int M, int N, int K, const float* __restrict__ A, const float* __restrict__ B,
                  float* __restrict__ C) {
  extern __shared__ __align__(16) float gv_smem[];
  float(*Bs)[GV_KS][GV_W] = reinterpret_cast<float(*)[GV_KS][GV_W]>(gv_smem);
  float(*As)[GV_KS][4] = reinterpret_cast<float(*)[GV_KS][4]>(gv_smem + GV_STAGES * GV_KS * GV_W);

  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * GV_W;
  const int col = n0 + tid;  // compute threads: tid < 32
  const bool compute = tid < GV_W;

  float acc[4];
#pragma unroll
  for (int i = 0; i < 4; i++) acc[i] = (compute && i < M && col < N) ? C[(int64_t)i * N + col] : 0.f;

  const int nstages = (K + GV_KS - 1) / GV_KS;
  auto issue = [&](int st) {
    if (st < nstages) {
      const int buf = st % GV_STAGES, k0 = st * GV_KS;
      // B: 32 k-rows x 8 quads = 256 quads, 2 per thread
#pragma unroll
      for (int i = 0; i < 2; i++) {
        const int e = tid + i * GV_THREADS;
        const int kk = e >> 3, q = e & 7;
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
      // A chunk k-major: As[kk][row]
      if (tid < 4 * GV_KS) {
        const int r = tid / GV_KS, kk = tid % GV_KS;
        const bool ok = r < M && k0 + kk < K;
        ffma::cp_async4(&As[buf][kk][r], A + (ok ? (int64_t)r * K + k0 + kk : 0), ok);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  for (int st = 0; st < GV_STAGES - 1; st++) issue(st);
  for (int st = 0; st < nstages; st++) {
    asm volatile("cp.async.wait_group %0;" ::"n"(GV_STAGES - 2) : "memory");
    __syncthreads();
    issue(st + GV_STAGES - 1);
    if (compute) {
      const int buf = st % GV_STAGES;
      const int kmax = min(GV_KS, K - st * GV_KS);
      auto step = [&](int kk) {
        const float b = Bs[buf][kk][tid];
        const float4 a = *reinterpret_cast<const float4*>(&As[buf][kk][0]);
        acc[0] = fmaf(a.x, b, acc[0]);
        acc[1] = fmaf(a.y, b, acc[1]);
        acc[2] = fmaf(a.z, b, acc[2]);
        acc[3] = fmaf(a.w, b, acc[3]);
      };
      if (kmax == GV_KS) {
#pragma unroll
        for (int kk = 0; kk < GV_KS; kk++) step(kk);
      } else {
        for (int kk = 0; kk < kmax; kk++) step(kk);
      }
    }
  }
  if (compute && col < N) {
#pragma unroll
    for (int i = 0; i < 4; i++)
      if (i < M) C[(int64_t)i * N + col] = acc[i];
  }
}

// --------------------------------------------------------------------------
// GEMV-like kernel, TMA-fed (M <= 2, N % 4 == 0): the HBM-bound shape.
// B streams through a ring of 16 KB fp32 boxes (64 columns x 64 K-rows, or 32 x 128) filled by one producer thread
// with tiled TMA loads (one instruction per 16 KB instead of 1024 cp.async);
// full/empty mbarriers replace the per-stage CTA barrier, so the two consumer
// warps (thread = column) never wait for the loaders.  Each stage's slice of A's
// few rows rides the same ring (a bulk copy per row beside the box, when A is
// 16-byte aligned and K % 4 == 0; 1 x 4096 x 8192: 45.7 -> 40.9 us, 1 x 8192 x 8192:
// 58.4 -> 56.6 us); otherwise the consumers read them from global memory.  Chain
// order per output is unchanged: k ascending, starting from C.
constexpr int GT_STAGES = 6;
constexpr int GT_STAGE_BYTES = 16384;  // one box: W columns x (4096 / W) K-rows of fp32
constexpr int GT_A_STAGE_BYTES = 2 * 128 * 4;  // one stage's A values: <= 2 rows x <= 128 k
constexpr int GT_A_BYTES = GT_STAGES * GT_A_STAGE_BYTES;
constexpr int GT_SMEM = GT_STAGES * GT_STAGE_BYTES + GT_A_BYTES + 1024 + 128;

// Untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completion on an mbarrier.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// MR = M (1 or 2), unrolled without predicates; W = strip width: 64, or 32 when N
// is too small to give every SM a 64-column strip.
// a_bulk: A's base is 16-byte aligned and K % 4 == 0, so each stage's slice of A's rows rides the ring as well
// (a bulk copy per row beside the box of B); otherwise the consumers fetch A themselves.
template <int MR, int W>
__global__ void __launch_bounds__(W + 32)
sgemm_gemv_tma_kernel(const __grid_constant__ CUtensorMap tmB, int N, int K, const float* __restrict__ A,
                      float* __restrict__ C, DeviceStatus* status, int a_bulk) {
  constexpr int GT_W = W, GT_KS = 4096 / W, AR = GT_KS / 32;  // AR: A values per lane per row
  using namespace umma;
  extern __shared__ uint8_t gt_raw[];
  const uint32_t raw = smem_u32(gt_raw);
  const uint32_t base = (raw + 127u) & ~127u;
  const float* tiles = reinterpret_cast<const float*>(gt_raw + (base - raw));
  const uint32_t bars = base + GT_STAGES * GT_STAGE_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (GT_STAGES + s); };
  volatile int* abort_flag =
      reinterpret_cast<volatile int*>(gt_raw + (base - raw) + GT_STAGES * GT_STAGE_BYTES + 16 * GT_STAGES);
  // A values: GT_STAGES areas of MR x GT_KS floats (with a_bulk, filled by the producer per stage; without, the
  // first two areas serve as the per-warp scratch of the consumers)
  float* a_area = reinterpret_cast<float*>(gt_raw + (base - raw) + GT_STAGES * GT_STAGE_BYTES + 256);
  const uint32_t a_area_addr = base + GT_STAGES * GT_STAGE_BYTES + 256;

  const int tid = threadIdx.x, warp = tid >> 5;
  const int n0 = blockIdx.x * GT_W;
  if (tid == 0) {
    for (int s = 0; s < GT_STAGES; s++) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), W / 32);  // one arrival per consumer warp
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  __syncthreads();
  const int nstages = (K + GT_KS - 1) / GT_KS;

  if (warp == W / 32) {
    if (tid == W) {
      prefetch_tensormap(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      for (int st = 0; st < nstages; st++) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, tc::WAIT_LIMIT_NS)) {
          tc::report_timeout(status, abort_flag, 31);
          break;
        }
        const int k0 = st * GT_KS;
        const uint32_t a_bytes = a_bulk ? (uint32_t)min(GT_KS, K - k0) * 4u : 0u;
        mbar_arrive_expect_tx(full_bar(stage), GT_STAGE_BYTES + MR * a_bytes);
        tma_load_2d(base + stage * GT_STAGE_BYTES, &tmB, full_bar(stage), n0, k0);
        if (a_bulk) {
#pragma unroll
          for (int i = 0; i < MR; i++)
            bulk_load_1d(a_area_addr + (uint32_t)(stage * GT_A_STAGE_BYTES + i * GT_KS * 4), A + (int64_t)i * K + k0,
                         a_bytes, full_bar(stage));
        }
        if (++stage == GT_STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else {
    const int col = n0 + tid;
    const int lane = tid & 31;
    float acc[MR];
#pragma unroll
    for (int i = 0; i < MR; i++) acc[i] = (col < N) ? C[(int64_t)i * N + col] : 0.f;
    // A's K chunk for a stage lives in registers, 2 values per lane per row (lane l holds
    // k0 + l and k0 + 32 + l), and is handed out by warp shuffles; the next stage's
    // values are requested before the current stage is multiplied.
    auto load_a = [&](int k0, float (&ar)[MR][AR]) {
#pragma unroll
      for (int i = 0; i < MR; i++)
#pragma unroll
        for (int h = 0; h < AR; h++) {
          const int k = k0 + h * 32 + lane;
          ar[i][h] = k < K ? __ldg(A + (int64_t)i * K + k) : 0.f;
        }
    };
    float acur[MR][AR], anext[MR][AR];
    if (!a_bulk) load_a(0, acur);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int st = 0; st < nstages && ok; st++) {
      if (!a_bulk) load_a((st + 1) * GT_KS, anext);
      if (!mbar_wait(full_bar(stage), phase, abort_flag, tc::WAIT_LIMIT_NS)) {
        if (lane == 0) tc::report_timeout(status, abort_flag, 32);
        ok = false;
        break;
      }
      const float* bs = tiles + stage * (GT_KS * GT_W) + tid;
      const int kmax = min(GT_KS, K - st * GT_KS);
      if (kmax == GT_KS) {
        // This stage's A values go through a small per-warp area of shared memory: lane l
        // writes the values it holds, then every lane reads four consecutive k at a time
        // as one broadcast 128-bit load.  That is 1.25 shared-memory instructions per k
        // step instead of a load plus a shuffle (the loop is bound by that pipe and by the
        // 4-clock chain, not by issue slots).
        float* aw = a_bulk ? a_area + stage * (GT_A_STAGE_BYTES / 4) : a_area + warp * (GT_A_STAGE_BYTES / 4);
        if (!a_bulk) {
          __syncwarp();  // every lane is done with the previous stage's values
#pragma unroll
          for (int i = 0; i < MR; i++)
#pragma unroll
            for (int h = 0; h < AR; h++) aw[i * GT_KS + h * 32 + lane] = acur[i][h];
          __syncwarp();
        }
#pragma unroll
        for (int k0 = 0; k0 < GT_KS; k0 += 16) {
          float bv[16];
          float4 av[MR][4];
#pragma unroll
          for (int j = 0; j < 16; j++) bv[j] = bs[(k0 + j) * GT_W];
#pragma unroll
          for (int i = 0; i < MR; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) av[i][j] = *reinterpret_cast<const float4*>(aw + i * GT_KS + k0 + 4 * j);
#pragma unroll
          for (int j = 0; j < 4; j++)
#pragma unroll
            for (int i = 0; i < MR; i++) {
              acc[i] = fmaf(av[i][j].x, bv[4 * j + 0], acc[i]);
              acc[i] = fmaf(av[i][j].y, bv[4 * j + 1], acc[i]);
              acc[i] = fmaf(av[i][j].z, bv[4 * j + 2], acc[i]);
              acc[i] = fmaf(av[i][j].w, bv[4 * j + 3], acc[i]);
            }
        }
      } else {
        for (int kk = 0; kk < kmax; kk++) {  // ragged K tail: no padded steps
          const float b = bs[kk * GT_W];
#pragma unroll
          for (int i = 0; i < MR; i++) {
            float a = 0.f;
            if (a_bulk) {
              a = a_area[stage * (GT_A_STAGE_BYTES / 4) + i * GT_KS + kk];
            } else {
#pragma unroll
              for (int h = 0; h < AR; h++) {
                const float v = __shfl_sync(0xffffffffu, acur[i][h], kk & 31);
                if ((kk >> 5) == h) a = v;
              }
            }
            acc[i] = fmaf(a, b, acc[i]);
          }
        }
      }
      if (!a_bulk) {
#pragma unroll
        for (int i = 0; i < MR; i++)
#pragma unroll
          for (int h = 0; h < AR; h++) acur[i][h] = anext[i][h];
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar(stage));
      if (++stage == GT_STAGES) {
        stage = 0;
        phase ^= 1u;
      }
    }
    if (ok && col < N) {
#pragma unroll
      for (int i = 0; i < MR; i++) C[(int64_t)i * N + col] = acc[i];
    }
  }
}

// --------------------------------------------------------------------------
// Tall kernel (N <= 16, many rows): the mirror image of the skinny kernel.  A is
// streamed exactly once; a thread owns one row of C (all N columns, N <= 16
// accumulators), so the chain order is unchanged.  A CTA takes ROWS = 128 rows; the K chunk of A (ROWS x 32 k, row
// pitch 36 floats so that a quarter-warp's 128-bit reads are conflict free) and of B
// (32 k x 32 columns) flow through a cp.async ring.
constexpr int TL_KS = 32, TL_STAGES = 5, TL_PITCH = 36;
template <int ROWS>
__host__ __device__ constexpr int tl_stage_floats() { return ROWS * TL_PITCH + TL_KS * 32; }
template <int ROWS>
__host__ __device__ constexpr int tl_smem() { return TL_STAGES * tl_stage_floats<ROWS>() * (int)sizeof(float); }  // 110 KiB / 42.5 KiB

// NQ = ceil(N / 4): column quads per row, 1..4.  A thread owns QPT quads of one row (NQ / QPT threads per row,
// in adjacent lanes, which read the row's A value as one broadcast): with a whole row per thread there were
// only M / 32 warps, two per scheduler, and the k step waited on its shared-memory loads (ncu on
// 32768 x 8 x 512: short-scoreboard stalls 1.9 per issue, 33 % issue active).  Measured, us, quads per thread
// 1 / 2 / 4: 32768 x 8 x 512 21.1 / 24.6 / -; 16384 x 16 x 512 26.0 / 18.4 / 23.2; 32768 x 16 x 2048
// 178 / 102 / 118; 4096 x 8 x 4096 89.7 / 120.8 / -; 20000 x 12 x 300 (three quads) 26.1 for one, 20.5 for all
// three per thread.  Hence one quad per thread up to N = 8, two for N = 13 .. 16, the row for N = 9 .. 12.
template <int NQ, int QPT, int ROWS>  // QPT: quads per thread (NQ / QPT threads per row)
__global__ void __launch_bounds__(ROWS * (NQ / QPT))
sgemm_tall_kernel(int M, int N, int K, const float* __restrict__ A, const float* __restrict__ B,
                  float* __restrict__ C, int a_vec, int b_vec) {
  static_assert(NQ % QPT == 0, "whole threads per row");
  extern __shared__ __align__(16) float tl_smem_buf[];
  constexpr int STAGE = tl_stage_floats<ROWS>();
  constexpr int TPR = NQ / QPT;  // threads per row
  constexpr int THREADS = ROWS * TPR;
  const int tid = threadIdx.x;
  const int m0 = blockIdx.x * ROWS;
  const int r_local = tid / TPR, q0 = (tid % TPR) * QPT;
  const int row = m0 + r_local;

  uint64_t acc2[QPT][2];
#pragma unroll
  for (int q = 0; q < QPT; q++) {
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; j++)
      v[j] = (row < M && (q0 + q) * 4 + j < N) ? C[(int64_t)row * N + (q0 + q) * 4 + j] : 0.f;
    acc2[q][0] = ffma::pack2(v[0], v[1]);
    acc2[q][1] = ffma::pack2(v[2], v[3]);
  }

  const int nstages = (K + TL_KS - 1) / TL_KS;
  auto issue = [&](int st) {
    if (st < nstages) {
      float* as = tl_smem_buf + (st % TL_STAGES) * STAGE;
      float* bs = as + ROWS * TL_PITCH;
      const int k0 = st * TL_KS;
      // A: ROWS rows x 8 k-quads; 8 consecutive threads cover one row segment
#pragma unroll
      for (int i = 0; i < (ROWS * 8 + THREADS - 1) / THREADS; i++) {
        const int e = tid + i * THREADS;
        if ((ROWS * 8) % THREADS != 0 && e >= ROWS * 8) break;
        const int r = e >> 3, kq = (e & 7) * 4;
        const bool rin = m0 + r < M;
        const float* src = A + (rin ? (int64_t)(m0 + r) * K : 0);
        if (a_vec) {
          const bool ok = rin && k0 + kq < K;  // K % 4 == 0
          ffma::cp_async16(as + r * TL_PITCH + kq, src + (ok ? k0 + kq : 0), ok);
        } else {
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const bool ok = rin && k0 + kq + j < K;
            ffma::cp_async4(as + r * TL_PITCH + kq + j, src + (ok ? k0 + kq + j : 0), ok);
          }
        }
      }
      // B: 32 k x 32 columns (zero beyond N)
      if (b_vec) {  // N % 4 == 0
        for (int e = tid; e < TL_KS * 8; e += THREADS) {
          const int kk = e >> 3, c = (e & 7) * 4;
          const bool ok = k0 + kk < K && c < N;
          ffma::cp_async16(bs + kk * 32 + c, B + (ok ? (int64_t)(k0 + kk) * N + c : 0), ok);
        }
      } else {
        for (int e = tid; e < TL_KS * 32; e += THREADS) {
          const int kk = e >> 5, c = e & 31;
          const bool ok = k0 + kk < K && c < N;
          ffma::cp_async4(bs + kk * 32 + c, B + (ok ? (int64_t)(k0 + kk) * N + c : 0), ok);
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  for (int st = 0; st < TL_STAGES - 1; st++) issue(st);
  for (int st = 0; st < nstages; st++) {
    asm volatile("cp.async.wait_group %0;" ::"n"(TL_STAGES - 2) : "memory");
    __syncthreads();
    issue(st + TL_STAGES - 1);
    const float* as = tl_smem_buf + (st % TL_STAGES) * STAGE + r_local * TL_PITCH;
    const float* bs = tl_smem_buf + (st % TL_STAGES) * STAGE + ROWS * TL_PITCH + q0 * 4;
    const int kmax = min(TL_KS, K - st * TL_KS);
    auto step = [&](float a, int kk) {
      const uint64_t aa = ffma::pack2(a, a);
#pragma unroll
      for (int q = 0; q < QPT; q++) {
        const ulonglong2 bv = *reinterpret_cast<const ulonglong2*>(bs + kk * 32 + q * 4);
        acc2[q][0] = ffma::fma2(aa, bv.x, acc2[q][0]);
        acc2[q][1] = ffma::fma2(aa, bv.y, acc2[q][1]);
      }
    };
    if (kmax == TL_KS) {
#pragma unroll
      for (int k4 = 0; k4 < TL_KS; k4 += 4) {
        const float4 av = *reinterpret_cast<const float4*>(as + k4);
        step(av.x, k4 + 0);
        step(av.y, k4 + 1);
        step(av.z, k4 + 2);
        step(av.w, k4 + 3);
      }
    } else {
      for (int kk = 0; kk < kmax; kk++) step(as[kk], kk);  // ragged K tail: no padded steps
    }
  }
  if (row < M) {
#pragma unroll
    for (int q = 0; q < QPT; q++) {
      float v[4];
      ffma::unpack2(acc2[q][0], v[0], v[1]);
      ffma::unpack2(acc2[q][1], v[2], v[3]);
#pragma unroll
      for (int j = 0; j < 4; j++)
        if ((q0 + q) * 4 + j < N) C[(int64_t)row * N + (q0 + q) * 4 + j] = v[j];
    }
  }
}

template <int NQ, int QPT, int ROWS>
cudaError_t launch_tall_r(int device, cudaStream_t stream, int M, int N, int K, const float* A, const float* B,
                          float* C, int a_vec, int b_vec) {
  EXOB200_SMEM_ATTR_ONCE((sgemm_tall_kernel<NQ, QPT, ROWS>), tl_smem<ROWS>(), device);
  sgemm_tall_kernel<NQ, QPT, ROWS><<<(unsigned)((M + ROWS - 1) / ROWS), ROWS * (NQ / QPT), tl_smem<ROWS>(), stream>>>(
      M, N, K, A, B, C, a_vec, b_vec);
  return cudaGetLastError();
}

template <int NQ>
cudaError_t launch_tall(int device, cudaStream_t stream, int M, int N, int K, const float* A, const float* B, float* C,
                        int a_vec, int b_vec) {
  static const int force = [] {
    const char* e = getenv("EXOB200_TALL_QPT");  // quads per thread (timing experiments); 0 / unset: the default
    return e ? atoi(e) : 0;
  }();
  // 32-row (one warp) CTAs were measured too: slower than 128-row CTAs from 8192 rows up, equal below
  if constexpr (NQ == 1) {
    return launch_tall_r<1, 1, 128>(device, stream, M, N, K, A, B, C, a_vec, b_vec);
  } else if constexpr (NQ == 3) {  // three threads per row straddle warps: the whole row per thread is faster here
    if (force == 1) return launch_tall_r<3, 1, 128>(device, stream, M, N, K, A, B, C, a_vec, b_vec);
    return launch_tall_r<3, 3, 128>(device, stream, M, N, K, A, B, C, a_vec, b_vec);
  } else if constexpr (NQ == 2) {
    if (force == 2) return launch_tall_r<2, 2, 128>(device, stream, M, N, K, A, B, C, a_vec, b_vec);
    return launch_tall_r<2, 1, 128>(device, stream, M, N, K, A, B, C, a_vec, b_vec);
  } else {
    if (force == 1) return launch_tall_r<4, 1, 128>(device, stream, M, N, K, A, B, C, a_vec, b_vec);
    if (force == 4) return launch_tall_r<4, 4, 128>(device, stream, M, N, K, A, B, C, a_vec, b_vec);
    return launch_tall_r<4, 2, 128>(device, stream, M, N, K, A, B, C, a_vec, b_vec);
  }
}

}  // namespace

namespace {
int skinny_max_rows() {
  static const int n = [] {
    const char* e = getenv("EXOB200_SKINNY_MAX_M");  // rows up to which the skinny kernel is used (timing experiments)
    return e ? atoi(e) : 8;
  }();
  return n;
}
bool gemv_tma_enabled() {
  static const bool on = [] {
    const char* e = getenv("EXOB200_GEMV_TMA");  // =0: use the cp.async ring instead (timing experiments)
    return !(e && e[0] == '0');
  }();
  return on;
}
}  // namespace

// Which kernel the exact SGEMM takes for a shape (va / vb: 16-byte aligned operands with K % 4 == 0 / N % 4 == 0):
// 1 tall, 2 TMA-fed GEMV, 3 cp.async GEMV, 4 skinny, otherwise the tile engine's configuration id.
int sgemm_ffma_plan(int64_t M, int64_t N, int64_t K, bool va, bool vb) {
  (void)va;
  if (N <= 16 && M >= 1024) return 1;
  if (gemv_tma_enabled() && M <= 2 && vb && K >= 512) return 2;
  if (M <= 4) return 3;
  if (M <= skinny_max_rows() && ((N >= 8192 && N <= 16384) || skinny_max_rows() != 8)) return 4;
  return ffma::choose_tile(SgemmPolicy<true, true>{(int)M, (int)N, (int)K, nullptr, nullptr, nullptr});
}

cudaError_t launch_sgemm_ffma(exo_b200_Context* ctx, int64_t M, int64_t N, int64_t K, const float* A,
                              const float* B, float* C) {
  cudaStream_t stream = ctx->stream;
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return cudaErrorInvalidValue;
  const bool va = (K % 4 == 0) && ffma::aligned16(A);
  const bool vb = (N % 4 == 0) && ffma::aligned16(B) && ffma::aligned16(C);
  const int plan = sgemm_ffma_plan(M, N, K, va, vb);
  if (plan == 1) {  // wider rows reuse too little of each B fragment here; the tile kernel takes them
    const int a_vec = va ? 1 : 0, b_vec = vb ? 1 : 0;
    const int m = (int)M, n = (int)N, k = (int)K;
    switch ((n + 3) / 4) {
      case 1: return launch_tall<1>(ctx->device, stream, m, n, k, A, B, C, a_vec, b_vec);
      case 2: return launch_tall<2>(ctx->device, stream, m, n, k, A, B, C, a_vec, b_vec);
      case 3: return launch_tall<3>(ctx->device, stream, m, n, k, A, B, C, a_vec, b_vec);
      default: return launch_tall<4>(ctx->device, stream, m, n, k, A, B, C, a_vec, b_vec);
    }
  }
  if (plan == 2) {
    const int W = (N + 63) / 64 >= 200 ? 64 : 32;
    CUtensorMap mb;
    cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)K};
    cuuint64_t strides[1] = {(cuuint64_t)N * 4};
    cuuint32_t box[2] = {(cuuint32_t)W, (cuuint32_t)(4096 / W)};
    if (!tc::make_tiled_map(&mb, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, B, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE))
      return cudaErrorUnknown;
    const unsigned grid = (unsigned)((N + W - 1) / W);
#define EXOB200_GEMV(MR_, W_)                                                                                      \
  {                                                                                                                \
    EXOB200_SMEM_ATTR_ONCE((sgemm_gemv_tma_kernel<MR_, W_>), GT_SMEM, ctx->device);                                \
    sgemm_gemv_tma_kernel<MR_, W_><<<grid, W_ + 32, GT_SMEM, stream>>>(mb, (int)N, (int)K, A, C, ctx->status_dev, \
                                                                       va ? 1 : 0);                                \
  }
    if (M == 1 && W == 64) EXOB200_GEMV(1, 64)
    else if (M == 1) EXOB200_GEMV(1, 32)
    else if (W == 64) EXOB200_GEMV(2, 64)
    else EXOB200_GEMV(2, 32)
#undef EXOB200_GEMV
    return cudaGetLastError();
  }
  if (plan == 3) {
    const unsigned grid = (unsigned)((N + GV_W - 1) / GV_W);
    if (vb) {
      EXOB200_SMEM_ATTR_ONCE(sgemm_gemv_kernel<true>, GV_SMEM, ctx->device);
      sgemm_gemv_kernel<true><<<grid, GV_THREADS, GV_SMEM, stream>>>((int)M, (int)N, (int)K, A, B, C);
    } else {
      EXOB200_SMEM_ATTR_ONCE(sgemm_gemv_kernel<false>, GV_SMEM, ctx->device);
      sgemm_gemv_kernel<false><<<grid, GV_THREADS, GV_SMEM, stream>>>((int)M, (int)N, (int)K, A, B, C);
    }
    return cudaGetLastError();
  }
  // The skinny kernel (a CTA per 64 columns, all rows) only beats the tile engine when there are very few rows
  // and enough columns for every SM.  From a dozen rows on the tile
  // engine's 32 x 32 tiles win although most of their rows are padding, because they give the machine two to
  // four times the CTAs: 17 x 4099 x 513 18.2 against 21.6 us, 32 x 8192 x 512 18.5 against 22.4,
  // 24 x 4096 x 1024 28.6 against 38.4, 32 x 2048 x 2048 55.6 against 86.2 (12 x 1000 x 700: a tie).
  if (plan == 4) {
#define EXOB200_SKINNY(VB_, RPT_)                                                                            \
  {                                                                                                        \
    dim3 grid((unsigned)((N + SK_W - 1) / SK_W), (unsigned)((M + 8 * RPT_ - 1) / (8 * RPT_)));             \
    EXOB200_SMEM_ATTR_ONCE((sgemm_skinny_kernel<VB_, RPT_>), SK_SMEM, ctx->device);                        \
    sgemm_skinny_kernel<VB_, RPT_><<<grid, SK_THREADS, SK_SMEM, stream>>>((int)M, (int)N, (int)K, A, B, C); \
  }
    if (M <= 8 && vb) EXOB200_SKINNY(true, 2)
    else if (M <= 8) EXOB200_SKINNY(false, 2)
    else if (vb) EXOB200_SKINNY(true, 4)
    else EXOB200_SKINNY(false, 4)
#undef EXOB200_SKINNY
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
