// The exact-fp32 SIMT tile engine shared by the SGEMM and the implicit-GEMM
// convolution.  It computes, for a logical row-major problem
//     D[m, n] = finish( chain_k  fmaf(A(m, k), B(k, n), .) starting at init(m, n) )
// where each output element is owned by one thread for the whole reduction, so
// the reduction is one fused-multiply-add chain in increasing k -- the order
// the reference's generated microkernels use
// (tests/golden/test_apps/test_x86_sgemm.txt:437-454, test_x86_conv.txt:85-101).
// No split-K, and no padded steps along K (fmaf(0,0,c) would turn c = -0.0
// into +0.0), so results are bit-identical to the reference.
//
// Tiling: CTA tile 128x128, K step 16, 256 threads, each thread an 8x8
// register tile laid out as 2x2 quadrants of 4x4 so that every shared-memory
// read is a conflict-free 128-bit load.  A is stored k-major in shared memory
// so that the per-k A fragment is contiguous.  The next K tile is fetched
// (A into registers, B by cp.async) while the current one is multiplied, through
// a ring of shared-memory buffers with one barrier per tile: two buffers for the
// 8x8-per-thread configurations, three (two tiles of look-ahead) for the
// 4x4-per-thread ones, whose few warps per SM cannot hide a global load behind
// one tile's arithmetic.
//
// A Policy supplies the operand addressing:
//   int  M, N, K                       logical extents
//   RowCtx row_ctx(int m)              per-row state for the A loader (computed once)
//   KCtx k_ctx(int k), k_advance(KCtx&, int step)   a cursor along K: the engine walks K in steps of one
//                                      tile, so a policy whose k -> address map needs divisions (the
//                                      convolution's (ky, kx, ci)) pays them once and then only adds
//   float4 load_a(const RowCtx&, int m, const KCtx& k)   A(m, k..k+3), zero outside
//   void copy_b(float* smem, const KCtx& k, int n)   cp.async of B(k, n..n+3) into smem, zero outside
//   float4 init(int m, int n)          chain start for (m, n..n+3)
//   void store(int m, int n, float4)   applies the epilogue and writes (bounds-checked)
//   static constexpr bool kTransposedB B(k, n) is stored with k contiguous (an N x K row-major array):
//                                      the B tile then takes the A tile's route through registers,
//                                      with  float4 load_bt(int n, const KCtx& k)  = B(k..k+3, n), zero outside
//   static constexpr bool kUpperTriangle  only tiles that hold an element with n >= m exist: the grid
//                                      enumerates just those (a square problem, M == N)
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <algorithm>
#include <type_traits>

namespace exob200 {
namespace ffma {

constexpr int BK = 16;
// Tile sizes from one engine (TDY x TDX threads, each RM rows x 4 HN columns of outputs):
//   16 x 16 threads, 8 x 8 each -> 128 x 128, 256 threads: the throughput configuration;
//   16 x  8 threads, 8 x 8 each -> 128 x  64, 128 threads: medium problems, and when the 128 x 128 tiles
//     would leave a nearly empty last round;
//   16 x  8 threads, 4 x 8 each ->  64 x  64, 128 threads: when 128 x 64 tiles would put two CTAs on a few
//     SMs and one on the rest (tile counts just above the SM count);
//   16 x 16 threads, 4 x 4 each ->  64 x  64, 256 threads;
//    8 x  8 threads, 4 x 4 each ->  32 x  32,  64 threads, and
//   16 x  8 threads, 2 x 4 each ->  32 x  32, 128 threads, and
//    8 x 16 threads, 2 x 4 each ->  16 x  64, 128 threads (at most 16 rows), and
//    4 x 32 threads, 2 x 4 each ->   8 x 128, 128 threads (at most 8 rows): small problems.  Those are bound by the latency
//     of one warp's k loop, so spreading the same warps over more SMs (one or two per scheduler instead
//     of four) is what shortens them.
// launch_tiles() picks among them with a measured cost table.
// Without split-K, which the reference's per-element chain order rules out, parallelism only comes
// from M x N.

__device__ __forceinline__ float4 ldg4(const float* p) {
  return __ldg(reinterpret_cast<const float4*>(p));
}
__device__ __forceinline__ float4 zero4() { return make_float4(0.f, 0.f, 0.f, 0.f); }

// Asynchronous global -> shared copies; `valid` false zero-fills the destination.
__device__ __forceinline__ void cp_async16(float* smem, const float* g, bool valid) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(g), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async4(float* smem, const float* g, bool valid) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  const int n = valid ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(s), "l"(g), "r"(n) : "memory");
}

// Packed fp32 pairs: fma.rn.f32x2 performs two IEEE fused multiply-adds (one per
// 32-bit half, round-to-nearest, denormals kept) in ONE issue slot.  The SIMT
// SGEMM is issue-bound (one FFMA per slot, plus loads and address arithmetic),
// so pairing adjacent output columns halves the slots the FMAs need while every
// component still sees exactly fmaf(a, b, c).
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

// First tile column of tile row tm that holds an element on or above the diagonal (n >= m).
__host__ __device__ constexpr int first_live_tile_col(int tm, int bm, int bn) { return (tm * bm) / bn; }
// Number of tiles of an M x N problem; for an upper-triangular one only those that reach the diagonal.
template <class Policy>
inline int64_t count_tiles(const Policy& P, int bm, int bn) {
  const int64_t tiles_m = (P.M + bm - 1) / bm, tiles_n = (P.N + bn - 1) / bn;
  if (!Policy::kUpperTriangle) return tiles_m * tiles_n;
  int64_t n = 0;
  for (int64_t tm = 0; tm < tiles_m; tm++) n += std::max<int64_t>(0, tiles_n - first_live_tile_col((int)tm, bm, bn));
  return n;
}

// Resident CTAs per SM that the register budget is sized for.  8 x 8 outputs per thread need about
// 190 registers to keep a k step's fragments and the next tile's operands in flight without spilling:
// the 128-thread 128 x 64 configuration gets that (two CTAs per SM); the 256-thread 128 x 128 one is
// held to 128 registers so that two CTAs (16 warps) share an SM, which is worth more there than the
// few spilled values cost (measured at 8192^3: 55.3 against 48.4 TFLOP/s with one CTA per SM).
template <int RM, int HN, int THREADS>
__host__ __device__ constexpr int min_ctas() {
  return (RM * HN == 16 && THREADS == 128) ? 2 : 512 / THREADS;
}

// RM rows (2, 4 or 8) x 4 HN columns of outputs per thread, TDY x TDX threads.  The rows come as
// RM / QR quadrants of QR = min(RM, 4) consecutive rows, the columns as HN quadrants of 4.
template <class Policy, bool PACKED, int RM, int HN, int TDY, int TDX>
__global__ void __launch_bounds__(TDY * TDX, min_ctas<RM, HN, TDY * TDX>())
tile_kernel(const Policy P, int tiles_m, int tiles_n) {
  static_assert(RM == 2 || RM == 4 || RM == 8, "rows per thread");
  constexpr int THREADS = TDY * TDX;
  constexpr int QR = RM < 4 ? RM : 4, HM = RM / QR;
  constexpr int QSM = QR * TDY, QSN = 4 * TDX;  // rows / columns per quadrant
  constexpr int BM = QSM * HM, BN = QSN * HN;
  constexpr int AS_PITCH = BM + 4;  // floats; keeps 16-byte alignment, spreads the transposing stores
  constexpr int RN = 4 * HN;        // columns per thread
  static_assert((BM % (THREADS / 4) == 0 || BM < THREADS / 4) && BK % (THREADS / (BN / 4)) == 0,
                "the tile loaders cover whole passes (or, for A, part of one)");
  static_assert(!Policy::kTransposedB || BN % (THREADS / 4) == 0, "so does the register route of a transposed B");
  constexpr int BS_PITCH = Policy::kTransposedB ? BN + 4 : BN;  // the transposing stores want the same skew as A's
  // Shared-memory ring of STAGES k-tiles; operands of the next STAGES - 1 tiles are in flight (A in
  // registers, B as cp.async groups).  Three stages for the 4 x 4-per-thread configurations: those run
  // one or two warps per scheduler, a k-tile is over in ~800 cycles, and with a single tile of
  // look-ahead each k-tile waited about 570 cycles for its operands (ncu on 512^3: 35 of 89 cycles per
  // k step were long-scoreboard stalls; 256^3 13.7 -> 9.8 us, 512^3 26.2 -> 18.5 us, 4096 x 64 x 4096
  // 192 -> 128 us).  The 8 x 8-per-thread configurations keep two stages: their k-tile takes 2000
  // cycles, which already covers the latency, and the second register set cost them 10 %
  // (1024^3 72 -> 82 us).
  constexpr int STAGES = (RM * HN < 16 && !Policy::kTransposedB) ? 3 : 2;
  static_assert(STAGES * BK * (AS_PITCH + BS_PITCH) * 4 <= 48 * 1024, "static shared memory");
  static_assert(STAGES == 2 || STAGES == 3, "the k loop below is written for one or two tiles of look-ahead");
  constexpr int D = STAGES - 1;  // tiles of look-ahead = register sets for A
  __shared__ __align__(16) float As[STAGES][BK][AS_PITCH];
  __shared__ __align__(16) float Bs[STAGES][BK][BS_PITCH];

  int tm, tn;
  if constexpr (Policy::kUpperTriangle) {
    // CTA -> the bid-th tile that reaches the diagonal or lies above it, row by row: tile row tm holds
    // tile columns first_live_tile_col(tm) .. tiles_n - 1.  Enumerating only those keeps the block
    // scheduler's one-CTA-per-SM-first placement balanced (skipping dead CTAs of a full grid does not:
    // the live ones then share SMs at random).
    int rest = blockIdx.x;
    for (tm = 0; tm < tiles_m; tm++) {
      const int first = first_live_tile_col(tm, BM, BN);
      const int count = tiles_n > first ? tiles_n - first : 0;
      if (rest < count) {
        tn = first + rest;
        break;
      }
      rest -= count;
    }
    if (tm == tiles_m) return;
  } else {
    // CTA -> tile, grouped 8 tile-rows at a time so that CTAs resident together
    // share A rows and B columns in L2.
    constexpr int GM = 8;
    const int bid = blockIdx.x;
    const int per_group = GM * tiles_n;
    const int group = bid / per_group;
    const int first_m = group * GM;
    const int gm = min(GM, tiles_m - first_m);
    const int in_group = bid - group * per_group;
    tm = first_m + in_group % gm;
    tn = in_group / gm;
  }
  const int m0 = tm * BM, n0 = tn * BN;
  const int K = P.K;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  constexpr int WX = TDX / 8;                      // warps side by side
  const int ty = (warp / WX) * 4 + (lane >> 3);  // 0..TDY-1
  const int tx = (warp % WX) * 8 + (lane & 7);   // 0..TDX-1

  // global -> register staging coordinates
  // A tile: BM rows x 16 k.  thread -> rows tid/4 (+ THREADS/4 per pass), k quad (tid%4)*4
  const int a_row = tid >> 2, a_kq = (tid & 3) * 4;
  constexpr int A_RSTEP = THREADS / 4, PA = (BM + A_RSTEP - 1) / A_RSTEP;  // passes over the A tile
  constexpr bool A_PART = BM < A_RSTEP;  // a tile with fewer rows than one pass covers: some threads load no A
  // B tile: 16 k x BN cols = 16 * BN/4 column quads, PB per thread
  constexpr int QPR = BN / 4;  // quads per k row
  const int b_k = tid / QPR, b_c4 = (tid % QPR) * 4;
  constexpr int B_KSTEP = THREADS / QPR, PB = BK / B_KSTEP;  // k rows covered per pass, passes

  typename Policy::RowCtx rc[PA];
#pragma unroll
  for (int h = 0; h < PA; h++) rc[h] = P.row_ctx(m0 + a_row + h * A_RSTEP);
  // K cursors of this thread's loads: tiles are requested in increasing k, one BK apart
  typename Policy::KCtx ka = P.k_ctx(a_kq);
  typename Policy::KCtx kb[PB];
#pragma unroll
  for (int h = 0; h < PB; h++) kb[h] = P.k_ctx(b_k + h * B_KSTEP);

  // A goes through registers (it is transposed on the way into shared memory);
  // B is copied global -> shared asynchronously, 16 bytes (or 4 x 4) per thread.
  float4 pa[D][PA];
  constexpr int PBT = Policy::kTransposedB ? BN / A_RSTEP : 1;  // passes over a k-contiguous B tile
  float4 pbt[D][PBT];
  // `set` is a std::integral_constant: the register set is chosen at compile time
  auto load_tile = [&](auto set, int buf, bool live) {  // the next tile along K
    constexpr int S = decltype(set)::value;
    if (live) {
#pragma unroll
      for (int h = 0; h < PA; h++)
        if (!A_PART || a_row < BM) pa[S][h] = P.load_a(rc[h], m0 + a_row + h * A_RSTEP, ka);
      if constexpr (Policy::kTransposedB) {
#pragma unroll
        for (int h = 0; h < PBT; h++) pbt[S][h] = P.load_bt(n0 + a_row + h * A_RSTEP, ka);
      } else {
#pragma unroll
        for (int h = 0; h < PB; h++) P.copy_b(&Bs[buf][b_k + h * B_KSTEP][b_c4], kb[h], n0 + b_c4);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");  // one group per tile, empty past the last one
    P.k_advance(ka, BK);
    if constexpr (!Policy::kTransposedB) {
#pragma unroll
      for (int h = 0; h < PB; h++) P.k_advance(kb[h], BK);
    }
  };
  auto store_tile = [&](auto set, int buf) {
    constexpr int S = decltype(set)::value;
    if constexpr (Policy::kTransposedB) {
#pragma unroll
      for (int h = 0; h < PBT; h++) {
        const int r = a_row + h * A_RSTEP;
        Bs[buf][a_kq + 0][r] = pbt[S][h].x;
        Bs[buf][a_kq + 1][r] = pbt[S][h].y;
        Bs[buf][a_kq + 2][r] = pbt[S][h].z;
        Bs[buf][a_kq + 3][r] = pbt[S][h].w;
      }
    }
#pragma unroll
    for (int h = 0; h < PA; h++) {
      const int r = a_row + h * A_RSTEP;
      if (A_PART && r >= BM) continue;
      As[buf][a_kq + 0][r] = pa[S][h].x;
      As[buf][a_kq + 1][r] = pa[S][h].y;
      As[buf][a_kq + 2][r] = pa[S][h].z;
      As[buf][a_kq + 3][r] = pa[S][h].w;
    }
    // all but the D - 1 most recent groups have landed: the tile being published is complete
    asm volatile("cp.async.wait_group %0;" ::"n"(D - 1) : "memory");
  };

  // accumulators start at the chain's first operand
  float acc[PACKED ? 1 : RM][PACKED ? 1 : RN];
  uint64_t acc2[PACKED ? RM : 1][PACKED ? RN / 2 : 1];  // [row][column pair]
#pragma unroll
  for (int i = 0; i < RM; i++) {
    const int row = m0 + (i / QR) * QSM + ty * QR + (i % QR);
#pragma unroll
    for (int jq = 0; jq < HN; jq++) {
      const float4 v = P.init(row, n0 + jq * QSN + tx * 4);
      if (PACKED) {
        acc2[i][jq * 2 + 0] = pack2(v.x, v.y);
        acc2[i][jq * 2 + 1] = pack2(v.z, v.w);
      } else {
        acc[i][jq * 4 + 0] = v.x;
        acc[i][jq * 4 + 1] = v.y;
        acc[i][jq * 4 + 2] = v.z;
        acc[i][jq * 4 + 3] = v.w;
      }
    }
  }

  const int ktiles = (K + BK - 1) / BK;
  // The loop over the look-ahead is written out for D = 1 and D = 2.  (A compile-time loop over D
  // through a generic lambda compiled to a slower k loop: 1024^3 65.5 -> 71.6 us with 128 x 64 tiles;
  // rings of four and five stages, tried that way, were within 1 % of three.)
  using Set0 = std::integral_constant<int, 0>;
  using Set1 = std::integral_constant<int, D - 1>;  // the second set (the first again when D == 1)
  // prologue: tiles 0 .. D - 1 requested, tile 0 published
  load_tile(Set0{}, 0, true);
  if (D > 1) load_tile(Set1{}, 1, 1 < ktiles);
  store_tile(Set0{}, 0);
  __syncthreads();

  // One k-tile: request tile t + D into the register set / ring slot that tile t's predecessor freed,
  // multiply tile t, publish tile t + 1.  `set` = t % D.
  auto iteration = [&](auto set, auto next_set, int t, int buf) {
    load_tile(set, (buf + D) % STAGES, t + D < ktiles);  // tile t + D

    const int kmax = min(BK, K - t * BK);
    auto step = [&](int kk) {
      float a[RM];
      if constexpr (QR == 4) {
#pragma unroll
        for (int h = 0; h < HM; h++) {
          const float4 av = *reinterpret_cast<const float4*>(&As[buf][kk][h * QSM + ty * 4]);
          a[h * 4 + 0] = av.x;
          a[h * 4 + 1] = av.y;
          a[h * 4 + 2] = av.z;
          a[h * 4 + 3] = av.w;
        }
      } else {
        const float2 av = *reinterpret_cast<const float2*>(&As[buf][kk][ty * 2]);
        a[0] = av.x;
        a[1] = av.y;
      }
      if (PACKED) {
        uint64_t b[RN / 2];
#pragma unroll
        for (int h = 0; h < HN; h++) {
          const ulonglong2 bv = *reinterpret_cast<const ulonglong2*>(&Bs[buf][kk][h * QSN + tx * 4]);
          b[h * 2 + 0] = bv.x;
          b[h * 2 + 1] = bv.y;
        }
#pragma unroll
        for (int i = 0; i < RM; i++) {
          const uint64_t aa = pack2(a[i], a[i]);
#pragma unroll
          for (int j = 0; j < RN / 2; j++) acc2[i][j] = fma2(aa, b[j], acc2[i][j]);
        }
      } else {
        float b[RN];
#pragma unroll
        for (int h = 0; h < HN; h++) {
          const float4 bv = *reinterpret_cast<const float4*>(&Bs[buf][kk][h * QSN + tx * 4]);
          b[h * 4 + 0] = bv.x;
          b[h * 4 + 1] = bv.y;
          b[h * 4 + 2] = bv.z;
          b[h * 4 + 3] = bv.w;
        }
#pragma unroll
        for (int i = 0; i < RM; i++)
#pragma unroll
          for (int j = 0; j < RN; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
    };
    if (kmax == BK) {
#pragma unroll
      for (int kk = 0; kk < BK; kk++) step(kk);
    } else {
      for (int kk = 0; kk < kmax; kk++) step(kk);  // ragged K tail: no padded steps
    }

    if (t + 1 < ktiles) store_tile(next_set, (buf + 1) % STAGES);
    __syncthreads();
  };
  int buf = 0;
  for (int t = 0; t < ktiles; t += D) {
    iteration(Set0{}, Set1{}, t, buf);
    buf = (buf + 1) % STAGES;
    if (D > 1 && t + 1 < ktiles) {
      iteration(Set1{}, Set0{}, t + 1, buf);
      buf = (buf + 1) % STAGES;
    }
  }

#pragma unroll
  for (int i = 0; i < RM; i++) {
    const int row = m0 + (i / QR) * QSM + ty * QR + (i % QR);
#pragma unroll
    for (int jq = 0; jq < HN; jq++) {
      float4 v;
      if (PACKED) {
        unpack2(acc2[i][jq * 2 + 0], v.x, v.y);
        unpack2(acc2[i][jq * 2 + 1], v.z, v.w);
      } else {
        v = make_float4(acc[i][jq * 4], acc[i][jq * 4 + 1], acc[i][jq * 4 + 2], acc[i][jq * 4 + 3]);
      }
      P.store(row, n0 + jq * QSN + tx * 4, v);
    }
  }
}

// EXOB200_FFMA_SCALAR=1 selects the one-FMA-per-instruction variant (for A/B timing).
inline bool use_packed() {
  static const bool packed = [] {
    const char* e = getenv("EXOB200_FFMA_SCALAR");
    return !(e && e[0] == '1');
  }();
  return packed;
}

template <class Policy, int RM, int HN, int TDY, int TDX>
cudaError_t launch_tiles_h(cudaStream_t stream, const Policy& P) {
  constexpr int TM = TDY * RM, TN = 4 * TDX * HN;
  const int64_t tiles_m = (P.M + TM - 1) / TM, tiles_n = (P.N + TN - 1) / TN;
  if (tiles_m * tiles_n > INT32_MAX) return cudaErrorInvalidValue;
  const unsigned grid = (unsigned)count_tiles(P, TM, TN);
  if (use_packed())
    tile_kernel<Policy, true, RM, HN, TDY, TDX><<<grid, TDY * TDX, 0, stream>>>(P, (int)tiles_m, (int)tiles_n);
  else
    tile_kernel<Policy, false, RM, HN, TDY, TDX><<<grid, TDY * TDX, 0, stream>>>(P, (int)tiles_m, (int)tiles_n);
  return cudaGetLastError();
}

// Tile choice.  Without split-K the only freedom is the tile shape, and which one is fastest depends
// on how many CTAs end up sharing an SM.  Each configuration was timed on a B200 with 1 .. max resident
// CTAs per SM (cubes 256^3 .. 2048^3 and 4096 x 64 x 4096, fixed launch cost removed); the table holds
// the nanoseconds ONE k step of the whole SM takes at that residency.  A launch is modelled as full
// rounds at the maximum residency plus one round for the remainder, CTAs spread evenly over the SMs
// (the block scheduler fills breadth first), and the cheapest configuration wins.  The model reproduces
// what was found shape by shape before it: 1024^3 -> 128 x 64 (62 us; 128 x 128: 110), 1088^3 -> 64 x 64
// with 4 x 8 per thread (77 us; 128 x 64: 111), 1536^3 -> 128 x 64 or 128 x 128 (155 / 160), 2048^3 and
// up -> 128 x 128 unless its last round would be nearly empty (324 tiles: 578 -> 517 us with 128 x 64).
struct TileConfig {
  int id;             // value of EXOB200_FFMA_TILE that forces it
  int bm, bn;         // tile extents
  int max_resident;   // CTAs per SM by registers / threads
  float ns[8];        // ns per k step of one SM holding 1 .. max_resident CTAs
};
constexpr TileConfig kTileConfigs[] = {
    {128, 128, 128, 2, {102.5f, 185.f}},
    {12864, 128, 64, 2, {58.f, 99.f}},
    {6464, 64, 64, 4, {47.f, 66.f, 87.5f, 114.5f}},  // 128 threads, 4 x 8 outputs each
    {64, 64, 64, 2, {40.5f, 71.5f}},                  // 256 threads, 4 x 4 outputs each
    {32, 32, 32, 8, {24.f, 27.5f, 37.3f, 40.6f, 54.2f, 57.7f, 72.3f, 76.2f}},  // 64 threads, 4 x 4 each
    // 128 threads, 2 x 4 outputs each: twice the warps of the row above on the same tile.  Alone on an SM
    // they hide each other's latency (256^3: 9.4 -> 7.7 us); from two CTAs per SM on, the shared-memory
    // pipe is the limit (ncu on 512^3: 76 % of its peak while active) and the 4 x 4 threads win.
    {3224, 32, 32, 4, {18.f, 28.5f, 43.f, 56.5f}},
    // 16 x 64, 128 threads, 2 x 4 outputs each: problems of up to 16 rows, which leave half of a 32-row tile
    // empty (16 x 16384 x 512: 18.8 against 22.6 us on 32 x 32 tiles; 16 x 32768 x 512: 33.1 against 39.9)
    {1664, 16, 64, 4, {21.f, 30.f, 44.f, 58.f}},
    // 8 x 128, 128 threads, 2 x 4 outputs each: at most 8 rows (8 x 32768 x 512: 19.4 us; 30.8 on 16 x 64 tiles)
    {8128, 8, 128, 4, {21.f, 30.f, 44.f, 58.f}},
};

// Predicted ns per k step of the slowest SM for `tiles` CTAs of configuration c.
inline double predicted_ns_per_k(const TileConfig& c, int64_t tiles, int sm_count) {
  const int64_t per_round = (int64_t)sm_count * c.max_resident;
  const int64_t rounds = tiles / per_round, rest = tiles - rounds * per_round;
  double t = (double)rounds * c.ns[c.max_resident - 1];
  if (rest > 0) t += c.ns[(rest + sm_count - 1) / sm_count - 1];
  return t;
}

// The configuration (TileConfig::id) launch_tiles uses for this problem.
template <class Policy>
int choose_tile(const Policy& P, int sm_count = 148) {
  static const int force = [] {
    const char* e = getenv("EXOB200_FFMA_TILE");  // a TileConfig id forces a tile size (timing experiments)
    return e ? atoi(e) : 0;
  }();
  for (const TileConfig& c : kTileConfigs)
    if (force == c.id) return force;
  int tile = 0;
  double best = 0;
  for (const TileConfig& c : kTileConfigs) {
    if (c.bn > 64 && P.N <= 64) continue;    // a 128-wide tile would be half empty
    if (c.bm <= 16 && P.M > c.bm) continue;  // measured only where they are meant for
    const double t = predicted_ns_per_k(c, count_tiles(P, c.bm, c.bn), sm_count);
    if (tile == 0 || t < best) best = t, tile = c.id;
  }
  return tile;
}

template <class Policy>
cudaError_t launch_tiles(cudaStream_t stream, const Policy& P, int sm_count = 148) {
  const int tile = choose_tile(P, sm_count);
  if (tile == 128) return launch_tiles_h<Policy, 8, 2, 16, 16>(stream, P);
  if (tile == 12864) return launch_tiles_h<Policy, 8, 2, 16, 8>(stream, P);
  if (tile == 6464) return launch_tiles_h<Policy, 4, 2, 16, 8>(stream, P);    // 64 x 64, 128 threads, 4 x 8 per thread
  if (tile == 64) return launch_tiles_h<Policy, 4, 1, 16, 16>(stream, P);
  if (tile == 3224) return launch_tiles_h<Policy, 2, 1, 16, 8>(stream, P);  // 32 x 32, 128 threads, 2 x 4 per thread
  if (tile == 1664) return launch_tiles_h<Policy, 2, 1, 8, 16>(stream, P);  // 16 x 64, 128 threads, 2 x 4 per thread
  if (tile == 8128) return launch_tiles_h<Policy, 2, 1, 4, 32>(stream, P);  // 8 x 128, 128 threads, 2 x 4 per thread
  return launch_tiles_h<Policy, 4, 1, 8, 8>(stream, P);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace ffma
}  // namespace exob200
