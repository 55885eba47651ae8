// Tensor-core GEMMs on tcgen05 / tensor memory, fed by TMA.
//
// One persistent, warp-specialised kernel template serves three arithmetic
// modes; all operands reach it K-major (rows of K-contiguous elements):
//   BF16    C(bf16) = A(bf16) * B(bf16), fp32 accumulation      -> gemm_bf16_exo
//   I8      int8 x int8 -> int32 in tensor memory, then the Gemmini output
//           stage (scale, round-half-even, clamp, ReLU) fused in the epilogue
//           (apps/gemmini/src/exo/matmul.py:18-43)                -> matmul_on_cpu & co
//   TF32X3  fp32 operands pre-split into TF32 hi + lo terms; per product three
//           MMAs (lo*hi, hi*lo, hi*hi) into one fp32 accumulator; C += result
//           (apps/x86/sgemm/sgemm.py:20-23)                       -> sgemm_exo_3xtf32
//
// CTA = 6 warps: warp 0 issues TMA loads into a ring of shared-memory stages
// (mbarrier full/empty pairs), one thread of warp 1 issues tcgen05.mma into one
// of two 128 x 256 fp32/int32 accumulators in tensor memory (512 columns) and
// commits stage releases, warps 2-5 drain the other accumulator with tcgen05.ld
// and write C, so the epilogue of tile i overlaps the main loop of tile i+1.
// Grid = one CTA per SM; tiles are handed out round-robin in an order that keeps
// 16 tile-rows of A and the matching B columns hot in L2.  Ragged M / N / K:
// TMA zero-fills out-of-range rows and K, stores are bounds-checked.
//
// Every wait is bounded: on expiry the role records EXO_B200_ERR_TIMEOUT in the
// status word, raises the CTA's abort flag so the other roles leave their loops
// too, the producer waits (bounded) for its TMA copies in flight, and the CTA
// frees its tensor memory and returns.
//
// Operand layouts that are not K-major in the caller's memory (B of the int8
// matmul and of the SGEMM are row-major K x N) are transposed into a scratch
// buffer by a bandwidth-bound pre-pass, which for TF32X3 also performs the
// hi/lo split and pads the row pitch to TMA's 16-byte rule, so ragged K and N
// need no special case.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdlib>
#include <mutex>

#include "i8_epilogue.cuh"
#include "kernels.cuh"
#include "tc_common.cuh"
#include "umma.cuh"

namespace exob200 {
namespace {

using namespace umma;

enum Mode { MODE_BF16 = 0, MODE_I8 = 1, MODE_TF32X3 = 2 };

using namespace tc;
constexpr int BN = 256;
constexpr int TMEM_COLS = 512;            // two BN-column accumulators

template <int MODE>
struct Cfg;
template <>
struct Cfg<MODE_BF16> {
  static constexpr int ELEM = 2, NA = 1, NB = 1, NPROD = 1, STAGES = 4, KIND = KIND_F16;
  static constexpr int CHUNK_KB = 1 << 30;  // k-blocks accumulated in tensor memory before a drain: all
  static constexpr uint32_t IDESC = make_idesc(1, 1, 1, BM, BN);
};
template <>
struct Cfg<MODE_I8> {
  static constexpr int ELEM = 1, NA = 1, NB = 1, NPROD = 1, STAGES = 4, KIND = KIND_I8;
  static constexpr int CHUNK_KB = 1 << 30;
  static constexpr uint32_t IDESC = make_idesc(2, 1, 1, BM, BN);
};
template <>
struct Cfg<MODE_TF32X3> {
  static constexpr int ELEM = 4, NA = 2, NB = 2, NPROD = 3, STAGES = 2, KIND = KIND_TF32;
  // The tensor core adds into its fp32 accumulator without round-to-nearest, a bias that
  // grows with the number of accumulation steps.  So K is accumulated in tensor memory in
  // chunks of 32 k-blocks (1024 elements); each chunk's partial sum is then added to C by
  // the epilogue warps with ordinary round-to-nearest fp32 adds (the epilogue is "C +="
  // anyway, and it overlaps the next chunk's MMAs through the second accumulator).
  static constexpr int CHUNK_KB = 32;
  static constexpr uint32_t IDESC = make_idesc(1, 2, 2, BM, BN);
};

constexpr int B_TILE_BYTES = BN * ROW_BYTES;  // 32 KiB

template <int MODE>
__host__ __device__ constexpr int stage_bytes() {
  return Cfg<MODE>::NA * A_TILE_BYTES + Cfg<MODE>::NB * B_TILE_BYTES;
}
// 3xTF32 epilogue staging: per epilogue warp a 32-row x 16-column fp32 patch (pitch 20
// floats) through which the tile's running sums are transposed, so that the final
// "C += sum" reads and writes C in row-contiguous pieces instead of one row per lane.
constexpr int EPI_PITCH = 20;
constexpr int EPI_PATCH_BYTES = 32 * EPI_PITCH * 4;
template <int MODE>
__host__ __device__ constexpr int smem_bytes() {
  return Cfg<MODE>::STAGES * stage_bytes<MODE>() + 1024 /* alignment slack */ + 256 /* barriers */ +
         (MODE == MODE_TF32X3 ? 8 * EPI_PATCH_BYTES : 0);
}

struct EpiParams {
  void* C;
  int64_t ldc;   // elements
  float scale;   // I8
  int act;       // I8
  int vec_ok;    // 16-byte stores allowed
  int tri;       // TF32X3: 1 = only the upper triangle (col >= row) of a square C is updated (SSYRK)
};

// ------------------------------------------------------------- epilogues
template <int MODE>
__device__ __forceinline__ void store_chunk(const EpiParams& ep, const uint32_t (&r)[32], int row, int col,
                                            int M, int N) {
  if (row >= M || col >= N) return;
  if (MODE == MODE_BF16) {
    __nv_bfloat16* p = static_cast<__nv_bfloat16*>(ep.C) + (int64_t)row * ep.ldc + col;
    if (ep.vec_ok) {
#pragma unroll
      for (int v = 0; v < 4; v++) {
        if (col + v * 8 + 8 > N) break;
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * j]),
                                                         __uint_as_float(r[v * 8 + 2 * j + 1]));
          w[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(p + v * 8) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; j++)
        if (col + j < N) p[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
    }
  } else if (MODE == MODE_I8) {
    int8_t* p = static_cast<int8_t*>(ep.C) + (int64_t)row * ep.ldc + col;
    if (ep.vec_ok) {
#pragma unroll
      for (int v = 0; v < 2; v++) {
        if (col + v * 16 + 16 > N) break;
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
          uint32_t x = 0;
#pragma unroll
          for (int b = 0; b < 4; b++) {
            const int8_t q = i8_epilogue((int32_t)r[v * 16 + j * 4 + b], ep.scale, ep.act != 0);
            x |= (uint32_t)(uint8_t)q << (8 * b);
          }
          w[j] = x;
        }
        *reinterpret_cast<uint4*>(p + v * 16) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; j++)
        if (col + j < N) p[j] = i8_epilogue((int32_t)r[j], ep.scale, ep.act != 0);
    }
  } else {  // MODE_TF32X3: C += acc
    float* p = static_cast<float*>(ep.C) + (int64_t)row * ep.ldc + col;
    if (ep.vec_ok) {
#pragma unroll
      for (int v = 0; v < 8; v++) {
        if (col + v * 4 + 4 > N) break;
        float4 c = *reinterpret_cast<const float4*>(p + v * 4);
        c.x += __uint_as_float(r[v * 4 + 0]);
        c.y += __uint_as_float(r[v * 4 + 1]);
        c.z += __uint_as_float(r[v * 4 + 2]);
        c.w += __uint_as_float(r[v * 4 + 3]);
        *reinterpret_cast<float4*>(p + v * 4) = c;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; j++)
        if (col + j < N) p[j] += __uint_as_float(r[j]);
    }
  }
}

// ------------------------------------------------------------ the kernel
// BMN: B is read MN-major straight from the caller's row-major K x N array (no
// transposing pre-pass): per stage BN*ELEM/128 TMA boxes {128 bytes of N, BK rows
// of K}, and the B descriptor / instruction descriptor say "MN-major".
template <int MODE>
__host__ __device__ constexpr int epi_warps() {
  return MODE == MODE_TF32X3 ? 8 : 4;  // 3xTF32 keeps a tile's running sum in registers: 128 columns per thread
}
template <int MODE>
__host__ __device__ constexpr int tc_threads() {
  return 64 + 32 * epi_warps<MODE>();
}

template <int MODE, bool BMN = false>
__global__ void __launch_bounds__(tc_threads<MODE>(), 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
               const __grid_constant__ CUtensorMap tmB0, const __grid_constant__ CUtensorMap tmB1, int M, int N,
               int K, EpiParams ep, DeviceStatus* status, int tiles_m, int tiles_n, int chunk_kb) {
  using C = Cfg<MODE>;
  constexpr int STAGES = C::STAGES;
  constexpr int STAGE_BYTES = stage_bytes<MODE>();
  constexpr int BK = ROW_BYTES / C::ELEM;  // elements of K per stage

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
  uint8_t* ctrl = smem_raw + (tiles - raw) + STAGES * STAGE_BYTES;
  const uint32_t bars = tiles + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bars + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(ctrl + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl + 8 * (2 * STAGES + 4) + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), epi_warps<MODE>());  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
    prefetch_tensormap(&tmA0);
    prefetch_tensormap(&tmB0);
    if (C::NA > 1) prefetch_tensormap(&tmA1);
    if (C::NB > 1) prefetch_tensormap(&tmB1);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_dep_wait();  // operands may come from a pre-pass kernel that this launch was allowed to overlap

  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  constexpr int GM = 16;
  auto tile_coord = [&](int t, int& tm, int& tn) {
    const int per_group = GM * tiles_n;
    const int group = t / per_group;
    const int first_m = group * GM;
    const int gm = min(GM, tiles_m - first_m);
    const int in_group = t - group * per_group;
    tm = first_m + in_group % gm;
    tn = in_group / gm;
  };

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t armed = 0, armed_parity = 0;  // per-stage: has a load in flight / its phase parity
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn;
        tile_coord(t, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        if (ep.tri && n0 + BN <= m0) continue;  // entirely below the diagonal: every role skips it
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
            report_timeout(status, abort_flag, 1);
            ok = false;
            break;
          }
          const uint32_t bar = full_bar(stage);
          const uint32_t dst = tiles + stage * STAGE_BYTES;
          mbar_arrive_expect_tx(bar, STAGE_BYTES);
          armed |= 1u << stage;
          armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
          const int k0 = kb * BK;
          tma_load_2d(dst, &tmA0, bar, k0, m0);
          if (C::NA > 1) tma_load_2d(dst + A_TILE_BYTES, &tmA1, bar, k0, m0);
          if (BMN) {
            constexpr int NBOX = BN * C::ELEM / ROW_BYTES;  // 128-byte chunks of N per tile
            constexpr int BOX_BYTES = BK * ROW_BYTES;
#pragma unroll
            for (int j = 0; j < NBOX; j++)
              tma_load_2d(dst + C::NA * A_TILE_BYTES + j * BOX_BYTES, &tmB0, bar, n0 + j * (ROW_BYTES / C::ELEM), k0);
          } else {
            tma_load_2d(dst + C::NA * A_TILE_BYTES, &tmB0, bar, k0, n0);
            if (C::NB > 1) tma_load_2d(dst + C::NA * A_TILE_BYTES + B_TILE_BYTES, &tmB1, bar, k0, n0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok || *abort_flag) {
        // error path: let the copies already issued land before the CTA exits
        volatile int never = 0;
        for (int s = 0; s < STAGES; s++)
          if (armed & (1u << s)) mbar_wait(full_bar(s), (armed_parity >> s) & 1u, &never, DRAIN_LIMIT_NS);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (ep.tri) {
          int tm, tn;
          tile_coord(t, tm, tn);
          if (tn * BN + BN <= tm * BM) continue;
        }
        for (int kb0 = 0; kb0 < num_kb && ok; kb0 += chunk_kb) {
          const int kb1 = min(num_kb, kb0 + chunk_kb);
          if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
            report_timeout(status, abort_flag, 2);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d = tmem_base + (uint32_t)(acc * BN);
          for (int kb = kb0; kb < kb1; kb++) {
            if (!mbar_wait(full_bar(stage), phase, abort_flag, WAIT_LIMIT_NS)) {
              report_timeout(status, abort_flag, 3);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t a0 = tiles + stage * STAGE_BYTES;
            const uint32_t b0 = a0 + C::NA * A_TILE_BYTES;
            const uint64_t da_hi = smem_desc_k_sw128(a0);
            const uint64_t db_hi = BMN ? smem_desc_mn_sw128(b0, BK) : smem_desc_k_sw128(b0);
            constexpr uint32_t IDESC = C::IDESC | (BMN ? IDESC_B_MN_MAJOR : 0u);
            // one MMA consumes 32 bytes of K: K-major that is 32 bytes along the row;
            // MN-major it is (32 / ELEM) K-rows of 128 bytes
            constexpr uint64_t B_ADV = BMN ? (uint64_t)((32 / C::ELEM) * ROW_BYTES / 16) : 2u;
            const uint32_t first = (kb == kb0) ? 0u : 1u;  // the chunk's first MMA overwrites the accumulator
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ks++) {
              const uint64_t adv = (uint64_t)(ks * 2);  // 32 bytes, in 16-byte units
              if (C::NPROD == 1) {
                tc_mma<C::KIND>(d, da_hi + adv, db_hi + ks * B_ADV, IDESC, first | (uint32_t)ks);
              } else {
                const uint64_t da_lo = smem_desc_k_sw128(a0 + A_TILE_BYTES);
                const uint64_t db_lo = smem_desc_k_sw128(b0 + B_TILE_BYTES);
                // small terms first, then the leading term
                tc_mma<C::KIND>(d, da_lo + adv, db_hi + adv, C::IDESC, first | (uint32_t)ks);
                tc_mma<C::KIND>(d, da_hi + adv, db_lo + adv, C::IDESC, 1);
                tc_mma<C::KIND>(d, da_hi + adv, db_hi + adv, C::IDESC, 1);
              }
            }
            tc_commit(empty_bar(stage));  // stage reusable once these MMAs have read it
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if (!ok) break;
          tc_commit(tfull_bar(acc));  // this chunk's accumulator is complete
          acc ^= 1;
          if (acc == 0) acc_phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------ epilogue warps 2..5
    const int q = warp & 3;  // tensor-memory lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int tm, tn;
      tile_coord(t, tm, tn);
      const int m0 = tm * BM, n0 = tn * BN;
      if (ep.tri && n0 + BN <= m0) continue;
      const int row = m0 + q * 32 + lane;
      bool ok = true;
      const int half = (warp - 2) >> 2;  // 3xTF32 only: which 128 columns of the tile this warp owns
      float part[MODE == MODE_TF32X3 ? 128 : 1];
      if (MODE == MODE_TF32X3) {
#pragma unroll
        for (int j = 0; j < 128; j++) part[j] = 0.f;
      }
      // one pass per K chunk: a single pass that writes C, except for 3xTF32, whose passes
      // each add the chunk's partial sums to per-thread running sums (same thread, same
      // elements in every pass) that are added to C once, after the last chunk
      for (int kb0 = 0; kb0 < num_kb; kb0 += chunk_kb) {
        if (!mbar_wait_warp(tfull_bar(acc), acc_phase, abort_flag, WAIT_LIMIT_NS)) {
          if (lane == 0) report_timeout(status, abort_flag, 4);
          ok = false;
          break;
        }
        tc_fence_after();
        if (MODE == MODE_TF32X3) {
          // add this chunk's partial sums (tensor memory) to the tile's running sums
          // (registers, round-to-nearest adds); this warp owns columns [half*128, +128)
#pragma unroll
          for (int cc = 0; cc < 8; cc++) {
            if (n0 + half * 128 + cc * 16 < N) {  // warp-uniform
              uint32_t r[16];
              tmem_ld_32x16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + half * 128 + cc * 16), r);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 16; j++) part[cc * 16 + j] += __uint_as_float(r[j]);
            }
          }
        } else {
#pragma unroll 1
          for (int ch = 0; ch < BN / 32; ch++) {
            const int col = n0 + ch * 32;
            if (col >= N) break;  // warp-uniform
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + ch * 32), r);
            tmem_ld_wait();
            store_chunk<MODE>(ep, r, row, col, M, N);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      if (!ok) break;
      if (MODE == MODE_TF32X3) {
        // C += running sums, once per tile.  A lane owns a row, but reading and writing C
        // one row per lane (32 rows, a power-of-two pitch apart, per instruction) is an
        // order of magnitude slower than row-contiguous access, so each 16-column group
        // is transposed through a shared-memory patch: afterwards one instruction covers
        // 8 rows x 64 contiguous bytes.
        float* patch = reinterpret_cast<float*>(ctrl + 256) + (warp - 2) * (EPI_PATCH_BYTES / 4);
        const int row0 = m0 + q * 32;
        const int colbase = n0 + half * 128;
#pragma unroll
        for (int g = 0; g < 8; g++) {
          const int col0 = colbase + g * 16;
          if (col0 >= N) continue;  // warp-uniform
#pragma unroll
          for (int v = 0; v < 4; v++)
            *reinterpret_cast<float4*>(patch + lane * EPI_PITCH + v * 4) = make_float4(
                part[g * 16 + v * 4], part[g * 16 + v * 4 + 1], part[g * 16 + v * 4 + 2], part[g * 16 + v * 4 + 3]);
          __syncwarp();
          float4 c[4], p4[4];
          float* gptr[4];
          bool okk[4];
#pragma unroll
          for (int it = 0; it < 4; it++) {
            const int idx = it * 32 + lane;
            const int r = idx >> 2, c4 = (idx & 3) * 4;
            p4[it] = *reinterpret_cast<const float4*>(patch + r * EPI_PITCH + c4);
            gptr[it] = static_cast<float*>(ep.C) + (int64_t)(row0 + r) * ep.ldc + col0 + c4;
            okk[it] = row0 + r < M && col0 + c4 < N && !(ep.tri && col0 + c4 + 3 < row0 + r);
            // a quad that straddles the diagonal takes the element-wise path below
            const bool whole = ep.vec_ok && !(ep.tri && col0 + c4 < row0 + r);
            if (okk[it]) {
              if (whole) {
                c[it] = *reinterpret_cast<const float4*>(gptr[it]);
              } else {
                c[it].x = gptr[it][0];
                c[it].y = col0 + c4 + 1 < N ? gptr[it][1] : 0.f;
                c[it].z = col0 + c4 + 2 < N ? gptr[it][2] : 0.f;
                c[it].w = col0 + c4 + 3 < N ? gptr[it][3] : 0.f;
              }
            }
          }
#pragma unroll
          for (int it = 0; it < 4; it++) {
            if (!okk[it]) continue;
            const int c4 = ((it * 32 + lane) & 3) * 4;
            c[it].x += p4[it].x;
            c[it].y += p4[it].y;
            c[it].z += p4[it].z;
            c[it].w += p4[it].w;
            const int rr = row0 + ((it * 32 + lane) >> 2);
            const int lim = ep.tri ? rr : -1;  // columns below lim are not part of the update
            if (ep.vec_ok && col0 + c4 >= lim) {
              *reinterpret_cast<float4*>(gptr[it]) = c[it];
            } else {
              if (col0 + c4 + 0 >= lim) gptr[it][0] = c[it].x;
              if (col0 + c4 + 1 < N && col0 + c4 + 1 >= lim) gptr[it][1] = c[it].y;
              if (col0 + c4 + 2 < N && col0 + c4 + 2 >= lim) gptr[it][2] = c[it].z;
              if (col0 + c4 + 3 < N && col0 + c4 + 3 >= lim) gptr[it][3] = c[it].w;
            }
          }
          __syncwarp();
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ----------------------------------------------------- pre-pass kernels
// A (M x K row-major) -> hi, lo (M x Kp), zero in the pad columns.
__global__ void split_rows_kernel(const float* __restrict__ A, int64_t M, int K, int Kp, float* __restrict__ hi,
                                  float* __restrict__ lo) {
  grid_dep_launch();
  const int64_t total = M * Kp;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = i / Kp;
    const int k = (int)(i - row * Kp);
    float h = 0.f, l = 0.f;
    if (k < K) split_tf32(__ldg(A + row * K + k), h, l);
    hi[i] = h;
    lo[i] = l;
  }
}

// B (K x N row-major) -> hi^T, lo^T (N x Kp): 32 x 32 tiles through shared memory.
__global__ void split_transpose_kernel(const float* __restrict__ B, int K, int N, int Kp, float* __restrict__ hi,
                                       float* __restrict__ lo) {
  __shared__ float th[32][33], tl[32][33];
  grid_dep_launch();
  const int k0 = blockIdx.x * 32, n0 = blockIdx.y * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;  // 32 x 8
  for (int r = ty; r < 32; r += 8) {
    const int k = k0 + r, n = n0 + tx;
    float h = 0.f, l = 0.f;
    if (k < K && n < N) split_tf32(__ldg(B + (int64_t)k * N + n), h, l);
    th[r][tx] = h;
    tl[r][tx] = l;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int n = n0 + r, k = k0 + tx;
    if (n < N && k < Kp) {
      hi[(int64_t)n * Kp + k] = th[tx][r];
      lo[(int64_t)n * Kp + k] = tl[tx][r];
    }
  }
}

// int8 B (K x N row-major) -> B^T (N x Kp), zero pad.  128 x 128 byte tiles,
// 32-bit global accesses on both sides.
__global__ void __launch_bounds__(256) transpose_i8_kernel(const int8_t* __restrict__ B, int K, int N, int Kp,
                                                           int8_t* __restrict__ Bt, int vec_in) {
  __shared__ int8_t t[128][128 + 4];
  grid_dep_launch();
  const int k0 = blockIdx.x * 128, n0 = blockIdx.y * 128;
  const int tid = threadIdx.x;
  // read: 128 k rows x 32 words
  for (int e = tid; e < 128 * 32; e += 256) {
    const int r = e >> 5, w = e & 31;
    const int k = k0 + r, n = n0 + w * 4;
    uint32_t v = 0;
    if (k < K) {
      const int8_t* p = B + (int64_t)k * N + n;
      if (vec_in && n + 4 <= N) {
        v = __ldg(reinterpret_cast<const uint32_t*>(p));
      } else {
#pragma unroll
        for (int b = 0; b < 4; b++)
          if (n + b < N) v |= (uint32_t)(uint8_t)__ldg(p + b) << (8 * b);
      }
    }
    *reinterpret_cast<uint32_t*>(&t[r][w * 4]) = v;
  }
  __syncthreads();
  // write: 128 n rows x 32 words of k
  for (int e = tid; e < 128 * 32; e += 256) {
    const int r = e >> 5, w = e & 31;
    const int n = n0 + r, k = k0 + w * 4;
    if (n < N && k < Kp) {  // Kp % 16 == 0, so a word is entirely inside
      const uint32_t v = (uint32_t)(uint8_t)t[w * 4 + 0][r] | ((uint32_t)(uint8_t)t[w * 4 + 1][r] << 8) |
                         ((uint32_t)(uint8_t)t[w * 4 + 2][r] << 16) | ((uint32_t)(uint8_t)t[w * 4 + 3][r] << 24);
      *reinterpret_cast<uint32_t*>(Bt + (int64_t)n * Kp + k) = v;
    }
  }
}

// ------------------------------------------------------------ host side
// K-major operand: `rows` rows of `k_elems` elements, row pitch `pitch_bytes`;
// box = 128 bytes of K x box_rows rows.
bool make_kmajor_map(CUtensorMap* m, CUtensorMapDataType dt, int elem, const void* base, int64_t rows,
                     int64_t k_elems, int64_t pitch_bytes, int box_rows) {
  cuuint64_t dims[2] = {(cuuint64_t)k_elems, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)pitch_bytes};
  cuuint32_t box[2] = {(cuuint32_t)(ROW_BYTES / elem), (cuuint32_t)box_rows};
  return make_tiled_map(m, dt, 2, base, dims, strides, box);
}

// MN-major operand: a row-major `k_rows` x `n_elems` array, row pitch
// `pitch_bytes`; box = 128 bytes of N x box_k rows of K.
bool make_mnmajor_map(CUtensorMap* m, CUtensorMapDataType dt, int elem, const void* base, int64_t k_rows,
                      int64_t n_elems, int64_t pitch_bytes, int box_k) {
  cuuint64_t dims[2] = {(cuuint64_t)n_elems, (cuuint64_t)k_rows};
  cuuint64_t strides[1] = {(cuuint64_t)pitch_bytes};
  cuuint32_t box[2] = {(cuuint32_t)(ROW_BYTES / elem), (cuuint32_t)box_k};
  return make_tiled_map(m, dt, 2, base, dims, strides, box);
}

// k-blocks accumulated in tensor memory between drains (EXOB200_TF32_CHUNK overrides the
// 3xTF32 value, in k-blocks of 32 elements; timing / accuracy experiments)
template <int MODE>
int chunk_kb() {
  if (MODE != MODE_TF32X3) return Cfg<MODE>::CHUNK_KB;
  static const int v = [] {
    const char* e = getenv("EXOB200_TF32_CHUNK");
    const int n = e ? atoi(e) : 0;
    return n > 0 ? n : Cfg<MODE_TF32X3>::CHUNK_KB;
  }();
  return v;
}

template <int MODE, bool BMN = false>
cudaError_t launch_tc(exo_b200_Context* ctx, const CUtensorMap& a0, const CUtensorMap& a1, const CUtensorMap& b0,
                      const CUtensorMap& b1, int64_t M, int64_t N, int64_t K, const EpiParams& ep, int chunk_override = 0,
                      bool after_prepass = false) {
  EXOB200_SMEM_ATTR_ONCE((gemm_tc_kernel<MODE, BMN>), smem_bytes<MODE>(), ctx->device);
  const int64_t tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  if (tiles_m * tiles_n > INT32_MAX || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX)
    return cudaErrorInvalidValue;
  const int grid = (int)std::min<int64_t>(tiles_m * tiles_n, ctx->sm_count);
  const int chunk = chunk_override > 0 ? chunk_override : chunk_kb<MODE>();
  if (after_prepass)  // set-up overlaps the tail of the pre-pass that was enqueued just before
    return launch_dependent(gemm_tc_kernel<MODE, BMN>, dim3(grid), dim3(tc_threads<MODE>()), smem_bytes<MODE>(),
                            ctx->stream, a0, a1, b0, b1, (int)M, (int)N, (int)K, ep, ctx->status_dev, (int)tiles_m,
                            (int)tiles_n, chunk);
  gemm_tc_kernel<MODE, BMN><<<grid, tc_threads<MODE>(), smem_bytes<MODE>(), ctx->stream>>>(
      a0, a1, b0, b1, (int)M, (int)N, (int)K, ep, ctx->status_dev, (int)tiles_m, (int)tiles_n, chunk);
  return cudaGetLastError();
}

}  // namespace

// ---------------------------------------------------------------- bf16
bool tc_supported_bf16(int64_t, int64_t, int64_t K, const void* A, const void* B, const void*) {
  return K % 8 == 0 && aligned16(A) && aligned16(B);
}

namespace {
// rows x K 16-bit elements -> rows x Kp, zero in the pad columns (Kp % 8 == 0, dst 16-byte aligned)
__global__ void pad_rows_u16_kernel(const uint16_t* __restrict__ src, int64_t rows, int K, int Kp,
                                    uint16_t* __restrict__ dst) {
  const int64_t total = rows * Kp;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / Kp;
    const int k = (int)(i - r * Kp);
    dst[i] = k < K ? __ldg(src + r * K + k) : (uint16_t)0;
  }
}
}  // namespace

cudaError_t launch_gemm_bf16_tc(exo_b200_Context* ctx, int64_t M, int64_t N, int64_t K, const uint16_t* A,
                                const uint16_t* B, uint16_t* C) {
  if (!tc_supported_bf16(M, N, K, A, B, C)) {
    // TMA needs a 16-byte row pitch and base.  K % 8 != 0 or an odd base: copy both operands into
    // scratch with the pitch rounded up to 8 elements (zero padding adds exact zeros to every sum)
    // and multiply those.  Costs one extra pass over A and B; ragged K is not the fast case.
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX - 8) return cudaErrorInvalidValue;
    const int64_t Kp = (K + 7) / 8 * 8;
    if (!acquire_scratch(ctx, 0, (size_t)(M * Kp) * 2)) return cudaErrorMemoryAllocation;
    if (!acquire_scratch(ctx, 1, (size_t)(N * Kp) * 2)) return cudaErrorMemoryAllocation;
    uint16_t* Ap = static_cast<uint16_t*>(ctx->scratch[0]);
    uint16_t* Bp = static_cast<uint16_t*>(ctx->scratch[1]);
    const int ba = (int)std::min<int64_t>((M * Kp + 255) / 256, (int64_t)ctx->sm_count * 16);
    const int bb = (int)std::min<int64_t>((N * Kp + 255) / 256, (int64_t)ctx->sm_count * 16);
    pad_rows_u16_kernel<<<ba, 256, 0, ctx->stream>>>(A, M, (int)K, (int)Kp, Ap);
    pad_rows_u16_kernel<<<bb, 256, 0, ctx->stream>>>(B, N, (int)K, (int)Kp, Bp);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = launch_gemm_bf16_tc(ctx, M, N, Kp, Ap, Bp, C);
    release_scratch(ctx, 0);
    release_scratch(ctx, 1);
    return e;
  }
  if (tc2_wanted(M, N, 128)) return launch_gemm_bf16_tc2(ctx, M, N, K, A, B, C);
  CUtensorMap ma, mb;
  if (!make_kmajor_map(&ma, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, M, K, K * 2, BM)) return cudaErrorUnknown;
  if (!make_kmajor_map(&mb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, N, K, K * 2, BN)) return cudaErrorUnknown;
  EpiParams ep{C, N, 0.f, 0, (N % 8 == 0 && aligned16(C)) ? 1 : 0};
  return launch_tc<MODE_BF16>(ctx, ma, ma, mb, mb, M, N, K, ep);
}

// ---------------------------------------------------------------- int8
bool tc_supported_i8(int64_t, int64_t, int64_t K, const void* A, const void*, const void*) {
  return K % 16 == 0 && aligned16(A);
}

cudaError_t launch_matmul_i8_tc(exo_b200_Context* ctx, int64_t N, int64_t M, int64_t K, float scale, bool act,
                                const int8_t* A, const int8_t* B, int8_t* C) {
  // Exo's names: A is N x K (rows N), B is K x M, C is N x M.  GEMM view: rows = N, cols = M.
  const int64_t rows = N, cols = M;
  const int64_t Kp = K;  // K % 16 == 0 already
  static const bool allow_mn = [] {
    const char* e = getenv("EXOB200_I8_TRANSPOSE");  // =1 forces the transposing pre-pass (A/B timing)
    return !(e && e[0] == '1');
  }();
  if (allow_mn && cols % 16 == 0 && aligned16(B)) {
    // B's pitch satisfies TMA: read it MN-major in place, no pre-pass, no scratch
    if (tc2_wanted(rows, cols, 4 * 74)) return launch_matmul_i8_tc2(ctx, rows, cols, K, scale, act, A, B, C);
    CUtensorMap ma, mb;
    if (!make_kmajor_map(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, rows, K, K, BM)) return cudaErrorUnknown;
    if (!make_mnmajor_map(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B, K, cols, cols, ROW_BYTES)) return cudaErrorUnknown;
    EpiParams ep{C, cols, scale, act ? 1 : 0, (cols % 16 == 0 && aligned16(C)) ? 1 : 0};
    return launch_tc<MODE_I8, true>(ctx, ma, ma, mb, mb, rows, cols, K, ep);
  }
  if (!acquire_scratch(ctx, 1, (size_t)(cols * Kp))) return cudaErrorMemoryAllocation;
  int8_t* Bt = static_cast<int8_t*>(ctx->scratch[1]);
  {
    dim3 grid((unsigned)((K + 127) / 128), (unsigned)((cols + 127) / 128));
    if (grid.y > 65535) return cudaErrorInvalidValue;
    const int vec_in = (cols % 4 == 0 && (reinterpret_cast<uintptr_t>(B) & 3u) == 0) ? 1 : 0;
    transpose_i8_kernel<<<grid, 256, 0, ctx->stream>>>(B, (int)K, (int)cols, (int)Kp, Bt, vec_in);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  CUtensorMap ma, mb;
  if (!make_kmajor_map(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, rows, K, K, BM)) return cudaErrorUnknown;
  if (!make_kmajor_map(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, Bt, cols, K, Kp, BN)) return cudaErrorUnknown;
  EpiParams ep{C, cols, scale, act ? 1 : 0, (cols % 16 == 0 && aligned16(C)) ? 1 : 0};
  const cudaError_t e = launch_tc<MODE_I8>(ctx, ma, ma, mb, mb, rows, cols, K, ep, 0, true);
  release_scratch(ctx, 1);
  return e;
}

// -------------------------------------------------------------- 3xTF32
bool tc_supported_tf32(int64_t, int64_t, int64_t, const void*, const void*, const void*) { return true; }

cudaError_t launch_sgemm_3xtf32_tc(exo_b200_Context* ctx, int64_t M, int64_t N, int64_t K, const float* A,
                                   const float* B, float* C) {
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX - 64) return cudaErrorInvalidValue;
  const int64_t Kp = (K + 3) / 4 * 4;  // pitch multiple of 16 bytes
  const size_t a_elems = (size_t)(M * Kp), b_elems = (size_t)(N * Kp);
  if (!acquire_scratch(ctx, 0, 2 * a_elems * sizeof(float))) return cudaErrorMemoryAllocation;
  if (!acquire_scratch(ctx, 1, 2 * b_elems * sizeof(float))) return cudaErrorMemoryAllocation;
  float* a_hi = static_cast<float*>(ctx->scratch[0]);
  float* a_lo = a_hi + a_elems;
  float* b_hi = static_cast<float*>(ctx->scratch[1]);
  float* b_lo = b_hi + b_elems;
  {
    const int64_t total = M * Kp;
    const int blocks = (int)std::min<int64_t>((total + 255) / 256, (int64_t)ctx->sm_count * 16);
    split_rows_kernel<<<blocks, 256, 0, ctx->stream>>>(A, M, (int)K, (int)Kp, a_hi, a_lo);
    dim3 grid((unsigned)((Kp + 31) / 32), (unsigned)((N + 31) / 32));
    if (grid.y > 65535) return cudaErrorInvalidValue;
    split_transpose_kernel<<<grid, dim3(32, 8), 0, ctx->stream>>>(B, (int)K, (int)N, (int)Kp, b_hi, b_lo);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  CUtensorMap ma0, ma1, mb0, mb1;
  const CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  if (!make_kmajor_map(&ma0, dt, 4, a_hi, M, Kp, Kp * 4, BM)) return cudaErrorUnknown;
  if (!make_kmajor_map(&ma1, dt, 4, a_lo, M, Kp, Kp * 4, BM)) return cudaErrorUnknown;
  if (!make_kmajor_map(&mb0, dt, 4, b_hi, N, Kp, Kp * 4, BN)) return cudaErrorUnknown;
  if (!make_kmajor_map(&mb1, dt, 4, b_lo, N, Kp, Kp * 4, BN)) return cudaErrorUnknown;
  EpiParams ep{C, N, 0.f, 0, (N % 4 == 0 && aligned16(C)) ? 1 : 0};
  const cudaError_t e = launch_tc<MODE_TF32X3>(ctx, ma0, ma1, mb0, mb1, M, N, Kp, ep, 0, true);
  release_scratch(ctx, 0);
  release_scratch(ctx, 1);
  return e;
}

// ---------------------------------------------------------------- SSYRK (3xTF32)
// C += A * A^T on the upper triangle.  Both operands of the product are rows of A with k
// contiguous -- the layout the kernel wants for either side -- so ONE hi/lo split of A serves
// as the A operand (boxes of 128 rows) and as the B operand (boxes of 256 rows); tiles below
// the diagonal are skipped by every role and the epilogue masks the diagonal tiles.
cudaError_t launch_ssyrk_3xtf32_tc(exo_b200_Context* ctx, int64_t N, int64_t K, const float* A, float* C) {
  if (N > INT32_MAX || K > INT32_MAX - 64) return cudaErrorInvalidValue;
  const int64_t Kp = (K + 3) / 4 * 4;
  const size_t a_elems = (size_t)(N * Kp);
  if (!acquire_scratch(ctx, 0, 2 * a_elems * sizeof(float))) return cudaErrorMemoryAllocation;
  float* a_hi = static_cast<float*>(ctx->scratch[0]);
  float* a_lo = a_hi + a_elems;
  const int blocks = (int)std::min<int64_t>((N * Kp + 255) / 256, (int64_t)ctx->sm_count * 16);
  split_rows_kernel<<<blocks, 256, 0, ctx->stream>>>(A, N, (int)K, (int)Kp, a_hi, a_lo);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  CUtensorMap ma0, ma1, mb0, mb1;
  const CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  if (!make_kmajor_map(&ma0, dt, 4, a_hi, N, Kp, Kp * 4, BM)) return cudaErrorUnknown;
  if (!make_kmajor_map(&ma1, dt, 4, a_lo, N, Kp, Kp * 4, BM)) return cudaErrorUnknown;
  if (!make_kmajor_map(&mb0, dt, 4, a_hi, N, Kp, Kp * 4, BN)) return cudaErrorUnknown;
  if (!make_kmajor_map(&mb1, dt, 4, a_lo, N, Kp, Kp * 4, BN)) return cudaErrorUnknown;
  EpiParams ep{C, N, 0.f, 0, (N % 4 == 0 && aligned16(C)) ? 1 : 0, 1};
  // The tensor core adds into its accumulator without round-to-nearest; on the diagonal of A A^T every
  // product has the same sign, so that bias is coherent there instead of averaging out.  Draining the
  // accumulator every 8 k-blocks (256 elements of K) instead of every 32 keeps it four times smaller.
  e = launch_tc<MODE_TF32X3>(ctx, ma0, ma1, mb0, mb1, N, N, Kp, ep, 8, true);
  release_scratch(ctx, 0);
  return e;
}

// --------------------------------------------------------------------------
// Self-test of the bounded-wait machinery: one CTA waits on an mbarrier that
// nothing ever arrives on.  The wait must run out after `limit_ns`, record
// EXO_B200_ERR_TIMEOUT in the context's status word and return normally, leaving
// the context usable.  (No trap, no fault: this is how a lost producer or
// consumer would surface in the GEMM kernels.)
namespace {
__global__ void bounded_wait_selftest_kernel(DeviceStatus* status, uint64_t limit_ns) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!mbar_wait(smem_u32(&bar), 0, &abort_flag, limit_ns)) report_timeout(status, &abort_flag, 99);
  }
  __syncthreads();
}
}  // namespace

cudaError_t launch_bounded_wait_selftest(exo_b200_Context* ctx, uint64_t limit_ns) {
  bounded_wait_selftest_kernel<<<1, 32, 0, ctx->stream>>>(ctx->status_dev, limit_ns);
  return cudaGetLastError();
}

// --------------------------------------------------------------------------
// matmul_on_cpu_static: the int8 matmul for callers that must not allocate.
//
// Some callers cannot call cudaMalloc at the point where they need a matmul:
// code that has handed all device memory to its own arena and must never see
// the driver allocator move under it, processes held to a fixed memory budget,
// and latency-critical loops where an allocation's implicit device
// synchronisation is not acceptable.  The regular entry points
// keep a grow-only scratch buffer in their context (for the K-major copy of B
// that the tensor-core kernel reads), so their first call with a new size
// allocates.  This variant keeps that scratch in a fixed array inside the
// library image instead: every GPU that loads the library holds
// EXO_B200_STATIC_SCRATCH_BYTES of it until the process exits.
//
// The array's name is only a host-side handle for the symbol; the kernels need
// its device address, which is looked up once per device (cudaGetSymbolAddress,
// with that device current) on the first call made on that device.  That first
// call also loads the kernels and sets their shared-memory attribute, so make
// it before starting any stream capture.
//
// All calls share the one array: two calls whose kernels overlap on the GPU
// (different streams, no dependency) race on it.  Nothing in it has to start at
// zero -- the transpose pre-pass overwrites every byte the GEMM then reads.
constexpr size_t kStaticScratchBytes = 4u << 20;  // K * M <= 4 Mi int8 elements
static __device__ __align__(256) int8_t g_static_bt_scratch[kStaticScratchBytes];
// The status word of this entry point's kernels lives in the library image too (the regular
// entry points use a mapped host allocation of their context).  A bounded wait that runs out
// records EXO_B200_ERR_TIMEOUT here; exo_b200_synchronize() copies it back and reports it.
static __device__ DeviceStatus g_static_status;

namespace {

struct StaticDeviceState {
  bool ready = false;
  int8_t* scratch = nullptr;  // device address of g_static_bt_scratch on this device
  DeviceStatus* status = nullptr;  // device address of g_static_status on this device
  int sm_count = 0;
};
constexpr int kMaxDevices = 64;
StaticDeviceState g_static_state[kMaxDevices];
std::mutex g_static_mutex;

// Once per device, with that device current.  Allocates nothing.
StaticDeviceState* static_state_for_current_device() {
  int dev = 0;
  if (!check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return nullptr;
  if (dev < 0 || dev >= kMaxDevices) {
    set_error(EXO_B200_ERR_UNSUPPORTED, "matmul_on_cpu_static: device ordinal out of range");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_static_mutex);
  StaticDeviceState& st = g_static_state[dev];
  if (st.ready) return &st;
  int major = 0;
  if (!check_cuda(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev), "cudaDeviceGetAttribute"))
    return nullptr;
  if (major != 10) {
    set_error(EXO_B200_ERR_UNSUPPORTED, "matmul_on_cpu_static: this library contains sm_100a code only");
    return nullptr;
  }
  if (!check_cuda(cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, dev),
                  "cudaDeviceGetAttribute"))
    return nullptr;
  void* ptr = nullptr;
  if (!check_cuda(cudaGetSymbolAddress(&ptr, g_static_bt_scratch), "cudaGetSymbolAddress(static scratch)"))
    return nullptr;
  if (!check_cuda(cudaFuncSetAttribute(gemm_tc_kernel<MODE_I8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       smem_bytes<MODE_I8>()),
                  "cudaFuncSetAttribute"))
    return nullptr;
  void* status_ptr = nullptr;
  if (!check_cuda(cudaGetSymbolAddress(&status_ptr, g_static_status), "cudaGetSymbolAddress(static status)"))
    return nullptr;
  st.scratch = static_cast<int8_t*>(ptr);
  st.status = static_cast<DeviceStatus*>(status_ptr);
  st.ready = true;
  return &st;
}

// Where a device pointer lives: its device ordinal, -1 for managed memory (reachable from every
// device), -2 for anything that is not device memory.
int device_of(const void* p) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
    cudaGetLastError();
    return -2;
  }
  if (attr.type == cudaMemoryTypeManaged) return -1;
  return attr.type == cudaMemoryTypeDevice ? attr.device : -2;
}

}  // namespace

// Called by exo_b200_synchronize: reports a timeout that a kernel of matmul_on_cpu_static has
// recorded on the current device.  A plain blocking 16-byte copy: it sees what kernels that
// have completed wrote (the caller synchronises its own stream first), and allocates nothing.
bool collect_static_status() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return true;
  DeviceStatus* word = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_state[dev].ready) return true;
    word = g_static_state[dev].status;
  }
  DeviceStatus h;
  if (!check_cuda(cudaMemcpy(&h, word, sizeof(h), cudaMemcpyDeviceToHost), "cudaMemcpy(static status)")) return false;
  if (h.code == 0) return true;
  cudaMemset(word, 0, sizeof(h));
  set_error(h.code, "matmul_on_cpu_static: device-side wait ran out (kernel location " + std::to_string(h.where) +
                        ", block " + std::to_string(h.block) + "); its output is incomplete");
  return false;
}

}  // namespace exob200

extern "C" __attribute__((visibility("default"))) void matmul_on_cpu_static(
    void* stream, int_fast32_t N, int_fast32_t M, int_fast32_t K, const float* scale, bool act, const int8_t* A,
    const int8_t* B, int8_t* C) {
  using namespace exob200;
  const char* fn = "matmul_on_cpu_static";
  clear_error();
  if (N < 1 || M < 1 || K < 1 || !scale || !A || !B || !C) {
    set_error(EXO_B200_ERR_INVALID_ARGUMENT, std::string(fn) + ": sizes must be >= 1 and pointers non-NULL");
    return;
  }
  if (N > INT32_MAX || M > INT32_MAX || K > INT32_MAX) {
    set_error(EXO_B200_ERR_INVALID_ARGUMENT, std::string(fn) + ": size out of range");
    return;
  }
  if ((size_t)K * (size_t)M > kStaticScratchBytes) {
    set_error(EXO_B200_ERR_UNSUPPORTED,
              std::string(fn) + ": K * M = " + std::to_string((size_t)K * (size_t)M) + " exceeds the static scratch of " +
                  std::to_string(kStaticScratchBytes) + " int8 elements; use matmul_on_cpu");
    return;
  }
  const int where[3] = {device_of(A), device_of(B), device_of(C)};
  if (where[0] == -2 || where[1] == -2 || where[2] == -2 || is_device_pointer(scale)) {
    set_error(EXO_B200_ERR_INVALID_ARGUMENT,
              std::string(fn) + ": A, B, C must be device memory (host buffers would need staging allocations) "
                                "and scale host memory (it is read when the call is made)");
    return;
  }
  int cur = 0;
  if (!check_cuda(cudaGetDevice(&cur), "cudaGetDevice")) return;
  for (int i = 0; i < 3; i++)
    if (where[i] >= 0 && where[i] != cur) {
      // the scratch array, the SM count and the launch are the current device's
      set_error(EXO_B200_ERR_INVALID_ARGUMENT,
                std::string(fn) + ": operand " + "ABC"[i] + " lives on device " + std::to_string(where[i]) +
                    " but device " + std::to_string(cur) + " is current; make the operands' device current first");
      return;
    }
  StaticDeviceState* st = static_state_for_current_device();
  if (!st) return;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const float sc = *scale;
  if (K % 16 != 0 || (reinterpret_cast<uintptr_t>(A) & 15u) != 0) {
    // pitches TMA cannot express: the SIMT kernel needs no scratch at all
    check_cuda(launch_matmul_i8_simt(s, N, M, K, sc, act, A, B, C), fn);
    return;
  }
  const int64_t rows = N, cols = M;
  dim3 tgrid((unsigned)((K + 127) / 128), (unsigned)((cols + 127) / 128));
  const int vec_in = (cols % 4 == 0 && (reinterpret_cast<uintptr_t>(B) & 3u) == 0) ? 1 : 0;
  transpose_i8_kernel<<<tgrid, 256, 0, s>>>(B, (int)K, (int)cols, (int)K, st->scratch, vec_in);
  if (!check_cuda(cudaGetLastError(), fn)) return;
  CUtensorMap ma, mb;
  if (!make_kmajor_map(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, rows, K, K, BM)) return;
  if (!make_kmajor_map(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, st->scratch, cols, K, K, BN)) return;
  EpiParams ep{C, cols, sc, act ? 1 : 0, (cols % 16 == 0 && (reinterpret_cast<uintptr_t>(C) & 15u) == 0) ? 1 : 0};
  const int64_t tiles_m = (rows + BM - 1) / BM, tiles_n = (cols + BN - 1) / BN;
  const int grid = (int)std::min<int64_t>(tiles_m * tiles_n, st->sm_count);
  // a bounded device-side wait that runs out is recorded in the static status word; this call only
  // enqueues, so the report comes from the next exo_b200_synchronize()
  gemm_tc_kernel<MODE_I8><<<grid, NUM_THREADS, smem_bytes<MODE_I8>(), s>>>(ma, ma, mb, mb, (int)rows, (int)cols,
                                                                           (int)K, ep, st->status, (int)tiles_m,
                                                                           (int)tiles_n, 1 << 30);
  check_cuda(cudaGetLastError(), fn);
}

