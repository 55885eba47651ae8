// Tensor-core GEMM with CTA pairs (tcgen05 cta_group::2).
//
// Same pipeline as tc_gemm.cu -- TMA -> mbarrier ring -> tcgen05.mma -> two
// accumulators in tensor memory -> epilogue warps -- but two CTAs on neighbouring
// SMs form a cluster and share one 256 x 256 output tile: CTA r of the pair loads
// A rows [128 r, 128 r + 128) and B rows (columns of the product) [128 r, 128 r +
// 128) of the tile, one thread of the even CTA issues a single 256 x 256 x (32
// bytes of K) MMA that reads both CTAs' shared memory, and each CTA ends up with
// its 128 x 256 half of the accumulator in its own tensor memory.  Per SM that
// halves the B traffic into and out of shared memory (128 instead of 192 bytes
// per tensor clock), which is what limits the single-CTA kernel, and leaves room
// for a six-stage ring.
//
// Synchronisation inside the pair:
//   full[s]    lives in the even CTA; armed by its producer for the bytes of BOTH
//              CTAs; each CTA's TMA loads complete on it (cp.async.bulk.tensor
//              with .cta_group::2, no multicast)
//   empty[s], tfull[b]   one in each CTA, signalled together by the issuing
//              thread's tcgen05.commit (multicast arrive to the pair)
//   tempty[b]  lives in the even CTA; the eight epilogue warps of the pair arrive
//              on it (the odd CTA's through a cluster-scope remote arrive)
// Every wait is bounded as in tc_gemm.cu; a CTA that gives up also raises the
// abort flag of its partner.  The pair leaves together (cluster barrier) so
// neither CTA's shared memory disappears under the other.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>

#include "i8_epilogue.cuh"
#include "kernels.cuh"
#include "tc_common.cuh"
#include "umma.cuh"

namespace exob200 {
namespace {

using namespace tc;
using namespace umma;

enum Mode2 { M2_BF16 = 0, M2_I8 = 1 };

template <int MODE>
struct Cfg2;
template <>
struct Cfg2<M2_BF16> {
  static constexpr int ELEM = 2, KIND = KIND_F16;
  static constexpr bool BMN = false;
  static constexpr uint32_t D_FMT = 1, AB_FMT = 1;
};
template <>
struct Cfg2<M2_I8> {
  static constexpr int ELEM = 1, KIND = KIND_I8;
  static constexpr bool BMN = true;
  static constexpr uint32_t D_FMT = 2, AB_FMT = 1;
};

constexpr int BN2 = 256;                          // columns of the pair's tile
constexpr int BHALF = BN2 / 2;                    // B rows each CTA loads
constexpr int STAGE2_BYTES = A_TILE_BYTES + BHALF * ROW_BYTES;  // 32 KiB per CTA
constexpr int STAGES2 = 6;
constexpr int SMEM2_BYTES = STAGES2 * STAGE2_BYTES + 1024 + 256;
constexpr uint32_t TMEM2_COLS = 512;

// ---- cluster / pair primitives
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `local_addr` in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapa(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on a barrier of another CTA of the cluster.  Default semantics (release at CTA scope): the
// barrier only hands a tensor-memory accumulator back, and the tcgen05 fences on both sides order those
// accesses.  With .release.cluster the instruction held its thread for about 1.3 us each time (it waits
// for the thread's earlier global and bulk stores to be visible cluster-wide), which kept the issuing
// thread -- and the tensor pipe -- waiting at every tile boundary.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// TMA load whose completion is signalled on a barrier of the even CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar_cluster, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y)
      : "memory");
}
// L2 eviction-priority policies for the TMA loads: the operand panel that the next
// waves of tiles will read again is kept (evict_last), the one that streams
// through is marked evict_first so it does not push the panel out.
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_load_2d_pair_hint(uint32_t dst, const CUtensorMap* m, uint32_t bar_cluster, int x,
                                                      int y, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrive on the barrier at this shared-memory offset in both CTAs of the pair
// once all MMAs issued so far by this thread have completed
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"(mask)
      : "memory");
}
template <int KIND>
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  if (KIND == KIND_F16) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

struct Epi2 {
  void* C;
  int64_t ldc;
  float scale;
  int act;
  int vec_ok;
};

template <int MODE>
__device__ __forceinline__ void store_chunk2(const Epi2& ep, const uint32_t (&r)[32], int row, int col, int M,
                                             int N) {
  if (row >= M || col >= N) return;
  if (MODE == M2_BF16) {
    __nv_bfloat16* p = static_cast<__nv_bfloat16*>(ep.C) + (int64_t)row * ep.ldc + col;
    if (ep.vec_ok) {
#pragma unroll
      for (int v = 0; v < 4; v++) {
        if (col + v * 8 + 8 > N) break;
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const __nv_bfloat162 h =
              __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * j]), __uint_as_float(r[v * 8 + 2 * j + 1]));
          w[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(p + v * 8) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; j++)
        if (col + j < N) p[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
    }
  } else {
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
          for (int b = 0; b < 4; b++)
            x |= (uint32_t)(uint8_t)i8_epilogue((int32_t)r[v * 16 + j * 4 + b], ep.scale, ep.act != 0) << (8 * b);
          w[j] = x;
        }
        *reinterpret_cast<uint4*>(p + v * 16) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; j++)
        if (col + j < N) p[j] = i8_epilogue((int32_t)r[j], ep.scale, ep.act != 0);
    }
  }
}

template <int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, int M, int N, int K,
                Epi2 ep, DeviceStatus* status, int tiles_m, int tiles_n, int GM, int use_hints, int stages,
                int plain_leader) {
  using C = Cfg2<MODE>;
  constexpr int BK = ROW_BYTES / C::ELEM;
  constexpr uint32_t IDESC =
      make_idesc(C::D_FMT, C::AB_FMT, C::AB_FMT, 2 * BM, BN2) | (C::BMN ? IDESC_B_MN_MAJOR : 0u);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  uint8_t* ctrl = smem_raw + (tiles - raw) + STAGES2 * STAGE2_BYTES;
  const uint32_t bars = tiles + STAGES2 * STAGE2_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES2 + s); };
  auto tfull_bar = [&](int b) { return bars + 8u * (2 * STAGES2 + b); };
  auto tempty_bar = [&](int b) { return bars + 8u * (2 * STAGES2 + 2 + b); };
  const uint32_t slot_addr = bars + 8u * (2 * STAGES2 + 4);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(ctrl + 8 * (2 * STAGES2 + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl + 8 * (2 * STAGES2 + 4) + 4);
  const uint32_t abort_addr = slot_addr + 4;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = even CTA: owns full[] / tempty[] and issues the MMAs
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; s++) {
      mbar_init(full_bar(s), 1);   // the even CTA's producer; bytes of both CTAs ride on the tx count
      mbar_init(empty_bar(s), 1);  // one multicast commit
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 8);  // four epilogue warps in each CTA of the pair
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc2(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM2_COLS);
    tmem_relinquish2();
  }
  tc_fence_before();
  cluster_sync_all();  // barriers of both CTAs initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = tiles_m * tiles_n;  // 256 x 256 tiles
  const int num_kb = (K + BK - 1) / BK;
  auto tile_coord = [&](int t, int& tm, int& tn) {
    const int per_group = GM * tiles_n;
    const int group = t / per_group;
    const int first_m = group * GM;
    const int gm = min(GM, tiles_m - first_m);
    const int in_group = t - group * per_group;
    tm = first_m + in_group % gm;
    tn = in_group / gm;
  };
  auto give_up = [&](int where) {
    report_timeout(status, abort_flag, where);
    st_cluster_u32(mapa(abort_addr, rank ^ 1u), 1u);  // take the partner down too
  };

  if (warp == 0) {
    // ------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint64_t keep = l2_policy_evict_last(), stream_through = l2_policy_evict_first();
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        int tm, tn;
        tile_coord(t, tm, tn);
        const int m0 = tm * 2 * BM + (int)rank * BM;      // this CTA's A rows
        const int n0 = tn * BN2 + (int)rank * BHALF;       // this CTA's half of the tile's columns
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
            give_up(21);
            ok = false;
            break;
          }
          const uint32_t bar0 = mapa(full_bar(stage), 0);  // the even CTA's barrier
          const uint32_t dst = tiles + stage * STAGE2_BYTES;
          if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * STAGE2_BYTES);
          const int k0 = kb * BK;
          if (use_hints) {
            // experiment knob (1: A evict_last + B evict_first, 2: A evict_last only); both
            // measured worse than the default policy and are off by default
            tma_load_2d_pair_hint(dst, &tmA, bar0, k0, m0, keep);
            if (use_hints == 2) {
              if (C::BMN)
                tma_load_2d_pair(dst + A_TILE_BYTES, &tmB, bar0, n0, k0);
              else
                tma_load_2d_pair(dst + A_TILE_BYTES, &tmB, bar0, k0, n0);
            } else if (C::BMN)
              tma_load_2d_pair_hint(dst + A_TILE_BYTES, &tmB, bar0, n0, k0, stream_through);
            else
              tma_load_2d_pair_hint(dst + A_TILE_BYTES, &tmB, bar0, k0, n0, stream_through);
          } else if (plain_leader && rank == 0) {
            // experiment: the even CTA's own loads as ordinary (single-CTA) TMA loads
            tma_load_2d(dst, &tmA, full_bar(stage), k0, m0);
            if (C::BMN)
              tma_load_2d(dst + A_TILE_BYTES, &tmB, full_bar(stage), n0, k0);
            else
              tma_load_2d(dst + A_TILE_BYTES, &tmB, full_bar(stage), k0, n0);
          } else {
            tma_load_2d_pair(dst, &tmA, bar0, k0, m0);
            if (C::BMN)
              tma_load_2d_pair(dst + A_TILE_BYTES, &tmB, bar0, n0, k0);  // {128 bytes of N, BK rows of K}
            else
              tma_load_2d_pair(dst + A_TILE_BYTES, &tmB, bar0, k0, n0);
          }
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok || *abort_flag) {
        // error path: give copies in flight time to land (they complete on the even
        // CTA's barrier, which this CTA may not be able to poll)
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer (even CTA only)
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
          give_up(22);
          break;
        }
        tc_fence_after();
        const uint32_t d = tmem_base + (uint32_t)(acc * BN2);
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, WAIT_LIMIT_NS)) {
            give_up(23);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a0 = tiles + stage * STAGE2_BYTES;
          const uint32_t b0 = a0 + A_TILE_BYTES;
          const uint64_t da = smem_desc_k_sw128(a0);
          const uint64_t db = C::BMN ? smem_desc_mn_sw128(b0, BK) : smem_desc_k_sw128(b0);
          constexpr uint64_t B_ADV = C::BMN ? (uint64_t)((32 / C::ELEM) * ROW_BYTES / 16) : 2u;
#pragma unroll
          for (int ks = 0; ks < KSTEPS; ks++)
            tc_mma_pair<C::KIND>(d, da + (uint64_t)(ks * 2), db + ks * B_ADV, IDESC, (kb | ks) != 0);
          tc_commit_pair(empty_bar(stage));
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        tc_commit_pair(tfull_bar(acc));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------ epilogue warps 2..5 (both CTAs)
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = pair; t < num_tiles; t += num_pairs) {
      int tm, tn;
      tile_coord(t, tm, tn);
      const int m0 = tm * 2 * BM + (int)rank * BM, n0 = tn * BN2;
      if (!mbar_wait_warp(tfull_bar(acc), acc_phase, abort_flag, WAIT_LIMIT_NS)) {
        if (lane == 0) give_up(24);
        break;
      }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
#pragma unroll 1
      for (int ch = 0; ch < BN2 / 32; ch++) {
        const int col = n0 + ch * 32;
        if (col >= N) break;
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN2 + ch * 32), r);
        tmem_ld_wait();
        store_chunk2<MODE>(ep, r, row, col, M, N);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa(tempty_bar(acc), 0));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  tc_fence_before();
  cluster_sync_all();  // the pair leaves together
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, TMEM2_COLS);
  }
}

// --------------------------------------------------------------------------
// Tall variant: one pair computes a 512 x 256 tile as two 256 x 256 halves that
// share every B stage.  Each CTA holds two 128 x 256 accumulators (all 512
// tensor-memory columns), so there is no second tile to fill while one drains,
// but a stage of A0 | A1 | B-half (48 KiB, four stages) feeds twice the FLOPs:
// 24 instead of 32 bytes into shared memory per 128 x 256 x 64 block, and half
// the DRAM reads (6.3 instead of 10.9 - 13.6 GB per launch of the 32768 x 16384
// x 8192 problem).  Those bytes are power under the cap.  The price is an
// epilogue that is no longer hidden behind the next tile's MMAs; the lower half
// therefore runs `skew` k-blocks behind the upper one, so that the upper
// accumulator drains while the lower one still multiplies, and the next tile's
// upper half starts while the lower accumulator drains.
//
// More elaborate versions were built and measured slower than this one: separate
// rings for A0, A1 and B (more barrier waits and commits per k-block for the one
// issuing thread) and other orders of the two halves' MMAs.
constexpr int STAGE2T_BYTES = 2 * A_TILE_BYTES + BHALF * ROW_BYTES;  // 48 KiB per CTA
constexpr int STAGES2T = 4;
static_assert(STAGES2T * STAGE2T_BYTES <= STAGES2 * STAGE2_BYTES, "tall ring must fit the same allocation");
// Epilogue staging for TMA stores: per epilogue warp two buffers of 32 rows x 64 bytes, behind the control block.
constexpr int T_STAGING_OFFSET = STAGES2 * STAGE2_BYTES + 1024;
constexpr int T_EPI_WARPS = 8;  // two per tensor-memory lane quarter: each takes half of the tile's columns
constexpr int THREADS2T = 32 * (2 + T_EPI_WARPS);
constexpr int T_STAGING_BYTES = T_EPI_WARPS * 2 * 2048;
constexpr int SMEM2T_BYTES = T_STAGING_OFFSET + T_STAGING_BYTES + 1024;
static_assert(SMEM2T_BYTES <= 232448, "exceeds the shared memory a CTA can opt in to");

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all but the most recent bulk store of this thread have finished READING shared memory
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

template <int MODE>
__global__ void __launch_bounds__(THREADS2T, 1)
gemm_tc2t_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, int M, int N, int K, Epi2 ep, DeviceStatus* status,
                 int tiles_m, int tiles_n, int GM, int skew, int relax, int tma_store, int split_tail) {
  using C = Cfg2<MODE>;
  constexpr int BK = ROW_BYTES / C::ELEM;
  constexpr uint32_t IDESC =
      make_idesc(C::D_FMT, C::AB_FMT, C::AB_FMT, 2 * BM, BN2) | (C::BMN ? IDESC_B_MN_MAJOR : 0u);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  uint8_t* ctrl = smem_raw + (tiles - raw) + STAGES2 * STAGE2_BYTES;
  const uint32_t bars = tiles + STAGES2 * STAGE2_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES2 + s); };
  auto tfull_bar = [&](int b) { return bars + 8u * (2 * STAGES2 + b); };
  auto tempty_bar = [&](int b) { return bars + 8u * (2 * STAGES2 + 2 + b); };
  const uint32_t slot_addr = bars + 8u * (2 * STAGES2 + 4);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(ctrl + 8 * (2 * STAGES2 + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl + 8 * (2 * STAGES2 + 4) + 4);
  const uint32_t abort_addr = slot_addr + 4;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2T; s++) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 2 * T_EPI_WARPS);  // the epilogue warps of both CTAs of the pair
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
    prefetch_tensormap(&tmC);
  }
  if (warp == 1) {
    tmem_alloc2(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM2_COLS);
    tmem_relinquish2();
  }
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = tiles_m * tiles_n;  // 512 x 256 tiles
  const int num_kb = (K + BK - 1) / BK;
  const int d = min(skew, num_kb);
  // Work items of this pair: tiles pair, pair + num_pairs, ... as long as a whole round of pairs has one each.
  // A last, partial round of `rest` tiles would keep `rest` pairs busy for a whole tile while the others wait;
  // when there are pairs enough (2 rest <= num_pairs) it is split into 2 rest half tiles (the 256 x 256 upper or
  // lower half), one per pair, and takes half as long.  32768 x 16384: 4096 tiles on 74 pairs = 55 rounds + 26
  // tiles, i.e. 55.5 instead of 56 rounds.
  const int full_tiles = (num_tiles / num_pairs) * num_pairs;
  const int rest = num_tiles - full_tiles;
  const bool split_rest = split_tail && rest > 0 && 2 * rest <= num_pairs;
  // the item after this pair's full rounds: tile index (or -1) and which halves (0 = both, 1 = upper only, 2 = lower only)
  int last_tile = -1, last_mode = 0;
  if (split_rest) {
    if (pair < 2 * rest) last_tile = full_tiles + (pair >> 1), last_mode = 1 + (pair & 1);
  } else if (pair < rest) {
    last_tile = full_tiles + pair;
  }
  const int my_items = full_tiles / num_pairs + (last_tile >= 0 ? 1 : 0);
  auto item = [&](int i, int& t, int& mode) {
    if (i < full_tiles / num_pairs) {
      t = pair + i * num_pairs;
      mode = 0;
    } else {
      t = last_tile;
      mode = last_mode;
    }
  };
  auto tile_coord = [&](int t, int& tm, int& tn) {
    const int per_group = GM * tiles_n;
    const int group = t / per_group;
    const int first_m = group * GM;
    const int gm = min(GM, tiles_m - first_m);
    const int in_group = t - group * per_group;
    tm = first_m + in_group % gm;
    tn = in_group / gm;
  };
  auto give_up = [&](int where) {
    report_timeout(status, abort_flag, where);
    st_cluster_u32(mapa(abort_addr, rank ^ 1u), 1u);
  };

  if (warp == 0) {
    // ------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int it = 0; it < my_items && ok; it++) {
        int t, mode, tm, tn;
        item(it, t, mode);
        tile_coord(t, tm, tn);
        // this CTA's rows of the upper half (lower half: + 2 BM); a half tile's rows go where the upper half's do
        const int m0 = tm * 4 * BM + (int)rank * BM + (mode == 2 ? 2 * BM : 0);
        const int n0 = tn * BN2 + (int)rank * BHALF;
        for (int kb = 0; kb < num_kb; kb++) {
          // this thread is normally a ring ahead: sleeping between polls (relax ns) instead of
          // spinning is worth about 2 % under the power cap
          if (!(relax ? mbar_wait_relaxed(empty_bar(stage), phase ^ 1u, abort_flag, WAIT_LIMIT_NS, (uint32_t)relax)
                      : mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, WAIT_LIMIT_NS))) {
            give_up(41);
            ok = false;
            break;
          }
          const uint32_t bar0 = mapa(full_bar(stage), 0);
          const uint32_t dst = tiles + stage * STAGE2T_BYTES;
          if (rank == 0)
            mbar_arrive_expect_tx(full_bar(stage), 2 * (mode == 0 ? STAGE2T_BYTES : STAGE2T_BYTES - A_TILE_BYTES));
          const int k0 = kb * BK;
          tma_load_2d_pair(dst, &tmA, bar0, k0, m0);
          if (mode == 0) tma_load_2d_pair(dst + A_TILE_BYTES, &tmA, bar0, k0, m0 + 2 * BM);
          if (C::BMN)
            tma_load_2d_pair(dst + 2 * A_TILE_BYTES, &tmB, bar0, n0, k0);
          else
            tma_load_2d_pair(dst + 2 * A_TILE_BYTES, &tmB, bar0, k0, n0);
          if (++stage == STAGES2T) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok || *abort_flag) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer (even CTA only)
    if (lane == 0 && rank == 0) {
      // two cursors into the ring: `hi` (upper half, accumulator 0) runs d k-blocks
      // ahead of `lo` (lower half, accumulator 1); a stage is released by lo
      int hi_stage = 0, lo_stage = 0;
      uint32_t hi_phase = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      constexpr uint64_t B_ADV = C::BMN ? (uint64_t)((32 / C::ELEM) * ROW_BYTES / 16) : 2u;
      auto issue = [&](int stage, int half, bool first) {
        const uint32_t a0 = tiles + stage * STAGE2T_BYTES + half * A_TILE_BYTES;
        const uint32_t b0 = tiles + stage * STAGE2T_BYTES + 2 * A_TILE_BYTES;
        const uint64_t da = smem_desc_k_sw128(a0);
        const uint64_t db = C::BMN ? smem_desc_mn_sw128(b0, BK) : smem_desc_k_sw128(b0);
        const uint32_t dtm = tmem_base + (uint32_t)(half * BN2);
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++)
          tc_mma_pair<C::KIND>(dtm, da + (uint64_t)(ks * 2), db + ks * B_ADV, IDESC, !(first && ks == 0));
      };
      auto hi_step = [&](int kb) -> bool {  // upper half of k-block kb: wait for its stage, multiply
        if (!mbar_wait(full_bar(hi_stage), hi_phase, abort_flag, WAIT_LIMIT_NS)) {
          give_up(43);
          return false;
        }
        tc_fence_after();
        issue(hi_stage, 0, kb == 0);
        if (++hi_stage == STAGES2T) {
          hi_stage = 0;
          hi_phase ^= 1u;
        }
        return true;
      };
      for (int it = 0; it < my_items && ok; it++) {
        int t, mode;
        item(it, t, mode);
        if (!mbar_wait(tempty_bar(0), acc_phase ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
          give_up(42);
          break;
        }
        tc_fence_after();
        if (mode != 0) {
          // a half tile (always this pair's last item): accumulator 0 only, and the stage is released right away
          for (int kb = 0; kb < num_kb && ok; kb++) {
            const int stage = hi_stage;
            ok = hi_step(kb);
            if (ok) tc_commit_pair(empty_bar(stage));
          }
          if (ok) tc_commit_pair(tfull_bar(0));
          break;
        }
        // The upper half starts as soon as its accumulator is free and keeps going while the lower
        // accumulator still drains: at least d k-blocks ahead, at most STAGES2T - 1 (a stage is only
        // released by the lower half, and the producer needs one to load into).
        int hi_kb = 0;
        while (ok && hi_kb < num_kb && hi_kb < STAGES2T - 1 &&
               (hi_kb < d || !mbar_try_wait(tempty_bar(1), acc_phase ^ 1u))) {
          ok = hi_step(hi_kb++);
          if (ok && hi_kb == num_kb) tc_commit_pair(tfull_bar(0));  // upper accumulator complete
        }
        if (!ok) break;
        if (!mbar_wait(tempty_bar(1), acc_phase ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
          give_up(44);
          break;
        }
        tc_fence_after();
        for (int kb = 0; kb < num_kb; kb++) {
          // steady state: the upper half d k-blocks ahead (the lead of the start shrinks back to d)
          if (hi_kb < num_kb && hi_kb - kb <= d) {
            if (!hi_step(hi_kb++)) {
              ok = false;
              break;
            }
            if (hi_kb == num_kb) tc_commit_pair(tfull_bar(0));
          }
          // the lower half's stage was waited for when the upper half used it
          issue(lo_stage, 1, kb == 0);
          tc_commit_pair(empty_bar(lo_stage));
          if (++lo_stage == STAGES2T) lo_stage = 0;
        }
        if (!ok) break;
        tc_commit_pair(tfull_bar(1));
        acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------ epilogue warps 2..9 (both CTAs)
    // warp w may read tensor-memory lanes 32 (w % 4) .. + 31; the two warps of a lane quarter split the columns
    const int q = warp & 3, part = (warp - 2) >> 2;
    uint32_t acc_phase = 0;
    bool ok = true;
    // Output through shared memory and TMA stores (bf16, 16-byte pitch): a warp's 32 x 32 chunk is
    // written as whole 64-byte rows by the copy engine instead of as 16-byte pieces of 32 different
    // lines per store instruction; the engine clips at the edges of C.  Two staging buffers per
    // warp, 64-byte swizzle so that the 128-bit shared-memory writes are conflict free.
    const uint32_t stg = tiles + T_STAGING_OFFSET + (uint32_t)(warp - 2) * 4096u;
    int stg_buf = 0;
    // p: this lane's 32 columns as 16 packed bf16 pairs
    auto stage_store = [&](const uint32_t (&p)[16], int row0, int col) {
      if (row0 >= M || col >= N) return;  // warp-uniform
      if (lane == 0) bulk_wait_read_1();  // the store that last used this buffer has read it
      __syncwarp();
      const uint32_t buf = stg + (uint32_t)stg_buf * 2048u;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const uint32_t dst = buf + (uint32_t)lane * 64u + (uint32_t)((j ^ ((lane >> 1) & 3)) * 16);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(p[4 * j]), "r"(p[4 * j + 1]),
                     "r"(p[4 * j + 2]), "r"(p[4 * j + 3])
                     : "memory");
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        tma_store_2d(&tmC, buf, col, row0);
        bulk_commit();
      }
      stg_buf ^= 1;
    };
    auto pack = [&](const uint32_t (&r)[32], uint32_t (&p)[16]) {
#pragma unroll
      for (int i = 0; i < 16; i++) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
        p[i] = *reinterpret_cast<const uint32_t*>(&h);
      }
    };
    auto wait_full = [&](int half) -> bool {
      if (!mbar_wait_warp(tfull_bar(half), acc_phase, abort_flag, WAIT_LIMIT_NS)) {
        if (lane == 0) give_up(45);
        return false;
      }
      tc_fence_after();
      return true;
    };
    auto hand_back = [&](int half) {  // after the last tcgen05.wait::ld of this warp's share
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa(tempty_bar(half), 0));
    };
    auto acc_addr = [&](int half) {
      return tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(half * BN2 + part * (BN2 / 2));
    };
    for (int it = 0; it < my_items && ok; it++) {
      int t, mode, tm, tn;
      item(it, t, mode);
      tile_coord(t, tm, tn);
      const int n0 = tn * BN2;
      const int c0 = n0 + part * (BN2 / 2);
      // this warp's first row of the upper half (of the one half, for a half tile) and of the lower half
      const int mu = tm * 4 * BM + (int)rank * BM + q * 32 + (mode == 2 ? 2 * BM : 0);
      const int ml = mu + 2 * BM;
      uint32_t r0[32], r1[32], r2[32], r3[32];
      if (mode != 0) {
        // a half tile: accumulator 0 only
        if (!(ok = wait_full(0))) break;
        tmem_ld_32x32(acc_addr(0), r0);
        tmem_ld_32x32(acc_addr(0) + 32, r1);
        tmem_ld_32x32(acc_addr(0) + 64, r2);
        tmem_ld_32x32(acc_addr(0) + 96, r3);
        tmem_ld_wait();
        hand_back(0);
        if (MODE == M2_BF16 && tma_store) {
          uint32_t p0[16], p1[16], p2[16], p3[16];
          pack(r0, p0);
          pack(r1, p1);
          pack(r2, p2);
          pack(r3, p3);
          stage_store(p0, mu, c0);
          stage_store(p1, mu, c0 + 32);
          stage_store(p2, mu, c0 + 64);
          stage_store(p3, mu, c0 + 96);
        } else {
          store_chunk2<MODE>(ep, r0, mu + lane, c0, M, N);
          store_chunk2<MODE>(ep, r1, mu + lane, c0 + 32, M, N);
          store_chunk2<MODE>(ep, r2, mu + lane, c0 + 64, M, N);
          store_chunk2<MODE>(ep, r3, mu + lane, c0 + 96, M, N);
        }
        break;
      }
      if (MODE == M2_BF16 && tma_store) {
        // Upper accumulator: this warp's four 32-column chunks, all loads in flight at once, then the
        // accumulator goes back to the MMA thread; conversion and stores follow off the critical path.
        uint32_t p0[16], p1[16], p2[16], p3[16];
        if (!(ok = wait_full(0))) break;
        tmem_ld_32x32(acc_addr(0), r0);
        tmem_ld_32x32(acc_addr(0) + 32, r1);
        tmem_ld_32x32(acc_addr(0) + 64, r2);
        tmem_ld_32x32(acc_addr(0) + 96, r3);
        tmem_ld_wait();
        hand_back(0);
        pack(r0, p0);
        pack(r1, p1);
        pack(r2, p2);
        pack(r3, p3);
        // The lower accumulator completes a k-block or so after the upper one, and the next tile's
        // lower half cannot start before it is handed back.  So only two of the upper half's stores go
        // first; the other two chunks wait, packed, in 32 registers while the lower accumulator is read,
        // two chunks at a time so that everything stays in registers.  (With all four stores first,
        // 1.6 - 2.0 us of them, the hand-back came 2.8 us after the tile's last MMA was issued and the
        // tensor pipe idled for about half of that.)
        stage_store(p0, mu, c0);
        stage_store(p1, mu, c0 + 32);
        if (!(ok = wait_full(1))) break;
        tmem_ld_32x32(acc_addr(1), r0);
        tmem_ld_32x32(acc_addr(1) + 32, r1);
        tmem_ld_wait();
        pack(r0, p0);
        pack(r1, p1);
        tmem_ld_32x32(acc_addr(1) + 64, r0);
        tmem_ld_32x32(acc_addr(1) + 96, r1);
        tmem_ld_wait();
        hand_back(1);
        stage_store(p2, mu, c0 + 64);
        stage_store(p3, mu, c0 + 96);
        pack(r0, p2);
        pack(r1, p3);
        stage_store(p0, ml, c0);
        stage_store(p1, ml, c0 + 32);
        stage_store(p2, ml, c0 + 64);
        stage_store(p3, ml, c0 + 96);
      } else {
        for (int half = 0; half < 2 && ok; half++) {
          if (!(ok = wait_full(half))) break;
          tmem_ld_32x32(acc_addr(half), r0);
          tmem_ld_32x32(acc_addr(half) + 32, r1);
          tmem_ld_32x32(acc_addr(half) + 64, r2);
          tmem_ld_32x32(acc_addr(half) + 96, r3);
          tmem_ld_wait();
          hand_back(half);
          const int row = (half ? ml : mu) + lane;
          store_chunk2<MODE>(ep, r0, row, c0, M, N);
          store_chunk2<MODE>(ep, r1, row, c0 + 32, M, N);
          store_chunk2<MODE>(ep, r2, row, c0 + 64, M, N);
          store_chunk2<MODE>(ep, r3, row, c0 + 96, M, N);
        }
        if (!ok) break;
      }
      acc_phase ^= 1u;
    }
    if (lane == 0) bulk_wait_all();  // shared memory must outlive the stores that read it
    __syncwarp();
  }

  tc_fence_before();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, TMEM2_COLS);
  }
}

template <int MODE>
cudaError_t launch_tc2t(exo_b200_Context* ctx, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc,
                        int tma_store, int64_t M, int64_t N, int64_t K, const Epi2& ep) {
  EXOB200_SMEM_ATTR_ONCE((gemm_tc2t_kernel<MODE>), SMEM2T_BYTES, ctx->device);
  cudaError_t e;
  const int64_t tiles_m = (M + 4 * BM - 1) / (4 * BM), tiles_n = (N + BN2 - 1) / BN2;
  if (tiles_m * tiles_n > INT32_MAX || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return cudaErrorInvalidValue;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(THREADS2T);
  cfg.dynamicSmemBytes = SMEM2T_BYTES;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int& max_clusters = ctx->max_pairs[2 + MODE];  // per context, i.e. per device; the caller holds the context's mutex
  if (max_clusters == 0) {
    cfg.gridDim = dim3(2 * ctx->sm_count);
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, gemm_tc2t_kernel<MODE>, &cfg);
    if (e != cudaSuccess) return e;
    max_clusters = std::max(1, n);
  }
  const int pairs = (int)std::min<int64_t>(tiles_m * tiles_n, max_clusters);
  cfg.gridDim = dim3(2 * pairs);
  static const int gm = [] {
    const char* e = getenv("EXOB200_TC2T_GM");  // tile rows (of 512) per group
    return e ? std::max(1, atoi(e)) : 6;
  }();
  static const int skew = [] {
    const char* e = getenv("EXOB200_TC2T_SKEW");
    const int n = e ? atoi(e) : 1;
    return n >= 0 && n <= STAGES2T - 1 ? n : 1;
  }();
  static const int relax = [] {
    const char* e = getenv("EXOB200_TC2T_RELAX");  // ns the producer sleeps between polls (0: spin)
    return e ? std::max(0, atoi(e)) : 50;
  }();
  static const int direct = [] {
    const char* e = getenv("EXOB200_TC2T_DIRECT");  // 1: 16-byte global stores instead of staged TMA stores
    return e ? atoi(e) : 0;
  }();
  static const int split_tail = [] {
    const char* e = getenv("EXOB200_TC2T_SPLIT_TAIL");  // 0: a partial last round keeps whole tiles
    return e ? atoi(e) : 1;
  }();
  return cudaLaunchKernelEx(&cfg, gemm_tc2t_kernel<MODE>, ma, mb, mc, (int)M, (int)N, (int)K, ep, ctx->status_dev,
                            (int)tiles_m, (int)tiles_n, gm, skew, relax, (tma_store && !direct) ? 1 : 0, split_tail);
}

template <int MODE>
cudaError_t launch_tc2(exo_b200_Context* ctx, const CUtensorMap& ma, const CUtensorMap& mb, int64_t M, int64_t N,
                       int64_t K, const Epi2& ep) {
  EXOB200_SMEM_ATTR_ONCE((gemm_tc2_kernel<MODE>), SMEM2_BYTES, ctx->device);
  cudaError_t e;
  const int64_t tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = (N + BN2 - 1) / BN2;
  if (tiles_m * tiles_n > INT32_MAX || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return cudaErrorInvalidValue;
  // launched as clusters of two CTAs; size the grid to the number of pairs that
  // can be resident at once (a pair needs two SMs of the same GPC)
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = SMEM2_BYTES;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int& max_clusters = ctx->max_pairs[MODE];  // per context, i.e. per device; the caller holds the context's mutex
  if (max_clusters == 0) {
    cfg.gridDim = dim3(2 * ctx->sm_count);
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, gemm_tc2_kernel<MODE>, &cfg);
    if (e != cudaSuccess) return e;
    max_clusters = std::max(1, n);
  }
  const int pairs = (int)std::min<int64_t>(tiles_m * tiles_n, max_clusters);
  cfg.gridDim = dim3(2 * pairs);
  static const int gm = [] {
    const char* e = getenv("EXOB200_TC2_GM");
    return e ? std::max(1, atoi(e)) : 8;
  }();
  static const int hints = [] {
    const char* e = getenv("EXOB200_TC2_HINT");
    return e ? atoi(e) : 0;
  }();
  // Ring depth actually used (the shared-memory layout always has room for STAGES2).
  // Measured on the 32768 x 16384 x 8192 bf16 problem: 6 stages let the pairs drift so
  // far apart in K that L2 sharing drops (13.0 GB of DRAM reads per launch), 4 stages
  // read 8.2 GB, 3 stages starve the tensor pipe; 5 is the fastest both cold and under
  // the power cap.  EXOB200_TC2_STAGES overrides it.
  static const int stages = [] {
    const char* e = getenv("EXOB200_TC2_STAGES");
    const int n = e ? atoi(e) : 5;
    return n >= 2 && n <= STAGES2 ? n : 5;
  }();
  static const int plain_leader = [] {
    const char* e = getenv("EXOB200_TC2_PLAIN");
    return e ? atoi(e) : 0;
  }();
  return cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<MODE>, ma, mb, (int)M, (int)N, (int)K, ep, ctx->status_dev,
                            (int)tiles_m, (int)tiles_n, gm, hints, stages, plain_leader);
}

}  // namespace

// The pair kernel keeps the tensor pipe busier (96 % against 81 % active in ncu
// captures of the bf16 GEMM) and is used once there are enough 256 x 256 tiles;
// smaller problems quantise better on the 128 x 256 tiles of the single-CTA
// kernel.  Measured crossover, bf16 (TFLOP/s pair / single): 64 tiles 896 / 932,
// 128 tiles 1375 / 1360, 144 tiles 1375 / 1349, 192 tiles 1382 / 1287, 256 tiles
// 1396 / 1287; int8 at 256 tiles (4096^3) still favours the single-CTA kernel
// (52.1 against 53.9 us), so it keeps the threshold of four tiles per pair.
// EXOB200_TC2=0 switches the pair kernels off, =1 forces them.
bool tc2_wanted(int64_t M, int64_t N, int64_t min_tiles) {
  static const int mode = [] {
    const char* e = getenv("EXOB200_TC2");
    return e ? atoi(e) : -1;
  }();
  if (mode == 0) return false;
  if (mode == 1) return true;
  const int64_t tiles = ((M + 255) / 256) * ((N + 255) / 256);
  return tiles >= min_tiles;
}

cudaError_t launch_gemm_bf16_tc2(exo_b200_Context* ctx, int64_t M, int64_t N, int64_t K, const uint16_t* A,
                                 const uint16_t* B, uint16_t* C) {
  CUtensorMap ma, mb;
  cuuint64_t da[2] = {(cuuint64_t)K, (cuuint64_t)M}, db[2] = {(cuuint64_t)K, (cuuint64_t)N};
  cuuint64_t st[1] = {(cuuint64_t)K * 2};
  cuuint32_t boxa[2] = {64, (cuuint32_t)BM}, boxb[2] = {64, (cuuint32_t)BHALF};
  if (!make_tiled_map(&ma, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, da, st, boxa)) return cudaErrorUnknown;
  if (!make_tiled_map(&mb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, db, st, boxb)) return cudaErrorUnknown;
  Epi2 ep{C, N, 0.f, 0, (N % 8 == 0 && aligned16(C)) ? 1 : 0};
  // The tall variant (512 x 256 per pair) once every pair gets several such tiles: measured against
  // the 256 x 256 variant on one GPU, 32768 x 16384 x 8192: +1.4 % for a single cold launch, +2-3 %
  // over 20 launches, +7 % over 100, +6 % over 400 (1333 against 1255 TFLOP/s; the SM clock settles at
  // 1395 instead of 1113 MHz under the 1 kW cap).  EXOB200_TC2_TALL=0 / 1 forces the choice.
  static const int tall = [] {
    const char* e = getenv("EXOB200_TC2_TALL");
    return e ? atoi(e) : -1;
  }();
  const int64_t tall_tiles = ((M + 4 * BM - 1) / (4 * BM)) * ((N + BN2 - 1) / BN2);
  // (256 such tiles: 1414 against 1483 TFLOP/s for the 256 x 256 variant, the fourth round is half empty;
  // 288: 1527 against 1468; 384: 1475 against 1457; 512: 1484 against 1442)
  if (tall == 1 || (tall == -1 && tall_tiles >= 280)) {
    // C as 32 x 32 boxes of 64-byte rows for the staged epilogue; needs a 16-byte pitch and base
    CUtensorMap mc = ma;
    const int tma_store = ep.vec_ok;
    if (tma_store) {
      cuuint64_t dc[2] = {(cuuint64_t)N, (cuuint64_t)M};
      cuuint64_t sc[1] = {(cuuint64_t)N * 2};
      cuuint32_t boxc[2] = {32, 32};
      if (!make_tiled_map(&mc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, C, dc, sc, boxc, CU_TENSOR_MAP_SWIZZLE_64B))
        return cudaErrorUnknown;
    }
    return launch_tc2t<M2_BF16>(ctx, ma, mb, mc, tma_store, M, N, K, ep);
  }
  return launch_tc2<M2_BF16>(ctx, ma, mb, M, N, K, ep);
}

// The 512 x 256 variant for int8, from four such tiles per pair: 8192^3 350 us against 362 (256 x 256 per
// pair) and 367 (single CTA); at 4096^3 (128 tiles, a 73 % full second round) it loses, 56.2 against 52.9
// and 51.6 us, and 6144^3 (288 tiles) is a tie.
constexpr int64_t I8_TALL_MIN_TILES = 4 * 74;

cudaError_t launch_matmul_i8_tc2(exo_b200_Context* ctx, int64_t rows, int64_t cols, int64_t K, float scale, bool act,
                                 const int8_t* A, const int8_t* B, int8_t* C) {
  CUtensorMap ma, mb;
  cuuint64_t da[2] = {(cuuint64_t)K, (cuuint64_t)rows}, db[2] = {(cuuint64_t)cols, (cuuint64_t)K};
  cuuint64_t sa[1] = {(cuuint64_t)K}, sb[1] = {(cuuint64_t)cols};
  cuuint32_t boxa[2] = {128, (cuuint32_t)BM}, boxb[2] = {128, 128};
  if (!make_tiled_map(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, A, da, sa, boxa)) return cudaErrorUnknown;
  if (!make_tiled_map(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, B, db, sb, boxb)) return cudaErrorUnknown;
  Epi2 ep{C, cols, scale, act ? 1 : 0, (cols % 16 == 0 && aligned16(C)) ? 1 : 0};
  static const int tall = [] {
    const char* e = getenv("EXOB200_TC2_TALL");
    return e ? atoi(e) : -1;
  }();
  const int64_t tall_tiles = ((rows + 4 * BM - 1) / (4 * BM)) * ((cols + BN2 - 1) / BN2);
  if (tall == 1 || (tall == -1 && tall_tiles >= I8_TALL_MIN_TILES))
    return launch_tc2t<M2_I8>(ctx, ma, mb, ma, 0, rows, cols, K, ep);  // 16-byte global stores: no map for C
  return launch_tc2<M2_I8>(ctx, ma, mb, rows, cols, K, ep);
}

}  // namespace exob200
