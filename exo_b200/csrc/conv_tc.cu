// NHWC convolution as an implicit GEMM on tcgen05 tensor cores, with the im2col
// addressing done by the TMA producer.
//
// GEMM view (tests/test_im2col.py:41-62 states the decomposition: marshal, then
// a matmul whose reduction runs over channel x tap): M = output pixels, N = Co,
// K = (ky, kx, ci).  The im2col matrix is never built.  A CTA tile is a TH x TW
// patch of output pixels of one image (TH * TW <= 128 rows); for tap (ky, kx) and
// a 128-byte block of channels the producer issues ONE 4-D tiled TMA load of the
// input box {channels, TW, TH, 1} at coordinates (c0, ox0 + kx - pad,
// oy0 + ky - pad, n): the box lands in shared memory as TH*TW rows of 128 bytes
// -- exactly a K-major, 128-byte-swizzled A tile -- and every coordinate outside
// the image (padding, ragged patch edge, channels beyond Ci) is zero-filled by
// the TMA unit.  Weights [K, Co] row-major are read in place as the MN-major B
// operand (int8), or from a K-major hi/lo copy made by a small pre-pass (fp32).
//
// Two arithmetic modes on the same pipeline as the GEMM kernels (TMA -> mbarrier
// ring -> tcgen05.mma -> double-buffered accumulators in tensor memory ->
// epilogue warps):
//   I8      the Gemmini convolution, apps/gemmini/src/exo/conv.py:6-55: int32
//           accumulation (bias added in the epilogue: integer sums are order
//           independent), then scale / round-half-even / clamp / ReLU.  Bit-exact.
//   TF32X3  fp32 convolution of apps/x86/conv/conv.py:10-45 with each operand
//           split into TF32 hi + lo; bias + ReLU in the epilogue.  Not bit-exact;
//           the exact path is the FFMA kernel in conv_ffma.cu.
//
// Rows of the A tile beyond TH*TW are never written by TMA; they hold stale
// shared memory, produce garbage in their own accumulator rows only (rows of an
// MMA are independent) and are never stored.
#include <cuda.h>

#include <algorithm>
#include <cstring>

#include "i8_epilogue.cuh"
#include "kernels.cuh"
#include "tc_common.cuh"
#include "umma.cuh"

namespace exob200 {
namespace {

using namespace tc;
using namespace umma;

enum ConvMode { CONV_I8 = 0, CONV_TF32X3 = 1 };

template <int MODE>
struct CCfg;
template <>
struct CCfg<CONV_I8> {
  static constexpr int ELEM = 1, NA = 1, NB = 1, NPROD = 1, KIND = KIND_I8;
  static constexpr bool BMN = true;
  static constexpr uint32_t D_FMT = 2, AB_FMT = 1;
};
template <>
struct CCfg<CONV_TF32X3> {
  static constexpr int ELEM = 4, NA = 2, NB = 2, NPROD = 3, KIND = KIND_TF32;
  static constexpr bool BMN = false;
  static constexpr uint32_t D_FMT = 1, AB_FMT = 2;
};

template <int MODE, int BN>
__host__ __device__ constexpr int conv_stage_bytes() {
  return CCfg<MODE>::NA * A_TILE_BYTES + CCfg<MODE>::NB * BN * ROW_BYTES;
}
template <int MODE, int BN>
__host__ __device__ constexpr int conv_stages() {
  return (200 * 1024) / conv_stage_bytes<MODE, BN>() > 6 ? 6 : (200 * 1024) / conv_stage_bytes<MODE, BN>();
}
template <int MODE, int BN>
__host__ __device__ constexpr int conv_smem_bytes() {
  return conv_stages<MODE, BN>() * conv_stage_bytes<MODE, BN>() + 1024 + 256;
}

struct ConvTcParams {
  int batch, out_h, out_w, co, ci, kdim, pad;
  int TW, TH;              // output patch of a CTA tile
  int tiles_w, tiles_h, tiles_n;
  int cblocks;             // 128-byte channel blocks per tap
  void* out;
  const void* bias;        // int32 (I8) or float (TF32X3); may be null
  float scale;
  int act;                 // ReLU
};

template <int MODE, int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
               const __grid_constant__ CUtensorMap tmB0, const __grid_constant__ CUtensorMap tmB1,
               const ConvTcParams p, DeviceStatus* status) {
  using C = CCfg<MODE>;
  constexpr int STAGES = conv_stages<MODE, BN>();
  constexpr int STAGE_BYTES = conv_stage_bytes<MODE, BN>();
  constexpr int B_TILE = BN * ROW_BYTES;
  constexpr int BK = ROW_BYTES / C::ELEM;  // channels per stage
  constexpr uint32_t TMEM_COLS = 2 * BN;
  constexpr uint32_t IDESC = make_idesc(C::D_FMT, C::AB_FMT, C::AB_FMT, BM, BN) | (C::BMN ? IDESC_B_MN_MAJOR : 0u);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
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
      mbar_init(tempty_bar(b), 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
    prefetch_tensormap(&tmA0);
    prefetch_tensormap(&tmB0);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_dep_wait();  // the fp32 path's operands come from the split pre-pass that this launch may overlap

  const int tiles_per_image = p.tiles_h * p.tiles_w;
  const int num_tiles = p.batch * tiles_per_image * p.tiles_n;
  const int num_kb = p.kdim * p.kdim * p.cblocks;
  const uint32_t a_box_bytes = (uint32_t)(p.TW * p.TH * ROW_BYTES);
  const uint32_t tx_bytes = C::NA * a_box_bytes + C::NB * B_TILE;
  // tile index -> (n-tile fastest, so CTAs running together share the input patch)
  auto tile_coord = [&](int t, int& img, int& oy0, int& ox0, int& n0) {
    const int tn = t % p.tiles_n;
    int r = t / p.tiles_n;
    img = r / tiles_per_image;
    r -= img * tiles_per_image;
    oy0 = (r / p.tiles_w) * p.TH;
    ox0 = (r % p.tiles_w) * p.TW;
    n0 = tn * BN;
  };

  if (warp == 0) {
    // ---------------------------------- TMA producer: the implicit im2col
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t armed = 0, armed_parity = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int img, oy0, ox0, n0;
        tile_coord(t, img, oy0, ox0, n0);
        for (int kb = 0; kb < num_kb; kb++) {
          const int tap = kb / p.cblocks, cb = kb - tap * p.cblocks;
          const int ky = tap / p.kdim, kx = tap - ky * p.kdim;
          const int c0 = cb * BK;
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
            report_timeout(status, abort_flag, 11);
            ok = false;
            break;
          }
          const uint32_t bar = full_bar(stage);
          const uint32_t dst = tiles + stage * STAGE_BYTES;
          mbar_arrive_expect_tx(bar, tx_bytes);
          armed |= 1u << stage;
          armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
          // input patch shifted by the tap; everything outside the image reads as zero
          tma_load_4d(dst, &tmA0, bar, c0, ox0 + kx - p.pad, oy0 + ky - p.pad, img);
          if (C::NA > 1) tma_load_4d(dst + A_TILE_BYTES, &tmA1, bar, c0, ox0 + kx - p.pad, oy0 + ky - p.pad, img);
          const int krow = tap * p.ci + c0;  // first row of the [K, Co] weight matrix for this stage
          const uint32_t bdst = dst + C::NA * A_TILE_BYTES;
          if (C::BMN) {
            constexpr int NBOX = BN * C::ELEM / ROW_BYTES;
            constexpr int BOX_BYTES = BK * ROW_BYTES;
#pragma unroll
            for (int j = 0; j < NBOX; j++)
              tma_load_2d(bdst + j * BOX_BYTES, &tmB0, bar, n0 + j * (ROW_BYTES / C::ELEM), krow);
          } else {
            tma_load_2d(bdst, &tmB0, bar, krow, n0);
            if (C::NB > 1) tma_load_2d(bdst + B_TILE, &tmB1, bar, krow, n0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok || *abort_flag) {
        volatile int never = 0;
        for (int s = 0; s < STAGES; s++)
          if (armed & (1u << s)) mbar_wait(full_bar(s), (armed_parity >> s) & 1u, &never, DRAIN_LIMIT_NS);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------- MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, WAIT_LIMIT_NS)) {
          report_timeout(status, abort_flag, 12);
          break;
        }
        tc_fence_after();
        const uint32_t d = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, WAIT_LIMIT_NS)) {
            report_timeout(status, abort_flag, 13);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a0 = tiles + stage * STAGE_BYTES;
          const uint32_t b0 = a0 + C::NA * A_TILE_BYTES;
          const uint64_t da_hi = smem_desc_k_sw128(a0);
          const uint64_t db_hi = C::BMN ? smem_desc_mn_sw128(b0, BK) : smem_desc_k_sw128(b0);
          constexpr uint64_t B_ADV = C::BMN ? (uint64_t)((32 / C::ELEM) * ROW_BYTES / 16) : 2u;
#pragma unroll
          for (int ks = 0; ks < KSTEPS; ks++) {
            const uint64_t adv = (uint64_t)(ks * 2);
            if (C::NPROD == 1) {
              tc_mma<C::KIND>(d, da_hi + adv, db_hi + ks * B_ADV, IDESC, (kb | ks) != 0);
            } else {
              const uint64_t da_lo = smem_desc_k_sw128(a0 + A_TILE_BYTES);
              const uint64_t db_lo = smem_desc_k_sw128(b0 + B_TILE);
              tc_mma<C::KIND>(d, da_lo + adv, db_hi + adv, IDESC, (kb | ks) != 0);
              tc_mma<C::KIND>(d, da_hi + adv, db_lo + adv, IDESC, 1);
              tc_mma<C::KIND>(d, da_hi + adv, db_hi + adv, IDESC, 1);
            }
          }
          tc_commit(empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        tc_commit(tfull_bar(acc));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------- epilogue warps 2..5
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int img, oy0, ox0, n0;
      tile_coord(t, img, oy0, ox0, n0);
      if (!mbar_wait_warp(tfull_bar(acc), acc_phase, abort_flag, WAIT_LIMIT_NS)) {
        if (lane == 0) report_timeout(status, abort_flag, 14);
        break;
      }
      tc_fence_after();
      const int r = q * 32 + lane;  // row of the tile = pixel of the patch
      const int hl = r / p.TW, wl = r - hl * p.TW;
      const int oy = oy0 + hl, ox = ox0 + wl;
      const bool live = r < p.TW * p.TH && oy < p.out_h && ox < p.out_w;
      const int64_t pix = ((int64_t)img * p.out_h + oy) * p.out_w + ox;
#pragma unroll 1
      for (int ch = 0; ch < BN / 32; ch++) {
        const int col = n0 + ch * 32;
        if (col >= p.co) break;  // warp-uniform
        uint32_t v[32];
        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + ch * 32), v);
        tmem_ld_wait();
        if (!live) continue;
        if (MODE == CONV_I8) {
          int8_t* o = static_cast<int8_t*>(p.out) + pix * p.co + col;
          const int32_t* bias = static_cast<const int32_t*>(p.bias);
          if (p.co % 16 == 0) {
#pragma unroll
            for (int g = 0; g < 2; g++) {
              if (col + g * 16 + 16 > p.co) break;
              uint32_t w[4];
#pragma unroll
              for (int j = 0; j < 4; j++) {
                uint32_t x = 0;
#pragma unroll
                for (int b = 0; b < 4; b++) {
                  const int e = g * 16 + j * 4 + b;
                  const int32_t a = (int32_t)v[e] + (bias ? __ldg(bias + col + e) : 0);
                  x |= (uint32_t)(uint8_t)i8_epilogue(a, p.scale, p.act != 0) << (8 * b);
                }
                w[j] = x;
              }
              *reinterpret_cast<uint4*>(o + g * 16) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; e++)
              if (col + e < p.co)
                o[e] = i8_epilogue((int32_t)v[e] + (bias ? __ldg(bias + col + e) : 0), p.scale, p.act != 0);
          }
        } else {
          float* o = static_cast<float*>(p.out) + pix * p.co + col;
          const float* bias = static_cast<const float*>(p.bias);
#pragma unroll
          for (int g = 0; g < 8; g++) {
            float f[4];
#pragma unroll
            for (int b = 0; b < 4; b++) {
              const int e = g * 4 + b;
              float x = __uint_as_float(v[e]) + ((bias && col + e < p.co) ? __ldg(bias + col + e) : 0.f);
              f[b] = p.act ? (x > 0.f ? x : 0.f) : x;
            }
            if (p.co % 4 == 0) {
              if (col + g * 4 + 4 <= p.co) *reinterpret_cast<float4*>(o + g * 4) = make_float4(f[0], f[1], f[2], f[3]);
            } else {
#pragma unroll
              for (int b = 0; b < 4; b++)
                if (col + g * 4 + b < p.co) o[g * 4 + b] = f[b];
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// fp32 pre-pass, one launch for both operands.  Blocks [0, x_blocks): elementwise hi/lo split of the input
// (layout unchanged).  The remaining blocks: weights (either layout, given as strides) -> hi, lo as a
// K-major [Co][Kp] matrix with K ordered (ky, kx, ci), zero in the pad columns; skipped (w_blocks = 0)
// when the context still holds the split of these weights.
__global__ void conv_split_kernel(const float* __restrict__ x, int64_t n, float* __restrict__ x_hi,
                                  float* __restrict__ x_lo, int x_blocks, const float* __restrict__ w, ConvShape s,
                                  int K, int Kp, float* __restrict__ w_hi, float* __restrict__ w_lo) {
  grid_dep_launch();
  if ((int)blockIdx.x < x_blocks) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)x_blocks * blockDim.x) {
      float h, l;
      split_tf32(__ldg(x + i), h, l);
      x_hi[i] = h;
      x_lo[i] = l;
    }
    return;
  }
  const int w_blocks = (int)gridDim.x - x_blocks;
  const int64_t total = (int64_t)s.out_c * Kp;
  for (int64_t i = (blockIdx.x - x_blocks) * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)w_blocks * blockDim.x) {
    const int co = (int)(i / Kp), k = (int)(i - (int64_t)co * Kp);
    float h = 0.f, l = 0.f;
    if (k < K) {
      const int tap = k / s.in_c, ci = k - tap * s.in_c;
      const int ky = tap / s.kdim, kx = tap - ky * s.kdim;
      split_tf32(__ldg(w + ky * s.w_stride_ky + kx * s.w_stride_kx + ci * s.w_stride_ci + co), h, l);
    }
    w_hi[i] = h;
    w_lo[i] = l;
  }
}

void choose_patch(const ConvShape& s, ConvTcParams* p) {
  // widest patch that fits 128 rows: whole output rows when they fit
  p->TW = std::min(s.out_w, 128);
  p->TH = std::max(1, std::min(s.out_h, 128 / p->TW));
  p->tiles_w = (s.out_w + p->TW - 1) / p->TW;
  p->tiles_h = (s.out_h + p->TH - 1) / p->TH;
}

bool make_input_map(CUtensorMap* m, CUtensorMapDataType dt, int elem, const void* base, const ConvShape& s,
                    const ConvTcParams& p) {
  cuuint64_t dims[4] = {(cuuint64_t)s.in_c, (cuuint64_t)s.in_w, (cuuint64_t)s.in_h, (cuuint64_t)s.batch};
  cuuint64_t strides[3] = {(cuuint64_t)s.in_c * elem, (cuuint64_t)s.in_w * s.in_c * elem,
                           (cuuint64_t)s.in_h * s.in_w * s.in_c * elem};
  cuuint32_t box[4] = {(cuuint32_t)(ROW_BYTES / elem), (cuuint32_t)p.TW, (cuuint32_t)p.TH, 1};
  return make_tiled_map(m, dt, 4, base, dims, strides, box);
}

template <int MODE, int BN>
cudaError_t launch_conv(exo_b200_Context* ctx, const CUtensorMap& a0, const CUtensorMap& a1, const CUtensorMap& b0,
                        const CUtensorMap& b1, ConvTcParams p, bool after_prepass = false) {
  EXOB200_SMEM_ATTR_ONCE((conv_tc_kernel<MODE, BN>), (conv_smem_bytes<MODE, BN>()), ctx->device);
  p.tiles_n = (p.co + BN - 1) / BN;
  const int64_t num_tiles = (int64_t)p.batch * p.tiles_h * p.tiles_w * p.tiles_n;
  if (num_tiles > INT32_MAX) return cudaErrorInvalidValue;
  const int grid = (int)std::min<int64_t>(num_tiles, ctx->sm_count);
  if (after_prepass)
    return launch_dependent(conv_tc_kernel<MODE, BN>, dim3(grid), dim3(NUM_THREADS), conv_smem_bytes<MODE, BN>(),
                            ctx->stream, a0, a1, b0, b1, p, ctx->status_dev);
  conv_tc_kernel<MODE, BN><<<grid, NUM_THREADS, conv_smem_bytes<MODE, BN>(), ctx->stream>>>(a0, a1, b0, b1, p,
                                                                                           ctx->status_dev);
  return cudaGetLastError();
}

ConvTcParams base_params(const ConvShape& s, int elem) {
  ConvTcParams p;
  p.batch = s.batch;
  p.out_h = s.out_h;
  p.out_w = s.out_w;
  p.co = s.out_c;
  p.ci = s.in_c;
  p.kdim = s.kdim;
  p.pad = s.pad;
  p.cblocks = (s.in_c * elem + ROW_BYTES - 1) / ROW_BYTES;
  p.tiles_n = 0;
  choose_patch(s, &p);
  return p;
}

}  // namespace

// int8: needs the [K, Co] weight matrix contiguous (Kh,Kw,Ci,Co layout) with a
// 16-byte pitch, and a 16-byte channel pitch in the input.
bool tc_supported_conv_i8(const ConvShape& s, const void* inp, const void* weights) {
  return s.stride == 1 && s.in_c % 16 == 0 && s.out_c % 16 == 0 && aligned16(inp) && aligned16(weights) &&
         s.w_stride_ci == s.out_c && s.w_stride_kx == (int64_t)s.in_c * s.out_c &&
         s.w_stride_ky == (int64_t)s.kdim * s.in_c * s.out_c;
}

cudaError_t launch_conv_i8_tc(exo_b200_Context* ctx, const ConvShape& s, float scale, bool act, const int8_t* inp,
                              int8_t* out, const int8_t* weights, const int32_t* bias) {
  ConvTcParams p = base_params(s, 1);
  p.out = out;
  p.bias = bias;
  p.scale = scale;
  p.act = act ? 1 : 0;
  const int64_t K = (int64_t)s.kdim * s.kdim * s.in_c;
  CUtensorMap ma, mb;
  if (!make_input_map(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, inp, s, p)) return cudaErrorUnknown;
  {
    cuuint64_t dims[2] = {(cuuint64_t)s.out_c, (cuuint64_t)K};
    cuuint64_t strides[1] = {(cuuint64_t)s.out_c};
    cuuint32_t box[2] = {(cuuint32_t)ROW_BYTES, (cuuint32_t)ROW_BYTES};  // 128 bytes of Co x 128 K-rows
    if (!make_tiled_map(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, weights, dims, strides, box)) return cudaErrorUnknown;
  }
  if (s.out_c <= 128) return launch_conv<CONV_I8, 128>(ctx, ma, ma, mb, mb, p);
  return launch_conv<CONV_I8, 256>(ctx, ma, ma, mb, mb, p);
}

bool tc_supported_conv_tf32(const ConvShape& s, const void* inp) {
  return s.stride == 1 && s.in_c % 4 == 0 && aligned16(inp);
}

cudaError_t launch_conv_3xtf32_tc(exo_b200_Context* ctx, const ConvShape& s, const float* inp, float* out,
                                  const float* weights, const float* bias) {
  ConvTcParams p = base_params(s, 4);
  p.out = out;
  p.bias = bias;
  p.scale = 0.f;
  p.act = s.relu ? 1 : 0;
  const int64_t in_elems = (int64_t)s.batch * s.in_h * s.in_w * s.in_c;
  const int64_t K = (int64_t)s.kdim * s.kdim * s.in_c;
  const int64_t Kp = (K + 3) / 4 * 4;
  const int64_t w_elems = (int64_t)s.out_c * Kp;
  if (!acquire_scratch(ctx, 0, 2 * (size_t)in_elems * sizeof(float))) return cudaErrorMemoryAllocation;
  if (!acquire_scratch(ctx, 2, 2 * (size_t)w_elems * sizeof(float))) return cudaErrorMemoryAllocation;
  float* x_hi = static_cast<float*>(ctx->scratch[0]);
  float* x_lo = x_hi + in_elems;
  float* w_hi = static_cast<float*>(ctx->scratch[2]);  // a slot of its own: it may outlive the call (weight cache)
  float* w_lo = w_hi + w_elems;
  {
    // With the weight cache switched on (exo_b200_context_cache_weights) the split of these weights is
    // reused while the pointer, the shape and the layout stay the same.
    WeightKey key{weights, s.in_c, s.out_c, s.kdim, s.w_stride_ky, s.w_stride_kx, s.w_stride_ci};
    const bool cached = ctx->cache_weights && ctx->wkey_valid && memcmp(&ctx->wkey, &key, sizeof(key)) == 0;
    const int b1 = (int)std::min<int64_t>((in_elems + 255) / 256, (int64_t)ctx->sm_count * 16);
    const int b2 = cached ? 0 : (int)std::min<int64_t>((w_elems + 255) / 256, (int64_t)ctx->sm_count * 4);
    conv_split_kernel<<<b1 + b2, 256, 0, ctx->stream>>>(inp, in_elems, x_hi, x_lo, b1, weights, s, (int)K, (int)Kp,
                                                       w_hi, w_lo);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    ctx->wkey = key;
    ctx->wkey_valid = ctx->cache_weights;
  }
  CUtensorMap ma0, ma1, mb0, mb1;
  const CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  if (!make_input_map(&ma0, dt, 4, x_hi, s, p)) return cudaErrorUnknown;
  if (!make_input_map(&ma1, dt, 4, x_lo, s, p)) return cudaErrorUnknown;
  // the narrowest instruction shape that covers Co: with Co = 64 a 128-wide MMA would spend half of
  // its columns on padding
  const int bn = s.out_c <= 64 ? 64 : s.out_c <= 128 ? 128 : 256;
  {
    cuuint64_t dims[2] = {(cuuint64_t)Kp, (cuuint64_t)s.out_c};
    cuuint64_t strides[1] = {(cuuint64_t)Kp * 4};
    cuuint32_t box[2] = {(cuuint32_t)(ROW_BYTES / 4), (cuuint32_t)bn};
    if (!make_tiled_map(&mb0, dt, 2, w_hi, dims, strides, box)) return cudaErrorUnknown;
    if (!make_tiled_map(&mb1, dt, 2, w_lo, dims, strides, box)) return cudaErrorUnknown;
  }
  const cudaError_t e = bn == 64    ? launch_conv<CONV_TF32X3, 64>(ctx, ma0, ma1, mb0, mb1, p, true)
                        : bn == 128 ? launch_conv<CONV_TF32X3, 128>(ctx, ma0, ma1, mb0, mb1, p, true)
                                    : launch_conv<CONV_TF32X3, 256>(ctx, ma0, ma1, mb0, mb1, p, true);
  release_scratch(ctx, 0);
  release_scratch(ctx, 2);
  return e;
}

}  // namespace exob200
