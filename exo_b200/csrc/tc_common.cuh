// Pieces shared by the tensor-core kernels (tc_gemm.cu, conv_tc.cu): tile
// constants, the bounded-wait bookkeeping, the TF32 split, and the host-side
// tensor-map encoder.
#pragma once
#include <cstdlib>
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstring>
#include <mutex>
#include <string>

#include "common.cuh"
#include "umma.cuh"

namespace exob200 {
namespace tc {

constexpr int BM = 128;                   // rows per CTA tile = tensor-memory lanes
constexpr int ROW_BYTES = 128;            // one swizzle row: the K extent of a stage
constexpr int KSTEPS = ROW_BYTES / 32;    // every tcgen05.mma consumes 32 bytes of K
constexpr int NUM_THREADS = 192;          // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue
constexpr int A_TILE_BYTES = BM * ROW_BYTES;  // 16 KiB
constexpr uint64_t WAIT_LIMIT_NS = 1000ull * 1000ull * 1000ull;  // 1 s per wait
constexpr uint64_t DRAIN_LIMIT_NS = 1000ull * 1000ull;           // 1 ms per stage on the error path

__device__ __forceinline__ void report_timeout(DeviceStatus* st, volatile int* abort, int where) {
  *abort = 1;
  if (st != nullptr && st->code == 0) {
    st->where = where;
    st->block = (int)blockIdx.x;
    st->code = EXO_B200_ERR_TIMEOUT;
  }
}

// TF32 split of one fp32 value: hi = rna_tf32(x), lo = rna_tf32(x - hi).
// x - hi is exact in fp32.  Non-finite x keeps lo = 0 so inf stays inf.
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
  uint32_t h;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
  hi = __uint_as_float(h);
  const float d = x - hi;
  uint32_t l;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(d));
  lo = (fabsf(hi) <= 3.402823466e38f) ? __uint_as_float(l) : 0.f;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Tiled tensor map, 128-byte swizzle, zero fill outside the tensor.  dims/box are
// innermost first; strides (bytes) are for dimensions 1..rank-1.
inline bool make_tiled_map(CUtensorMap* m, CUtensorMapDataType dt, int rank, const void* base,
                           const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box,
                           CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  // Callers that repeat a call (a layer of a network, a benchmark loop) ask for the same maps
  // again and again; the driver's encoder takes a microsecond or two per map, which is a large
  // part of the host time of a 10 us kernel.  A map is a pure function of the arguments below,
  // so the last few are kept per thread.
  struct Key {
    const void* base;
    int dt, rank, swizzle;
    cuuint64_t dims[5], strides[4];
    cuuint32_t box[5];
  };
  struct Entry {
    Key key;
    CUtensorMap map;
    bool valid;
  };
  constexpr int kCached = 16;
  static thread_local Entry cache[kCached];
  static thread_local int next_slot = 0;
  Key key;
  memset(&key, 0, sizeof(key));
  key.base = base;
  key.dt = (int)dt;
  key.rank = rank;
  key.swizzle = (int)swizzle;
  for (int i = 0; i < rank; i++) {
    key.dims[i] = dims[i];
    key.box[i] = box[i];
    if (i + 1 < rank) key.strides[i] = strides[i];
  }
  for (int i = 0; i < kCached; i++)
    if (cache[i].valid && memcmp(&cache[i].key, &key, sizeof(Key)) == 0) {
      *m = cache[i].map;
      return true;
    }
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_error(EXO_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    return false;
  }
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  // EXOB200_L2_PROMOTION=0|64|128|256: how much L2 fetches from DRAM around a missing line (experiments)
  static const CUtensorMapL2promotion promo = [] {
    const char* e = getenv("EXOB200_L2_PROMOTION");
    const int v = e ? atoi(e) : 256;
    return v == 0     ? CU_TENSOR_MAP_L2_PROMOTION_NONE
           : v == 64  ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
           : v == 128 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                      : CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
  }();
  CUresult r = fn(m, dt, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error(EXO_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r));
    return false;
  }
  Entry& slot = cache[next_slot];
  next_slot = (next_slot + 1) % kCached;
  slot.key = key;
  slot.map = *m;
  slot.valid = true;
  return true;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Launches `kernel` so that it may begin before the preceding kernel of the stream has finished (the
// kernel calls grid_dep_wait() before it touches that kernel's output).  EXOB200_PDL=0 turns the
// attribute off (plain stream order).
template <class... KArgs, class... Args>
cudaError_t launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args&&... args) {
  static const bool pdl = [] {
    const char* e = getenv("EXOB200_PDL");
    return !(e && e[0] == '0');
  }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace tc
}  // namespace exob200

// Opt a kernel in to `bytes` of dynamic shared memory once per device instead of on every
// launch (the attribute is per function and device; the call costs about a microsecond).
// Used inside functions that return cudaError_t.
#define EXOB200_SMEM_ATTR_ONCE(kernel, bytes, device)                                                         \
  do {                                                                                                        \
    static std::atomic<uint64_t> done_{0};                                                                    \
    const uint64_t bit_ = 1ull << ((device) & 63);                                                            \
    if (!(done_.load(std::memory_order_acquire) & bit_)) {                                                    \
      cudaError_t e_ = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (bytes));    \
      if (e_ != cudaSuccess) return e_;                                                                       \
      done_.fetch_or(bit_, std::memory_order_release);                                                        \
    }                                                                                                         \
  } while (0)

