// Measured ceilings for the roofline fractions this library reports.
//
// The reference ships no peak numbers; the denominators a benchmark divides by have to
// be measured on the GPU at hand.  exo_b200_measure_peak() times two kinds of probe
// kernels that do nothing but the instruction whose rate is the ceiling:
//   FP32 SIMT    every thread runs 16 independent chains of fma.rn.f32x2 (two IEEE fused
//                multiply-adds per instruction), 32 warps per SM, operands in registers;
//   tensor core  one thread per CTA issues tcgen05.mma (cta_group::1, M = 128, N = 256,
//                32 bytes of K per instruction) back to back into two accumulators in tensor
//                memory, operands resident in shared memory (filled with a byte pattern, not
//                zeros, so that the power drawn resembles real data), one CTA per SM;
//                kind::i8, kind::f16 (bf16) or kind::tf32.
// The result is the rate over the whole launch (CUDA events), i.e. at whatever clock the
// GPU sustains for a launch of the requested length.
#include <algorithm>

#include "kernels.cuh"
#include "tc_common.cuh"
#include "umma.cuh"

namespace exob200 {
namespace {

using namespace tc;
using namespace umma;

__global__ void __launch_bounds__(512, 2) simt_peak_kernel(int iters, float* sink) {
  uint64_t acc[16];
#pragma unroll
  for (int i = 0; i < 16; i++) {
    const float lo = (float)(threadIdx.x + i) * 1e-3f, hi = (float)(threadIdx.x + 2 * i) * 1e-3f;
    asm("mov.b64 %0, {%1, %2};" : "=l"(acc[i]) : "f"(lo), "f"(hi));
  }
  uint64_t a, b;
  asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(1.0001f), "f"(0.9999f));
  asm("mov.b64 %0, {%1, %2};" : "=l"(b) : "f"(1e-6f), "f"(-1e-6f));
  for (int it = 0; it < iters; it++) {
#pragma unroll
    for (int u = 0; u < 4; u++)
#pragma unroll
      for (int i = 0; i < 16; i++) asm volatile("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(acc[i]) : "l"(a), "l"(b));
  }
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 16; i++) {
    float lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(acc[i]));
    s += lo + hi;
  }
  if (s == 123.456f) sink[0] = s;  // keeps the chains alive; practically never true
}
constexpr double kSimtFmaPerThreadPerIter = 4.0 * 16.0 * 2.0;

constexpr int PROBE_BN = 256;
constexpr int PROBE_SMEM = A_TILE_BYTES + PROBE_BN * ROW_BYTES + 1024 + 64;

template <int KIND>
__global__ void __launch_bounds__(128, 1) tensor_peak_kernel(int iters, uint32_t idesc, DeviceStatus* status) {
  extern __shared__ uint8_t probe_raw[];
  const uint32_t raw = smem_u32(probe_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  uint8_t* base = probe_raw + (tiles - raw);
  const uint32_t bar = tiles + A_TILE_BYTES + PROBE_BN * ROW_BYTES;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base + A_TILE_BYTES + PROBE_BN * ROW_BYTES + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base + A_TILE_BYTES + PROBE_BN * ROW_BYTES + 12);
  // operands: a byte pattern with small magnitudes in every format (no NaN / Inf patterns for bf16 / tf32)
  for (int i = threadIdx.x; i < (A_TILE_BYTES + PROBE_BN * ROW_BYTES) / 4; i += blockDim.x) {
    uint32_t x = (uint32_t)i * 2654435761u + blockIdx.x;
    x ^= x >> 13;
    reinterpret_cast<uint32_t*>(base)[i] = x & 0x3F7F3F7Fu;
  }
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  fence_proxy_async();  // generic-proxy writes of the operands before the tensor core reads them
  if (threadIdx.x < 32) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) {
    const uint64_t da = smem_desc_k_sw128(tiles);
    const uint64_t db = smem_desc_k_sw128(tiles + A_TILE_BYTES);
    for (int it = 0; it < iters; it++) {
      const uint32_t d = tmem_base + (uint32_t)((it & 1) * PROBE_BN);
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ks++) tc_mma<KIND>(d, da + (uint64_t)(ks * 2), db + (uint64_t)(ks * 2), idesc, it > 1 || ks > 0);
    }
    tc_commit(bar);
    if (!mbar_wait(bar, 0, abort_flag, 2 * WAIT_LIMIT_NS)) report_timeout(status, abort_flag, 77);
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <class Launch>
double timed(exo_b200_Context* c, Launch launch, double work_per_iter, int milliseconds) {
  cudaEvent_t e0, e1;
  if (!check_cuda(cudaEventCreate(&e0), "cudaEventCreate") || !check_cuda(cudaEventCreate(&e1), "cudaEventCreate"))
    return -1.0;
  double rate = -1.0;
  int iters = 256;
  for (int round = 0; round < 4; round++) {  // calibrate the loop count, then measure
    cudaEventRecord(e0, c->stream);
    launch(iters);
    cudaEventRecord(e1, c->stream);
    if (!check_cuda(cudaGetLastError(), "probe launch") ||
        !check_cuda(cudaStreamSynchronize(c->stream), "cudaStreamSynchronize"))
      break;
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    rate = work_per_iter * iters / (ms * 1e-3) / 1e12;
    if (round >= 1 && ms >= 0.6f * (float)milliseconds) break;
    const double want = (double)iters * (double)milliseconds / std::max(ms, 0.01f);
    iters = (int)std::min<double>(std::max(want, 256.0), 4.0e6);
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return rate;
}

}  // namespace
}  // namespace exob200

using namespace exob200;

extern "C" __attribute__((visibility("default"))) double exo_b200_measure_peak(int what, int milliseconds) {
  clear_error();
  ContextUse use(default_context());
  exo_b200_Context* c = use.get();
  if (!c) return -1.0;
  if (milliseconds < 1 || milliseconds > 500 || what < 0 || what > 3) {
    set_error(EXO_B200_ERR_INVALID_ARGUMENT, "exo_b200_measure_peak: what in 0..3, milliseconds in 1..500");
    return -1.0;
  }
  const int sms = c->sm_count;
  double rate = -1.0;
  if (what == EXO_B200_PEAK_FP32_SIMT) {
    float* sink = nullptr;
    if (!check_cuda(cudaMalloc(&sink, 256), "cudaMalloc")) return -1.0;
    const int grid = 2 * sms, threads = 512;
    rate = timed(c, [&](int iters) { simt_peak_kernel<<<grid, threads, 0, c->stream>>>(iters, sink); },
                 2.0 * kSimtFmaPerThreadPerIter * threads * grid, milliseconds);
    cudaFree(sink);
  } else {
    const double flop_per_iter = (double)KSTEPS * 2.0 * BM * PROBE_BN * sms;  // x elements of K per instruction, below
    auto run = [&](auto kernel, uint32_t idesc, int k_per_instr) {
      if (!check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PROBE_SMEM),
                      "cudaFuncSetAttribute"))
        return -1.0;
      return timed(c, [&](int iters) { kernel<<<sms, 128, PROBE_SMEM, c->stream>>>(iters, idesc, c->status_dev); },
                   flop_per_iter * k_per_instr, milliseconds);
    };
    if (what == EXO_B200_PEAK_INT8_TENSOR) rate = run(tensor_peak_kernel<KIND_I8>, make_idesc(2, 1, 1, BM, PROBE_BN), 32);
    else if (what == EXO_B200_PEAK_BF16_TENSOR) rate = run(tensor_peak_kernel<KIND_F16>, make_idesc(1, 1, 1, BM, PROBE_BN), 16);
    else rate = run(tensor_peak_kernel<KIND_TF32>, make_idesc(1, 2, 2, BM, PROBE_BN), 8);
  }
  if (rate < 0) return -1.0;
  if (c->status_host && c->status_host->code != 0) {
    c->status_host->code = 0;
    set_error(EXO_B200_ERR_TIMEOUT, "exo_b200_measure_peak: the probe's bounded wait ran out");
    return -1.0;
  }
  return rate;
}
