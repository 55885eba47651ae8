// Device-pointer launchers of every kernel in the library.  All pointers are
// device memory; launches are asynchronous on `stream`.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace exob200 {

// ---- exact fp32 SIMT kernels (sgemm_ffma.cu, conv_ffma.cu)
cudaError_t launch_sgemm_ffma(exo_b200_Context* ctx, int64_t M, int64_t N, int64_t K, const float* A,
                              const float* B, float* C);

// C += A * A^T on the upper triangle (ssyrk_ffma.cu); the 3xTF32 variant is in tc_gemm.cu
cudaError_t launch_ssyrk_ffma(exo_b200_Context* ctx, int64_t N, int64_t K, const float* A, float* C);
// which kernel launch_sgemm_ffma takes: 1 tall, 2 TMA GEMV, 3 cp.async GEMV, 4 skinny, else the tile configuration id
int sgemm_ffma_plan(int64_t M, int64_t N, int64_t K, bool va, bool vb);
cudaError_t launch_ssyrk_3xtf32_tc(exo_b200_Context* ctx, int64_t N, int64_t K, const float* A, float* C);

struct ConvShape {
  int batch, in_h, in_w, in_c, out_h, out_w, out_c, kdim, pad;
  int stride = 1;  // spatial stride (exact FFMA path only; the tensor-core paths take stride 1)
  // element strides of the weight tensor for (ky, kx, ci); co is contiguous
  int64_t w_stride_ky, w_stride_kx, w_stride_ci;
  bool relu;
};
cudaError_t launch_conv_ffma(cudaStream_t stream, const ConvShape& s, const float* inp, float* out,
                             const float* weights, const float* bias);

// ---- exact int8 SIMT kernels for shapes the tensor path cannot address (i8_simt.cu)
cudaError_t launch_matmul_i8_simt(cudaStream_t stream, int64_t N, int64_t M, int64_t K, float scale,
                                  bool act, const int8_t* A, const int8_t* B, int8_t* C);
cudaError_t launch_conv_i8_simt(cudaStream_t stream, const ConvShape& s, float scale, bool act,
                                const int8_t* inp, int8_t* out, const int8_t* weights,
                                const int32_t* bias);

// ---- tcgen05 / TMEM / TMA kernels (tc_gemm.cu)
// Each returns cudaErrorNotSupported when the operands do not meet TMA's
// address rules (16-byte aligned base and row pitch); callers then repack or
// use the SIMT kernel.
bool tc_supported_bf16(int64_t M, int64_t N, int64_t K, const void* A, const void* B, const void* C);
cudaError_t launch_gemm_bf16_tc(exo_b200_Context* ctx, int64_t M, int64_t N, int64_t K,
                                const uint16_t* A, const uint16_t* B, uint16_t* C);
bool tc_supported_i8(int64_t N, int64_t M, int64_t K, const void* A, const void* B, const void* C);
cudaError_t launch_matmul_i8_tc(exo_b200_Context* ctx, int64_t N, int64_t M, int64_t K, float scale,
                                bool act, const int8_t* A, const int8_t* B, int8_t* C);
bool tc_supported_tf32(int64_t M, int64_t N, int64_t K, const void* A, const void* B, const void* C);
cudaError_t launch_sgemm_3xtf32_tc(exo_b200_Context* ctx, int64_t M, int64_t N, int64_t K,
                                   const float* A, const float* B, float* C);

// one CTA waits on a barrier nobody signals; must end with EXO_B200_ERR_TIMEOUT in the status word
cudaError_t launch_bounded_wait_selftest(exo_b200_Context* ctx, uint64_t limit_ns);

// status word of matmul_on_cpu_static on the current device (tc_gemm.cu); false with the error set if a
// timeout was recorded there
bool collect_static_status();

// ---- CTA-pair (cta_group::2) variants of the bf16 and int8 GEMMs (tc_gemm2.cu)
bool tc2_wanted(int64_t M, int64_t N, int64_t min_tiles);
cudaError_t launch_gemm_bf16_tc2(exo_b200_Context* ctx, int64_t M, int64_t N, int64_t K, const uint16_t* A,
                                 const uint16_t* B, uint16_t* C);
cudaError_t launch_matmul_i8_tc2(exo_b200_Context* ctx, int64_t rows, int64_t cols, int64_t K, float scale, bool act,
                                 const int8_t* A, const int8_t* B, int8_t* C);

// ---- implicit-GEMM convolution on tensor cores, im2col done by TMA (conv_tc.cu)
bool tc_supported_conv_i8(const ConvShape& s, const void* inp, const void* weights);
cudaError_t launch_conv_i8_tc(exo_b200_Context* ctx, const ConvShape& s, float scale, bool act, const int8_t* inp,
                              int8_t* out, const int8_t* weights, const int32_t* bias);
bool tc_supported_conv_tf32(const ConvShape& s, const void* inp);
cudaError_t launch_conv_3xtf32_tc(exo_b200_Context* ctx, const ConvShape& s, const float* inp, float* out,
                                  const float* weights, const float* bias);

}  // namespace exob200
