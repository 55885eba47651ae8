// The C-ABI entry points: argument checks, host/device operand staging, and
// the choice of kernel.  Every computation runs on the GPU; an entry point that
// cannot reach a device reports an error through exo_b200_last_error() and
// leaves its output untouched -- there is no CPU path.
#include <cstdlib>
#include <cstring>

#include "../../include/exo_b200_gemmini_shim.h"
#include "common.cuh"
#include "kernels.cuh"

using namespace exob200;

namespace {

// Row pipeline for host operands: worth it from about 64 MB of row traffic; chunks of
// about 96 MB (rounded to 256 rows) keep four buffers under 400 MB of device memory.
bool want_row_pipeline(int64_t rows, const void* host_a, const void* host_c, size_t bytes_per_row) {
  static const bool off = [] {
    const char* e = getenv("EXOB200_NO_PIPELINE");
    return e && e[0] == '1';
  }();
  if (off) return false;
  if (!((double)rows * (double)bytes_per_row >= 64.0e6 && rows >= 1024)) return false;  // cheap test first
  return !is_device_pointer(host_a) && !is_device_pointer(host_c);
}
// The two-dimensional pipeline pays when the second operand is a sizeable part of the
// upload (the row pipeline cannot start before all of it is in place) and there are
// enough blocks to overlap.  EXOB200_PIPELINE=rows keeps the row pipeline (A/B timing).
bool want_block_pipeline(int64_t rows, int64_t cols, size_t k_bytes, const void* host_a, const void* host_b,
                         const void* host_c) {
  static const bool off = [] {
    const char* e = getenv("EXOB200_NO_PIPELINE");
    const char* m = getenv("EXOB200_PIPELINE");
    return (e && e[0] == '1') || (m && !strcmp(m, "rows"));
  }();
  if (off) return false;
  const double a_bytes = (double)rows * (double)k_bytes, b_bytes = (double)cols * (double)k_bytes;
  if (!(rows >= 8192 && cols >= 8192 && b_bytes >= 32.0e6 && a_bytes + b_bytes <= 8.0e9)) return false;
  return !is_device_pointer(host_a) && !is_device_pointer(host_b) && !is_device_pointer(host_c);
}
int64_t pipeline_chunk_rows(int64_t rows, size_t bytes_per_row) {
  int64_t r = (int64_t)(96.0e6 / (double)bytes_per_row);
  r = r / 256 * 256;
  if (r < 256) r = 256;
  // at least four chunks so the pipeline has something to overlap
  while (r > 256 && (rows + r - 1) / r < 4) r = (r / 2) / 256 * 256 > 0 ? (r / 2) / 256 * 256 : 256;
  return r;
}

bool bad_args(const char* fn, bool cond, const char* what) {
  if (!cond) return false;
  set_error(EXO_B200_ERR_INVALID_ARGUMENT, std::string(fn) + ": " + what);
  return true;
}

// ---------------------------------------------------------------- SGEMM
void sgemm_dispatch(const char* fn, void* ctxt, int path, int_fast32_t M, int_fast32_t N, int_fast32_t K,
                    const float* A, const float* B, float* C, bool path_by_name = false) {
  clear_error();
  if (bad_args(fn, M < 1 || N < 1 || K < 1, "M, N, K must be >= 1")) return;
  if (bad_args(fn, !A || !B || !C, "NULL tensor")) return;
  ContextUse use(resolve_context(ctxt));
  exo_b200_Context* c = use.get();
  if (!c) return;
  if (path < 0) path = c->sgemm_path;
  Operand a, b, cc;
  if (want_row_pipeline(M, A, C, ((size_t)K + 2 * (size_t)N) * 4)) {
    if (!stage_in(c, 1, B, sizeof(float) * (size_t)K * N, true, &b)) return;
    const float* dB = static_cast<const float*>(b.dev);
    RowPipeline p{M, pipeline_chunk_rows(M, ((size_t)K + 2 * (size_t)N) * 4), A, (size_t)K * 4, C, (size_t)N * 4, true};
    const bool tensor = path == EXO_B200_SGEMM_3XTF32;
    if (!run_row_pipeline(c, p, [&](int64_t rows, const void* dA, void* dC) {
          if (tensor && rows >= 128 && N >= 64)
            return launch_sgemm_3xtf32_tc(c, rows, N, K, static_cast<const float*>(dA), dB, static_cast<float*>(dC));
          return launch_sgemm_ffma(c, rows, N, K, static_cast<const float*>(dA), dB, static_cast<float*>(dC));
        }))
      return;
    finish(c, true);
    return;
  }
  if (!stage_in(c, 0, A, sizeof(float) * (size_t)M * K, true, &a)) return;
  if (!stage_in(c, 1, B, sizeof(float) * (size_t)K * N, true, &b)) return;
  if (!stage_in(c, 2, C, sizeof(float) * (size_t)M * N, true, &cc)) return;  // C is read: +=
  const float* dA = static_cast<const float*>(a.dev);
  const float* dB = static_cast<const float*>(b.dev);
  float* dC = static_cast<float*>(cc.dev);
  cudaError_t e;
  // The tensor path has fixed costs (two split pre-passes, 128 x 256 tiles); for
  // skinny or small problems the exact FFMA kernels are faster and more accurate,
  // so the context-wide "3xTF32" setting means "tensor cores where they pay"; the
  // entry point that names the path (sgemm_exo_3xtf32) always takes it.
  const bool tensor_pays =
      path_by_name || (M >= 128 && N >= 64 && 2.0 * (double)M * (double)N * (double)K >= 1.0e9);
  if (path == EXO_B200_SGEMM_3XTF32 && tensor_pays && tc_supported_tf32(M, N, K, dA, dB, dC))
    e = launch_sgemm_3xtf32_tc(c, M, N, K, dA, dB, dC);
  else
    e = launch_sgemm_ffma(c, M, N, K, dA, dB, dC);
  if (!check_cuda(e, fn)) return;
  if (!stage_out(c, cc)) return;
  finish(c, a.staged || b.staged || cc.staged);
}

// ---------------------------------------------------------------- SSYRK
void ssyrk_dispatch(const char* fn, void* ctxt, int path, int_fast32_t N, int_fast32_t K, const float* A, float* C) {
  clear_error();
  if (bad_args(fn, N < 1 || K < 1, "N, K must be >= 1")) return;
  if (bad_args(fn, !A || !C, "NULL tensor")) return;
  ContextUse use(resolve_context(ctxt));
  exo_b200_Context* c = use.get();
  if (!c) return;
  if (path < 0) path = c->sgemm_path;
  Operand a, cc;
  if (!stage_in(c, 0, A, sizeof(float) * (size_t)N * K, true, &a)) return;
  if (!stage_in(c, 2, C, sizeof(float) * (size_t)N * N, true, &cc)) return;  // read (+=) and written
  const float* dA = static_cast<const float*>(a.dev);
  float* dC = static_cast<float*>(cc.dev);
  const cudaError_t e = path == EXO_B200_SGEMM_3XTF32 ? launch_ssyrk_3xtf32_tc(c, N, K, dA, dC)
                                                      : launch_ssyrk_ffma(c, N, K, dA, dC);
  if (!check_cuda(e, fn)) return;
  // a staged C travels back whole: its lower triangle went up unchanged and comes back unchanged
  if (!stage_out(c, cc)) return;
  finish(c, a.staged || cc.staged);
}

// ----------------------------------------------------------------- conv
void conv_dispatch(const char* fn, void* ctxt, const ConvShape& s, const float* inp, float* output,
                   const float* weights, const float* bias, int path = -1) {
  clear_error();
  if (bad_args(fn, s.batch < 1 || s.in_h < 1 || s.in_w < 1 || s.in_c < 1 || s.out_c < 1 || s.kdim < 1 ||
                       s.pad < 0 || s.out_h < 1 || s.out_w < 1,
               "sizes must be >= 1 (pad >= 0) and the kernel must fit the padded input"))
    return;
  if (bad_args(fn, !inp || !output || !weights, "NULL tensor")) return;
  ContextUse use(resolve_context(ctxt));
  exo_b200_Context* c = use.get();
  if (!c) return;
  Operand i, o, w, b;
  const size_t in_elems = (size_t)s.batch * s.in_h * s.in_w * s.in_c;
  const size_t out_elems = (size_t)s.batch * s.out_h * s.out_w * s.out_c;
  const size_t w_elems = (size_t)s.kdim * s.kdim * s.in_c * s.out_c;
  if (!stage_in(c, 0, inp, sizeof(float) * in_elems, true, &i)) return;
  if (!stage_in(c, 1, weights, sizeof(float) * w_elems, true, &w)) return;
  if (!stage_in(c, 2, output, sizeof(float) * out_elems, false, &o)) return;
  b.dev = nullptr;
  b.staged = false;
  if (bias && !stage_in(c, 3, bias, sizeof(float) * (size_t)s.out_c, true, &b)) return;
  if (path < 0) path = c->sgemm_path;  // one switch selects exact FFMA or 3xTF32 for every fp32 kernel
  cudaError_t e;
  if (path == EXO_B200_SGEMM_3XTF32 && tc_supported_conv_tf32(s, i.dev))
    e = launch_conv_3xtf32_tc(c, s, static_cast<const float*>(i.dev), static_cast<float*>(o.dev),
                              static_cast<const float*>(w.dev), static_cast<const float*>(b.dev));
  else
    e = launch_conv_ffma(c->stream, s, static_cast<const float*>(i.dev), static_cast<float*>(o.dev),
                         static_cast<const float*>(w.dev), static_cast<const float*>(b.dev));
  if (!check_cuda(e, fn)) return;
  if (!stage_out(c, o)) return;
  finish(c, i.staged || w.staged || o.staged || b.staged);
}

ConvShape x86_conv_shape(int_fast32_t out_h, int_fast32_t out_w, int_fast32_t out_channel, int_fast32_t in_h,
                         int_fast32_t in_w, int_fast32_t in_channel, int_fast32_t kernel_dim,
                         int_fast32_t batch_size) {
  ConvShape s;
  s.batch = (int)batch_size;
  s.in_h = (int)in_h;
  s.in_w = (int)in_w;
  s.in_c = (int)in_channel;
  s.out_h = (int)out_h;
  s.out_w = (int)out_w;
  s.out_c = (int)out_channel;
  s.kdim = (int)kernel_dim;
  s.pad = 0;
  // weights f32[in_channel, kernel_dim, kernel_dim, out_channel] (apps/x86/conv/conv.py:22)
  s.w_stride_kx = out_channel;
  s.w_stride_ky = kernel_dim * out_channel;
  s.w_stride_ci = kernel_dim * kernel_dim * out_channel;
  s.relu = true;
  return s;
}

// ----------------------------------------------------------- int8 matmul
void matmul_i8_dispatch(const char* fn, int_fast32_t N, int_fast32_t M, int_fast32_t K, const float* scale,
                        bool act, const int8_t* A, const int8_t* B, int8_t* C) {
  clear_error();
  if (bad_args(fn, N < 1 || M < 1 || K < 1, "N, M, K must be >= 1")) return;
  if (bad_args(fn, !A || !B || !C || !scale, "NULL tensor or scale")) return;
  ContextUse use(default_context());  // ctxt may be an uninitialised pointer: never read it
  exo_b200_Context* c = use.get();
  if (!c) return;
  float s;
  if (is_device_pointer(scale)) {
    if (!check_cuda(cudaMemcpyAsync(&s, scale, sizeof(float), cudaMemcpyDeviceToHost, c->stream), fn)) return;
    if (!check_cuda(cudaStreamSynchronize(c->stream), fn)) return;
  } else {
    s = *scale;
  }
  Operand a, b, cc;
  if (want_row_pipeline(N, A, C, (size_t)K + (size_t)M) && K % 16 == 0) {
    if (!stage_in(c, 1, B, (size_t)K * M, true, &b)) return;
    const int8_t* dB = static_cast<const int8_t*>(b.dev);
    RowPipeline p{N, pipeline_chunk_rows(N, (size_t)K + (size_t)M), A, (size_t)K, C, (size_t)M, false};
    if (!run_row_pipeline(c, p, [&](int64_t rows, const void* dA, void* dC) {
          return launch_matmul_i8_tc(c, rows, M, K, s, act, static_cast<const int8_t*>(dA), dB, static_cast<int8_t*>(dC));
        }))
      return;
    finish(c, true);
    return;
  }
  if (!stage_in(c, 0, A, (size_t)N * K, true, &a)) return;
  if (!stage_in(c, 1, B, (size_t)K * M, true, &b)) return;
  if (!stage_in(c, 2, C, (size_t)N * M, false, &cc)) return;
  const int8_t* dA = static_cast<const int8_t*>(a.dev);
  const int8_t* dB = static_cast<const int8_t*>(b.dev);
  int8_t* dC = static_cast<int8_t*>(cc.dev);
  cudaError_t e;
  if (tc_supported_i8(N, M, K, dA, dB, dC))
    e = launch_matmul_i8_tc(c, N, M, K, s, act, dA, dB, dC);
  else
    e = launch_matmul_i8_simt(c->stream, N, M, K, s, act, dA, dB, dC);
  if (!check_cuda(e, fn)) return;
  if (!stage_out(c, cc)) return;
  finish(c, a.staged || b.staged || cc.staged);
}

// ------------------------------------------------------------- int8 conv
void conv_i8_dispatch(const char* fn, int_fast32_t batch_size, int_fast32_t out_dim, int_fast32_t out_channel,
                      int_fast32_t kernel_dim, int_fast32_t in_channel, int_fast32_t in_dim, int8_t* output,
                      const int32_t* bias, const int8_t* inp, const int8_t* weights, bool act,
                      const float* scale) {
  clear_error();
  if (bad_args(fn, batch_size < 1 || out_dim < 1 || out_channel < 1 || kernel_dim < 1 || in_channel < 1 ||
                       in_dim < 1,
               "sizes must be >= 1"))
    return;
  if (bad_args(fn, out_dim != in_dim - kernel_dim + 1, "out_dim must equal in_dim - kernel_dim + 1")) return;
  if (bad_args(fn, !output || !bias || !inp || !weights || !scale, "NULL tensor or scale")) return;
  ContextUse use(default_context());
  exo_b200_Context* c = use.get();
  if (!c) return;
  float sc;
  if (is_device_pointer(scale)) {
    if (!check_cuda(cudaMemcpyAsync(&sc, scale, sizeof(float), cudaMemcpyDeviceToHost, c->stream), fn)) return;
    if (!check_cuda(cudaStreamSynchronize(c->stream), fn)) return;
  } else {
    sc = *scale;
  }
  ConvShape s;
  s.batch = (int)batch_size;
  s.in_h = s.in_w = (int)in_dim;
  s.in_c = (int)in_channel;
  s.out_h = s.out_w = (int)out_dim;
  s.out_c = (int)out_channel;
  s.kdim = (int)kernel_dim;
  s.pad = 0;
  // weights i8[kernel_dim, kernel_dim, in_channel, out_channel] (apps/gemmini/src/exo/conv.py:17)
  s.w_stride_ci = out_channel;
  s.w_stride_kx = in_channel * out_channel;
  s.w_stride_ky = kernel_dim * in_channel * out_channel;
  s.relu = act;
  Operand i, o, w, b;
  if (!stage_in(c, 0, inp, (size_t)batch_size * in_dim * in_dim * in_channel, true, &i)) return;
  if (!stage_in(c, 1, weights, (size_t)kernel_dim * kernel_dim * in_channel * out_channel, true, &w)) return;
  if (!stage_in(c, 2, output, (size_t)batch_size * out_dim * out_dim * out_channel, false, &o)) return;
  if (!stage_in(c, 3, bias, sizeof(int32_t) * (size_t)out_channel, true, &b)) return;
  cudaError_t e;
  if (tc_supported_conv_i8(s, i.dev, w.dev))
    e = launch_conv_i8_tc(c, s, sc, act, static_cast<const int8_t*>(i.dev), static_cast<int8_t*>(o.dev),
                          static_cast<const int8_t*>(w.dev), static_cast<const int32_t*>(b.dev));
  else
    e = launch_conv_i8_simt(c->stream, s, sc, act, static_cast<const int8_t*>(i.dev),
                            static_cast<int8_t*>(o.dev), static_cast<const int8_t*>(w.dev),
                            static_cast<const int32_t*>(b.dev));
  if (!check_cuda(e, fn)) return;
  if (!stage_out(c, o)) return;
  finish(c, i.staged || w.staged || o.staged || b.staged);
}

}  // namespace

extern "C" {

void sgemm_exo(void* ctxt, int_fast32_t M, int_fast32_t N, int_fast32_t K, const float* A, const float* B,
               float* C) {
  sgemm_dispatch("sgemm_exo", ctxt, -1, M, N, K, A, B, C);
}
void sgemm_exo_ffma(void* ctxt, int_fast32_t M, int_fast32_t N, int_fast32_t K, const float* A, const float* B,
                    float* C) {
  sgemm_dispatch("sgemm_exo_ffma", ctxt, EXO_B200_SGEMM_FFMA, M, N, K, A, B, C);
}
void sgemm_exo_3xtf32(void* ctxt, int_fast32_t M, int_fast32_t N, int_fast32_t K, const float* A,
                      const float* B, float* C) {
  sgemm_dispatch("sgemm_exo_3xtf32", ctxt, EXO_B200_SGEMM_3XTF32, M, N, K, A, B, C, true);
}

void ssyrk_exo(void* ctxt, int_fast32_t N, int_fast32_t K, const float* A, float* C) {
  ssyrk_dispatch("ssyrk_exo", ctxt, EXO_B200_SGEMM_FFMA, N, K, A, C);
}
void ssyrk_exo_ffma(void* ctxt, int_fast32_t N, int_fast32_t K, const float* A, float* C) {
  ssyrk_dispatch("ssyrk_exo_ffma", ctxt, EXO_B200_SGEMM_FFMA, N, K, A, C);
}
void ssyrk_exo_3xtf32(void* ctxt, int_fast32_t N, int_fast32_t K, const float* A, float* C) {
  ssyrk_dispatch("ssyrk_exo_3xtf32", ctxt, EXO_B200_SGEMM_3XTF32, N, K, A, C);
}

void conv_specialized(void* ctxt, const float* inp, float* output, const float* weights, const float* bias) {
  // inp f32[5,82,102,128], output f32[5,80,100,128], weights f32[128,3,3,128], bias f32[128]
  clear_error();
  if (bad_args("conv_specialized", !bias, "NULL bias")) return;
  conv_dispatch("conv_specialized", ctxt, x86_conv_shape(80, 100, 128, 82, 102, 128, 3, 5), inp, output,
                weights, bias);
}

void conv(void* ctxt, int_fast32_t out_h, int_fast32_t out_w, int_fast32_t out_channel, int_fast32_t in_h,
          int_fast32_t in_w, int_fast32_t in_channel, int_fast32_t kernel_dim, int_fast32_t batch_size,
          const float* inp, float* output, const float* weights, const float* bias) {
  clear_error();
  // assert out_h == in_h - kernel_dim + 1, out_w == in_w - kernel_dim + 1 (apps/x86/conv/conv.py:26-27)
  if (bad_args("conv", out_h != in_h - kernel_dim + 1 || out_w != in_w - kernel_dim + 1,
               "out_h/out_w must equal in - kernel_dim + 1"))
    return;
  if (bad_args("conv", !bias, "NULL bias")) return;
  conv_dispatch("conv", ctxt,
                x86_conv_shape(out_h, out_w, out_channel, in_h, in_w, in_channel, kernel_dim, batch_size), inp,
                output, weights, bias);
}

static ConvShape nhwc_conv_shape(int_fast32_t batch_size, int_fast32_t in_h, int_fast32_t in_w,
                                 int_fast32_t in_channel, int_fast32_t out_channel, int_fast32_t kernel_dim,
                                 int_fast32_t pad, bool relu, int_fast32_t stride = 1) {
  ConvShape s;
  if (stride < 1) stride = 0;  // rejected below: out_h / out_w come out as 0
  s.batch = (int)batch_size;
  s.in_h = (int)in_h;
  s.in_w = (int)in_w;
  s.in_c = (int)in_channel;
  s.out_c = (int)out_channel;
  s.kdim = (int)kernel_dim;
  s.pad = (int)pad;
  s.stride = (int)stride;
  s.out_h = stride ? (int)((in_h + 2 * pad - kernel_dim) / stride + 1) : 0;
  s.out_w = stride ? (int)((in_w + 2 * pad - kernel_dim) / stride + 1) : 0;
  if (in_h + 2 * pad < kernel_dim || in_w + 2 * pad < kernel_dim) s.out_h = s.out_w = 0;
  s.w_stride_ci = out_channel;
  s.w_stride_kx = in_channel * out_channel;
  s.w_stride_ky = kernel_dim * in_channel * out_channel;
  s.relu = relu;
  return s;
}

void conv_nhwc_exo(void* ctxt, int_fast32_t batch_size, int_fast32_t in_h, int_fast32_t in_w,
                   int_fast32_t in_channel, int_fast32_t out_channel, int_fast32_t kernel_dim, int_fast32_t pad,
                   bool relu, const float* inp, float* output, const float* weights, const float* bias) {
  conv_dispatch("conv_nhwc_exo", ctxt,
                nhwc_conv_shape(batch_size, in_h, in_w, in_channel, out_channel, kernel_dim, pad, relu), inp, output,
                weights, bias);
}

void conv_nhwc_strided_exo(void* ctxt, int_fast32_t batch_size, int_fast32_t in_h, int_fast32_t in_w,
                           int_fast32_t in_channel, int_fast32_t out_channel, int_fast32_t kernel_dim, int_fast32_t pad,
                           int_fast32_t stride, bool relu, const float* inp, float* output, const float* weights,
                           const float* bias) {
  conv_dispatch("conv_nhwc_strided_exo", ctxt,
                nhwc_conv_shape(batch_size, in_h, in_w, in_channel, out_channel, kernel_dim, pad, relu, stride), inp,
                output, weights, bias, EXO_B200_SGEMM_FFMA);
}

void conv_nhwc_exo_3xtf32(void* ctxt, int_fast32_t batch_size, int_fast32_t in_h, int_fast32_t in_w,
                          int_fast32_t in_channel, int_fast32_t out_channel, int_fast32_t kernel_dim,
                          int_fast32_t pad, bool relu, const float* inp, float* output, const float* weights,
                          const float* bias) {
  conv_dispatch("conv_nhwc_exo_3xtf32", ctxt,
                nhwc_conv_shape(batch_size, in_h, in_w, in_channel, out_channel, kernel_dim, pad, relu), inp, output,
                weights, bias, EXO_B200_SGEMM_3XTF32);
}

void matmul_on_cpu(void* ctxt, int_fast32_t N, int_fast32_t M, int_fast32_t K, const float* scale, bool act,
                   const int8_t* A, const int8_t* B, int8_t* C) {
  (void)ctxt;
  matmul_i8_dispatch("matmul_on_cpu", N, M, K, scale, act, A, B, C);
}

#define EXOB200_MATMUL_INSTANCE(NAME, N_, M_, K_)                                                          \
  void cpu_matmul_##NAME(void* ctxt, const float* scale, bool act, const int8_t* A, const int8_t* B,       \
                         int8_t* C) {                                                                      \
    (void)ctxt;                                                                                            \
    matmul_i8_dispatch("cpu_matmul_" #NAME, N_, M_, K_, scale, act, A, B, C);                              \
  }                                                                                                        \
  void matmul_##NAME(void* ctxt, const float* scale, bool act, const int8_t* A, const int8_t* B, int8_t* C) { \
    (void)ctxt;                                                                                            \
    matmul_i8_dispatch("matmul_" #NAME, N_, M_, K_, scale, act, A, B, C);                                  \
  }
// shapes: apps/gemmini/src/exo/matmul.py:166-170,228-232,284-288,349-353,414-418,487-507
EXOB200_MATMUL_INSTANCE(512x512x512, 512, 512, 512)
EXOB200_MATMUL_INSTANCE(4, 12544, 256, 64)
EXOB200_MATMUL_INSTANCE(6, 12544, 64, 256)
EXOB200_MATMUL_INSTANCE(14, 3136, 512, 128)
EXOB200_MATMUL_INSTANCE(16, 3136, 128, 512)
EXOB200_MATMUL_INSTANCE(27, 784, 1024, 256)
#undef EXOB200_MATMUL_INSTANCE

void conv_on_cpu_stride_1(void* ctxt, int_fast32_t batch_size, int_fast32_t out_dim, int_fast32_t out_channel,
                          int_fast32_t kernel_dim, int_fast32_t in_channel, int_fast32_t in_dim, int8_t* output,
                          const int32_t* bias, const int8_t* inp, const int8_t* weights, bool act,
                          const float* scale) {
  (void)ctxt;
  conv_i8_dispatch("conv_on_cpu_stride_1", batch_size, out_dim, out_channel, kernel_dim, in_channel, in_dim,
                   output, bias, inp, weights, act, scale);
}

#define EXOB200_CONV_INSTANCE(NAME, B_, OD_, OC_, KD_, IC_, ID_)                                           \
  void conv_##NAME##_cpu(void* ctxt, int8_t* output, const int32_t* bias, const int8_t* inp,               \
                         const int8_t* weights, bool act, const float* scale) {                            \
    (void)ctxt;                                                                                            \
    conv_i8_dispatch("conv_" #NAME "_cpu", B_, OD_, OC_, KD_, IC_, ID_, output, bias, inp, weights, act,   \
                     scale);                                                                               \
  }                                                                                                        \
  void conv_##NAME(void* ctxt, int8_t* output, const int32_t* bias, const int8_t* inp,                     \
                   const int8_t* weights, bool act, const float* scale) {                                  \
    (void)ctxt;                                                                                            \
    conv_i8_dispatch("conv_" #NAME, B_, OD_, OC_, KD_, IC_, ID_, output, bias, inp, weights, act, scale);  \
  }
// shapes: apps/gemmini/src/exo/conv.py (conv_3 / conv_17 / conv_30 schedules)
EXOB200_CONV_INSTANCE(3, 4, 56, 64, 3, 64, 58)
EXOB200_CONV_INSTANCE(17, 4, 28, 128, 3, 128, 30)
EXOB200_CONV_INSTANCE(30, 4, 14, 256, 3, 256, 16)
#undef EXOB200_CONV_INSTANCE

// ---------------------------------------------------------------------------
// The Gemmini software library's two "auto" entry points, as the reference's shim
// overrides them (apps/gemmini/test/bare-metal/shims/gemmini.c): shape switch to the
// generated instances; other shapes run on the generic kernels when the call asks for
// nothing beyond what those compute, and are refused otherwise.
void tiled_matmul_auto(size_t dim_I, size_t dim_J, size_t dim_K, const elem_t* A, const elem_t* B, const void* D,
                       void* C, size_t stride_A, size_t stride_B, size_t stride_D, size_t stride_C,
                       scale_t A_scale_factor, scale_t B_scale_factor, scale_acc_t D_scale_factor, int act,
                       acc_scale_t scale, acc_scale_t bert_scale, bool repeating_bias, bool transpose_A,
                       bool transpose_B, bool full_C, bool low_D, uint8_t weightA,
                       exo_b200_tiled_matmul_type tiled_matmul_type) {
  (void)stride_D, (void)D_scale_factor, (void)bert_scale, (void)repeating_bias, (void)low_D, (void)weightA,
      (void)tiled_matmul_type;
  const float c_scale = (float)scale;
  const bool act_ = act != 0;
  int8_t* out = static_cast<int8_t*>(C);
  struct Instance {
    size_t i, j, k;
    const char* name;
  };
  // shapes: gemmini.c:20-51
  static const Instance instances[] = {{512, 512, 512, "tiled_matmul_auto -> matmul_512x512x512"},
                                       {12544, 256, 64, "tiled_matmul_auto -> matmul_4"},
                                       {12544, 64, 256, "tiled_matmul_auto -> matmul_6"},
                                       {3136, 512, 128, "tiled_matmul_auto -> matmul_14"},
                                       {3136, 128, 512, "tiled_matmul_auto -> matmul_16"},
                                       {784, 1024, 256, "tiled_matmul_auto -> matmul_27"}};
  for (const Instance& in : instances)
    if (dim_I == in.i && dim_J == in.j && dim_K == in.k) {
      // like the reference shim, an instance takes A, B, C as dense and ignores D and the strides
      matmul_i8_dispatch(in.name, (int_fast32_t)dim_I, (int_fast32_t)dim_J, (int_fast32_t)dim_K, &c_scale, act_, A, B,
                         out);
      return;
    }
  clear_error();
  const char* why = nullptr;
  if (D != nullptr) why = "a bias matrix D";
  else if (transpose_A || transpose_B) why = "transposed operands";
  else if (full_C) why = "full-width (int32) output";
  else if (stride_A != dim_K || stride_B != dim_J || stride_C != dim_J) why = "strided operands";
  else if (act != 0 && act != 1) why = "an activation other than none / ReLU";
  else if (A_scale_factor != 1.0f || B_scale_factor != 1.0f) why = "input scale factors other than 1";
  if (why) {
    set_error(EXO_B200_ERR_UNSUPPORTED, std::string("tiled_matmul_auto: no generated instance for ") +
                                            std::to_string(dim_I) + " x " + std::to_string(dim_J) + " x " +
                                            std::to_string(dim_K) + ", and the generic kernel does not take " + why);
    return;
  }
  matmul_i8_dispatch("tiled_matmul_auto -> matmul_on_cpu", (int_fast32_t)dim_I, (int_fast32_t)dim_J,
                     (int_fast32_t)dim_K, &c_scale, act_, A, B, out);
}

void tiled_conv_auto(int batch_size, int in_row_dim, int in_col_dim, int in_channels, int out_channels,
                     int out_row_dim, int out_col_dim, int stride, int input_dilation, int kernel_dilation,
                     int padding, int kernel_dim, bool wrot180, bool trans_output_1203, bool trans_input_3120,
                     bool trans_weight_1203, bool trans_weight_0132, const elem_t* input, const elem_t* weights,
                     const acc_t* bias, elem_t* output, int act, acc_scale_t scale, int pool_size, int pool_stride,
                     int pool_padding, exo_b200_tiled_matmul_type tiled_conv_type) {
  (void)pool_stride, (void)pool_padding, (void)tiled_conv_type;
  clear_error();
  // the restrictions the reference shim enforces by exiting (gemmini.c:73-90), reported instead
  const char* why = nullptr;
  if (input_dilation != 1 || kernel_dilation != 1) why = "dilation must be 1";
  else if (wrot180 || trans_output_1203 || trans_input_3120 || trans_weight_1203 || trans_weight_0132)
    why = "transposed / rotated tensors are not supported";
  else if (out_row_dim != out_col_dim || in_row_dim != in_col_dim) why = "images must be square";
  if (why) {
    set_error(EXO_B200_ERR_UNSUPPORTED, std::string("tiled_conv_auto: ") + why);
    return;
  }
  const float c_scale = (float)scale;
  const bool act_ = act != 0;
  // shape switch of gemmini.c:120-131 (it tests only these three fields; an instance then
  // takes its other sizes from its own definition, as there)
  if (stride == 1 && out_row_dim == 56 && out_channels == 64) {
    conv_i8_dispatch("tiled_conv_auto -> conv_3", 4, 56, 64, 3, 64, 58, output, bias, input, weights, act_, &c_scale);
    return;
  }
  if (stride == 1 && out_row_dim == 28 && out_channels == 128) {
    conv_i8_dispatch("tiled_conv_auto -> conv_17", 4, 28, 128, 3, 128, 30, output, bias, input, weights, act_,
                     &c_scale);
    return;
  }
  if (stride == 1 && out_row_dim == 14 && out_channels == 256) {
    conv_i8_dispatch("tiled_conv_auto -> conv_30", 4, 14, 256, 3, 256, 16, output, bias, input, weights, act_,
                     &c_scale);
    return;
  }
  if (stride != 1) why = "stride must be 1";
  else if (padding != 0) why = "padding must be 0 (pad the input, as the generated instances expect)";
  else if (pool_size > 1) why = "pooling is not supported";
  else if (out_row_dim != in_row_dim - kernel_dim + 1) why = "out_dim must equal in_dim - kernel_dim + 1";
  if (why) {
    set_error(EXO_B200_ERR_UNSUPPORTED, std::string("tiled_conv_auto: no generated instance for this shape, and ") + why);
    return;
  }
  conv_i8_dispatch("tiled_conv_auto -> conv_on_cpu_stride_1", batch_size, out_row_dim, out_channels, kernel_dim,
                   in_channels, in_row_dim, output, bias, input, weights, act_, &c_scale);
}

int exo_b200_sgemm_kernel_choice(int_fast32_t M, int_fast32_t N, int_fast32_t K) {
  if (M < 1 || N < 1 || K < 1 || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return -1;
  const int plan = sgemm_ffma_plan(M, N, K, K % 4 == 0, N % 4 == 0);
  if (plan <= EXO_B200_SGEMM_SKINNY) return plan;
  int rows = plan, cols = plan;  // square configurations are named by their edge
  switch (plan) {
    case 12864: rows = 128, cols = 64; break;
    case 6464: rows = cols = 64; break;
    case 3224: rows = cols = 32; break;
    case 1664: rows = 16, cols = 64; break;
    case 8128: rows = 8, cols = 128; break;
    default: break;
  }
  return EXO_B200_SGEMM_TILES + 1000 * rows + cols;
}

int exo_b200_selftest_bounded_wait(exo_b200_Context* ctxt, int limit_us) {
  clear_error();
  ContextUse use(resolve_context(ctxt));
  exo_b200_Context* c = use.get();
  if (!c) return exo_b200_last_error();
  if (limit_us < 1 || limit_us > 2000000) {
    set_error(EXO_B200_ERR_INVALID_ARGUMENT, "exo_b200_selftest_bounded_wait: limit_us must be in [1, 2000000]");
    return exo_b200_last_error();
  }
  if (check_cuda(launch_bounded_wait_selftest(c, (uint64_t)limit_us * 1000ull), "selftest launch"))
    exo_b200_synchronize(ctxt);  // reads the status word: expected to report the timeout
  return exo_b200_last_error();
}

void gemm_bf16_exo(void* ctxt, int_fast32_t M, int_fast32_t N, int_fast32_t K, const uint16_t* A,
                   const uint16_t* B, uint16_t* C) {
  const char* fn = "gemm_bf16_exo";
  clear_error();
  if (bad_args(fn, M < 1 || N < 1 || K < 1, "M, N, K must be >= 1")) return;
  if (bad_args(fn, !A || !B || !C, "NULL tensor")) return;
  ContextUse use(resolve_context(ctxt));
  exo_b200_Context* c = use.get();
  if (!c) return;
  Operand a, b, cc;
  // (K % 8 != 0 goes through a padded copy of the operands in the launcher, which wants them whole:
  // such calls skip the chunked pipelines)
  if (K % 8 == 0 && want_block_pipeline(M, N, (size_t)K * 2, A, B, C)) {
    // everything on the host and B large too: upload both operands piecewise and let
    // output blocks leave as soon as their row chunk and column block are on the device
    static const int64_t br = getenv("EXOB200_BLOCK_ROWS") ? atoll(getenv("EXOB200_BLOCK_ROWS")) : 2048;
    // 2048 x 4096 blocks measured best on the 32768 x 16384 x 8192 problem (25.0 ms against 26.1 ms for the row
    // pipeline); 2048-wide blocks lose to it (28.0 ms): their 4 KB rows make the strided copy-out slow
    static const int64_t bc = getenv("EXOB200_BLOCK_COLS") ? atoll(getenv("EXOB200_BLOCK_COLS")) : 4096;
    BlockPipeline p{M, N, br, bc, A, (size_t)K * 2, B, (size_t)K * 2, C, 2};
    if (!run_block_pipeline(c, p, [&](int64_t rows, int64_t cols, const void* dA, const void* dB, void* dC) {
          return launch_gemm_bf16_tc(c, rows, cols, K, static_cast<const uint16_t*>(dA),
                                     static_cast<const uint16_t*>(dB), static_cast<uint16_t*>(dC));
        }))
      return;
    finish(c, true);
    return;
  }
  if (K % 8 == 0 && want_row_pipeline(M, A, C, (size_t)K * 2 + (size_t)N * 2) &&
      (!is_device_pointer(B) || (reinterpret_cast<uintptr_t>(B) & 15u) == 0)) {
    // host A and C: rows are independent, so stream them through in chunks
    if (!stage_in(c, 1, B, sizeof(uint16_t) * (size_t)K * N, true, &b)) return;
    RowPipeline p{M, pipeline_chunk_rows(M, (size_t)K * 2 + (size_t)N * 2), A, (size_t)K * 2, C, (size_t)N * 2, false};
    const uint16_t* dB = static_cast<const uint16_t*>(b.dev);
    if (!run_row_pipeline(c, p, [&](int64_t rows, const void* dA, void* dC) {
          return launch_gemm_bf16_tc(c, rows, N, K, static_cast<const uint16_t*>(dA), dB, static_cast<uint16_t*>(dC));
        }))
      return;
    finish(c, true);
    return;
  }
  if (!stage_in(c, 0, A, sizeof(uint16_t) * (size_t)M * K, true, &a)) return;
  if (!stage_in(c, 1, B, sizeof(uint16_t) * (size_t)K * N, true, &b)) return;
  if (!stage_in(c, 2, C, sizeof(uint16_t) * (size_t)M * N, false, &cc)) return;
  cudaError_t e = launch_gemm_bf16_tc(c, M, N, K, static_cast<const uint16_t*>(a.dev),
                                      static_cast<const uint16_t*>(b.dev), static_cast<uint16_t*>(cc.dev));
  if (!check_cuda(e, fn)) return;
  if (!stage_out(c, cc)) return;
  finish(c, a.staged || b.staged || cc.staged);
}

}  // extern "C"
