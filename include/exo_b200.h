/*
 * exo_b200 -- B200 (sm_100a) GEMM / convolution kernels behind the C ABI that
 * Exo's compiler `exocc` writes into its generated headers.
 *
 * Every "reference-identical" prototype below is the one exocc emits for the
 * corresponding Exo procedure (sgemm_exo and conv_specialized character for
 * character; the Gemmini-typed ones up to the type of the context pointer, see
 * EXO_B200_GEMMINI_CONTEXT), so this library links wherever the generated C was
 * linked (the `add_exo_library` CMake target, src/exo/cmake/AddExoLibrary.cmake:29-31).  ABI rules, from
 * src/exo/backend/LoopIR_compiler.py:524-619 and src/exo/core/LoopIR.py:436-466:
 *   - first parameter `ctxt`; sizes are int_fast32_t by value; bool by value;
 *   - numeric scalars (e.g. `scale : f32`) are passed BY POINTER;
 *   - tensors are raw pointers to dense row-major data; the callee allocates
 *     nothing the caller has to free; arguments must not alias;
 *   - return type is void: there is no error channel in the reference.  This
 *     library adds one that existing callers may ignore: exo_b200_last_error().
 *
 * Pointers may be host memory (as in the reference; data is staged to the GPU
 * and back inside the call, which returns when the result is in place) or
 * CUDA device memory (used in place; the kernel is enqueued on the context's
 * stream and the call returns without synchronising).  All work is done on the
 * GPU; there is no CPU code path.
 *
 * `ctxt`: the `void *ctxt` functions accept NULL (process default context) or
 * an exo_b200_Context* made by exo_b200_context_create().  The Gemmini-typed
 * functions receive an UNINITIALISED pointer from their reference callers
 * (apps/gemmini/test/run_matmul.c:49-52), so they never look at ctxt.
 *
 * Thread safety: every entry point holds its context's mutex for the length of
 * the call, so host threads may call into one context -- the default one
 * included -- at the same time; they take turns.  (The reference's sgemm_exo is
 * not reentrant at all: it keeps tiles in function statics,
 * tests/golden/test_apps/test_x86_sgemm.txt:797,804.)  A call with device
 * pointers only enqueues kernels; kernels enqueued through ONE context on
 * DIFFERENT streams may overlap on the GPU and share that context's scratch,
 * so give each stream its own context.
 */
#pragma once
#ifndef EXO_B200_H
#define EXO_B200_H

#ifdef __cplusplus
extern "C" {
#endif

#include <stdbool.h>
#include <stdint.h>

#if defined(__GNUC__)
#pragma GCC visibility push(default) /* the library itself is built with hidden visibility */
#endif

/* ------------------------------------------------------------------------
 * Reference-identical entry points
 * --------------------------------------------------------------------- */

/* sgemm_exo(M, N, K : size, A : f32[M,K], B : f32[K,N], C : f32[M,N]):  C += A * B
 * Replaces tests/golden/test_apps/test_x86_sgemm.txt:69 (apps/x86/sgemm/sgemm.py:11-23,194).
 * Default arithmetic: exact fp32 FFMA, one fused-multiply-add chain per output
 * in increasing k starting from the incoming C -- bit-identical to the
 * generated AVX-512 code.  EXOB200_SGEMM_PATH=3xtf32 (or the context setting)
 * selects the tensor-core path instead. */
void sgemm_exo( void *ctxt, int_fast32_t M, int_fast32_t N, int_fast32_t K, const float* A, const float* B, float* C );

/* conv_specialized(inp : f32[5,82,102,128], output : f32[5,80,100,128],
 *                  weights : f32[128,3,3,128], bias : f32[128])
 * Replaces tests/golden/test_apps/test_x86_conv.txt:53 (apps/x86/conv/conv.py:53-119). */
void conv_specialized( void *ctxt, const float* inp, float* output, const float* weights, const float* bias );

/* conv: the unspecialised procedure of apps/x86/conv/conv.py:10-45 (argument
 * order :11-24; call shape at apps/x86/conv/exo_conv.cpp:12-14).  NHWC input,
 * weights f32[in_channel, kernel_dim, kernel_dim, out_channel], stride 1, no
 * padding, bias, ReLU.  Requires out_h == in_h - kernel_dim + 1 (same for w). */
void conv( void *ctxt, int_fast32_t out_h, int_fast32_t out_w, int_fast32_t out_channel, int_fast32_t in_h, int_fast32_t in_w, int_fast32_t in_channel, int_fast32_t kernel_dim, int_fast32_t batch_size, const float* inp, float* output, const float* weights, const float* bias );

/* Gemmini-style int8 matmul (apps/gemmini/src/exo/matmul.py:7-43):
 *   acc = sum_k (i32)A[i,k] * (i32)B[k,j];  t = round_half_even((f32)acc * *scale);
 *   q = (int8)clamp(t, -128, 127);  if (act) q = max(q, 0);  C[i,j] = q
 * A : i8[N,K], B : i8[K,M], C : i8[N,M] (Exo names the rows N and the columns M).
 * Generic sizes; prototype shape confirmed by
 * tests/golden/asplos25/test_gemmini_matmul_old/test_matmul.txt:92. */
void matmul_on_cpu( void *ctxt, int_fast32_t N, int_fast32_t M, int_fast32_t K, const float* scale, bool act, const int8_t* A, const int8_t* B, int8_t* C );

/* Type of the context pointer in the Gemmini-typed prototypes.  exocc names it after
 * the library stem (`gemmini_lib_Context` in the app build, apps/gemmini/src/CMakeLists.txt:10-13;
 * `test_case_Context` in tests/golden/test_apps/test_gemmini_matmul.txt:32-56).  The pointer is
 * never dereferenced here, so the default is void; a translation unit that also includes the
 * generated header defines EXO_B200_GEMMINI_CONTEXT to that header's type first
 * (-DEXO_B200_GEMMINI_CONTEXT=gemmini_lib_Context) and the declarations below then repeat the
 * generated ones token for token instead of conflicting with them. */
#ifndef EXO_B200_GEMMINI_CONTEXT
#define EXO_B200_GEMMINI_CONTEXT void
#endif

/* The size-specialised instances the Gemmini app exports
 * (tests/golden/test_apps/test_gemmini_matmul.txt:99-198): `cpu_matmul_*` is the
 * plain-C twin, `matmul_*` the accelerator version; both compute the same
 * result (apps/gemmini/test/run_matmul.c:63 asserts equality) and both map to
 * the same GPU kernel here.  ctxt is never dereferenced. */
void cpu_matmul_512x512x512( EXO_B200_GEMMINI_CONTEXT *ctxt, const float* scale, bool act, const int8_t* A, const int8_t* B, int8_t* C );
void matmul_512x512x512( EXO_B200_GEMMINI_CONTEXT *ctxt, const float* scale, bool act, const int8_t* A, const int8_t* B, int8_t* C );
void cpu_matmul_4( EXO_B200_GEMMINI_CONTEXT *ctxt, const float* scale, bool act, const int8_t* A, const int8_t* B, int8_t* C );   /* 12544 x 256, K = 64 */
void matmul_4( EXO_B200_GEMMINI_CONTEXT *ctxt, const float* scale, bool act, const int8_t* A, const int8_t* B, int8_t* C );
void cpu_matmul_6( EXO_B200_GEMMINI_CONTEXT *ctxt, const float* scale, bool act, const int8_t* A, const int8_t* B, int8_t* C );   /* 12544 x 64, K = 256 */
void matmul_6( EXO_B200_GEMMINI_CONTEXT *ctxt, const float* scale, bool act, const int8_t* A, const int8_t* B, int8_t* C );
void cpu_matmul_14( EXO_B200_GEMMINI_CONTEXT *ctxt, const float* scale, bool act, const int8_t* A, const int8_t* B, int8_t* C );  /* 3136 x 512, K = 128 */
void matmul_14( EXO_B200_GEMMINI_CONTEXT *ctxt, const float* scale, bool act, const int8_t* A, const int8_t* B, int8_t* C );
void cpu_matmul_16( EXO_B200_GEMMINI_CONTEXT *ctxt, const float* scale, bool act, const int8_t* A, const int8_t* B, int8_t* C );  /* 3136 x 128, K = 512 */
void matmul_16( EXO_B200_GEMMINI_CONTEXT *ctxt, const float* scale, bool act, const int8_t* A, const int8_t* B, int8_t* C );
void cpu_matmul_27( EXO_B200_GEMMINI_CONTEXT *ctxt, const float* scale, bool act, const int8_t* A, const int8_t* B, int8_t* C );  /* 784 x 1024, K = 256 */
void matmul_27( EXO_B200_GEMMINI_CONTEXT *ctxt, const float* scale, bool act, const int8_t* A, const int8_t* B, int8_t* C );

/* Gemmini-style int8 NHWC convolution (apps/gemmini/src/exo/conv.py:6-55):
 * weights i8[kernel_dim,kernel_dim,in_channel,out_channel], bias i32[1,out_channel]
 * is the accumulator's start value, stride 1, caller-padded input
 * (out_dim == in_dim - kernel_dim + 1), same epilogue as the matmul. */
void conv_on_cpu_stride_1( void *ctxt, int_fast32_t batch_size, int_fast32_t out_dim, int_fast32_t out_channel, int_fast32_t kernel_dim, int_fast32_t in_channel, int_fast32_t in_dim, int8_t* output, const int32_t* bias, const int8_t* inp, const int8_t* weights, bool act, const float* scale );

/* Size-specialised instances, tests/golden/test_apps/test_gemmini_conv.txt:96-146:
 * conv_3: batch 4, 58->56, 64->64, 3x3;  conv_17: batch 4, 30->28, 128->128;
 * conv_30: batch 4, 16->14, 256->256. */
void conv_3_cpu( EXO_B200_GEMMINI_CONTEXT *ctxt, int8_t* output, const int32_t* bias, const int8_t* inp, const int8_t* weights, bool act, const float* scale );
void conv_3( EXO_B200_GEMMINI_CONTEXT *ctxt, int8_t* output, const int32_t* bias, const int8_t* inp, const int8_t* weights, bool act, const float* scale );
void conv_17_cpu( EXO_B200_GEMMINI_CONTEXT *ctxt, int8_t* output, const int32_t* bias, const int8_t* inp, const int8_t* weights, bool act, const float* scale );
void conv_17( EXO_B200_GEMMINI_CONTEXT *ctxt, int8_t* output, const int32_t* bias, const int8_t* inp, const int8_t* weights, bool act, const float* scale );
void conv_30_cpu( EXO_B200_GEMMINI_CONTEXT *ctxt, int8_t* output, const int32_t* bias, const int8_t* inp, const int8_t* weights, bool act, const float* scale );
void conv_30( EXO_B200_GEMMINI_CONTEXT *ctxt, int8_t* output, const int32_t* bias, const int8_t* inp, const int8_t* weights, bool act, const float* scale );

/* ------------------------------------------------------------------------
 * Entry points with no generated counterpart, same conventions
 * --------------------------------------------------------------------- */

/* sgemm_exo with the arithmetic path fixed by name (same contract as
 * tests/golden/test_apps/test_x86_sgemm.txt:69).  _ffma: exact fp32 chain.
 * _3xtf32: tcgen05 tensor cores, each fp32 operand split into two TF32 terms,
 * three MMAs per product, fp32 accumulation in tensor memory; not bit-identical,
 * error comparable to fp32 accumulation in a different order. */
void sgemm_exo_ffma( void *ctxt, int_fast32_t M, int_fast32_t N, int_fast32_t K, const float* A, const float* B, float* C );
void sgemm_exo_3xtf32( void *ctxt, int_fast32_t M, int_fast32_t N, int_fast32_t K, const float* A, const float* B, float* C );

/* gemm_bf16_exo(M, N, K, A : ui16[M,K] row-major, B : ui16 column-major KxN
 * (element (k,j) at B[j*K + k]), C : ui16[M,N] row-major):  C = A * B.
 * Exo has no bf16 type (src/exo/core/LoopIR.py:446-462 maps ui16 -> uint16_t), so
 * bf16 bit patterns travel as uint16_t.  fp32 accumulation, one round-to-
 * nearest-even to bf16 on output. */
void gemm_bf16_exo( void *ctxt, int_fast32_t M, int_fast32_t N, int_fast32_t K, const uint16_t* A, const uint16_t* B, uint16_t* C );

/* conv_nhwc_exo: apps/x86/conv/conv.py:10-45 generalised the way the
 * convolution workload needs it: weights f32[kernel_dim,kernel_dim,in_channel,out_channel]
 * (the layout of apps/gemmini/src/exo/conv.py:17), symmetric zero padding `pad`,
 * stride 1, bias (may be NULL = zeros), optional ReLU.  Output is
 * f32[batch, in_h + 2 pad - kernel_dim + 1, in_w + 2 pad - kernel_dim + 1, out_channel].
 * Exact fp32: bias-initialised FMA chain in ky -> kx -> ci order. */
void conv_nhwc_exo( void *ctxt, int_fast32_t batch_size, int_fast32_t in_h, int_fast32_t in_w, int_fast32_t in_channel, int_fast32_t out_channel, int_fast32_t kernel_dim, int_fast32_t pad, bool relu, const float* inp, float* output, const float* weights, const float* bias );

/* conv_nhwc_exo with a spatial stride >= 1: output f32[batch, (in_h + 2 pad - kernel_dim) / stride + 1,
 * (in_w + 2 pad - kernel_dim) / stride + 1, out_channel] -- the output size of the reference's
 * convolution harness (apps/x86/conv/conv_instance.hpp:44-45), whose layer list has two stride-2 layers
 * (apps/x86/conv/bench_conv.cpp:47-49) that the Exo procedure does not cover ("todo: add padding,
 * stride", apps/x86/conv/conv.py:37).  Always the exact fp32 FFMA path. */
void conv_nhwc_strided_exo( void *ctxt, int_fast32_t batch_size, int_fast32_t in_h, int_fast32_t in_w, int_fast32_t in_channel, int_fast32_t out_channel, int_fast32_t kernel_dim, int_fast32_t pad, int_fast32_t stride, bool relu, const float* inp, float* output, const float* weights, const float* bias );

/* Same contract as conv_nhwc_exo on the tensor cores: implicit GEMM whose im2col
 * addressing is done by TMA (the decomposition of tests/test_im2col.py:41-62),
 * operands split into TF32 hi + lo terms, bias and ReLU in the epilogue.  Not
 * bit-identical; error like sgemm_exo_3xtf32.  conv / conv_specialized /
 * conv_nhwc_exo take this path too when the context's SGEMM path is 3xTF32. */
void conv_nhwc_exo_3xtf32( void *ctxt, int_fast32_t batch_size, int_fast32_t in_h, int_fast32_t in_w, int_fast32_t in_channel, int_fast32_t out_channel, int_fast32_t kernel_dim, int_fast32_t pad, bool relu, const float* inp, float* output, const float* weights, const float* bias );

/* matmul_on_cpu_static: the int8 matmul of matmul_on_cpu for callers that cannot
 * allocate device memory where they need the result -- under an arena that has
 * taken all device memory for itself, in a process that must stay inside a fixed
 * memory budget, or in a loop that must not meet an allocation's implicit
 * synchronisation.  It has no counterpart in the reference
 * (whose C code never allocates on a device); same arithmetic and same result
 * as matmul_on_cpu.
 *   - The first parameter is the cudaStream_t to launch on (NULL = default
 *     stream), not a context: contexts own allocations.
 *   - A, B, C must be device memory of the CURRENT device (the scratch array and
 *     the launch are the current device's; operands of another device are
 *     rejected); scale is host memory, read during the call.
 *   - Scratch for the K-major copy of B is a fixed array in the library image,
 *     EXO_B200_STATIC_SCRATCH_BYTES per GPU for the life of the process;
 *     K * M beyond it is rejected (EXO_B200_ERR_UNSUPPORTED, output untouched).
 *   - The first call on each device looks up the array's device address and
 *     loads the kernels: make that call before any stream capture begins.
 *   - All calls share the array: calls whose kernels may overlap on the GPU
 *     race; order them on one stream or with events.
 *   - The call only enqueues.  If a bounded device-side wait of its kernel ever
 *     runs out, the kernel ends with C partly written and records that in a
 *     status word that also lives in the library image; the call itself cannot
 *     report it.  exo_b200_synchronize() picks it up (EXO_B200_ERR_TIMEOUT), so
 *     call that after synchronising your stream where you need to know.
 *   - Calls no cudaMalloc / cudaFree / cudaHostAlloc and creates no context. */
#define EXO_B200_STATIC_SCRATCH_BYTES (4u << 20)
void matmul_on_cpu_static( void *stream, int_fast32_t N, int_fast32_t M, int_fast32_t K, const float* scale, bool act, const int8_t* A, const int8_t* B, int8_t* C );

/* SSYRK: C += A * A^T on the upper triangle (j >= i), A : f32[N,K], C : f32[N,N] row-major; the
 * strict lower triangle of C is not modified.  The computation that the reference's
 * MKL comparison benchmark measures (apps/x86/ssyrk/bench_ssyrk.cpp:11-13,49-65: cblas_ssyrk,
 * CblasRowMajor, CblasUpper, CblasNoTrans, alpha = beta = 1); there is no Exo procedure for it in
 * the reference, so the name and signature follow sgemm_exo's conventions.  Arithmetic as in
 * sgemm_exo: per element one fused-multiply-add chain in increasing k from the incoming C value
 * (_ffma, which ssyrk_exo always takes: bit-identical to sgemm_exo(N, N, K, A, A^T, C) on the
 * triangle), or 3xTF32 tensor cores (_3xtf32; error bound of sgemm_exo_3xtf32). */
void ssyrk_exo( void *ctxt, int_fast32_t N, int_fast32_t K, const float* A, float* C );
void ssyrk_exo_ffma( void *ctxt, int_fast32_t N, int_fast32_t K, const float* A, float* C );
void ssyrk_exo_3xtf32( void *ctxt, int_fast32_t N, int_fast32_t K, const float* A, float* C );

/* ------------------------------------------------------------------------
 * Context and error side channel (additions; the reference has neither)
 * --------------------------------------------------------------------- */

typedef struct exo_b200_Context exo_b200_Context;

enum {
  EXO_B200_OK = 0,
  EXO_B200_ERR_INVALID_ARGUMENT = 1, /* size < 1, NULL tensor, broken size relation */
  EXO_B200_ERR_CUDA = 2,             /* a CUDA runtime / driver call failed */
  EXO_B200_ERR_TIMEOUT = 3,          /* a bounded device-side wait ran out */
  EXO_B200_ERR_UNSUPPORTED = 4       /* no sm_100 device / shape not supported by this path */
};

enum { EXO_B200_SGEMM_FFMA = 0, EXO_B200_SGEMM_3XTF32 = 1 };

/* device < 0: the current CUDA device.  stream: a cudaStream_t (NULL = the
 * legacy default stream).  Returns NULL on failure (see last_error). */
exo_b200_Context* exo_b200_context_create( int device, void* stream );
void exo_b200_context_destroy( exo_b200_Context* ctxt );
void exo_b200_context_set_stream( exo_b200_Context* ctxt, void* stream );
void exo_b200_context_set_sgemm_path( exo_b200_Context* ctxt, int path );
/* Weight cache of the tensor-core fp32 convolution (conv_nhwc_exo_3xtf32, and conv / conv_specialized /
 * conv_nhwc_exo on a 3xTF32 context).  That path multiplies TF32 hi + lo copies of both operands; the
 * copy of the weights is the same from call to call while the weights are.  With the cache on
 * (enable != 0; it is OFF by default) the context keeps the copy of the last weight tensor and reuses it
 * when a call passes the same pointer, shape and layout -- so the caller promises not to rewrite that
 * memory in place, or calls exo_b200_context_invalidate() after doing so.  ctxt == NULL: the default
 * context of the current device. */
void exo_b200_context_cache_weights( exo_b200_Context* ctxt, int enable );
void exo_b200_context_invalidate( exo_b200_Context* ctxt );
/* Stream used by calls that pass ctxt == NULL (and by the Gemmini-typed calls). */
void exo_b200_set_default_stream( void* stream );
/* Wait for the context's stream (NULL: default context) and collect device-side status. */
int exo_b200_synchronize( exo_b200_Context* ctxt );

/* Diagnostic: launches one CTA that waits, with a limit of limit_us microseconds, on
 * a barrier that nothing signals, then synchronises.  The expected result is
 * EXO_B200_ERR_TIMEOUT (also left in last_error) with the context still usable:
 * it shows that a wait that cannot complete ends as an error code, not a hang. */
int exo_b200_selftest_bounded_wait( exo_b200_Context* ctxt, int limit_us );

/* Measures a ceiling of the GPU that the default context is on, for roofline fractions: a probe
 * kernel that issues nothing but the instruction in question (packed fp32 FMA from registers;
 * tcgen05.mma with operands resident in shared memory) runs for about `milliseconds` (1..500) and
 * the achieved rate is returned in TFLOP/s (int8: Tera-ops/s), or a negative value on failure
 * (see last_error).  Allocates a few bytes and synchronises the default stream. */
enum { EXO_B200_PEAK_FP32_SIMT = 0, EXO_B200_PEAK_INT8_TENSOR = 1, EXO_B200_PEAK_BF16_TENSOR = 2,
       EXO_B200_PEAK_TF32_TENSOR = 3 };
double exo_b200_measure_peak( int what, int milliseconds );

/* Which kernel sgemm_exo_ffma takes for a problem whose operands are 16-byte aligned (no counterpart in the
 * reference; needs no GPU): EXO_B200_SGEMM_TALL / _GEMV_TMA / _GEMV / _SKINNY for the kernels that serve few
 * columns or few rows, otherwise the tile engine's configuration as 1000 * tile_rows + tile_cols plus
 * EXO_B200_SGEMM_TILES (e.g. 128064 + EXO_B200_SGEMM_TILES for 128 x 64 tiles); two 64 x 64 and two 32 x 32
 * configurations differ in threads per tile and report the same value.  -1 for sizes below 1. */
enum { EXO_B200_SGEMM_TALL = 1, EXO_B200_SGEMM_GEMV_TMA = 2, EXO_B200_SGEMM_GEMV = 3, EXO_B200_SGEMM_SKINNY = 4,
       EXO_B200_SGEMM_TILES = 1000000 };
int exo_b200_sgemm_kernel_choice( int_fast32_t M, int_fast32_t N, int_fast32_t K );

/* Error of the most recent call on this thread (EXO_B200_OK if it succeeded). */
int exo_b200_last_error( void );
const char* exo_b200_last_error_string( void );
const char* exo_b200_version( void );

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
}
#endif
#endif /* EXO_B200_H */
