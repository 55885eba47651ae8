/*
 * exo_b200_gemmini_shim.h -- the two entry points through which applications
 * written against the upstream Gemmini software library reach the Exo kernels.
 *
 * The reference builds a shim (apps/gemmini/test/bare-metal/shims/gemmini.c:5-58 and
 * :60-141, declared in shims/include/gemmini.h.in:16-35) that overrides the upstream
 * library's `tiled_matmul_auto` / `tiled_conv_auto`: it switches on the problem shape,
 * calls the matching Exo-generated instance (matmul_4/6/14/16/27/512x512x512, conv_3/17/30)
 * and hands every other shape back to the upstream implementation.  libexo_b200.so exports
 * the same two symbols with the same parameter lists.  They dispatch the same way; a shape
 * that has no generated instance does not fall through to third-party code but runs on
 * this library's generic kernels (matmul_on_cpu / conv_on_cpu_stride_1), provided the call
 * uses only what those compute:
 *   matmul:  C = clamp(round_half_even(scale * (A * B))) (+ ReLU if act == 1); no bias D,
 *            no transposes, dense operands (stride_A == dim_K, stride_B == stride_C == dim_J),
 *            int8 output (full_C false)
 *   conv:    stride 1, no dilation, no transposes, no pooling, padding 0 (the caller pads,
 *            as the Exo instances expect: out_dim == in_dim - kernel_dim + 1), square images
 * Anything else is refused: EXO_B200_ERR_UNSUPPORTED in exo_b200_last_error(), outputs
 * untouched.  (The reference prints a line and aborts on the conv restrictions,
 * gemmini.c:73-90.)  As in the reference shim, the instances ignore D and the strides.
 *
 * The scalar types come from the upstream header when a caller has it.  Define
 * EXO_B200_HAVE_GEMMINI_H after including it; otherwise the typedefs below are used,
 * with the widths this library's kernels compute in (int8 elements, int32 accumulators,
 * float scales).  The enum parameter travels as an int either way.
 */
#pragma once
#ifndef EXO_B200_GEMMINI_SHIM_H
#define EXO_B200_GEMMINI_SHIM_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef EXO_B200_HAVE_GEMMINI_H
typedef int8_t elem_t;
typedef int32_t acc_t;
typedef float scale_t;
typedef float scale_acc_t;
typedef float acc_scale_t;
typedef int exo_b200_tiled_matmul_type; /* stands in for `enum tiled_matmul_type_t` */
#else
typedef enum tiled_matmul_type_t exo_b200_tiled_matmul_type;
#endif

#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

/* Replaces tiled_matmul_auto of apps/gemmini/test/bare-metal/shims/gemmini.c:5-58.
 * A : dim_I x dim_K, B : dim_K x dim_J, C : dim_I x dim_J, all int8 row-major. */
void tiled_matmul_auto( size_t dim_I, size_t dim_J, size_t dim_K,
    const elem_t* A, const elem_t* B, const void* D, void* C, size_t stride_A,
    size_t stride_B, size_t stride_D, size_t stride_C, scale_t A_scale_factor,
    scale_t B_scale_factor, scale_acc_t D_scale_factor, int act,
    acc_scale_t scale, acc_scale_t bert_scale, bool repeating_bias,
    bool transpose_A, bool transpose_B, bool full_C, bool low_D,
    uint8_t weightA, exo_b200_tiled_matmul_type tiled_matmul_type );

/* Replaces tiled_conv_auto of apps/gemmini/test/bare-metal/shims/gemmini.c:60-141.
 * input : int8 NHWC, weights : int8 [kernel_dim, kernel_dim, in_channels, out_channels],
 * bias : int32 [out_channels], output : int8 NHWC. */
void tiled_conv_auto( int batch_size, int in_row_dim, int in_col_dim,
    int in_channels, int out_channels, int out_row_dim, int out_col_dim, int stride,
    int input_dilation, int kernel_dilation, int padding, int kernel_dim,
    bool wrot180, bool trans_output_1203, bool trans_input_3120,
    bool trans_weight_1203, bool trans_weight_0132,
    const elem_t* input, const elem_t* weights, const acc_t* bias,
    elem_t* output,
    int act, acc_scale_t scale,
    int pool_size, int pool_stride, int pool_padding,
    exo_b200_tiled_matmul_type tiled_conv_type );

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif

#ifdef __cplusplus
}
#endif
#endif /* EXO_B200_GEMMINI_SHIM_H */
