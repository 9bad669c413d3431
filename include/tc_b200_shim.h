/*
 * tc_b200_shim.h -- the reference's generated entry point, served by libtc_b200.so.
 *
 * COGENT emits, per expression, a .cu file whose only entry is
 *     extern "C" void sd_t_d2_fusion_(int size_<idx>..., T* t3, T* t2, T* v2,
 *                                     int cond_kernel_1, int opt_register_transpose)
 * (cogent/src/codes/kernels/tc_interface.py:1444-1598) and the drivers call it through an implicit
 * declaration (cogent/drivers/tccg/code_main_tccg_02.c:71).  One translation unit that contains
 *
 *     #include "tc_b200_shim.h"
 *     TC_DEFINE_SD_T_D2_FUSION_4("t3 [a,16,b,16,c,16] += sum(d,16) * t2 [d,c,a] * v2 [b,d];", double, TC_F64)
 *
 * linked with -ltc_b200 in place of the generated object gives an unmodified driver the same symbol.
 * The digit is the number of size arguments (output indices in written order, then contraction
 * indices); the last two ints of the reference signature are accepted and ignored, as its
 * single-contraction code ignores them.  Failures are reported on stderr (the reference entry is void).
 */
#ifndef TC_B200_SHIM_H_
#define TC_B200_SHIM_H_

#include <stdio.h>

#include "tc_b200.h"

#ifdef __cplusplus
#define TC_SHIM_EXTERN extern "C"
#else
#define TC_SHIM_EXTERN
#endif

#define TC_SHIM_BODY_(EXPR, DTYPE, N, ...)                                                         \
  {                                                                                                \
    const int tc_sizes_[] = {__VA_ARGS__};                                                         \
    const int tc_st_ = tc_sd_t_d2_fusion(EXPR, DTYPE, N, tc_sizes_, t3, t2, v2);                   \
    (void)cond_kernel_1;                                                                           \
    (void)opt_register_transpose;                                                                  \
    if (tc_st_ != TC_OK)                                                                           \
      fprintf(stderr, "sd_t_d2_fusion_: %s %s\n", tc_status_string(tc_st_), tc_last_cuda_error()); \
  }

#define TC_DEFINE_SD_T_D2_FUSION_2(EXPR, T, DTYPE) \
  TC_SHIM_EXTERN void sd_t_d2_fusion_(int s0, int s1, T* t3, T* t2, T* v2, int cond_kernel_1, int opt_register_transpose) TC_SHIM_BODY_(EXPR, DTYPE, 2, s0, s1)
#define TC_DEFINE_SD_T_D2_FUSION_3(EXPR, T, DTYPE) \
  TC_SHIM_EXTERN void sd_t_d2_fusion_(int s0, int s1, int s2, T* t3, T* t2, T* v2, int cond_kernel_1, int opt_register_transpose) TC_SHIM_BODY_(EXPR, DTYPE, 3, s0, s1, s2)
#define TC_DEFINE_SD_T_D2_FUSION_4(EXPR, T, DTYPE) \
  TC_SHIM_EXTERN void sd_t_d2_fusion_(int s0, int s1, int s2, int s3, T* t3, T* t2, T* v2, int cond_kernel_1, int opt_register_transpose) TC_SHIM_BODY_(EXPR, DTYPE, 4, s0, s1, s2, s3)
#define TC_DEFINE_SD_T_D2_FUSION_5(EXPR, T, DTYPE) \
  TC_SHIM_EXTERN void sd_t_d2_fusion_(int s0, int s1, int s2, int s3, int s4, T* t3, T* t2, T* v2, int cond_kernel_1, int opt_register_transpose) TC_SHIM_BODY_(EXPR, DTYPE, 5, s0, s1, s2, s3, s4)
#define TC_DEFINE_SD_T_D2_FUSION_6(EXPR, T, DTYPE) \
  TC_SHIM_EXTERN void sd_t_d2_fusion_(int s0, int s1, int s2, int s3, int s4, int s5, T* t3, T* t2, T* v2, int cond_kernel_1, int opt_register_transpose) TC_SHIM_BODY_(EXPR, DTYPE, 6, s0, s1, s2, s3, s4, s5)
#define TC_DEFINE_SD_T_D2_FUSION_7(EXPR, T, DTYPE) \
  TC_SHIM_EXTERN void sd_t_d2_fusion_(int s0, int s1, int s2, int s3, int s4, int s5, int s6, T* t3, T* t2, T* v2, int cond_kernel_1, int opt_register_transpose) TC_SHIM_BODY_(EXPR, DTYPE, 7, s0, s1, s2, s3, s4, s5, s6)
#define TC_DEFINE_SD_T_D2_FUSION_8(EXPR, T, DTYPE) \
  TC_SHIM_EXTERN void sd_t_d2_fusion_(int s0, int s1, int s2, int s3, int s4, int s5, int s6, int s7, T* t3, T* t2, T* v2, int cond_kernel_1, int opt_register_transpose) TC_SHIM_BODY_(EXPR, DTYPE, 8, s0, s1, s2, s3, s4, s5, s6, s7)

#endif /* TC_B200_SHIM_H_ */
