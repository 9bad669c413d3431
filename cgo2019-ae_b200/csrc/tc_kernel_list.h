// The compiled contraction kernels: one line per (arithmetic, dtype, CTA tile,
// warp layout).  build.py turns every line into its own translation unit
// (csrc/_obj/gen_<name>.cu) so they compile in parallel; tc_api.cu expands the
// same list into the dispatch registry.
//
//   X(name, T, MATH, BM, BN, WARPS_M, WARPS_N, STAGES, MIN_CTAS_PER_SM, VARIANT)
//
// DMMA / TF32X3: WARPS_M x WARPS_N warps, warp tile (BM/WARPS_M) x (BN/WARPS_N), both
// multiples of 16.  SIMT: (BM/8) x (BN/8) threads with 8 x 8 outputs each
// (WARPS_* unused).  VARIANT distinguishes warp layouts of the same tile.
#ifndef TC_KERNEL_LIST_H_
#define TC_KERNEL_LIST_H_

#define TC_KERNEL_LIST(X)                                                  \
  X(dmma_128x128_w8, double, TC_MATH_DMMA, 128, 128, 2, 4, 4, 1, 0)        \
  X(dmma_128x128_w16, double, TC_MATH_DMMA, 128, 128, 4, 4, 4, 1, 1)       \
  X(dmma_128x64_w4, double, TC_MATH_DMMA, 128, 64, 2, 2, 3, 2, 0)          \
  X(dmma_128x64_w8, double, TC_MATH_DMMA, 128, 64, 4, 2, 3, 2, 1)          \
  X(dmma_128x96_w8, double, TC_MATH_DMMA, 128, 96, 4, 2, 3, 1, 0)          \
  X(dmma_64x96_w4, double, TC_MATH_DMMA, 64, 96, 2, 2, 3, 3, 0)            \
  X(dmma_64x64_w4, double, TC_MATH_DMMA, 64, 64, 2, 2, 3, 4, 0)            \
  X(dfma_128x128, double, TC_MATH_SIMT, 128, 128, 1, 1, 3, 1, 0)           \
  X(dfma_64x64, double, TC_MATH_SIMT, 64, 64, 1, 1, 4, 1, 0)               \
  X(ffma_128x128, float, TC_MATH_SIMT, 128, 128, 1, 1, 4, 2, 0)            \
  X(ffma_128x64, float, TC_MATH_SIMT, 128, 64, 1, 1, 4, 3, 0)              \
  X(ffma_96x128, float, TC_MATH_SIMT, 96, 128, 1, 1, 4, 3, 0)              \
  X(ffma_96x64, float, TC_MATH_SIMT, 96, 64, 1, 1, 4, 5, 0)                \
  X(ffma_64x64, float, TC_MATH_SIMT, 64, 64, 1, 1, 4, 4, 0)               \
  X(tf32_128x128, float, TC_MATH_TF32X3, 128, 128, 2, 4, 4, 2, 0)          \
  X(tf32_96x128, float, TC_MATH_TF32X3, 96, 128, 2, 4, 4, 2, 0)            \
  X(tf32tc_96x128, float, TC_MATH_TF32TC, 96, 128, 2, 4, 2, 3, 0)          \
  X(tf32tc_128x128, float, TC_MATH_TF32TC, 128, 128, 2, 4, 2, 3, 0)        \
  X(tf32_64x64, float, TC_MATH_TF32X3, 64, 64, 2, 2, 4, 4, 0)

// Persistent warp-specialised fp64 kernels (tc_ws_kernel.cuh): two consumer groups of 2 x 2 warps,
// each on its own BM x BN tile, plus four producer warps.
//   X(name, BM, BN, STAGES, VARIANT)
#define TC_WS_KERNEL_LIST(X) \
  X(dmma_ws_128x64, 128, 64, 3, 2)     \
  X(dmma_ws_128x32, 128, 32, 4, 2)     \
  X(dmma_ws_64x96, 64, 96, 3, 2)

// Persistent fp64 kernels that keep the output tile resident in shared memory (tc_wc_kernel.cuh): GROUPS consumer
// groups of WGM x WGN warps, each on its own BM x 64 tile.
//   X(name, BM, GROUPS, WGM, WGN, STAGES, VARIANT)
#define TC_WC_KERNEL_LIST(X)            \
  X(dmma_wc_128x64, 128, 1, 4, 2, 3, 3)

// Persistent fp32 kernels on tcgen05 (tc_wt_kernel.cuh): BM x 128 tiles, two accumulators in tensor memory, the
// output tile resident in shared memory.
//   X(name, BM, VARIANT)
#define TC_WT_KERNEL_LIST(X)   \
  X(tf32wt_96x128, 96, 1)      \
  X(tf32wt_128x128, 128, 1)

#endif  // TC_KERNEL_LIST_H_
