// Instantiation helper: one translation unit per line of tc_kernel_list.h
// so the variants compile in parallel.  Each unit exports one dispatcher that
// selects the loader variant (16-byte loads along the external index of X / Y
// or element-wise loads) and either launches, prepares (opt-in shared memory)
// or reports the launch shape.
#pragma once
#include "tc_kernels.cuh"
#include "tc_ws_kernel.cuh"
#include "tc_wc_kernel.cuh"
#include "tc_wt_kernel.cuh"

// TC_INST_CARVE (persistent tcgen05 kernel): *threads = operand stages that fit beside args->out_bufs output tile
// buffers and args->img_sets image sets.
enum TcInstMode { TC_INST_LAUNCH = 0, TC_INST_PREPARE = 1, TC_INST_QUERY = 2, TC_INST_OCCUPANCY = 3, TC_INST_CARVE = 4 };

// mode_x / mode_y: 0 element loads, 1 16-byte loads along the external index, 2 16-byte loads along the
// contraction index, 3 one tiled TMA copy per stage (kernels without these images treat 2 and 3 as 0).
typedef int (*tc_inst_fn)(int mode_x, int mode_y, const TcKernelArgs* args, void* C, const void* X, const void* Y,
                          cudaStream_t stream, int mode, int* threads, int* smem_bytes);

namespace tck {

template <class CF>
int run_variant(const TcKernelArgs* a, void* C, const void* X, const void* Y, cudaStream_t stream, int mode,
                int* threads, int* smem_bytes) {
  using T = typename CF::T;
  auto kern = tc_contract_kernel<CF>;
  if (mode == TC_INST_QUERY) {
    if (threads) *threads = CF::THREADS;
    if (smem_bytes) *smem_bytes = CF::SMEM_BYTES;
    return TC_OK;
  }
  if (mode == TC_INST_OCCUPANCY) {  // resident CTAs per SM -> *threads
    int n = 0;
    TC_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, CF::THREADS, CF::SMEM_BYTES));
    if (threads) *threads = n;
    return TC_OK;
  }
  if (mode == TC_INST_PREPARE) {
    TC_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, CF::SMEM_BYTES));
    // as much of the unified L1/shared array as shared memory as the device allows: residency is bounded by it
    TC_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    return TC_OK;
  }
  const unsigned grid = a->tiles_m * a->tiles_n * a->ksplit;
  kern<<<grid, CF::THREADS, CF::SMEM_BYTES, stream>>>(*a, static_cast<T*>(C), static_cast<const T*>(X),
                                                       static_cast<const T*>(Y));
  TC_CUDA_OK(cudaGetLastError());
  return TC_OK;
}

template <class CF, class Kern>
int run_persistent(Kern kern, const TcKernelArgs* a, void* C, const void* X, const void* Y, cudaStream_t stream,
                   int mode, int* threads, int* smem_bytes) {
  using T = typename CF::T;
  if (mode == TC_INST_QUERY) {
    if (threads) *threads = CF::CTA_THREADS;
    if (smem_bytes) *smem_bytes = CF::SMEM_BYTES;
    return TC_OK;
  }
  if (mode == TC_INST_OCCUPANCY) {
    if (threads) *threads = 1;
    return TC_OK;
  }
  if (mode == TC_INST_PREPARE) {
    TC_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, CF::SMEM_BYTES));
    return TC_OK;
  }
  int dev = 0, sms = 0;
  TC_CUDA_OK(cudaGetDevice(&dev));
  TC_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  // work items: tiles, times the K slices where the plan has them; a CTA's groups take consecutive items
  const unsigned tiles = a->tiles_m * a->tiles_n * (a->ksplit > 1 ? a->ksplit : 1u), per_cta = CF::GROUPS;
  const unsigned grid = (tiles + per_cta - 1) / per_cta < (unsigned)sms ? (tiles + per_cta - 1) / per_cta : (unsigned)sms;  // one persistent CTA per SM
  kern<<<grid, CF::CTA_THREADS, CF::SMEM_BYTES, stream>>>(*a, static_cast<T*>(C), static_cast<const T*>(X),
                                                           static_cast<const T*>(Y));
  TC_CUDA_OK(cudaGetLastError());
  return TC_OK;
}

template <class CF>
int run_ws_variant(const TcKernelArgs* a, void* C, const void* X, const void* Y, cudaStream_t stream, int mode,
                   int* threads, int* smem_bytes) {
  return run_persistent<CF>(tc_ws_dmma_kernel<CF>, a, C, X, Y, stream, mode, threads, smem_bytes);
}
template <class CF>
int run_wc_variant(const TcKernelArgs* a, void* C, const void* X, const void* Y, cudaStream_t stream, int mode,
                   int* threads, int* smem_bytes) {
  return run_persistent<CF>(tc_wc_dmma_kernel<CF>, a, C, X, Y, stream, mode, threads, smem_bytes);
}
template <class CF>
int run_wt_variant(const TcKernelArgs* a, void* C, const void* X, const void* Y, cudaStream_t stream, int mode,
                   int* threads, int* smem_bytes) {
  if (mode == TC_INST_CARVE) {
    if (!a || !threads || a->out_bufs < 1 || a->out_bufs > CF::MAX_CBUFS || a->img_sets < 1 || a->img_sets > CF::MAX_IMGS) return TC_ERR_INVALID_ARG;
    *threads = CF::stages_for(a->out_bufs, a->img_sets);
    return *threads >= 2 ? TC_OK : TC_ERR_UNSUPPORTED;
  }
  return run_persistent<CF>(tc_wt_tf32_kernel<CF>, a, C, X, Y, stream, mode, threads, smem_bytes);
}
}  // namespace tck

// Persistent fp32 kernel: loader modes 0 element, 1 external vector, 2 contraction vector, 3 / 4 one tiled TMA box per
// stage (contraction index fastest / external index fastest).
#define TC_WT_CASE(MX, MY, BM) \
  if (vx == MX && vy == MY) return tck::run_wt_variant<tck::WtCfg<BM, MX, MY>>(a, C, X, Y, s, mode, threads, smem);
#define TC_WT_ROW(MX, BM) TC_WT_CASE(MX, 0, BM) TC_WT_CASE(MX, 1, BM) TC_WT_CASE(MX, 2, BM) TC_WT_CASE(MX, 3, BM) TC_WT_CASE(MX, 4, BM)
#define TC_DEFINE_WT_INST(NAME, BM)                                                                          \
  extern "C" int NAME(int vx, int vy, const TcKernelArgs* a, void* C, const void* X, const void* Y,         \
                      cudaStream_t s, int mode, int* threads, int* smem) {                                  \
    TC_WT_ROW(0, BM) TC_WT_ROW(1, BM) TC_WT_ROW(2, BM) TC_WT_ROW(3, BM) TC_WT_ROW(4, BM)                    \
    return TC_ERR_INVALID_ARG;                                                                              \
  }

#define TC_WC_CASE(MX, MY, BM, GROUPS, WGM, WGN, STAGES) \
  if (vx == MX && vy == MY) return tck::run_wc_variant<tck::WcCfg<BM, GROUPS, WGM, WGN, STAGES, MX, MY>>(a, C, X, Y, s, mode, threads, smem);
#define TC_WC_ROW(MX, BM, GROUPS, WGM, WGN, STAGES) \
  TC_WC_CASE(MX, 0, BM, GROUPS, WGM, WGN, STAGES) TC_WC_CASE(MX, 1, BM, GROUPS, WGM, WGN, STAGES) \
  TC_WC_CASE(MX, 2, BM, GROUPS, WGM, WGN, STAGES) TC_WC_CASE(MX, 3, BM, GROUPS, WGM, WGN, STAGES)
#define TC_DEFINE_WC_INST(NAME, BM, GROUPS, WGM, WGN, STAGES)                                               \
  extern "C" int NAME(int vx, int vy, const TcKernelArgs* a, void* C, const void* X, const void* Y,         \
                      cudaStream_t s, int mode, int* threads, int* smem) {                                  \
    TC_WC_ROW(0, BM, GROUPS, WGM, WGN, STAGES) TC_WC_ROW(1, BM, GROUPS, WGM, WGN, STAGES)                   \
    TC_WC_ROW(2, BM, GROUPS, WGM, WGN, STAGES) TC_WC_ROW(3, BM, GROUPS, WGM, WGN, STAGES)                   \
    return TC_ERR_INVALID_ARG;                                                                              \
  }

#define TC_WS_CASE(MX, MY, BM, BN, STAGES) \
  if (vx == MX && vy == MY) return tck::run_ws_variant<tck::WsCfg<BM, BN, STAGES, MX, MY>>(a, C, X, Y, s, mode, threads, smem);
#define TC_DEFINE_WS_INST(NAME, BM, BN, STAGES)                                                              \
  extern "C" int NAME(int vx, int vy, const TcKernelArgs* a, void* C, const void* X, const void* Y,         \
                      cudaStream_t s, int mode, int* threads, int* smem) {                                  \
    TC_WS_CASE(0, 0, BM, BN, STAGES) TC_WS_CASE(0, 1, BM, BN, STAGES) TC_WS_CASE(0, 2, BM, BN, STAGES) TC_WS_CASE(0, 3, BM, BN, STAGES) \
    TC_WS_CASE(1, 0, BM, BN, STAGES) TC_WS_CASE(1, 1, BM, BN, STAGES) TC_WS_CASE(1, 2, BM, BN, STAGES) TC_WS_CASE(1, 3, BM, BN, STAGES) \
    TC_WS_CASE(2, 0, BM, BN, STAGES) TC_WS_CASE(2, 1, BM, BN, STAGES) TC_WS_CASE(2, 2, BM, BN, STAGES) TC_WS_CASE(2, 3, BM, BN, STAGES) \
    TC_WS_CASE(3, 0, BM, BN, STAGES) TC_WS_CASE(3, 1, BM, BN, STAGES) TC_WS_CASE(3, 2, BM, BN, STAGES) TC_WS_CASE(3, 3, BM, BN, STAGES) \
    return TC_ERR_INVALID_ARG;                                                                              \
  }

// Kernels with a third loader per operand (16 bytes along the contraction index): modes 0 element, 1 external
// vector, 2 contraction vector.
#define TC_KV_CASE(MX, MY, T, MATH, BM, BN, WMN, WNN, STAGES, MINB)                                                   \
  if (vx == MX && vy == MY)                                                                                           \
    return tck::run_variant<tck::Cfg<T, MATH, BM, BN, WMN, WNN, STAGES, MINB, MX == 1, MY == 1, MX == 2, MY == 2>>(     \
        a, C, X, Y, s, mode, threads, smem);
#define TC_DEFINE_INST_KV(NAME, T, MATH, BM, BN, WMN, WNN, STAGES, MINB)                                              \
  extern "C" int NAME(int vx, int vy, const TcKernelArgs* a, void* C, const void* X, const void* Y,                  \
                      cudaStream_t s, int mode, int* threads, int* smem) {                                           \
    TC_KV_CASE(0, 0, T, MATH, BM, BN, WMN, WNN, STAGES, MINB) TC_KV_CASE(0, 1, T, MATH, BM, BN, WMN, WNN, STAGES, MINB) \
    TC_KV_CASE(0, 2, T, MATH, BM, BN, WMN, WNN, STAGES, MINB) TC_KV_CASE(1, 0, T, MATH, BM, BN, WMN, WNN, STAGES, MINB) \
    TC_KV_CASE(1, 1, T, MATH, BM, BN, WMN, WNN, STAGES, MINB) TC_KV_CASE(1, 2, T, MATH, BM, BN, WMN, WNN, STAGES, MINB) \
    TC_KV_CASE(2, 0, T, MATH, BM, BN, WMN, WNN, STAGES, MINB) TC_KV_CASE(2, 1, T, MATH, BM, BN, WMN, WNN, STAGES, MINB) \
    TC_KV_CASE(2, 2, T, MATH, BM, BN, WMN, WNN, STAGES, MINB)                                                         \
    return TC_ERR_INVALID_ARG;                                                                                        \
  }

#define TC_DEFINE_INST(NAME, T, MATH, BM, BN, WMN, WNN, STAGES, MINB)                                                  \
  extern "C" int NAME(int vx, int vy, const TcKernelArgs* a, void* C, const void* X, const void* Y,              \
                      cudaStream_t s, int mode, int* threads, int* smem) {                                       \
    vx = vx == 1; vy = vy == 1;                                                                                  \
    if (vx && vy) return tck::run_variant<tck::Cfg<T, MATH, BM, BN, WMN, WNN, STAGES, MINB, true, true>>(a, C, X, Y, s, mode, threads, smem);   \
    if (vx) return tck::run_variant<tck::Cfg<T, MATH, BM, BN, WMN, WNN, STAGES, MINB, true, false>>(a, C, X, Y, s, mode, threads, smem);        \
    if (vy) return tck::run_variant<tck::Cfg<T, MATH, BM, BN, WMN, WNN, STAGES, MINB, false, true>>(a, C, X, Y, s, mode, threads, smem);        \
    return tck::run_variant<tck::Cfg<T, MATH, BM, BN, WMN, WNN, STAGES, MINB, false, false>>(a, C, X, Y, s, mode, threads, smem);               \
  }
