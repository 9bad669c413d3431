// C ABI: plan / execute / free, the seeded input generator and small utilities.
// Declarations and the reference interfaces they replace are in include/tc_b200.h.
#include <cuda.h>  // types of the tensor-map encoder only; the entry point is looked up at run time
#include <cuda_runtime.h>
#include <stdlib.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>

#include "tc_inst.cuh"
#include "tc_internal.h"

// ---------------------------------------------------------------- errors ----
static thread_local char g_cuda_error[256] = "";

void tc_note_cuda_error(int code, const char* what) {
  std::snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s (%d)", what, cudaGetErrorString((cudaError_t)code), code);
}

extern "C" const char* tc_last_cuda_error(void) { return g_cuda_error; }

extern "C" const char* tc_status_string(int s) {
  switch (s) {
    case TC_OK: return "ok";
    case TC_ERR_PARSE: return "expression rejected by the grammar";
    case TC_ERR_INVALID_ARG: return "invalid argument";
    case TC_ERR_UNSUPPORTED: return "unsupported contraction";
    case TC_ERR_EXTENT: return "bad extent or stride";
    case TC_ERR_CUDA: return "CUDA error";
    case TC_ERR_ALIGNMENT: return "misaligned tensor pointer";
    case TC_ERR_STATE: return "call order violated";
    case TC_ERR_WORKSPACE: return "workspace missing or too small";
    default: return "unknown status";
  }
}

extern "C" const char* tc_version(void) { return "tc_b200 0.1 (sm_100a)"; }

static void copy_out(const std::string& s, char* buf, size_t cap) {
  if (!buf || cap == 0) return;
  const size_t n = std::min(cap - 1, s.size());
  std::memcpy(buf, s.data(), n);
  buf[n] = '\0';
}

// ------------------------------------------------------------ expression ----
extern "C" int tc_expr_describe(const char* expr, char* buf, size_t cap) {
  TcExpr e;
  std::string why;
  const int st = tc_parse_expr(expr, &e, &why);
  copy_out(st == TC_OK ? tc_expr_to_json(e) : "{\"error\":\"" + why + "\"}", buf, cap);
  return st;
}

// -------------------------------------------------------- kernel dispatch ----
#include "tc_kernel_list.h"

#define TC_DECLARE(NAME, T, MATH, BM, BN, WMN, WNN, STAGES, MINB, VARIANT) \
  extern "C" int tc_inst_##NAME(int, int, const TcKernelArgs*, void*, const void*, const void*, cudaStream_t, int, int*, int*);
TC_KERNEL_LIST(TC_DECLARE)
#undef TC_DECLARE
#define TC_DECLARE_WS(NAME, BM, BN, STAGES, VARIANT) \
  extern "C" int tc_inst_##NAME(int, int, const TcKernelArgs*, void*, const void*, const void*, cudaStream_t, int, int*, int*);
TC_WS_KERNEL_LIST(TC_DECLARE_WS)
#undef TC_DECLARE_WS

namespace {
struct KernelEntry {
  const char* name;
  int dtype, math, bm, bn, variant;
  tc_inst_fn fn;
};
template <typename T> constexpr int dtype_of() { return sizeof(T) == 8 ? TC_F64 : TC_F32; }
#define TC_ENTRY(NAME, T, MATH, BM, BN, WMN, WNN, STAGES, MINB, VARIANT) {#NAME, dtype_of<T>(), MATH, BM, BN, VARIANT, tc_inst_##NAME},
#define TC_WS_ENTRY(NAME, BM, BN, STAGES, VARIANT) {#NAME, TC_F64, TC_MATH_DMMA, BM, BN, VARIANT, tc_inst_##NAME},
const KernelEntry kKernels[] = {TC_KERNEL_LIST(TC_ENTRY) TC_WS_KERNEL_LIST(TC_WS_ENTRY)};
#undef TC_ENTRY
#undef TC_WS_ENTRY

const KernelEntry* find_kernel(int dtype, int math, int bm, int bn, int variant) {
  for (const KernelEntry& k : kKernels)
    if (k.dtype == dtype && k.math == math && k.bm == bm && k.bn == bn && k.variant == variant) return &k;
  return nullptr;
}
}  // namespace

bool tc_kernel_exists(int dtype, int math, int bm, int bn, int variant) {
  return find_kernel(dtype, math, bm, bn, variant) != nullptr;
}

const char* tc_kernel_name(const TcKernelChoice& c) {
  const KernelEntry* k = find_kernel(c.dtype, c.math, c.bm, c.bn, c.variant);
  return k ? k->name : "?";
}

static tc_inst_fn pick_inst(const TcKernelChoice& c) {
  const KernelEntry* k = find_kernel(c.dtype, c.math, c.bm, c.bn, c.variant);
  return k ? k->fn : nullptr;
}

static int mode_of(bool ext_vec, bool k_vec) { return ext_vec ? 1 : k_vec ? 2 : 0; }

// Tiled TMA descriptor of an operand seen as a 2-D fp64 matrix: dimension 0 = contraction index (stride 1),
// dimension 1 = flattened external index at `pitch` elements; box = 16 x rows, 128-byte swizzle, zero fill
// outside the tensor.  cuTensorMapEncodeTiled is resolved through the runtime (no link against libcuda).
static bool encode_operand_map(TcTensorMap* out, const void* base, uint64_t k_extent, uint64_t ext_extent,
                               uint64_t pitch, uint32_t rows) {
  typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static encode_fn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<encode_fn>(f);
  }();
  if (!fn || (reinterpret_cast<uintptr_t>(base) & 15) || (pitch * 8) % 16 != 0 || rows > 256) return false;
  const cuuint64_t dims[2] = {k_extent, ext_extent};
  const cuuint64_t strides[1] = {pitch * 8};
  const cuuint32_t box[2] = {16, rows};
  const cuuint32_t estr[2] = {1, 1};
  static_assert(sizeof(CUtensorMap) == sizeof(TcTensorMap), "tensor map storage");
  return fn(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 2, const_cast<void*>(base), dims,
            strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Rank-5 tiled TMA descriptor of the fp64 output for the persistent kernel's epilogue.  Dimensions, fastest
// first: the contiguous run of the fastest M dimensions; the parity of n; n / 2 inside N's fastest dimensions;
// then the remaining N and M dimensions (at most two together, padded with extent 1).
// Box = (bw, bh, bq, 1, 1): (warp rows, 1, 8) for the 8 rows one consumer warp stages at a time, or
// (bm, 2, bn / 2) for a whole tile.  No swizzle, no fill.
static bool encode_output_map(TcTensorMap* out, const void* base, const TcOutMap& o, uint32_t bw, uint32_t bh,
                              uint32_t bq) {
  typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static encode_fn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<encode_fn>(f);
  }();
  if (!fn || (reinterpret_cast<uintptr_t>(base) & 15) || bw > 256 || bq > 256 || o.e0 == 0 || o.f0 < 2 || o.ne + o.me > 2) return false;
  cuuint64_t dims[5] = {o.e0, 2, o.f0 / 2, 1, 1};
  cuuint64_t strides[4] = {(cuuint64_t)o.stride_n * 8, (cuuint64_t)o.stride_n * 16, 0, 0};
  int r = 3;
  for (int d = 0; d < o.ne + o.me; ++d, ++r) { dims[r] = o.ext[d]; strides[r - 1] = (cuuint64_t)o.stride[d] * 8; }
  for (; r < 5; ++r) strides[r - 1] = strides[r - 2] * dims[r - 1];  // extent-1 padding: any aligned stride
  for (int i = 0; i < 4; ++i)
    if (strides[i] % 16 != 0 || strides[i] >= (cuuint64_t(1) << 40)) return false;
  const cuuint32_t box[5] = {bw, bh, bq, 1, 1};
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  return fn(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 5, const_cast<void*>(base), dims,
            strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int tc_kernel_shape(const TcKernelChoice& c, int* threads, int* smem_bytes, int* bk) {
  if (bk) *bk = TC_BK;
  tc_inst_fn fn = pick_inst(c);
  if (!fn) return TC_ERR_UNSUPPORTED;
  return fn(mode_of(c.vec_x, c.kvec_x), mode_of(c.vec_y, c.kvec_y), nullptr, nullptr, nullptr, nullptr, nullptr, TC_INST_QUERY, threads, smem_bytes);
}

int tc_kernels_prepare(const TcKernelChoice& c) {
  // Both loader variants of each operand: a misaligned base pointer at execute
  // time demotes 16-byte loads to element loads.
  tc_inst_fn fn = pick_inst(c);
  if (!fn) return TC_ERR_UNSUPPORTED;
  const int mx = mode_of(c.vec_x, c.kvec_x), my = mode_of(c.vec_y, c.kvec_y);
  const bool ws = tc_kernel_is_persistent(c) && c.math == TC_MATH_DMMA;
  const int xs[3] = {0, mx, (ws && c.tma_x) ? 3 : 0}, ys[3] = {0, my, (ws && c.tma_y) ? 3 : 0};
  for (int vx : xs)
    for (int vy : ys) {
      const int st = fn(vx, vy, nullptr, nullptr, nullptr, nullptr, nullptr, TC_INST_PREPARE, nullptr, nullptr);
      if (st != TC_OK) return st;
    }
  return TC_OK;
}

// Resident CTAs of the chosen kernel on the whole device (0 on failure).
static int resident_ctas(const TcKernelChoice& c) {
  tc_inst_fn fn = pick_inst(c);
  int per_sm = 0, dev = 0, sms = 0;
  if (!fn || fn(mode_of(c.vec_x, c.kvec_x), mode_of(c.vec_y, c.kvec_y), nullptr, nullptr, nullptr, nullptr, nullptr, TC_INST_OCCUPANCY, &per_sm, nullptr) != TC_OK) return 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  return per_sm * sms;
}

int tc_launch_contraction(const tc_plan& p, const TcKernelArgs& args, void* C, const void* X, const void* Y,
                          cudaStream_t stream) {
  const TcKernelChoice& c = p.choice;
  TcKernelArgs a = args;
  // Alignment-driven demotions (base pointers are the only run-time unknowns).
  const bool x16 = (reinterpret_cast<uintptr_t>(X) & 15) == 0, y16 = (reinterpret_cast<uintptr_t>(Y) & 15) == 0;
  const uintptr_t cu = reinterpret_cast<uintptr_t>(C);
  if ((cu & 15) != 0) a.vec_c = 1;
  int vx = x16 ? mode_of(c.vec_x, c.kvec_x) : 0, vy = y16 ? mode_of(c.vec_y, c.kvec_y) : 0;
  // Persistent kernels fetch operands that are plain 2-D matrices with one tiled TMA copy per stage.
  if (tc_kernel_is_persistent(c) && c.math == TC_MATH_DMMA && p.opt.tma != 1) {
    const bool operands = p.opt.tma == 0 || p.opt.tma == 2 || p.opt.tma == 4, output = p.opt.tma == 0 || p.opt.tma == 3 || p.opt.tma == 4;
    if (operands && c.tma_x && encode_operand_map(&a.tmap_x, X, a.Kflat, a.Mflat, (uint64_t)a.M.s_in[0], (uint32_t)a.bm)) vx = 3;
    if (operands && c.tma_y && encode_operand_map(&a.tmap_y, Y, a.Kflat, a.Nflat, (uint64_t)a.N.s_in[0], (uint32_t)a.bn)) vy = 3;
    a.c_tensor = (output && c.tma_c && a.c_mode == 2 &&
                  encode_output_map(&a.tmap_c, C, a.cmap, (uint32_t)a.bm / 2 /* rows of a consumer warp's block */, 1, 8)) ? 1 : 0;
    if (a.c_tensor == 1 && c.tma_ct && p.opt.tma != 4 &&
        encode_output_map(&a.tmap_ct, C, a.cmap, (uint32_t)a.bm, 2, (uint32_t)a.bn / 2))
      a.c_tensor = 2;
  }
  tc_inst_fn fn = pick_inst(c);
  if (!fn) return TC_ERR_UNSUPPORTED;
  int st = fn(vx, vy, &a, C, X, Y, stream, TC_INST_LAUNCH, nullptr, nullptr);
  if (st != TC_OK) return st;
  if (a.ksplit > 1) {
    const unsigned grid = a.tiles_m * a.tiles_n;
    const size_t smem = (size_t)(a.bm + a.bn) * sizeof(int64_t);
    if (p.dtype == TC_F64) tck::tc_combine_kernel<double><<<grid, 256, smem, stream>>>(a, static_cast<double*>(C));
    else tck::tc_combine_kernel<float><<<grid, 256, smem, stream>>>(a, static_cast<float*>(C));
    TC_CUDA_OK(cudaGetLastError());
  }
  return TC_OK;
}

// ------------------------------------------------------------------ plan ----
extern "C" int tc_plan_create(const char* expr, int dtype, const tc_options* options, tc_plan** out) {
  if (!expr || !out) return TC_ERR_INVALID_ARG;
  *out = nullptr;
  if (dtype != TC_F64 && dtype != TC_F32) return TC_ERR_INVALID_ARG;
  TcExpr e;
  std::string why;
  const int st = tc_parse_expr(expr, &e, &why);
  if (st != TC_OK) return st;
  tc_plan* p = new (std::nothrow) tc_plan();
  if (!p) return TC_ERR_INVALID_ARG;
  p->expr = e;
  p->dtype = dtype;
  if (options) p->opt = *options;
  if (p->opt.path < TC_PATH_AUTO || p->opt.path > TC_PATH_TCGEN05 || p->opt.split_k < 0) {
    delete p;
    return TC_ERR_INVALID_ARG;
  }
  for (size_t i = 0; i < e.out_idx.size(); ++i) { p->idx_names.push_back(e.out_idx[i]); p->idx_extent.push_back(e.out_ext[i]); }
  for (size_t i = 0; i < e.sum_idx.size(); ++i) { p->idx_names.push_back(e.sum_idx[i]); p->idx_extent.push_back(e.sum_ext[i]); }
  *out = p;
  return TC_OK;
}

extern "C" int tc_plan_set_extents(tc_plan* p, int n, const char* const* names, const int64_t* extents) {
  if (!p || n < 0 || (n > 0 && (!names || !extents))) return TC_ERR_INVALID_ARG;
  if (p->committed) return TC_ERR_STATE;
  std::vector<int64_t> next = p->idx_extent;
  for (int i = 0; i < n; ++i) {
    if (!names[i]) return TC_ERR_INVALID_ARG;
    if (extents[i] <= 0) return TC_ERR_EXTENT;
    size_t j = 0;
    for (; j < p->idx_names.size(); ++j)
      if (p->idx_names[j] == names[i]) break;
    if (j == p->idx_names.size()) return TC_ERR_INVALID_ARG;
    next[j] = extents[i];
  }
  p->idx_extent = next;
  return TC_OK;
}

extern "C" int tc_plan_set_extents_ordered(tc_plan* p, int n, const int64_t* extents) {
  if (!p || n < 0 || (n > 0 && !extents)) return TC_ERR_INVALID_ARG;
  if (p->committed) return TC_ERR_STATE;
  if ((size_t)n != p->idx_names.size()) return TC_ERR_INVALID_ARG;
  for (int i = 0; i < n; ++i)
    if (extents[i] <= 0) return TC_ERR_EXTENT;
  p->idx_extent.assign(extents, extents + n);
  return TC_OK;
}

extern "C" int tc_plan_set_strides(tc_plan* p, int tensor, int n, const int64_t* strides) {
  if (!p || tensor < 0 || tensor > 2 || n < 0 || (n > 0 && !strides)) return TC_ERR_INVALID_ARG;
  if (p->committed) return TC_ERR_STATE;
  const size_t rank = tensor == 0 ? p->expr.out_idx.size() : tensor == 1 ? p->expr.left_idx.size() : p->expr.right_idx.size();
  if ((size_t)n != rank) return TC_ERR_INVALID_ARG;
  for (int i = 0; i < n; ++i)
    if (strides[i] <= 0) return TC_ERR_EXTENT;
  p->strides[tensor].assign(strides, strides + n);
  p->custom_strides[tensor] = true;
  return TC_OK;
}

extern "C" int tc_plan_commit(tc_plan* p) {
  if (!p) return TC_ERR_INVALID_ARG;
  if (p->committed) return TC_OK;
  int st = tc_plan_build(p, &p->why);
  if (st != TC_OK) return st;
  int dev = 0;
  TC_CUDA_OK(cudaGetDevice(&dev));
  st = tc_kernels_prepare(p->choice);
  if (st != TC_OK) return st;
  // How the result reaches C (tc_options.c_path) and whether output tiles are prefetched into L2.
  // Defaults follow the B200 measurements: persistent kernels hand their tiles to the memory system as
  // bulk reduce-adds and need no prefetch; the one-CTA-per-tile kernels read-modify-write behind a prefetch.
  const bool persistent = tc_kernel_is_persistent(p->choice);
  const int c_path = p->opt.c_path;
  p->args.c_mode = c_path > 0 ? c_path - 1 : ((persistent || p->choice.math != TC_MATH_DMMA) ? 2 : 0);
  p->args.c_stream = 0;
  const bool bulk_out = p->args.c_mode == 2 && (persistent || p->args.epi_run > 0);
  // ... unless the whole problem is a fraction of one wave: then the tile is in flight anyway and the prefetch
  // only lengthens a latency-bound kernel (measured on the 64 x 48 x 32 configuration: 10.7 -> 9.4 us).
  const bool tiny = (int64_t)p->args.tiles_m * p->args.tiles_n * p->args.ksplit < 148;
  const bool prefetch = p->opt.l2_prefetch == 2 || (p->opt.l2_prefetch == 0 && !bulk_out && !tiny);
  p->args.prefetch_dist = prefetch ? (uint32_t)resident_ctas(p->choice) : 0u;
  const size_t kb = p->h_koff_x.size() * sizeof(int64_t);
  TC_CUDA_OK(cudaMalloc(&p->d_koff, 2 * kb));
  TC_CUDA_OK(cudaMemcpy(p->d_koff, p->h_koff_x.data(), kb, cudaMemcpyHostToDevice));
  TC_CUDA_OK(cudaMemcpy(static_cast<char*>(p->d_koff) + kb, p->h_koff_y.data(), kb, cudaMemcpyHostToDevice));
  p->args.koff_x = static_cast<const int64_t*>(p->d_koff);
  p->args.koff_y = p->args.koff_x + p->h_koff_x.size();
  if (p->ws_bytes) TC_CUDA_OK(cudaMalloc(&p->d_ws, p->ws_bytes));
  TC_CUDA_OK(cudaMalloc(&p->d_status, sizeof(int)));
  TC_CUDA_OK(cudaMemset(p->d_status, 0, sizeof(int)));
  p->args.status = p->d_status;
  p->device = dev;
  p->committed = true;
  return TC_OK;
}

struct TcHostPipe;
static void host_pipe_destroy(TcHostPipe* h);

extern "C" void tc_plan_destroy(tc_plan* p) {
  if (!p) return;
  if (p->d_koff) cudaFree(p->d_koff);
  if (p->d_ws) cudaFree(p->d_ws);
  if (p->d_status) cudaFree(p->d_status);
  host_pipe_destroy(p->host);
  delete p;
}

extern "C" int tc_plan_describe(const tc_plan* p, char* buf, size_t cap) {
  if (!p) return TC_ERR_INVALID_ARG;
  if (p->committed) { copy_out(tc_plan_to_json(*p), buf, cap); return TC_OK; }
  // Not committed yet: run the host-side planner on a copy (needs no GPU).
  tc_plan tmp = *p;
  std::string why;
  const int st = tc_plan_build(&tmp, &why);
  if (st != TC_OK) { copy_out("{\"error\":\"" + why + "\"}", buf, cap); return st; }
  tmp.committed = true;
  std::string js = tc_plan_to_json(tmp);
  tmp.committed = false;
  copy_out(js, buf, cap);
  return TC_OK;
}

extern "C" int tc_plan_cost(const tc_plan* p, double* flops, double* bytes) {
  if (!p) return TC_ERR_INVALID_ARG;
  tc_plan tmp = *p;
  if (!p->committed) {
    std::string why;
    const int st = tc_plan_build(&tmp, &why);
    if (st != TC_OK) return st;
  }
  if (flops) *flops = tmp.flops;
  if (bytes) *bytes = tmp.bytes;
  return TC_OK;
}

extern "C" int tc_plan_status(tc_plan* p, int* device_status) {
  if (!p || !device_status) return TC_ERR_INVALID_ARG;
  if (!p->committed) return TC_ERR_STATE;
  TC_CUDA_OK(cudaMemcpy(device_status, p->d_status, sizeof(int), cudaMemcpyDeviceToHost));
  return TC_OK;
}

extern "C" int tc_plan_launches(const tc_plan* p) { return p && p->committed ? p->launches : -1; }

extern "C" int tc_plan_workspace_bytes(const tc_plan* p, size_t* bytes) {
  if (!p || !bytes) return TC_ERR_INVALID_ARG;
  if (!p->committed) return TC_ERR_STATE;
  *bytes = p->ws_bytes;
  return TC_OK;
}

// --------------------------------------------------------------- execute ----
static int execute_impl(tc_plan* p, void* C, const void* A, const void* B, void* ws, size_t ws_bytes, void* stream) {
  if (!p || !C || !A || !B) return TC_ERR_INVALID_ARG;
  if (!p->committed) {
    const int st = tc_plan_commit(p);
    if (st != TC_OK) return st;
  }
  int dev = 0;
  TC_CUDA_OK(cudaGetDevice(&dev));
  if (dev != p->device) return TC_ERR_STATE;
  const uintptr_t es = p->dtype == TC_F64 ? 8 : 4;
  if ((reinterpret_cast<uintptr_t>(C) | reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & (es - 1))
    return TC_ERR_ALIGNMENT;
  TcKernelArgs a = p->args;
  if (a.ksplit > 1) {
    if (!ws || ws_bytes < p->ws_bytes || (reinterpret_cast<uintptr_t>(ws) & 15)) return TC_ERR_WORKSPACE;
    a.ws = ws;
  }
#ifdef TC_WS_TIMING
  a.ws = ws;
#endif
  const void* X = p->swapped ? B : A;
  const void* Y = p->swapped ? A : B;
  return tc_launch_contraction(*p, a, C, X, Y, static_cast<cudaStream_t>(stream));
}

extern "C" int tc_execute(tc_plan* p, void* C, const void* A, const void* B, void* stream) {
  if (p && !p->committed) {
    const int st = tc_plan_commit(p);
    if (st != TC_OK) return st;
  }
  return execute_impl(p, C, A, B, p ? p->d_ws : nullptr, p ? p->ws_bytes : 0, stream);
}

extern "C" int tc_execute_ws(tc_plan* p, void* C, const void* A, const void* B, void* ws, size_t ws_bytes, void* stream) {
  return execute_impl(p, C, A, B, ws, ws_bytes, stream);
}

// ---------------------------------------------------- execute without allocating ----
// K-slice scratch that lives in the library image instead of in allocated memory.  Every GPU that
// loads the library carries these 8 MiB until the process exits.
static __device__ __align__(256) unsigned char g_tc_static_ws[TC_NOALLOC_MAX_WORKSPACE_BYTES];

namespace {
constexpr int kMaxDevices = 64;
// Device address of g_tc_static_ws per device.  In host code the array's name is only a handle for
// the runtime, not an address a kernel can use; the real address comes from cudaGetSymbolAddress,
// asked once per device with that device current.
void* g_static_ws_addr[kMaxDevices] = {};
}  // namespace

// For callers that must not allocate device memory at call time and have none to lend: an application
// whose own pool already owns the whole device (the reference's competitors pre-claim memory this way,
// nwchem-tccg/memory.cu:74-163), or a latency-critical loop where cudaMalloc's implicit device-wide
// synchronisation is not acceptable.  Same work as tc_execute on a committed plan; a plan that slices
// the contraction takes its slice scratch from the static array above.
//   * The plan must already be committed (committing uploads tables, which allocates): TC_ERR_STATE otherwise.
//   * Plans that need more than TC_NOALLOC_MAX_WORKSPACE_BYTES of scratch are refused with TC_ERR_WORKSPACE.
//   * The first call on each device looks up the array's device address; make that call before any
//     stream capture begins.
//   * All calls on a device share the one array and it keeps whatever the last call left in it.  Nothing
//     in it has to start at zero: every slice overwrites its whole partial tile before the combine step
//     reads it.  Two calls whose kernels overlap on the GPU (different streams) race on it: serialise them.
extern "C" int tc_execute_noalloc(tc_plan* p, void* C, const void* A, const void* B, void* stream) {
  if (!p || !C || !A || !B) return TC_ERR_INVALID_ARG;
  if (!p->committed) return TC_ERR_STATE;
  if (p->ws_bytes > (size_t)TC_NOALLOC_MAX_WORKSPACE_BYTES) return TC_ERR_WORKSPACE;
  int dev = 0;
  TC_CUDA_OK(cudaGetDevice(&dev));
  if (dev != p->device || dev < 0 || dev >= kMaxDevices) return TC_ERR_STATE;
  void* ws = nullptr;
  if (p->ws_bytes) {
    ws = __atomic_load_n(&g_static_ws_addr[dev], __ATOMIC_ACQUIRE);
    if (!ws) {
      void* addr = nullptr;
      TC_CUDA_OK(cudaGetSymbolAddress(&addr, g_tc_static_ws));
      if (!addr) return TC_ERR_CUDA;
      __atomic_store_n(&g_static_ws_addr[dev], addr, __ATOMIC_RELEASE);  // same value from every thread
      ws = addr;
    }
  }
  return execute_impl(p, C, A, B, ws, (size_t)TC_NOALLOC_MAX_WORKSPACE_BYTES, stream);
}

// Host-pointer path.  The reference's wrapper copies everything in, runs, copies the output back
// (cogent/src/codes/others/tc_pre_CUDA_Malloc.py:6-47, tc_interface.py:1368-1388).  Here the output's
// slowest index is cut into slabs and the slabs are pipelined over two streams: while slab i computes, slab
// i+1 is on its way in and slab i-1 on its way out, so a pass costs about max(bytes in, bytes out) over
// PCIe instead of their sum.  Inputs that carry the cut index as THEIR slowest index travel slab by slab
// too; the others go first, whole.  Device buffers, streams and the slab plans are created on the first
// call and kept with the plan.
struct TcHostPipe {
  void *dC = nullptr, *dA = nullptr, *dB = nullptr;
  cudaStream_t stream[2] = {nullptr, nullptr};
  cudaEvent_t inputs_ready = nullptr;
  int cut = -1;                 // position of the cut index in idx_names (-1: no slabs)
  int64_t extent = 1, slab = 1; // extent of the cut index, values per slab
  int64_t step[3] = {0, 0, 0};  // elements per value of the cut index where the tensor travels slab by slab (0: whole, first)
  int64_t view[3] = {0, 0, 0};  // element stride of the cut index in C, A, B (0: the tensor does not carry it)
  tc_plan* plan_slab = nullptr; // slab-sized sub-plan (strides of the full tensors)
  tc_plan* plan_tail = nullptr; // last, shorter slab
};

static void host_pipe_destroy(TcHostPipe* h) {
  if (!h) return;
  if (h->dC) cudaFree(h->dC);
  if (h->dA) cudaFree(h->dA);
  if (h->dB) cudaFree(h->dB);
  for (cudaStream_t s : h->stream)
    if (s) cudaStreamDestroy(s);
  if (h->inputs_ready) cudaEventDestroy(h->inputs_ready);
  if (h->plan_slab) tc_plan_destroy(h->plan_slab);
  if (h->plan_tail) tc_plan_destroy(h->plan_tail);
  delete h;
}

static int make_slab_plan(const tc_plan* p, int cut, int64_t count, tc_plan** out) {
  tc_plan* q = new (std::nothrow) tc_plan();
  if (!q) return TC_ERR_INVALID_ARG;
  q->expr = p->expr;
  q->dtype = p->dtype;
  q->opt = p->opt;
  q->idx_names = p->idx_names;
  q->idx_extent = p->idx_extent;
  q->idx_extent[cut] = count;
  // views into the full (compact) device tensors
  const std::vector<std::string>* tidx[3] = {&p->expr.out_idx, &p->expr.left_idx, &p->expr.right_idx};
  for (int t = 0; t < 3; ++t) {
    int64_t acc = 1;
    for (const std::string& n : *tidx[t]) {
      q->strides[t].push_back(acc);
      for (size_t j = 0; j < p->idx_names.size(); ++j)
        if (p->idx_names[j] == n) acc *= p->idx_extent[j];
    }
    q->custom_strides[t] = true;
  }
  const int st = tc_plan_commit(q);
  if (st != TC_OK) { tc_plan_destroy(q); return st; }
  *out = q;
  return TC_OK;
}

static int host_pipe_create(tc_plan* p) {
  TcHostPipe* h = new (std::nothrow) TcHostPipe();
  if (!h) return TC_ERR_INVALID_ARG;
  p->host = h;
  const size_t es = p->dtype == TC_F64 ? 8 : 4;
  TC_CUDA_OK(cudaMalloc(&h->dC, p->size_c * es));
  TC_CUDA_OK(cudaMalloc(&h->dA, p->size_a * es));
  TC_CUDA_OK(cudaMalloc(&h->dB, p->size_b * es));
  for (cudaStream_t& s : h->stream) TC_CUDA_OK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  TC_CUDA_OK(cudaEventCreateWithFlags(&h->inputs_ready, cudaEventDisableTiming));
  // Slabs only for compact tensors, outputs worth pipelining (>= 32 MB) and plans that do not slice K.
  const bool compact = !p->custom_strides[0] && !p->custom_strides[1] && !p->custom_strides[2];
  const TcExpr& e = p->expr;
  if (!compact || e.out_idx.empty() || p->count_c * (int64_t)es < (32 << 20) || p->args.ksplit > 1) return TC_OK;
  const std::string& name = e.out_idx.back();
  int cut = -1;
  for (size_t j = 0; j < p->idx_names.size(); ++j)
    if (p->idx_names[j] == name) cut = (int)j;
  const int64_t extent = p->idx_extent[cut];
  if (extent < 4) return TC_OK;
  const int64_t nslabs = std::min<int64_t>(extent, 12);
  h->slab = (extent + nslabs - 1) / nslabs;
  h->extent = extent;
  h->step[0] = h->view[0] = p->count_c / extent;
  if (!e.left_idx.empty() && e.left_idx.back() == name) h->step[1] = p->count_a / extent;
  if (!e.right_idx.empty() && e.right_idx.back() == name) h->step[2] = p->count_b / extent;
  const std::vector<std::string>* in_idx[2] = {&e.left_idx, &e.right_idx};
  for (int t = 0; t < 2; ++t) {
    int64_t acc = 1;
    for (const std::string& n : *in_idx[t]) {
      if (n == name) h->view[t + 1] = acc;
      for (size_t j = 0; j < p->idx_names.size(); ++j)
        if (p->idx_names[j] == n) acc *= p->idx_extent[j];
    }
  }
  int st = make_slab_plan(p, cut, h->slab, &h->plan_slab);
  if (st != TC_OK) return st;
  if (extent % h->slab) {
    st = make_slab_plan(p, cut, extent % h->slab, &h->plan_tail);
    if (st != TC_OK) return st;
  }
  if (h->plan_slab->args.ksplit > 1 || (h->plan_tail && h->plan_tail->args.ksplit > 1)) return TC_OK;  // keep one stream
  h->cut = cut;
  return TC_OK;
}

extern "C" int tc_execute_host(tc_plan* p, void* C, const void* A, const void* B) {
  if (!p || !C || !A || !B) return TC_ERR_INVALID_ARG;
  if (!p->committed) {
    const int st = tc_plan_commit(p);
    if (st != TC_OK) return st;
  }
  int dev = 0;
  TC_CUDA_OK(cudaGetDevice(&dev));
  if (dev != p->device) return TC_ERR_STATE;
  if (!p->host) {
    const int st = host_pipe_create(p);
    if (st != TC_OK) { host_pipe_destroy(p->host); p->host = nullptr; return st; }
  }
  TcHostPipe* h = p->host;
  const size_t es = p->dtype == TC_F64 ? 8 : 4;
  char* hC = static_cast<char*>(C);
  const char* hA = static_cast<const char*>(A);
  const char* hB = static_cast<const char*>(B);
  char *dC = static_cast<char*>(h->dC), *dA = static_cast<char*>(h->dA), *dB = static_cast<char*>(h->dB);
  const bool read_c = p->args.beta || p->size_c != p->count_c;
  cudaStream_t s0 = h->stream[0];
  if (h->cut < 0) {  // one piece
    TC_CUDA_OK(cudaMemcpyAsync(dA, hA, p->size_a * es, cudaMemcpyHostToDevice, s0));
    TC_CUDA_OK(cudaMemcpyAsync(dB, hB, p->size_b * es, cudaMemcpyHostToDevice, s0));
    if (read_c) TC_CUDA_OK(cudaMemcpyAsync(dC, hC, p->size_c * es, cudaMemcpyHostToDevice, s0));
    const int st = execute_impl(p, dC, dA, dB, p->d_ws, p->ws_bytes, s0);
    if (st != TC_OK) return st;
    TC_CUDA_OK(cudaMemcpyAsync(hC, dC, p->size_c * es, cudaMemcpyDeviceToHost, s0));
    TC_CUDA_OK(cudaStreamSynchronize(s0));
    return TC_OK;
  }
  // inputs that are not sliced go first, whole
  if (!h->step[1]) TC_CUDA_OK(cudaMemcpyAsync(dA, hA, p->size_a * es, cudaMemcpyHostToDevice, s0));
  if (!h->step[2]) TC_CUDA_OK(cudaMemcpyAsync(dB, hB, p->size_b * es, cudaMemcpyHostToDevice, s0));
  TC_CUDA_OK(cudaEventRecord(h->inputs_ready, s0));
  int i = 0;
  for (int64_t v = 0; v < h->extent; v += h->slab, ++i) {
    const int64_t n = std::min(h->slab, h->extent - v);
    tc_plan* q = n == h->slab ? h->plan_slab : h->plan_tail;
    cudaStream_t s = h->stream[i & 1];
    const size_t oc = (size_t)(v * h->step[0]) * es, oa = (size_t)(v * h->step[1]) * es, ob = (size_t)(v * h->step[2]) * es;
    if (read_c) TC_CUDA_OK(cudaMemcpyAsync(dC + oc, hC + oc, (size_t)(n * h->step[0]) * es, cudaMemcpyHostToDevice, s));
    if (h->step[1]) TC_CUDA_OK(cudaMemcpyAsync(dA + oa, hA + oa, (size_t)(n * h->step[1]) * es, cudaMemcpyHostToDevice, s));
    if (h->step[2]) TC_CUDA_OK(cudaMemcpyAsync(dB + ob, hB + ob, (size_t)(n * h->step[2]) * es, cudaMemcpyHostToDevice, s));
    if (s != s0) TC_CUDA_OK(cudaStreamWaitEvent(s, h->inputs_ready, 0));
    const int st = execute_impl(q, dC + oc, dA + (size_t)(v * h->view[1]) * es, dB + (size_t)(v * h->view[2]) * es, q->d_ws,
                                q->ws_bytes, s);
    if (st != TC_OK) return st;
    TC_CUDA_OK(cudaMemcpyAsync(hC + oc, dC + oc, (size_t)(n * h->step[0]) * es, cudaMemcpyDeviceToHost, s));
  }
  TC_CUDA_OK(cudaStreamSynchronize(h->stream[0]));
  TC_CUDA_OK(cudaStreamSynchronize(h->stream[1]));
  return TC_OK;
}

// ------------------------------------------- drop-in for sd_t_d2_fusion_ ----
#include <map>
#include <mutex>
extern "C" int tc_sd_t_d2_fusion(const char* expr, int dtype, int n_sizes, const int* sizes, void* t3, const void* t2,
                                 const void* v2) {
  if (!expr || !sizes || !t3 || !t2 || !v2 || n_sizes < 0) return TC_ERR_INVALID_ARG;
  static std::mutex mu;
  static std::map<std::string, tc_plan*> cache;  // plans live for the process, like the generated code's statics
  std::string key = std::string(expr) + "|" + std::to_string(dtype);
  for (int i = 0; i < n_sizes; ++i) key += "," + std::to_string(sizes[i]);
  tc_plan* plan = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) plan = it->second;
  }
  if (!plan) {
    int st = tc_plan_create(expr, dtype, nullptr, &plan);
    if (st != TC_OK) return st;
    std::vector<int64_t> ext(sizes, sizes + n_sizes);
    st = tc_plan_set_extents_ordered(plan, n_sizes, ext.data());
    if (st == TC_OK) st = tc_plan_commit(plan);
    if (st != TC_OK) { tc_plan_destroy(plan); return st; }
    std::lock_guard<std::mutex> lock(mu);
    auto ins = cache.emplace(key, plan);
    if (!ins.second) { tc_plan_destroy(plan); plan = ins.first->second; }
  }
  return tc_execute_host(plan, t3, t2, v2);
}

// -------------------------------------------------------- seeded inputs ----
namespace {

__host__ __device__ inline uint64_t splitmix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

template <typename T>
__global__ void fill_kernel(T* dst, int64_t count, uint64_t key, int64_t first) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < count; i += stride) {
    const uint64_t x = splitmix64(key ^ (uint64_t)(first + i));
    if constexpr (sizeof(T) == 8) dst[i] = (double)(x >> 11) * (1.0 / 9007199254740992.0) * 2.0 - 1.0;
    else dst[i] = (float)(x >> 40) * (1.0f / 16777216.0f) * 2.0f - 1.0f;
  }
}

template <typename T>
__global__ void axpy_kernel(T* y, const T* x, int64_t count, T alpha) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < count; i += stride) y[i] += alpha * x[i];
}

int grid_for(int64_t count) {
  int64_t g = (count + 255) / 256;
  return (int)std::max<int64_t>(1, std::min<int64_t>(g, 148 * 16));
}

}  // namespace

extern "C" int tc_fill_uniform(void* dst, int64_t count, int dtype, uint64_t seed, int tensor_id, int64_t first_index,
                               void* stream) {
  if (!dst || count < 0 || tensor_id < 0 || tensor_id > 15 || (dtype != TC_F64 && dtype != TC_F32)) return TC_ERR_INVALID_ARG;
  if (count == 0) return TC_OK;
  const uint64_t key = (seed * 0x9E3779B97F4A7C15ull) ^ ((uint64_t)tensor_id << 60);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == TC_F64) fill_kernel<double><<<grid_for(count), 256, 0, s>>>(static_cast<double*>(dst), count, key, first_index);
  else fill_kernel<float><<<grid_for(count), 256, 0, s>>>(static_cast<float*>(dst), count, key, first_index);
  TC_CUDA_OK(cudaGetLastError());
  return TC_OK;
}

extern "C" int tc_axpy(void* y, const void* x, int64_t count, int dtype, double alpha, void* stream) {
  if (!y || !x || count < 0 || (dtype != TC_F64 && dtype != TC_F32)) return TC_ERR_INVALID_ARG;
  if (count == 0) return TC_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == TC_F64) axpy_kernel<double><<<grid_for(count), 256, 0, s>>>(static_cast<double*>(y), static_cast<const double*>(x), count, alpha);
  else axpy_kernel<float><<<grid_for(count), 256, 0, s>>>(static_cast<float*>(y), static_cast<const float*>(x), count, (float)alpha);
  TC_CUDA_OK(cudaGetLastError());
  return TC_OK;
}
