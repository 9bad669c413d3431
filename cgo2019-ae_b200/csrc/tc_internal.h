// Internal declarations shared by the parser, the planner, the kernels and the C ABI.
#ifndef TC_INTERNAL_H_
#define TC_INTERNAL_H_

#include <stdint.h>
#include <stddef.h>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/tc_b200.h"

#ifdef __CUDACC__
#include <cuda_runtime.h>
#endif

// ---------------------------------------------------------------- errors ----
void tc_note_cuda_error(int code, const char* what);  // stores text for tc_last_cuda_error()

#define TC_CUDA_OK(call)                                   \
  do {                                                     \
    cudaError_t tc_e_ = (call);                            \
    if (tc_e_ != cudaSuccess) {                            \
      tc_note_cuda_error((int)tc_e_, #call);               \
      return TC_ERR_CUDA;                                  \
    }                                                      \
  } while (0)

// ------------------------------------------------------------ expression ----
// One parsed line of the contraction grammar
// (reference: cogent/src/algs/bases/tc_gen_inputs.py:28-108).
struct TcExpr {
  std::string out_name, left_name, right_name;
  std::vector<std::string> out_idx;    // output indices, first = fastest
  std::vector<std::string> sum_idx;    // contraction indices in sum(...) order
  std::vector<std::string> left_idx;   // left input's indices, first = fastest
  std::vector<std::string> right_idx;  // right input's indices
  std::vector<int64_t> out_ext;        // extents written next to out_idx
  std::vector<int64_t> sum_ext;        // extents written inside sum(...)
  int op = 0;                          // +1 for "+=", -1 for "-=", 0 for "="
};

// Returns TC_OK / TC_ERR_PARSE / TC_ERR_UNSUPPORTED; `why` gets a one-line reason.
int tc_parse_expr(const char* line, TcExpr* out, std::string* why);
std::string tc_expr_to_json(const TcExpr& e);

// ------------------------------------------------------------------ plan ----
constexpr int TC_MAX_DIMS = 8;  // fused dimensions per index class
constexpr int TC_DEFAULT_SMS = 148;   // B200; only used to describe a plan before a device is known
constexpr uint32_t TC_SPIN_LIMIT = 1u << 24;
constexpr int TC_TF32_CHAIN = 512;    // longest fp32 accumulation chain the tensor-core paths may run

// One index class (rows of the left operand, rows of the right operand) as a
// mixed-radix number: dimension 0 is the fastest digit of the flattened index.
struct TcDims {
  int32_t n;
  uint32_t extent[TC_MAX_DIMS];
  int64_t s_in[TC_MAX_DIMS];   // element stride in the input that carries the class
  int64_t s_out[TC_MAX_DIMS];  // element stride in the output
};

// Opaque storage of a CUtensorMap (128 bytes, 64-byte aligned), so host-only sources need no CUDA headers.
struct alignas(64) TcTensorMap { uint64_t opaque[16]; };

// The output seen as a tensor of rank <= 5 for tiled TMA copies: dimension 0 is the contiguous run of the
// fastest M dimensions (fused as far as they are contiguous in C), dimensions 1 and 2 the parity of n and
// n / 2 inside N's fastest dimensions (fused likewise), then `ne` further N dimensions and `me` further M
// dimensions (ne + me <= 2).
struct TcOutMap {
  uint32_t e0, f0;     // extents of the fused fastest M / N dimensions
  int32_t ne, me;      // slower dimensions of N / M that follow
  uint32_t ext[2];     // their extents, N's first
  int64_t stride_n;    // element stride of n inside f0
  int64_t stride[2];   // element strides of ext[]
};

// Everything a kernel launch needs besides the three tensor pointers.
// "M" is the external class of operand X (the one holding the output's fastest
// index after the planner's optional operand swap), "N" the class of operand Y.
struct TcKernelArgs {
  TcDims M, N;
  uint32_t Mflat, Nflat, Kflat;
  uint32_t tiles_m, tiles_n;
  uint32_t mblock_w;  // persistent kernels walk the tiles in column blocks of this many M tiles (0: M fastest over all of M)
  int32_t bm, bn;    // CTA tile of the chosen kernel
  int32_t c_mode;    // 0: read-modify-write epilogue, 1: accumulators start from C,
                     // 2: bulk asynchronous reduce-add from shared memory (persistent kernels)
  int32_t c_stream;  // cache-streaming hints on accesses to C
  uint32_t prefetch_dist;  // blocks ahead whose output tile is prefetched into L2 (0 = off)
  uint32_t k_chunk;  // flattened contraction range per K slice (multiple of the K step)
  uint32_t ksplit;   // number of K slices (1 = the kernel applies the result to C itself)
  uint32_t k_first;  // first flattened contraction index of this launch (plans that run K in sequential passes)
  uint32_t spin_limit;  // polls a bounded wait may take before it gives up
  int32_t test_fault;   // tests only: 1 = the persistent kernel's producers leave one stage unannounced
  int32_t out_bufs, img_sets, ring_stages;  // persistent tcgen05 kernel: how its shared memory is carved (set at launch)
  const int64_t* koff_x;  // [Kflat] offset of flattened contraction index k inside X
  const int64_t* koff_y;  // [Kflat] the same inside Y
  int32_t lanes_k_x;  // element-wise loader: consecutive lanes that walk k (1 = lanes walk the external index)
  int32_t lanes_k_y;
  int32_t vec_c;     // contiguous output elements a thread may touch with one access (1, 2 or 4)
  int32_t beta;      // 1: C is read and accumulated into; 0: C is overwritten
  double alpha;      // +1 or -1
  void* ws;          // K-slice partials: [ksplit][tiles][BN][BM]
  int32_t epi_run;       // staged bulk epilogue: run length E0 in elements (0 = not available)
  int32_t epi_n_span;    // ... F0 > 0: consecutive n are adjacent in the output within blocks of F0 (0: never)
  TcTensorMap tmap_x, tmap_y;  // tiled TMA descriptors of X / Y as 2-D (k, flattened external) tensors, when used
  int32_t c_tensor;      // persistent kernels: output leaves as tiled TMA reduce/store boxes: 1 = one box per
                         // consumer warp and batch of 8 rows (tmap_c), 2 = one box per tile (tmap_ct) where the
                         // kernel has room to stage a whole tile, else as 1
  TcOutMap cmap;         // ... the view of C they are boxes of
  TcTensorMap tmap_c;    // its rank-5 descriptor with box (warp rows, 1, 8, 1, 1)
  TcTensorMap tmap_ct;   // the same tensor with box (bm, 2, bn / 2, 1, 1)
  int* status;       // device word: 0, or the code of a wait that ran out of polls (persistent kernels)
};

enum TcMath { TC_MATH_DMMA = 0, TC_MATH_SIMT = 1, TC_MATH_TF32X3 = 2, TC_MATH_TF32TC = 3 };

struct TcKernelChoice {
  int dtype;      // tc_dtype
  int math;       // TcMath
  int bm, bn;     // CTA tile
  int variant;    // warp layout of the tile (0-based)
  bool vec_x, vec_y;    // 16-byte loads along the external index of X / Y are legal
  bool kvec_x, kvec_y;  // 16-byte loads along the contraction index of X / Y are legal
  bool tma_x, tma_y;    // X / Y is a plain 2-D (k fastest, flattened external) matrix: tiles are TMA boxes
  bool tma_xe, tma_ye;  // ... with the flattened external index fastest and k at a constant pitch (fp32 persistent kernel)
  bool tma_c;           // a warp's 8-row output batch is a box of a rank-5 tensor over C
  bool tma_ct;          // ... and so is a whole bm x bn tile
};

struct TcHostPipe;

// Host-side plan.
struct tc_plan {
  TcExpr expr;
  int dtype = TC_F64;
  tc_options opt{};
  // current extents by index name (out_idx then sum_idx order)
  std::vector<std::string> idx_names;
  std::vector<int64_t> idx_extent;
  bool custom_strides[3] = {false, false, false};
  std::vector<int64_t> strides[3];  // per tensor, per written index

  // ---- filled by commit ----
  bool committed = false;
  int device = -1;
  bool swapped = false;  // X = right input, Y = left input
  TcKernelArgs args{};
  TcDims kdims{};  // the contraction class (s_in: stride in X, s_out: stride in Y); the kernels see it as offset tables
  TcKernelChoice choice{};
  std::vector<int64_t> h_koff_x, h_koff_y;
  void* d_koff = nullptr;      // device copy of both tables
  void* d_ws = nullptr;        // plan-owned K-slice workspace
  int* d_status = nullptr;     // device status word
  struct TcHostPipe* host = nullptr;  // device buffers, streams and slab plans of the host-pointer path
  size_t ws_bytes = 0;
  int sm_count = TC_DEFAULT_SMS;  // multiprocessors of the device the plan is committed on
  int passes = 1;   // sequential launches over consecutive contraction ranges, each accumulating into C
  std::mutex* host_mu = nullptr;  // serialises tc_execute_host on this plan (its device buffers are shared)
  int64_t size_c = 0, size_a = 0, size_b = 0;  // elements spanned (max offset + 1)
  int64_t count_c = 0, count_a = 0, count_b = 0;  // logical element counts
  double flops = 0, bytes = 0;
  double estimate_s = 0;  // the planner's own estimate of one execute (persistent fp64 kernels; 0: none made)
  int launches = 1;
  std::string why;  // last planner message
};

int tc_plan_build(tc_plan* p, std::string* why);           // host-only part of commit
std::string tc_plan_to_json(const tc_plan& p);

// ------------------------------------------------------------- kernels ----
#ifdef __CUDACC__
// Enqueues the contraction (and, for K-sliced plans, the combine step).
int tc_launch_contraction(const tc_plan& p, const TcKernelArgs& args, void* C, const void* X,
                          const void* Y, cudaStream_t stream);
// Shared memory bytes / threads of the chosen kernel (for tc_plan_describe).
int tc_kernel_shape(const TcKernelChoice& c, int* threads, int* smem_bytes, int* bk);
int tc_kernels_prepare(const TcKernelChoice& c);  // opt-in shared memory attribute
#endif

// Compiled kernels (registry built from tc_kernel_list.h).
bool tc_kernel_exists(int dtype, int math, int bm, int bn, int variant);
const char* tc_kernel_name(const TcKernelChoice& c);
// fp32 on tcgen05 with the output tile resident in shared memory (tc_wt_kernel.cuh)
inline bool tc_kernel_is_tmem_persistent(const TcKernelChoice& c) { return c.math == TC_MATH_TF32TC && c.variant == 1; }
inline bool tc_kernel_is_persistent(const TcKernelChoice& c) {
  return (c.math == TC_MATH_DMMA && c.variant >= 2) || tc_kernel_is_tmem_persistent(c);
}
// ... and keeps its output tile resident in shared memory (tc_wc_kernel.cuh)
inline bool tc_kernel_is_c_resident(const TcKernelChoice& c) { return c.math == TC_MATH_DMMA && c.variant == 3; }
constexpr int TC_BK = 16;  // contraction step of every kernel

#endif  // TC_INTERNAL_H_
