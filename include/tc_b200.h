/*
 * tc_b200.h -- C ABI of the B200 tensor-contraction engine.
 *
 * One binary contraction  C[ext...] (+=|-=|=) sum(int...) A[...] * B[...]  on
 * column-major (first index fastest) tensors, described by COGENT's one-line
 * expression grammar.  The reference turns such a line into a generated .cu
 * file whose only entry is
 *     extern "C" void sd_t_d2_fusion_(int size_<idx>..., T* t3, T* t2, T* v2,
 *                                     int cond_kernel_1, int opt_register_transpose)
 * (emitted by cogent/src/codes/kernels/tc_interface.py:1444-1598); this header
 * replaces that generate-compile-link cycle with plan / execute / free calls.
 *
 * Plain pointers and sizes only.  All functions return a tc_status (0 = ok) and
 * never throw, exit or print.  The library has no CPU compute path: when no
 * CUDA device is usable every compute call returns TC_ERR_CUDA.
 */
#ifndef TC_B200_H_
#define TC_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum tc_status {
  TC_OK = 0,
  TC_ERR_PARSE = 1,        /* expression rejected by the grammar                       */
  TC_ERR_INVALID_ARG = 2,  /* null pointer, unknown index name, bad enum value         */
  TC_ERR_UNSUPPORTED = 3,  /* well-formed but outside the engine's limits              */
  TC_ERR_EXTENT = 4,       /* extent <= 0, or layouts that make output elements alias  */
  TC_ERR_CUDA = 5,         /* a CUDA runtime call failed (tc_last_cuda_error has it)   */
  TC_ERR_ALIGNMENT = 6,    /* a tensor base pointer is not aligned to its element size */
  TC_ERR_STATE = 7,        /* call order violated (e.g. changing a committed plan)     */
  TC_ERR_WORKSPACE = 8,    /* workspace too small or missing                           */
  TC_ERR_DEVICE_WAIT = 9   /* a bounded wait inside a kernel gave up: the output of that
                              execute is invalid (tc_plan_status has the wait's code)  */
} tc_status;

typedef enum tc_dtype { TC_F64 = 0, TC_F32 = 1 } tc_dtype;

/* Arithmetic path.  AUTO picks per dtype what measured fastest on B200. */
typedef enum tc_path {
  TC_PATH_AUTO = 0,
  TC_PATH_DMMA = 1,  /* fp64 on the tensor pipe (mma.sync f64)     */
  TC_PATH_DFMA = 2,  /* fp64 on the vector pipe                    */
  TC_PATH_FFMA = 3,  /* fp32 on the vector pipe                    */
  TC_PATH_3XTF32 = 4, /* fp32 as three TF32 tensor-core products (mma.sync), fp32 accumulate */
  TC_PATH_TCGEN05 = 5 /* the same three products issued as tcgen05.mma with the accumulators in tensor memory;
                         problems too small for its 128-wide tiles run on TC_PATH_3XTF32 */
} tc_path;

typedef struct tc_options {
  int path;       /* tc_path                                                          */
  int tile_m;     /* 0 = planner's choice; otherwise force the CTA tile (must be one  */
  int tile_n;     /*     of the compiled shapes, see tc_plan_describe)                */
  int split_k;    /* 0 = planner's choice, 1 = never split, >1 = that many K slices   */
  int variant;    /* 0 = planner's choice; otherwise 1-based warp layout of the tile  */
  int l2_prefetch; /* output tiles are prefetched into L2 ahead of their read-modify-write:  */
                   /*   0 = planner's choice, 1 = off, 2 = on                                */
  int c_path;      /* how `+=`/`-=` reach the output: 0 = planner's choice, 1 = read-modify- */
                   /*   write in the epilogue, 2 = accumulators start from the output,       */
                   /*   3 = bulk asynchronous reduce-add from shared memory (persistent      */
                   /*   kernels, rows contiguous in the output; falls back to 1 elsewhere).  */
                   /*   The persistent fp32 kernel stages its tile in shared memory either   */
                   /*   way: 0 and 3 send it as reduce-adds, 1 fetches the old values and    */
                   /*   stores the sums, 2 runs the tiles one CTA per tile instead.          */
  int tma;         /* tiled TMA copies in the persistent kernels (operand tiles that are plain 2-D boxes, fp64 and
                      fp32; fp64 output batches that are boxes of a rank-5 view of C): 0 = both, 1 = neither,
                      2 = operands only, 3 = output only, 4 = both but the output per warp, never per tile */
  int test_fault;  /* tests only, 0 in production.  1: the persistent fp64 kernel's producers leave one stage
                      unannounced and every device-side wait gives up after 2^14 polls instead of 2^24, so the
                      give-up path (status word, TC_ERR_DEVICE_WAIT) can be exercised without a long stall */
} tc_options;

typedef struct tc_plan tc_plan;

/* ---- expression front end -------------------------------------------------
 * Same whitespace-sensitive grammar as the reference parser
 * (cogent/src/algs/bases/tc_gen_inputs.py:28-108): after '[', ']' and ';' are
 * removed the line must split on blanks into
 *   name  idx,ext,idx,ext..  (+=|-=|=)  sum(idx,ext,..)  *  name  idx,..  *  name  idx,..
 * Index names may be any length; tensor names are free.
 *
 * tc_expr_describe writes a JSON description of the parsed line into buf
 * (always NUL terminated, truncated to cap) and returns TC_OK or TC_ERR_PARSE.
 * It needs no GPU. */
int tc_expr_describe(const char* expr, char* buf, size_t cap);

/* ---- plan -----------------------------------------------------------------
 * Replaces running tc_code_generator.py + nvcc on one expression
 * (cogent/tc_code_generator.py:13-60).  The extents written in the expression
 * are the defaults; tc_plan_set_extents overrides them by index name, as the
 * reference drivers do from argv (cogent/drivers/tccg/code_main_tccg_02.c:32-38). */
int tc_plan_create(const char* expr, int dtype, const tc_options* options, tc_plan** out);
int tc_plan_set_extents(tc_plan* plan, int n, const char* const* index_names, const int64_t* extents);

/* Extents by position: output indices in written order, then the contraction indices in sum(...)
 * order -- the order of the size arguments of the reference entry sd_t_d2_fusion_
 * (cogent/src/codes/kernels/tc_interface.py:1451-1516). */
int tc_plan_set_extents_ordered(tc_plan* plan, int n, const int64_t* extents);

/* Optional strided views.  tensor: 0 = output, 1 = left input, 2 = right input.
 * strides[i] is the element stride of the tensor's i-th index as written in the
 * expression.  Default: compact column-major from the current extents.  Used to
 * run one slab of a larger tensor (sharding an external or a contraction index
 * across GPUs) without copying. */
int tc_plan_set_strides(tc_plan* plan, int tensor, int n, const int64_t* strides);

/* Freezes extents/strides, chooses the tiling for the current device, uploads
 * the plan's tables.  Implied by the first execute.  After it the plan is
 * immutable and may be executed from several threads/streams at once. */
int tc_plan_commit(tc_plan* plan);

void tc_plan_destroy(tc_plan* plan);

/* JSON: index classes, fused dimensions, tile shape, kernel variant, grid,
 * algorithmic flops and bytes. */
int tc_plan_describe(const tc_plan* plan, char* buf, size_t cap);
/* 2 * prod(all extents), and elemsize * (2|C| + |A| + |B|)  ('=' reads C zero times: |C|). */
int tc_plan_cost(const tc_plan* plan, double* flops, double* bytes);
/* Kernel launches one tc_execute enqueues. */
int tc_plan_launches(const tc_plan* plan);
/* Synchronises the whole device (cudaDeviceSynchronize, so work on non-blocking streams is covered too)
 * and reads this plan's status word: 0 = every kernel of the plan ran to completion; non-zero = the code
 * of the first bounded wait inside a kernel that gave up (the output of that execute is invalid).  The
 * word is sticky until tc_plan_status_reset.  No counterpart in the reference. */
int tc_plan_status(tc_plan* plan, int* device_status);
int tc_plan_status_reset(tc_plan* plan);
/* Bytes of caller-provided workspace tc_execute_ws needs (0 when the plan does not split K). */
int tc_plan_workspace_bytes(const tc_plan* plan, size_t* bytes);

/* ---- execute --------------------------------------------------------------
 * Replaces the generated host wrapper sd_t_d2_fusion (kernel launch part,
 * cogent/src/codes/kernels/tc_interface.py:284-362,1147-1352).  Pointers are
 * DEVICE pointers to the first element of each tensor; the call only enqueues
 * work on `stream` (a cudaStream_t, 0 = default stream) and never allocates.
 * The output must not alias an input.  True accumulate semantics: C += sum
 * (the reference's generated kernel overwrites C and relies on the driver
 * having zeroed it; its CPU check accumulates, which is what this does). */
int tc_execute(tc_plan* plan, void* C, const void* A, const void* B, void* stream);
/* Same with an explicit workspace (plans with split K use the plan-owned
 * workspace in tc_execute; concurrent executes of such a plan must each bring
 * their own through this call). */
int tc_execute_ws(tc_plan* plan, void* C, const void* A, const void* B, void* workspace,
                  size_t workspace_bytes, void* stream);

/* No counterpart in the reference.  tc_execute for callers that can neither allocate device memory
 * when they call nor spare any for a workspace: programs whose own memory pool already owns the
 * device, and latency-critical loops that cannot take cudaMalloc's device-wide synchronisation.
 * The scratch of K-sliced plans comes from a fixed array inside the library image
 * (TC_NOALLOC_MAX_WORKSPACE_BYTES, held by every GPU that loads the library until exit); the call
 * itself never allocates or frees.  The plan must already be committed (TC_ERR_STATE otherwise);
 * plans needing more scratch than the array return TC_ERR_WORKSPACE.  tc_plan_commit of a K-sliced plan
 * resolves the array's device address and loads the kernels of the combine step, so that nothing is
 * loaded or looked up at call time; should a plan committed by an older code path lack the address,
 * the first call on that device resolves it, so issue one call before any stream capture.  Calls on
 * one device share the array, so calls whose kernels may overlap on the GPU must be serialised by the
 * caller. */
#define TC_NOALLOC_MAX_WORKSPACE_BYTES (8u << 20)
int tc_execute_noalloc(tc_plan* plan, void* C, const void* A, const void* B, void* stream);

/* Blocking convenience over HOST pointers: allocate, copy in (C too), run,
 * copy C back, free -- what the reference's sd_t_d2_fusion does around its
 * kernel (cogent/src/codes/others/tc_pre_CUDA_Malloc.py:6-47,
 * cogent/src/codes/kernels/tc_interface.py:1368-1388).  The output's slowest index is cut into slabs
 * that are pipelined over two streams.  Pinned (page-locked) host buffers are copied from directly;
 * pageable ones (plain malloc, what the reference drivers pass) travel through two plan-owned pinned
 * bounce buffers per direction.  Calls on one plan are serialised by a lock inside the plan (they share
 * its device buffers); use one plan per thread to run them concurrently.  Returns TC_ERR_DEVICE_WAIT
 * when a kernel of the call reported a wait that gave up. */
int tc_execute_host(tc_plan* plan, void* C, const void* A, const void* B);

/* ---- several contractions into one output ----------------------------------------------
 * n expression lines that accumulate (+= / -=) into the SAME output tensor -- same name, same indices in the same
 * order -- each with its own two inputs and its own assignment of the output's indices to them: the CCSD(T)
 * triples terms (cogent/input_strings/ccsd_t/original-expressions/sd_t_d2.in:4-30; checker
 * cogent/drivers/ccsd_t/code_main_sd2_1.c:561-613).  The reference meant to fuse such terms in one kernel but only
 * stubbed it (cogent/src/codes/kernels/tc_code_kernel_fusion.py:6-205).  Here one kernel keeps a box of the output in
 * shared memory, runs every term's product for that box on the FP64 tensor pipe and adds the box to C once: the
 * output is read and written once instead of n times.  fp64; at most 16 terms; every input of a term may carry at
 * most as many output indices as fit 64 rows of a box (TC_ERR_UNSUPPORTED otherwise).  Extents written in the
 * first line are the defaults; index names are shared by all lines.
 * A[k], B[k]: device pointers to the left / right input of term k (compact column-major). */
typedef struct tc_fused_plan tc_fused_plan;
int tc_plan_create_fused(int n, const char* const* exprs, int dtype, tc_fused_plan** out);
int tc_fused_set_extents(tc_fused_plan* plan, int n, const char* const* index_names, const int64_t* extents);
int tc_fused_commit(tc_fused_plan* plan);
/* JSON: box shape, boxes, rows x cols per term, flops, bytes moved fused and term by term. */
int tc_fused_describe(tc_fused_plan* plan, char* buf, size_t cap);
int tc_execute_fused(tc_fused_plan* plan, void* C, const void* const* A, const void* const* B, void* stream);
void tc_fused_destroy(tc_fused_plan* plan);

/* ---- one contraction over several GPUs from one process ----------------------------------
 * One plan, one stream and (contraction kind) one NCCL communicator per device; the calling thread drives all
 * devices.  The reference is single-GPU (nwchem-tccg/tccg_kernels.cu:228 is the only stream it creates), so
 * nothing there is replaced; the geometry is the one cgo2019-ae_b200/shard.py uses with one process per GPU.
 *   TC_SHARD_EXTERNAL     an output index (`index`, NULL = the largest, ties to the slowest) is cut into contiguous
 *                         ranges, one per device: no communication.
 *   TC_SHARD_CONTRACTION  a contraction index (NULL = the largest) is cut: every device writes a full-size partial
 *                         result into scratch the plan owns, one reduce-scatter (NCCL, found at run time as
 *                         libnccl.so.2; TC_ERR_UNSUPPORTED at commit if absent) sums them, and device d adds chunk d
 *                         (ceil(|C| / n_devices) elements) into chunk d of its output.
 * device_ids NULL means 0 .. n_devices - 1.  tc_sharded_describe works before commit and without a GPU (JSON:
 * kind, index, per-device range, element offsets of the device's views, local expression, chunk).
 * tc_execute_sharded: C[d], A[d], B[d] are pointers in device d's memory to the FULL tensors (compact, column-
 * major); with TC_SHARD_C_IS_SLAB (external kind, cut along the output's slowest index) C[d] is only device d's
 * contiguous slab.  The call is asynchronous on the plan's streams; tc_sharded_synchronize waits for all of them and
 * returns TC_ERR_DEVICE_WAIT if a kernel reported a wait that gave up. */
#define TC_SHARD_EXTERNAL 0
#define TC_SHARD_CONTRACTION 1
#define TC_SHARD_C_IS_SLAB 1
typedef struct tc_sharded_plan tc_sharded_plan;
int tc_plan_create_sharded(const char* expr, int dtype, int n_devices, const int* device_ids, int kind,
                           const char* index, tc_sharded_plan** out);
int tc_sharded_set_extents(tc_sharded_plan* plan, int n, const char* const* index_names, const int64_t* extents);
int tc_sharded_describe(tc_sharded_plan* plan, char* buf, size_t cap);
int tc_sharded_commit(tc_sharded_plan* plan);
int tc_execute_sharded(tc_sharded_plan* plan, void* const* C, const void* const* A, const void* const* B, int flags);
int tc_sharded_synchronize(tc_sharded_plan* plan);
void tc_sharded_destroy(tc_sharded_plan* plan);

/* ---- drop-in for the reference's generated entry ------------------------------------
 * What the generated sd_t_d2_fusion_ does for ONE expression (cogent/src/codes/kernels/tc_interface.py:
 * 1444-1598 -> 10-101): sizes in the order above, host pointers t3 (in/out), t2, v2; allocate, copy in,
 * contract, copy t3 back.  Plans are cached per (expression, dtype, sizes).  include/tc_b200_shim.h
 * wraps this into a symbol with the reference's exact name and argument list. */
int tc_sd_t_d2_fusion(const char* expr, int dtype, int n_sizes, const int* sizes, void* t3, const void* t2,
                      const void* v2);

/* ---- diagnostics ------------------------------------------------------------ */
const char* tc_status_string(int status);
/* Last CUDA error text seen by the calling thread inside this library. */
const char* tc_last_cuda_error(void);
const char* tc_version(void);

/* ---- seeded inputs ------------------------------------------------------------
 * Counter-based uniform[-1,1) generator shared by tests, bench and shards:
 * element i of tensor `tensor_id` (0 = C, 1 = A, 2 = B) is a pure function of
 * (seed, tensor_id, first_index + i), so any slab can be produced in place on
 * any GPU.  dst is a device pointer to `count` elements. */
int tc_fill_uniform(void* dst, int64_t count, int dtype, uint64_t seed, int tensor_id,
                    int64_t first_index, void* stream);
/* y[i] += alpha * x[i] on device (combines reduce-scattered partial sums into C). */
int tc_axpy(void* y, const void* x, int64_t count, int dtype, double alpha, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TC_B200_H_ */
