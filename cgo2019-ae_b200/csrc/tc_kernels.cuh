// Contraction kernel template for sm_100a.
//
// One CTA computes a BM x BN tile of the FLATTENED external index spaces
// (M = external indices of operand X, N = external indices of operand Y) and
// walks the flattened contraction range in steps of BK.  It takes over the
// roles of the reference's generated kernel pieces:
//   * prologue / index decode   cogent/src/codes/kernels/tc_code_kernel.py:166-552
//   * permuted global->shared   cogent/src/codes/kernels/tc_code_kernel_load_inputs_abstract.py:32-317
//   * register-tile product     cogent/src/codes/kernels/tc_code_kernel_compute.py:4-204
//   * guarded store             cogent/src/codes/kernels/tc_code_kernel_store_output.py:6-89
// but not their structure: tiles are ranges of the flattened index (no partial
// tiles inside the tensor, whatever the extents), addresses are separable sums
// off_ext[m] + off_k[k] looked up from a per-CTA table in shared memory and a
// per-plan table in global memory, the staging is an asynchronous multi-stage
// cp.async pipeline, fp64 products run on the tensor pipe (DMMA m8n8k4), and the
// epilogue is a true read-modify-write with up to 32 contiguous bytes per thread.
//
// fp32 products run as three TF32 tensor-core products per product: on tcgen05.mma with the accumulators in
// tensor memory (TC_MATH_TF32TC, one elected thread issues, tcgen05.ld feeds the epilogue) or on mma.sync
// (TC_MATH_TF32X3); FFMA / DFMA kernels remain for comparison.
//
// Shared-memory image of both operands is "external-index major":
//   Xs[stage][k][m], row pitch BM+4; Ys[stage][k][n], row pitch BN+4.
// The pitch makes the 16-byte DMMA fragment reads, the 16-byte SIMT reads and
// the element-wise transposing writes all bank-conflict free.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "tc_internal.h"

namespace tck {

// ------------------------------------------------------------- primitives ----
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  const int sz = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src, bool pred) {
  const int sz = pred ? 8 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, bool pred) {
  const int sz = pred ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
template <int ES>
__device__ __forceinline__ void cp_async_elem(uint32_t dst, const void* src, bool pred) {
  if constexpr (ES == 8) cp_async8(dst, src, pred);
  else cp_async4(dst, src, pred);
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// ---- mbarriers (shared memory), every wait bounded ----

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.shared::cta.b64 st, [%0];\n}\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false (and *status = code) if the phase does not complete within `limit` polls.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  atomicCAS(status, 0, code);  // the first wait that gives up names the cause; the others follow from it
  return false;
}

// ---- tcgen05: tensor memory and the 5th-generation MMA (inline PTX, one CTA per MMA) ----
// Tensor-memory address: lane in bits [31:16], column in bits [15:0]; a column holds one 32-bit value per lane.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {  // one whole warp; cols a power of two >= 32
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {  // the warp that allocated
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// One arrival on `bar` once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void tc05_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A * B^T, A and B in shared memory behind matrix descriptors, TF32 inputs, fp32 accumulate.
__device__ __forceinline__ void tc05_mma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
      : "memory");
}
// The same with A in tensor memory: row i of A in lane i, one column per k (32-bit elements), from column `a_tmem` on.
__device__ __forceinline__ void tc05_mma_tf32_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
      : "memory");
}
// Four consecutive columns of this thread's lane (lane = 32 * (warp % 4) + lane id) from registers; asynchronous
// until tc05_wait_st().
__device__ __forceinline__ void tc05_st4(uint32_t taddr, const float4& v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(taddr), "r"(__float_as_uint(v.x)),
               "r"(__float_as_uint(v.y)), "r"(__float_as_uint(v.z)), "r"(__float_as_uint(v.w))
               : "memory");
}
__device__ __forceinline__ void tc05_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
// 16 consecutive columns of this thread's lane (lane = 32 * (warp % 4) + lane id) into registers.  The load is
// asynchronous: nothing may touch the destination registers (not even a move) before tc05_wait_ld(), so the
// values land directly in the caller's floats.
__device__ __forceinline__ void tc05_ld16(uint32_t taddr, float* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
      : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]), "=f"(v[8]),
        "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc05_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
// Shared-memory matrix descriptor, no swizzle, K-major: 16 bytes hold 4 consecutive k of one row (external), 8
// rows are contiguous (a 128-byte core matrix); `lbo` bytes lead to the next 4 k, `sbo` bytes to the next 8 rows.
// (The MN-major form without swizzle returned zeros for TF32 on B200; this form is exact.)
__device__ __forceinline__ uint64_t umma_desc_k(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) |
         (1ull << 46);
}
// Instruction descriptor of kind::tf32: fp32 accumulate, TF32 inputs, both operands K-major, D is m x n.
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int m, int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// v = hi + lo: hi is v rounded to TF32 (nearest, on the 13 dropped bits, as cvt.rna.tf32 does); lo = v - hi is exact
// in fp32 and is left as it is -- the tensor core reads its upper 19 bits, an error of at most 2^-21 |v|.
__device__ __forceinline__ void split_tf32_bits(float v, float& hi, float& lo) {
  hi = __uint_as_float((__float_as_uint(v) + 0x1000u) & 0xFFFFE000u);
  lo = v - hi;
}


// D(16x8) += A(16x8) * B(8x8), TF32 inputs, fp32 accumulate.
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// v = hi + lo with hi, lo representable in TF32 (10-bit mantissa): hi*hi' + hi*lo' + lo*hi' recovers the
// fp32 product to about 2^-21 relative.
__device__ __forceinline__ void split_tf32(float v, uint32_t& hi, uint32_t& lo) {
  asm("cvt.rna.tf32.f32 %0, %1;\n" : "=r"(hi) : "f"(v));
  const float r = v - __uint_as_float(hi);
  asm("cvt.rna.tf32.f32 %0, %1;\n" : "=r"(lo) : "f"(r));
}

__device__ __forceinline__ void dmma884(double& d0, double& d1, double a, double b) {
  asm("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};\n"
      : "+d"(d0), "+d"(d1)
      : "d"(a), "d"(b));
}

template <typename T> struct Vec16;
template <> struct Vec16<double> { using type = double2; static constexpr int W = 2; };
template <> struct Vec16<float> { using type = float4; static constexpr int W = 4; };

// ------------------------------------------------------------ configuration ----
template <typename T_, int MATH_, int BM_, int BN_, int WARPS_M_, int WARPS_N_, int STAGES_, int MINB_, bool VECX_, bool VECY_,
          bool KVX_ = false, bool KVY_ = false>
struct Cfg {
  using T = T_;
  static constexpr int MATH = MATH_;
  static constexpr int BM = BM_, BN = BN_, BK = 16;
  static constexpr int STAGES = STAGES_;
  static constexpr int MIN_CTAS = MINB_;
  static constexpr bool VECX = VECX_, VECY = VECY_;
  // tcgen05 path only: the operand's fastest index is the contracted one and is fetched 16 bytes at a time into a
  // contraction-major image [external][k], pitch BK + 4 (conflict-free 16-byte reads by consecutive rows)
  static constexpr bool KVX = KVX_, KVY = KVY_;
  static constexpr int LDKV = 16 + 4;
  static constexpr int ES = (int)sizeof(T);
  static constexpr int VW = 16 / ES;  // elements per 16 bytes
  // DMMA: WARPS_M x WARPS_N warps, each a (BM/WARPS_M) x (BN/WARPS_N) tile.
  // SIMT: (BM/8) x (BN/8) threads, each an 8 x 8 tile.
  static constexpr int THREADS = MATH == TC_MATH_SIMT ? (BM / 8) * (BN / 8) : 32 * WARPS_M_ * WARPS_N_;
  static constexpr int WARPS = THREADS / 32;
  static constexpr int WM = BM / WARPS_M_, WN = BN / WARPS_N_;
  static constexpr int WARPS_M = WARPS_M_, WARPS_N = WARPS_N_;
  // row pitch: +4 words keeps the fp64 / vector-pipe reads conflict-free, the TF32 fragment reads want +8
  static constexpr int PAD = MATH == TC_MATH_TF32X3 ? 8 : 4;
  static constexpr int LDX = BM + PAD, LDY = BN + PAD;
  // tcgen05 path: hi and lo TF32 images of both operands for one K step, in the layout the MMA's matrix
  // descriptors expect; one mbarrier and the tensor-memory address follow them.
  static constexpr bool TCGEN = MATH == TC_MATH_TF32TC;
  static constexpr int UMMA_ELEMS = TCGEN ? 2 * BK * (BM + BN) : 0;
  static constexpr int TMEM_COLS = BM <= 32 ? 32 : BM <= 64 ? 64 : BM <= 128 ? 128 : 256;
  // Contraction offsets of the stages in flight live in a shared ring (filled by
  // cp.async one pipeline depth ahead), so the loaders never wait on global memory.
  static constexpr int KRING = 2 * STAGES - 2;
  // + output offsets of the tile whose C is prefetched into L2 (BM + BN entries)
  static constexpr int TABLE_BYTES = (3 * BM + 3 * BN + KRING * 2 * BK) * 8;
  static constexpr int XIMG = KVX ? BM * LDKV : BK * LDX, YIMG = KVY ? BN * LDKV : BK * LDY;
  static constexpr int STAGE_ELEMS = XIMG + YIMG;
  static constexpr int SMEM_BYTES = TABLE_BYTES + (STAGES * STAGE_ELEMS + UMMA_ELEMS) * ES + (TCGEN ? 16 : 0);
  static_assert(!TCGEN || (BN == 128 && BM % 16 == 0 && BM <= 256 && sizeof(T) == 4 && WARPS_M_ * WARPS_N_ == 8),
                "tcgen05 path: D is BN (=128 lanes) x BM columns, eight warps");
};

// ------------------------------------------------------- offset tables ----
// Entry i of a class table: flattened index base+i decomposed over the class's
// dimensions; -1 marks "outside the tensor".
__device__ __forceinline__ void decode(const TcDims& d, uint32_t flat, uint32_t limit, int64_t* off_in, int64_t* off_out) {
  if (flat >= limit) { *off_in = -1; *off_out = -1; return; }
  if (d.n == 1) {  // one fused dimension: the flattened index is the coordinate
    *off_in = (int64_t)flat * d.s_in[0];
    *off_out = (int64_t)flat * d.s_out[0];
    return;
  }
  int64_t oi = 0, oo = 0;
#pragma unroll 1
  for (int i = 0; i < d.n; ++i) {
    const uint32_t q = flat / d.extent[i];
    const uint32_t c = flat - q * d.extent[i];
    flat = q;
    oi += (int64_t)c * d.s_in[i];
    oo += (int64_t)c * d.s_out[i];
  }
  *off_in = oi;
  *off_out = oo;
}

// Tile number -> tile coordinates for the persistent kernels.  Plain order: M fastest over all of M.  With
// mblock_w = w > 0 the tiles are walked in column blocks of w M tiles: inside a block M is fastest, then N, and a
// block is finished over all of N before the next begins.  The tiles in flight at any time (one per consumer group
// and SM, consecutive numbers) then share a handful of operand tiles -- w tiles of X that stay hot in L2 for the
// whole sweep over N, and a few tiles of Y -- instead of sweeping ALL of X once per row of tiles, which for large
// outputs pushes the operands out of L2 behind the stream of C (measured: 26.6 -> 22.2 TFLOP/s as the output grew
// from 4 to 33 GB).
__device__ __forceinline__ void tile_coords(const TcKernelArgs& p, uint32_t tile, uint32_t* tm, uint32_t* tn) {
  const uint32_t w = p.mblock_w;
  if (w == 0) { *tm = tile % p.tiles_m; *tn = tile / p.tiles_m; return; }
  const uint32_t per_block = w * p.tiles_n;
  const uint32_t blk = tile / per_block, r = tile - blk * per_block;
  const uint32_t left = p.tiles_m - blk * w, wb = left < w ? left : w;  // the last block may be narrower
  *tn = r / wb;
  *tm = blk * w + (r - *tn * wb);
}

// ------------------------------------------------------------- loaders ----
// 16-byte loads along the external index: thread -> (vector of VW externals, k).
template <class CF, int ROWS, int LD>
__device__ __forceinline__ void load_stage_vec(typename CF::T* s_stage, const typename CF::T* __restrict__ g,
                                               const int64_t* s_off, const int64_t* s_koff,
                                               uint32_t k0, uint32_t kend, int tid) {
  constexpr int VPR = ROWS / CF::VW;            // vectors per k row
  constexpr int SLOTS = VPR * CF::BK;
  constexpr int PER = (SLOTS + CF::THREADS - 1) / CF::THREADS;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int s = tid + j * CF::THREADS;
    if (SLOTS % CF::THREADS != 0 && s >= SLOTS) break;
    const int ev = s % VPR, kk = s / VPR;
    const int64_t eo = s_off[ev * CF::VW];
    const uint32_t k = k0 + kk;
    const bool ok = eo >= 0 && k < kend;
    const typename CF::T* src = ok ? g + eo + s_koff[kk] : g;
    cp_async16(smem_u32(s_stage + kk * LD + ev * CF::VW), src, ok);
  }
}

// Element-wise loads.  A warp covers `lanes_k` consecutive k by 32/lanes_k
// consecutive externals, so that the lanes that walk the tensor's fastest index
// read whole 32-byte sectors; the write into the external-major image is a
// transposing scatter.  The thread -> element map does not change from stage to
// stage, so it is computed once (elem_slots) and kept packed in registers:
//   bits 0-15 element offset inside the stage image, 16-23 k, 24-31 external.
// 16-byte loads along the contraction index into a contraction-major image [row][k] (pitch CF::LDKV): four lanes
// fetch the 64 bytes one row contributes to a K step.  Needs 4 consecutive flattened k to be contiguous and aligned.
template <class CF, int ROWS>
__device__ __forceinline__ void load_stage_kvec(typename CF::T* s_stage, const typename CF::T* __restrict__ g,
                                                const int64_t* s_off, const int64_t* koff, uint32_t k0, uint32_t kend,
                                                int tid) {
  static_assert(CF::ES == 4, "fp32 only");
  constexpr int CH = CF::BK / 4;  // chunks per row
  const uint32_t sbase = smem_u32(s_stage);
  for (int f = tid; f < ROWS * CH; f += CF::THREADS) {
    const int r = f / CH, kc = f % CH;
    const int64_t eo = s_off[r];
    const bool ok = eo >= 0 && k0 + 4 * kc < kend;
    const typename CF::T* src = ok ? g + eo + koff[4 * kc] : g;
    cp_async16(sbase + (uint32_t)(r * CF::LDKV + 4 * kc) * 4u, src, ok);
  }
}

template <class CF, int ROWS, int LD>
struct ElemSlots {
  static constexpr int SLABS = ROWS * CF::BK / 32;                      // warp-wide groups of 32 elements
  static constexpr int PER = (SLABS + CF::WARPS - 1) / CF::WARPS;      // slabs (= elements per thread) per stage
  static constexpr uint32_t kNoSlot = 0xffffffffu;
  static_assert(CF::BK * LD < 65536 && ROWS <= 256, "slot packing");
  uint32_t slot[PER];
  // lg = log2(lanes walking k); BK and the warp size are powers of two, so the
  // slab arithmetic is shifts and masks.
  __device__ __forceinline__ void init(int tid, int lg) {
    static_assert(CF::BK == 16, "slab arithmetic assumes BK = 16");
    const int lane = tid & 31, warp = tid >> 5;
    const int lk = lane & ((1 << lg) - 1), le = lane >> lg;
    const int ks_bits = 4 - lg;  // log2(slabs along k)
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int slab = warp * PER + j;
      const int kk = ((slab & ((1 << ks_bits) - 1)) << lg) + lk;
      const int el = ((slab >> ks_bits) << (5 - lg)) + le;
      slot[j] = slab < SLABS ? ((uint32_t)(kk * LD + el) | ((uint32_t)kk << 16) | ((uint32_t)el << 24)) : kNoSlot;
    }
  }
  __device__ __forceinline__ void load(typename CF::T* s_stage, const typename CF::T* __restrict__ g,
                                       const int64_t* s_off, const int64_t* s_koff, uint32_t k0,
                                       uint32_t kend) const {
    const uint32_t sbase = smem_u32(s_stage);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const uint32_t sl = slot[j];
      if (SLABS % CF::WARPS != 0 && sl == kNoSlot) continue;
      const int64_t eo = s_off[sl >> 24];
      const uint32_t kk = (sl >> 16) & 0xffu;
      const bool ok = eo >= 0 && k0 + kk < kend;
      const typename CF::T* src = ok ? g + eo + s_koff[kk] : g;
      cp_async_elem<CF::ES>(sbase + (sl & 0xffffu) * CF::ES, src, ok);
    }
  }
};

// Issues the bulk asynchronous copies of a staged output tile (layout: see the staged epilogue) and
// waits until they have read shared memory.  Chunks: per run of E0 rows either one per n, or -- when
// consecutive n are adjacent in the output inside blocks of F0 -- one per such block (at most two per tile).
template <class CF>
__device__ __forceinline__ void bulk_out_tile(const TcKernelArgs& p, typename CF::T* __restrict__ C,
                                              const typename CF::T* ctile, const int64_t* offc_m,
                                              const int64_t* offc_n, uint32_t n0, int tid) {
  using T = typename CF::T;
  constexpr int BM = CF::BM, BN = CF::BN;
  const int E0 = p.epi_run, run_elems = E0 * BN, runs = BM / E0;
  const int F0 = p.epi_n_span;
  int nb = BN, nseg = BN;
  if (F0 > 0) {
    const int left = F0 - (int)(n0 % (uint32_t)F0);
    nb = left < BN ? left : BN;
    nseg = nb < BN ? 2 : 1;
  }
  for (int c = tid; c < runs * nseg; c += CF::THREADS) {
    const int r = c / nseg, sgi = c % nseg;
    const int n = F0 > 0 ? (sgi == 0 ? 0 : nb) : sgi;
    const int len = F0 > 0 ? (sgi == 0 ? nb : BN - nb) : 1;
    T* dstg = C + offc_m[r * E0] + offc_n[n];
    const uint32_t src = smem_u32(ctile + r * run_elems + n * E0);
    const uint32_t bytes = (uint32_t)(E0 * len) * CF::ES;
    if (p.beta) {
      if constexpr (CF::ES == 4)
        asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;\n" ::"l"(dstg), "r"(src), "r"(bytes) : "memory");
      else
        asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f64 [%0], [%1], %2;\n" ::"l"(dstg), "r"(src), "r"(bytes) : "memory");
    } else {
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n" ::"l"(dstg), "r"(src), "r"(bytes) : "memory");
    }
  }
  asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
  asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");  // shared memory is released at exit
}

// The same staged tile, applied with plain 16-byte loads and stores: every chunk (a run of E0 outputs times the
// adjacent n) is contiguous in C, so the whole CTA walks it with one float4 / double2 per thread and step.
template <class CF>
__device__ __forceinline__ void rmw_out_tile(const TcKernelArgs& p, typename CF::T* __restrict__ C,
                                             const typename CF::T* ctile, const int64_t* offc_m,
                                             const int64_t* offc_n, uint32_t n0, int tid) {
  using T = typename CF::T;
  using V = typename Vec16<T>::type;
  constexpr int BM = CF::BM, BN = CF::BN, VW = CF::VW;
  const int E0 = p.epi_run, run_elems = E0 * BN, runs = BM / E0;
  const int F0 = p.epi_n_span;
  int nb = BN, nseg = BN;
  if (F0 > 0) {
    const int left = F0 - (int)(n0 % (uint32_t)F0);
    nb = left < BN ? left : BN;
    nseg = nb < BN ? 2 : 1;
  }
  const bool acc = p.beta != 0;
  for (int c = 0; c < runs * nseg; ++c) {
    const int r = c / nseg, sgi = c % nseg;
    const int n = F0 > 0 ? (sgi == 0 ? 0 : nb) : sgi;
    const int len = F0 > 0 ? (sgi == 0 ? nb : BN - nb) : 1;
    V* dst = reinterpret_cast<V*>(C + offc_m[r * E0] + offc_n[n]);
    const V* src = reinterpret_cast<const V*>(ctile + r * run_elems + n * E0);
    const int nv = E0 * len / VW;
    for (int i = tid; i < nv; i += CF::THREADS) {
      V v = src[i];
      if (acc) {
        const V o = dst[i];
        if constexpr (CF::ES == 4) { v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w; }
        else { v.x += o.x; v.y += o.y; }
      }
      dst[i] = v;
    }
  }
}

// --------------------------------------------------------------- kernel ----
template <class CF>
__global__ void __launch_bounds__(CF::THREADS, CF::MIN_CTAS) tc_contract_kernel(const __grid_constant__ TcKernelArgs p,
                                                                   typename CF::T* __restrict__ C,
                                                                   const typename CF::T* __restrict__ X,
                                                                   const typename CF::T* __restrict__ Y) {
  using T = typename CF::T;
  constexpr int BM = CF::BM, BN = CF::BN, BK = CF::BK, LDX = CF::LDX, LDY = CF::LDY, STAGES = CF::STAGES;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int64_t* offx_m = reinterpret_cast<int64_t*>(smem_raw);
  int64_t* offc_m = offx_m + BM;
  int64_t* offy_n = offc_m + BM;
  int64_t* offc_n = offy_n + BN;
  int64_t* kring = offc_n + BN;  // [KRING][2][BK]
  int64_t* pf_m = kring + CF::KRING * 2 * BK;
  int64_t* pf_n = pf_m + BM;
  T* Xs = reinterpret_cast<T*>(pf_n + BN);
  T* Ys = Xs + STAGES * CF::XIMG;

  const int tid = threadIdx.x;
  const uint32_t bid = blockIdx.x;
  const uint32_t tile_m = bid % p.tiles_m;
  const uint32_t rest = bid / p.tiles_m;
  const uint32_t tile_n = rest % p.tiles_n;
  const uint32_t slice = rest / p.tiles_n;
  const uint32_t m0 = tile_m * BM, n0 = tile_n * BN;
  const uint32_t kbeg = p.k_first + slice * p.k_chunk;
  const uint32_t kend = min(p.Kflat, kbeg + p.k_chunk);

  for (int i = tid; i < BM + BN; i += CF::THREADS) {
    if (i < BM) decode(p.M, m0 + i, p.Mflat, &offx_m[i], &offc_m[i]);
    else decode(p.N, n0 + (i - BM), p.Nflat, &offy_n[i - BM], &offc_n[i - BM]);
  }
  // Contraction offsets of the first KRING stages, read directly.
  for (int i = tid; i < CF::KRING * 2 * BK; i += CF::THREADS) {
    const int st = i / (2 * BK), r = i % (2 * BK);
    const uint32_t k = kbeg + st * BK + (r % BK);
    kring[i] = k < kend ? (r < BK ? p.koff_x[k] : p.koff_y[k]) : 0;
  }
  __syncthreads();

  const int nk = (int)((kend - kbeg + BK - 1) / BK);
  ElemSlots<CF, BM, LDX> slots_x;
  ElemSlots<CF, BN, LDY> slots_y;
  if constexpr (!CF::VECX && !CF::KVX) slots_x.init(tid, p.lanes_k_x == 1 ? 0 : (CF::ES == 8 ? 2 : 3));
  if constexpr (!CF::VECY && !CF::KVY) slots_y.init(tid, p.lanes_k_y == 1 ? 0 : (CF::ES == 8 ? 2 : 3));
  auto issue = [&](int it) {
    if (it < nk) {
      const int st = it % STAGES;
      const uint32_t k0 = kbeg + it * BK;
      T* xs = Xs + st * CF::XIMG;
      T* ys = Ys + st * CF::YIMG;
      const int64_t* kx = kring + (it % CF::KRING) * 2 * BK;
      if constexpr (CF::KVX) load_stage_kvec<CF, BM>(xs, X, offx_m, kx, k0, kend, tid);
      else if constexpr (CF::VECX) load_stage_vec<CF, BM, LDX>(xs, X, offx_m, kx, k0, kend, tid);
      else slots_x.load(xs, X, offx_m, kx, k0, kend);
      if constexpr (CF::KVY) load_stage_kvec<CF, BN>(ys, Y, offy_n, kx + BK, k0, kend, tid);
      else if constexpr (CF::VECY) load_stage_vec<CF, BN, LDY>(ys, Y, offy_n, kx + BK, k0, kend, tid);
      else slots_y.load(ys, Y, offy_n, kx + BK, k0, kend);
    }
    cp_async_commit();
  };
  // Stage `it`'s data group also carries the offsets of stage it + KRING, into the
  // ring slot whose last reader (the issue of stage `it`) is behind a barrier.
  auto issue_koff = [&](int it) {
    const int nx = it + CF::KRING;
    if (tid < 2 * BK && nx < nk) {
      const uint32_t k = kbeg + nx * BK + (tid % BK);
      const int64_t* src = (tid < BK ? p.koff_x : p.koff_y) + (k < kend ? k : 0);
      cp_async8(smem_u32(kring + (nx % CF::KRING) * 2 * BK + tid), src, k < kend);
    }
  };
  // How `+=` / `-=` reaches C when K is not split (p.c_mode):
  //   0  read-modify-write in the epilogue; the CTA prefetches its own C tile into
  //      L2 before the pipeline fills, so the epilogue loads wait on L2, not DRAM;
  //   1  the accumulators START as alpha*C (alpha = +-1, exact), the epilogue only
  //      stores alpha*acc; the C tile of a CTA one wave ahead is prefetched into L2.
  const bool accumulate = p.ksplit == 1 && p.beta != 0;
  const bool init_from_c = accumulate && p.c_mode == 1;
  const bool rmw = accumulate && p.c_mode != 1;
  const bool stream = p.c_stream != 0;  // cache-streaming hints on the accesses to C

  auto prefetch_tile = [&](const int64_t* tm, const int64_t* tn) {
    constexpr int SEC = 32 / CF::ES;  // elements per 32-byte sector
    constexpr int SPR = BM / SEC;     // sectors per tile row
    for (int i = tid; i < SPR * BN; i += CF::THREADS) {
      const int64_t cm = tm[(i % SPR) * SEC], cn = tn[i / SPR];
      if (cm >= 0 && cn >= 0) asm volatile("prefetch.global.L2 [%0];\n" ::"l"(C + cn + cm));
    }
  };
  auto prefetch_next = [&]() {
    if (!accumulate || p.prefetch_dist == 0) return;
    if (rmw) { prefetch_tile(offc_m, offc_n); return; }
    const uint32_t nb = bid + p.prefetch_dist;
    if (nb >= p.tiles_m * p.tiles_n) return;  // uniform across the CTA
    const uint32_t pm0 = (nb % p.tiles_m) * BM, pn0 = (nb / p.tiles_m) * BN;
    for (int i = tid; i < BM + BN; i += CF::THREADS) {
      int64_t dummy;
      if (i < BM) decode(p.M, pm0 + i, p.Mflat, &dummy, &pf_m[i]);
      else decode(p.N, pn0 + (i - BM), p.Nflat, &dummy, &pf_n[i - BM]);
    }
    __syncthreads();
    prefetch_tile(pf_m, pf_n);
  };
  auto ld_c2 = [&](const double2* q) { return stream ? __ldcs(q) : *q; };
  auto st_c2 = [&](double2* q, double2 v) { if (stream) __stcs(q, v); else *q = v; };

  if constexpr (CF::MATH == TC_MATH_DMMA) {
    // ---------------- fp64 on the tensor pipe ----------------
    // D(8x8) += Aop(8x4) * Bop(4x8) with rows of D = n, columns of D = m, so a
    // thread's two D registers are consecutive m (the output's fastest index).
    // MMA row/column r of block b is mapped to tile element 16*(b/2) + 2r + (b&1):
    // one 16-byte shared load feeds two blocks, and the four D values a thread
    // holds for a block pair are four CONSECUTIVE m.
    // Thread holds, per n row (nb = 2j+h -> n = wn0 + 16j + 2g + h) and block
    // pair i, the four m = wm0 + 16i + 4t + {0,1,2,3}:
    //   acc[nb][2i][0], acc[nb][2i+1][0], acc[nb][2i][1], acc[nb][2i+1][1].
    constexpr int WM = CF::WM, WN = CF::WN;
    constexpr int MB2 = WM / 16, NB2 = WN / 16;
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int wm0 = (warp % CF::WARPS_M) * WM, wn0 = (warp / CF::WARPS_M) * WN;
    const double alpha = p.alpha;
    double acc[2 * NB2][2 * MB2][2];
#pragma unroll
    for (int j = 0; j < 2 * NB2; ++j)
#pragma unroll
      for (int i = 0; i < 2 * MB2; ++i) { acc[j][i][0] = 0.0; acc[j][i][1] = 0.0; }

    if (init_from_c) {
#pragma unroll
      for (int nb = 0; nb < 2 * NB2; ++nb) {
        const int64_t cn = offc_n[wn0 + 16 * (nb >> 1) + 2 * g + (nb & 1)];
        if (cn < 0) continue;
        if (p.vec_c == 4) {
#pragma unroll
          for (int i = 0; i < MB2; ++i) {
            const int64_t co = offc_m[wm0 + 16 * i + 4 * t];
            if (co < 0) continue;
            const double2* src = reinterpret_cast<const double2*>(C + cn + co);
            const double2 v0 = ld_c2(src), v1 = ld_c2(src + 1);
            acc[nb][2 * i][0] = alpha * v0.x;
            acc[nb][2 * i + 1][0] = alpha * v0.y;
            acc[nb][2 * i][1] = alpha * v1.x;
            acc[nb][2 * i + 1][1] = alpha * v1.y;
          }
        } else if (p.vec_c == 2) {
#pragma unroll
          for (int i = 0; i < MB2; ++i)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int64_t co = offc_m[wm0 + 16 * i + 4 * t + 2 * e];
              if (co < 0) continue;
              const double2 v = ld_c2(reinterpret_cast<const double2*>(C + cn + co));
              acc[nb][2 * i][e] = alpha * v.x;
              acc[nb][2 * i + 1][e] = alpha * v.y;
            }
        } else {
#pragma unroll
          for (int i = 0; i < MB2; ++i)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int64_t co = offc_m[wm0 + 16 * i + 4 * t + q];
              if (co < 0) continue;
              acc[nb][2 * i + (q & 1)][q >> 1] = alpha * C[cn + co];
            }
        }
      }
    }

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) issue(s);
    prefetch_next();

    for (int it = 0; it < nk; ++it) {
      cp_async_wait<STAGES - 2>();
      __syncthreads();
      issue_koff(it);
      issue(it + STAGES - 1);
      const int st = it % STAGES;
      const T* xs = Xs + st * BK * LDX + wm0 + 2 * g;
      const T* ys = Ys + st * BK * LDY + wn0 + 2 * g;
      const int kleft = (int)(kend - (kbeg + it * BK));
      const int nks = kleft >= BK ? BK / 4 : (kleft + 3) / 4;
#pragma unroll
      for (int ks = 0; ks < BK / 4; ++ks) {
        if (ks < nks) {
          const int k = ks * 4 + t;
          double2 xf[MB2], yf[NB2];
#pragma unroll
          for (int i = 0; i < MB2; ++i) xf[i] = *reinterpret_cast<const double2*>(xs + k * LDX + i * 16);
#pragma unroll
          for (int j = 0; j < NB2; ++j) yf[j] = *reinterpret_cast<const double2*>(ys + k * LDY + j * 16);
#pragma unroll
          for (int j = 0; j < NB2; ++j)
#pragma unroll
            for (int i = 0; i < MB2; ++i) {
              dmma884(acc[2 * j][2 * i][0], acc[2 * j][2 * i][1], yf[j].x, xf[i].x);
              dmma884(acc[2 * j][2 * i + 1][0], acc[2 * j][2 * i + 1][1], yf[j].x, xf[i].y);
              dmma884(acc[2 * j + 1][2 * i][0], acc[2 * j + 1][2 * i][1], yf[j].y, xf[i].x);
              dmma884(acc[2 * j + 1][2 * i + 1][0], acc[2 * j + 1][2 * i + 1][1], yf[j].y, xf[i].y);
            }
        }
      }
    }
    cp_async_wait<0>();

    // ---------------- epilogue: stores only ----------------
    if (p.ksplit > 1) {
      double* ws = reinterpret_cast<double*>(p.ws) +
                   ((size_t)slice * p.tiles_m * p.tiles_n + (size_t)tile_n * p.tiles_m + tile_m) * (size_t)(BM * BN);
#pragma unroll
      for (int nb = 0; nb < 2 * NB2; ++nb) {
        const int nl = wn0 + 16 * (nb >> 1) + 2 * g + (nb & 1);
#pragma unroll
        for (int i = 0; i < MB2; ++i) {
          const int ml = wm0 + 16 * i + 4 * t;
          double2* dst = reinterpret_cast<double2*>(ws + (size_t)nl * BM + ml);
          dst[0] = make_double2(acc[nb][2 * i][0], acc[nb][2 * i + 1][0]);
          dst[1] = make_double2(acc[nb][2 * i][1], acc[nb][2 * i + 1][1]);
        }
      }
      return;
    }
    if (p.vec_c == 4) {
      // Two n rows (the pair fed by one Y fragment) per batch: all their loads are
      // issued before the first store, so a batch pays one L2 round trip.
      int64_t co[MB2];
#pragma unroll
      for (int i = 0; i < MB2; ++i) co[i] = offc_m[wm0 + 16 * i + 4 * t];
#pragma unroll
      for (int j = 0; j < NB2; ++j) {
        int64_t cn[2];
        double2 c0[2][MB2], c1[2][MB2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          cn[h] = offc_n[wn0 + 16 * j + 2 * g + h];
#pragma unroll
          for (int i = 0; i < MB2; ++i) {
            c0[h][i] = make_double2(0.0, 0.0);
            c1[h][i] = make_double2(0.0, 0.0);
            if (rmw && cn[h] >= 0 && co[i] >= 0) {
              const double2* src = reinterpret_cast<const double2*>(C + cn[h] + co[i]);
              c0[h][i] = ld_c2(src);
              c1[h][i] = ld_c2(src + 1);
            }
          }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int nb = 2 * j + h;
#pragma unroll
          for (int i = 0; i < MB2; ++i) {
            if (cn[h] < 0 || co[i] < 0) continue;
            double2* dst = reinterpret_cast<double2*>(C + cn[h] + co[i]);
            st_c2(dst, make_double2(fma(alpha, acc[nb][2 * i][0], c0[h][i].x), fma(alpha, acc[nb][2 * i + 1][0], c0[h][i].y)));
            st_c2(dst + 1, make_double2(fma(alpha, acc[nb][2 * i][1], c1[h][i].x), fma(alpha, acc[nb][2 * i + 1][1], c1[h][i].y)));
          }
        }
      }
      return;
    }
#pragma unroll
    for (int nb = 0; nb < 2 * NB2; ++nb) {
      const int64_t cn = offc_n[wn0 + 16 * (nb >> 1) + 2 * g + (nb & 1)];
      if (cn < 0) continue;
      if (p.vec_c == 2) {
#pragma unroll
        for (int i = 0; i < MB2; ++i)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int64_t co = offc_m[wm0 + 16 * i + 4 * t + 2 * e];
            if (co < 0) continue;
            double2* dst = reinterpret_cast<double2*>(C + cn + co);
            double2 c = make_double2(0.0, 0.0);
            if (rmw) c = ld_c2(dst);
            st_c2(dst, make_double2(fma(alpha, acc[nb][2 * i][e], c.x), fma(alpha, acc[nb][2 * i + 1][e], c.y)));
          }
      } else {
#pragma unroll
        for (int i = 0; i < MB2; ++i)
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int64_t co = offc_m[wm0 + 16 * i + 4 * t + q];
            if (co < 0) continue;
            const double c = rmw ? C[cn + co] : 0.0;
            C[cn + co] = fma(alpha, acc[nb][2 * i + (q & 1)][q >> 1], c);
          }
      }
    }
  } else if constexpr (CF::MATH == TC_MATH_TF32X3) {
    // ---------------- fp32 as three TF32 tensor-core products ----------------
    // mma.sync m16n8k8: D rows (16) = n, D columns (8) = m; column c of m-block 2i+h is tile element
    // 16i + 2c + h, so one 8-byte shared load feeds two blocks and a thread's D values of a block pair are
    // four consecutive m (16 bytes of the output).  Every operand value is split v = hi + lo (both TF32)
    // and the product is hi*hi + hi*lo + lo*hi accumulated in fp32.
    constexpr int WM = CF::WM, WN = CF::WN;
    constexpr int MB2 = WM / 16, NB = WN / 16;
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int wm0 = (warp % CF::WARPS_M) * WM, wn0 = (warp / CF::WARPS_M) * WN;
    const float alpha = (float)p.alpha;
    const bool rmw = accumulate;  // this path has no "accumulators start from C" mode: c_mode 1 means 0 here
    float acc[NB][2 * MB2][4];
#pragma unroll
    for (int j = 0; j < NB; ++j)
#pragma unroll
      for (int i = 0; i < 2 * MB2; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][i][e] = 0.f;

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) issue(s);
    prefetch_next();

    for (int it = 0; it < nk; ++it) {
      cp_async_wait<STAGES - 2>();
      __syncthreads();
      issue_koff(it);
      issue(it + STAGES - 1);
      const int st = it % STAGES;
      const float* xs = Xs + st * BK * LDX + wm0 + 2 * g;
      const float* ys = Ys + st * BK * LDY + wn0 + g;
      const int kleft = (int)(kend - (kbeg + it * BK));
      const int nk8 = kleft >= BK ? BK / 8 : (kleft + 7) / 8;
#pragma unroll
      for (int k8 = 0; k8 < BK / 8; ++k8) {
        if (k8 < nk8) {
          const int k = k8 * 8 + t;
          uint32_t ahi[NB][4], alo[NB][4];
#pragma unroll
          for (int j = 0; j < NB; ++j) {
            split_tf32(ys[k * LDY + 16 * j], ahi[j][0], alo[j][0]);
            split_tf32(ys[k * LDY + 16 * j + 8], ahi[j][1], alo[j][1]);
            split_tf32(ys[(k + 4) * LDY + 16 * j], ahi[j][2], alo[j][2]);
            split_tf32(ys[(k + 4) * LDY + 16 * j + 8], ahi[j][3], alo[j][3]);
          }
#pragma unroll
          for (int i = 0; i < MB2; ++i) {
            const float2 x0 = *reinterpret_cast<const float2*>(xs + k * LDX + 16 * i);
            const float2 x1 = *reinterpret_cast<const float2*>(xs + (k + 4) * LDX + 16 * i);
            uint32_t bhi[2][2], blo[2][2];
            split_tf32(x0.x, bhi[0][0], blo[0][0]);
            split_tf32(x1.x, bhi[0][1], blo[0][1]);
            split_tf32(x0.y, bhi[1][0], blo[1][0]);
            split_tf32(x1.y, bhi[1][1], blo[1][1]);
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
              for (int j = 0; j < NB; ++j) {
                mma_tf32(acc[j][2 * i + h], alo[j], bhi[h]);
                mma_tf32(acc[j][2 * i + h], ahi[j], blo[h]);
                mma_tf32(acc[j][2 * i + h], ahi[j], bhi[h]);
              }
          }
        }
      }
    }
    cp_async_wait<0>();

    // Thread holds, for n = wn0 + 16j + g + 8r (r = 0, 1) and block pair i, the four
    // m = wm0 + 16i + 4t + q:  acc[j][2i + (q & 1)][2r + (q >> 1)].
    if (p.ksplit > 1) {
      float* ws = reinterpret_cast<float*>(p.ws) +
                  ((size_t)slice * p.tiles_m * p.tiles_n + (size_t)tile_n * p.tiles_m + tile_m) * (size_t)(BM * BN);
#pragma unroll
      for (int j = 0; j < NB; ++j)
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
          for (int i = 0; i < MB2; ++i) {
            const int nl = wn0 + 16 * j + g + 8 * r, ml = wm0 + 16 * i + 4 * t;
            *reinterpret_cast<float4*>(ws + (size_t)nl * BM + ml) =
                make_float4(acc[j][2 * i][2 * r], acc[j][2 * i + 1][2 * r], acc[j][2 * i][2 * r + 1], acc[j][2 * i + 1][2 * r + 1]);
          }
      return;
    }
    if constexpr (STAGES * CF::STAGE_ELEMS >= BM * BN) {
      const int E0 = p.epi_run;
      if (p.c_mode == 2 && E0 > 0 && p.vec_c >= 4 && m0 + BM <= p.Mflat && n0 + BN <= p.Nflat) {
        __syncthreads();
        float* ctile = Xs;
        const int run_elems = E0 * BN;
#pragma unroll
        for (int i = 0; i < MB2; ++i) {
          const int m = wm0 + 16 * i + 4 * t;
          float* col = ctile + (m / E0) * run_elems + (m % E0);
#pragma unroll
          for (int j = 0; j < NB; ++j)
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              const int n = wn0 + 16 * j + g + 8 * r;
              *reinterpret_cast<float4*>(col + n * E0) =
                  make_float4(alpha * acc[j][2 * i][2 * r], alpha * acc[j][2 * i + 1][2 * r],
                              alpha * acc[j][2 * i][2 * r + 1], alpha * acc[j][2 * i + 1][2 * r + 1]);
            }
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        __syncthreads();
        bulk_out_tile<CF>(p, C, ctile, offc_m, offc_n, n0, tid);
        return;
      }
    }
#pragma unroll
    for (int j = 0; j < NB; ++j)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int64_t cn = offc_n[wn0 + 16 * j + g + 8 * r];
        if (cn < 0) continue;
#pragma unroll
        for (int i = 0; i < MB2; ++i) {
          if (p.vec_c == 4) {
            const int64_t co = offc_m[wm0 + 16 * i + 4 * t];
            if (co < 0) continue;
            float4* dst = reinterpret_cast<float4*>(C + cn + co);
            float4 c = make_float4(0.f, 0.f, 0.f, 0.f);
            if (rmw) c = *dst;
            *dst = make_float4(fmaf(alpha, acc[j][2 * i][2 * r], c.x), fmaf(alpha, acc[j][2 * i + 1][2 * r], c.y),
                               fmaf(alpha, acc[j][2 * i][2 * r + 1], c.z), fmaf(alpha, acc[j][2 * i + 1][2 * r + 1], c.w));
          } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int64_t co = offc_m[wm0 + 16 * i + 4 * t + q];
              if (co < 0) continue;
              const float c = rmw ? C[cn + co] : 0.f;
              C[cn + co] = fmaf(alpha, acc[j][2 * i + (q & 1)][2 * r + (q >> 1)], c);
            }
          }
        }
      }
  } else if constexpr (CF::MATH == TC_MATH_TF32TC) {
    // ---------------- fp32 as three TF32 products on tcgen05, accumulators in tensor memory ----------------
    // D (tensor memory) has one lane per n (BN = 128) and one column per m (BM): D += Y * X^T.  Each K step the
    // gathered fp32 images are split once per element into hi and lo TF32 images laid out as 128-byte core
    // matrices (8 externals x 4 k), one elected thread issues lo*hi, hi*lo and hi*hi for each group of 8 k, and a
    // commit on an mbarrier tells when the images may be overwritten.  The epilogue reads each lane's BM values
    // with tcgen05.ld and leaves through the same staged bulk reduce as the other fp32 kernels.
    constexpr int TCOLS = CF::TMEM_COLS;
    const int warp = tid >> 5, lane = tid & 31;
    float* ua_hi = Ys + STAGES * CF::YIMG;   // Y: BN rows
    float* ua_lo = ua_hi + BK * BN;
    float* ub_hi = ua_lo + BK * BN;          // X: BM rows
    float* ub_lo = ub_hi + BK * BM;
    uint64_t* mbar = reinterpret_cast<uint64_t*>(ub_lo + BK * BM);
    uint32_t* slot = reinterpret_cast<uint32_t*>(mbar + 1);
    volatile uint32_t* flag = slot + 1;      // 0, or 1 after a wait that ran out of polls
    const float alpha = (float)p.alpha;
    if (warp == 0) {
      tmem_alloc(slot, TCOLS);
      tmem_relinquish();
    }
    if (tid == 0) {
      mbar_init(mbar, 1);
      *flag = 0;
      asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    tc05_fence_before();
    __syncthreads();
    tc05_fence_after();
    const uint32_t tmem = *slot;
    constexpr uint32_t IDESC = umma_idesc_tf32(BN, BM);

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) issue(s);
    prefetch_next();

    bool gave_up = false;
    for (int it = 0; it < nk; ++it) {
      cp_async_wait<STAGES - 2>();
      // the MMAs of the previous step must have read the images before they are rewritten
      if (tid == 0 && it > 0 && !mbar_wait(mbar, (uint32_t)(it - 1) & 1u, p.status, 8, p.spin_limit)) *flag = 1;
      __syncthreads();
      if (*flag) { gave_up = true; break; }  // uniform
      issue_koff(it);
      issue(it + STAGES - 1);
      const int st = it % STAGES;
      const float* xs = Xs + st * CF::XIMG;
      const float* ys = Ys + st * CF::YIMG;
      // Chunk f of an operand with R rows: row r = f % R, the four k = 4 * (f / R) .. + 3; its 16 bytes go to
      // core matrix (r / 8, f / R), row r % 8.  Lanes walk r: conflict-free reads and writes.
      for (int f = tid; f < BN * (BK / 4); f += CF::THREADS) {
        const int r = f % BN, kc = f / BN;
        float4 v4;
        if constexpr (CF::KVY) v4 = *reinterpret_cast<const float4*>(ys + r * CF::LDKV + 4 * kc);
        else {
          const float* src = ys + (4 * kc) * LDY + r;
          v4 = make_float4(src[0], src[LDY], src[2 * LDY], src[3 * LDY]);
        }
        float4 h, l;
        split_tf32_bits(v4.x, h.x, l.x); split_tf32_bits(v4.y, h.y, l.y);
        split_tf32_bits(v4.z, h.z, l.z); split_tf32_bits(v4.w, h.w, l.w);
        const int d = ((r >> 3) * (BK / 4) + kc) * 8 + (r & 7);
        reinterpret_cast<float4*>(ua_hi)[d] = h;
        reinterpret_cast<float4*>(ua_lo)[d] = l;
      }
      for (int f = tid; f < BM * (BK / 4); f += CF::THREADS) {
        const int r = f % BM, kc = f / BM;
        float4 v4;
        if constexpr (CF::KVX) v4 = *reinterpret_cast<const float4*>(xs + r * CF::LDKV + 4 * kc);
        else {
          const float* src = xs + (4 * kc) * LDX + r;
          v4 = make_float4(src[0], src[LDX], src[2 * LDX], src[3 * LDX]);
        }
        float4 h, l;
        split_tf32_bits(v4.x, h.x, l.x); split_tf32_bits(v4.y, h.y, l.y);
        split_tf32_bits(v4.z, h.z, l.z); split_tf32_bits(v4.w, h.w, l.w);
        const int d = ((r >> 3) * (BK / 4) + kc) * 8 + (r & 7);
        reinterpret_cast<float4*>(ub_hi)[d] = h;
        reinterpret_cast<float4*>(ub_lo)[d] = l;
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // generic writes -> the MMA's reads
      tc05_fence_before();
      __syncthreads();
      if (tid == 0) {
        tc05_fence_after();
        const int kleft = (int)(kend - (kbeg + it * BK));
        const int nk8 = kleft >= BK ? BK / 8 : (kleft + 7) / 8;
        for (int kg = 0; kg < nk8; ++kg) {
          // two 4-k chunks per MMA: 128 bytes apart; 8-row groups (BK / 4) * 128 bytes apart
          const uint64_t ah = umma_desc_k(smem_u32(ua_hi) + kg * 256, 128, (BK / 4) * 128);
          const uint64_t al = umma_desc_k(smem_u32(ua_lo) + kg * 256, 128, (BK / 4) * 128);
          const uint64_t bh = umma_desc_k(smem_u32(ub_hi) + kg * 256, 128, (BK / 4) * 128);
          const uint64_t bl = umma_desc_k(smem_u32(ub_lo) + kg * 256, 128, (BK / 4) * 128);
          tc05_mma_tf32(tmem, al, bh, IDESC, (it > 0 || kg > 0) ? 1u : 0u);
          tc05_mma_tf32(tmem, ah, bl, IDESC, 1u);
          tc05_mma_tf32(tmem, ah, bh, IDESC, 1u);
        }
        tc05_commit(mbar);
      }
    }
    cp_async_wait<0>();
    if (!gave_up) {
      if (tid == 0 && nk > 0 && !mbar_wait(mbar, (uint32_t)(nk - 1) & 1u, p.status, 9, p.spin_limit)) *flag = 1;
      __syncthreads();
      gave_up = *flag != 0;
    }
    // This thread's lane of D: n = 32 * (warp % 4) + lane; warps 0-3 take the first half of the columns, 4-7 the second.
    constexpr int CPT = BM / 2;
    static_assert(CPT % 16 == 0, "columns per thread");
    float v[CPT];
    const int nl = 32 * (warp & 3) + lane, mbase = (warp >> 2) * CPT;
    if (!gave_up && nk > 0) {
      tc05_fence_after();
#pragma unroll
      for (int c = 0; c < CPT / 16; ++c)
        tc05_ld16(tmem + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)(mbase + 16 * c), v + 16 * c);
      tc05_wait_ld();
    } else {
#pragma unroll
      for (int c = 0; c < CPT; ++c) v[c] = 0.f;
    }
    tc05_fence_before();
    __syncthreads();  // every warp has its values: tensor memory and the operand images are free
    if (warp == 0) tmem_dealloc(tmem, TCOLS);
    if (gave_up) return;

    if (p.ksplit > 1) {
      float* ws = reinterpret_cast<float*>(p.ws) +
                  ((size_t)slice * p.tiles_m * p.tiles_n + (size_t)tile_n * p.tiles_m + tile_m) * (size_t)(BM * BN);
#pragma unroll
      for (int c = 0; c < CPT; c += 4)
        *reinterpret_cast<float4*>(ws + (size_t)nl * BM + mbase + c) = make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]);
      return;
    }
    const int E0 = p.epi_run;
    const bool staged_rmw = p.c_mode == 0 && p.epi_n_span > 0;  // read-modify-write of long contiguous chunks
    if ((p.c_mode == 2 || staged_rmw) && E0 > 0 && p.vec_c >= 4 && m0 + BM <= p.Mflat && n0 + BN <= p.Nflat) {
      float* ctile = Xs;  // BM * BN floats: fits in the stage images plus the MMA images
      const int run_elems = E0 * BN;
      // m = mbase + c walks the runs of E0 outputs: one division, then steps of 4 (E0 is a multiple of 4)
      int rem = mbase % E0;
      float* dst = ctile + (mbase / E0) * run_elems + nl * E0;
#pragma unroll
      for (int c = 0; c < CPT; c += 4) {
        *reinterpret_cast<float4*>(dst + rem) = make_float4(alpha * v[c], alpha * v[c + 1], alpha * v[c + 2], alpha * v[c + 3]);
        rem += 4;
        if (rem >= E0) { rem -= E0; dst += run_elems; }
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      __syncthreads();
      if (staged_rmw) rmw_out_tile<CF>(p, C, ctile, offc_m, offc_n, n0, tid);
      else bulk_out_tile<CF>(p, C, ctile, offc_m, offc_n, n0, tid);
      return;
    }
    {
      // Ragged tiles, unaligned or non-contiguous outputs: the tile goes through shared memory ([n][m], odd pitch)
      // so that a row of C is read and written by consecutive lanes on consecutive m.
      static_assert(STAGES * CF::STAGE_ELEMS + CF::UMMA_ELEMS >= BN * (BM + 1), "staging room");
      float* ctile = Xs;
      constexpr int CP = BM + 1;
#pragma unroll
      for (int c = 0; c < CPT; ++c) ctile[nl * CP + mbase + c] = alpha * v[c];
      __syncthreads();
      for (int row = warp; row < BN; row += CF::WARPS) {
        const int64_t cn = offc_n[row];
        if (cn < 0) continue;  // uniform across the warp
#pragma unroll
        for (int m = lane; m < BM; m += 32) {
          const int64_t co = offc_m[m];
          if (co < 0) continue;
          float* q = C + cn + co;
          const float r = ctile[row * CP + m];
          *q = accumulate ? r + *q : r;
        }
      }
    }
  } else {
    // ---------------- vector pipe (FFMA / DFMA) ----------------
    // (BM/8) x (BN/8) threads, 8 x 8 outputs each, as groups of VW contiguous
    // elements: m(q,e) = q*TX*VW + tx*VW + e, same along n.
    using V = typename Vec16<T>::type;
    constexpr int VW = CF::VW, GR = 8 / VW;
    constexpr int TX = BM / 8, TY = BN / 8;
    const int tx = tid % TX, ty = tid / TX;
    const T alpha = (T)p.alpha;
    const bool vec_c = p.vec_c >= VW;
    T acc[8][8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[j][i] = T(0);

    if (init_from_c) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int64_t cn = offc_n[(j / VW) * TY * VW + ty * VW + (j % VW)];
        if (cn < 0) continue;
#pragma unroll
        for (int q = 0; q < GR; ++q) {
          if (vec_c) {
            const int64_t co = offc_m[q * TX * VW + tx * VW];
            if (co < 0) continue;
            const V v = stream ? __ldcs(reinterpret_cast<const V*>(C + cn + co)) : *reinterpret_cast<const V*>(C + cn + co);
            const T* vp = reinterpret_cast<const T*>(&v);
#pragma unroll
            for (int e = 0; e < VW; ++e) acc[j][q * VW + e] = alpha * vp[e];
          } else {
#pragma unroll
            for (int e = 0; e < VW; ++e) {
              const int64_t co = offc_m[q * TX * VW + tx * VW + e];
              if (co >= 0) acc[j][q * VW + e] = alpha * C[cn + co];
            }
          }
        }
      }
    }

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) issue(s);
    prefetch_next();

    for (int it = 0; it < nk; ++it) {
      cp_async_wait<STAGES - 2>();
      __syncthreads();
      issue_koff(it);
      issue(it + STAGES - 1);
      const int st = it % STAGES;
      const T* xs = Xs + st * BK * LDX + tx * VW;
      const T* ys = Ys + st * BK * LDY + ty * VW;
      const int kleft = (int)(kend - (kbeg + it * BK));
      const int kv = kleft >= BK ? BK : kleft;
#pragma unroll
      for (int kk = 0; kk < BK; ++kk) {
        if (kk < kv) {
          T xv[8], yv[8];
#pragma unroll
          for (int q = 0; q < GR; ++q) {
            *reinterpret_cast<V*>(&xv[q * VW]) = *reinterpret_cast<const V*>(xs + kk * LDX + q * TX * VW);
            *reinterpret_cast<V*>(&yv[q * VW]) = *reinterpret_cast<const V*>(ys + kk * LDY + q * TY * VW);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[j][i] = fma(yv[j], xv[i], acc[j][i]);
        }
      }
    }
    cp_async_wait<0>();

    // ---------------- epilogue: stores only ----------------
    if (p.ksplit > 1) {
      T* ws = reinterpret_cast<T*>(p.ws) +
              ((size_t)slice * p.tiles_m * p.tiles_n + (size_t)tile_n * p.tiles_m + tile_m) * (size_t)(BM * BN);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int nl = (j / VW) * TY * VW + ty * VW + (j % VW);
#pragma unroll
        for (int q = 0; q < GR; ++q) {
          const int ml = q * TX * VW + tx * VW;
          *reinterpret_cast<V*>(ws + (size_t)nl * BM + ml) = *reinterpret_cast<const V*>(&acc[j][q * VW]);
        }
      }
      return;
    }
    // Staged bulk epilogue (c_mode 2, plans with args.epi_run = E0 > 0, tiles wholly inside the tensor).
    // The tile is laid out in the freed stage buffers in the ORDER IT HAS IN THE OUTPUT and leaves as bulk
    // asynchronous copies (reduce-add for `+=`/`-=`, plain copy for `=`): the SM never loads C.  The BM rows
    // split into BM/E0 runs of E0 elements contiguous in C; staging index of (m, n) is
    //   (m / E0) * (E0 * BN) + n * E0 + (m % E0).
    // If consecutive n are adjacent in C inside blocks of F0 (args.epi_n_span: the output's second index
    // belongs to the other operand), a run is one chunk per such block (at most two per tile), otherwise
    // one chunk per (run, n).
    if constexpr (STAGES * CF::STAGE_ELEMS >= BM * BN) {
      const int E0 = p.epi_run;
      if (p.c_mode == 2 && E0 > 0 && p.vec_c >= VW && m0 + BM <= p.Mflat && n0 + BN <= p.Nflat) {
        __syncthreads();  // every warp is done with the stage buffers
        T* ctile = Xs;
        const int run_elems = E0 * BN;
#pragma unroll
        for (int q = 0; q < GR; ++q) {
          const int m = q * TX * VW + tx * VW;
          T* col = ctile + (m / E0) * run_elems + (m % E0);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int n = (j / VW) * TY * VW + ty * VW + (j % VW);
            T r[VW];
#pragma unroll
            for (int e = 0; e < VW; ++e) r[e] = alpha * acc[j][q * VW + e];
            *reinterpret_cast<V*>(col + n * E0) = *reinterpret_cast<const V*>(r);
          }
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        __syncthreads();
        bulk_out_tile<CF>(p, C, ctile, offc_m, offc_n, n0, tid);
        return;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int64_t cn = offc_n[(j / VW) * TY * VW + ty * VW + (j % VW)];
      if (cn < 0) continue;
      if (vec_c) {
        int64_t co[GR];
        V cv[GR];
#pragma unroll
        for (int q = 0; q < GR; ++q) {
          co[q] = offc_m[q * TX * VW + tx * VW];
          if (rmw && co[q] >= 0) {
            const V* src = reinterpret_cast<const V*>(C + cn + co[q]);
            cv[q] = stream ? __ldcs(src) : *src;
          }
        }
#pragma unroll
        for (int q = 0; q < GR; ++q) {
          if (co[q] < 0) continue;
          T r[VW];
          const T* cp = reinterpret_cast<const T*>(&cv[q]);
#pragma unroll
          for (int e = 0; e < VW; ++e) r[e] = rmw ? fma(alpha, acc[j][q * VW + e], cp[e]) : alpha * acc[j][q * VW + e];
          V* dst = reinterpret_cast<V*>(C + cn + co[q]);
          if (stream) __stcs(dst, *reinterpret_cast<const V*>(r)); else *dst = *reinterpret_cast<const V*>(r);
        }
      } else {
#pragma unroll
        for (int q = 0; q < GR; ++q)
#pragma unroll
          for (int e = 0; e < VW; ++e) {
            const int64_t co = offc_m[q * TX * VW + tx * VW + e];
            if (co < 0) continue;
            const T c = rmw ? C[cn + co] : T(0);
            C[cn + co] = fma(alpha, acc[j][q * VW + e], c);
          }
      }
    }
  }
}

// K-slice combine: C (op)= sum over slices of the partial tiles, slices in
// ascending order (deterministic).  One CTA per output tile; the tile shape is
// the producing kernel's (args.bm x args.bn).
template <typename T>
__global__ void __launch_bounds__(256) tc_combine_kernel(const __grid_constant__ TcKernelArgs p, T* __restrict__ C) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int BM = p.bm, BN = p.bn;
  int64_t* offc_m = reinterpret_cast<int64_t*>(smem_raw);
  int64_t* offc_n = offc_m + BM;
  const uint32_t bid = blockIdx.x;
  const uint32_t tile_m = bid % p.tiles_m, tile_n = bid / p.tiles_m;
  const size_t tiles = (size_t)p.tiles_m * p.tiles_n;
  for (int i = threadIdx.x; i < BM + BN; i += 256) {
    int64_t dummy;
    if (i < BM) decode(p.M, tile_m * BM + i, p.Mflat, &dummy, &offc_m[i]);
    else decode(p.N, tile_n * BN + (i - BM), p.Nflat, &dummy, &offc_n[i - BM]);
  }
  __syncthreads();
  const size_t tile_elems = (size_t)BM * BN;
  const T* ws = reinterpret_cast<const T*>(p.ws) + (size_t)bid * tile_elems;
  const T alpha = (T)p.alpha;
  for (int e = threadIdx.x; e < BM * BN; e += 256) {
    const int ml = e % BM, nl = e / BM;
    const int64_t cm = offc_m[ml], cn = offc_n[nl];
    if (cm < 0 || cn < 0) continue;
    T s = T(0);
    for (uint32_t sl = 0; sl < p.ksplit; ++sl) s += ws[sl * tiles * tile_elems + e];
    T r = alpha * s;
    if (p.beta) r += C[cn + cm];
    C[cn + cm] = r;
  }
}

}  // namespace tck
