// Persistent, warp-specialised fp64 contraction kernel for sm_100a.
//
// Same tiling, address scheme, shared-memory image and DMMA fragment mapping as
// tc_contract_kernel (tc_kernels.cuh); what changes is WHO does what and WHEN:
//
//   * one CTA per SM lives for the whole contraction and walks a strided list of
//     output tiles;
//   * the first 2*CW warps are two CONSUMER groups (CW = 4, 6 or 8 warps, one per
//     32 x 32 block of the group's BM x BN tile), each group owning its own tile
//     and its own stage ring: shared loads, DMMA and the output of C, nothing
//     else;
//   * the last four warps are the PRODUCERS, two per group: they decode the tile's
//     offset tables, optionally prefetch its C tile into L2 and issue every copy of
//     its stages (cp.async, or one tiled TMA box per operand), running ahead of
//     the consumers by the depth of the ring -- across tile boundaries, so the
//     set-up and load latency of tile i+1 hide behind the products of tile i, and
//     one group's epilogue overlaps the other group's products;
//   * on the 64 x 96 tile one more warpgroup exists; its first lane is the STORE thread: the consumers write
//     whole output tiles into one staging area shared by both groups, the store thread issues one tiled TMA
//     reduce-add / store per tile and frees the area when the copy engine has read it;
//   * stages and tables are handed over through mbarriers in shared memory
//     (cp.async.mbarrier.arrive makes a stage "full" when its copies land);
//   * registers follow the roles (setmaxnreg): producers shrink, consumers grow;
//     every warp executes its setmaxnreg (all four warps of a warpgroup must, or
//     the instruction never completes).
//
// Every mbarrier wait is bounded: a wait that does not complete within
// args.spin_limit polls records an error code in *args.status and the thread leaves
// the kernel; its partners then run out of polls the same way, so the kernel
// always terminates.  The host reads the status word after synchronising.
#pragma once
#include "tc_kernels.cuh"

namespace tck {

// Arrival that fires when all cp.async issued so far by this thread have landed.
__device__ __forceinline__ void mbar_arrive_on_copies(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// One arrival that also announces `bytes` of asynchronous (TMA) traffic for the current phase.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("{\n .reg .b64 st;\n mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n}\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Tiled TMA load of one 2-D box into this CTA only: box corner (c0 = innermost coordinate, c1) of the tensor
// described by `tmap` into shared memory at `dst`; completion is signalled on `bar` as transferred bytes.
// c0 times the element size must be a multiple of 16 bytes; `dst` must be 1024-byte aligned for the
// 128-byte swizzle the descriptor asks for.
__device__ __forceinline__ void tma_load_2d(void* dst, const TcTensorMap* tmap, int c0, int c1, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
               ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void group_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(threads) : "memory");
}
template <int R> __device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(R)); }
template <int R> __device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(R)); }

// Loader / shared-image mode of one operand.
//   LM_ELEM     element copies, external-major image  [k][ext], pitch ROWS+4
//   LM_EXT_VEC  16-byte copies along the external index, same image
//   LM_K_VEC    16-byte copies along the contraction index, contraction-major image [ext][k], pitch 18
//   LM_TMA_K    one tiled TMA copy (cp.async.bulk.tensor.2d) per stage for operands that are plain 2-D
//               matrices: dense contraction-major image [ext][16] with the 128-byte swizzle, i.e. the
//               16-byte chunk c of row e sits at chunk position c ^ (e & 7)
enum { LM_ELEM = 0, LM_EXT_VEC = 1, LM_K_VEC = 2, LM_TMA_K = 3 };

template <int BM_, int BN_, int STAGES_, int MODEX_, int MODEY_>
struct WsCfg {
  using T = double;
  static constexpr int BM = BM_, BN = BN_, BK = 16, STAGES = STAGES_;
  static constexpr int MODEX = MODEX_, MODEY = MODEY_;
  static constexpr int ES = 8, VW = 2;
  static constexpr int GROUPS = 2;
  // Consumer warps of a group: 2 x 2 blocks of 64 x 32 outputs on a 128 x 64 tile, 2 x 3 blocks of 32 x 32
  // on 64 x 96 (six warps: measured faster there than four warps of 32 x 48), 2 x 2 of 32 x 32 on 64 x 64.
  static constexpr int WGM = 2, WGN = BN == 96 ? 3 : 2, CW = WGM * WGN;  // consumer warps per group
  static constexpr int WM = BM / WGM, WN = BN / WGN;
  static constexpr int CONSUMER_THREADS = CW * 32;
  // producer threads per group: two warps where every operand arrives 16 bytes (or a tiled copy) at a time, four
  // where one is gathered element by element (48 eight-byte copies per thread and stage with two warps: the
  // producers, not the tensor pipe, set the pace)
  // (not on the 64 x 96 tile, whose store warpgroup already makes the CTA 640 threads)
  static constexpr int THREADS = ((MODEX == LM_ELEM || MODEY == LM_ELEM) && BN != 96) ? 128 : 64;
  // Whole-tile output (below) pays on the 64 x 96 tile, whose six consumer warps otherwise queue 24 small
  // copies per tile; on 128 x 64 the extra warpgroup costs the consumers registers and measured slower.
  static constexpr bool TILE_OUT = BN == 96;
  static constexpr int STORE_THREADS = TILE_OUT ? 128 : 0;  // one more warpgroup: its first lane issues those copies
  static constexpr int CTA_THREADS = GROUPS * (CONSUMER_THREADS + THREADS) + STORE_THREADS;
  static constexpr int LDK = BK + 2;            // pitch of a contraction-major image (18 = 2 mod 16: conflict-free)
  static constexpr int LDX = MODEX == LM_K_VEC ? LDK : MODEX == LM_TMA_K ? BK : BM + 4;
  static constexpr int LDY = MODEY == LM_K_VEC ? LDK : MODEY == LM_TMA_K ? BK : BN + 4;
  static constexpr bool ANY_TMA = MODEX == LM_TMA_K || MODEY == LM_TMA_K;
  static constexpr int round128(int x) { return (x + 127) / 128 * 128; }  // TMA images start on 1024 bytes
  static constexpr int XIMG_RAW = MODEX == LM_K_VEC ? BM * LDK : MODEX == LM_TMA_K ? BM * BK : BK * (BM + 4);
  static constexpr int YIMG_RAW = MODEY == LM_K_VEC ? BN * LDK : MODEY == LM_TMA_K ? BN * BK : BK * (BN + 4);
  static constexpr int XIMG = ANY_TMA ? round128(XIMG_RAW) : XIMG_RAW;
  static constexpr int YIMG = ANY_TMA ? round128(YIMG_RAW) : YIMG_RAW;
  static constexpr int STAGE_ELEMS = XIMG + YIMG;
  static constexpr uint32_t TMA_BYTES = (MODEX == LM_TMA_K ? BM * BK * 8 : 0) + (MODEY == LM_TMA_K ? BN * BK * 8 : 0);
  static constexpr int FULL_ARRIVALS = THREADS + (ANY_TMA ? 1 : 0);
  static constexpr int TABLE_ELEMS = 2 * BM + 2 * BN;            // offx_m, offc_m, offy_n, offc_n
  // per group: full[STAGES], empty[STAGES], tab_full[2], tab_empty[2]; then staged[2], cfree[2], and eight
  // words used as the mailbox of tile coordinates (two groups x eight ints)
  static constexpr int NBARS = GROUPS * (2 * STAGES + 4) + 4 + 8;
  // Epilogue staging for the bulk reduce: per consumer warp 8 rows of WM outputs, pitch WM+2
  // (16-byte aligned rows, conflict-free 16-byte writes).
  static constexpr int CPITCH = WM + 2;
  static constexpr int CBATCH_ELEMS = 8 * CPITCH;
  static constexpr int BASE_BYTES = NBARS * 8 + GROUPS * 2 * TABLE_ELEMS * 8 + GROUPS * STAGES * STAGE_ELEMS * 8;
  // two staging batches per warp (the copies of one batch drain while the next is written) where they fit
  static constexpr int CBUF = BASE_BYTES + GROUPS * CW * 2 * CBATCH_ELEMS * 8 <= 232448 - 1024 ? 2 : 1;
  static constexpr int CSTAGE_ELEMS = CBUF * CBATCH_ELEMS;
  // Where a whole BM x BN tile fits beside the stages, ONE staging area shared by both groups takes a tile at
  // a time ([n][m], dense): the consumers only write it, a separate thread issues the single tiled TMA copy
  // and waits for it to be read, so no consumer waits for the copy engine.
  static constexpr bool TILE_OK = TILE_OUT && BASE_BYTES + BM * BN * 8 <= 232448 - 1024;
  static constexpr int CREGION_ELEMS =
      (TILE_OK && BM * BN > GROUPS * CW * CSTAGE_ELEMS) ? BM * BN : GROUPS * CW * CSTAGE_ELEMS;
  static constexpr int SMEM_BYTES = BASE_BYTES + CREGION_ELEMS * 8;
  // Registers follow the roles.  The CTA starts with LAUNCH_REGS per thread (what fits 64 K registers, in
  // units of 8); producers shrink to PRODUCER_REGS and the consumers share what that frees.
  static constexpr int LAUNCH_REGS = (65536 / CTA_THREADS) / 8 * 8 > 255 ? 248 : (65536 / CTA_THREADS) / 8 * 8;
  static constexpr int PRODUCER_REGS = 56, STORE_REGS = 40;
  static constexpr int CONSUMER_REGS_RAW =
      (LAUNCH_REGS * CTA_THREADS - PRODUCER_REGS * GROUPS * THREADS - STORE_REGS * STORE_THREADS) /
      (GROUPS * CONSUMER_THREADS) / 8 * 8;
  static constexpr int CONSUMER_REGS = CONSUMER_REGS_RAW > 224 ? 224 : CONSUMER_REGS_RAW;
};

// Producer loaders.  A producer thread keeps what does not change inside a stage in
// registers (its external offsets or its contraction offsets), so that one element
// costs an add, a predicate and the copy.

// 16 bytes along the external index, external-major image.
template <class CF, int ROWS>
__device__ __forceinline__ void ws_load_ext_vec(double* img, const double* __restrict__ g, const int64_t* s_off,
                                                const int64_t* __restrict__ koff, uint32_t k0, uint32_t kend, int ptid) {
  constexpr int LD = ROWS + 4, VPR = ROWS / 2, T = CF::THREADS;
  const uint32_t sbase = smem_u32(img);
  if constexpr (VPR >= T && VPR % T == 0) {
#pragma unroll
    for (int c = 0; c < VPR / T; ++c) {
      const int ev = ptid + c * T;
      const int64_t eo = s_off[ev * 2];
#pragma unroll 8
      for (int kk = 0; kk < CF::BK; ++kk) {
        const bool ok = eo >= 0 && k0 + kk < kend;
        const double* src = ok ? g + eo + koff[k0 + kk] : g;
        cp_async16(sbase + (uint32_t)(kk * LD + ev * 2) * 8u, src, ok);
      }
    }
  } else if constexpr (T % VPR == 0) {
    const int ev = ptid % VPR;
    const int64_t eo = s_off[ev * 2];
#pragma unroll 8
    for (int kk = ptid / VPR; kk < CF::BK; kk += T / VPR) {
      const bool ok = eo >= 0 && k0 + kk < kend;
      const double* src = ok ? g + eo + koff[k0 + kk] : g;
      cp_async16(sbase + (uint32_t)(kk * LD + ev * 2) * 8u, src, ok);
    }
  } else {  // tile widths that neither divide nor are divided by the producer count
    static_assert(VPR * CF::BK % T == 0, "loader shape");
#pragma unroll 4
    for (int sl = ptid; sl < VPR * CF::BK; sl += T) {
      const int ev = sl % VPR, kk = sl / VPR;
      const int64_t eo = s_off[ev * 2];
      const bool ok = eo >= 0 && k0 + kk < kend;
      const double* src = ok ? g + eo + koff[k0 + kk] : g;
      cp_async16(sbase + (uint32_t)(kk * LD + ev * 2) * 8u, src, ok);
    }
  }
}

// 16 bytes along the contraction index, contraction-major image.
template <class CF, int ROWS>
__device__ __forceinline__ void ws_load_k_vec(double* img, const double* __restrict__ g, const int64_t* s_off,
                                              const int64_t* __restrict__ koff, uint32_t k0, uint32_t kend, int ptid) {
  constexpr int KV = CF::BK / 2, T = CF::THREADS;
  static_assert(T % KV == 0 && ROWS % (T / KV) == 0, "loader shape");
  const int kv = ptid % KV;
  const uint32_t k = k0 + kv * 2;
  const bool kok = k < kend;
  const int64_t ko = kok ? koff[k] : 0;
  const uint32_t sbase = smem_u32(img) + (uint32_t)(kv * 2) * 8u;
#pragma unroll 8
  for (int r = ptid / KV; r < ROWS; r += T / KV) {
    const int64_t eo = s_off[r];
    const bool ok = kok && eo >= 0;
    const double* src = ok ? g + eo + ko : g;
    cp_async16(sbase + (uint32_t)(r * CF::LDK) * 8u, src, ok);
  }
}

// Element copies, external-major image.  lg = log2(lanes walking k): a warp covers 2^lg consecutive k
// by 32 >> lg consecutive externals (whole 32-byte sectors along the operand's fastest index).
template <class CF, int ROWS>
__device__ __forceinline__ void ws_load_elem(double* img, const double* __restrict__ g, const int64_t* s_off,
                                             const int64_t* __restrict__ koff, uint32_t k0, uint32_t kend, int ptid,
                                             int lg) {
  constexpr int LD = ROWS + 4, WARPS = CF::THREADS / 32;
  const int lane = ptid & 31, warp = ptid >> 5;
  const uint32_t sbase = smem_u32(img);
  if (lg == 0) {  // lanes walk the external index: few externals, all 16 k per thread
    constexpr int EG = ROWS / 32;  // groups of 32 externals
#pragma unroll
    for (int eg = warp; eg < EG; eg += WARPS) {
      const int el = eg * 32 + lane;
      const int64_t eo = s_off[el];
#pragma unroll 8
      for (int kk = 0; kk < CF::BK; ++kk) {
        const bool ok = eo >= 0 && k0 + kk < kend;
        const double* src = ok ? g + eo + koff[k0 + kk] : g;
        cp_async8(sbase + (uint32_t)(kk * LD + el) * 8u, src, ok);
      }
    }
  } else {  // 4 lanes walk k, 8 lanes walk the external index: 4 contraction offsets live in registers
    const int lk = lane & 3, le = lane >> 2;
    int64_t ko[4];
    bool kok[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t k = k0 + q * 4 + lk;
      kok[q] = k < kend;
      ko[q] = kok[q] ? koff[k] : 0;
    }
#pragma unroll 4
    for (int eg = warp; eg < ROWS / 8; eg += WARPS) {
      const int el = eg * 8 + le;
      const int64_t eo = s_off[el];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const bool ok = kok[q] && eo >= 0;
        const double* src = ok ? g + eo + ko[q] : g;
        cp_async8(sbase + (uint32_t)((q * 4 + lk) * LD + el) * 8u, src, ok);
      }
    }
  }
}

template <class CF, int ROWS, int MODE>
__device__ __forceinline__ void ws_load(double* img, const double* __restrict__ g, const int64_t* s_off,
                                        const int64_t* __restrict__ koff, uint32_t k0, uint32_t kend, int ptid, int lg) {
  if constexpr (MODE == LM_EXT_VEC) ws_load_ext_vec<CF, ROWS>(img, g, s_off, koff, k0, kend, ptid);
  else if constexpr (MODE == LM_K_VEC) ws_load_k_vec<CF, ROWS>(img, g, s_off, koff, k0, kend, ptid);
  else if constexpr (MODE == LM_TMA_K) return;  // fetched by the producer's TMA copy
  else ws_load_elem<CF, ROWS>(img, g, s_off, koff, k0, kend, ptid, lg);
}

// Fragment pair of the DMMA mapping: tile elements (e, e+1) at contraction index k.
template <int MODE, int LD>
__device__ __forceinline__ double2 ws_frag(const double* img, int e, int k) {
  if constexpr (MODE == LM_K_VEC) return make_double2(img[e * LD + k], img[(e + 1) * LD + k]);
  else if constexpr (MODE == LM_TMA_K) {
    // rows e and e+1 (e even): swizzled chunk position of k differs by the row's low bits
    const int c = k >> 1, w = k & 1;
    return make_double2(img[e * 16 + (((c ^ (e & 7)) << 1) | w)], img[(e + 1) * 16 + (((c ^ ((e + 1) & 7)) << 1) | w)]);
  } else return *reinterpret_cast<const double2*>(img + k * LD + e);
}

template <class CF>
__global__ void __launch_bounds__(CF::CTA_THREADS, 1) tc_ws_dmma_kernel(const __grid_constant__ TcKernelArgs p,
                                                                         double* __restrict__ C,
                                                                         const double* __restrict__ X,
                                                                         const double* __restrict__ Y) {
  constexpr int BM = CF::BM, BN = CF::BN, BK = CF::BK, LDX = CF::LDX, LDY = CF::LDY, STAGES = CF::STAGES;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  double* stages = reinterpret_cast<double*>(smem_raw);  // first: TMA images need 1024-byte alignment
  double* cstages = stages + CF::GROUPS * CF::STAGES * CF::STAGE_ELEMS;
  int64_t* tables = reinterpret_cast<int64_t*>(cstages + CF::CREGION_ELEMS);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tables + CF::GROUPS * 2 * CF::TABLE_ELEMS);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  constexpr int CW = CF::CW;
  constexpr int PW = CF::THREADS / 32;  // producer warps per group
  const bool is_store = CF::STORE_THREADS > 0 && warp >= 2 * CW + 2 * PW;
  const bool is_producer = !is_store && warp >= 2 * CW;
  const int gi = is_producer ? (warp - 2 * CW) / PW : is_store ? 0 : warp / CW;  // group served
  uint64_t* staged = bars + CF::GROUPS * (2 * STAGES + 4);  // [2] a group's tile is in the shared staging area
  uint64_t* cfree = staged + 2;                             // [2] group g's staged tile has been read out
  int* mailbox = reinterpret_cast<int*>(cfree + 2);         // [2][8] tensor coordinates of the staged tile
  uint64_t* full = bars + gi * (2 * STAGES + 4);             // [STAGES]
  uint64_t* empty = full + STAGES;                           // [STAGES]
  uint64_t* tab_full = empty + STAGES;                       // [2]
  uint64_t* tab_empty = tab_full + 2;                        // [2]
  int64_t* gtab = tables + gi * 2 * CF::TABLE_ELEMS;         // two table sets, alternating per tile
  double* gstage = stages + gi * STAGES * CF::STAGE_ELEMS;

  if (tid == 32) {  // descriptors into the copy engine's cache before the first copy needs them
    if constexpr (CF::MODEX == LM_TMA_K) asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&p.tmap_x)) : "memory");
    if constexpr (CF::MODEY == LM_TMA_K) asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&p.tmap_y)) : "memory");
    if (p.c_tensor >= 1) asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&p.tmap_c)) : "memory");
    if (p.c_tensor == 2) asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&p.tmap_ct)) : "memory");
  }
  if (tid == 0) {
    for (int q = 0; q < CF::GROUPS; ++q) {
      uint64_t* b = bars + q * (2 * STAGES + 4);
      for (int s = 0; s < STAGES; ++s) { mbar_init(b + s, CF::FULL_ARRIVALS); mbar_init(b + STAGES + s, CW); }
      for (int s = 0; s < 2; ++s) { mbar_init(b + 2 * STAGES + s, CF::THREADS); mbar_init(b + 2 * STAGES + 2 + s, CW); }
    }
    mbar_init(staged, CW);
    mbar_init(staged + 1, CW);
    mbar_init(cfree, 1);
    mbar_init(cfree + 1, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();

  // Work items: output tiles, or -- where the planner sliced the contraction (few tiles, long K) -- (slice, tile)
  // pairs, slices of one tile spread over the CTAs; a slice's result goes to the plan's workspace as a partial tile
  // and tc_combine_kernel adds the slices in ascending order.
  const uint32_t tiles = p.tiles_m * p.tiles_n;
  const uint32_t total = tiles * p.ksplit;
  const bool sliced = p.ksplit > 1;
  const uint32_t first = 2u * blockIdx.x + gi, step = 2u * gridDim.x;
  const bool accumulate = p.beta != 0;
  // contraction range [kb, ke) and number of K steps of work item `item`
  auto k_range = [&](uint32_t item, uint32_t* kb, uint32_t* ke) {
    const uint32_t slice = item / tiles;
    *kb = slice * p.k_chunk;
    *ke = min(p.Kflat, *kb + p.k_chunk);
    return (int)((*ke - *kb + BK - 1) / BK);
  };

  // Whole-tile output: the geometry allows it, the kernel has the room, and the epilogue is the bulk one.
  const bool tile_out = CF::TILE_OK && p.c_tensor == 2 && p.c_mode == 2 && !sliced;

  if (is_store) {
    // --------------------------------------------------------------- store ----
    // One thread takes the staged tiles in the fixed order group 0, group 1, group 0, ... (the order in which
    // the consumers are allowed to fill the area), issues one tiled TMA reduce-add / store per tile and
    // releases the area once the copy engine has read it.
    reg_dec<CF::STORE_REGS>();
    if (!tile_out || warp != 2 * CW + 2 * PW || (tid & 31) != 0) return;
    const uint64_t tmap = reinterpret_cast<uint64_t>(&p.tmap_ct);
    const uint32_t src = smem_u32(cstages);
    for (uint32_t t = 0;; ++t) {
      bool any = false;
      for (int g = 0; g < 2; ++g) {
        if (2u * blockIdx.x + g + t * step >= total) continue;
        any = true;
        if (!mbar_wait(&staged[g], t & 1, p.status, 6, p.spin_limit)) return;
        const int* mb = mailbox + g * 8;
        if (accumulate)
          asm volatile(
              "cp.reduce.async.bulk.tensor.5d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2, %3, %4, %5}], [%6];\n" ::"l"(tmap),
              "r"(mb[0]), "r"(0), "r"(mb[2]), "r"(mb[3]), "r"(mb[4]), "r"(src)
              : "memory");
        else
          asm volatile(
              "cp.async.bulk.tensor.5d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3, %4, %5}], [%6];\n" ::"l"(tmap),
              "r"(mb[0]), "r"(0), "r"(mb[2]), "r"(mb[3]), "r"(mb[4]), "r"(src)
              : "memory");
        asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
        mbar_arrive(&cfree[g]);
      }
      if (!any) break;
    }
    asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");
    return;
  }

  if (is_producer) {
    // ------------------------------------------------------------ producer ----
    reg_dec<CF::PRODUCER_REGS>();
    const int ptid = tid - 2 * CF::CONSUMER_THREADS - gi * CF::THREADS;
    const int lgx = p.lanes_k_x == 1 ? 0 : 2, lgy = p.lanes_k_y == 1 ? 0 : 2;
    uint32_t it = 0, titer = 0;
    for (uint32_t tile = first; tile < total; tile += step, ++titer) {
      const uint32_t par = titer & 1;
      int64_t* offx_m = gtab + par * CF::TABLE_ELEMS;
      int64_t* offc_m = offx_m + BM;
      int64_t* offy_n = offc_m + BM;
      int64_t* offc_n = offy_n + BN;
      if (!mbar_wait(&tab_empty[par], ((titer >> 1) & 1) ^ 1, p.status, 1, p.spin_limit)) return;
      uint32_t tm, tn, kbeg, kend;
      tile_coords(p, tile % tiles, &tm, &tn);
      const int nk = k_range(tile, &kbeg, &kend);
      const uint32_t m0 = tm * BM, n0 = tn * BN;
      for (int i = ptid; i < BM + BN; i += CF::THREADS) {
        if (i < BM) decode(p.M, m0 + i, p.Mflat, &offx_m[i], &offc_m[i]);
        else decode(p.N, n0 + (i - BM), p.Nflat, &offy_n[i - BM], &offc_n[i - BM]);
      }
      mbar_arrive(&tab_full[par]);            // consumers may read the tables once all 64 have arrived
      group_bar_sync(1 + gi, CF::THREADS);    // ... and so may this group's producers
      auto prefetch_c = [&]() {
        constexpr int SEC = 4;                // doubles per 32-byte sector
        constexpr int SPR = BM / SEC;
        for (int i = ptid; i < SPR * BN; i += CF::THREADS) {
          const int64_t cm = offc_m[(i % SPR) * SEC], cn = offc_n[i / SPR];
          if (cm >= 0 && cn >= 0) asm volatile("prefetch.global.L2 [%0];\n" ::"l"(C + cn + cm));
        }
      };
      const bool pf = accumulate && p.prefetch_dist != 0 && !sliced;
      if (pf && !p.c_stream) prefetch_c();
      for (int ks = 0; ks < nk; ++ks, ++it) {
        const uint32_t s = it % STAGES;
        if (!mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, p.status, 2, p.spin_limit)) return;
        double* xs = gstage + s * CF::STAGE_ELEMS;
        double* ys = xs + CF::XIMG;
        const uint32_t k0 = kbeg + (uint32_t)ks * BK;
        if constexpr (CF::ANY_TMA) {
          if (ptid == 0) {
            mbar_arrive_expect_tx(&full[s], CF::TMA_BYTES);
            if constexpr (CF::MODEX == LM_TMA_K) tma_load_2d(xs, &p.tmap_x, (int)k0, (int)m0, &full[s]);
            if constexpr (CF::MODEY == LM_TMA_K) tma_load_2d(ys, &p.tmap_y, (int)k0, (int)n0, &full[s]);
          }
        }
        ws_load<CF, BM, CF::MODEX>(xs, X, offx_m, p.koff_x, k0, kend, ptid, lgx);
        ws_load<CF, BN, CF::MODEY>(ys, Y, offy_n, p.koff_y, k0, kend, ptid, lgy);
        // tests only: one producer thread of CTA 0 never announces its copies of one stage, so that stage stays
        // "not full" and every thread that depends on it runs out of polls
        if (p.test_fault == 1 && blockIdx.x == 0 && gi == 0 && it == 1 && ptid == 7) continue;
        mbar_arrive_on_copies(&full[s]);
      }
      if (pf && p.c_stream) prefetch_c();
    }
    return;
  }

  // -------------------------------------------------------------- consumer ----
  reg_inc<CF::CONSUMER_REGS>();
  constexpr int WM = CF::WM, WN = CF::WN;
  constexpr int MB2 = WM / 16, NB2 = WN / 16;
  const int lane = tid & 31, cw = warp % CW;
  const int g = lane >> 2, t = lane & 3;
  const int wm0 = (cw % CF::WGM) * WM, wn0 = (cw / CF::WGM) * WN;
  const double alpha = p.alpha;
  uint32_t it = 0, titer = 0;
  for (uint32_t tile = first; tile < total; tile += step, ++titer) {
    const uint32_t par = titer & 1;
    const int64_t* offc_m = gtab + par * CF::TABLE_ELEMS + BM;
    const int64_t* offc_n = offc_m + BM + BN;
    double acc[2 * NB2][2 * MB2][2];
#pragma unroll
    for (int j = 0; j < 2 * NB2; ++j)
#pragma unroll
      for (int i = 0; i < 2 * MB2; ++i) { acc[j][i][0] = 0.0; acc[j][i][1] = 0.0; }
    // Optional (c_mode 1, 32-byte-contiguous output): the accumulators start as alpha*C.  The producers
    // prefetched this tile's C into L2 a whole tile ago, all loads go out at once and overlap the wait for
    // the first stage; the epilogue is then stores only.
    uint32_t kbeg, kend;
    const int nk = k_range(tile, &kbeg, &kend);
    const bool from_c = accumulate && p.c_mode == 1 && p.vec_c == 4 && !sliced;
    if (from_c) {
      if (!mbar_wait(&tab_full[par], (titer >> 1) & 1, p.status, 5, p.spin_limit)) return;
#pragma unroll
      for (int nb = 0; nb < 2 * NB2; ++nb) {
        const int64_t cn = offc_n[wn0 + 16 * (nb >> 1) + 2 * g + (nb & 1)];
#pragma unroll
        for (int i = 0; i < MB2; ++i) {
          const int64_t co = offc_m[wm0 + 16 * i + 4 * t];
          if (cn < 0 || co < 0) continue;
          const double2* src = reinterpret_cast<const double2*>(C + cn + co);
          const double2 v0 = src[0], v1 = src[1];
          acc[nb][2 * i][0] = alpha * v0.x;
          acc[nb][2 * i + 1][0] = alpha * v0.y;
          acc[nb][2 * i][1] = alpha * v1.x;
          acc[nb][2 * i + 1][1] = alpha * v1.y;
        }
      }
    }

    for (int ks = 0; ks < nk; ++ks, ++it) {
      const uint32_t s = it % STAGES;
      if (!mbar_wait(&full[s], (it / STAGES) & 1, p.status, 3, p.spin_limit)) return;
      const double* xs = gstage + s * CF::STAGE_ELEMS;
      const double* ys = xs + CF::XIMG;
      const int kleft = (int)(kend - kbeg) - ks * BK;
      const int nks = kleft >= BK ? BK / 4 : (kleft + 3) / 4;
#pragma unroll
      for (int kq = 0; kq < BK / 4; ++kq) {
        if (kq < nks) {
          const int k = kq * 4 + t;
          double2 xf[MB2], yf[NB2];
#pragma unroll
          for (int i = 0; i < MB2; ++i) xf[i] = ws_frag<CF::MODEX, LDX>(xs, wm0 + 2 * g + i * 16, k);
#pragma unroll
          for (int j = 0; j < NB2; ++j) yf[j] = ws_frag<CF::MODEY, LDY>(ys, wn0 + 2 * g + j * 16, k);
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
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);  // this warp no longer reads the stage
    }

    // ---- epilogue: read-modify-write of C (the tile was prefetched into L2 by the producers) ----
    if (!from_c && !mbar_wait(&tab_full[par], (titer >> 1) & 1, p.status, 4, p.spin_limit)) return;
    const bool rmw = accumulate && !from_c;
    // c_mode 2: the warp's tile leaves through shared memory as bulk asynchronous copies, one per output
    // row (WM contiguous elements): `+=`/`-=` become reduce-adds performed by the memory system, so the SM
    // neither loads C nor waits for it.  Needs the warp's WM outputs of a row to be contiguous in C.
    bool bulk = false;
    if (p.c_mode == 2 && p.vec_c == 4 && !from_c) {
      const int64_t c_lo = offc_m[wm0], c_hi = offc_m[wm0 + WM - 1];
      bulk = c_lo >= 0 && c_hi == c_lo + WM - 1;  // uniform across the warp
    }
    // Tensor form of the same idea: a batch of 8 rows is one box of the rank-5 descriptor of C, so one tiled
    // TMA reduce-add (or store) per batch replaces eight per-row copies.  Rows and columns beyond the tensor are
    // clipped by the copy engine; boxes that lie outside altogether are not issued.
    uint32_t tm, tn;
    tile_coords(p, tile % tiles, &tm, &tn);
    const uint32_t m_idx = tm * BM + wm0, n_base = tn * BN + wn0;
    if (sliced) {
      // partial tile of this slice, [n][m] as tc_combine_kernel reads it (every element, padding included)
      double* ws = reinterpret_cast<double*>(p.ws) +
                   ((size_t)(tile / tiles) * tiles + (size_t)tn * p.tiles_m + tm) * (size_t)(BM * BN);
#pragma unroll
      for (int nb = 0; nb < 2 * NB2; ++nb) {
        double* row = ws + (size_t)(wn0 + 16 * (nb >> 1) + 2 * g + (nb & 1)) * BM + wm0 + 4 * t;
#pragma unroll
        for (int i = 0; i < MB2; ++i) {
          double2* dst = reinterpret_cast<double2*>(row + 16 * i);
          dst[0] = make_double2(acc[nb][2 * i][0], acc[nb][2 * i + 1][0]);
          dst[1] = make_double2(acc[nb][2 * i][1], acc[nb][2 * i + 1][1]);
        }
      }
    } else if (tile_out) {
      // Whole tile through the shared staging area, filled in the order g0, g1, g0, ...: use number u may start
      // once use u - 1 has been read out.  After the first wait the two groups stay out of phase.
      // The area is used in the order (0,g0) (0,g1) (1,g0) (1,g1) ...: group 1 may write tile t once group 0's tile
      // t has been read out, group 0 may write tile t once group 1's tile t - 1 has (which implies everything
      // before it).  One barrier per group keeps every waiter within one phase of what it waits for -- with a
      // single barrier a group that returns quickly (short contractions) could be two phases off, which a parity
      // wait cannot tell apart.
      if (gi == 1) { if (!mbar_wait(&cfree[0], titer & 1, p.status, 7, p.spin_limit)) return; }
      else if (titer > 0) { if (!mbar_wait(&cfree[1], (titer - 1) & 1, p.status, 7, p.spin_limit)) return; }
      double* tb = cstages;
#pragma unroll
      for (int nb = 0; nb < 2 * NB2; ++nb) {
        double* row = tb + (wn0 + 16 * (nb >> 1) + 2 * g + (nb & 1)) * BM + wm0 + 4 * t;
#pragma unroll
        for (int i = 0; i < MB2; ++i) {
          double2* dst = reinterpret_cast<double2*>(row + 16 * i);
          dst[0] = make_double2(alpha * acc[nb][2 * i][0], alpha * acc[nb][2 * i + 1][0]);
          dst[1] = make_double2(alpha * acc[nb][2 * i][1], alpha * acc[nb][2 * i + 1][1]);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        if (cw == 0) {
          const uint32_t m0t = m_idx - wm0, n0t = n_base - wn0;
          const uint32_t e0 = p.cmap.e0, f0 = p.cmap.f0;
          const int ne = p.cmap.ne, me = p.cmap.me;
          int x3 = 0, x4 = 0;
          const uint32_t rm = m0t / e0, rn = n0t / f0;
          if (me == 2) { x3 = (int)(rm % p.cmap.ext[0]); x4 = (int)(rm / p.cmap.ext[0]); }
          else if (me == 1) { if (ne == 0) x3 = (int)rm; else x4 = (int)rm; }
          if (ne == 2) { x3 = (int)(rn % p.cmap.ext[0]); x4 = (int)(rn / p.cmap.ext[0]); }
          else if (ne == 1) x3 = (int)rn;
          int* mb = mailbox + gi * 8;
          mb[0] = (int)(m0t % e0);
          mb[2] = (int)((n0t % f0) >> 1);
          mb[3] = x3;
          mb[4] = x4;
        }
        mbar_arrive(&staged[gi]);  // release: the mailbox and this warp's part of the tile are visible
      }
    } else if (p.c_tensor && p.c_mode == 2 && !from_c) {
      if (m_idx < p.Mflat) {
        double* cst = cstages + (gi * CW + cw) * CF::CSTAGE_ELEMS;
        const uint64_t tmap = reinterpret_cast<uint64_t>(&p.tmap_c);
        const uint32_t e0 = p.cmap.e0, f0 = p.cmap.f0;
        const int ne = p.cmap.ne, me = p.cmap.me;
        int xm[2] = {0, 0};  // coordinates 3 and 4: slower N dimensions first, then slower M dimensions
        {
          const uint32_t r = m_idx / e0;
          if (me == 2) { xm[0] = (int)(r % p.cmap.ext[0]); xm[1] = (int)(r / p.cmap.ext[0]); }
          else if (me == 1) { if (ne == 0) xm[0] = (int)r; else xm[1] = (int)r; }
        }
        const int c0 = (int)(m_idx % e0);
#pragma unroll
        for (int j = 0; j < NB2; ++j) {
          const uint32_t n_idx = n_base + 16 * j;
          if (n_idx >= p.Nflat) break;  // uniform across the warp
          int x3 = xm[0], x4 = xm[1];
          {
            const uint32_t r = n_idx / f0;
            if (ne == 2) { x3 = (int)(r % p.cmap.ext[0]); x4 = (int)(r / p.cmap.ext[0]); }
            else if (ne == 1) x3 = (int)r;
          }
          const int q = (int)((n_idx % f0) >> 1);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int nb = 2 * j + h;
            asm volatile("cp.async.bulk.wait_group.read %0;\n" ::"n"(CF::CBUF - 1) : "memory");
            __syncwarp();
            double* cbuf = cst + (nb % CF::CBUF) * CF::CBATCH_ELEMS;  // dense rows of WM: the box image
#pragma unroll
            for (int i = 0; i < MB2; ++i) {
              double2* dst = reinterpret_cast<double2*>(cbuf + g * WM + 16 * i + 4 * t);
              dst[0] = make_double2(alpha * acc[nb][2 * i][0], alpha * acc[nb][2 * i + 1][0]);
              dst[1] = make_double2(alpha * acc[nb][2 * i][1], alpha * acc[nb][2 * i + 1][1]);
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              const uint32_t src = smem_u32(cbuf);
              if (accumulate)
                asm volatile(
                    "cp.reduce.async.bulk.tensor.5d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2, %3, %4, %5}], [%6];\n" ::"l"(tmap),
                    "r"(c0), "r"(h), "r"(q), "r"(x3), "r"(x4), "r"(src)
                    : "memory");
              else
                asm volatile(
                    "cp.async.bulk.tensor.5d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3, %4, %5}], [%6];\n" ::"l"(tmap),
                    "r"(c0), "r"(h), "r"(q), "r"(x3), "r"(x4), "r"(src)
                    : "memory");
              asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
            }
          }
        }
      }
    } else if (bulk) {
      double* cst = cstages + (gi * CW + cw) * CF::CSTAGE_ELEMS;
      const int64_t c_lo = offc_m[wm0];
#pragma unroll
      for (int nb = 0; nb < 2 * NB2; ++nb) {
        // the batch that last used this staging buffer must have been read out of it
        asm volatile("cp.async.bulk.wait_group.read %0;\n" ::"n"(CF::CBUF - 1) : "memory");
        __syncwarp();
        double* cbuf = cst + (nb % CF::CBUF) * CF::CBATCH_ELEMS;
#pragma unroll
        for (int i = 0; i < MB2; ++i) {
          double2* dst = reinterpret_cast<double2*>(cbuf + g * CF::CPITCH + 16 * i + 4 * t);
          dst[0] = make_double2(alpha * acc[nb][2 * i][0], alpha * acc[nb][2 * i + 1][0]);
          dst[1] = make_double2(alpha * acc[nb][2 * i][1], alpha * acc[nb][2 * i + 1][1]);
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        __syncwarp();
        if (lane < 8) {
          const int64_t cn = offc_n[wn0 + 16 * (nb >> 1) + 2 * lane + (nb & 1)];
          if (cn >= 0) {
            const uint32_t src = smem_u32(cbuf + lane * CF::CPITCH);
            double* dstg = C + cn + c_lo;
            if (accumulate)
              asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f64 [%0], [%1], %2;\n" ::"l"(dstg),
                           "r"(src), "n"(WM * 8)
                           : "memory");
            else
              asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n" ::"l"(dstg), "r"(src),
                           "n"(WM * 8)
                           : "memory");
          }
          asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
        }
      }
    } else if (p.vec_c == 4) {
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
              c0[h][i] = src[0];
              c1[h][i] = src[1];
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
            dst[0] = make_double2(fma(alpha, acc[nb][2 * i][0], c0[h][i].x), fma(alpha, acc[nb][2 * i + 1][0], c0[h][i].y));
            dst[1] = make_double2(fma(alpha, acc[nb][2 * i][1], c1[h][i].x), fma(alpha, acc[nb][2 * i + 1][1], c1[h][i].y));
          }
        }
      }
    } else {
      // Any alignment, any strides: the warp's rows pass through its staging buffer so that the read-modify-write
      // of a row is done by consecutive lanes on consecutive m -- whole sectors per instruction wherever
      // consecutive m are contiguous in C, which fragment-order accesses of 8 bytes are not.
      double* cst = cstages + (gi * CW + cw) * CF::CSTAGE_ELEMS;
      asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");  // an earlier tile's copies may still read it
      __syncwarp();
#pragma unroll
      for (int nb = 0; nb < 2 * NB2; ++nb) {
#pragma unroll
        for (int i = 0; i < MB2; ++i) {
          double2* dst = reinterpret_cast<double2*>(cst + g * CF::CPITCH + 16 * i + 4 * t);
          dst[0] = make_double2(alpha * acc[nb][2 * i][0], alpha * acc[nb][2 * i + 1][0]);
          dst[1] = make_double2(alpha * acc[nb][2 * i][1], alpha * acc[nb][2 * i + 1][1]);
        }
        __syncwarp();
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const int64_t cn = offc_n[wn0 + 16 * (nb >> 1) + 2 * r + (nb & 1)];
          if (cn < 0) continue;  // uniform across the warp
#pragma unroll
          for (int m = lane; m < WM; m += 32) {
            const int64_t co = offc_m[wm0 + m];
            if (co < 0) continue;
            double* q = C + cn + co;
            const double v = cst[r * CF::CPITCH + m];
            *q = accumulate ? v + *q : v;
          }
        }
        __syncwarp();
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&tab_empty[par]);  // the producers may overwrite this table set
  }
  asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");  // outstanding bulk copies of this thread
}

}  // namespace tck
