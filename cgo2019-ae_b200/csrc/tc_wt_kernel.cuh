// Persistent, warp-specialised fp32 contraction kernel for sm_100a: three TF32 products per fp32 product on
// tcgen05.mma, two accumulators and the A operand in tensor memory, the output tile staged in shared memory.
//
// Same tiling, address scheme, split (v = hi + lo) and X images as the one-CTA-per-tile tcgen05 path of
// tc_contract_kernel (tc_kernels.cuh); what changes is WHO does what and WHEN, and where the A operand lives.  One CTA per SM lives
// for the whole contraction and walks a strided list of BM x 128 output tiles; its warps have fixed roles that meet
// only through mbarriers in shared memory:
//
//   warps 0-7   EPILOGUE  one thread per lane of D (n) and half of its columns (m).  Waits for an accumulator, reads
//                         its columns with tcgen05.ld, frees the accumulator, and puts alpha * D into the tile buffer
//                         in shared memory.  A contraction longer than SEG_STEPS K steps is cut into segments that
//                         alternate between the two accumulators and are added into the buffer one after another in
//                         round-to-nearest fp32, so no tensor-core accumulation chain exceeds 512 products and the
//                         output still moves once.
//   warps 8-15  SPLIT     turn the gathered fp32 stage into the hi and lo TF32 values the MMA reads; one 16-byte chunk
//                         of each operand per thread and group of eight k.  X (the MMA's B operand) goes into
//                         images in shared memory (128-byte core matrices, K-major); Y (its A operand) goes
//                         straight into tensor memory with tcgen05.st -- row n in lane n, one column per k -- so
//                         its images are neither written to shared memory nor read from it three times.
//   warps 16-19 LOADERS   issue every cp.async of the stages (the three loader shapes of tc_kernels.cuh) -- or, for an
//                         operand that is a plain 2-D matrix with the contraction index fastest, one tiled TMA box
//                         per stage from a single thread -- running ahead across tile boundaries by the depth of the
//                         ring.  Row offsets live in registers, the
//                         contraction offsets of a step in shared memory (a dependent global load per copy would
//                         serialise the issue).
//   warp 20     MMA       owns tensor memory; its first lane issues lo*hi, hi*lo, hi*hi for every group of eight k
//                         and commits onto the barriers that free the images and publish the accumulator.  Images
//                         change hands eight k at a time (short contractions) or a K step at a time (long ones).
//   warp 21     FETCH     only where the caller asked for sums to be stored (tc_options.c_path 1): brings the tile's
//                         old values from C up to CBUFS tiles ahead into the tile buffer with bulk asynchronous
//                         copies.  By default nothing is fetched: the buffer holds the products alone.
//   warp 22     STORE     sends a finished tile to C with bulk asynchronous copies -- reduce-adds for `+=` / `-=`
//                         (the memory system adds; measured faster than fetching and storing on every shape tried),
//                         plain stores for `=` -- and frees its buffer when they have read it (one tile late where
//                         there are several buffers, so that the read-out overlaps the next tile's copies).
//   warp 23               no work.
//
// The tile lies in shared memory in the order it has in C: rows split into runs of E0 = args.epi_run elements that
// are contiguous in C; element (m, n) sits at (m / E0) * run_stride + n * pitch + m % E0.  Where consecutive n are
// adjacent in C (args.epi_n_span) and E0 is short, pitch = E0 and a run leaves as one or two large chunks; otherwise
// every (run, n) is one chunk and pitch = E0 + 4 where that makes it 4 mod 8 words (conflict-free 16-byte accesses by
// lanes on consecutive n).
//
// Every mbarrier wait is bounded (args.spin_limit polls); a wait that gives up records its code in *args.status and the
// role leaves its loop; the others then run out of polls the same way.  The MMA warp frees tensor memory after the
// epilogue warps have left, on every path.
#pragma once
#include "tc_ws_kernel.cuh"

namespace tck {

template <int BM_, int MODEX_, int MODEY_>
struct WtCfg {
  using T = float;
  static constexpr int BM = BM_, BN = 128, BK = 16;
  // 0 element copies, 1 16 bytes along the external index, 2 16 bytes along k, 3 one tiled TMA box per stage (rows of
  // 16 k, 64-byte swizzle), 4 the same for an operand whose external index is the fastest (16 rows of k, dense)
  static constexpr int MODEX = MODEX_, MODEY = MODEY_;
  static constexpr bool VECX = MODEX == 1, VECY = MODEY == 1, KVX = MODEX == 2, KVY = MODEY == 2;
  static constexpr bool TMAX = MODEX == 3, TMAY = MODEY == 3, TMAXE = MODEX == 4, TMAYE = MODEY == 4;
  static constexpr bool ANY_TMA = TMAX || TMAY || TMAXE || TMAYE;
  static constexpr int ES = 4, VW = 4, LDKV = 16 + 4;
  static constexpr int THREADS = 128, WARPS = 4;  // the LOADER role, as the shared loaders see it
  static constexpr int LDX = TMAXE ? BM : BM + 4, LDY = TMAYE ? BN : BN + 4;  // a box is dense
  // A TMA box lands as rows of 16 k (64 bytes) under the 64-byte swizzle, whose pattern repeats every 512 bytes:
  // with a box in the stage, both images are rounded to 1024 bytes and the stages lead the shared memory.
  static constexpr int XIMG_RAW = KVX ? BM * LDKV : TMAX ? BM * BK : BK * LDX;  // (mode 4: BK rows of BM)
  static constexpr int YIMG_RAW = KVY ? BN * LDKV : TMAY ? BN * BK : BK * LDY;
  static constexpr int XIMG = ANY_TMA ? (XIMG_RAW + 255) / 256 * 256 : XIMG_RAW;
  static constexpr int YIMG = ANY_TMA ? (YIMG_RAW + 255) / 256 * 256 : YIMG_RAW;
  static constexpr int STAGE_ELEMS = XIMG + YIMG;
  static constexpr uint32_t TMA_BYTES = (TMAX || TMAXE ? BM * BK * 4 : 0) + (TMAY || TMAYE ? BN * BK * 4 : 0);
  static constexpr int FULL_ARRIVALS = THREADS + (ANY_TMA ? 1 : 0);  // the loaders' copies, and the announcement of the boxes
  static constexpr int UMMA_ELEMS = 2 * BK * BM;         // hi and lo images of X for one K step (those of Y live in tensor memory)
  static constexpr int GROUPS = 1;                       // tiles a CTA works on at a time (launch arithmetic)
  // Six warpgroups: epilogue, epilogue, split, split, loaders, {MMA, fetch, store, a warp without work}.
  static constexpr int CTA_THREADS = 24 * 32;
  static constexpr int SPLIT_WARPS = 8, SPLIT_THREADS = 256, EPI_WARPS = 8;
  // Registers follow the roles (setmaxnreg, every warp of a warpgroup executes it): the CTA starts with 80 per thread
  // (65536 / 768, in units of 8); split, MMA, fetch and store warps shrink, the epilogue and the loaders grow.
  // What the growing warps take must have been given up by the shrinking ones of the same CTA: an increase waits for
  // registers released inside the CTA, not for the multiprocessor's spare ones.
  static constexpr int LAUNCH_REGS = 80, SMALL_REGS = 48, EPILOGUE_REGS = 104, LOADER_REGS = 128;
  static_assert(256 * (EPILOGUE_REGS - LAUNCH_REGS) + 128 * (LOADER_REGS - LAUNCH_REGS) <= 384 * (LAUNCH_REGS - SMALL_REGS),
                "register increases must be covered by the decreases");
  static_assert(CTA_THREADS * LAUNCH_REGS <= 65536 && (65536 / CTA_THREADS) / 8 * 8 == LAUNCH_REGS, "launch registers");
  static constexpr int SEG_STEPS = 32;                   // K steps per accumulation chain: 512 products
  // Tensor memory: two accumulators of 128 columns, then the hi / lo values of Y (the MMA's A operand: row n in lane
  // n, one column per k): per image slot 2 groups of 8 k x (8 hi + 8 lo) columns.
  static constexpr int TMEM_COLS = 512, A_COLS = 256, A_SLOT_COLS = 32;
  // output tile buffers: room for the padded layout (pitch E0 + 4 only where E0 >= 64: at most BM / 64 runs)
  static constexpr int CTILE_ELEMS = BN * (BM + 4 * (BM / 64));
  // Shared memory is carved at run time (args.out_bufs tile buffers, args.img_sets image sets, args.ring_stages
  // stages, chosen at launch): short contractions want tile buffers (the output stream is what has to be kept in flight),
  // long ones want operand stages and a second image set (the MMAs are).
  static constexpr int MAX_STAGES = 8, MAX_CBUFS = 3, MAX_IMGS = 2;
  static constexpr int NBARS = (2 * MAX_STAGES + 4 * MAX_IMGS + 4 + 3 * MAX_CBUFS + 1) / 2 * 2;  // even: what follows stays 16-byte aligned
  static constexpr int KSTEPS_KEPT = 8;  // contractions of at most this many steps keep all their offsets in shared memory
  static constexpr int HEAD_BYTES = NBARS * 8 + 16 + KSTEPS_KEPT * 32 * 8;  // barriers, tensor-memory slot, contraction offsets
  static constexpr int SMEM_BYTES = 232448;
  static_assert(HEAD_BYTES % 16 == 0 && (STAGE_ELEMS * 4) % 16 == 0, "barriers, images and tile buffers start on 16 bytes");
  static_assert(!ANY_TMA || (XIMG * 4) % 1024 == 0 && (YIMG * 4) % 1024 == 0, "boxes start on the swizzle's period");
  static_assert(BM % 32 == 0 && BM <= 128, "a warp reads BM / 2 columns, 16 at a time; an accumulator has 128 columns");
  // stages that fit beside `cbufs` tile buffers and `imgs` image sets
  static constexpr int stages_for(int cbufs, int imgs) {
    const int left = SMEM_BYTES - HEAD_BYTES - cbufs * CTILE_ELEMS * 4 - imgs * UMMA_ELEMS * 4;
    const int n = left / (STAGE_ELEMS * 4);
    return n > MAX_STAGES ? MAX_STAGES : n;
  }
  static_assert(stages_for(BM <= 96 ? 3 : 2, 1) >= 2 && stages_for(1, MAX_IMGS) >= 2, "shared memory");
};

// What one loader thread copies per stage, fixed for the whole kernel: up to PER slots, each a cp.async of 16 bytes
// (along the external index: mode 1; along k: mode 2) or of one element (mode 0, lanes arranged as in ElemSlots so
// that whole 32-byte sectors are fetched).  A slot packs its element offset inside the stage image (bits 0-15), its
// k inside the step (16-23) and its row (24-31).  The rows' operand offsets are computed once per tile, straight from
// the tile's first flattened index (classes of one or two fused dimensions need one division per tile and a
// multiply-add per row; the row's digits inside the first dimension are fixed per thread), and stay in registers; a
// step then costs one shared-memory read (the contraction offset) and the copy.
template <class CF, int ROWS, int MODE, int LD>
struct WtSlots {
  static constexpr int PER = MODE == 0 ? ROWS * 16 / 128 : (ROWS * 4 + 127) / 128;
  static constexpr uint32_t kNone = 0xffffffffu;
  // Element slots come in pairs on the same row (two groups of k): one offset per pair.
  static constexpr int NROW = MODE == 0 ? PER / 2 : PER;
  static_assert(MODE != 0 || PER % 2 == 0, "element slots pair up");
  __host__ __device__ static constexpr int row_of(int j) { return MODE == 0 ? j >> 1 : j; }
  uint32_t slot[PER];
  uint32_t digit[NROW];  // row / e0 (bits 8-15) and row % e0 (bits 0-7), e0 = extent of the class's first dimension
  int64_t eo[NROW];
  __device__ __forceinline__ void init(int ptid, int lg, uint32_t e0) {
    const int lane = ptid & 31, warp = ptid >> 5;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      int kk, el, off;
      bool valid = true;
      if constexpr (MODE >= 3) {
        kk = 0; el = 0; off = 0; valid = false;  // the box is fetched by one thread's TMA copy
      } else if constexpr (MODE == 2) {
        const int f = ptid + 128 * j;
        el = f >> 2; kk = 4 * (f & 3); off = el * CF::LDKV + kk;
        valid = el < ROWS;
      } else if constexpr (MODE == 1) {
        constexpr int VPR = ROWS / 4;
        const int sidx = ptid + 128 * j;
        kk = sidx / VPR; el = 4 * (sidx % VPR); off = kk * LD + el;
        valid = kk < 16;
      } else {
        const int lk = lane & ((1 << lg) - 1), le = lane >> lg, ks_bits = 4 - lg;
        const int slab = warp * PER + j;
        kk = ((slab & ((1 << ks_bits) - 1)) << lg) + lk;
        el = ((slab >> ks_bits) << (5 - lg)) + le;
        off = kk * LD + el;
      }
      slot[j] = valid ? ((uint32_t)off | ((uint32_t)kk << 16) | ((uint32_t)el << 24)) : kNone;
      digit[row_of(j)] = (((uint32_t)el / e0) << 8) | ((uint32_t)el % e0);
      eo[row_of(j)] = -1;
    }
  }
  // Operand offsets of this thread's rows in the tile that starts at flattened index `flat0` of class `d`.
  __device__ __forceinline__ void rows(const TcDims& d, uint32_t flat0, uint32_t limit) {
    if constexpr (MODE >= 3) return;
    const uint32_t e0 = d.extent[0];
    const uint32_t rest0 = flat0 / e0, b0 = flat0 - rest0 * e0;
#pragma unroll
    for (int r = 0; r < NROW; ++r) {
      const uint32_t sl = slot[MODE == 0 ? 2 * r : r], el = sl >> 24;
      if (sl == kNone || flat0 + el >= limit) { eo[r] = -1; continue; }
      if (d.n <= 2) {
        uint32_t d0 = b0 + (digit[r] & 0xffu), carry = digit[r] >> 8;
        if (d0 >= e0) { d0 -= e0; ++carry; }
        eo[r] = (int64_t)d0 * d.s_in[0] + (d.n == 2 ? (int64_t)(rest0 + carry) * d.s_in[1] : 0);
      } else {
        int64_t unused;
        decode(d, flat0 + el, limit, &eo[r], &unused);
      }
    }
  }
  // (a last step of at most eight k is split and multiplied as one group of eight: nobody reads its k >= 8)
  __device__ __forceinline__ void issue(float* img, const float* __restrict__ g, const int64_t* kr, uint32_t k0, uint32_t kend) const {
    if constexpr (MODE >= 3) return;
    const uint32_t sbase = smem_u32(img);
    const uint32_t kmax = kend - k0 <= 8u ? 8u : 16u;
    int64_t ko[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) ko[j] = kr[(slot[j] >> 16) & 0xffu];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      if (slot[j] == kNone || ((slot[j] >> 16) & 0xffu) >= kmax) continue;
      const bool ok = eo[row_of(j)] >= 0 && k0 + ((slot[j] >> 16) & 0xffu) < kend;
      const float* src = ok ? g + eo[row_of(j)] + ko[j] : g;
      if constexpr (MODE == 0) cp_async4(sbase + (slot[j] & 0xffffu) * 4u, src, ok);
      else cp_async16(sbase + (slot[j] & 0xffffu) * 4u, src, ok);
    }
  }
};

// Bulk asynchronous copy global -> shared, completion counted in bytes on an mbarrier of this CTA.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void bulk_reduce_add(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;\n" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}

template <class CF>
__global__ void __launch_bounds__(CF::CTA_THREADS, 1) tc_wt_tf32_kernel(const __grid_constant__ TcKernelArgs p,
                                                                         float* __restrict__ C,
                                                                         const float* __restrict__ X,
                                                                         const float* __restrict__ Y) {
  constexpr int BM = CF::BM, BN = CF::BN, BK = CF::BK;
  const int STAGES = p.ring_stages, CBUFS = p.out_bufs, IMGS = p.img_sets;
  // Image units, handed from the split warps to the MMA thread through two slots.  With one image set a unit is a
  // group of eight k (the two halves of the set take turns: finer hand-over, which short contractions want); with two
  // sets a unit is a whole K step of sixteen and a slot is a set (half as many waits, fences and commits per product,
  // which is what bounds long contractions).
  const bool whole = IMGS == 2;
  constexpr uint32_t SLOTS = 2;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  float* stages = reinterpret_cast<float*>(smem_raw);                        // [STAGES][XIMG + YIMG]
  uint64_t* bars = reinterpret_cast<uint64_t*>(stages + STAGES * CF::STAGE_ELEMS);
  uint64_t* full = bars;                             // [STAGES] a stage's copies have landed
  uint64_t* empty = full + CF::MAX_STAGES;           // [STAGES] the split warps have read it
  uint64_t* img_full = empty + CF::MAX_STAGES;       // [SLOTS] hi / lo images of eight k are written
  uint64_t* img_free = img_full + 2 * CF::MAX_IMGS;  // [SLOTS] ... and the MMAs that read them have completed
  uint64_t* acc_full = img_free + 2 * CF::MAX_IMGS;  // [2] an accumulator holds a finished segment
  uint64_t* acc_free = acc_full + 2;                 // [2] ... and has been read out
  uint64_t* c_ready = acc_free + 2;                  // [CBUFS] the tile's contents have arrived from C
  uint64_t* c_staged = c_ready + CF::MAX_CBUFS;      // [CBUFS] the tile is finished and may be written back
  uint64_t* c_free = c_staged + CF::MAX_CBUFS;       // [CBUFS] ... and has been read out: the buffer is free
  uint32_t* slot = reinterpret_cast<uint32_t*>(bars + CF::NBARS);
  int64_t* kring = reinterpret_cast<int64_t*>(slot + 4);                     // [steps][X 16 | Y 16] contraction offsets
  // One image set: X hi, X lo (BM rows each) for one K step.
  float* images = reinterpret_cast<float*>(kring + CF::KSTEPS_KEPT * 32);    // [IMGS][UMMA_ELEMS]
  float* ctiles = images + IMGS * CF::UMMA_ELEMS;                            // [CBUFS][CTILE_ELEMS]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, CF::FULL_ARRIVALS); mbar_init(empty + s, CF::SPLIT_WARPS); }
    for (uint32_t h = 0; h < SLOTS; ++h) { mbar_init(img_full + h, CF::SPLIT_WARPS); mbar_init(img_free + h, 1); }
    for (int h = 0; h < 2; ++h) { mbar_init(acc_full + h, 1); mbar_init(acc_free + h, CF::EPI_WARPS); }
    for (int b = 0; b < CBUFS; ++b) { mbar_init(c_ready + b, 1); mbar_init(c_staged + b, CF::EPI_WARPS); mbar_init(c_free + b, 1); }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    if constexpr (CF::TMAX || CF::TMAXE) asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&p.tmap_x)) : "memory");
    if constexpr (CF::TMAY || CF::TMAYE) asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&p.tmap_y)) : "memory");
  }
  if (warp == 20) {
    tmem_alloc(slot, CF::TMEM_COLS);
    tmem_relinquish();
  }
  tc05_fence_before();
  __syncthreads();
  tc05_fence_after();
  const uint32_t tmem = *slot;

  const uint32_t total = p.tiles_m * p.tiles_n;
  const uint32_t first = blockIdx.x, step = gridDim.x;
  const uint32_t kbeg = p.k_first, kend = min(p.Kflat, kbeg + p.k_chunk);
  const int nk = (int)((kend - kbeg + BK - 1) / BK);
  const int nseg = (nk + CF::SEG_STEPS - 1) / CF::SEG_STEPS;
  auto seg_begin = [&](int seg) { return (int)((int64_t)seg * nk / nseg); };  // segments of (almost) equal length, none empty
  const bool accumulate = p.beta != 0;
  // `+=` / `-=` reach C as bulk reduce-adds of the products alone (args.c_mode 2, the default: nothing is fetched) or
  // as sums (args.c_mode 0: the tile's old values are fetched into the buffer first, the sums are stored).
  const bool reduce = accumulate && p.c_mode == 2;
  const bool fetch_old = accumulate && !reduce;
  const uint32_t limit = p.spin_limit;

  // Layout of a tile buffer (see the head of this file).
  const int E0 = p.epi_run, runs = BM / E0;
  const bool dense = p.epi_n_span > 0 && E0 < 64;
  const int pitch = (dense || E0 % 8 == 4) ? E0 : E0 + 4, run_stride = pitch * BN;  // 4 mod 8 words: conflict-free

  if (warp < 8) {
    // ------------------------------------------------------------ epilogue ----
    // Warp w reads lanes 32 (w % 4) .. + 31 of D (a warp reaches only its own quarter of tensor memory) and the
    // columns of half w / 4.
    reg_inc<CF::EPILOGUE_REGS>();
    constexpr int CPW = BM / 2;  // columns per warp
    static_assert(CPW % 16 == 0, "columns are read 16 at a time");
    const int nl = 32 * (warp & 3) + lane, cbase = (warp >> 2) * CPW;
    const float alpha = (float)p.alpha;
    uint32_t unit = 0, j = 0;
    bool alive = true;
    for (uint32_t tile = first; alive && tile < total; tile += step, ++j) {
      const uint32_t b = j % CBUFS;
      float* ct = ctiles + b * CF::CTILE_ELEMS;
      for (int seg = 0; seg < nseg; ++seg, ++unit) {
        const uint32_t a = unit & 1u;
        if (!mbar_wait(acc_full + a, (unit >> 1) & 1u, p.status, 10, limit)) { alive = false; break; }
        tc05_fence_after();
        // the buffer holds the tile's old values (`+=`, `-=`) or is simply free (`=`)
        if (seg == 0 && !mbar_wait(c_ready + b, (j / CBUFS) & 1u, p.status, 11, limit)) { alive = false; break; }
        const bool overwrite = !fetch_old && seg == 0;
        float v[CPW];
        const uint32_t taddr = tmem + ((uint32_t)(32 * (warp & 3)) << 16) + a * 128u + (uint32_t)cbase;
#pragma unroll
        for (int c = 0; c < CPW; c += 16) tc05_ld16(taddr + c, v + c);
        tc05_wait_ld();
        // the accumulator is in registers: the next segment but one may overwrite it
        tc05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_free + a);
        int rem = cbase % E0;
        float* dst = ct + (cbase / E0) * run_stride + nl * pitch;
#pragma unroll
        for (int c = 0; c < CPW; c += 4) {
          float4* q = reinterpret_cast<float4*>(dst + rem);
          float4 t = make_float4(alpha * v[c], alpha * v[c + 1], alpha * v[c + 2], alpha * v[c + 3]);
          if (!overwrite) {
            const float4 old = *q;
            t.x += old.x; t.y += old.y; t.z += old.z; t.w += old.w;
          }
          *q = t;
          rem += 4;
          if (rem >= E0) { rem -= E0; dst += run_stride; }
        }
      }
      if (!alive) break;
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // these writes -> the bulk copies that read the tile
      __syncwarp();
      if (lane == 0) mbar_arrive(c_staged + b);
    }
    tc05_fence_before();
    group_bar_sync(1, 288);  // tensor memory may go
    return;
  }

  if (warp < 16) {
    // --------------------------------------------------------------- split ----
    reg_dec<CF::SMALL_REGS>();
    // Thread -> one 16-byte chunk of each operand per group of eight k: row r (lanes walk r: conflict-free reads and
    // writes) and the four k = 4 * kc .. + 3 with kc = 2 h + kq; it goes to core matrix (r / 8, kc), row r % 8.
    const int stid = tid - 256;
    const int ry = stid % BN, qy = stid / BN;
    const bool has_x = stid < 2 * BM;
    const int rx = has_x ? stid % BM : 0, qx = has_x ? stid / BM : 0;
    auto chunk = [&](const float* img, int r, int kc, int mode, int ld) {
      if (mode == 2) return *reinterpret_cast<const float4*>(img + r * CF::LDKV + 4 * kc);
      // a TMA box: row r holds its 16 k in 16-byte chunks, chunk c at position c ^ ((r / 2) % 4) (64-byte swizzle)
      if (mode == 3) return *reinterpret_cast<const float4*>(img + r * BK + 4 * (kc ^ ((r >> 1) & 3)));
      const float* src = img + (4 * kc) * ld + r;
      return make_float4(src[0], src[ld], src[2 * ld], src[3 * ld]);
    };
    // Y: this thread's lane of tensor memory is its row (warp w holds rows 32 (w % 4) .. + 31), its columns the four k
    // of its chunk, hi values in the group's first eight columns, lo values in the next eight.
    const uint32_t ylane = tmem + ((uint32_t)(32 * (warp & 3)) << 16) + CF::A_COLS + 4u * (uint32_t)qy;
    auto put_y = [&](uint32_t set, uint32_t pos, const float4& v4) {
      float4 hi, lo;
      split_tf32_bits(v4.x, hi.x, lo.x); split_tf32_bits(v4.y, hi.y, lo.y);
      split_tf32_bits(v4.z, hi.z, lo.z); split_tf32_bits(v4.w, hi.w, lo.w);
      const uint32_t col = ylane + set * CF::A_SLOT_COLS + pos * 16u;
      tc05_st4(col, hi);
      tc05_st4(col + 8u, lo);
    };
    auto put = [&](float* hi_img, float* lo_img, int r, int kc, const float4& v4) {
      float4 hi, lo;
      split_tf32_bits(v4.x, hi.x, lo.x); split_tf32_bits(v4.y, hi.y, lo.y);
      split_tf32_bits(v4.z, hi.z, lo.z); split_tf32_bits(v4.w, hi.w, lo.w);
      const int d = ((r >> 3) * (BK / 4) + kc) * 8 + (r & 7);
      reinterpret_cast<float4*>(hi_img)[d] = hi;
      reinterpret_cast<float4*>(lo_img)[d] = lo;
    };
    uint32_t g = 0, u = 0;  // stages and image units (eight k each) so far
    for (uint32_t tile = first; tile < total; tile += step) {
      for (int it = 0; it < nk; ++it, ++g) {
        const uint32_t s = g % STAGES;
        const int nh = (kend - (kbeg + (uint32_t)it * BK)) > 8u ? 2 : 1;  // a last step of at most eight k is one unit
        if (!mbar_wait(full + s, (g / STAGES) & 1u, p.status, 12, limit)) return;
        const float* xs = stages + s * CF::STAGE_ELEMS;
        const float* ys = xs + CF::XIMG;
        float4 vy[2], vx[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          vy[h] = chunk(ys, ry, 2 * h + qy, CF::MODEY, CF::LDY);
          vx[h] = has_x ? chunk(xs, rx, 2 * h + qx, CF::MODEX, CF::LDX) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        // The stage goes back to the loaders only after its values have been written into the images.  With a release
        // straight after the loads (the values then wait in registers for an image slot), rows at the head of a TMA
        // box came out wrong about once in 400 stages where both operands arrive in boxes and a tile has three or
        // more segments.  How a refill could overtake loads that precede the arrival in program order was not
        // established; releasing after the stores removed it (five lengths, 40 executions each, all exact).  The
        // release now also follows the thread's fence.proxy.async, the order the memory model asks for between
        // generic-proxy reads and an overwrite by the asynchronous proxy.
        if (whole) {
          const uint32_t sl = u % SLOTS, use = u / SLOTS;
          ++u;
          if (use > 0 && !mbar_wait(img_free + sl, (use - 1) & 1u, p.status, 13, limit)) return;
          float* ub_hi = images + sl * CF::UMMA_ELEMS;
          float* ub_lo = ub_hi + BK * BM;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (h >= nh) break;
            put_y(sl, (uint32_t)h, vy[h]);
            if (has_x) put(ub_hi, ub_lo, rx, 2 * h + qx, vx[h]);
          }
          __syncwarp();
          tc05_wait_st();
          tc05_fence_before();
          asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // generic writes -> the MMA's reads
          __syncwarp();
          if (lane == 0) { mbar_arrive(empty + s); mbar_arrive(img_full + sl); }
          continue;
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (h >= nh) break;
          // unit u (eight k) goes to slot sl = u % 2: position sl among the image set's two groups of 8 k
          const uint32_t sl = u % SLOTS, use = u / SLOTS;
          ++u;
          if (use > 0 && !mbar_wait(img_free + sl, (use - 1) & 1u, p.status, 13, limit)) return;
          float* ub_hi = images;
          float* ub_lo = ub_hi + BK * BM;
          put_y(0u, sl, vy[h]);
          if (has_x) put(ub_hi, ub_lo, rx, 2 * (int)sl + qx, vx[h]);
          __syncwarp();
          tc05_wait_st();
          tc05_fence_before();
          asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // generic writes -> the MMA's reads
          __syncwarp();
          if (lane == 0) {
            if (h == nh - 1) mbar_arrive(empty + s);
            mbar_arrive(img_full + sl);
          }
        }
      }
    }
    return;
  }

  if (warp < 20) {
    // -------------------------------------------------------------- loaders ----
    reg_inc<CF::LOADER_REGS>();
    const int ptid = tid - 512;
    WtSlots<CF, BM, CF::MODEX, CF::LDX> slots_x;
    WtSlots<CF, BN, CF::MODEY, CF::LDY> slots_y;
    slots_x.init(ptid, p.lanes_k_x == 1 ? 0 : 3, p.M.extent[0]);
    slots_y.init(ptid, p.lanes_k_y == 1 ? 0 : 3, p.N.extent[0]);
    // Contraction offsets (entry t of a step: X for t < 16, Y for the rest).  They do not depend on the tile.
    // Short contractions keep all their steps' offsets in shared memory; longer ones pass them through a two-slot
    // ring that 32 threads fill one step ahead (the steps repeat from tile to tile, so "ahead" wraps around).
    const bool keep_all = nk <= CF::KSTEPS_KEPT;
    auto koff_of = [&](int it, int t) -> int64_t {
      const uint32_t k = kbeg + (uint32_t)it * BK + (uint32_t)(t & 15);
      return k < kend ? (t < 16 ? p.koff_x : p.koff_y)[k] : 0;
    };
    int64_t knext = 0;
    if (keep_all) {
      for (int i = ptid; i < nk * 32; i += 128) kring[i] = koff_of(i >> 5, i & 31);
      group_bar_sync(2, 128);
    } else if (ptid < 32) {
      knext = koff_of(0, ptid);
    }
    uint32_t g = 0;
    bool alive = true;  // a loader whose wait gave up keeps meeting the others at the role's barrier, without work
    for (uint32_t tile = first; tile < total; tile += step) {
      uint32_t tm, tn;
      tile_coords(p, tile, &tm, &tn);
      slots_x.rows(p.M, tm * BM, p.Mflat);
      slots_y.rows(p.N, tn * BN, p.Nflat);
      for (int it = 0; it < nk; ++it, ++g) {
        const int64_t* kr = kring + (keep_all ? it : (int)(g & 1u)) * 32;
        if (!keep_all) {
          if (ptid < 32) {
            kring[(g & 1u) * 32 + ptid] = knext;
            knext = koff_of(it + 1 < nk ? it + 1 : 0, ptid);
          }
          group_bar_sync(2, 128);  // the ring slot is written (its last readers passed the previous barrier)
        }
        if (!alive) continue;
        const uint32_t s = g % STAGES;
        if (g >= (uint32_t)STAGES && !mbar_wait(empty + s, ((g / STAGES) - 1) & 1u, p.status, 14, limit)) { alive = false; continue; }
        const uint32_t k0 = kbeg + it * BK;
        float* xs = stages + s * CF::STAGE_ELEMS;
        float* ys = xs + CF::XIMG;
        if constexpr (CF::ANY_TMA) {
          if (ptid == 0) {
            mbar_arrive_expect_tx(full + s, CF::TMA_BYTES);
            if constexpr (CF::TMAX) tma_load_2d(xs, &p.tmap_x, (int)k0, (int)(tm * BM), full + s);
            if constexpr (CF::TMAY) tma_load_2d(ys, &p.tmap_y, (int)k0, (int)(tn * BN), full + s);
            if constexpr (CF::TMAXE) tma_load_2d(xs, &p.tmap_x, (int)(tm * BM), (int)k0, full + s);
            if constexpr (CF::TMAYE) tma_load_2d(ys, &p.tmap_y, (int)(tn * BN), (int)k0, full + s);
          }
        }
        slots_x.issue(xs, X, kr, k0, kend);
        slots_y.issue(ys, Y, kr + 16, k0, kend);
        // tests only: one thread leaves one stage unannounced, so that the waits on it run out
        if (p.test_fault == 1 && blockIdx.x == 0 && g == 1 && ptid == 7) continue;
        mbar_arrive_on_copies(full + s);
      }
    }
    cp_async_wait<0>();
    return;
  }

  reg_dec<CF::SMALL_REGS>();  // the last warpgroup: MMA, fetch, store and a warp without work
  if (warp == 20) {
    // ------------------------------------------------------------------ MMA ----
    if (lane == 0) {
      constexpr uint32_t IDESC = umma_idesc_tf32(BN, BM);
      uint32_t u = 0, unit = 0;  // image units and accumulator segments so far
      const uint32_t a0 = tmem + CF::A_COLS;
      const uint64_t bh0 = umma_desc_k(smem_u32(images), 128, (BK / 4) * 128);
      bool alive = true;
        for (uint32_t tile = first; alive && tile < total; tile += step) {
        for (int seg = 0; alive && seg < nseg; ++seg, ++unit) {
          const uint32_t a = unit & 1u;
          if (unit >= 2 && !mbar_wait(acc_free + a, ((unit >> 1) - 1) & 1u, p.status, 15, limit)) { alive = false; break; }
          tc05_fence_after();
          const uint32_t d_tmem = tmem + a * 128u;
          const int it_begin = seg_begin(seg), it_end = seg_begin(seg + 1);
          for (int it = it_begin; alive && it < it_end; ++it) {
            const int nh = (kend - (kbeg + (uint32_t)it * BK)) > 8u ? 2 : 1;
            // per group of 8 k: two 4-k chunks per MMA, 128 bytes apart; 8-row groups (BK / 4) * 128 bytes apart.
            // The descriptors of a set's groups differ from the first one's only in the address field (16-byte
            // units, no carry out of it: the images lie in the first 256 KB): one addition each.
            auto three = [&](uint32_t set, uint32_t pos, uint32_t acc) {
              const uint32_t ah = a0 + set * CF::A_SLOT_COLS + pos * 16u, al = ah + 8u;
              const uint64_t bh = bh0 + (uint64_t)(set * (uint32_t)(CF::UMMA_ELEMS * 4 / 16) + pos * 16u);
              const uint64_t bl = bh + (uint64_t)(BK * BM * 4 / 16);
              tc05_mma_tf32_ta(d_tmem, al, bh, IDESC, acc);
              tc05_mma_tf32_ta(d_tmem, ah, bl, IDESC, 1u);
              tc05_mma_tf32_ta(d_tmem, ah, bh, IDESC, 1u);
            };
            if (whole) {
              const uint32_t sl = u % SLOTS, use = u / SLOTS;
              ++u;
              if (!mbar_wait(img_full + sl, use & 1u, p.status, 16, limit)) { alive = false; break; }
              tc05_fence_after();
              three(sl, 0u, it > it_begin ? 1u : 0u);
              if (nh == 2) three(sl, 1u, 1u);
              tc05_commit(img_free + sl);
              continue;
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              if (h >= nh) break;
              const uint32_t sl = u % SLOTS, use = u / SLOTS;
              ++u;
              if (!mbar_wait(img_full + sl, use & 1u, p.status, 16, limit)) { alive = false; break; }
              tc05_fence_after();
              three(0u, sl, (it > it_begin || h > 0) ? 1u : 0u);
              tc05_commit(img_free + sl);
            }
          }
          if (alive) tc05_commit(acc_full + a);
        }
      }
    }
    __syncwarp();
    tc05_fence_before();
    group_bar_sync(1, 288);  // the epilogue warps have left: nobody reads tensor memory any more
    tc05_fence_after();
    tmem_dealloc(tmem, CF::TMEM_COLS);
    return;
  }

  // Chunks of tile (m0, n0) in C and in its buffer: per run r either one per n (pitch > E0), or the n that are adjacent
  // in C inside the current block of F0 = args.epi_n_span and then the rest (at most two chunks per run).  Lane-
  // parallel: chunk c of the tile is described by lane c % 32 in round c / 32.
  const int F0 = p.epi_n_span;
  const uint32_t ntiles = first < total ? (total - first + step - 1) / step : 0;
  struct Chunk { const float* g; uint32_t s, bytes; };
  // Offset in C of flattened index `flat` of a class: one division for classes of one or two fused dimensions.
  auto out_off = [&](const TcDims& d, uint32_t flat) -> int64_t {
    if (d.n == 1) return (int64_t)flat * d.s_out[0];
    if (d.n == 2) {
      const uint32_t q = flat / d.extent[0];
      return (int64_t)(flat - q * d.extent[0]) * d.s_out[0] + (int64_t)q * d.s_out[1];
    }
    int64_t unused, o;
    decode(d, flat, 0xffffffffu, &unused, &o);
    return o;
  };
  auto chunk_count = [&](uint32_t j, int* vruns, int* vn, int* nb, int* nchunk, uint32_t* m0, uint32_t* n0) {
    uint32_t tm, tn;
    tile_coords(p, first + j * step, &tm, &tn);
    *m0 = tm * BM; *n0 = tn * BN;
    *vruns = min(runs, (int)((p.Mflat - *m0 + E0 - 1) / E0));  // runs and n inside the tensor
    *vn = min(BN, (int)(p.Nflat - *n0));
    *nb = *vn; *nchunk = *vn;
    if (dense) {
      const int left = F0 - (int)(*n0 % (uint32_t)F0);
      *nb = left < *vn ? left : *vn;
      *nchunk = *nb < *vn ? 2 : 1;
    }
    return *vruns * *nchunk;
  };
  auto chunk_of = [&](int c, uint32_t b, int vn, int nb, int nchunk, uint32_t m0, uint32_t n0) {
    const int r = c / nchunk, q = c % nchunk;
    const int n = dense ? (q == 0 ? 0 : nb) : q;
    const int len = dense ? (q == 0 ? nb : vn - nb) : 1;
    Chunk k;
    k.g = C + out_off(p.M, m0 + r * E0) + out_off(p.N, n0 + n);
    k.s = smem_u32(ctiles + b * CF::CTILE_ELEMS) + (uint32_t)(r * run_stride + n * pitch) * 4u;
    k.bytes = (uint32_t)(E0 * len) * 4u;
    return k;
  };

  if (warp == 23) return;
  if (warp == 21) {
    // ---------------------------------------------------------------- fetch ----
    for (uint32_t j = 0; j < ntiles; ++j) {
      const uint32_t b = j % CBUFS;
      if (j >= (uint32_t)CBUFS && !mbar_wait(c_free + b, ((j / CBUFS) - 1) & 1u, p.status, 17, limit)) break;
      if (fetch_old) {
        int vruns, vn, nb, nchunk;
        uint32_t m0, n0;
        const int total_chunks = chunk_count(j, &vruns, &vn, &nb, &nchunk, &m0, &n0);
        if (lane == 0) mbar_arrive_expect_tx(c_ready + b, (uint32_t)(vruns * vn * E0) * 4u);
        __syncwarp();
        for (int c = lane; c < total_chunks; c += 32) {
          const Chunk k = chunk_of(c, b, vn, nb, nchunk, m0, n0);
          bulk_load(k.s, k.g, k.bytes, c_ready + b);
        }
      } else if (lane == 0) {
        mbar_arrive(c_ready + b);  // nothing to fetch: the buffer is simply free
      }
    }
    return;
  }

  {
    // ---------------------------------------------------------------- store ----
    // With several buffers, the buffer of tile j - 1 is released after tile j's copies have been issued: its read-out
    // overlaps them.  With one buffer the next tile cannot be finished before this one is released: no deferring.
    const bool defer = CBUFS > 1;
    uint32_t j = 0;
    for (; j < ntiles; ++j) {
      const uint32_t b = j % CBUFS;
      if (!mbar_wait(c_staged + b, (j / CBUFS) & 1u, p.status, 18, limit)) break;
      int vruns, vn, nb, nchunk;
      uint32_t m0, n0;
      const int total_chunks = chunk_count(j, &vruns, &vn, &nb, &nchunk, &m0, &n0);
      for (int c = lane; c < total_chunks; c += 32) {
        const Chunk k = chunk_of(c, b, vn, nb, nchunk, m0, n0);
        if (reduce) bulk_reduce_add(const_cast<float*>(k.g), k.s, k.bytes);
        else bulk_store(const_cast<float*>(k.g), k.s, k.bytes);
      }
      asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
      if (!defer) {
        asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(c_free + b);
      } else if (j > 0) {
        asm volatile("cp.async.bulk.wait_group.read 1;\n" ::: "memory");  // all but the newest group have read their buffer
        __syncwarp();
        if (lane == 0) mbar_arrive(c_free + (j - 1) % CBUFS);
      }
    }
    asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");
    __syncwarp();
    if (defer && j > 0 && lane == 0) mbar_arrive(c_free + (j - 1) % CBUFS);
    asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");
  }
}

}  // namespace tck
