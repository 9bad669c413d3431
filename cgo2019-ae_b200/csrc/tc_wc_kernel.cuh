// Persistent fp64 contraction kernel for outputs that dominate the memory traffic (short contractions):
// the output tile is RESIDENT in shared memory while it is updated.
//
// Same tiling, address tables, operand images and DMMA fragment mapping as tc_ws_dmma_kernel
// (tc_ws_kernel.cuh); what differs is the way the result meets C:
//
//   * a consumer group (eight warps of 32 x 32 on a 128 x 64 tile) owns TWO output-tile buffers in shared memory,
//     used alternately;
//   * one thread per group (the "C thread", first lane of a warp of its own) moves whole output tiles with tiled TMA
//     copies of the rank-5 view of C: it LOADS the tile of C a whole tile ahead of its use
//     (cp.async.bulk.tensor.5d into the group's free buffer, completion on an mbarrier), waits until the
//     consumers have added their products into the buffer, STORES it back (cp.async.bulk.tensor.5d, plain
//     store) and, once the copy engine has read the buffer, issues the load of the tile after next;
//   * the consumers never touch global memory and never wait for the copy engine in their epilogue: they wait
//     for "tile loaded" (issued a tile ago), do `buffer += alpha * acc` with 16-byte shared loads and stores
//     (the two halves of a thread's 32 bytes are visited in opposite order by even and odd row groups, which
//     makes the accesses bank-conflict free on the dense rows the copy engine wants), and go on to
//     their next tile;
//   * producer warps fill the group's operand ring exactly as in tc_ws_dmma_kernel.
//
// Why: on B200 the reduce-add stream of the copy engine (cp.reduce.async.bulk.tensor ... add) tops out near
// 5.2 TB/s of read+write traffic for this access pattern, while tiled loads plus tiled stores through the SM
// reach 6.1 TB/s; and an epilogue that stages through two small per-warp buffers waits once per batch for the
// copy engine's read-out latency, during which the tensor pipe idles.  `=` uses the same path without loads.
// One group of eight warps (two per scheduler) with a three-stage operand ring measured faster than two groups
// of four or eight warps with two-stage rings, which is all that fits beside 128 KB of output buffers: a group
// that runs alone is then starved by its own ring (a refill takes about 2400 cycles, a stage lasts 1000), and
// letting the groups take turns on the tensor pipe made that worse.  What is left exposed is the epilogue itself:
// 128 KB of shared-memory traffic per tile, about 1000 cycles beside 5600 of products at K = 40.
//
// Needs the output to be a rank-<=5 tensor in which a BM x 64 tile is one box (the planner's tma_ct test) and
// 16-byte aligned; rows and columns beyond the tensor are filled with zeros on load and clipped on store by
// the copy engine.  Every mbarrier wait is bounded (args.spin_limit) and reports through args.status.
#pragma once
#include "tc_ws_kernel.cuh"

namespace tck {

// GROUPS consumer groups, each with its own tile, operand ring and output buffers, of WGM x WGN warps.
template <int BM_, int GROUPS_, int WGM_, int WGN_, int STAGES_, int MODEX_, int MODEY_>
struct WcCfg {
  using T = double;
  static constexpr int BM = BM_, BN = 64, BK = 16, STAGES = STAGES_;
  static constexpr int MODEX = MODEX_, MODEY = MODEY_;
  static constexpr int GROUPS = GROUPS_, WGM = WGM_, WGN = WGN_, CW = WGM * WGN;  // consumer warps per group
  static constexpr int WM = BM / WGM, WN = BN / WGN;
  static constexpr int CONSUMER_THREADS = CW * 32;
  static constexpr int PWARPS = GROUPS == 1 ? 2 : 1;  // producer warps per group
  static constexpr int THREADS = 32 * PWARPS;    // producer threads per group
  // last warpgroup: the producer warps, then one warp per group whose first lane is the group's C thread
  static constexpr int CTA_THREADS = GROUPS * CONSUMER_THREADS + 128;
  static_assert(GROUPS * (PWARPS + 1) <= 4 && (GROUPS * CW) % 4 == 0, "warp roles");
  static constexpr int LDK = BK + 2;
  static constexpr int LDX = MODEX == LM_K_VEC ? LDK : MODEX == LM_TMA_K ? BK : BM + 4;
  static constexpr int LDY = MODEY == LM_K_VEC ? LDK : MODEY == LM_TMA_K ? BK : BN + 4;
  static constexpr bool ANY_TMA = MODEX == LM_TMA_K || MODEY == LM_TMA_K;
  static constexpr int round128(int x) { return (x + 127) / 128 * 128; }  // images start on 1024 bytes
  static constexpr int XIMG = round128(MODEX == LM_K_VEC ? BM * LDK : MODEX == LM_TMA_K ? BM * BK : BK * (BM + 4));
  static constexpr int YIMG = round128(MODEY == LM_K_VEC ? BN * LDK : MODEY == LM_TMA_K ? BN * BK : BK * (BN + 4));
  static constexpr int STAGE_ELEMS = XIMG + YIMG;
  static constexpr uint32_t TMA_BYTES = (MODEX == LM_TMA_K ? BM * BK * 8 : 0) + (MODEY == LM_TMA_K ? BN * BK * 8 : 0);
  static constexpr int FULL_ARRIVALS = THREADS + (ANY_TMA ? 1 : 0);
  static constexpr int TABLE_ELEMS = BM + BN;    // offx_m, offy_n (the output is addressed by the copy engine)
  static constexpr int CBUFS = 2;                // output-tile buffers per group
  static constexpr int CTILE_ELEMS = BM * BN;
  static constexpr int NBARS = GROUPS * (2 * STAGES + 2 * CBUFS);
  static constexpr int SMEM_BYTES = (GROUPS * STAGES * STAGE_ELEMS + GROUPS * CBUFS * CTILE_ELEMS + GROUPS * 2 * TABLE_ELEMS) * 8 +
                                    NBARS * 8;
  static constexpr int PRODUCER_REGS = 56;
  static_assert(SMEM_BYTES <= 232448, "shared memory");
};

// Coordinates of the box of the rank-5 view of C (TcOutMap) that holds the tile starting at (m0, n0):
// {run offset, 0, (n inside N's fastest dimension) / 2, slower dimension, slowest dimension}.
__device__ __forceinline__ void tile_box_coords(const TcKernelArgs& p, uint32_t m0, uint32_t n0, int (&c)[4]) {
  const uint32_t e0 = p.cmap.e0, f0 = p.cmap.f0;
  const int ne = p.cmap.ne, me = p.cmap.me;
  int x3 = 0, x4 = 0;
  const uint32_t rm = m0 / e0, rn = n0 / f0;
  if (me == 2) { x3 = (int)(rm % p.cmap.ext[0]); x4 = (int)(rm / p.cmap.ext[0]); }
  else if (me == 1) { if (ne == 0) x3 = (int)rm; else x4 = (int)rm; }
  if (ne == 2) { x3 = (int)(rn % p.cmap.ext[0]); x4 = (int)(rn / p.cmap.ext[0]); }
  else if (ne == 1) x3 = (int)rn;
  c[0] = (int)(m0 % e0);
  c[1] = (int)((n0 % f0) >> 1);
  c[2] = x3;
  c[3] = x4;
}

template <class CF>
__global__ void __launch_bounds__(CF::CTA_THREADS, 1) tc_wc_dmma_kernel(const __grid_constant__ TcKernelArgs p,
                                                                         double* __restrict__ C,
                                                                         const double* __restrict__ X,
                                                                         const double* __restrict__ Y) {
  constexpr int BM = CF::BM, BN = CF::BN, BK = CF::BK, LDX = CF::LDX, LDY = CF::LDY, STAGES = CF::STAGES;
  constexpr int CW = CF::CW;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  double* stages = reinterpret_cast<double*>(smem_raw);  // first: TMA images need 1024-byte alignment
  double* cbufs = stages + CF::GROUPS * STAGES * CF::STAGE_ELEMS;
  int64_t* tables = reinterpret_cast<int64_t*>(cbufs + CF::GROUPS * CF::CBUFS * CF::CTILE_ELEMS);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tables + CF::GROUPS * 2 * CF::TABLE_ELEMS);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  constexpr int CWARPS = CF::GROUPS * CW, PW = CF::PWARPS;
  const bool is_producer = warp >= CWARPS && warp < CWARPS + CF::GROUPS * PW;
  const bool is_cwg = warp >= CWARPS + CF::GROUPS * PW;  // C threads (first lanes of the first GROUPS warps here), idle warps
  const int gi = warp < CWARPS ? warp / CW : is_producer ? (warp - CWARPS) / PW : (warp - CWARPS - CF::GROUPS * PW) % CF::GROUPS;
  uint64_t* full = bars + gi * (2 * STAGES + 2 * CF::CBUFS);  // [STAGES] operands of a stage have landed
  uint64_t* empty = full + STAGES;                            // [STAGES] the consumers are done with a stage
  uint64_t* c_ready = empty + STAGES;                         // [CBUFS] the buffer holds the tile of C (or is free, for `=`)
  uint64_t* c_staged = c_ready + CF::CBUFS;                   // [CBUFS] the consumers have added their products
  int64_t* gtab = tables + gi * 2 * CF::TABLE_ELEMS;          // two table sets, alternating per tile
  double* gstage = stages + gi * STAGES * CF::STAGE_ELEMS;
  double* gcbuf = cbufs + gi * CF::CBUFS * CF::CTILE_ELEMS;

  if (tid == 32) {  // descriptors into the copy engine's cache before the first copy needs them
    if constexpr (CF::MODEX == LM_TMA_K) asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&p.tmap_x)) : "memory");
    if constexpr (CF::MODEY == LM_TMA_K) asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&p.tmap_y)) : "memory");
    asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(&p.tmap_ct)) : "memory");
  }
  if (tid == 0) {
    for (int q = 0; q < CF::GROUPS; ++q) {
      uint64_t* b = bars + q * (2 * STAGES + 2 * CF::CBUFS);
      for (int s = 0; s < STAGES; ++s) { mbar_init(b + s, CF::FULL_ARRIVALS); mbar_init(b + STAGES + s, CW); }
      for (int s = 0; s < CF::CBUFS; ++s) { mbar_init(b + 2 * STAGES + s, 1); mbar_init(b + 2 * STAGES + CF::CBUFS + s, CW); }
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();

  const uint32_t total = p.tiles_m * p.tiles_n;
  const uint32_t first = (uint32_t)CF::GROUPS * blockIdx.x + gi, step = (uint32_t)CF::GROUPS * gridDim.x;
  const int nk = (int)((p.Kflat + BK - 1) / BK);
  const uint32_t kend = p.Kflat;
  const bool accumulate = p.beta != 0;

  if (is_cwg) {
    // --------------------------------------------------------------- C thread ----
    reg_dec<CF::PRODUCER_REGS>();  // one value for the whole warpgroup
    if ((tid & 31) != 0 || warp >= CWARPS + CF::GROUPS * (PW + 1)) return;
    const uint64_t tmap = reinterpret_cast<uint64_t>(&p.tmap_ct);
    const uint32_t ntiles = first < total ? (total - first + step - 1) / step : 0u;
    auto fetch = [&](uint32_t j) {  // tile j of this group into buffer j & 1 (or just: the buffer is free)
      const uint32_t b = j & 1u;
      if (!accumulate) { mbar_arrive(&c_ready[b]); return; }
      uint32_t tm, tn;
      tile_coords(p, first + j * step, &tm, &tn);
      int c[4];
      tile_box_coords(p, tm * BM, tn * BN, c);
      mbar_arrive_expect_tx(&c_ready[b], BM * BN * 8);
      asm volatile(
          "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];\n" ::"r"(
              smem_u32(gcbuf + b * CF::CTILE_ELEMS)),
          "l"(tmap), "r"(c[0]), "r"(0), "r"(c[1]), "r"(c[2]), "r"(c[3]), "r"(smem_u32(&c_ready[b]))
          : "memory");
    };
    for (uint32_t j = 0; j < ntiles && j < (uint32_t)CF::CBUFS; ++j) fetch(j);
    for (uint32_t j = 0; j < ntiles; ++j) {
      const uint32_t b = j & 1u;
      if (!mbar_wait(&c_staged[b], (j >> 1) & 1u, p.status, 6, p.spin_limit)) return;
      uint32_t tm, tn;
      tile_coords(p, first + j * step, &tm, &tn);
      int c[4];
      tile_box_coords(p, tm * BM, tn * BN, c);
      asm volatile("cp.async.bulk.tensor.5d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3, %4, %5}], [%6];\n" ::"l"(tmap),
                   "r"(c[0]), "r"(0), "r"(c[1]), "r"(c[2]), "r"(c[3]), "r"(smem_u32(gcbuf + b * CF::CTILE_ELEMS))
                   : "memory");
      asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
      if (j + CF::CBUFS < ntiles) {
        asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");  // the store has read the buffer: it may be refilled
        fetch(j + CF::CBUFS);
      }
    }
    asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory");
    return;
  }

  if (is_producer) {
    // ------------------------------------------------------------ producer ----
    reg_dec<CF::PRODUCER_REGS>();
    const int ptid = tid - (CWARPS + gi * PW) * 32;
    const int lgx = p.lanes_k_x == 1 ? 0 : 2, lgy = p.lanes_k_y == 1 ? 0 : 2;
    uint32_t it = 0, titer = 0;
    for (uint32_t tile = first; tile < total; tile += step, ++titer) {
      // Two table sets used alternately: the barrier below is passed only when every producer of the group has
      // issued the previous tile's loads, so the set written now (last read two tiles ago) is free.
      int64_t* offx_m = gtab + (titer & 1) * CF::TABLE_ELEMS;
      int64_t* offy_n = offx_m + BM;
      uint32_t tm, tn;
      tile_coords(p, tile, &tm, &tn);
      const uint32_t m0 = tm * BM, n0 = tn * BN;
      for (int i = ptid; i < BM + BN; i += CF::THREADS) {
        int64_t unused;
        if (i < BM) decode(p.M, m0 + i, p.Mflat, &offx_m[i], &unused);
        else decode(p.N, n0 + (i - BM), p.Nflat, &offy_n[i - BM], &unused);
      }
      group_bar_sync(1 + gi, CF::THREADS);
      for (int ks = 0; ks < nk; ++ks, ++it) {
        const uint32_t s = it % STAGES;
        if (!mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, p.status, 2, p.spin_limit)) return;
        double* xs = gstage + s * CF::STAGE_ELEMS;
        double* ys = xs + CF::XIMG;
        const uint32_t k0 = (uint32_t)ks * BK;
        if constexpr (CF::ANY_TMA) {
          if (ptid == 0) {
            mbar_arrive_expect_tx(&full[s], CF::TMA_BYTES);
            if constexpr (CF::MODEX == LM_TMA_K) tma_load_2d(xs, &p.tmap_x, (int)k0, (int)m0, &full[s]);
            if constexpr (CF::MODEY == LM_TMA_K) tma_load_2d(ys, &p.tmap_y, (int)k0, (int)n0, &full[s]);
          }
        }
        ws_load<CF, BM, CF::MODEX>(xs, X, offx_m, p.koff_x, k0, kend, ptid, lgx);
        ws_load<CF, BN, CF::MODEY>(ys, Y, offy_n, p.koff_y, k0, kend, ptid, lgy);
        // tests only: one producer thread of CTA 0 never announces its copies of one stage
        if (p.test_fault == 1 && blockIdx.x == 0 && gi == 0 && it == 1 && ptid == 7) continue;
        mbar_arrive_on_copies(&full[s]);
      }
    }
    return;
  }

  // -------------------------------------------------------------- consumer ----
  constexpr int WM = CF::WM, WN = CF::WN;
  constexpr int MB2 = WM / 16, NB2 = WN / 16;
  const int lane = tid & 31, cw = warp % CW;
  const int g = lane >> 2, t = lane & 3;
  const int wm0 = (cw % CF::WGM) * WM, wn0 = (cw / CF::WGM) * WN;
  const double alpha = p.alpha;
  const int h0 = g & 1;  // which 16-byte half of its 32 bytes a thread visits first (see the header)
  uint32_t it = 0, titer = 0;
  for (uint32_t tile = first; tile < total; tile += step, ++titer) {
    // acc[nb][2i + e][h]: row n = wn0 + 16 (nb >> 1) + 2 g + (nb & 1), column m = wm0 + 16 i + 4 t + e + 2 h
    // (the fragment mapping of tc_ws_dmma_kernel: four consecutive m per thread and row)
    double acc[2 * NB2][2 * MB2][2];
#pragma unroll
    for (int j = 0; j < 2 * NB2; ++j)
#pragma unroll
      for (int i = 0; i < 2 * MB2; ++i) { acc[j][i][0] = 0.0; acc[j][i][1] = 0.0; }

    for (int ks = 0; ks < nk; ++ks, ++it) {
      const uint32_t s = it % STAGES;
      if (!mbar_wait(&full[s], (it / STAGES) & 1, p.status, 3, p.spin_limit)) return;
      const double* xs = gstage + s * CF::STAGE_ELEMS;
      const double* ys = xs + CF::XIMG;
      const int kleft = (int)kend - ks * BK;
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
    // ---- epilogue: buffer (+)= alpha * acc in shared memory; the C thread stores the buffer ----
    const uint32_t b = titer & 1u;
    if (!mbar_wait(&c_ready[b], (titer >> 1) & 1u, p.status, 4, p.spin_limit)) return;
    double* tb = gcbuf + b * CF::CTILE_ELEMS;
#pragma unroll
    for (int nb = 0; nb < 2 * NB2; ++nb) {
      double* row = tb + (wn0 + 16 * (nb >> 1) + 2 * g + (nb & 1)) * BM + wm0 + 4 * t;
#pragma unroll
      for (int i = 0; i < MB2; ++i) {
        double2* q = reinterpret_cast<double2*>(row + 16 * i);
        // the thread's four consecutive outputs: lo = (m, m+1), hi = (m+2, m+3)
        const double2 lo = make_double2(alpha * acc[nb][2 * i][0], alpha * acc[nb][2 * i + 1][0]);
        const double2 hi = make_double2(alpha * acc[nb][2 * i][1], alpha * acc[nb][2 * i + 1][1]);
        double2 first_v = h0 ? hi : lo, second_v = h0 ? lo : hi;
        if (accumulate) {
          const double2 c0 = q[h0], c1 = q[h0 ^ 1];
          first_v.x += c0.x; first_v.y += c0.y;
          second_v.x += c1.x; second_v.y += c1.y;
        }
        q[h0] = first_v;
        q[h0 ^ 1] = second_v;
      }
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    __syncwarp();
    if (lane == 0) mbar_arrive(&c_staged[b]);  // release: this warp's part of the tile is in the buffer
  }
}

}  // namespace tck
