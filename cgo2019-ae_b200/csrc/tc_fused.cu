// Several contractions accumulated into ONE output in a single pass over it.
//
// The reference's application case is CCSD(T): nine contractions, each with its own pair of inputs and its own
// assignment of the output's indices to the two inputs, all accumulating into one 6-D tensor
// (cogent/input_strings/ccsd_t/original-expressions/sd_t_d2.in:4-30, checker
// cogent/drivers/ccsd_t/code_main_sd2_1.c:561-613).  The reference planned to fuse them ("register transpose") but
// its emitter for that is a stub (cogent/src/codes/kernels/tc_code_kernel_fusion.py:6-205); executed one by one they
// read and write the output nine times, and on outputs of this shape the output traffic IS the run time.
//
// Here a CTA owns one BOX of the output -- b_i consecutive values of every output index i, 4096 elements at most --
// kept in shared memory in the output's own order.  For every term the box is a (rows x cols) matrix product, rows
// being the box coordinates of the indices the term's left input carries and cols those of its right input (both at
// most 64, e.g. 4 x 4 x 4 for the 3 + 3 index splits of CCSD(T)); the term's operand slabs are gathered through
// per-term offset tables (cp.async, two stages in flight across term boundaries), multiplied on the FP64 tensor pipe
// (DMMA m8n8k4, same fragment mapping as tc_contract_kernel) and the accumulators are scattered into the box with
// the term's own (row, col) -> box-offset tables.  After the last term the box is added to C once.
// fp64 only.  Operator per term: += or -=.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <new>
#include <sstream>
#include <string>
#include <vector>

#include "tc_kernels.cuh"

namespace {

constexpr int kMaxTerms = 16;     // terms per fused plan
constexpr int kMaxRank = 8;       // output indices
constexpr int kBox = 64;          // rows / cols of a term inside a box, at most
constexpr int kBoxElems = 4096;   // elements of a box, at most
constexpr int kThreads = 256;
constexpr int kStages = 3;        // operand stages in flight
constexpr int kTabK = 64;         // contraction offsets per term kept in shared memory

// One term as the kernel sees it (device memory).
struct FusedTerm {
  int64_t rowoff_x[kBox], rowoff_y[kBox];   // element offset of box row r / box column c inside the left / right input
  uint64_t coord_m[kBox], coord_n[kBox];    // their box coordinates, one byte per output index (0 where the index is absent)
  int32_t boxoff_m[kBox], boxoff_n[kBox];   // their contribution to the element's position inside the box
  int64_t sx[kMaxRank], sy[kMaxRank];       // stride of output index i in the left / right input (0: not carried)
  const int64_t* koff_x;                    // [kflat] offset of flattened contraction index k in the left input
  const int64_t* koff_y;
  uint32_t kflat;
  int32_t rows, cols;                       // box rows / columns of this term (<= 64)
  int32_t kfast_x, kfast_y;                 // loader mode of the left / right input (see the kernel)
  double alpha;                             // +1 or -1
};

struct FusedArgs {
  int32_t n_terms, rank;
  uint32_t b[kMaxRank], ext[kMaxRank], tiles[kMaxRank], boxstride[kMaxRank];
  int64_t sc[kMaxRank];
  uint32_t box_elems;
  uint64_t total_boxes;
  const FusedTerm* terms;
  const int64_t* box_off;   // [box_elems] offset of box element e from the box's corner inside the output
  int32_t beta;  // 1: the box is added to C, 0: it overwrites C
};

struct FusedPtrs { const double* x[kMaxTerms]; const double* y[kMaxTerms]; };

constexpr int LD = kBox + 4;   // pitch of an operand image [k][row]: conflict-free 16-byte fragment reads
constexpr int LDK = TC_BK + 2; // pitch of an operand image [row][k] (inputs whose fastest index is contracted)
constexpr int IMG = kBox * LDK > TC_BK * LD ? kBox * LDK : TC_BK * LD;  // doubles per image, either layout

// Position of box element e in shared memory.  The box is kept in the output's order, but its low four position
// bits are XORed with bits of the higher coordinates: a term's accumulators scatter over three output indices at
// once (one of the left input's, two of the right input's), most of them with strides of 16 elements and more,
// which in the plain order fall on one or two banks (measured: 73 % of all shared-memory wavefronts were conflicts).
__device__ __forceinline__ uint32_t box_pos(uint32_t e) { return e ^ (((e >> 4) ^ (e >> 8)) & 15u); }

__global__ void __launch_bounds__(kThreads, 2) tc_fused_kernel(const __grid_constant__ FusedArgs p,
                                                                const __grid_constant__ FusedPtrs ptrs,
                                                                double* __restrict__ C) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  double* box = reinterpret_cast<double*>(smem_raw);            // [box_elems], the output's order inside the box
  double* xs = box + kBoxElems;                                  // [kStages][IMG]
  double* ys = xs + kStages * IMG;                               // [kStages][IMG]
  // per-term tables, copied from global memory once per CTA: every later look-up is a shared-memory read
  int64_t* s_rowx = reinterpret_cast<int64_t*>(ys + kStages * IMG);  // [terms][64]
  int64_t* s_rowy = s_rowx + p.n_terms * kBox;                   // [terms][64]
  int64_t* s_kox = s_rowy + p.n_terms * kBox;                    // [terms][kTabK] offsets of the first kTabK contraction positions
  int64_t* s_koy = s_kox + p.n_terms * kTabK;
  int32_t* s_bom = reinterpret_cast<int32_t*>(s_koy + p.n_terms * kTabK);  // [terms][64]
  int32_t* s_bon = s_bom + p.n_terms * kBox;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int wm0 = (warp & 1) * 32, wn0 = (warp >> 1) * 16;       // 2 x 4 warps of 32 x 16
  constexpr int BK = TC_BK;

  // this CTA's box: coordinates of its corner, and how much of the box lies inside the tensor
  uint32_t tc[kMaxRank];
  uint64_t limits = 0, full = 0;  // byte i: valid values of index i inside this box / in a whole box
  int64_t base_c = 0;
  {
    uint64_t r = blockIdx.x;
    for (int i = 0; i < p.rank; ++i) {
      tc[i] = (uint32_t)(r % p.tiles[i]) * p.b[i];
      r /= p.tiles[i];
      const uint32_t left = p.ext[i] - tc[i];
      limits |= (uint64_t)(left < p.b[i] ? left : p.b[i]) << (8 * i);
      full |= (uint64_t)p.b[i] << (8 * i);
      base_c += (int64_t)tc[i] * p.sc[i];
    }
  }
  const bool whole = limits == full;  // uniform: most boxes lie wholly inside the tensor
  auto inside = [&](uint64_t coord) {  // every byte of coord below the matching byte of limits
    if (whole) return true;
    bool ok = true;
    for (int i = 0; i < p.rank; ++i) ok = ok && ((coord >> (8 * i)) & 0xff) < ((limits >> (8 * i)) & 0xff);
    return ok;
  };
  for (int e = tid; e < kBoxElems; e += kThreads) box[e] = 0.0;
  for (int i = tid; i < p.n_terms * kBox; i += kThreads) {
    const FusedTerm& T = p.terms[i / kBox];
    const int r = i % kBox;
    s_rowx[i] = T.rowoff_x[r];
    s_rowy[i] = T.rowoff_y[r];
    s_bom[i] = r < T.rows ? T.boxoff_m[r] : -1;
    s_bon[i] = r < T.cols ? T.boxoff_n[r] : -1;
  }
  for (int i = tid; i < p.n_terms * kTabK; i += kThreads) {
    const FusedTerm& T = p.terms[i / kTabK];
    const uint32_t k = i % kTabK;
    s_kox[i] = k < T.kflat ? T.koff_x[k] : 0;
    s_koy[i] = k < T.kflat ? T.koff_y[k] : 0;
  }
  __syncthreads();

  // Loader state of the term whose stages are being ISSUED (it may be up to kStages - 1 stages ahead of the one
  // being multiplied), set up once per term so that a stage costs a handful of instructions per thread:
  //   mode 0  image [k][row], 8-byte copies: the thread keeps its row and walks four k per stage;
  //   mode 1  image [row][k] (the input's fastest index is contracted), 8-byte copies: the thread keeps its k
  //           position and walks four rows;
  //   mode 2  the same with 16-byte copies of two consecutive k: two rows per thread.
  const double* xsrc[4];
  const double* ysrc[4];       // global address of this thread's rows at k = 0 (the input's base where the row is outside)
  uint32_t xok = 0, yok = 0;   // bit q: row q lies inside the tensor
  uint32_t xdst, ydst;         // byte offset of its first copy inside an image; further copies follow at xstep / ystep
  uint32_t xstep, ystep;
  int xmode = 0, ymode = 0;
  const int64_t* skx = nullptr;  // contraction offsets of the term (shared-memory copy of the first kTabK, else global)
  const int64_t* sky = nullptr;
  const int64_t* gkx = nullptr;
  const int64_t* gky = nullptr;
  uint32_t kfl = 0;
  auto setup = [&](int k) {
    const FusedTerm& T = p.terms[k];
    int64_t bx = 0, by = 0;
    for (int i = 0; i < p.rank; ++i) { bx += (int64_t)tc[i] * T.sx[i]; by += (int64_t)tc[i] * T.sy[i]; }
    const double* xb = ptrs.x[k] + bx;
    const double* yb = ptrs.y[k] + by;
    xmode = T.kfast_x;
    ymode = T.kfast_y;
    gkx = T.koff_x;
    gky = T.koff_y;
    skx = s_kox + k * kTabK;
    sky = s_koy + k * kTabK;
    kfl = T.kflat;
    auto rows = [&](int mode, const int32_t* s_bo, const int64_t* s_row, const uint64_t* coord, const double* base,
                    const double* (&src)[4], uint32_t* okbits, uint32_t* dst, uint32_t* step) {
      *okbits = 0;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int r = mode == 2 ? tid / 8 + 32 * q : mode == 1 ? tid / 16 + 16 * q : tid % kBox;
        const bool ok = r < kBox && s_bo[k * kBox + r] >= 0 && (whole || inside(coord[r]));
        src[q] = ok ? base + s_row[k * kBox + r] : base;
        *okbits |= (ok ? 1u : 0u) << q;
      }
      *dst = mode == 2 ? ((tid / 8) * LDK + 2 * (tid % 8)) * 8 : mode == 1 ? ((tid / 16) * LDK + tid % 16) * 8 : ((tid / kBox) * LD + tid % kBox) * 8;
      *step = mode == 2 ? 32 * LDK * 8 : mode == 1 ? 16 * LDK * 8 : 4 * LD * 8;
    };
    rows(xmode, s_bom, s_rowx, T.coord_m, xb, xsrc, &xok, &xdst, &xstep);
    rows(ymode, s_bon, s_rowy, T.coord_n, yb, ysrc, &yok, &ydst, &ystep);
  };
  auto fetch = [&](uint32_t img, const double* const (&src)[4], uint32_t okbits, uint32_t dst, uint32_t dstep, int mode, const int64_t* sk,
                   const int64_t* gk, uint32_t k0) {
    auto ko_of = [&](uint32_t k) { return k < (uint32_t)kTabK ? sk[k] : gk[k]; };
    if (mode == 2) {
      const uint32_t k = k0 + 2 * (tid % 8);
      const bool kok = k < kfl;
      const int64_t ko = kok ? ko_of(k) : 0;
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const bool ok = kok && ((okbits >> q) & 1u);
        tck::cp_async16(img + dst + q * dstep, ok ? src[q] + ko : src[q], ok);
      }
    } else if (mode == 1) {
      const uint32_t k = k0 + tid % 16;
      const bool kok = k < kfl;
      const int64_t ko = kok ? ko_of(k) : 0;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const bool ok = kok && ((okbits >> q) & 1u);
        tck::cp_async8(img + dst + q * dstep, ok ? src[q] + ko : src[q], ok);
      }
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t k = k0 + tid / kBox + 4 * q;
        const bool ok = k < kfl && (okbits & 1u);
        tck::cp_async8(img + dst + q * dstep, ok ? src[0] + ko_of(k) : src[0], ok);
      }
    }
  };
  const uint32_t xs_u32 = tck::smem_u32(xs), ys_u32 = tck::smem_u32(ys);
  auto issue = [&](int k, int step, int buf) {
    if (step == 0) setup(k);
    fetch(xs_u32 + buf * IMG * 8, xsrc, xok, xdst, xstep, xmode, skx, gkx, (uint32_t)step * BK);
    fetch(ys_u32 + buf * IMG * 8, ysrc, yok, ydst, ystep, ymode, sky, gky, (uint32_t)step * BK);
    tck::cp_async_commit();
  };
  // Fragment addressing of the term being MULTIPLIED, in either image layout: element (row e, position k) sits at
  // e * se + k * sk doubles; a fragment pair is rows e and e + 1.
  int fx0 = 0, fx1 = 0, fy0 = 0, sex = 1, sey = 1, skx4 = 0, sky4 = 0;
  auto frag_setup = [&](int k) {
    const int mx = p.terms[k].kfast_x, my = p.terms[k].kfast_y;
    sex = mx ? LDK : 1;
    sey = my ? LDK : 1;
    const int kx1 = mx ? 1 : LD, ky1 = my ? 1 : LD;
    fx0 = (wm0 + 2 * g) * sex + t * kx1;
    fx1 = (wm0 + 2 * g + 16) * sex + t * kx1;
    fy0 = (wn0 + 2 * g) * sey + t * ky1;
    skx4 = 4 * kx1;
    sky4 = 4 * ky1;
  };

  double acc[2][4][2];
  auto zero = [&]() {
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) { acc[j][i][0] = 0.0; acc[j][i][1] = 0.0; }
  };
  zero();
  // scatter offsets of the term being multiplied, fetched when it begins (their latency hides behind its products)
  int bom[8], bon[2];
  double alpha = 1.0;
  auto scatter_setup = [&](int k) {
    const FusedTerm& T = p.terms[k];
    alpha = T.alpha;
#pragma unroll
    for (int h = 0; h < 2; ++h) bon[h] = s_bon[k * kBox + wn0 + 2 * g + h];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int q = 0; q < 4; ++q) bom[4 * i + q] = s_bom[k * kBox + wm0 + 16 * i + 4 * t + q];
  };
  scatter_setup(0);
  // The flattened sequence of (term, K step) stages runs through a ring of kStages buffers: one barrier per stage.
  int term = 0, ks = 0, buf = 0;            // the stage being multiplied
  int iterm = 0, iks = 0, ibuf = 0;         // the next stage to be issued
  int steps = (int)((p.terms[0].kflat + BK - 1) / BK);
  frag_setup(0);
  int ckfl = (int)p.terms[0].kflat, isteps = steps;
  auto issue_next = [&]() {
    if (iterm < p.n_terms) {
      issue(iterm, iks, ibuf);
      ibuf = ibuf + 1 == kStages ? 0 : ibuf + 1;
      if (++iks >= isteps) {
        iks = 0;
        ++iterm;
        if (iterm < p.n_terms) isteps = (int)((p.terms[iterm].kflat + BK - 1) / BK);
      }
    } else {
      tck::cp_async_commit();  // keeps the group count in step
    }
  };
#pragma unroll
  for (int s0 = 0; s0 < kStages - 1; ++s0) issue_next();
  while (term < p.n_terms) {
    tck::cp_async_wait<kStages - 2>();
    __syncthreads();  // the stage is complete for every thread; the buffer issued into below was read a stage ago
    issue_next();
    {
      const double* x = xs + buf * IMG;
      const double* y = ys + buf * IMG;
      const int kleft = ckfl - ks * BK;
      const int nq = kleft >= BK ? BK / 4 : (kleft + 3) / 4;
#pragma unroll
      for (int q = 0; q < BK / 4; ++q) {
        if (q < nq) {
          const double* xq = x + q * skx4;
          const double* yq = y + q * sky4;
          const double2 x0 = make_double2(xq[fx0], xq[fx0 + sex]), x1 = make_double2(xq[fx1], xq[fx1 + sex]);
          const double2 y0 = make_double2(yq[fy0], yq[fy0 + sey]);
          tck::dmma884(acc[0][0][0], acc[0][0][1], y0.x, x0.x);
          tck::dmma884(acc[0][1][0], acc[0][1][1], y0.x, x0.y);
          tck::dmma884(acc[1][0][0], acc[1][0][1], y0.y, x0.x);
          tck::dmma884(acc[1][1][0], acc[1][1][1], y0.y, x0.y);
          tck::dmma884(acc[0][2][0], acc[0][2][1], y0.x, x1.x);
          tck::dmma884(acc[0][3][0], acc[0][3][1], y0.x, x1.y);
          tck::dmma884(acc[1][2][0], acc[1][2][1], y0.y, x1.x);
          tck::dmma884(acc[1][3][0], acc[1][3][1], y0.y, x1.y);
        }
      }
    }
    buf = buf + 1 == kStages ? 0 : buf + 1;
    if (++ks >= steps) {
      // The term is complete: its 64 x 64 products go into the box.  acc[h][2 i + e][h2] is box column
      // n = wn0 + 2 g + h and box row m = wm0 + 16 i + 4 t + e + 2 h2; every (m, n) is one distinct box element, and
      // the next term's scatter is at least one stage (one barrier) away.
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (bon[h] >= 0) {
#pragma unroll
          for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int e = 0; e < 2; ++e)
#pragma unroll
              for (int h2 = 0; h2 < 2; ++h2) {
                const int bo = bom[4 * i + 2 * h2 + e];
                if (bo >= 0) box[box_pos((uint32_t)(bo + bon[h]))] += alpha * acc[h][2 * i + e][h2];
              }
        }
      }
      zero();
      ks = 0;
      ++term;
      if (term < p.n_terms) {
        scatter_setup(term);
        steps = (int)((p.terms[term].kflat + BK - 1) / BK);
        ckfl = (int)p.terms[term].kflat;
        frag_setup(term);
      }
    }
  }
  tck::cp_async_wait<0>();
  __syncthreads();  // every term's scatter is in the box

  // ---- the box meets C once ----
  if (whole) {
    for (uint32_t e = tid; e < p.box_elems; e += kThreads) {
      double* q = C + base_c + p.box_off[e];
      *q = p.beta ? *q + box[box_pos(e)] : box[box_pos(e)];
    }
  } else {
    for (uint32_t e = tid; e < p.box_elems; e += kThreads) {
      uint32_t r = e;
      bool ok = true;
      for (int i = 0; i < p.rank; ++i) {
        const uint32_t c = r % p.b[i];
        r /= p.b[i];
        ok = ok && c < ((limits >> (8 * i)) & 0xff);
      }
      if (ok) {
        double* q = C + base_c + p.box_off[e];
        *q = p.beta ? *q + box[box_pos(e)] : box[box_pos(e)];
      }
    }
  }
}

}  // namespace

// ------------------------------------------------------------------ host ----
struct tc_fused_plan {
  std::vector<TcExpr> terms;
  std::vector<std::string> idx_names;   // output indices in written order, then every contraction index once
  std::vector<int64_t> idx_extent;
  bool committed = false;
  int device = -1;
  FusedArgs args{};
  std::vector<FusedTerm> h_terms;
  FusedTerm* d_terms = nullptr;
  int64_t* d_box_off = nullptr;
  std::vector<int64_t*> d_koff;
  double flops = 0, bytes_fused = 0, bytes_separate = 0;
  std::string why;
};

static int find_name(const std::vector<std::string>& v, const std::string& s) {
  for (size_t i = 0; i < v.size(); ++i)
    if (v[i] == s) return (int)i;
  return -1;
}

extern "C" int tc_plan_create_fused(int n, const char* const* exprs, int dtype, tc_fused_plan** out) {
  if (!exprs || !out || n < 1) return TC_ERR_INVALID_ARG;
  *out = nullptr;
  if (n > kMaxTerms) return TC_ERR_UNSUPPORTED;
  if (dtype != TC_F64) return TC_ERR_UNSUPPORTED;  // the application case (CCSD(T)) is fp64
  tc_fused_plan* p = new (std::nothrow) tc_fused_plan();
  if (!p) return TC_ERR_INVALID_ARG;
  for (int k = 0; k < n; ++k) {
    TcExpr e;
    std::string why;
    const int st = exprs[k] ? tc_parse_expr(exprs[k], &e, &why) : TC_ERR_INVALID_ARG;
    if (st != TC_OK) { delete p; return st; }
    if (e.op == 0) { delete p; return TC_ERR_UNSUPPORTED; }  // every term accumulates
    if (k > 0 && (e.out_name != p->terms[0].out_name || e.out_idx != p->terms[0].out_idx || e.out_ext != p->terms[0].out_ext)) {
      delete p;
      return TC_ERR_INVALID_ARG;  // all terms write the same output, indices in the same order
    }
    p->terms.push_back(e);
  }
  const TcExpr& e0 = p->terms[0];
  if ((int)e0.out_idx.size() > kMaxRank) { delete p; return TC_ERR_UNSUPPORTED; }
  for (size_t i = 0; i < e0.out_idx.size(); ++i) { p->idx_names.push_back(e0.out_idx[i]); p->idx_extent.push_back(e0.out_ext[i]); }
  for (const TcExpr& e : p->terms)
    for (size_t i = 0; i < e.sum_idx.size(); ++i) {
      const int j = find_name(p->idx_names, e.sum_idx[i]);
      if (j < 0) { p->idx_names.push_back(e.sum_idx[i]); p->idx_extent.push_back(e.sum_ext[i]); }
      else if (j < (int)e0.out_idx.size() || p->idx_extent[j] != e.sum_ext[i]) { delete p; return TC_ERR_INVALID_ARG; }
    }
  *out = p;
  return TC_OK;
}

extern "C" int tc_fused_set_extents(tc_fused_plan* p, int n, const char* const* names, const int64_t* extents) {
  if (!p || n < 0 || (n > 0 && (!names || !extents))) return TC_ERR_INVALID_ARG;
  if (p->committed) return TC_ERR_STATE;
  std::vector<int64_t> next = p->idx_extent;
  for (int i = 0; i < n; ++i) {
    const int j = names[i] ? find_name(p->idx_names, names[i]) : -1;
    if (j < 0) return TC_ERR_INVALID_ARG;
    if (extents[i] <= 0) return TC_ERR_EXTENT;
    next[j] = extents[i];
  }
  p->idx_extent = next;
  return TC_OK;
}

// Host part of commit: box shape and per-term tables (needs no GPU).
static int fused_build(tc_fused_plan* p) {
  const TcExpr& e0 = p->terms[0];
  const int rank = (int)e0.out_idx.size();
  auto ext_of = [&](const std::string& n) { return p->idx_extent[find_name(p->idx_names, n)]; };
  // Box: b values of every output index, b the largest power of two with b^s <= 64 where s is the largest number
  // of output indices one input of one term carries (3 + 3 splits of a 6-D output: 4 x 4 x 4 rows and columns).
  size_t s = 1;
  for (const TcExpr& e : p->terms) {
    size_t m = 0, n = 0;
    for (const std::string& i : e.out_idx) (find_name(e.left_idx, i) >= 0 ? m : n) += 1;
    s = std::max(s, std::max(m, n));
  }
  uint32_t b = 64;
  while (b > 1) {
    uint64_t pw = 1;
    for (size_t i = 0; i < s; ++i) pw *= b;
    if (pw <= (uint64_t)kBox) break;
    b >>= 1;
  }
  FusedArgs& a = p->args;
  std::memset(&a, 0, sizeof(a));
  a.n_terms = (int)p->terms.size();
  a.rank = rank;
  a.beta = 1;
  uint64_t boxes = 1, elems = 1;
  int64_t stride = 1;
  for (int i = 0; i < rank; ++i) {
    const int64_t ext = ext_of(e0.out_idx[i]);
    if (ext >= (int64_t(1) << 31)) { p->why = "extent too large"; return TC_ERR_UNSUPPORTED; }
    a.ext[i] = (uint32_t)ext;
    a.b[i] = (uint32_t)std::min<int64_t>(b, ext);
    a.tiles[i] = (uint32_t)((ext + a.b[i] - 1) / a.b[i]);
    a.boxstride[i] = (uint32_t)elems;
    a.sc[i] = stride;
    stride *= ext;
    elems *= a.b[i];
    boxes *= a.tiles[i];
  }
  if (elems > (uint64_t)kBoxElems || boxes >= (uint64_t(1) << 31)) { p->why = "box or grid too large"; return TC_ERR_UNSUPPORTED; }
  a.box_elems = (uint32_t)elems;
  a.total_boxes = boxes;
  p->h_terms.assign(p->terms.size(), FusedTerm{});
  double out_elems = 1;
  for (int i = 0; i < rank; ++i) out_elems *= (double)a.ext[i];
  p->flops = 0;
  p->bytes_fused = 2.0 * 8 * out_elems;
  p->bytes_separate = 0;
  for (size_t k = 0; k < p->terms.size(); ++k) {
    const TcExpr& e = p->terms[k];
    FusedTerm& T = p->h_terms[k];
    T.alpha = e.op < 0 ? -1.0 : 1.0;
    // strides of the term's inputs (compact column-major)
    std::vector<int64_t> sl(e.left_idx.size()), sr(e.right_idx.size());
    int64_t acc = 1;
    for (size_t i = 0; i < e.left_idx.size(); ++i) { sl[i] = acc; acc *= ext_of(e.left_idx[i]); }
    const double count_l = (double)acc;
    acc = 1;
    for (size_t i = 0; i < e.right_idx.size(); ++i) { sr[i] = acc; acc *= ext_of(e.right_idx[i]); }
    const double count_r = (double)acc;
    // classes: output indices by the input that carries them, ordered by their stride in that input
    struct Cls { int out_pos; int64_t s_in; };
    std::vector<Cls> cm, cn;
    for (int i = 0; i < rank; ++i) {
      const int il = find_name(e.left_idx, e0.out_idx[i]), ir = find_name(e.right_idx, e0.out_idx[i]);
      if (il >= 0) { cm.push_back({i, sl[il]}); T.sx[i] = sl[il]; }
      else if (ir >= 0) { cn.push_back({i, sr[ir]}); T.sy[i] = sr[ir]; }
      else { p->why = "an output index appears in neither input"; return TC_ERR_PARSE; }
    }
    auto by_stride = [](const Cls& x, const Cls& y) { return x.s_in < y.s_in; };
    std::sort(cm.begin(), cm.end(), by_stride);
    std::sort(cn.begin(), cn.end(), by_stride);
    auto fill = [&](const std::vector<Cls>& cls, int64_t* rowoff, uint64_t* coord, int32_t* boxoff, int32_t* count) {
      int64_t n = 1;
      for (const Cls& c : cls) n *= a.b[c.out_pos];
      if (n > kBox) return false;
      *count = (int32_t)n;
      for (int r = 0; r < kBox; ++r) {
        rowoff[r] = 0; coord[r] = 0; boxoff[r] = 0;
        if (r >= n) continue;
        int q = r;
        for (const Cls& c : cls) {
          const int v = q % a.b[c.out_pos];
          q /= a.b[c.out_pos];
          rowoff[r] += (int64_t)v * c.s_in;
          coord[r] |= (uint64_t)v << (8 * c.out_pos);
          boxoff[r] += v * (int32_t)a.boxstride[c.out_pos];
        }
      }
      return true;
    };
    if (!fill(cm, T.rowoff_x, T.coord_m, T.boxoff_m, &T.rows) || !fill(cn, T.rowoff_y, T.coord_n, T.boxoff_n, &T.cols)) {
      p->why = "a term's box has more than 64 rows or columns";
      return TC_ERR_UNSUPPORTED;
    }
    // contraction offsets, flattened in sum(...) order
    int64_t kf = 1;
    for (const std::string& n : e.sum_idx) kf *= ext_of(n);
    if (kf >= (int64_t(1) << 31)) { p->why = "contraction too long"; return TC_ERR_UNSUPPORTED; }
    T.kflat = (uint32_t)kf;
    // loader mode per input: 0 = [k][row] image, 1 = [row][k] image (its fastest index is contracted), 2 = the same
    // with 16-byte copies of two consecutive k (that index has an even extent, so rows stay 16-byte aligned)
    // (k is flattened with the contraction index that is fastest in the LEFT input first: an input is walked along
    // k only when that very index is its own fastest one)
    std::string kfirst;
    for (const std::string& n : e.sum_idx)
      if (kfirst.empty() || sl[find_name(e.left_idx, n)] < sl[find_name(e.left_idx, kfirst)]) kfirst = n;
    auto mode_of = [&](const std::vector<std::string>& idx) {
      if (kfirst.empty() || idx[0] != kfirst) return 0;
      return ext_of(kfirst) % 2 == 0 ? 2 : 1;
    };
    T.kfast_x = mode_of(e.left_idx);
    T.kfast_y = mode_of(e.right_idx);
    double prod = out_elems * (double)kf;
    p->flops += 2.0 * prod;
    p->bytes_fused += 8.0 * (count_l + count_r);
    p->bytes_separate += 8.0 * (2.0 * out_elems + count_l + count_r);
  }
  return TC_OK;
}

static void fused_koff(const tc_fused_plan* p, size_t k, std::vector<int64_t>* kx, std::vector<int64_t>* ky) {
  const TcExpr& e = p->terms[k];
  auto ext_of = [&](const std::string& n) { return p->idx_extent[find_name(p->idx_names, n)]; };
  std::vector<int64_t> sl(e.left_idx.size()), sr(e.right_idx.size());
  int64_t acc = 1;
  for (size_t i = 0; i < e.left_idx.size(); ++i) { sl[i] = acc; acc *= ext_of(e.left_idx[i]); }
  acc = 1;
  for (size_t i = 0; i < e.right_idx.size(); ++i) { sr[i] = acc; acc *= ext_of(e.right_idx[i]); }
  // order the contraction indices so that the flattened k walks the faster input index first
  std::vector<std::string> order = e.sum_idx;
  std::stable_sort(order.begin(), order.end(), [&](const std::string& x, const std::string& y) {
    return sl[find_name(e.left_idx, x)] < sl[find_name(e.left_idx, y)];
  });
  const uint32_t kf = p->h_terms[k].kflat;
  kx->assign(kf, 0);
  ky->assign(kf, 0);
  for (uint32_t f = 0; f < kf; ++f) {
    int64_t r = f;
    for (const std::string& n : order) {
      const int64_t ext = ext_of(n), v = r % ext;
      r /= ext;
      (*kx)[f] += v * sl[find_name(e.left_idx, n)];
      (*ky)[f] += v * sr[find_name(e.right_idx, n)];
    }
  }
}

static int fused_smem_bytes(int n_terms) { return (kBoxElems + 2 * kStages * IMG) * 8 + n_terms * (2 * kBox * 8 + 2 * kTabK * 8 + 2 * kBox * 4); }

extern "C" int tc_fused_commit(tc_fused_plan* p) {
  if (!p) return TC_ERR_INVALID_ARG;
  if (p->committed) return TC_OK;
  int st = fused_build(p);
  if (st != TC_OK) return st;
  int dev = 0;
  TC_CUDA_OK(cudaGetDevice(&dev));
  TC_CUDA_OK(cudaFuncSetAttribute(tc_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fused_smem_bytes(kMaxTerms)));
  for (size_t k = 0; k < p->terms.size(); ++k) {
    std::vector<int64_t> kx, ky;
    fused_koff(p, k, &kx, &ky);
    int64_t* d = nullptr;
    TC_CUDA_OK(cudaMalloc(&d, 2 * kx.size() * sizeof(int64_t)));
    p->d_koff.push_back(d);
    TC_CUDA_OK(cudaMemcpy(d, kx.data(), kx.size() * sizeof(int64_t), cudaMemcpyHostToDevice));
    TC_CUDA_OK(cudaMemcpy(d + kx.size(), ky.data(), ky.size() * sizeof(int64_t), cudaMemcpyHostToDevice));
    p->h_terms[k].koff_x = d;
    p->h_terms[k].koff_y = d + kx.size();
  }
  TC_CUDA_OK(cudaMalloc(&p->d_terms, p->h_terms.size() * sizeof(FusedTerm)));
  TC_CUDA_OK(cudaMemcpy(p->d_terms, p->h_terms.data(), p->h_terms.size() * sizeof(FusedTerm), cudaMemcpyHostToDevice));
  p->args.terms = p->d_terms;
  {
    std::vector<int64_t> off(p->args.box_elems);
    for (uint32_t e = 0; e < p->args.box_elems; ++e) {
      uint32_t r = e;
      int64_t o = 0;
      for (int i = 0; i < p->args.rank; ++i) { o += (int64_t)(r % p->args.b[i]) * p->args.sc[i]; r /= p->args.b[i]; }
      off[e] = o;
    }
    TC_CUDA_OK(cudaMalloc(&p->d_box_off, off.size() * sizeof(int64_t)));
    TC_CUDA_OK(cudaMemcpy(p->d_box_off, off.data(), off.size() * sizeof(int64_t), cudaMemcpyHostToDevice));
    p->args.box_off = p->d_box_off;
  }
  p->device = dev;
  p->committed = true;
  return TC_OK;
}

extern "C" int tc_execute_fused(tc_fused_plan* p, void* C, const void* const* A, const void* const* B, void* stream) {
  if (!p || !C || !A || !B) return TC_ERR_INVALID_ARG;
  if (!p->committed) {
    const int st = tc_fused_commit(p);
    if (st != TC_OK) return st;
  }
  int dev = 0;
  TC_CUDA_OK(cudaGetDevice(&dev));
  if (dev != p->device) return TC_ERR_STATE;
  FusedPtrs ptrs{};
  for (size_t k = 0; k < p->terms.size(); ++k) {
    if (!A[k] || !B[k]) return TC_ERR_INVALID_ARG;
    // inputs walked with 16-byte copies must start on 16 bytes (their rows then do too: the plan checked the extents)
    const uintptr_t need_a = p->h_terms[k].kfast_x == 2 ? 15 : 7, need_b = p->h_terms[k].kfast_y == 2 ? 15 : 7;
    if ((reinterpret_cast<uintptr_t>(A[k]) & need_a) || (reinterpret_cast<uintptr_t>(B[k]) & need_b)) return TC_ERR_ALIGNMENT;
    ptrs.x[k] = static_cast<const double*>(A[k]);
    ptrs.y[k] = static_cast<const double*>(B[k]);
  }
  if (reinterpret_cast<uintptr_t>(C) & 7) return TC_ERR_ALIGNMENT;
  tc_fused_kernel<<<(unsigned)p->args.total_boxes, kThreads, fused_smem_bytes(p->args.n_terms), static_cast<cudaStream_t>(stream)>>>(
      p->args, ptrs, static_cast<double*>(C));
  TC_CUDA_OK(cudaGetLastError());
  return TC_OK;
}

extern "C" void tc_fused_destroy(tc_fused_plan* p) {
  if (!p) return;
  for (int64_t* d : p->d_koff) cudaFree(d);
  if (p->d_terms) cudaFree(p->d_terms);
  if (p->d_box_off) cudaFree(p->d_box_off);
  delete p;
}

extern "C" int tc_fused_describe(tc_fused_plan* p, char* buf, size_t cap) {
  if (!p || !buf || cap == 0) return TC_ERR_INVALID_ARG;
  tc_fused_plan tmp;
  const tc_fused_plan* q = p;
  if (!p->committed) {  // run the host part on a copy (needs no GPU)
    tmp.terms = p->terms;
    tmp.idx_names = p->idx_names;
    tmp.idx_extent = p->idx_extent;
    const int st = fused_build(&tmp);
    if (st != TC_OK) {
      std::snprintf(buf, cap, "{\"error\":\"%s\"}", tmp.why.c_str());
      return st;
    }
    q = &tmp;
  }
  std::ostringstream o;
  o.precision(17);
  o << "{\"terms\":" << q->args.n_terms << ",\"rank\":" << q->args.rank << ",\"box\":[";
  for (int i = 0; i < q->args.rank; ++i) o << (i ? "," : "") << q->args.b[i];
  o << "],\"boxes\":" << q->args.total_boxes << ",\"box_elems\":" << q->args.box_elems << ",\"rows_cols\":[";
  for (size_t k = 0; k < q->h_terms.size(); ++k) o << (k ? "," : "") << "[" << q->h_terms[k].rows << "," << q->h_terms[k].cols << "]";
  o << "],\"flops\":" << q->flops << ",\"bytes\":" << q->bytes_fused << ",\"bytes_term_by_term\":" << q->bytes_separate
    << ",\"kernel\":\"tc_fused_kernel\",\"launches\":1}";
  const std::string s = o.str();
  const size_t n = std::min(cap - 1, s.size());
  std::memcpy(buf, s.data(), n);
  buf[n] = '\0';
  return TC_OK;
}
