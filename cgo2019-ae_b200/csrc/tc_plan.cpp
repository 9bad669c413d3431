// Planner: from a parsed expression + extents to the launch description.
//
// This replaces the reference's offline search
// (cogent/src/generators/configurations.py:15-289 -> enumeration.py:15-278 ->
// cost_models.py:11-39), which enumerates thread-block / register-tile index
// groups and ranks them by estimated DRAM transactions.  The B200 kernels tile
// the FLATTENED external index spaces instead of per-index boxes, so the search
// collapses to: classify and order the indices, fuse what is contiguous, pick
// the loader per operand, pick a CTA tile and (for small outputs) a K split.
//
//   M  = external indices of X, ordered by their stride in the output
//   N  = external indices of Y, ordered by their stride in the output
//   K  = contraction indices, ordered by their stride in whichever operand has
//        a contraction index as its fastest index
// where X is the operand that carries the output's fastest index (operands are
// swapped if that is the right one; the product is commutative).  The reference
// makes the same choice when it maps the input holding the output's fastest
// index to the thread-block X dimension (enumeration.py:72-100).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <numeric>
#include <sstream>

#include "tc_internal.h"

namespace {

struct Dim {
  int64_t extent, s_in, s_out;  // for K: s_in = stride in X, s_out = stride in Y
};

int find(const std::vector<std::string>& v, const std::string& s) {
  for (size_t i = 0; i < v.size(); ++i)
    if (v[i] == s) return (int)i;
  return -1;
}

std::vector<int64_t> compact_strides(const std::vector<std::string>& idx, const tc_plan& p) {
  std::vector<int64_t> s(idx.size());
  int64_t acc = 1;
  for (size_t i = 0; i < idx.size(); ++i) {
    s[i] = acc;
    acc *= p.idx_extent[find(p.idx_names, idx[i])];
  }
  return s;
}

// Drops unit extents and merges neighbours that are contiguous in both tensors.
std::vector<Dim> fuse(std::vector<Dim> d) {
  std::vector<Dim> out;
  for (const Dim& x : d) {
    if (x.extent == 1) continue;
    if (!out.empty()) {
      Dim& b = out.back();
      if (x.s_in == b.s_in * b.extent && x.s_out == b.s_out * b.extent) {
        b.extent *= x.extent;
        continue;
      }
    }
    out.push_back(x);
  }
  return out;
}

bool to_dims(const std::vector<Dim>& d, TcDims* t, int64_t* flat) {
  if ((int)d.size() > TC_MAX_DIMS) return false;
  std::memset(t, 0, sizeof(*t));
  t->n = (int)d.size();
  int64_t f = 1;
  for (size_t i = 0; i < d.size(); ++i) {
    t->extent[i] = (uint32_t)d[i].extent;
    t->s_in[i] = d[i].s_in;
    t->s_out[i] = d[i].s_out;
    f *= d[i].extent;
    if (f >= (int64_t(1) << 31)) return false;
  }
  *flat = f;
  return true;
}

int64_t span(const std::vector<int64_t>& ext, const std::vector<int64_t>& str) {
  int64_t s = 1;
  for (size_t i = 0; i < ext.size(); ++i) s += (ext[i] - 1) * str[i];
  return s;
}

// A consumer warp's batch of 8 output rows (n = base + 2g + parity, WM consecutive m) of the persistent fp64
// kernels is one box of a rank-5 view of C when, with each class's dimensions fused as far as they are
// contiguous IN C (the flattened index does not change by that),
//   * the warp's WM outputs of a row sit inside one contiguous run: the fastest fused M dimension has
//     stride 1 and is the only one, or a multiple of the tile,
//   * the 16 rows of two batches stay inside N's fastest fused dimension (the only one, or a multiple of
//     16), which must be even so that n splits into (parity, n / 2),
//   * what is left of both classes fits the two remaining tensor dimensions, and every stride keeps
//     16-byte alignment.
// Then one tiled TMA reduce-add (or store) replaces eight per-row bulk copies (*per_warp); a whole bm x bn tile
// is a box too when its bn rows stay inside N's fastest fused dimension (*per_tile).
void out_box_view(const TcKernelArgs& a, int es, int bm, int bn, TcOutMap* map, bool* per_warp, bool* per_tile) {
  *per_warp = false;
  *per_tile = false;
  *map = TcOutMap{};
  if (!(es == 8 && a.vec_c == 4 && a.M.n >= 1 && a.N.n >= 1 && a.M.s_out[0] == 1)) return;
  auto fuse_out = [](const TcDims& cls, std::vector<int64_t>* ext, std::vector<int64_t>* str) {
    for (int d = 0; d < cls.n; ++d) {
      if (!ext->empty() && cls.s_out[d] == str->back() * ext->back()) ext->back() *= cls.extent[d];
      else { ext->push_back(cls.extent[d]); str->push_back(cls.s_out[d]); }
    }
  };
  std::vector<int64_t> me, ms, ne, ns;
  fuse_out(a.M, &me, &ms);
  fuse_out(a.N, &ne, &ns);
  bool ok = (me.size() == 1 || me[0] % bm == 0) && ne[0] % 2 == 0 && (ne.size() == 1 || ne[0] % 16 == 0) &&
            (me.size() - 1) + (ne.size() - 1) <= 2;
  for (size_t d = 0; d < ne.size(); ++d) ok = ok && ns[d] % 2 == 0 && ns[d] > 0 && ns[d] < (int64_t(1) << 36) && ne[d] < (int64_t(1) << 31);
  for (size_t d = 1; d < me.size(); ++d) ok = ok && ms[d] % 2 == 0 && ms[d] > 0 && ms[d] < (int64_t(1) << 36) && me[d] < (int64_t(1) << 31);
  ok = ok && me[0] < (int64_t(1) << 31);
  if (!ok) return;
  TcOutMap& o = *map;
  o.e0 = (uint32_t)me[0];
  o.f0 = (uint32_t)ne[0];
  o.stride_n = ns[0];
  o.ne = (int32_t)ne.size() - 1;
  o.me = (int32_t)me.size() - 1;
  int r = 0;
  for (size_t d = 1; d < ne.size(); ++d, ++r) { o.ext[r] = (uint32_t)ne[d]; o.stride[r] = ns[d]; }
  for (size_t d = 1; d < me.size(); ++d, ++r) { o.ext[r] = (uint32_t)me[d]; o.stride[r] = ms[d]; }
  *per_warp = true;
  *per_tile = ne.size() == 1 || ne[0] % bn == 0;
}

// The staged output layout of the fp32 kernels: a tile's rows split into runs of E0 elements that are contiguous in
// the output (E0 a multiple of 4, tiles 16-byte aligned); `n_adjacent`: consecutive n are adjacent in the output
// inside blocks of N's fastest extent, so a run and its n leave as one chunk.  Returns E0, or 0 where bulk copies do
// not pay (chunks under 256 bytes) or are not possible.
int64_t staged_run(const TcKernelArgs& a, int bm, int bn, int es, bool* n_adjacent) {
  const int V = 16 / es;
  *n_adjacent = false;
  if (!(a.M.n > 0 && a.M.s_out[0] == 1 && a.vec_c >= V)) return 0;
  const int64_t e = a.M.extent[0];
  const int64_t e0 = e % bm == 0 ? bm : (bm % e == 0 ? e : std::gcd<int64_t>(bm, e));
  if (e0 % V != 0 || e0 < V) return 0;
  *n_adjacent = e0 == e && a.N.n > 0 && a.N.s_out[0] == e && (int64_t)a.N.extent[0] >= bn;
  return (*n_adjacent || e0 * es >= 256) ? e0 : 0;
}
bool wt_eligible(const TcKernelArgs& a, int bm, int es) {
  bool adj;
  return es == 4 && staged_run(a, bm, 128, es, &adj) > 0;
}

}  // namespace

int tc_plan_build(tc_plan* p, std::string* why) {
  std::string dummy;
  if (!why) why = &dummy;
  const TcExpr& e = p->expr;
  const int es = p->dtype == TC_F64 ? 8 : 4;
  auto ext_of = [&](const std::string& n) { return p->idx_extent[find(p->idx_names, n)]; };

  // Per-tensor extents and strides in written order.
  const std::vector<std::string>* tidx[3] = {&e.out_idx, &e.left_idx, &e.right_idx};
  std::vector<int64_t> text[3], tstr[3];
  for (int t = 0; t < 3; ++t) {
    for (const std::string& n : *tidx[t]) text[t].push_back(ext_of(n));
    if (p->custom_strides[t]) {
      if (p->strides[t].size() != tidx[t]->size()) { *why = "stride count does not match tensor rank"; return TC_ERR_INVALID_ARG; }
      tstr[t] = p->strides[t];
      for (int64_t s : tstr[t])
        if (s <= 0) { *why = "strides must be positive"; return TC_ERR_EXTENT; }
      // strides that merely restate the compact layout keep the plan eligible for everything compact plans get
      if (tstr[t] == compact_strides(*tidx[t], *p)) p->custom_strides[t] = false;
    } else {
      tstr[t] = compact_strides(*tidx[t], *p);
    }
  }
  // The output must not alias itself: sorted by stride, each stride must clear the previous extent.
  {
    std::vector<std::pair<int64_t, int64_t>> se;
    for (size_t i = 0; i < text[0].size(); ++i)
      if (text[0][i] > 1) se.push_back({tstr[0][i], text[0][i]});
    std::sort(se.begin(), se.end());
    int64_t need = 1;
    for (auto& x : se) {
      if (x.first < need) { *why = "output strides make elements alias"; return TC_ERR_EXTENT; }
      need = x.first * x.second;
    }
  }
  p->count_c = std::accumulate(text[0].begin(), text[0].end(), int64_t(1), std::multiplies<int64_t>());
  p->count_a = std::accumulate(text[1].begin(), text[1].end(), int64_t(1), std::multiplies<int64_t>());
  p->count_b = std::accumulate(text[2].begin(), text[2].end(), int64_t(1), std::multiplies<int64_t>());
  p->size_c = span(text[0], tstr[0]);
  p->size_a = span(text[1], tstr[1]);
  p->size_b = span(text[2], tstr[2]);

  // Which operand carries the output's fastest (non-unit) index?
  int fvi = -1;
  for (size_t i = 0; i < e.out_idx.size(); ++i)
    if (text[0][i] > 1 && (fvi < 0 || tstr[0][i] < tstr[0][fvi])) fvi = (int)i;
  p->swapped = fvi >= 0 && find(e.left_idx, e.out_idx[fvi]) < 0;
  const int X = p->swapped ? 2 : 1, Y = p->swapped ? 1 : 2;

  std::vector<Dim> dm, dn, dk;
  for (size_t i = 0; i < e.out_idx.size(); ++i) {
    const std::string& n = e.out_idx[i];
    const int ix = find(*tidx[X], n), iy = find(*tidx[Y], n);
    if (ix >= 0) dm.push_back({text[0][i], tstr[X][ix], tstr[0][i]});
    else dn.push_back({text[0][i], tstr[Y][iy], tstr[0][i]});
  }
  for (const std::string& n : e.sum_idx) {
    const int ix = find(*tidx[X], n), iy = find(*tidx[Y], n);
    dk.push_back({ext_of(n), tstr[X][ix], tstr[Y][iy]});
  }
  auto by_out = [](const Dim& a, const Dim& b) { return a.s_out < b.s_out; };
  std::stable_sort(dm.begin(), dm.end(), by_out);
  std::stable_sort(dn.begin(), dn.end(), by_out);
  bool x_k_unit = false, y_k_unit = false;
  for (const Dim& d : dk) {
    if (d.extent > 1 && d.s_in == 1) x_k_unit = true;
    if (d.extent > 1 && d.s_out == 1) y_k_unit = true;
  }
  if (!x_k_unit && y_k_unit)
    std::stable_sort(dk.begin(), dk.end(), [](const Dim& a, const Dim& b) { return a.s_out < b.s_out; });
  else
    std::stable_sort(dk.begin(), dk.end(), [](const Dim& a, const Dim& b) { return a.s_in < b.s_in; });
  dm = fuse(dm);
  dn = fuse(dn);
  dk = fuse(dk);

  // Operand-friendly orders.  By output stride alone, an operand whose own fastest index is an external one that
  // comes late in the output would be gathered 8 bytes per sector (the reference's mapping search blocks two
  // indices in that situation, cogent/src/algs/bases/enumeration.py:72-278).  Tiles here are ranges of the
  // flattened class, so the same effect comes from the ORDER of the class's dimensions:
  //   * N, fp64 (never holds the output's fastest index): ordered by stride in Y when Y's fastest index is external;
  //   * M, fp64: the output's fastest index a and X's fastest external index x are both split by 4 and the digits
  //     ordered (a_lo, x_lo, a_hi, ..., x_hi): a thread still owns 4 consecutive output elements (32 bytes), and
  //     the 4 lanes that share an a_lo fetch 4 consecutive x, one whole sector of X.  (Putting x_lo first made
  //     the loads 16-byte vectors but sent the output through the element-wise epilogue: measured slower.)
  if (p->dtype == TC_F64 && !y_k_unit && dn.size() > 1) {  // (the fp32 epilogues lean on N's order in the output)
    bool y_ext_unit = false;
    for (const Dim& d : dn) y_ext_unit = y_ext_unit || (d.extent > 1 && d.s_in == 1);
    if (y_ext_unit && dn[0].s_in != 1) {
      std::stable_sort(dn.begin(), dn.end(), [](const Dim& a, const Dim& b) { return a.s_in < b.s_in; });
      dn = fuse(dn);
    }
  }
  if (p->dtype == TC_F64 && !x_k_unit && dm.size() > 1 && dm[0].s_in != 1 && dm[0].s_out == 1 && dm[0].extent % 4 == 0) {
    for (size_t j = 1; j < dm.size(); ++j) {
      if (dm[j].s_in != 1 || dm[j].extent < 4 || dm[j].extent % 4 != 0) continue;
      if (dm.size() + 2 > (size_t)TC_MAX_DIMS) break;
      // only when a 128-row tile in output order would hold at most two values of x: with short faster
      // dimensions the tile reaches x by itself and keeps the cheaper row-wise output
      int64_t before = 1;
      for (size_t i = 0; i < j; ++i) before *= dm[i].extent;
      if (before < 64) break;
      const Dim o = dm[0], x = dm[j];
      std::vector<Dim> r;
      r.push_back({4, o.s_in, o.s_out});            // 4 consecutive output elements: 32 bytes of C per thread
      r.push_back({4, x.s_in, x.s_out});            // 4 consecutive x: one whole sector of X per 4 lanes
      if (o.extent / 4 > 1) r.push_back({o.extent / 4, o.s_in * 4, o.s_out * 4});
      for (size_t i = 1; i < dm.size(); ++i) {
        if (i != j) r.push_back(dm[i]);
        else if (x.extent / 4 > 1) r.push_back({x.extent / 4, x.s_in * 4, x.s_out * 4});
      }
      dm = r;
      break;
    }
  }

  TcKernelArgs& a = p->args;
  std::memset(&a, 0, sizeof(a));
  int64_t mf = 1, nf = 1, kf = 1;
  TcDims kd;
  if (!to_dims(dm, &a.M, &mf) || !to_dims(dn, &a.N, &nf) || !to_dims(dk, &kd, &kf)) {
    *why = "a fused index class has more than 8 dimensions or 2^31 elements";
    return TC_ERR_UNSUPPORTED;
  }
  a.Mflat = (uint32_t)mf;
  a.Nflat = (uint32_t)nf;
  a.Kflat = (uint32_t)kf;
  p->kdims = kd;

  // Contraction offset tables (one entry per flattened k).
  p->h_koff_x.assign(kf, 0);
  p->h_koff_y.assign(kf, 0);
  for (int64_t k = 0; k < kf; ++k) {
    int64_t r = k, ox = 0, oy = 0;
    for (int d = 0; d < kd.n; ++d) {
      const int64_t c = r % kd.extent[d];
      r /= kd.extent[d];
      ox += c * kd.s_in[d];
      oy += c * kd.s_out[d];
    }
    p->h_koff_x[k] = ox;
    p->h_koff_y[k] = oy;
  }

  // Kernel family.
  TcKernelChoice& c = p->choice;
  c.dtype = p->dtype;
  const int path = p->opt.path;
  if (p->dtype == TC_F64) {
    if (path == TC_PATH_FFMA || path == TC_PATH_3XTF32 || path == TC_PATH_TCGEN05) { *why = "fp32 path requested for an fp64 plan"; return TC_ERR_INVALID_ARG; }
    c.math = path == TC_PATH_DFMA ? TC_MATH_SIMT : TC_MATH_DMMA;
  } else {
    if (path == TC_PATH_DMMA || path == TC_PATH_DFMA) { *why = "fp64 path requested for an fp32 plan"; return TC_ERR_INVALID_ARG; }
    // AUTO: three TF32 tensor-core products per fp32 product measured faster than FFMA on B200 (the
    // vector-pipe kernel is issue-bound on short contractions) at the same observed error (~3e-7).
    // The tcgen05 form of the same arithmetic (TMEM accumulators) is opt-in: measured beside the mma.sync one.
    c.math = path == TC_PATH_FFMA ? TC_MATH_SIMT : path == TC_PATH_TCGEN05 ? TC_MATH_TF32TC : TC_MATH_TF32X3;
  }

  // Loader per operand.
  const int V = 16 / es;
  auto loader = [&](const TcDims& ext, bool k_is_in, bool* vec, bool* kvec, int32_t* lanes_k) {
    *vec = false;
    *kvec = false;
    *lanes_k = 1;
    auto ks = [&](int d) { return k_is_in ? kd.s_in[d] : kd.s_out[d]; };
    if (ext.n > 0 && ext.s_in[0] == 1) {
      bool ok = ext.extent[0] % V == 0;
      for (int d = 1; d < ext.n; ++d) ok = ok && ext.s_in[d] % V == 0;
      for (int d = 0; d < kd.n; ++d) ok = ok && ks(d) % V == 0;
      *vec = ok;
    } else if (kd.n > 0 && ks(0) == 1) {
      *lanes_k = 32 / es;
      bool ok = kd.extent[0] % V == 0;
      for (int d = 1; d < kd.n; ++d) ok = ok && ks(d) % V == 0;
      for (int d = 0; d < ext.n; ++d) ok = ok && ext.s_in[d] % V == 0;
      *kvec = ok;
    }
  };
  loader(a.M, true, &c.vec_x, &c.kvec_x, &a.lanes_k_x);
  loader(a.N, false, &c.vec_y, &c.kvec_y, &a.lanes_k_y);
  // An operand is a plain 2-D matrix (k fastest, then the flattened external index at a constant pitch)
  // when it has one fused contraction dimension of stride 1 and its external dimensions are contiguous
  // among themselves: then a tile of the flattened class is a box, which TMA can fetch (rows 16 bytes apart or more).
  auto affine = [&](const TcDims& ext, bool k_is_in) {
    if (kd.n != 1 || (k_is_in ? kd.s_in[0] : kd.s_out[0]) != 1 || ext.n < 1) return false;
    for (int d = 1; d < ext.n; ++d)
      if (ext.s_in[d] != ext.s_in[d - 1] * (int64_t)ext.extent[d - 1]) return false;
    return ext.s_in[0] % (16 / es) == 0 && ext.s_in[0] >= (int64_t)kd.extent[0];
  };
  c.tma_x = affine(a.M, true);
  c.tma_y = affine(a.N, false);
  // The transposed case: the whole external class is one contiguous run and the single contraction dimension lies
  // at a constant pitch (rows of the box are then k, 16 bytes apart or more).
  auto affine_ext = [&](const TcDims& ext, bool k_is_in) {
    if (kd.n != 1 || ext.n < 1 || ext.s_in[0] != 1) return false;
    int64_t run = 1;
    for (int d = 0; d < ext.n; ++d) {
      if (ext.s_in[d] != run) return false;
      run *= (int64_t)ext.extent[d];
    }
    const int64_t pitch = k_is_in ? kd.s_in[0] : kd.s_out[0];
    return pitch % (16 / es) == 0 && pitch >= run;
  };
  c.tma_xe = es == 4 && affine_ext(a.M, true);
  c.tma_ye = es == 4 && affine_ext(a.N, false);

  // Contiguous output elements per thread access.
  a.vec_c = 1;
  if (a.M.n > 0 && a.M.s_out[0] == 1) {
    for (int v : {4, 2}) {
      bool ok = a.M.extent[0] % v == 0;
      for (int d = 1; d < a.M.n; ++d) ok = ok && a.M.s_out[d] % v == 0;
      for (int d = 0; d < a.N.n; ++d) ok = ok && a.N.s_out[d] % v == 0;
      if (ok && v * es >= 8) { a.vec_c = v; break; }
    }
  }
  a.alpha = e.op < 0 ? -1.0 : 1.0;
  a.beta = e.op == 0 ? 0 : 1;

  // CTA tile and kernel variant.  Rules distilled from tile sweeps on B200 over the
  // benchmark configurations (they replace the reference's transaction-count
  // cost model, cogent/src/algs/bases/cost_models.py:191-574):
  //   * fp64 tensor pipe: the persistent warp-specialised kernel (variant 2), N tile
  //     64 or 96, whichever wastes less of Nflat (128 x 64 or 64 x 96 per consumer group);
  //   * vector pipe: 128 x 128;
  //   * anything that would leave most SMs without a tile: 64 x 64, one CTA per tile.
  const int64_t sms = p->sm_count > 0 ? p->sm_count : TC_DEFAULT_SMS;
  int bm = 128, bn = 128, variant = 0;
  bool slice_persistent = false;  // the persistent reduce-add kernel with K slices (few tiles, long contraction)
  if (p->opt.tile_m > 0 || p->opt.tile_n > 0) {
    bm = p->opt.tile_m;
    bn = p->opt.tile_n;
    variant = p->opt.variant > 0 ? p->opt.variant - 1 : 0;
  } else {
    if (c.math == TC_MATH_DMMA) {
      // fp64 on the tensor pipe: the persistent kernels, chosen by a small cost model (this takes the place of the
      // reference's ranking of mappings by estimated DRAM transactions, cogent/src/algs/bases/cost_models.py:191-574).
      // Per candidate (tile, kernel) the time of one SM is  tiles per SM  x  max(products + idle, output bytes / rate):
      //   products   2 bm bn K / (DMMA rate of one SM x the share of it the kernel's main loop reaches), K rounded up to 4;
      //   idle       cycles per tile during which the pipe waits (epilogue, hand-overs), measured per kernel;
      //   rate       what the kernel's way of reaching C sustains: reduce-adds of the copy engine 0.76 of the
      //              measured copy bandwidth, tiled loads + stores of a resident tile 0.92;
      //   tiles per SM is rounded up (wave quantisation) and edge tiles count in full (waste).
      // Constants come from the B200 measurements recorded beside the kernels; the device's SM count is the plan's.
      struct Cand { int bm, bn, variant; double idle, rate, eff; };  // eff: share of the DMMA rate its main loop reaches
      const Cand cands[] = {{128, 64, 2, 2100.0, 0.76, 0.90}, {64, 96, 2, 800.0, 0.76, 0.86}, {128, 32, 2, 1500.0, 0.76, 0.84},
                            {128, 64, 3, 1450.0, 0.92, 0.92}};
      const double clk = 1.9e9, flop_per_clk = 37.0e12 / 148.0 / clk, byte_per_clk = 6.5e12 / 148.0 / clk;
      const double kpad = (double)((kf + 3) / 4 * 4);
      double best = 0;
      p->why.clear();
      for (const Cand& k : cands) {
        if (!tc_kernel_exists(TC_F64, TC_MATH_DMMA, k.bm, k.bn, k.variant)) continue;
        if (k.variant == 3) {  // needs whole tiles to be boxes of a rank-5 view of C, and nothing that pins the epilogue
          TcOutMap view;
          bool per_warp = false, per_tile = false;
          out_box_view(a, es, k.bm, k.bn, &view, &per_warp, &per_tile);
          if (!per_tile || p->opt.tma == 1 || p->opt.tma == 2 || p->opt.c_path != 0) continue;
          // ... and pays only where the output traffic is the longer side: per output element the memory system moves
          // 16 bytes while the pipe does 2 K flops, equal near K = 46.  On long contractions its single consumer group
          // and two producer warps measured a third slower than the two-group kernel (21 against 31 TFLOP/s).
          if (2.0 * es / 6.5e12 < 0.85 * 2.0 * (double)kf / 37.0e12) continue;
        }
        const double tiles_c = (double)((mf + k.bm - 1) / k.bm) * (double)((nf + k.bn - 1) / k.bn);
        const double products = 2.0 * k.bm * k.bn * kpad / (flop_per_clk * k.eff);
        const double out_bytes = (e.op == 0 ? 1.0 : 2.0) * k.bm * k.bn * es;
        const double per_tile = std::max(products + k.idle, out_bytes / (byte_per_clk * k.rate));
        const double t = std::ceil(tiles_c / (double)sms) * per_tile / clk;
        // the first candidate (128 x 64, two groups) stays unless another is estimated a tenth faster: the model knows
        // tiles, waste and waves, not how well each loader shape feeds each tile
        // (the output-resident kernel has its own gate above and the same tile: any estimated gain counts)
        if (best == 0 || t < best * (k.variant == 3 ? 0.98 : 0.90)) { best = t; bm = k.bm; bn = k.bn; variant = k.variant; }
      }
      p->estimate_s = best;
    }
    if (c.math != TC_MATH_DMMA && c.dtype == TC_F32) {
      // fp32: 96 rows instead of 128 when that makes the tile a whole number of the output's contiguous
      // runs (e.g. a fastest output index of extent 24), which the bulk epilogue wants.
      const int64_t e0 = (a.M.n > 0 && a.M.s_out[0] == 1) ? a.M.extent[0] : 0;
      if (e0 > 0 && e0 % 128 != 0 && 128 % e0 != 0 && (96 % e0 == 0 || e0 % 96 == 0)) bm = 96;
    }
    if (c.math == TC_MATH_TF32X3 && path == TC_PATH_AUTO && p->opt.split_k <= 1) {
      // The same three products as tcgen05.mma with the accumulators in tensor memory measured 10 % (K = 24)
      // to 80 % (K = 2048) faster than the mma.sync form on B200.  Its tiles are bm x 128; it is chosen when
      // they fill the GPU, almost all of them are whole (ragged tiles leave row by row through shared memory) and whole
      // tiles can leave through the staged bulk epilogue.
      auto mostly_whole = [](int64_t n, int64_t b) { return n % b == 0 || n >= 16 * b; };
      bool bulk_ok = false;
      if (a.M.n > 0 && a.M.s_out[0] == 1 && a.vec_c >= 4) {
        const int64_t e = a.M.extent[0];
        const int64_t e0 = e % bm == 0 ? bm : (bm % e == 0 ? e : std::gcd<int64_t>(bm, e));
        const bool n_adjacent = e0 == e && a.N.n > 0 && a.N.s_out[0] == e && (int64_t)a.N.extent[0] >= 128;
        bulk_ok = e0 % 4 == 0 && (n_adjacent || e0 * es >= 256);
      }
      const int64_t ctas_tc = ((mf + bm - 1) / bm) * ((nf + 127) / 128);
      if (bulk_ok && ctas_tc >= 2 * sms && mostly_whole(mf, bm) && mostly_whole(nf, 128) &&
          tc_kernel_exists(TC_F32, TC_MATH_TF32TC, bm, 128, 0)) {
        c.math = TC_MATH_TF32TC;
        bn = 128;
      }
    }
    if (c.math == TC_MATH_TF32TC && p->opt.split_k == 0 && p->opt.c_path != 2) {
      // ... as the persistent kernel (two accumulators in tensor memory, output tile staged in shared memory)
      // wherever its tile buffers can hold the output in runs that leave as bulk copies and both operands are
      // fetched 16 bytes at a time: its four loader warps issue element gathers slower than the 24 warps of three
      // resident one-tile CTAs do (measured on the fp32 items of the reference's benchmark list, one operand
      // gathered by element: 12.0-14.7 against 15.5-16.7 TFLOP/s; with vector loads on both sides it is 8-27 % ahead).
      const int tbm = (bm == 96 || bm == 128) ? bm : 128;
      const bool vector_loads = (c.vec_x || c.kvec_x) && (c.vec_y || c.kvec_y);
      if (vector_loads && wt_eligible(a, tbm, es) && tc_kernel_exists(TC_F32, TC_MATH_TF32TC, tbm, 128, 1)) { bm = tbm; bn = 128; variant = 1; }
    }
    const int64_t ctas = ((mf + bm - 1) / bm) * ((nf + bn - 1) / bn);
    if (ctas < 2 * sms) {
      // Too few tiles to fill the GPU.  fp64 with a long contraction stays on the persistent 128 x 64 kernel and
      // slices K over its CTAs instead (16-byte loads along k, tiled TMA operands and two consumer groups are worth
      // more than small tiles: measured 3-4 x on few-tile, long-K items of the reference's list); everything else
      // runs one CTA per 64 x 64 tile, with K slices where K is long.
      const int64_t t128 = ((mf + 127) / 128) * ((nf + 63) / 64), t64 = ((mf + 63) / 64) * ((nf + 63) / 64);
      // ... unless its 128-row tiles pad the problem much more than 64-row ones would while the small kernel can
      // at least load one operand by vector (measured on 312 x 296 outputs: 20 % more padded work cost 20 %)
      const bool padding_ok = 2 * t128 * 100 <= t64 * 112 || (!c.vec_x && !c.vec_y);
      if (c.math == TC_MATH_DMMA && p->opt.split_k == 0 && (kf + TC_BK - 1) / TC_BK >= 64 && t128 * ((kf + TC_BK - 1) / TC_BK / 16) >= 2 * sms &&
          padding_ok && tc_kernel_exists(TC_F64, TC_MATH_DMMA, 128, 64, 2)) {
        bm = 128; bn = 64; variant = 2;
        slice_persistent = true;
      } else {
        bm = 64; bn = 64; variant = 0;
        if (c.math == TC_MATH_TF32TC) c.math = TC_MATH_TF32X3;  // no 64-wide tcgen05 tile: same arithmetic on mma.sync
      }
    }
    if (p->opt.variant > 0) variant = p->opt.variant - 1;
  }
  c.bm = bm;
  c.bn = bn;
  c.variant = variant;
  if (tc_kernel_is_tmem_persistent(c) && !wt_eligible(a, bm, es)) {
    *why = "the persistent tcgen05 kernel needs an output whose tile rows are 16-byte aligned contiguous runs";
    return TC_ERR_UNSUPPORTED;
  }
  if (!tc_kernel_exists(c.dtype, c.math, bm, bn, c.variant)) { *why = "requested CTA tile / variant is not compiled in"; return TC_ERR_UNSUPPORTED; }
  a.bm = bm;
  a.bn = bn;
  a.tiles_m = (uint32_t)((mf + bm - 1) / bm);
  a.tiles_n = (uint32_t)((nf + bn - 1) / bn);
  const int64_t tiles = (int64_t)a.tiles_m * a.tiles_n;
  const int bk = TC_BK;
  // Persistent kernels: walk the tiles in column blocks of 32 M tiles when one sweep over all of M would drag more
  // than a few MB of X through L2 per row of tiles (see tile_coords in tc_kernels.cuh).
  a.mblock_w = 0;
  if (tc_kernel_is_persistent(c) && a.tiles_m > 64 && a.tiles_n > 1 && (double)mf * (double)kf * es > 4.0e6) a.mblock_w = 32;

  // K split: only when the tile count cannot fill the GPU and K is long.
  int64_t ksplit = 1;
  const int64_t ksteps = (kf + bk - 1) / bk;
  const bool persistent = tc_kernel_is_persistent(c);
  // Persistent kernels do not split K, except the fp64 reduce-add kernel: on request (forced tile and split_k), or
  // where the planner kept it for a problem of few tiles (about four work items per SM, slices of at least 16 steps).
  const bool ws_kernel = c.math == TC_MATH_DMMA && c.variant == 2;
  if (persistent && ws_kernel && p->opt.split_k > 1) ksplit = std::min<int64_t>(p->opt.split_k, ksteps);
  else if (persistent && ws_kernel && slice_persistent)
    ksplit = std::max<int64_t>(1, std::min<int64_t>((4 * sms + tiles - 1) / tiles, ksteps / 16));
  else if (persistent) ksplit = 1;
  else if (p->opt.split_k > 1) ksplit = std::min<int64_t>(p->opt.split_k, ksteps);
  else if (p->opt.split_k == 0 && tiles * 2 <= sms && ksteps >= 16)
    ksplit = std::max<int64_t>(1, std::min<int64_t>((2 * sms) / tiles, ksteps / 8));
  // The tensor cores accumulate fp32 with truncation: measured against exact sums on B200 the relative error of
  // one accumulation chain grows linearly with its length (2e-6 at K = 256, 7e-6 at 1024, 3e-5 at 4096), for
  // mma.sync and tcgen05 alike, while FFMA stays at 1e-6.  No tensor-core plan therefore runs a chain longer
  // than TC_TF32_CHAIN products (tc_options.split_k >= 1 overrides this, as does TC_PATH_FFMA):
  //   * where the slices' partial tiles fit 1 GiB of plan-owned scratch, the contraction is K-sliced and the
  //     combine kernel adds the slices in round-to-nearest fp32;
  //   * larger outputs run the contraction as sequential PASSES over consecutive ranges of at most that many
  //     products, every pass accumulating into the output itself (the first with the expression's operator,
  //     the others with `+=`; the additions into C are round-to-nearest).  A pass re-reads and re-writes C,
  //     which at 512 products per element is noise beside the arithmetic.
  p->passes = 1;
  // (the persistent tcgen05 kernel cuts its chains itself: segments of at most 32 K steps that alternate between
  // two accumulators and are added into the output tile in shared memory)
  if ((c.math == TC_MATH_TF32X3 || c.math == TC_MATH_TF32TC) && p->opt.split_k == 0 && !persistent) {
    const int64_t per_slice = tiles * bm * bn * (int64_t)es;
    const int64_t want = std::min<int64_t>((kf + TC_TF32_CHAIN - 1) / TC_TF32_CHAIN, ksteps);
    if (want > 1 && want * per_slice > (int64_t(1) << 30) && ksplit == 1) p->passes = (int)std::min<int64_t>(want, 1 << 20);
    else ksplit = std::max<int64_t>(ksplit, want);
  }
  if (p->passes > 1) {
    const int64_t steps_per_pass = (ksteps + p->passes - 1) / p->passes;
    p->passes = (int)((ksteps + steps_per_pass - 1) / steps_per_pass);
    a.k_chunk = (uint32_t)(steps_per_pass * bk);
    a.ksplit = 1;
  }
  if (p->passes == 1) {
    int64_t chunk_steps = (ksteps + ksplit - 1) / ksplit;
    ksplit = (ksteps + chunk_steps - 1) / chunk_steps;
    a.ksplit = (uint32_t)ksplit;
    a.k_chunk = (uint32_t)(chunk_steps * bk);
  }
  if (tiles * ksplit >= (int64_t(1) << 31)) { *why = "too many tiles"; return TC_ERR_UNSUPPORTED; }
  p->ws_bytes = ksplit > 1 ? (size_t)(ksplit * tiles * bm * bn) * es : 0;
  p->launches = ksplit > 1 ? 2 : p->passes;

  // Staged bulk epilogue of the vector-pipe kernels: the tile's rows split into runs of E0 elements
  // contiguous in the output; if the output's next index belongs to the other operand (its stride equals
  // the extent of the fastest one), consecutive n are adjacent too within blocks of that index's extent.
  a.epi_run = 0;
  a.epi_n_span = 0;
  if (c.math != TC_MATH_DMMA && ksplit == 1) {
    // bulk copies pay off from a few hundred bytes per chunk; shorter runs keep the read-modify-write
    bool n_adjacent = false;
    const int64_t e0 = staged_run(a, bm, bn, es, &n_adjacent);
    if (e0 > 0) {
      a.epi_run = (int32_t)e0;
      if (n_adjacent) a.epi_n_span = (int32_t)a.N.extent[0];
    }
  }

  // Persistent fp64 kernels: which output batches / tiles are boxes of a rank-5 view of C (see out_box_view).
  c.tma_c = false;
  c.tma_ct = false;
  a.cmap = TcOutMap{};
  if (persistent) out_box_view(a, es, bm, bn, &a.cmap, &c.tma_c, &c.tma_ct);

  double prod = 1.0;
  for (int64_t x : p->idx_extent) prod *= (double)x;
  p->flops = 2.0 * prod;
  p->bytes = (double)es * ((e.op == 0 ? 1.0 : 2.0) * p->count_c + p->count_a + p->count_b);
  return TC_OK;
}

std::string tc_plan_to_json(const tc_plan& p) {
  std::ostringstream o;
  o.precision(17);
  const TcKernelArgs& a = p.args;
  auto dims = [&](const TcDims& d) {
    o << "[";
    for (int i = 0; i < d.n; ++i)
      o << (i ? "," : "") << "{\"extent\":" << d.extent[i] << ",\"s_in\":" << d.s_in[i] << ",\"s_out\":" << d.s_out[i] << "}";
    o << "]";
  };
  o << "{\"expr\":" << tc_expr_to_json(p.expr) << ",\"dtype\":\"" << (p.dtype == TC_F64 ? "f64" : "f32")
    << "\",\"committed\":" << (p.committed ? "true" : "false");
  // longest tensor-core accumulation chain of the plan
  uint32_t chain = std::min<uint32_t>(a.k_chunk, a.Kflat);
  if (tc_kernel_is_tmem_persistent(p.choice)) {
    const uint32_t steps = (a.Kflat + TC_BK - 1) / TC_BK, segs = (steps + 31) / 32;
    chain = std::min<uint32_t>(a.Kflat, ((steps + segs - 1) / segs) * TC_BK);
  }
  if (p.committed) {
    o << ",\"swapped\":" << (p.swapped ? "true" : "false") << ",\"M\":";
    dims(a.M);
    o << ",\"N\":";
    dims(a.N);
    o << ",\"K\":";
    dims(p.kdims);
    o << ",\"Mflat\":" << a.Mflat << ",\"Nflat\":" << a.Nflat << ",\"Kflat\":" << a.Kflat
      << ",\"math\":\"" << (p.choice.math == TC_MATH_DMMA ? "dmma" : p.choice.math == TC_MATH_TF32X3 ? "tf32x3" : p.choice.math == TC_MATH_TF32TC ? "tf32x3_tcgen05" : (p.dtype == TC_F64 ? "dfma" : "ffma"))
      << "\",\"kernel\":\"" << tc_kernel_name(p.choice) << "\",\"tile\":[" << p.choice.bm << "," << p.choice.bn << "," << TC_BK
      << "],\"variant\":" << p.choice.variant << ",\"tiles\":[" << a.tiles_m << "," << a.tiles_n << "],\"estimate_us\":" << p.estimate_s * 1e6 << ",\"mblock_w\":" << a.mblock_w << ",\"ksplit\":" << a.ksplit
      << ",\"k_chunk\":" << a.k_chunk << ",\"passes\":" << p.passes << ",\"chain\":" << chain << ",\"vec_x\":" << (p.choice.vec_x ? "true" : "false")
      << ",\"vec_y\":" << (p.choice.vec_y ? "true" : "false") << ",\"kvec_x\":" << (p.choice.kvec_x ? "true" : "false")
      << ",\"kvec_y\":" << (p.choice.kvec_y ? "true" : "false") << ",\"tma_x\":" << (p.choice.tma_x ? "true" : "false")
      << ",\"tma_y\":" << (p.choice.tma_y ? "true" : "false") << ",\"tma_xe\":" << (p.choice.tma_xe ? "true" : "false")
      << ",\"tma_ye\":" << (p.choice.tma_ye ? "true" : "false") << ",\"tma_c\":" << (p.choice.tma_c ? "true" : "false") << ",\"tma_ct\":" << (p.choice.tma_ct ? "true" : "false")
      << ",\"lanes_k_x\":" << a.lanes_k_x
      << ",\"lanes_k_y\":" << a.lanes_k_y << ",\"vec_c\":" << a.vec_c << ",\"epi_run\":" << a.epi_run << ",\"epi_n_span\":" << a.epi_n_span << ",\"beta\":" << a.beta
      << ",\"alpha\":" << a.alpha << ",\"workspace_bytes\":" << p.ws_bytes << ",\"launches\":" << p.launches
      << ",\"flops\":" << p.flops << ",\"bytes\":" << p.bytes;
  }
  o << "}";
  return o.str();
}
