// One contraction over several GPUs of a box from ONE host process: one plan, one stream and (for the
// contraction split) one NCCL communicator per device.
//
// Two splits, both strided views of the FULL tensors, so nothing is repacked (the geometry is the one
// cgo2019-ae_b200/shard.py uses for one process per GPU):
//   external     an index of the output is cut into contiguous ranges, one per device; every output element is an
//                independent sum, so there is no exchange: each device runs the same kernels on its slab;
//   contraction  a contraction index is cut; each device writes a full-size partial result into scratch it owns,
//                one reduce-scatter (NCCL, all devices in one group call) leaves device d with the summed chunk d,
//                which the library's axpy kernel applies to chunk d of that device's output.
// The reference is single-GPU (its only stream: nwchem-tccg/tccg_kernels.cu:228); this layer has no counterpart
// there.  NCCL is looked up at run time (dlopen of libnccl.so.2) and only by plans of the contraction kind.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <cstring>
#include <mutex>
#include <sstream>
#include <string>
#include <vector>

#include "tc_internal.h"

namespace {

// The few NCCL entry points used, declared here so that the library has no link-time dependency on NCCL.
typedef struct ncclComm* ncclComm_t;
struct Nccl {
  int (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  int (*ReduceScatter)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  bool ok = false;
};
constexpr int kNcclFloat32 = 7, kNcclFloat64 = 8, kNcclSum = 0;  // ncclDataType_t / ncclRedOp_t values of nccl.h

Nccl* nccl() {
  static Nccl n;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return;
    n.CommInitAll = reinterpret_cast<decltype(n.CommInitAll)>(dlsym(h, "ncclCommInitAll"));
    n.CommDestroy = reinterpret_cast<decltype(n.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
    n.GroupStart = reinterpret_cast<decltype(n.GroupStart)>(dlsym(h, "ncclGroupStart"));
    n.GroupEnd = reinterpret_cast<decltype(n.GroupEnd)>(dlsym(h, "ncclGroupEnd"));
    n.ReduceScatter = reinterpret_cast<decltype(n.ReduceScatter)>(dlsym(h, "ncclReduceScatter"));
    n.ok = n.CommInitAll && n.CommDestroy && n.GroupStart && n.GroupEnd && n.ReduceScatter;
  });
  return &n;
}

struct Shard {
  int device = 0;
  int64_t start = 0, count = 0;      // range of the cut index
  int64_t offset[3] = {0, 0, 0};      // element offset of the device's view inside C, A, B
  std::string local_expr;
  tc_plan* plan = nullptr;
  cudaStream_t stream = nullptr;
  void* partial = nullptr;            // contraction kind: padded full-size partial result
  void* reduced = nullptr;            // ... and this device's summed chunk
  ncclComm_t comm = nullptr;
};

std::vector<int64_t> compact(const std::vector<std::string>& idx, const std::vector<std::string>& names,
                             const std::vector<int64_t>& ext) {
  std::vector<int64_t> s;
  int64_t acc = 1;
  for (const std::string& i : idx) {
    s.push_back(acc);
    acc *= ext[std::find(names.begin(), names.end(), i) - names.begin()];
  }
  return s;
}

}  // namespace

struct tc_sharded_plan {
  TcExpr e;
  int dtype = TC_F64;
  int kind = TC_SHARD_EXTERNAL;
  std::string cut;                    // the index that is cut ("" until chosen)
  bool cut_given = false;
  std::vector<std::string> names;     // out_idx then sum_idx
  std::vector<int64_t> extent;        // full extents
  std::vector<Shard> shards;
  std::vector<int64_t> stride[3];     // strides of the FULL tensors
  int64_t full_size[3] = {0, 0, 0};
  int64_t chunk = 0, padded = 0;      // contraction kind: elements of C per device (last one may be short)
  bool committed = false;
  std::string why;
};

namespace {

int64_t extent_of(const tc_sharded_plan& p, const std::string& n) {
  return p.extent[std::find(p.names.begin(), p.names.end(), n) - p.names.begin()];
}

std::string rewrite(const tc_sharded_plan& p, const std::string& cut, int64_t local, int op) {
  auto ext = [&](const std::string& n) { return n == cut ? local : extent_of(p, n); };
  std::ostringstream o;
  o << p.e.out_name << " [";
  for (size_t i = 0; i < p.e.out_idx.size(); ++i) o << (i ? "," : "") << p.e.out_idx[i] << "," << ext(p.e.out_idx[i]);
  o << "] " << (op > 0 ? "+=" : op < 0 ? "-=" : "=") << " sum(";
  for (size_t i = 0; i < p.e.sum_idx.size(); ++i) o << (i ? "," : "") << p.e.sum_idx[i] << "," << ext(p.e.sum_idx[i]);
  o << ") * " << p.e.left_name << " [";
  for (size_t i = 0; i < p.e.left_idx.size(); ++i) o << (i ? "," : "") << p.e.left_idx[i];
  o << "] * " << p.e.right_name << " [";
  for (size_t i = 0; i < p.e.right_idx.size(); ++i) o << (i ? "," : "") << p.e.right_idx[i];
  o << "];";
  return o.str();
}

// Ranges, views and local expressions of every device (host arithmetic only).
int build_geometry(tc_sharded_plan* p) {
  const std::vector<std::string>& pool = p->kind == TC_SHARD_EXTERNAL ? p->e.out_idx : p->e.sum_idx;
  if (pool.empty()) { p->why = "nothing to cut"; return TC_ERR_UNSUPPORTED; }
  if (!p->cut_given) {
    // the largest index of the kind; among equal output indices the slowest one (its slabs of C are contiguous),
    // among equal contraction indices the first one
    p->cut = pool[0];
    for (const std::string& n : pool) {
      const int64_t a = extent_of(*p, n), b = extent_of(*p, p->cut);
      if (a > b || (a == b && p->kind == TC_SHARD_EXTERNAL)) p->cut = n;
    }
  } else if (std::find(pool.begin(), pool.end(), p->cut) == pool.end()) {
    p->why = p->kind == TC_SHARD_EXTERNAL ? "the cut index is not an output index" : "the cut index is not a contraction index";
    return TC_ERR_INVALID_ARG;
  }
  const std::vector<std::string>* tidx[3] = {&p->e.out_idx, &p->e.left_idx, &p->e.right_idx};
  for (int t = 0; t < 3; ++t) {
    p->stride[t] = compact(*tidx[t], p->names, p->extent);
    p->full_size[t] = 1;
    for (const std::string& n : *tidx[t]) p->full_size[t] *= extent_of(*p, n);
  }
  const int64_t world = (int64_t)p->shards.size(), full = extent_of(*p, p->cut);
  const int64_t base = full / world, rem = full % world;
  for (int64_t r = 0; r < world; ++r) {
    Shard& s = p->shards[r];
    s.start = r * base + std::min(r, rem);
    s.count = base + (r < rem ? 1 : 0);
    for (int t = 0; t < 3; ++t) {
      const auto it = std::find(tidx[t]->begin(), tidx[t]->end(), p->cut);
      s.offset[t] = it == tidx[t]->end() ? 0 : s.start * p->stride[t][it - tidx[t]->begin()];
    }
    // every device of the contraction kind writes its partial sum with `=` into scratch
    s.local_expr = rewrite(*p, p->cut, std::max<int64_t>(s.count, 1), p->kind == TC_SHARD_CONTRACTION ? 0 : p->e.op);
  }
  p->chunk = (p->full_size[0] + world - 1) / world;
  p->padded = p->chunk * world;
  return TC_OK;
}

void release(tc_sharded_plan* p) {
  for (Shard& s : p->shards) {
    if (s.plan || s.stream || s.partial || s.reduced || s.comm) cudaSetDevice(s.device);
    if (s.comm && nccl()->ok) nccl()->CommDestroy(s.comm);
    if (s.plan) tc_plan_destroy(s.plan);
    if (s.partial) cudaFree(s.partial);
    if (s.reduced) cudaFree(s.reduced);
    if (s.stream) cudaStreamDestroy(s.stream);
    s.comm = nullptr; s.plan = nullptr; s.partial = nullptr; s.reduced = nullptr; s.stream = nullptr;
  }
  p->committed = false;
}

}  // namespace

extern "C" int tc_plan_create_sharded(const char* expr, int dtype, int n_devices, const int* device_ids, int kind,
                                      const char* index, tc_sharded_plan** out) {
  if (!expr || !out || n_devices < 1 || n_devices > 64) return TC_ERR_INVALID_ARG;
  *out = nullptr;
  if ((dtype != TC_F64 && dtype != TC_F32) || (kind != TC_SHARD_EXTERNAL && kind != TC_SHARD_CONTRACTION)) return TC_ERR_INVALID_ARG;
  TcExpr e;
  std::string why;
  const int st = tc_parse_expr(expr, &e, &why);
  if (st != TC_OK) return st;
  tc_sharded_plan* p = new (std::nothrow) tc_sharded_plan();
  if (!p) return TC_ERR_INVALID_ARG;
  p->e = e;
  p->dtype = dtype;
  p->kind = kind;
  if (index && *index) { p->cut = index; p->cut_given = true; }
  for (size_t i = 0; i < e.out_idx.size(); ++i) { p->names.push_back(e.out_idx[i]); p->extent.push_back(e.out_ext[i]); }
  for (size_t i = 0; i < e.sum_idx.size(); ++i) { p->names.push_back(e.sum_idx[i]); p->extent.push_back(e.sum_ext[i]); }
  p->shards.resize(n_devices);
  for (int d = 0; d < n_devices; ++d) p->shards[d].device = device_ids ? device_ids[d] : d;
  *out = p;
  return TC_OK;
}

extern "C" int tc_sharded_set_extents(tc_sharded_plan* p, int n, const char* const* names, const int64_t* extents) {
  if (!p || n < 0 || (n > 0 && (!names || !extents))) return TC_ERR_INVALID_ARG;
  if (p->committed) return TC_ERR_STATE;
  std::vector<int64_t> next = p->extent;
  for (int i = 0; i < n; ++i) {
    if (!names[i]) return TC_ERR_INVALID_ARG;
    if (extents[i] <= 0) return TC_ERR_EXTENT;
    const auto it = std::find(p->names.begin(), p->names.end(), std::string(names[i]));
    if (it == p->names.end()) return TC_ERR_INVALID_ARG;
    next[it - p->names.begin()] = extents[i];
  }
  p->extent = next;
  return TC_OK;
}

extern "C" int tc_sharded_describe(tc_sharded_plan* p, char* buf, size_t cap) {
  if (!p || !buf || cap == 0) return TC_ERR_INVALID_ARG;
  int st = TC_OK;
  if (!p->committed) st = build_geometry(p);
  std::ostringstream o;
  if (st != TC_OK) {
    o << "{\"error\":\"" << p->why << "\"}";
  } else {
    o << "{\"kind\":\"" << (p->kind == TC_SHARD_EXTERNAL ? "external" : "contraction") << "\",\"index\":\"" << p->cut
      << "\",\"dtype\":\"" << (p->dtype == TC_F64 ? "f64" : "f32") << "\",\"committed\":" << (p->committed ? "true" : "false")
      << ",\"full_sizes\":[" << p->full_size[0] << "," << p->full_size[1] << "," << p->full_size[2] << "],\"chunk\":" << p->chunk
      << ",\"padded\":" << p->padded << ",\"c_slab_contiguous\":"
      << ((p->kind == TC_SHARD_EXTERNAL && (p->e.out_idx.back() == p->cut || p->shards.size() == 1)) ? "true" : "false") << ",\"strides\":[";
    for (int t = 0; t < 3; ++t) {
      o << (t ? "," : "") << "[";
      for (size_t i = 0; i < p->stride[t].size(); ++i) o << (i ? "," : "") << p->stride[t][i];
      o << "]";
    }
    o << "],\"shards\":[";
    for (size_t r = 0; r < p->shards.size(); ++r) {
      const Shard& s = p->shards[r];
      o << (r ? "," : "") << "{\"device\":" << s.device << ",\"start\":" << s.start << ",\"count\":" << s.count << ",\"empty\":"
        << (s.count == 0 ? "true" : "false") << ",\"offsets\":[" << s.offset[0] << "," << s.offset[1] << "," << s.offset[2]
        << "],\"local_expr\":\"" << s.local_expr << "\"}";
    }
    o << "]}";
  }
  const std::string text = o.str();
  if (text.size() + 1 > cap) return TC_ERR_INVALID_ARG;
  std::memcpy(buf, text.c_str(), text.size() + 1);
  return st;
}

extern "C" int tc_sharded_commit(tc_sharded_plan* p) {
  if (!p) return TC_ERR_INVALID_ARG;
  if (p->committed) return TC_OK;
  int st = build_geometry(p);
  if (st != TC_OK) return st;
  const size_t es = p->dtype == TC_F64 ? 8 : 4;
  if (p->kind == TC_SHARD_CONTRACTION && p->shards.size() > 1 && !nccl()->ok) {
    p->why = "libnccl.so.2 not found";
    return TC_ERR_UNSUPPORTED;
  }
  int prev = 0;
  cudaGetDevice(&prev);
  for (Shard& s : p->shards) {
    if (cudaSetDevice(s.device) != cudaSuccess) { st = TC_ERR_CUDA; break; }
    if (cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) != cudaSuccess) { st = TC_ERR_CUDA; break; }
    if (p->kind == TC_SHARD_CONTRACTION) {
      if (cudaMalloc(&s.partial, (size_t)p->padded * es) != cudaSuccess || cudaMalloc(&s.reduced, (size_t)p->chunk * es) != cudaSuccess ||
          cudaMemsetAsync(s.partial, 0, (size_t)p->padded * es, s.stream) != cudaSuccess) { st = TC_ERR_CUDA; break; }
    }
    if (s.count == 0) continue;  // more devices than index values: nothing to compute here
    st = tc_plan_create(s.local_expr.c_str(), p->dtype, nullptr, &s.plan);
    if (st != TC_OK) break;
    // views of the full tensors: the inputs always; the output too when it is the device's full copy
    for (int t = p->kind == TC_SHARD_CONTRACTION ? 1 : 0; t < 3 && st == TC_OK; ++t)
      st = tc_plan_set_strides(s.plan, t, (int)p->stride[t].size(), p->stride[t].data());
    if (st == TC_OK) st = tc_plan_commit(s.plan);
    if (st != TC_OK) break;
  }
  if (st == TC_OK && p->kind == TC_SHARD_CONTRACTION && p->shards.size() > 1) {
    std::vector<ncclComm_t> comms(p->shards.size());
    std::vector<int> devs;
    for (const Shard& s : p->shards) devs.push_back(s.device);
    if (nccl()->CommInitAll(comms.data(), (int)devs.size(), devs.data()) != 0) { p->why = "ncclCommInitAll failed"; st = TC_ERR_CUDA; }
    else for (size_t r = 0; r < comms.size(); ++r) p->shards[r].comm = comms[r];
  }
  cudaSetDevice(prev);
  if (st != TC_OK) { release(p); return st; }
  p->committed = true;
  return TC_OK;
}

extern "C" int tc_execute_sharded(tc_sharded_plan* p, void* const* C, const void* const* A, const void* const* B, int flags) {
  if (!p || !C || !A || !B) return TC_ERR_INVALID_ARG;
  if (!p->committed) return TC_ERR_STATE;
  const size_t es = p->dtype == TC_F64 ? 8 : 4;
  const bool c_is_slab = (flags & TC_SHARD_C_IS_SLAB) != 0;
  if (c_is_slab && !(p->kind == TC_SHARD_EXTERNAL && (p->e.out_idx.back() == p->cut || p->shards.size() == 1))) return TC_ERR_INVALID_ARG;
  int prev = 0, st = TC_OK;
  cudaGetDevice(&prev);
  for (size_t r = 0; r < p->shards.size() && st == TC_OK; ++r) {
    Shard& s = p->shards[r];
    if (cudaSetDevice(s.device) != cudaSuccess) { st = TC_ERR_CUDA; break; }
    const char* a = static_cast<const char*>(A[r]) + s.offset[1] * (int64_t)es;
    const char* b = static_cast<const char*>(B[r]) + s.offset[2] * (int64_t)es;
    if (p->kind == TC_SHARD_EXTERNAL) {
      if (!s.plan) continue;
      // (a slab of the slowest index is compact and has the full tensor's strides: the same plan serves both)
      char* c = static_cast<char*>(C[r]) + (c_is_slab ? 0 : s.offset[0] * (int64_t)es);
      st = tc_execute(s.plan, c, a, b, s.stream);
    } else if (s.plan) {
      st = tc_execute(s.plan, s.partial, a, b, s.stream);
    }
  }
  if (st == TC_OK && p->kind == TC_SHARD_CONTRACTION) {
    const int nt = p->dtype == TC_F64 ? kNcclFloat64 : kNcclFloat32;
    if (p->shards.size() > 1) {
      nccl()->GroupStart();
      for (Shard& s : p->shards)
        if (nccl()->ReduceScatter(s.partial, s.reduced, (size_t)p->chunk, nt, kNcclSum, s.comm, s.stream) != 0) st = TC_ERR_CUDA;
      if (nccl()->GroupEnd() != 0) st = TC_ERR_CUDA;
    }
    for (size_t r = 0; r < p->shards.size() && st == TC_OK; ++r) {
      Shard& s = p->shards[r];
      if (cudaSetDevice(s.device) != cudaSuccess) { st = TC_ERR_CUDA; break; }
      const int64_t lo = std::min<int64_t>((int64_t)r * p->chunk, p->full_size[0]), hi = std::min<int64_t>(lo + p->chunk, p->full_size[0]);
      if (hi <= lo) continue;
      const void* src = p->shards.size() > 1 ? s.reduced : s.partial;
      char* mine = static_cast<char*>(C[r]) + lo * (int64_t)es;
      if (p->e.op == 0) {
        if (cudaMemcpyAsync(mine, src, (size_t)(hi - lo) * es, cudaMemcpyDeviceToDevice, s.stream) != cudaSuccess) st = TC_ERR_CUDA;
      } else {
        st = tc_axpy(mine, src, hi - lo, p->dtype, p->e.op < 0 ? -1.0 : 1.0, s.stream);
      }
    }
  }
  cudaSetDevice(prev);
  return st;
}

extern "C" int tc_sharded_synchronize(tc_sharded_plan* p) {
  if (!p) return TC_ERR_INVALID_ARG;
  if (!p->committed) return TC_ERR_STATE;
  int prev = 0, st = TC_OK;
  cudaGetDevice(&prev);
  for (Shard& s : p->shards) {
    if (cudaSetDevice(s.device) != cudaSuccess || cudaStreamSynchronize(s.stream) != cudaSuccess) st = TC_ERR_CUDA;
    int code = 0;
    if (st == TC_OK && s.plan && tc_plan_status(s.plan, &code) == TC_OK && code != 0) st = TC_ERR_DEVICE_WAIT;
  }
  cudaSetDevice(prev);
  return st;
}

extern "C" void tc_sharded_destroy(tc_sharded_plan* p) {
  if (!p) return;
  int prev = 0;
  cudaGetDevice(&prev);
  release(p);
  cudaSetDevice(prev);
  delete p;
}
