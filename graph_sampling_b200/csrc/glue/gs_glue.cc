// TorchScript front end of the sampler: registers `gs_classes.Graph` and the `gs_ops` free operators with
// the method names of the reference's registry (src/pybind.cc:11-86) — CamelCase as registered there and the
// snake_case spelling its Python layer calls (python/gs/matrix_api/matrix.py) — so that
// `torch.classes.load_library("libgs.so")` gives the same object a user of the reference drives.
//
// This file holds only bookkeeping: which sparse formats a graph owns, its id maps, edge data, tuple orders.
// Every piece of arithmetic goes through the C ABI of gsb200.h with raw device pointers and torch's current
// stream.  The state kept per graph and the effect of each method on it follow gs::Graph
// (src/graph.h:113-126, src/graph.cc).  Where the reference aborts the process (LOG(FATAL)), TORCH_CHECK
// raises instead.
#include <c10/cuda/CUDAStream.h>
#include <torch/custom_class.h>
#include <torch/script.h>

#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <tuple>
#include <vector>

#include "../../../include/gsb200.h"

namespace gsglue {

using torch::Tensor;
using OptTensor = torch::optional<Tensor>;

constexpr int64_t kCOO = 1, kCSC = 2, kCSR = 4, kDCSC = 8, kDCSR = 16;

// ---- C ABI plumbing ---------------------------------------------------------------------------------------
static gsb_ctx* Ctx() {
  static thread_local gsb_ctx* ctx[64] = {nullptr};
  const int dev = c10::cuda::current_device();
  TORCH_CHECK(dev >= 0 && dev < 64, "unsupported device index ", dev);
  if (!ctx[dev]) {
    const int st = gsb_ctx_create(dev, &ctx[dev]);
    TORCH_CHECK(st == GSB_OK, "gsb_ctx_create failed: ", gsb_status_string(st), " (a CUDA device is required)");
  }
  return ctx[dev];
}
static void* Stream() { return (void*)c10::cuda::getCurrentCUDAStream().stream(); }
static void Check(int st, const char* what) {
  TORCH_CHECK(st == GSB_OK, what, ": ", gsb_status_string(st), " ", gsb_last_error_message(Ctx()));
}
static const int64_t* IP(const Tensor& t) { return t.defined() && t.numel() ? t.data_ptr<int64_t>() : nullptr; }
static int64_t* MP(Tensor& t) { return t.defined() && t.numel() ? t.data_ptr<int64_t>() : nullptr; }
static const float* FP(const Tensor& t) { return t.defined() && t.numel() ? t.data_ptr<float>() : nullptr; }
// Graph arrays may live in pinned host memory, which the kernels read in place over the unified address space
// (the reference accepts the same: src/graph_ops.cc:144,226, src/cuda/slicing.cu:128); results are always allocated
// on the current device.
static bool Pinned(const Tensor& t) { return !t.is_cuda() && t.is_pinned(); }
// Kernels are launched on the CURRENT device's stream with the current device's context: a tensor that lives on
// another GPU is refused here instead of being dereferenced from the wrong device.
static void SameDevice(const Tensor& t, const char* name) {
  TORCH_CHECK(!t.is_cuda() || t.device().index() == c10::cuda::current_device(), name, " is on cuda:",
              (int)t.device().index(), " while cuda:", (int)c10::cuda::current_device(),
              " is the current device; set the device (torch.cuda.device) before calling");
}
static Tensor Ids(const Tensor& t, const char* name) {
  TORCH_CHECK((t.is_cuda() || Pinned(t)) && t.scalar_type() == torch::kInt64, name, " must be an int64 CUDA (or pinned host) tensor");
  SameDevice(t, name);
  TORCH_CHECK(t.is_cuda() || t.is_contiguous(), name, ": a pinned host tensor must be contiguous");
  return t.contiguous();
}
static Tensor Floats(const Tensor& t, const char* name) {
  TORCH_CHECK((t.is_cuda() || Pinned(t)) && t.scalar_type() == torch::kFloat32, name, " must be a float32 CUDA (or pinned host) tensor");
  SameDevice(t, name);
  TORCH_CHECK(t.is_cuda() || t.is_contiguous(), name, ": a pinned host tensor must be contiguous");
  return t.contiguous();
}
static torch::Device DeviceOf(const Tensor& t) {
  return t.is_cuda() ? t.device() : torch::Device(torch::kCUDA, c10::cuda::current_device());
}
static c10::TensorOptions OnDevice(const Tensor& like) { return like.options().device(DeviceOf(like)); }
// src[index] for per-edge arrays that may be pinned (edge data: float32, edge ids: int64, copied as pairs of words):
// the GPU reads the pinned array in place, as gs::impl::IndexSelectCPUFromGPU does (src/graph.cc:296-306).
static Tensor Take(const Tensor& src, const Tensor& index);
static Tensor EmptyIds(int64_t n, const Tensor& like) { return torch::empty({n}, OnDevice(like).dtype(torch::kInt64)); }
static Tensor Take(const Tensor& src, const Tensor& index) {
  if (src.is_cuda()) return src.index({index});
  TORCH_CHECK(Pinned(src) && src.is_contiguous() && src.dim() == 1, "a host-side edge array must be pinned, contiguous and 1-D");
  const bool ids = src.scalar_type() == torch::kInt64;
  TORCH_CHECK(ids || src.scalar_type() == torch::kFloat32, "a pinned edge array must be int64 or float32");
  Tensor idx = Ids(index, "index");
  const int64_t n = idx.numel(), words = ids ? 2 : 1;
  Tensor out = torch::empty({n}, OnDevice(src));
  if (n)
    Check(gsb_gather_rows(Ctx(), Stream(), (const float*)src.data_ptr(), src.numel(), words, IP(idx), n, (float*)out.data_ptr()),
          "gsb_gather_rows");
  return out;
}

// Largest node count among the graphs loaded so far (0 = none): the id bound that operators without a graph
// argument (gs_ops.BatchCSRRelabel) may assume and verify.
static std::atomic<int64_t> g_node_bound{0};
static void NoteNodeBound(int64_t n) {
  int64_t cur = g_node_bound.load();
  while (n > cur && !g_node_bound.compare_exchange_weak(cur, n)) {
  }
}
static std::atomic<uint64_t> g_seed_base{7777};
static std::atomic<uint64_t> g_seed_counter{0};
static uint64_t NextSeed() { return g_seed_base.load() * 0x9E3779B97F4A7C15ull + g_seed_counter.fetch_add(1); }

// ---- storage (src/graph_storage.h:9-30) ------------------------------------------------------------------------
struct CSC {
  Tensor indptr, indices;
  OptTensor e_ids;
};
struct COO {
  Tensor row, col;
  OptTensor e_ids;
  bool row_sorted = false, col_sorted = false;
};
struct Sliced {  // {sub_indptr, other coordinate per edge (optional), sub_indices, select_index, gathered data (optional)}
  Tensor indptr, coo_other, indices, select, data;
};

// ---- operator wrappers ------------------------------------------------------------------------------------------
static Sliced ColSlice(const CSC& g, const Tensor& ids, bool with_coo, const OptTensor& data) {
  Tensor n_ids = Ids(ids, "node ids");
  const int64_t S = n_ids.numel();
  Sliced r;
  r.indptr = EmptyIds(S + 1, g.indptr);
  int64_t nnz = 0;
  const int64_t num_cols = g.indptr.numel() - 1;
  Check(gsb_col_slice_count(Ctx(), Stream(), IP(g.indptr), num_cols, IP(n_ids), S, MP(r.indptr), &nnz),
        "gsb_col_slice_count");
  r.indices = EmptyIds(nnz, g.indptr);
  r.select = EmptyIds(nnz, g.indptr);
  if (with_coo) r.coo_other = EmptyIds(nnz, g.indptr);
  Tensor d, e;
  if (data.has_value()) {
    d = Floats(data.value(), "edge data");
    r.data = torch::empty({nnz}, OnDevice(d));
    if (g.e_ids.has_value()) e = g.e_ids.value();
  }
  Check(gsb_col_slice_fill(Ctx(), Stream(), IP(g.indptr), IP(g.indices), num_cols, IP(n_ids), S, IP(r.indptr), nnz,
                           MP(r.indices),
                           MP(r.select), with_coo ? MP(r.coo_other) : nullptr, FP(d), IP(e),
                           r.data.defined() && nnz ? r.data.data_ptr<float>() : nullptr),
        "gsb_col_slice_fill");
  return r;
}

static Sliced Sample(const CSC& g, const Tensor* seeds, int64_t fanout, bool replace, bool with_coo,
                     const Tensor* probs, const OptTensor& data) {
  Tensor s;
  if (seeds) s = Ids(*seeds, "column ids");
  const int64_t S = seeds ? s.numel() : g.indptr.numel() - 1;
  const int64_t cap = S * fanout;
  Sliced r;
  r.indptr = EmptyIds(S + 1, g.indptr);
  r.indices = EmptyIds(cap, g.indptr);
  r.select = EmptyIds(cap, g.indptr);
  if (with_coo) r.coo_other = EmptyIds(cap, g.indptr);
  Tensor d, e, out_d, p;
  if (data.has_value()) {
    d = Floats(data.value(), "edge data");
    out_d = torch::empty({cap}, OnDevice(d));
    if (g.e_ids.has_value()) e = g.e_ids.value();
  }
  int64_t nnz = 0;
  if (probs) {
    p = Floats(*probs, "edge probabilities");
    TORCH_CHECK(p.numel() == g.indices.numel(), "edge_probs must have one entry per edge of the operand");
    Check(gsb_sample_weighted(Ctx(), Stream(), IP(g.indptr), IP(g.indices), g.indptr.numel() - 1, FP(p),
                              seeds ? IP(s) : nullptr, S, fanout,
                              replace, NextSeed(), MP(r.indptr), MP(r.indices), MP(r.select),
                              with_coo ? MP(r.coo_other) : nullptr, FP(d), IP(e),
                              out_d.defined() && cap ? out_d.data_ptr<float>() : nullptr, cap, &nnz),
          "gsb_sample_weighted");
  } else {
    Check(gsb_sample_uniform(Ctx(), Stream(), IP(g.indptr), IP(g.indices), g.indptr.numel() - 1,
                             seeds ? IP(s) : nullptr, S, fanout, replace,
                             NextSeed(), MP(r.indptr), MP(r.indices), MP(r.select),
                             with_coo ? MP(r.coo_other) : nullptr, FP(d), IP(e),
                             out_d.defined() && cap ? out_d.data_ptr<float>() : nullptr, cap, &nnz),
          "gsb_sample_uniform");
  }
  r.indices = r.indices.narrow(0, 0, nnz);
  r.select = r.select.narrow(0, 0, nnz);
  if (with_coo) r.coo_other = r.coo_other.narrow(0, 0, nnz);
  if (out_d.defined()) r.data = out_d.narrow(0, 0, nnz);
  return r;
}

static std::tuple<Tensor, std::vector<Tensor>> Relabel(const std::vector<Tensor>& mapping,
                                                       const std::vector<Tensor>& to_relabel) {
  TORCH_CHECK(!mapping.empty() && mapping.size() <= GSB_MAX_SEGMENTS && to_relabel.size() <= GSB_MAX_SEGMENTS,
              "relabel takes 1..", GSB_MAX_SEGMENTS, " mapping tensors and at most ", GSB_MAX_SEGMENTS, " tensors to relabel");
  std::vector<Tensor> maps, rels, outs;
  const int64_t* ip[GSB_MAX_SEGMENTS] = {nullptr};
  int64_t il[GSB_MAX_SEGMENTS] = {0};
  const int64_t* rp[GSB_MAX_SEGMENTS] = {nullptr};
  int64_t rl[GSB_MAX_SEGMENTS] = {0};
  int64_t* ro[GSB_MAX_SEGMENTS] = {nullptr};
  int64_t n = 0;
  for (size_t i = 0; i < mapping.size(); ++i) {
    maps.push_back(Ids(mapping[i], "mapping tensor"));
    ip[i] = IP(maps[i]);
    il[i] = maps[i].numel();
    n += il[i];
  }
  for (size_t i = 0; i < to_relabel.size(); ++i) {
    rels.push_back(Ids(to_relabel[i], "tensor to relabel"));
    outs.push_back(torch::empty_like(rels[i]));
    rp[i] = IP(rels[i]);
    rl[i] = rels[i].numel();
    ro[i] = MP(outs[i]);
  }
  Tensor unique = EmptyIds(n, maps[0]);
  int64_t nu = 0;
  Check(gsb_unique_relabel(Ctx(), Stream(), ip, il, (int)maps.size(), MP(unique), rp, rl, ro, (int)rels.size(), &nu),
        "gsb_unique_relabel");
  return {unique.narrow(0, 0, nu), outs};
}

static std::tuple<Tensor, Tensor, Tensor, Tensor> RowSliceCSC(const CSC& g, const Tensor& ids, bool with_coo) {
  Tensor rows = Ids(ids, "row ids");
  const int64_t nc = g.indptr.numel() - 1, E = g.indices.numel();
  Tensor out_indptr = EmptyIds(nc + 1, g.indptr), oi = EmptyIds(E, g.indptr), os = EmptyIds(E, g.indptr), oc;
  if (with_coo) oc = EmptyIds(E, g.indptr);
  int64_t nnz = 0;
  Check(gsb_row_slice_csc(Ctx(), Stream(), IP(g.indptr), IP(g.indices), nc, E, IP(rows), rows.numel(), MP(out_indptr),
                          MP(oi), MP(os), with_coo ? MP(oc) : nullptr, &nnz),
        "gsb_row_slice_csc");
  if (with_coo) oc = oc.narrow(0, 0, nnz);
  return {out_indptr, oc, oi.narrow(0, 0, nnz), os.narrow(0, 0, nnz)};
}

static std::tuple<Tensor, Tensor, Tensor> RowSliceCOO(const Tensor& key, const Tensor& other, const Tensor& ids) {
  Tensor rows = Ids(ids, "ids");
  const int64_t E = key.numel();
  Tensor o_k = EmptyIds(E, key), o_o = EmptyIds(E, key), o_s = EmptyIds(E, key);
  int64_t nnz = 0;
  Check(gsb_row_slice_coo(Ctx(), Stream(), IP(key), IP(other), E, IP(rows), rows.numel(), MP(o_k), MP(o_o), MP(o_s),
                          &nnz),
        "gsb_row_slice_coo");
  return {o_k.narrow(0, 0, nnz), o_o.narrow(0, 0, nnz), o_s.narrow(0, 0, nnz)};
}

static Tensor ExpandOffsets(const CSC& g) {
  Tensor col = EmptyIds(g.indices.numel(), g.indptr);
  Check(gsb_csc2coo(Ctx(), Stream(), IP(g.indptr), g.indptr.numel() - 1, MP(col)), "gsb_csc2coo");
  return col;
}

// (indptr, other sorted by key, permutation or nullopt): src/cuda/format_transform.cu:135-156
static std::tuple<Tensor, Tensor, OptTensor> SortByKey(const Tensor& key, const Tensor& other, int64_t num_keys,
                                                       bool sorted) {
  const int64_t E = key.numel();
  Tensor indptr = EmptyIds(num_keys + 1, key), out = EmptyIds(E, key), perm;
  if (!sorted) perm = EmptyIds(E, key);
  Check(gsb_coo2csc(Ctx(), Stream(), IP(key), IP(other), E, num_keys, sorted, MP(indptr), MP(out),
                    sorted ? nullptr : MP(perm)),
        "gsb_coo2csc");
  return {indptr, out, sorted ? OptTensor() : OptTensor(perm)};
}

struct Bcast {  // CalcBcastOff, src/bcast.cc:24-76
  int64_t lhs_len = 1, rhs_len = 1, out_len = 1, reduce_size = 1;
  std::vector<int64_t> lhs_off, rhs_off;
  bool use = false;
};
static Bcast CalcBcast(const std::string& op, const Tensor& lhs, const Tensor& rhs) {
  Bcast b;
  for (int64_t i = 1; i < lhs.dim(); ++i) b.lhs_len *= lhs.size(i);
  for (int64_t i = 1; i < rhs.dim(); ++i) b.rhs_len *= rhs.size(i);
  if (op != "copy_lhs" && op != "copy_rhs") {
    b.use = lhs.dim() != rhs.dim();
    for (int64_t i = 1; !b.use && i < lhs.dim(); ++i) b.use = lhs.size(i) != rhs.size(i);
  }
  if (b.use) {
    const int64_t max_ndim = std::max(lhs.dim(), rhs.dim()) - 1;
    int64_t out_len = 1, j = 0, stride_l = 1, stride_r = 1;
    if (op == "dot") {
      b.reduce_size = lhs.size(lhs.dim() - 1);
      j = 1;
    }
    b.lhs_off.push_back(0);
    b.rhs_off.push_back(0);
    for (; j < max_ndim; ++j) {
      const int64_t dl = (lhs.dim() - 1 - j < 1) ? 1 : lhs.size(lhs.dim() - 1 - j);
      const int64_t dr = (rhs.dim() - 1 - j < 1) ? 1 : rhs.size(rhs.dim() - 1 - j);
      for (int64_t i = 1; i < std::max(dl, dr); ++i)
        for (int64_t q = 0; q < out_len; ++q) {
          b.lhs_off.push_back(b.lhs_off[q] + i * (i < dl ? 1 : 0) * stride_l);
          b.rhs_off.push_back(b.rhs_off[q] + i * (i < dr ? 1 : 0) * stride_r);
        }
      out_len *= std::max(dl, dr);
      stride_l *= dl;
      stride_r *= dr;
    }
    b.out_len = out_len;
  } else {
    b.out_len = (op == "copy_rhs") ? b.rhs_len : b.lhs_len;
    if (op == "dot") {
      b.reduce_size = lhs.size(lhs.dim() - 1);
      b.out_len /= b.reduce_size;
    }
  }
  return b;
}

static void Sddmm(const std::string& op, const Tensor& row, const Tensor* col, const Tensor* indptr,
                  const OptTensor& e_ids, const Tensor& lhs_in, const Tensor& rhs_in, Tensor out, int64_t lt,
                  int64_t rt) {
  static const char* names[] = {"add", "sub", "mul", "div", "copy_lhs", "copy_rhs", "dot"};
  int code = -1;
  for (int i = 0; i < 7; ++i)
    if (op == names[i]) code = i;
  TORCH_CHECK(code >= 0, "unknown SDDMM op ", op);
  Tensor lhs = Floats(lhs_in, "lhs"), rhs = Floats(rhs_in, "rhs");
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == torch::kFloat32 && out.is_contiguous(),
              "out must be a contiguous float32 CUDA tensor");
  const Bcast b = CalcBcast(op, lhs, rhs);
  const int64_t E = row.numel();
  TORCH_CHECK(out.numel() == E * b.out_len, "out has ", out.numel(), " elements, expected ", E * b.out_len);
  Tensor lo, ro, e;
  if (b.use) {
    lo = torch::tensor(b.lhs_off, torch::dtype(torch::kInt64)).to(row.device());
    ro = torch::tensor(b.rhs_off, torch::dtype(torch::kInt64)).to(row.device());
  }
  if (e_ids.has_value()) e = e_ids.value();
  Check(gsb_sddmm(Ctx(), Stream(), code, IP(row), col ? IP(*col) : nullptr, indptr ? IP(*indptr) : nullptr,
                  indptr ? indptr->numel() - 1 : 0, IP(e), E, FP(lhs), FP(rhs), out.numel() ? out.data_ptr<float>() : nullptr,
                  (int)lt, (int)rt, b.lhs_len, b.rhs_len, b.out_len, b.reduce_size, IP(lo), IP(ro)),
        "gsb_sddmm");
}

// ---- Graph -----------------------------------------------------------------------------------------------------
class Graph : public torch::CustomClassHolder {
 public:
  explicit Graph(bool is_subgraph) : is_subgraph_(is_subgraph) {}
  Graph(bool is_subgraph, OptTensor col_ids, OptTensor row_ids, int64_t num_cols, int64_t num_rows)
      : is_subgraph_(is_subgraph), num_cols_(num_cols), num_rows_(num_rows), col_ids_(col_ids), row_ids_(row_ids) {}

  // loading (src/graph.cc:14-60)
  void LoadCSC(Tensor indptr, Tensor indices) {
    csc_ = std::make_shared<CSC>(CSC{Ids(indptr, "indptr"), Ids(indices, "indices"), torch::nullopt});
    num_cols_ = num_rows_ = indptr.numel() - 1;
    num_edges_ = indices.numel();
    NoteNodeBound(num_cols_);
  }
  void LoadCOO(Tensor row, Tensor col) {
    coo_ = std::make_shared<COO>(COO{Ids(row, "row"), Ids(col, "col"), torch::nullopt, false, false});
    const int64_t n = std::max(std::get<0>(torch::_unique(row)).numel(), std::get<0>(torch::_unique(col)).numel());
    num_cols_ = num_rows_ = n;
    num_edges_ = row.numel();
  }
  void LoadCSCWithColIds(Tensor column_ids, Tensor indptr, Tensor indices) {
    TORCH_CHECK(column_ids.numel() == indptr.numel() - 1, "length of column_ids is not aligned with indptr");
    csc_ = std::make_shared<CSC>(CSC{Ids(indptr, "indptr"), Ids(indices, "indices"), torch::nullopt});
    col_ids_ = column_ids;
    num_cols_ = column_ids.numel();
    num_rows_ = indices.numel() ? indices.max().item<int64_t>() + 1 : 0;
    num_edges_ = indices.numel();
  }
  void SetMetaData(OptTensor col_ids, OptTensor row_ids, int64_t num_cols, int64_t num_rows) {
    col_ids_ = col_ids;
    row_ids_ = row_ids;
    num_cols_ = num_cols;
    num_rows_ = num_rows;
  }
  void SetCOOByTensor(Tensor row, Tensor col, OptTensor e_ids, bool row_sorted, bool col_sorted) {
    coo_ = std::make_shared<COO>(COO{row, col, e_ids, row_sorted, col_sorted});
    known_csc_ = nullptr, known_csr_ = nullptr;
  }
  void SetData(Tensor data) { data_ = data; }
  int64_t GetNumRows() { return num_rows_; }
  int64_t GetNumCols() { return num_cols_; }
  int64_t GetNumEdges() { return num_edges_; }

  OptTensor GetData(std::string order) {
    Tensor data = DataOrOnes();
    if (order == "col") {
      CreateSparseFormat(kCSC);
      if (csc_->e_ids.has_value()) return data.index({csc_->e_ids.value()});
    } else if (order == "row") {
      CreateSparseFormat(kCSR);
      if (csr_->e_ids.has_value()) return data.index({csr_->e_ids.value()});
    }
    return data;
  }

  // lazy formats (src/graph.cc:585-644, src/graph_ops.cc:13-60)
  void CreateSparseFormat(int64_t format) {
    if (format == kCOO) {
      if (!coo_) coo_ = AnyToCOO();
    } else if (format == kCSC) {
      if (csc_) {
        TORCH_CHECK(!val_col_ids_.has_value(), "Require CSC, get DCSC instead");
        return;
      }
      if (known_csc_) {
        csc_ = known_csc_;
        return;
      }
      if (!coo_) coo_ = AnyToCOO();
      csc_ = FromCOO(*coo_, num_cols_, true);
    } else if (format == kDCSC) {
      if (csc_) {
        TORCH_CHECK(val_col_ids_.has_value(), "Require DCSC, get CSC instead");
        return;
      }
      if (!coo_) coo_ = AnyToCOO();
      Tensor val;
      std::tie(csc_, val) = CompactFromCOO(*coo_, num_cols_, true);
      val_col_ids_ = val;
    } else if (format == kCSR) {
      if (csr_) {
        TORCH_CHECK(!val_row_ids_.has_value(), "Require CSR, get DCSR instead");
        return;
      }
      if (known_csr_) {
        csr_ = known_csr_;
        return;
      }
      if (!coo_) coo_ = AnyToCOO();
      csr_ = FromCOO(*coo_, num_rows_, false);
    } else if (format == kDCSR) {
      if (csr_) {
        TORCH_CHECK(val_row_ids_.has_value(), "Require DCSR, get CSR instead");
        return;
      }
      if (!coo_) coo_ = AnyToCOO();
      Tensor val;
      std::tie(csr_, val) = CompactFromCOO(*coo_, num_rows_, false);
      val_row_ids_ = val;
    } else {
      TORCH_CHECK(false, "unknown sparse format");
    }
  }

  // Doubly compressed forms: offsets only over the columns (rows) that have edges, plus the list of those ids
  // (src/cuda/format_transform.cu:172-203, src/graph_ops.cc:62-110).
  static std::pair<std::shared_ptr<CSC>, Tensor> CompactFromCOO(const COO& c, int64_t num_items, bool to_csc) {
    std::shared_ptr<CSC> dense = FromCOO(c, num_items, to_csc);
    const int64_t n = dense->indptr.numel() - 1;
    Tensor degree = dense->indptr.slice(0, 1, n + 1) - dense->indptr.slice(0, 0, n);
    Tensor val = torch::nonzero(degree > 0).reshape({-1});
    Tensor indptr = torch::cat({dense->indptr.index({val}), dense->indptr.slice(0, n, n + 1)});
    return {std::make_shared<CSC>(CSC{indptr, dense->indices, dense->e_ids}), val};
  }
  std::shared_ptr<COO> AnyToCOO() {
    const bool from_csc = csc_ != nullptr;
    const CSC& g = from_csc ? *csc_ : *csr_;
    const OptTensor& val = from_csc ? val_col_ids_ : val_row_ids_;
    Tensor expanded = ExpandOffsets(g);
    if (val.has_value()) expanded = val.value().index({expanded});
    return from_csc ? std::make_shared<COO>(COO{g.indices, expanded, g.e_ids, false, true})
                    : std::make_shared<COO>(COO{expanded, g.indices, g.e_ids, true, false});
  }
  // DCSCColSlicingCUDA (src/cuda/slicing.cu:298-413): column slice of a doubly compressed form; a requested id
  // without edges is absent from val_ids and yields an empty segment.
  Sliced CompactColSlice(const CSC& g, const Tensor& val_ids, const Tensor& ids, bool with_coo, const OptTensor& data) {
    Tensor n_ids = Ids(ids, "node ids"), val = Ids(val_ids, "valid ids");
    Tensor pos = torch::empty_like(n_ids);
    Check(gsb_index_search(Ctx(), Stream(), IP(val), val.numel(), IP(n_ids), n_ids.numel(), MP(pos)), "gsb_index_search");
    Tensor present = torch::nonzero(pos >= 0).reshape({-1});
    Sliced r = ColSlice(g, pos.index({present}).contiguous(), with_coo, data);
    Tensor counts = torch::zeros({n_ids.numel() + 1}, n_ids.options());
    const int64_t m = r.indptr.numel() - 1;
    counts.index_put_({present + 1}, r.indptr.slice(0, 1, m + 1) - r.indptr.slice(0, 0, m));
    r.indptr = torch::cumsum(counts, 0);
    if (with_coo) r.coo_other = present.index({r.coo_other});
    return r;
  }

  // Slicing (src/graph.cc:173-310)
  c10::intrusive_ptr<Graph> Slicing(Tensor n_ids, int64_t axis, int64_t on_format, int64_t output_format,
                                    bool relabel) {
    CreateSparseFormat(on_format);
    const bool with_coo = output_format & kCOO;
    OptTensor new_col_ids, new_row_ids;
    int64_t new_cols, new_rows, new_edges = 0;
    if (axis == 0) {
      new_col_ids = col_ids_.has_value() ? col_ids_.value().index({n_ids}) : n_ids;
      new_row_ids = row_ids_;
      new_cols = n_ids.numel();
      new_rows = num_rows_;
    } else {
      new_col_ids = col_ids_;
      new_row_ids = row_ids_.has_value() ? row_ids_.value().index({n_ids}) : n_ids;
      new_cols = num_cols_;
      new_rows = n_ids.numel();
    }
    std::shared_ptr<CSC> csc, csr, known_csc, known_csr;
    std::shared_ptr<COO> coo;
    OptTensor new_val_cols, new_val_rows;
    Tensor out_data;
    auto gather = [&](const OptTensor& e_ids, const Tensor& select) {
      if (!data_.has_value()) return;
      Tensor idx = e_ids.has_value() ? Take(e_ids.value(), select) : select;
      out_data = Take(data_.value(), idx);
    };
    if (on_format == kCOO) {
      Tensor nr, nc, sel;
      if (axis == 1) std::tie(nr, nc, sel) = RowSliceCOO(coo_->row, coo_->col, n_ids);
      else std::tie(nc, nr, sel) = RowSliceCOO(coo_->col, coo_->row, n_ids);
      coo = std::make_shared<COO>(COO{nr, nc, torch::nullopt, coo_->row_sorted, coo_->col_sorted});
      new_edges = nr.numel();
      gather(coo_->e_ids, sel);
    } else if (on_format == kCSC || on_format == kCSR || on_format == kDCSC || on_format == kDCSR) {
      const bool on_csc = on_format == kCSC || on_format == kDCSC;
      const OptTensor& val_ids = on_csc ? val_col_ids_ : val_row_ids_;
      TORCH_CHECK(output_format != (on_csc ? kCSR : kCSC), "Error in Slicing, Not implementation [on_format = ",
                  on_csc ? "CSC, output_forat = CSR]" : "CSR, output_forat = CSC]");
      const CSC& g = on_csc ? *csc_ : *csr_;
      const bool slice_segments = (axis == 0) == on_csc;  // slicing along the format's own axis
      Tensor indptr, other, indices;
      if (slice_segments) {
        Sliced r = val_ids.has_value() ? CompactColSlice(g, val_ids.value(), n_ids, with_coo, data_)
                                       : ColSlice(g, n_ids, with_coo, data_);
        indptr = r.indptr, other = r.coo_other, indices = r.indices, out_data = r.data;
        if (relabel) {
          auto res = Relabel({indices}, {indices});
          indices = std::get<1>(res)[0];
          if (on_csc) new_row_ids = std::get<0>(res), new_rows = std::get<0>(res).numel();
          else new_col_ids = std::get<0>(res), new_cols = std::get<0>(res).numel();
        }
      } else {
        TORCH_CHECK(!relabel, "Not implemented warning");
        Tensor sel;
        std::tie(indptr, other, indices, sel) = RowSliceCSC(g, n_ids, with_coo);
        gather(g.e_ids, sel);
        (on_csc ? new_val_cols : new_val_rows) = val_ids;
      }
      if (output_format & (on_csc ? kCSC : kCSR))
        (on_csc ? csc : csr) = std::make_shared<CSC>(CSC{indptr, indices, torch::nullopt});
      else if (!(on_csc ? new_val_cols : new_val_rows).has_value())
        (on_csc ? known_csc : known_csr) = std::make_shared<CSC>(CSC{indptr, indices, torch::nullopt});
      if (with_coo)
        coo = on_csc ? std::make_shared<COO>(COO{indices, other, torch::nullopt, false, true})
                     : std::make_shared<COO>(COO{other, indices, torch::nullopt, true, false});
      new_edges = indices.numel();
    } else {
      TORCH_CHECK(false, "Not implemented warning");
    }
    auto ret = c10::make_intrusive<Graph>(true, new_col_ids, new_row_ids, new_cols, new_rows);
    ret->num_edges_ = new_edges;
    ret->csc_ = csc, ret->csr_ = csr, ret->coo_ = coo;
    // The slice computed these offsets anyway.  The child does not HOLD the format (which formats a graph holds
    // decides, e.g., what Relabel returns), but a later CreateSparseFormat adopts it instead of converting the COO:
    // the arrays are exactly what that conversion would produce from a COO sorted along this axis.
    ret->known_csc_ = known_csc, ret->known_csr_ = known_csr;
    ret->val_col_ids_ = new_val_cols, ret->val_row_ids_ = new_val_rows;
    if (out_data.defined()) ret->data_ = out_data;
    return ret;
  }

  // BatchSlicing (src/graph.cc:312-391): column slice for the seeds of many batches at once.
  std::tuple<c10::intrusive_ptr<Graph>, Tensor> BatchSlicing(Tensor n_ids_in, Tensor nid_ptr_in, int64_t axis,
                                                             int64_t on_format, int64_t output_format, bool relabel,
                                                             bool encoding) {
    TORCH_CHECK(axis == 0, "batch slicing only suppurt column slicing now");
    TORCH_CHECK(on_format == kCSC, "Not Implementatin Error");
    CreateSparseFormat(on_format);
    Tensor n_ids = Ids(n_ids_in, "node ids"), nid_ptr = Ids(nid_ptr_in, "nid_ptr");
    const bool with_coo = output_format & kCOO;
    const int64_t S = n_ids.numel(), G = nid_ptr.numel() - 1;
    OptTensor new_col_ids, new_row_ids = row_ids_;
    if (col_ids_.has_value()) {
      new_col_ids = col_ids_.value().index({n_ids});
    } else {
      Tensor enc = EmptyIds(S, n_ids);
      Check(gsb_batch_encode(Ctx(), Stream(), IP(n_ids), IP(nid_ptr), G, S, num_rows_, MP(enc)), "gsb_batch_encode");
      new_col_ids = enc;
    }
    int64_t new_rows = num_rows_ * G;
    const CSC& g = *csc_;
    Tensor sub_indptr = EmptyIds(S + 1, g.indptr);
    int64_t nnz = 0;
    Check(gsb_col_slice_count(Ctx(), Stream(), IP(g.indptr), g.indptr.numel() - 1, IP(n_ids), S, MP(sub_indptr), &nnz),
          "gsb_col_slice_count");
    Tensor indices = EmptyIds(nnz, g.indptr), select = EmptyIds(nnz, g.indptr), offsets = EmptyIds(G + 1, g.indptr);
    Tensor coo_col = with_coo ? EmptyIds(nnz, g.indptr) : Tensor();
    Tensor out_data;
    const float* data_in = nullptr;
    float* data_out = nullptr;
    if (data_.has_value()) {
      out_data = torch::empty({nnz}, OnDevice(data_.value()));
      data_in = FP(data_.value());
      data_out = nnz ? out_data.data_ptr<float>() : nullptr;
    }
    Tensor eids = g.e_ids.value_or(Tensor());
    Check(gsb_batch_col_slice_fill(Ctx(), Stream(), IP(g.indptr), IP(g.indices), g.indptr.numel() - 1, IP(n_ids), S,
                                   IP(nid_ptr), G,
                                   encoding ? num_rows_ : 0, IP(sub_indptr), MP(indices), MP(select), MP(coo_col),
                                   MP(offsets), data_in, IP(eids), data_out),
          "gsb_batch_col_slice_fill");
    if (relabel) {
      auto res = Relabel({indices}, {indices});
      indices = std::get<1>(res)[0];
      new_row_ids = std::get<0>(res);
      new_rows = std::get<0>(res).numel();
    }
    auto ret = c10::make_intrusive<Graph>(true, new_col_ids, new_row_ids, S, new_rows);
    ret->num_edges_ = nnz;
    if (output_format & kCSC) ret->csc_ = std::make_shared<CSC>(CSC{sub_indptr, indices, torch::nullopt});
    if (with_coo) ret->coo_ = std::make_shared<COO>(COO{indices, coo_col, torch::nullopt, false, true});
    if (out_data.defined()) ret->data_ = out_data;
    return {ret, offsets};
  }

  // FusedBidirSlicing / BatchFusedBidirSlicing (src/graph.cc:116-170): seed columns x listed rows in one pass.
  c10::intrusive_ptr<Graph> ColRowSliceImpl(Tensor column_seeds, const Tensor* col_ptr, Tensor row_seeds,
                                            const Tensor* row_ptr) {
    CreateSparseFormat(kCSC);
    const bool batched = col_ptr != nullptr;
    Tensor cs = Ids(column_seeds, "column seeds"), rs = Ids(row_seeds, "row seeds");
    Tensor col_ids = col_ids_.has_value() ? col_ids_.value().index({cs}) : cs;
    Tensor row_ids = batched ? rs : (row_ids_.has_value() ? row_ids_.value().index({rs}) : rs);
    Tensor cp = batched ? Ids(*col_ptr, "col_ptr") : Tensor(), rp = batched ? Ids(*row_ptr, "row_ptr") : Tensor();
    if (batched) TORCH_CHECK(cp.numel() == rp.numel(), "col_ptr and row_ptr must have the same length");
    const CSC& g = *csc_;
    const int64_t S = col_ids.numel(), R = row_ids.numel(), G = batched ? cp.numel() - 1 : 1;
    Tensor slice_indptr = EmptyIds(S + 1, g.indptr), sub_indptr = EmptyIds(S + 1, g.indptr);
    int64_t D = 0, nnz = 0;
    Check(gsb_col_slice_count(Ctx(), Stream(), IP(g.indptr), g.indptr.numel() - 1, IP(col_ids), S, MP(slice_indptr), &D),
          "gsb_col_slice_count");
    Tensor indices = EmptyIds(D, g.indptr), select = EmptyIds(D, g.indptr), out_data;
    const float* data_in = nullptr;
    float* data_out = nullptr;
    if (data_.has_value()) {
      out_data = torch::empty({D}, OnDevice(data_.value()));
      data_in = FP(data_.value());
      data_out = D ? out_data.data_ptr<float>() : nullptr;
    }
    Tensor eids = g.e_ids.value_or(Tensor());
    Check(gsb_col_row_slice(Ctx(), Stream(), IP(g.indptr), IP(g.indices), g.indptr.numel() - 1, IP(col_ids), S,
                            IP(slice_indptr), D,
                            IP(row_ids), R, IP(cp), IP(rp), G, num_rows_, batched ? 0 : 1, MP(sub_indptr), MP(indices),
                            MP(select), data_in, IP(eids), data_out, &nnz),
          "gsb_col_row_slice");
    indices = indices.narrow(0, 0, nnz);
    if (out_data.defined()) out_data = out_data.narrow(0, 0, nnz);
    auto ret = batched ? c10::make_intrusive<Graph>(true, col_ids, row_ids_, S, num_rows_)
                       : c10::make_intrusive<Graph>(true, col_ids, row_ids, S, R);
    ret->csc_ = std::make_shared<CSC>(CSC{sub_indptr, indices, torch::nullopt});
    ret->num_edges_ = nnz;
    if (out_data.defined()) ret->data_ = out_data;
    return ret;
  }
  c10::intrusive_ptr<Graph> FusedBidirSlicing(Tensor column_seeds, Tensor row_seeds) {
    return ColRowSliceImpl(column_seeds, nullptr, row_seeds, nullptr);
  }
  c10::intrusive_ptr<Graph> BatchFusedBidirSlicing(Tensor column_seeds, Tensor col_ptr, Tensor row_seeds,
                                                   Tensor row_ptr) {
    return ColRowSliceImpl(column_seeds, &col_ptr, row_seeds, &row_ptr);
  }

  // EDivUSum (src/graph.cc:732-755): data / divisor[row] and the per-column sums of the quotient.
  std::tuple<c10::intrusive_ptr<Graph>, Tensor> EDivUSum(Tensor divisor_in) {
    CreateSparseFormat(kCOO);
    Tensor divisor = Floats(divisor_in, "divisor");
    Tensor in = data_.has_value() ? data_.value() : Tensor();
    if (in.defined() && coo_->e_ids.has_value()) in = in.index({coo_->e_ids.value()});
    if (in.defined()) in = Floats(in, "edge data");
    Tensor out = torch::empty({num_edges_}, divisor.options());
    Tensor out_sum = torch::zeros({num_cols_}, divisor.options());
    Check(gsb_edge_div_u_sum(Ctx(), Stream(), IP(coo_->row), IP(coo_->col), num_edges_, FP(in), FP(divisor),
                             num_edges_ ? out.data_ptr<float>() : nullptr, num_cols_ ? out_sum.data_ptr<float>() : nullptr),
          "gsb_edge_div_u_sum");
    if (coo_->e_ids.has_value()) {
      Tensor full = torch::empty_like(out);
      full.index_put_({coo_->e_ids.value()}, out);
      out = full;
    }
    return {SameStructure(out), out_sum};
  }

  // Split (src/graph.cc:987-1017): consecutive chunks of split_size columns as separate graphs.
  std::vector<c10::intrusive_ptr<Graph>> Split(int64_t split_size) {
    CreateSparseFormat(kCSC);
    TORCH_CHECK(split_size > 0, "split_size must be positive");
    const int64_t n = csc_->indptr.numel() - 1;
    std::vector<int64_t> bounds;
    for (int64_t c = 0; c < n; c += split_size) bounds.push_back(c);
    bounds.push_back(n);
    const int64_t parts = (int64_t)bounds.size() - 1;
    Tensor offsets = torch::tensor(bounds, torch::dtype(torch::kInt64)).to(Device());
    Tensor out = EmptyIds(n + parts, csc_->indptr);
    Check(gsb_split_indptr(Ctx(), Stream(), IP(csc_->indptr), IP(offsets), parts, 0, MP(out)), "gsb_split_indptr");
    Tensor edge_bounds = csc_->indptr.index({offsets}).to(torch::kCPU);
    const int64_t* eb = edge_bounds.data_ptr<int64_t>();
    std::vector<c10::intrusive_ptr<Graph>> ret;
    for (int64_t i = 0; i < parts; ++i) {
      const int64_t cols = bounds[i + 1] - bounds[i];
      Tensor indptr = out.narrow(0, bounds[i] + i, cols + 1);
      Tensor indices = csc_->indices.narrow(0, eb[i], eb[i + 1] - eb[i]);
      OptTensor e_ids;
      if (csc_->e_ids.has_value()) e_ids = csc_->e_ids.value().narrow(0, eb[i], eb[i + 1] - eb[i]);
      OptTensor nid;
      if (col_ids_.has_value()) nid = col_ids_.value().narrow(0, bounds[i], cols);
      auto g = c10::make_intrusive<Graph>(true, nid, row_ids_, cols, num_rows_);
      g->csc_ = std::make_shared<CSC>(CSC{indptr, indices, e_ids});
      g->num_edges_ = indices.numel();
      ret.push_back(g);
    }
    return ret;
  }

  // Decode: strips the batch encoding from both id maps.  (The reference aborts whenever an id map is present and
  // dereferences it when it is absent, src/graph.cc:1035-1040; this does what the name says.)
  void Decode(int64_t encoding_size) {
    TORCH_CHECK(col_ids_.has_value() && row_ids_.has_value(), "Error: Decoding should have both row and column id");
    Tensor c = Ids(col_ids_.value(), "col ids"), r = Ids(row_ids_.value(), "row ids");
    Tensor oc = torch::empty_like(c), orow = torch::empty_like(r);
    Check(gsb_batch_decode(Ctx(), Stream(), IP(c), c.numel(), encoding_size, MP(oc)), "gsb_batch_decode");
    Check(gsb_batch_decode(Ctx(), Stream(), IP(r), r.numel(), encoding_size, MP(orow)), "gsb_batch_decode");
    col_ids_ = oc, row_ids_ = orow;
  }

  const CSC& CscForWalk() {
    CreateSparseFormat(kCSC);
    return *csc_;
  }

  // Sampling / SamplingProbs (src/graph.cc:393-529)
  c10::intrusive_ptr<Graph> SampleImpl(int64_t axis, const Tensor* probs, int64_t fanout, bool replace,
                                       int64_t on_format, int64_t output_format) {
    CreateSparseFormat(on_format);
    const bool with_coo = output_format & kCOO;
    const bool on_csc = axis == 0 && on_format == kCSC;
    TORCH_CHECK(on_csc || (axis == 1 && on_format == kCSR), "No implementation!");
    TORCH_CHECK(output_format != (on_csc ? kCSR : kCSC), "Error in Sampling, Not implementation [on_format / output_format]");
    const CSC& g = on_csc ? *csc_ : *csr_;
    Sliced r = Sample(g, nullptr, fanout, replace, with_coo, probs, data_);
    auto ret = c10::make_intrusive<Graph>(true, col_ids_, row_ids_, num_cols_, num_rows_);
    if (output_format & (on_csc ? kCSC : kCSR))
      (on_csc ? ret->csc_ : ret->csr_) = std::make_shared<CSC>(CSC{r.indptr, r.indices, torch::nullopt});
    if (with_coo)
      ret->coo_ = on_csc ? std::make_shared<COO>(COO{r.indices, r.coo_other, torch::nullopt, false, true})
                         : std::make_shared<COO>(COO{r.coo_other, r.indices, torch::nullopt, true, false});
    ret->num_edges_ = r.indices.numel();
    if (r.data.defined()) ret->data_ = r.data;
    return ret;
  }
  c10::intrusive_ptr<Graph> Sampling(int64_t axis, int64_t fanout, bool replace, int64_t on_format,
                                     int64_t output_format) {
    return SampleImpl(axis, nullptr, fanout, replace, on_format, output_format);
  }
  c10::intrusive_ptr<Graph> SamplingProbs(int64_t axis, Tensor edge_probs, int64_t fanout, bool replace,
                                          int64_t on_format, int64_t output_format) {
    return SampleImpl(axis, &edge_probs, fanout, replace, on_format, output_format);
  }

  // src/graph.cc:531-559 (keep-dim variant chosen like src/graph_ops.cc:223-247)
  c10::intrusive_ptr<Graph> ColumnwiseFusedSlicingAndSampling(Tensor column_index, int64_t fanout, bool replace) {
    TORCH_CHECK(csc_ != nullptr, "ColumnwiseFusedSlicingAndSampling needs a CSC graph");
    Tensor col_ids = col_ids_.has_value() ? col_ids_.value().index({column_index}) : column_index;
    auto ret = c10::make_intrusive<Graph>(true, col_ids, row_ids_, col_ids.numel(), num_rows_);
    if (fanout == 1 && replace) {
      Tensor seeds = Ids(column_index, "column ids");
      const int64_t S = seeds.numel();
      Tensor indptr = EmptyIds(S + 1, seeds), indices = EmptyIds(S, seeds), select = EmptyIds(S, seeds);
      Check(gsb_sample_one_keepdim(Ctx(), Stream(), IP(csc_->indptr), IP(csc_->indices), csc_->indptr.numel() - 1,
                                   IP(seeds), S, NextSeed(),
                                   MP(indptr), MP(indices), MP(select)),
            "gsb_sample_one_keepdim");
      ret->csc_ = std::make_shared<CSC>(CSC{indptr, indices, torch::nullopt});
      ret->num_edges_ = S;
      if (data_.has_value()) {
        Tensor safe = select.clamp_min(0);
        ret->data_ = Take(data_.value(), csc_->e_ids.has_value() ? Take(csc_->e_ids.value(), safe) : safe);
      }
      return ret;
    }
    Sliced r = Sample(*csc_, &column_index, fanout, replace, false, nullptr, data_);
    ret->csc_ = std::make_shared<CSC>(CSC{r.indptr, r.indices, torch::nullopt});
    ret->num_edges_ = r.indices.numel();
    if (r.data.defined()) ret->data_ = r.data;
    return ret;
  }

  // src/graph.cc:757-839
  Tensor AllValidNode() {
    TORCH_CHECK(col_ids_.has_value(), "For sampling, col_ids_ is necessary!");
    Tensor rows;
    if (csc_) rows = row_ids_.has_value() ? row_ids_.value() : csc_->indices;
    else {
      if (!coo_) coo_ = AnyToCOO();
      rows = row_ids_.has_value() ? row_ids_.value() : coo_->row;
    }
    return std::get<0>(Relabel({col_ids_.value(), rows}, {}));
  }
  std::tuple<Tensor, int64_t, int64_t, Tensor, Tensor, OptTensor, std::string> Relabel_() {
    TORCH_CHECK(col_ids_.has_value(), "For sampling, col_ids_ is necessary!");
    Tensor col_ids = col_ids_.value();
    if (csc_) {
      if (val_col_ids_.has_value()) col_ids = col_ids.index({val_col_ids_.value()});  // src/graph.cc:790-791
      Tensor rows = row_ids_.has_value() ? row_ids_.value().index({csc_->indices}) : csc_->indices;
      auto res = Relabel({col_ids, rows}, {rows});
      Tensor frontier = std::get<0>(res);
      return {frontier, frontier.numel(), col_ids.numel(), csc_->indptr.clone(), std::get<1>(res)[0], csc_->e_ids, "csc"};
    }
    TORCH_CHECK(csr_ || coo_, "Error in Relabel!");
    if (!coo_) coo_ = AnyToCOO();
    Tensor coo_col = col_ids.index({coo_->col});
    Tensor coo_row = row_ids_.has_value() ? row_ids_.value().index({coo_->row}) : coo_->row;
    auto res = Relabel({col_ids, coo_row}, {coo_col, coo_row});
    Tensor frontier = std::get<0>(res);
    return {frontier, frontier.numel(), col_ids.numel(), std::get<1>(res)[1], std::get<1>(res)[0], coo_->e_ids, "coo"};
  }

  // src/graph.cc:646-648: the reference's step-major memory viewed as [seeds, length + 1]
  Tensor RandomWalk(Tensor seeds, int64_t walk_length) {
    TORCH_CHECK(csc_ != nullptr, "RandomWalk needs a CSC graph");
    Tensor s = Ids(seeds, "seeds");
    Tensor out = EmptyIds(s.numel() * (walk_length + 1), s);
    Check(gsb_random_walk(Ctx(), Stream(), IP(csc_->indptr), IP(csc_->indices), csc_->indptr.numel() - 1, IP(s),
                          s.numel(), walk_length,
                          NextSeed(), 0, 0, MP(out)),
          "gsb_random_walk");
    return out.reshape({s.numel(), walk_length + 1});
  }

  // src/graph.cc:967-985
  void SDDMM(const std::string& op, Tensor lhs, Tensor rhs, Tensor out, int64_t lhs_target, int64_t rhs_target,
             int64_t on_format) {
    CreateSparseFormat(on_format);
    if (on_format == kDCSC || on_format == kDCSR) {
      // a compact form numbers its segments by position in val_*_ids_; the COO view has the node ids again and
      // carries the same edge ids, so the result lands in the same order
      CreateSparseFormat(kCOO);
      on_format = kCOO;
    }
    if (on_format == kCOO) {
      Sddmm(op, coo_->row, &coo_->col, nullptr, coo_->e_ids, lhs, rhs, out, lhs_target, rhs_target);
    } else if (on_format == kCSR) {
      const int64_t lt = lhs_target == 1 ? 1 : 2 - lhs_target, rt = rhs_target == 1 ? 1 : 2 - rhs_target;
      Sddmm(op, csr_->indices, nullptr, &csr_->indptr, csr_->e_ids, lhs, rhs, out, lt, rt);
    } else if (on_format == kCSC) {
      Sddmm(op, csc_->indices, nullptr, &csc_->indptr, csc_->e_ids, lhs, rhs, out, lhs_target, rhs_target);
    } else {
      TORCH_CHECK(false, "SDDMM only supports CSR and COO formats");
    }
  }

  // src/graph.cc:650-730
  Tensor Sum(int64_t axis, int64_t powk, int64_t on_format) {
    CreateSparseFormat(on_format);
    Tensor data;
    if (data_.has_value()) data = Floats(data_.value(), "edge data");
    Tensor out = torch::zeros({axis == 0 ? num_cols_ : num_rows_},
                              torch::dtype(torch::kFloat32).device(Device()));
    float* o = out.numel() ? out.data_ptr<float>() : nullptr;
    if (on_format == kCOO) {
      const bool by_row = (1 - axis) == 0;
      const Tensor& target = by_row ? coo_->row : coo_->col;
      Tensor e = coo_->e_ids.has_value() ? coo_->e_ids.value() : Tensor();
      Check(gsb_segment_sum_coo(Ctx(), Stream(), IP(target), target.numel(), IP(e), FP(data), powk,
                                (by_row ? coo_->row_sorted : coo_->col_sorted) ? 1 : 0, o),
            "gsb_segment_sum_coo");
    } else if ((axis == 0 && (on_format == kCSC || on_format == kDCSC)) ||
               (axis == 1 && (on_format == kCSR || on_format == kDCSR))) {
      const CSC& g = axis == 0 ? *csc_ : *csr_;
      const OptTensor& val = axis == 0 ? val_col_ids_ : val_row_ids_;
      Tensor e = g.e_ids.has_value() ? g.e_ids.value() : Tensor();
      if (!val.has_value()) {
        Check(gsb_segment_sum_csc(Ctx(), Stream(), IP(g.indptr), g.indptr.numel() - 1, IP(e), FP(data), powk, o),
              "gsb_segment_sum_csc");
      } else {  // segment c of a compact form belongs to node val[c] (src/cuda/graph_ops.cu:15-39)
        Tensor compact = torch::zeros({val.value().numel()}, out.options());
        Check(gsb_segment_sum_csc(Ctx(), Stream(), IP(g.indptr), g.indptr.numel() - 1, IP(e), FP(data), powk,
                                  compact.numel() ? compact.data_ptr<float>() : nullptr),
              "gsb_segment_sum_csc");
        out.index_put_({val.value()}, compact);
      }
    } else {
      TORCH_CHECK(false, "axis should be 0 or 1? on_format and axis do not match?");
    }
    return out;
  }
  c10::intrusive_ptr<Graph> Normalize(int64_t axis, int64_t on_format) {
    CreateSparseFormat(on_format);
    TORCH_CHECK((axis == 0 && (on_format == kCSC || on_format == kDCSC)) ||
                    (axis == 1 && (on_format == kCSR || on_format == kDCSR)),
                "Not Implementation Error");
    const CSC& g = axis == 0 ? *csc_ : *csr_;
    Tensor in = Floats(DataOrOnes(), "edge data");
    Tensor out = torch::empty_like(in);
    Tensor e = g.e_ids.has_value() ? g.e_ids.value() : Tensor();
    Check(gsb_segment_normalize_csc(Ctx(), Stream(), IP(g.indptr), g.indptr.numel() - 1, IP(e), FP(in),
                                    out.numel() ? out.data_ptr<float>() : nullptr),
          "gsb_segment_normalize_csc");
    return SameStructure(out);
  }
  c10::intrusive_ptr<Graph> Divide(Tensor divisor, int64_t axis, int64_t on_format) {
    CreateSparseFormat(on_format);
    Tensor in = DataOrOnes();
    Tensor out = torch::zeros({num_edges_}, in.options());
    if (on_format == kCOO) {
      Sddmm("div", coo_->row, &coo_->col, nullptr, coo_->e_ids, in, divisor, out, 1, (1 - axis) == 0 ? 0 : 2);
    } else if ((axis == 0 && (on_format == kCSC || on_format == kDCSC)) ||
               (axis == 1 && (on_format == kCSR || on_format == kDCSR))) {
      const CSC& g = axis == 0 ? *csc_ : *csr_;
      const OptTensor& val = axis == 0 ? val_col_ids_ : val_row_ids_;
      Tensor per_segment = val.has_value() ? divisor.index({val.value()}).contiguous() : divisor;
      Sddmm("div", g.indices, nullptr, &g.indptr, g.e_ids, in, per_segment, out, 1, 2);
    }
    return SameStructure(out);
  }

  // getters (src/graph.cc:841-965)
  Tensor GetRows() {
    return row_ids_.has_value() ? row_ids_.value() : torch::arange(num_rows_, torch::dtype(torch::kInt64).device(Device()));
  }
  Tensor GetCols() {
    return col_ids_.has_value() ? col_ids_.value() : torch::arange(num_cols_, torch::dtype(torch::kInt64).device(Device()));
  }
  Tensor GetCOORows(bool is_original) {
    Tensor rows;
    if (coo_) rows = coo_->row;
    else if (csc_ && !csc_->e_ids.has_value()) rows = csc_->indices;
    else {
      TORCH_CHECK(csr_ && !csr_->e_ids.has_value(), "Error in GetCOORows!");
      coo_ = AnyToCOO();
      rows = coo_->row;
    }
    return (is_original && row_ids_.has_value()) ? row_ids_.value().index({rows}) : rows;
  }
  Tensor GetCOOCols(bool is_original) {
    Tensor cols;
    if (coo_) cols = coo_->col;
    else if (csc_ && !csc_->e_ids.has_value()) {
      coo_ = AnyToCOO();
      cols = coo_->col;
    } else {
      TORCH_CHECK(csr_ && !csr_->e_ids.has_value(), "Error in GetCOOCols!");
      cols = csr_->indices;
    }
    return (is_original && col_ids_.has_value()) ? col_ids_.value().index({cols}) : cols;
  }
  Tensor GetValidRows() {
    Tensor local = val_row_ids_.has_value() ? val_row_ids_.value() : std::get<0>(torch::_unique(GetCOORows(false)));
    return row_ids_.has_value() ? row_ids_.value().index({local}) : local;
  }
  Tensor GetValidCols() {
    Tensor local = val_col_ids_.has_value() ? val_col_ids_.value() : std::get<0>(torch::_unique(GetCOOCols(false)));
    return col_ids_.has_value() ? col_ids_.value().index({local}) : local;
  }
  std::vector<Tensor> MetaData() {
    Tensor c = col_ids_.value_or(Tensor()), r = row_ids_.value_or(Tensor());
    if (csc_) return {c, r, DataOrOnes(), csc_->indptr, csc_->indices};
    if (csr_) return {c, r, DataOrOnes(), csr_->indptr, csr_->indices};
    return {coo_->row, coo_->col};
  }
  std::vector<Tensor> COOMetaData() {
    if (!coo_) return {};
    return {col_ids_.value_or(Tensor()), row_ids_.value_or(Tensor()), data_.value_or(Tensor()), coo_->row, coo_->col};
  }
  std::vector<Tensor> CSCMetaData() {
    if (!csc_) return {};
    return {col_ids_.value_or(Tensor()), row_ids_.value_or(Tensor()), data_.value_or(Tensor()), csc_->indptr, csc_->indices};
  }
  std::vector<Tensor> GetCSCTensor() {
    CreateSparseFormat(kCSC);
    return {csc_->indptr, csc_->indices, csc_->e_ids.value_or(Tensor())};
  }
  std::vector<Tensor> GetCOOTensor() {
    CreateSparseFormat(kCOO);
    TORCH_CHECK(coo_->col_sorted, "Check failed: coo_->col_sorted == true");
    return {coo_->row, coo_->col, coo_->e_ids.value_or(Tensor())};
  }

 private:
  torch::Device Device() const {
    if (csc_) return DeviceOf(csc_->indptr);
    if (csr_) return DeviceOf(csr_->indptr);
    return DeviceOf(coo_->row);
  }
  Tensor DataOrOnes() {
    return data_.has_value() ? data_.value()
                             : torch::ones({num_edges_}, torch::dtype(torch::kFloat32).device(Device()));
  }
  static std::shared_ptr<COO> ToCOO(const CSC& g, bool is_csc) {
    Tensor expanded = ExpandOffsets(g);
    return is_csc ? std::make_shared<COO>(COO{g.indices, expanded, g.e_ids, false, true})
                  : std::make_shared<COO>(COO{expanded, g.indices, g.e_ids, true, false});
  }
  static std::shared_ptr<CSC> FromCOO(const COO& c, int64_t num_items, bool to_csc) {
    Tensor indptr, indices;
    OptTensor perm;
    if (to_csc) std::tie(indptr, indices, perm) = SortByKey(c.col, c.row, num_items, c.col_sorted);
    else std::tie(indptr, indices, perm) = SortByKey(c.row, c.col, num_items, c.row_sorted);
    OptTensor e_ids = perm;
    if (c.e_ids.has_value()) e_ids = perm.has_value() ? c.e_ids.value().index({perm.value()}) : c.e_ids.value();
    return std::make_shared<CSC>(CSC{indptr, indices, e_ids});
  }
  c10::intrusive_ptr<Graph> SameStructure(Tensor data) {
    auto ret = c10::make_intrusive<Graph>(is_subgraph_, col_ids_, row_ids_, num_cols_, num_rows_);
    ret->csc_ = csc_, ret->csr_ = csr_, ret->coo_ = coo_;
    ret->num_edges_ = num_edges_;
    ret->data_ = data;
    ret->val_col_ids_ = val_col_ids_, ret->val_row_ids_ = val_row_ids_;
    return ret;
  }

  bool is_subgraph_ = false;
  int64_t num_cols_ = 0, num_rows_ = 0, num_edges_ = 0;
  std::shared_ptr<CSC> csc_, csr_;
  std::shared_ptr<CSC> known_csc_, known_csr_;  // offsets a slice computed but the graph does not hold (see Slicing)
  std::shared_ptr<COO> coo_;
  OptTensor data_, col_ids_, row_ids_;
  OptTensor val_col_ids_, val_row_ids_;  // ids that have edges, when csc_ / csr_ is doubly compressed (DCSC / DCSR)
};

// ---- HeteroGraph (src/hetero_graph.h:38-70, src/hetero_graph.cc:20-75) ----------------------------------------
class HeteroGraph : public torch::CustomClassHolder {
 public:
  HeteroGraph() {}
  void LoadFromHomo(const std::vector<std::string>& node_types,
                    const std::vector<std::tuple<std::string, std::string, std::string>>& edge_types,
                    const std::vector<c10::intrusive_ptr<Graph>>& edge_relations) {
    TORCH_CHECK(edge_types.size() == edge_relations.size(), "edge_types and edge_relations differ in length");
    TORCH_CHECK(edge_relations.size() <= GSB_MAX_RELATIONS, "at most ", GSB_MAX_RELATIONS, " relations");
    node_type_.clear(), edge_type_.clear(), relations_.clear();
    for (size_t i = 0; i < node_types.size(); ++i) node_type_[node_types[i]] = (int64_t)i;
    for (size_t i = 0; i < edge_types.size(); ++i) {
      edge_type_[std::get<1>(edge_types[i])] = (int64_t)i;
      relations_.push_back(edge_relations[i]);
    }
  }
  c10::intrusive_ptr<Graph> GetHomoGraph(const std::string& edge_type) const {
    auto it = edge_type_.find(edge_type);
    TORCH_CHECK(it != edge_type_.end(), "unknown edge type ", edge_type);
    return relations_[it->second];
  }
  Tensor MetapathRandomWalkFused(Tensor seeds, const std::vector<std::string>& metapath) {
    Tensor s = Ids(seeds, "seeds");
    const int64_t L = (int64_t)metapath.size();
    TORCH_CHECK(L <= GSB_MAX_METAPATH, "metapath longer than ", GSB_MAX_METAPATH);
    std::vector<int64_t> path;
    for (const auto& name : metapath) {
      auto it = edge_type_.find(name);
      TORCH_CHECK(it != edge_type_.end(), "unknown edge type ", name);
      path.push_back(it->second);
    }
    const int64_t* ip[GSB_MAX_RELATIONS];
    const int64_t* ix[GSB_MAX_RELATIONS];
    int64_t nn[GSB_MAX_RELATIONS];
    for (size_t i = 0; i < relations_.size(); ++i) {
      const CSC& g = relations_[i]->CscForWalk();
      ip[i] = IP(g.indptr), ix[i] = IP(g.indices), nn[i] = g.indptr.numel() - 1;
    }
    Tensor out = EmptyIds(s.numel() * (L + 1), s);
    Check(gsb_metapath_random_walk(Ctx(), Stream(), ip, ix, nn, (int)relations_.size(), path.data(), L, IP(s), s.numel(),
                                   NextSeed(), 0, 0, MP(out)),
          "gsb_metapath_random_walk");
    return out.reshape({s.numel(), L + 1});
  }

 private:
  std::map<std::string, int64_t> node_type_, edge_type_;
  std::vector<c10::intrusive_ptr<Graph>> relations_;
};

// ---- free operators (src/tensor_ops.cc:5-16, src/pybind.cc:62-85) ---------------------------------------------------
static std::tuple<Tensor, Tensor> ListSampleImpl(const Tensor& data_in, const Tensor* probs, int64_t k, bool replace) {
  Tensor data = Ids(data_in, "data"), p;
  if (probs) {
    p = Floats(*probs, "probs");
    TORCH_CHECK(p.numel() == data.numel(), "probs must have one entry per item");
  }
  const int64_t N = data.numel();
  const int64_t cap = std::max<int64_t>((!replace && N <= k) ? N : k, 1);
  Tensor out_d = EmptyIds(cap, data), out_i = EmptyIds(cap, data);
  int64_t n = 0;
  Check(gsb_list_sample(Ctx(), Stream(), IP(data), FP(p), N, k, replace, NextSeed(), MP(out_d), MP(out_i), &n),
        "gsb_list_sample");
  return {out_d.narrow(0, 0, n), out_i.narrow(0, 0, n)};
}
static std::tuple<Tensor, Tensor> ListSampling(Tensor data, int64_t num_picks, bool replace) {
  return ListSampleImpl(data, nullptr, num_picks, replace);
}
static std::tuple<Tensor, Tensor> ListSamplingProbs(Tensor data, Tensor probs, int64_t num_picks, bool replace) {
  return ListSampleImpl(data, &probs, num_picks, replace);
}
static Tensor Unique(Tensor node_ids) { return std::get<0>(Relabel({node_ids}, {})); }
static std::tuple<Tensor, Tensor, Tensor, Tensor> BatchCSRRelabel(Tensor seeds, Tensor seeds_ptr, Tensor indices,
                                                                  Tensor indices_ptr) {
  Tensor s = Ids(seeds, "seeds"), sp = Ids(seeds_ptr, "seeds_ptr"), ix = Ids(indices, "indices"),
         ixp = Ids(indices_ptr, "indices_ptr");
  const int64_t G = sp.numel() - 1;
  Tensor uniq = EmptyIds(s.numel() + ix.numel(), s), uniq_ptr = EmptyIds(G + 1, s), rel = EmptyIds(ix.numel(), s);
  int64_t nu = 0, ne = 0;
  // The operator's signature carries no id bound (src/tensor_ops.h), so the largest node count of the graphs loaded
  // so far serves as a hint: with it first occurrences are found in direct-address tables.  If an id turns out to
  // lie outside the hint, the device reports GSB_ERR_INDEX_RANGE and the call is redone with hash tables.
  const int64_t hint = g_node_bound.load();
  int st = gsb_batch_unique_relabel(Ctx(), Stream(), IP(s), IP(sp), s.numel(), IP(ix), IP(ixp), ix.numel(), G, hint, 0,
                                    MP(uniq), MP(uniq_ptr), MP(rel), &nu, &ne);
  if (hint > 0 && (st == GSB_ERR_INDEX_RANGE || st == GSB_ERR_OUT_OF_MEMORY))
    st = gsb_batch_unique_relabel(Ctx(), Stream(), IP(s), IP(sp), s.numel(), IP(ix), IP(ixp), ix.numel(), G, 0, 0,
                                  MP(uniq), MP(uniq_ptr), MP(rel), &nu, &ne);
  Check(st, "gsb_batch_unique_relabel");
  return {uniq.narrow(0, 0, nu), uniq_ptr, rel.narrow(0, 0, ne), ixp};
}
static std::vector<Tensor> SplitByOffset(Tensor data, Tensor offset) {  // src/tensor_ops.cc:33-45
  Tensor sizes = (offset.slice(0, 1, offset.numel()) - offset.slice(0, 0, offset.numel() - 1)).to(torch::kCPU);
  std::vector<int64_t> split(sizes.data_ptr<int64_t>(), sizes.data_ptr<int64_t>() + sizes.numel());
  return torch::split_with_sizes(data, split);
}
static std::vector<Tensor> IndptrSplitByOffset(Tensor indptr_in, Tensor offsets_in) {  // src/cuda/batch_split.cu:66-97
  Tensor indptr = Ids(indptr_in, "indptr"), offsets = Ids(offsets_in, "offsets");
  const int64_t G = offsets.numel() - 1;
  Tensor host = offsets.to(torch::kCPU);
  const int64_t* h = host.data_ptr<int64_t>();
  TORCH_CHECK(G >= 0 && (G == 0 || h[0] == 0), "offsets must start at 0");
  Tensor out = EmptyIds(G ? h[G] + G : 0, indptr);
  Check(gsb_split_indptr(Ctx(), Stream(), IP(indptr), IP(offsets), G, 0, MP(out)), "gsb_split_indptr");
  std::vector<int64_t> split;
  for (int64_t b = 0; b < G; ++b) split.push_back(h[b + 1] - h[b] + 1);
  return torch::split_with_sizes(out, split);
}
static std::vector<Tensor> IndptrSplitBySize(Tensor indptr_in, int64_t size) {  // src/cuda/batch_split.cu:11-48
  Tensor indptr = Ids(indptr_in, "indptr");
  const int64_t G = (indptr.numel() - 1) / size;
  Tensor out = EmptyIds(G * (size + 1), indptr);
  Check(gsb_split_indptr(Ctx(), Stream(), IP(indptr), nullptr, G, size, MP(out)), "gsb_split_indptr");
  return torch::split(out, size + 1);
}
// ---- the rest of the super-batch family (src/pybind.cc:65-84) ---------------------------------------------------
static Tensor BatchEncode(Tensor data_in, Tensor ptr_in, int64_t encoding_size) {
  Tensor data = Ids(data_in, "data"), ptr = Ids(ptr_in, "data_ptr");
  Tensor out = torch::empty_like(data);
  Check(gsb_batch_encode(Ctx(), Stream(), IP(data), IP(ptr), ptr.numel() - 1, data.numel(), encoding_size, MP(out)),
        "gsb_batch_encode");
  return out;
}
static Tensor BatchDecode(Tensor data_in, int64_t encoding_size) {
  Tensor data = Ids(data_in, "data");
  Tensor out = torch::empty_like(data);
  Check(gsb_batch_decode(Ctx(), Stream(), IP(data), data.numel(), encoding_size, MP(out)), "gsb_batch_decode");
  return out;
}
static std::tuple<Tensor, Tensor> GetBatchOffsets(Tensor data_in, int64_t num_batches, int64_t encoding_size) {
  Tensor data = Ids(data_in, "data");
  Tensor ptr = EmptyIds(num_batches + 1, data), dec = torch::empty_like(data);
  Check(gsb_get_batch_offsets(Ctx(), Stream(), IP(data), data.numel(), num_batches, encoding_size, MP(ptr), MP(dec)),
        "gsb_get_batch_offsets");
  return {ptr, dec};
}
static std::tuple<Tensor, Tensor, Tensor> BatchUniqueImpl(Tensor data_in, Tensor ptr_in, bool sorted) {
  Tensor data = Ids(data_in, "data"), ptr = Ids(ptr_in, "data_ptr");
  const int64_t n = data.numel(), G = ptr.numel() - 1;
  Tensor uniq = EmptyIds(n, data), key = EmptyIds(n, data), uptr = EmptyIds(G + 1, data);
  int64_t nu = 0;
  Check(gsb_batch_unique(Ctx(), Stream(), IP(data), IP(ptr), n, G, sorted ? 1 : 0, MP(uniq), MP(uptr), MP(key), &nu),
        "gsb_batch_unique");
  return {uniq.narrow(0, 0, nu), uptr, key.narrow(0, 0, nu)};
}
static std::tuple<Tensor, Tensor, Tensor> BatchUnique(Tensor data, Tensor ptr) { return BatchUniqueImpl(data, ptr, false); }
static std::tuple<Tensor, Tensor, Tensor> BatchUnique2(Tensor data, Tensor ptr) { return BatchUniqueImpl(data, ptr, true); }
// The ...ByKey forms take the batch number of every item as well; it is implied by the offset arrays (the
// reference derives one from the other with _RepeatKernel, src/cuda/batch_unique.cu:184-206), so it is not read.
static std::tuple<Tensor, Tensor, Tensor> BatchUniqueByKey(Tensor data, Tensor ptr, Tensor) {
  return BatchUniqueImpl(data, ptr, false);
}
static std::tuple<Tensor, Tensor, Tensor> BatchUniqueByKey2(Tensor data, Tensor ptr, Tensor) {
  return BatchUniqueImpl(data, ptr, true);
}
static std::tuple<Tensor, Tensor, Tensor, Tensor> BatchCSRRelabelByKey(Tensor seeds, Tensor seeds_ptr, Tensor,
                                                                       Tensor indices, Tensor indices_ptr, Tensor) {
  return BatchCSRRelabel(seeds, seeds_ptr, indices, indices_ptr);
}
static std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> BatchCOORelabel(Tensor seeds_in, Tensor seeds_ptr_in,
                                                                          Tensor coo_col_in, Tensor coo_row_in,
                                                                          Tensor coo_ptr_in) {
  Tensor s = Ids(seeds_in, "seeds"), sp = Ids(seeds_ptr_in, "seeds_ptr"), col = Ids(coo_col_in, "coo_col"),
         row = Ids(coo_row_in, "coo_row"), cp = Ids(coo_ptr_in, "coo_ptr");
  TORCH_CHECK(col.numel() == row.numel(), "coo_col and coo_row must have the same length");
  const int64_t G = sp.numel() - 1, E = row.numel();
  Tensor uniq = EmptyIds(s.numel() + E, s), uptr = EmptyIds(G + 1, s), orow = EmptyIds(E, s), ocol = EmptyIds(E, s);
  int64_t nu = 0;
  Check(gsb_batch_coo_relabel(Ctx(), Stream(), IP(s), IP(sp), s.numel(), IP(col), IP(row), IP(cp), E, G, MP(uniq),
                              MP(uptr), MP(orow), MP(ocol), &nu),
        "gsb_batch_coo_relabel");
  return {uniq.narrow(0, 0, nu), uptr, orow, ocol, cp};
}
static std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> BatchCOORelabelByKey(Tensor seeds, Tensor seeds_ptr, Tensor,
                                                                               Tensor coo_col, Tensor coo_row,
                                                                               Tensor coo_ptr, Tensor) {
  return BatchCOORelabel(seeds, seeds_ptr, coo_col, coo_row, coo_ptr);
}
static std::tuple<Tensor, Tensor, Tensor> CooSliceImpl(int64_t axis, Tensor row_in, Tensor col_in, const Tensor* edge_ptr,
                                                       Tensor members_in, const Tensor* members_ptr) {
  Tensor row = Ids(row_in, "coo_row"), col = Ids(col_in, "coo_col"), mem = Ids(members_in, "neighbors");
  TORCH_CHECK(axis == 0 || axis == 1, "axis must be 0 or 1");
  Tensor ep = edge_ptr ? Ids(*edge_ptr, "batch_ptr") : Tensor(), mp = members_ptr ? Ids(*members_ptr, "neighbors_ptr") : Tensor();
  const int64_t G = edge_ptr ? ep.numel() - 1 : 1, E = row.numel();
  Tensor orow = EmptyIds(E, row), ocol = EmptyIds(E, row), optr = EmptyIds(G + 1, row);
  int64_t n = 0;
  Check(gsb_batch_coo_slice(Ctx(), Stream(), (int)axis, IP(row), IP(col), IP(ep), E, IP(mem), IP(mp), mem.numel(), G,
                            MP(orow), MP(ocol), MP(optr), &n),
        "gsb_batch_coo_slice");
  return {orow.narrow(0, 0, n), ocol.narrow(0, 0, n), optr};
}
static std::tuple<Tensor, Tensor, Tensor> BatchCOOSlicing(int64_t axis, Tensor coo_row, Tensor coo_col, Tensor batch_ptr,
                                                          Tensor neighbors, Tensor neighbors_ptr) {
  return CooSliceImpl(axis, coo_row, coo_col, &batch_ptr, neighbors, &neighbors_ptr);
}
static std::tuple<Tensor, Tensor> COORowSlicingGlobalId(Tensor coo_row, Tensor coo_col, Tensor row_ids) {
  auto r = CooSliceImpl(1, coo_row, coo_col, nullptr, row_ids, nullptr);
  return {std::get<0>(r), std::get<1>(r)};
}
static std::tuple<Tensor, Tensor, Tensor> BatchConcat(std::vector<Tensor> data_tensors, std::vector<Tensor> offset_tensors) {
  const size_t n = data_tensors.size();
  TORCH_CHECK(n >= 1 && n == offset_tensors.size() && n <= GSB_MAX_CONCAT, "between 1 and ", GSB_MAX_CONCAT,
              " (data, offsets) pairs are required");
  std::vector<Tensor> d, o;
  const int64_t* dp[GSB_MAX_CONCAT];
  const int64_t* op[GSB_MAX_CONCAT];
  int64_t len[GSB_MAX_CONCAT], total = 0;
  for (size_t i = 0; i < n; ++i) {
    d.push_back(Ids(data_tensors[i], "data tensor"));
    o.push_back(Ids(offset_tensors[i], "offset tensor"));
    dp[i] = IP(d[i]), op[i] = IP(o[i]), len[i] = d[i].numel(), total += len[i];
  }
  const int64_t G = o[0].numel() - 1;
  Tensor out = EmptyIds(total, d[0]), key = EmptyIds(total, d[0]), ptr = EmptyIds(G + 1, d[0]);
  Check(gsb_batch_concat(Ctx(), Stream(), dp, op, len, (int)n, G, MP(out), MP(key), MP(ptr)), "gsb_batch_concat");
  return {out, key, ptr};
}
static std::tuple<std::vector<Tensor>, std::vector<Tensor>> BatchSplit(Tensor data_in, Tensor data_ptr_in, Tensor,
                                                                       std::vector<Tensor> out_tensors,
                                                                       std::vector<Tensor> out_ptr_tensors) {
  Tensor data = Ids(data_in, "data"), ptr = Ids(data_ptr_in, "data_ptr");
  const size_t n = out_tensors.size();
  TORCH_CHECK(n >= 1 && n == out_ptr_tensors.size() && n <= GSB_MAX_CONCAT, "between 1 and ", GSB_MAX_CONCAT,
              " (output, offsets) pairs are required");
  std::vector<Tensor> o;
  int64_t* outp[GSB_MAX_CONCAT];
  const int64_t* op[GSB_MAX_CONCAT];
  for (size_t i = 0; i < n; ++i) {
    TORCH_CHECK(out_tensors[i].is_cuda() && out_tensors[i].scalar_type() == torch::kInt64 && out_tensors[i].is_contiguous(),
                "output tensors must be contiguous int64 CUDA tensors");
    o.push_back(Ids(out_ptr_tensors[i], "output offsets"));
    outp[i] = MP(out_tensors[i]), op[i] = IP(o[i]);
  }
  Check(gsb_batch_split(Ctx(), Stream(), IP(data), IP(ptr), data.numel(), ptr.numel() - 1, outp, op, (int)n),
        "gsb_batch_split");
  return {out_tensors, out_ptr_tensors};
}
static std::tuple<Tensor, Tensor> BatchListSamplingProbs(Tensor probs_in, int64_t num_picks, bool replace, Tensor range_in) {
  TORCH_CHECK(!replace, "Not implemented warning");  // src/cuda/list_sampling_probs.cu:119-120 aborts as well
  Tensor probs = Floats(probs_in, "probs"), range = Ids(range_in, "range");
  const int64_t N = probs.numel(), G = range.numel() - 1;
  Tensor out = EmptyIds(std::min(N, G * num_picks), range), out_range = EmptyIds(G + 1, range);
  int64_t n = 0;
  Check(gsb_batch_list_sample(Ctx(), Stream(), FP(probs), N, IP(range), G, num_picks, NextSeed(), MP(out), MP(out_range), &n),
        "gsb_batch_list_sample");
  return {out.narrow(0, 0, n), out_range};
}
static Tensor IndexSearch(Tensor origin_in, Tensor keys_in) {  // src/tensor_ops.cc:23-31
  Tensor origin = Ids(origin_in, "origin_data"), keys = Ids(keys_in, "keys");
  Tensor out = torch::empty_like(keys);
  Check(gsb_index_search(Ctx(), Stream(), IP(origin), origin.numel(), IP(keys), keys.numel(), MP(out)), "gsb_index_search");
  return out;
}
static void SetSeed(int64_t seed) {
  g_seed_base.store((uint64_t)seed);
  g_seed_counter.store(0);
}

}  // namespace gsglue

using gsglue::Graph;
using gsglue::HeteroGraph;

#define GS_DEF2(camel, snake, fn) .def(camel, fn).def(snake, fn)

TORCH_LIBRARY(gs_classes, m) {
  m.class_<Graph>("Graph")
      .def(torch::init<bool>())
      GS_DEF2("_CAPI_SetData", "_CAPI_set_data", &Graph::SetData)
      GS_DEF2("_CAPI_GetData", "_CAPI_get_data", &Graph::GetData)
      GS_DEF2("_CAPI_GetNumRows", "_CAPI_get_num_rows", &Graph::GetNumRows)
      GS_DEF2("_CAPI_GetNumCols", "_CAPI_get_num_cols", &Graph::GetNumCols)
      GS_DEF2("_CAPI_GetNumEdges", "_CAPI_get_num_edges", &Graph::GetNumEdges)
      GS_DEF2("_CAPI_Slicing", "_CAPI_slicing", &Graph::Slicing)
      GS_DEF2("_CAPI_BatchSlicing", "_CAPI_batch_slicing", &Graph::BatchSlicing)
      GS_DEF2("_CAPI_FusionSlicing", "_CAPI_fusion_slicing", &Graph::FusedBidirSlicing)
      GS_DEF2("_CAPI_BatchFusionSlicing", "_CAPI_batch_fusion_slicing", &Graph::BatchFusedBidirSlicing)
      GS_DEF2("_CAPI_EDivUSum", "_CAPI_e_div_u_sum", &Graph::EDivUSum)
      GS_DEF2("_CAPI_Split", "_CAPI_split", &Graph::Split)
      GS_DEF2("_CAPI_Decode", "_CAPI_decode", &Graph::Decode)
      GS_DEF2("_CAPI_Sampling", "_CAPI_sampling", &Graph::Sampling)
      GS_DEF2("_CAPI_SamplingWithProbs", "_CAPI_sampling_with_probs", &Graph::SamplingProbs)
      GS_DEF2("_CAPI_FusedColumnwiseSlicingSampling", "_CAPI_fused_columnwise_slicing_sampling",
              &Graph::ColumnwiseFusedSlicingAndSampling)
      GS_DEF2("_CAPI_LoadCSC", "_CAPI_load_csc", &Graph::LoadCSC)
      GS_DEF2("_CAPI_LoadCOO", "_CAPI_load_coo", &Graph::LoadCOO)
      GS_DEF2("_CAPI_LoadCSCWithColIds", "_CAPI_load_csc_with_col_ids", &Graph::LoadCSCWithColIds)
      GS_DEF2("_CAPI_AllValidNode", "_CAPI_all_valid_node", &Graph::AllValidNode)
      .def("_CAPI_all_indices", &Graph::AllValidNode)
      GS_DEF2("_CAPI_GetRows", "_CAPI_get_rows", &Graph::GetRows)
      GS_DEF2("_CAPI_GetCols", "_CAPI_get_cols", &Graph::GetCols)
      GS_DEF2("_CAPI_GetValidRows", "_CAPI_get_valid_rows", &Graph::GetValidRows)
      GS_DEF2("_CAPI_GetValidCols", "_CAPI_get_valid_cols", &Graph::GetValidCols)
      GS_DEF2("_CAPI_GetCOORows", "_CAPI_get_coo_rows", &Graph::GetCOORows)
      GS_DEF2("_CAPI_GetCooCols", "_CAPI_get_coo_cols", &Graph::GetCOOCols)
      GS_DEF2("_CAPI_Relabel", "_CAPI_relabel", &Graph::Relabel_)
      GS_DEF2("_CAPI_Sum", "_CAPI_sum", &Graph::Sum)
      GS_DEF2("_CAPI_Normalize", "_CAPI_normalize", &Graph::Normalize)
      GS_DEF2("_CAPI_Divide", "_CAPI_divide", &Graph::Divide)
      GS_DEF2("_CAPI_Metadata", "_CAPI_metadata", &Graph::MetaData)
      GS_DEF2("_CAPI_COOMetadata", "_CAPI_coo_metadata", &Graph::COOMetaData)
      GS_DEF2("_CAPI_CSCMetadata", "_CAPI_csc_metadata", &Graph::CSCMetaData)
      GS_DEF2("_CAPI_RandomWalk", "_CAPI_random_walk", &Graph::RandomWalk)
      GS_DEF2("_CAPI_SDDMM", "_CAPI_sddmm", &Graph::SDDMM)
      GS_DEF2("_CAPI_GetCSC", "_CAPI_get_csc", &Graph::GetCSCTensor)
      GS_DEF2("_CAPI_GetCOO", "_CAPI_get_coo", &Graph::GetCOOTensor)
      GS_DEF2("_CAPI_SetCOO", "_CAPI_set_coo", &Graph::SetCOOByTensor)
      GS_DEF2("_CAPI_SetMetadata", "_CAPI_set_metadata", &Graph::SetMetaData);

  m.class_<HeteroGraph>("HeteroGraph")
      .def(torch::init<>())
      GS_DEF2("_CAPI_LoadFromHomo", "_CAPI_load_from_homo", &HeteroGraph::LoadFromHomo)
      GS_DEF2("_CAPI_GetHomoGraph", "_CAPI_get_homo_graph", &HeteroGraph::GetHomoGraph)
      GS_DEF2("_CAPI_MetapathRandomWalkFused", "_CAPI_metapath_random_walk_fused",
              &HeteroGraph::MetapathRandomWalkFused);
}

TORCH_LIBRARY(gs_ops, m) {
  m.def("_CAPI_ListSampling", &gsglue::ListSampling);
  m.def("list_sampling", &gsglue::ListSampling);
  m.def("_CAPI_ListSamplingWithProbs", &gsglue::ListSamplingProbs);
  m.def("list_sampling_with_probs", &gsglue::ListSamplingProbs);
  m.def("_CAPI_Unique", &gsglue::Unique);
  m.def("_CAPI_BatchCSRRelabel", &gsglue::BatchCSRRelabel);
  m.def("BatchCSRRelabel", &gsglue::BatchCSRRelabel);
  m.def("_CAPI_SplitByOffset", &gsglue::SplitByOffset);
  m.def("SplitByOffset", &gsglue::SplitByOffset);
  m.def("_CAPI_IndptrSplitByOffset", &gsglue::IndptrSplitByOffset);
  m.def("IndptrSplitByOffset", &gsglue::IndptrSplitByOffset);
  m.def("_CAPI_IndptrSplitBySize", &gsglue::IndptrSplitBySize);
  m.def("_CAPI_BatchListSamplingWithProbs", &gsglue::BatchListSamplingProbs);
  m.def("_CAPI_BatchConcat", &gsglue::BatchConcat);
  m.def("_CAPI_BatchUnique", &gsglue::BatchUnique);
  m.def("_CAPI_BatchUniqueByKey", &gsglue::BatchUniqueByKey);
  m.def("_CAPI_BatchUnique2", &gsglue::BatchUnique2);
  m.def("_CAPI_BatchUniqueByKey2", &gsglue::BatchUniqueByKey2);
  m.def("_CAPI_BatchCSRRelabelByKey", &gsglue::BatchCSRRelabelByKey);
  m.def("_CAPI_BatchCOORelabelByKey", &gsglue::BatchCOORelabelByKey);
  m.def("_CAPI_BatchCOORelabel", &gsglue::BatchCOORelabel);
  m.def("BatchCOORelabel", &gsglue::BatchCOORelabel);
  m.def("_CAPI_BatchSplit", &gsglue::BatchSplit);
  m.def("_CAPI_BatchCOOSlicing", &gsglue::BatchCOOSlicing);
  m.def("_CAPI_BatchEncode", &gsglue::BatchEncode);
  m.def("_CAPI_BatchDecode", &gsglue::BatchDecode);
  m.def("_CAPI_GetBatchOffsets", &gsglue::GetBatchOffsets);
  m.def("_CAPI_COORowSlicingGlobalId", &gsglue::COORowSlicingGlobalId);
  m.def("_CAPI_IndexSearch", &gsglue::IndexSearch);
  m.def("COORowSlicingGlobalId", &gsglue::COORowSlicingGlobalId);
  m.def("_CAPI_SetSeed", &gsglue::SetSeed);
}
