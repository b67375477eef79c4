// C interface of the compiler core (see ffi.h).
#include "ffi.h"

#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>

#include "builder.h"
#include "graph_algos.h"
#include "ir.h"
#include "models.h"
#include "search.h"
#include "substitutions.h"

using namespace ff;

struct ffc_builder {
  GraphBuilder b;
};
struct ffc_graph {
  Graph g;
};

namespace {
thread_local std::string g_error;

template <typename F>
int guarded(F &&f) {
  try {
    f();
    g_error.clear();
    return 0;
  } catch (const std::exception &e) {
    g_error = e.what();
    return 1;
  }
}
char *dup_string(const std::string &s) {
  char *p = (char *)std::malloc(s.size() + 1);
  if (p) std::memcpy(p, s.c_str(), s.size() + 1);
  return p;
}
ValueRef ref(ffc_value_t v) { return ValueRef{v.node, (Slot)v.slot}; }
ffc_value_t val(const ValueRef &v) { return ffc_value_t{v.node, (int)v.slot}; }
std::string str(const char *s) { return s ? std::string(s) : std::string(); }
std::optional<std::string> opt(const char *s) { return s && *s ? std::optional<std::string>(s) : std::nullopt; }
Json json_or_empty(const char *s) { return s && *s ? Json::parse(s) : Json::object(); }
}  // namespace

#define FFC_EXPORT extern "C" __attribute__((visibility("default")))

FFC_EXPORT const char *ffc_last_error(void) { return g_error.c_str(); }
FFC_EXPORT void ffc_string_free(char *s) { std::free(s); }
FFC_EXPORT const char *ffc_slot_name(int slot) {
  static thread_local std::string s;
  s = to_string((Slot)slot);
  return s.c_str();
}
FFC_EXPORT int ffc_slot_from_name(const char *name) {
  try {
    return (int)slot_from_string(str(name));
  } catch (const std::exception &e) {
    g_error = e.what();
    return -1;
  }
}

FFC_EXPORT ffc_builder_t *ffc_builder_create(void) { return new ffc_builder(); }
FFC_EXPORT void ffc_builder_destroy(ffc_builder_t *b) { delete b; }

FFC_EXPORT int ffc_builder_create_input(ffc_builder_t *b, const int64_t *dims, int ndims, const char *dtype, const char *name, ffc_value_t *out) {
  return guarded([&] {
    std::vector<int64_t> d(dims, dims + ndims);
    *out = val(b->b.create_input(d, datatype_from_string(dtype ? dtype : "FLOAT"), false, str(name)));
  });
}
FFC_EXPORT int ffc_builder_create_weight(ffc_builder_t *b, const int64_t *dims, int ndims, const char *dtype, const char *initializer_json,
                                         const char *name, ffc_value_t *out) {
  return guarded([&] {
    std::vector<int64_t> d(dims, dims + ndims);
    std::optional<Json> init;
    if (initializer_json && *initializer_json) init = Json::parse(initializer_json);
    *out = val(b->b.create_weight(d, datatype_from_string(dtype ? dtype : "FLOAT"), init, true, str(name)));
  });
}
FFC_EXPORT int ffc_builder_add_layer(ffc_builder_t *b, const char *op_type, const char *attrs_json, const ffc_value_t *inputs,
                                     const char *const *input_slots, int num_inputs, const char *name, ffc_value_t *outputs,
                                     int max_outputs, int *num_outputs) {
  return guarded([&] {
    std::vector<std::pair<Slot, ValueRef>> ins;
    for (int i = 0; i < num_inputs; ++i) ins.push_back({slot_from_string(str(input_slots[i])), ref(inputs[i])});
    auto outs = b->b.add_layer(optype_from_string(str(op_type)), json_or_empty(attrs_json), ins, str(name));
    if ((int)outs.size() > max_outputs) throw Error("ffc_builder_add_layer: operator has more outputs than max_outputs");
    for (size_t i = 0; i < outs.size(); ++i) outputs[i] = val(outs[i]);
    if (num_outputs) *num_outputs = (int)outs.size();
  });
}
FFC_EXPORT int ffc_builder_dense(ffc_builder_t *b, ffc_value_t x, int64_t out_channels, const char *activation, int use_bias, const char *name,
                                 ffc_value_t *out) {
  return guarded([&] { *out = val(b->b.dense(ref(x), out_channels, opt(activation), use_bias != 0, std::nullopt, std::nullopt, str(name))); });
}
FFC_EXPORT int ffc_builder_conv2d(ffc_builder_t *b, ffc_value_t x, int64_t out_channels, int kernel_h, int kernel_w, int stride_h, int stride_w,
                                  int padding_h, int padding_w, const char *activation, int groups, int use_bias, const char *name,
                                  ffc_value_t *out) {
  return guarded([&] {
    *out = val(b->b.conv2d(ref(x), out_channels, kernel_h, kernel_w, stride_h, stride_w, padding_h, padding_w, opt(activation), groups,
                           use_bias != 0, std::nullopt, std::nullopt, str(name)));
  });
}
FFC_EXPORT int ffc_builder_unary(ffc_builder_t *b, const char *op, ffc_value_t x, int has_scalar, double scalar, const char *name,
                                 ffc_value_t *out) {
  return guarded([&] {
    *out = val(b->b.unary(optype_from_string(str(op)), ref(x), has_scalar ? std::optional<double>(scalar) : std::nullopt, str(name)));
  });
}
FFC_EXPORT int ffc_builder_binary(ffc_builder_t *b, const char *op, ffc_value_t x, ffc_value_t y, const char *name, ffc_value_t *out) {
  return guarded([&] { *out = val(b->b.binary(optype_from_string(str(op)), ref(x), ref(y), str(name))); });
}
FFC_EXPORT int ffc_builder_softmax(ffc_builder_t *b, ffc_value_t x, int dim, const char *name, ffc_value_t *out) {
  return guarded([&] { *out = val(b->b.softmax(ref(x), dim, str(name))); });
}
FFC_EXPORT int ffc_builder_pool2d(ffc_builder_t *b, ffc_value_t x, int kernel_h, int kernel_w, int stride_h, int stride_w, int padding_h,
                                  int padding_w, const char *pool_type, const char *activation, const char *name, ffc_value_t *out) {
  return guarded([&] {
    *out = val(b->b.pool2d(ref(x), kernel_h, kernel_w, stride_h, stride_w, padding_h, padding_w, str(pool_type).empty() ? "MAX" : str(pool_type),
                           opt(activation), str(name)));
  });
}
FFC_EXPORT int ffc_builder_batch_norm(ffc_builder_t *b, ffc_value_t x, int affine, const char *activation, double eps, double momentum,
                                      const char *name, ffc_value_t *out) {
  return guarded([&] { *out = val(b->b.batch_norm(ref(x), affine != 0, opt(activation), eps, momentum, str(name))); });
}
FFC_EXPORT int ffc_builder_layer_norm(ffc_builder_t *b, ffc_value_t x, const int *axes, int num_axes, int affine, double eps, const char *name,
                                      ffc_value_t *out) {
  return guarded([&] { *out = val(b->b.layer_norm(ref(x), std::vector<int>(axes, axes + num_axes), affine != 0, eps, str(name))); });
}
FFC_EXPORT int ffc_builder_embedding(ffc_builder_t *b, ffc_value_t ids, int64_t num_entries, int64_t out_dim, const char *aggr, const char *dtype,
                                     const char *name, ffc_value_t *out) {
  return guarded([&] {
    *out = val(b->b.embedding(ref(ids), num_entries, out_dim, str(aggr).empty() ? "SUM" : str(aggr),
                              datatype_from_string(dtype && *dtype ? dtype : "FLOAT"), std::nullopt, str(name)));
  });
}
FFC_EXPORT int ffc_builder_multihead_attention(ffc_builder_t *b, ffc_value_t q, ffc_value_t k, ffc_value_t v, int64_t embed_dim,
                                               int64_t num_heads, int64_t kdim, int64_t vdim, double dropout, int bias, int add_bias_kv,
                                               int add_zero_attn, const char *name, ffc_value_t *out) {
  return guarded([&] {
    *out = val(b->b.multihead_attention(ref(q), ref(k), ref(v), embed_dim, num_heads, kdim > 0 ? std::optional<int64_t>(kdim) : std::nullopt,
                                        vdim > 0 ? std::optional<int64_t>(vdim) : std::nullopt, dropout, bias != 0, add_bias_kv != 0,
                                        add_zero_attn != 0, std::nullopt, str(name)));
  });
}
FFC_EXPORT int ffc_builder_batch_matmul(ffc_builder_t *b, ffc_value_t a, ffc_value_t bb, const char *name, ffc_value_t *out) {
  return guarded([&] { *out = val(b->b.batch_matmul(ref(a), ref(bb), str(name))); });
}
FFC_EXPORT int ffc_builder_dropout(ffc_builder_t *b, ffc_value_t x, double rate, uint64_t seed, const char *name, ffc_value_t *out) {
  return guarded([&] { *out = val(b->b.dropout(ref(x), rate, seed, str(name))); });
}
FFC_EXPORT int ffc_builder_cast(ffc_builder_t *b, ffc_value_t x, const char *dtype, const char *name, ffc_value_t *out) {
  return guarded([&] { *out = val(b->b.cast(ref(x), datatype_from_string(str(dtype)), str(name))); });
}
FFC_EXPORT int ffc_builder_concat(ffc_builder_t *b, const ffc_value_t *xs, int num, int axis, const char *name, ffc_value_t *out) {
  return guarded([&] {
    std::vector<ValueRef> v;
    for (int i = 0; i < num; ++i) v.push_back(ref(xs[i]));
    *out = val(b->b.concat(v, axis, str(name)));
  });
}
FFC_EXPORT int ffc_builder_split(ffc_builder_t *b, ffc_value_t x, const int64_t *sizes, int num, int axis, const char *name, ffc_value_t *outs) {
  return guarded([&] {
    auto r = b->b.split(ref(x), std::vector<int64_t>(sizes, sizes + num), axis, str(name));
    for (size_t i = 0; i < r.size(); ++i) outs[i] = val(r[i]);
  });
}
FFC_EXPORT int ffc_builder_flat(ffc_builder_t *b, ffc_value_t x, const char *name, ffc_value_t *out) {
  return guarded([&] { *out = val(b->b.flat(ref(x), 1, -1, str(name))); });
}
FFC_EXPORT int ffc_builder_transpose(ffc_builder_t *b, ffc_value_t x, const int *perm, int num, const char *name, ffc_value_t *out) {
  return guarded([&] { *out = val(b->b.transpose(ref(x), std::vector<int>(perm, perm + num), str(name))); });
}
FFC_EXPORT int ffc_builder_reshape(ffc_builder_t *b, ffc_value_t x, const int64_t *dims, int num, const char *name, ffc_value_t *out) {
  return guarded([&] { *out = val(b->b.reshape(ref(x), std::vector<int64_t>(dims, dims + num), str(name))); });
}
FFC_EXPORT int ffc_builder_reverse(ffc_builder_t *b, ffc_value_t x, int axis, const char *name, ffc_value_t *out) {
  return guarded([&] { *out = val(b->b.reverse(ref(x), axis, str(name))); });
}
FFC_EXPORT int ffc_builder_gather(ffc_builder_t *b, ffc_value_t x, ffc_value_t index, int dim, const char *name, ffc_value_t *out) {
  return guarded([&] { *out = val(b->b.gather(ref(x), ref(index), dim, str(name))); });
}
FFC_EXPORT int ffc_builder_top_k(ffc_builder_t *b, ffc_value_t x, int k, int sorted, const char *name, ffc_value_t *values,
                                 ffc_value_t *indices) {
  return guarded([&] {
    auto r = b->b.top_k(ref(x), k, sorted != 0, str(name));
    *values = val(r.at(0));
    *indices = val(r.at(1));
  });
}
FFC_EXPORT int ffc_builder_reduce(ffc_builder_t *b, const char *op, ffc_value_t x, const int *axes, int num_axes, int keepdims,
                                  const char *name, ffc_value_t *out) {
  return guarded([&] {
    *out = val(b->b.reduce(optype_from_string(str(op)), ref(x), std::vector<int>(axes, axes + num_axes), keepdims != 0, str(name)));
  });
}
FFC_EXPORT int ffc_builder_broadcast(ffc_builder_t *b, ffc_value_t x, const int64_t *target, int num, const char *name, ffc_value_t *out) {
  return guarded([&] { *out = val(b->b.broadcast(ref(x), std::vector<int64_t>(target, target + num), str(name))); });
}
FFC_EXPORT ffc_builder_t *ffc_builder_create_parallel(void) { return new ffc_builder{GraphBuilder(true)}; }
FFC_EXPORT int ffc_builder_parallel_partition(ffc_builder_t *b, ffc_value_t x, int dim, int degree, const char *name, ffc_value_t *out) {
  return guarded([&] { *out = val(b->b.parallel_partition(ref(x), dim, degree, str(name))); });
}
FFC_EXPORT int ffc_builder_parallel_combine(ffc_builder_t *b, ffc_value_t x, int dim, int degree, const char *name, ffc_value_t *out) {
  return guarded([&] { *out = val(b->b.parallel_combine(ref(x), dim, degree, str(name))); });
}
FFC_EXPORT int ffc_builder_parallel_replicate(ffc_builder_t *b, ffc_value_t x, int degree, const char *name, ffc_value_t *out) {
  return guarded([&] { *out = val(b->b.parallel_replicate(ref(x), degree, str(name))); });
}
FFC_EXPORT int ffc_builder_parallel_reduce(ffc_builder_t *b, ffc_value_t x, int degree, const char *name, ffc_value_t *out) {
  return guarded([&] { *out = val(b->b.parallel_reduce(ref(x), degree, str(name))); });
}
FFC_EXPORT int ffc_builder_value_degrees(const ffc_builder_t *b, ffc_value_t v, int *degrees, int max_dims, int *ndims, int *sum_degree,
                                         int *copy_degree) {
  return guarded([&] {
    const PShape &sh = b->b.graph.shape(ref(v));
    auto d = sh.degrees();
    if ((int)d.size() > max_dims) throw Error("ffc_builder_value_degrees: max_dims too small");
    for (size_t i = 0; i < d.size(); ++i) degrees[i] = (int)d[i];
    *ndims = (int)d.size();
    if (sum_degree) *sum_degree = (int)sh.sum_degree;
    if (copy_degree) *copy_degree = (int)sh.discard_copy_degree;
  });
}
FFC_EXPORT int ffc_builder_value_shape(const ffc_builder_t *b, ffc_value_t v, int64_t *dims, int max_dims, int *ndims) {
  return guarded([&] {
    auto sizes = b->b.graph.shape(ref(v)).sizes();
    if ((int)sizes.size() > max_dims) throw Error("ffc_builder_value_shape: max_dims too small");
    for (size_t i = 0; i < sizes.size(); ++i) dims[i] = sizes[i];
    *ndims = (int)sizes.size();
  });
}
FFC_EXPORT ffc_graph_t *ffc_builder_graph(const ffc_builder_t *b) { return new ffc_graph{b->b.graph}; }

FFC_EXPORT ffc_graph_t *ffc_model_build(const char *model_name, const char *config_json) {
  ffc_graph_t *g = nullptr;
  guarded([&] { g = new ffc_graph{build_model(str(model_name), json_or_empty(config_json))}; });
  return g;
}
FFC_EXPORT ffc_graph_t *ffc_graph_from_json(const char *v1_json) {
  ffc_graph_t *g = nullptr;
  guarded([&] { g = new ffc_graph{graph_from_v1(Json::parse(str(v1_json)))}; });
  return g;
}
FFC_EXPORT char *ffc_graph_to_json(const ffc_graph_t *g, int parallel, int indent) {
  char *r = nullptr;
  guarded([&] { r = dup_string(graph_to_v1(g->g, parallel != 0).dump(indent)); });
  return r;
}
FFC_EXPORT char *ffc_graph_to_dot(const ffc_graph_t *g) {
  char *r = nullptr;
  guarded([&] { r = dup_string(g->g.as_dot()); });
  return r;
}
FFC_EXPORT int ffc_graph_estimate(const ffc_graph_t *pcg, int num_nodes, int gpus_per_node, double *runtime_ms) {
  return guarded([&] {
    MachineSpec ms;
    ms.num_nodes = num_nodes;
    ms.num_gpus_per_node = gpus_per_node;
    CostParams cp;
    cp.nvlink_gbs = ms.intra_node_bandwidth;
    CostEstimator est(cp, ms);
    const double t = evaluate_pcg(pcg->g, ms, est).runtime_ms;
    if (!(t < 1e300)) throw Error("no machine mapping of this graph fits " + std::to_string(num_nodes * gpus_per_node) + " devices");
    *runtime_ms = t;
  });
}
FFC_EXPORT char *ffc_graph_sp_decomposition(const ffc_graph_t *g) {
  char *r = nullptr;
  guarded([&] {
    // exact when the graph is series-parallel, from SP-ization otherwise; JSON of the left-associative binary tree
    r = dup_string(sp_to_json(left_associative_binary_sp_tree(get_graph_sp_decomposition(g->g))).dump());
  });
  return r;
}
FFC_EXPORT int ffc_graph_num_nodes(const ffc_graph_t *g) { return (int)g->g.num_nodes(); }
FFC_EXPORT int ffc_graph_save_file(const ffc_graph_t *g, const char *path, int parallel, int indent) {
  return guarded([&] {
    std::ofstream f(str(path));
    if (!f) throw Error("cannot open " + str(path) + " for writing");
    f << graph_to_v1(g->g, parallel != 0).dump(indent);
    if (!f.flush()) throw Error("write to " + str(path) + " failed");
  });
}
FFC_EXPORT ffc_graph_t *ffc_graph_load_file(const char *path) {
  ffc_graph_t *g = nullptr;
  guarded([&] {
    std::ifstream f(str(path));
    if (!f) throw Error("cannot open " + str(path));
    std::stringstream ss;
    ss << f.rdbuf();
    g = new ffc_graph{graph_from_v1(Json::parse(ss.str()))};
  });
  return g;
}
FFC_EXPORT int ffc_graph_node_ids(const ffc_graph_t *g, int *ids, int max_ids, int *num) {
  return guarded([&] {
    auto order = g->g.topological_order();
    *num = (int)order.size();
    for (int i = 0; i < (int)order.size() && i < max_ids; ++i) ids[i] = (int)order[i];
  });
}
FFC_EXPORT char *ffc_graph_node_op_type(const ffc_graph_t *g, int node) {
  char *r = nullptr;
  guarded([&] { r = dup_string(to_string(g->g.node(node).type)); });
  return r;
}
FFC_EXPORT char *ffc_graph_node_name(const ffc_graph_t *g, int node) {
  char *r = nullptr;
  guarded([&] { r = dup_string(g->g.node(node).name); });
  return r;
}
FFC_EXPORT char *ffc_graph_node_attrs_json(const ffc_graph_t *g, int node) {
  char *r = nullptr;
  guarded([&] { r = dup_string(g->g.node(node).attrs.dump()); });
  return r;
}
FFC_EXPORT char *ffc_graph_node_view_json(const ffc_graph_t *g, int node) {
  char *r = nullptr;
  guarded([&] {
    const Node &n = g->g.node(node);
    if (!n.view) throw Error("node " + std::to_string(node) + " has no machine view (the graph is not mapped)");
    r = dup_string(n.view->to_json().dump());
  });
  return r;
}
FFC_EXPORT int ffc_graph_value_shape(const ffc_graph_t *g, ffc_value_t v, int64_t *dims, int max_dims, int *ndims) {
  return guarded([&] {
    auto sizes = g->g.shape(ref(v)).sizes();
    if ((int)sizes.size() > max_dims) throw Error("ffc_graph_value_shape: max_dims too small");
    for (size_t i = 0; i < sizes.size(); ++i) dims[i] = sizes[i];
    *ndims = (int)sizes.size();
  });
}
FFC_EXPORT const char *ffc_graph_value_dtype(const ffc_graph_t *g, ffc_value_t v) {
  static thread_local std::string s;
  if (guarded([&] { s = to_string(g->g.shape(ref(v)).dtype); })) return nullptr;
  return s.c_str();
}
FFC_EXPORT int ffc_graph_value_create_grad(const ffc_graph_t *g, ffc_value_t v, int *create_grad) {
  return guarded([&] { *create_grad = g->g.node(v.node).out((Slot)v.slot).create_grad ? 1 : 0; });
}
FFC_EXPORT int ffc_datatype_size(const char *dtype) {
  int n = -1;
  guarded([&] { n = dtype_bytes(datatype_from_string(str(dtype))); });
  return n;
}
FFC_EXPORT const char *ffc_builder_value_dtype(const ffc_builder_t *b, ffc_value_t v) {
  static thread_local std::string s;
  if (guarded([&] { s = to_string(b->b.graph.shape(ref(v)).dtype); })) return nullptr;
  return s.c_str();
}
FFC_EXPORT void ffc_graph_destroy(ffc_graph_t *g) { delete g; }

FFC_EXPORT int ffc_graph_optimize(const ffc_graph_t *cg, int num_nodes, int gpus_per_node, const char *algorithm, int budget, double alpha,
                                  unsigned seed, ffc_graph_t **out, double *runtime_ms) {
  return guarded([&] {
    MachineSpec ms;
    ms.num_nodes = num_nodes;
    ms.num_gpus_per_node = gpus_per_node;
    const int W = num_nodes * gpus_per_node;
    CostParams cp;
    cp.nvlink_gbs = ms.intra_node_bandwidth;
    CostEstimator est(cp, ms);
    std::vector<Substitution> rules = get_substitution_set(ms);
    Graph base = pcg_from_computation_graph(cg->g);
    SearchResult best = evaluate_pcg(base, ms, est);
    std::string algo = str(algorithm).empty() ? "unity" : str(algorithm);
    if (W > 1) {
      // seed: plain data parallelism expressed with the sample-dim partition rules and the cancellation rules
      std::vector<Substitution> dp;
      const std::string sfx = "_0_" + std::to_string(W);
      for (auto &r : rules) {
        const std::string &n = r.name;
        bool cancel = n.rfind("cancel", 0) == 0;
        bool batch = n.rfind("partition_", 0) == 0 && n.find("_combine") != std::string::npos &&
                     (n.size() >= sfx.size() && (n.compare(n.size() - sfx.size(), sfx.size(), sfx) == 0 ||
                                                 n.find(sfx + "_bias") != std::string::npos || n.find(sfx + "_affine") != std::string::npos));
        bool whole = (n.rfind("partition_attention_combine_", 0) == 0 || n.rfind("partition_conv2d_combine_", 0) == 0) &&
                     n.find("_" + std::to_string(W)) != std::string::npos;
        if (cancel || batch || whole) dp.push_back(r);
      }
      SearchResult dpr = evaluate_pcg(apply_rules_exhaustively(base, dp, 100000, W), ms, est);
      if (algo == "data_parallel" || dpr.runtime_ms < best.runtime_ms) best = dpr;
      if (algo == "unity" && budget > 0) {
        UnityConfig c;
        c.alpha = alpha;
        c.budget = budget;
        SearchResult r = unity_search(best.pcg, ms, est, rules, c);
        if (r.runtime_ms < best.runtime_ms) best = r;
      } else if (algo == "mcmc") {
        MCMCConfig c;
        c.seed = seed;
        c.num_iterations = budget > 0 ? budget : 100;
        SearchResult r = evaluate_pcg(mcmc_search(best.pcg, ms, est, rules, c).pcg, ms, est);
        if (r.runtime_ms < best.runtime_ms) best = r;
      }
    }
    *out = new ffc_graph{mapped_pcg_from_pcg_and_mapping(best.pcg, best.mapping)};
    if (runtime_ms) *runtime_ms = best.runtime_ms;
  });
}
