// C interface of the compiler core (see ffi.h).
#include "ffi.h"

#include <cstdlib>
#include <cstring>
#include <string>

#include "builder.h"
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
FFC_EXPORT int ffc_graph_num_nodes(const ffc_graph_t *g) { return (int)g->g.num_nodes(); }
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
