#include "builder.h"

#include <algorithm>

namespace ff {

static Json opt_str(const std::optional<std::string> &s) { return s ? Json(*s) : Json(); }

static Json plain_shape_json(const std::vector<int64_t> &dims, DataType dt) { return PShape::make(dims, dt).to_json_plain(); }

V GraphBuilder::create_input(const std::vector<int64_t> &dims, DataType dt, bool create_grad, const std::string &name) {
  Json a = Json::object();
  a["tensor_shape"] = plain_shape_json(dims, dt);
  NodeId n = graph.add_node(OpType::INPUT, a, name, {}, {{Slot::OUTPUT, PShape::make(dims, dt), create_grad}});
  return {n, Slot::OUTPUT};
}

V GraphBuilder::create_weight(const std::vector<int64_t> &dims, DataType dt, const OptInit &init, bool create_grad,
                              const std::string &name) {
  Json a = Json::object();
  a["tensor_shape"] = plain_shape_json(dims, dt);
  if (init) a["initializer"] = *init;
  else {
    Json z = Json::object();
    z["type"] = "zero";
    z["value"] = Json::object();
    a["initializer"] = z;
  }
  NodeId n = graph.add_node(OpType::WEIGHT, a, name, {}, {{Slot::OUTPUT, PShape::make(dims, dt), create_grad}});
  return {n, Slot::OUTPUT};
}

// A weight of the unparallel shape followed by the parallel ops that bring it to `goal`.
V GraphBuilder::weight_for(const PShape &goal, const Json &init, const std::string &name) {
  V w = create_weight(goal.sizes(), goal.dtype, init, true, name);
  if (!parallel_) return w;
  for (int d = 0; d < goal.ndim(); ++d)
    if (goal.dims[d].degree != 1) w = parallel_partition(w, d, goal.dims[d].degree);
  // A weight cannot be turned into partial sums; a slot that asks for sum degree s (the bias of a
  // row-parallel Linear) receives s further copies and the executor lets one of them contribute.
  int copies = goal.discard_copy_degree * goal.sum_degree;
  if (copies != 1) w = parallel_replicate(w, copies);
  return w;
}

std::vector<V> GraphBuilder::add_layer(OpType type, Json attrs, std::vector<std::pair<Slot, V>> inputs,
                                       const std::string &name, const std::map<Slot, Json> &initializers) {
  SlotShapes in_shapes;
  for (auto &p : inputs)
    if (!is_weight_slot(type, p.first)) in_shapes.push_back({p.first, graph.shape(p.second)});
  Inferred inf = infer_shapes(type, attrs, in_shapes);
  std::vector<InEdge> edges;
  for (auto &p : inputs) edges.push_back({p.first, p.second});
  for (auto &w : inf.weights) {
    bool given = false;
    for (auto &p : inputs) if (p.first == w.first) given = true;
    if (given) continue;
    auto it = initializers.find(w.first);
    Json init = it != initializers.end() ? it->second : default_initializer(type, w.first, attrs, in_shapes);
    std::string wname = name.empty() ? "" : name + "." + to_string(w.first);
    std::transform(wname.begin(), wname.end(), wname.begin(), [](unsigned char c) { return (char)std::tolower(c); });
    edges.push_back({w.first, weight_for(w.second, init, wname)});
  }
  std::vector<OutValue> outs;
  for (auto &o : inf.outputs) outs.push_back({o.first, o.second, true});
  NodeId n = graph.add_node(type, std::move(attrs), name, edges, outs);
  std::vector<V> r;
  for (auto &o : inf.outputs) r.push_back({n, o.first});
  return r;
}

V GraphBuilder::unary(OpType t, V x, std::optional<double> scalar, const std::string &name) {
  Json a = Json::object();
  a["op_type"] = to_string(t);
  a["scalar"] = scalar ? Json(*scalar) : Json();
  return add_layer(t, a, {{Slot::INPUT, x}}, name)[0];
}

V GraphBuilder::binary(OpType t, V lhs, V rhs, const std::string &name) {
  // like the reference builder, insert a cast when dtypes differ and a broadcast when ranks differ
  const PShape &ls = shape(lhs), &rs = shape(rhs);
  if (ls.dtype != rs.dtype) rhs = cast(rhs, ls.dtype);
  Json a = Json::object();
  a["type"] = to_string(t);
  a["compute_type"] = to_string(ls.dtype);
  a["should_broadcast_lhs"] = false;
  a["should_broadcast_rhs"] = ls.sizes() != shape(rhs).sizes();
  return add_layer(t, a, {{Slot::LHS_INPUT, lhs}, {Slot::RHS_INPUT, rhs}}, name)[0];
}

V GraphBuilder::dense(V x, int64_t out_channels, const std::optional<std::string> &activation, bool use_bias,
                      const OptInit &proj_init, const OptInit &bias_init, const std::string &name) {
  Json a = Json::object();
  a["out_channels"] = (long long)out_channels;
  a["use_bias"] = use_bias;
  a["data_type"] = to_string(shape(x).dtype);
  a["activation"] = opt_str(activation);
  a["regularizer"] = Json();
  std::map<Slot, Json> inits;
  if (proj_init) inits[Slot::WEIGHT] = *proj_init;
  if (bias_init) inits[Slot::BIAS] = *bias_init;
  return add_layer(OpType::LINEAR, a, {{Slot::INPUT, x}}, name, inits)[0];
}

V GraphBuilder::conv2d(V x, int64_t out_channels, int kh, int kw, int sh, int sw, int ph, int pw,
                       const std::optional<std::string> &activation, int groups, bool use_bias,
                       const OptInit &kernel_init, const OptInit &bias_init, const std::string &name) {
  Json a = Json::object();
  a["out_channels"] = (long long)out_channels;
  a["kernel_h"] = kh; a["kernel_w"] = kw; a["stride_h"] = sh; a["stride_w"] = sw;
  a["padding_h"] = ph; a["padding_w"] = pw; a["groups"] = groups;
  a["activation"] = opt_str(activation);
  a["use_bias"] = use_bias;
  std::map<Slot, Json> inits;
  if (kernel_init) inits[Slot::FILTER] = *kernel_init;
  if (bias_init) inits[Slot::BIAS] = *bias_init;
  return add_layer(OpType::CONV2D, a, {{Slot::INPUT, x}}, name, inits)[0];
}

V GraphBuilder::pool2d(V x, int kh, int kw, int sh, int sw, int ph, int pw, const std::string &pool_type,
                       const std::optional<std::string> &activation, const std::string &name) {
  Json a = Json::object();
  a["kernel_h"] = kh; a["kernel_w"] = kw; a["stride_h"] = sh; a["stride_w"] = sw;
  a["padding_h"] = ph; a["padding_w"] = pw;
  a["pool_type"] = pool_type;
  a["activation"] = opt_str(activation);
  return add_layer(OpType::POOL2D, a, {{Slot::INPUT, x}}, name)[0];
}

V GraphBuilder::adaptive_pool2d(V x, int out_h, int out_w, const std::string &pool_type, const std::string &name) {
  // lib/pcg/src/pcg/computation_graph_builder.cc (adaptive_pool2d): derive kernel and stride from the
  // input extent; the extent must be a multiple of the requested output extent.
  const PShape &s = shape(x);
  if (s.ndim() != 4) throw Error("adaptive_pool2d: input must be NCHW");
  int64_t h = s.dims[2].size, w = s.dims[3].size;
  if (h % out_h || w % out_w) throw Error("adaptive_pool2d: input extent must be a multiple of the output extent");
  int kh = (int)(h / out_h), kw = (int)(w / out_w);
  return pool2d(x, kh, kw, kh, kw, 0, 0, pool_type, std::nullopt, name);
}

V GraphBuilder::batch_norm(V x, bool affine, const std::optional<std::string> &activation, double eps,
                           std::optional<double> momentum, const std::string &name) {
  if (activation && *activation != "RELU") throw Error("batch_norm: only a fused RELU is supported");
  Json a = Json::object();
  a["relu"] = activation.has_value();
  a["affine"] = affine;
  a["eps"] = eps;
  a["momentum"] = momentum ? Json(*momentum) : Json();
  return add_layer(OpType::BATCHNORM, a, {{Slot::INPUT, x}}, name)[0];
}

V GraphBuilder::layer_norm(V x, const std::vector<int> &axes, bool affine, double eps, const std::string &name) {
  Json a = Json::object();
  std::vector<int> norm;
  for (int ax : axes) norm.push_back(shape(x).norm_dim(ax));
  std::sort(norm.begin(), norm.end());
  a["axes"] = Json::from_ints(norm);
  a["elementwise_affine"] = affine;
  a["eps"] = eps;
  return add_layer(OpType::LAYERNORM, a, {{Slot::INPUT, x}}, name)[0];
}

V GraphBuilder::embedding(V x, int64_t num_entries, int64_t out_dim, const std::string &aggr, DataType dt,
                          const OptInit &init, const std::string &name) {
  Json a = Json::object();
  a["num_entries"] = (long long)num_entries;
  a["out_channels"] = (long long)out_dim;
  a["aggr"] = aggr.empty() ? Json() : Json(aggr);
  a["data_type"] = to_string(dt);
  std::map<Slot, Json> inits;
  if (init) inits[Slot::WEIGHT] = *init;
  return add_layer(OpType::EMBEDDING, a, {{Slot::INPUT, x}}, name, inits)[0];
}

V GraphBuilder::multihead_attention(V q, V k, V v, int64_t embed_dim, int64_t num_heads, std::optional<int64_t> kdim,
                                    std::optional<int64_t> vdim, double dropout, bool bias, bool add_bias_kv,
                                    bool add_zero_attn, const OptInit &init, const std::string &name) {
  if (add_bias_kv || add_zero_attn) throw Error("multihead_attention: add_bias_kv / add_zero_attn are not supported");
  Json a = Json::object();
  a["embed_dim"] = (long long)embed_dim;
  a["num_heads"] = (long long)num_heads;
  a["kdim"] = (long long)kdim.value_or(embed_dim / num_heads);
  a["vdim"] = (long long)vdim.value_or(embed_dim / num_heads);
  a["dropout"] = dropout;
  a["bias"] = bias;
  a["add_bias_kv"] = add_bias_kv;
  a["add_zero_attn"] = add_zero_attn;
  std::map<Slot, Json> inits;
  if (init) inits[Slot::WEIGHT] = *init;
  // (the reference wires KEY<-query and QUERY<-key, computation_graph_builder.cc:752-764; not repeated here)
  return add_layer(OpType::MULTIHEAD_ATTENTION, a, {{Slot::QUERY, q}, {Slot::KEY, k}, {Slot::VALUE, v}}, name, inits)[0];
}

V GraphBuilder::batch_matmul(V a_, V b_, const std::string &name) {
  return add_layer(OpType::BATCHMATMUL, Json::object(), {{Slot::LHS_INPUT, a_}, {Slot::RHS_INPUT, b_}}, name)[0];
}

V GraphBuilder::dropout(V x, double rate, uint64_t seed, const std::string &name) {
  Json a = Json::object();
  a["rate"] = rate;
  a["seed"] = (unsigned long long)seed;
  return add_layer(OpType::DROPOUT, a, {{Slot::INPUT, x}}, name)[0];
}

V GraphBuilder::softmax(V x, int dim, const std::string &name) {
  Json a = Json::object();
  a["dim"] = shape(x).norm_dim(dim);
  return add_layer(OpType::SOFTMAX, a, {{Slot::INPUT, x}}, name)[0];
}

V GraphBuilder::cast(V x, DataType dt, const std::string &name) {
  Json a = Json::object();
  a["dtype"] = to_string(dt);
  return add_layer(OpType::CAST, a, {{Slot::INPUT, x}}, name)[0];
}

V GraphBuilder::concat(const std::vector<V> &xs, int axis, const std::string &name) {
  if (xs.size() < 2) throw Error("concat: needs at least two inputs");
  Json a = Json::object();
  a["axis"] = shape(xs[0]).norm_dim(axis);
  a["num_inputs"] = (int)xs.size();
  std::vector<std::pair<Slot, V>> ins;
  for (size_t i = 0; i < xs.size(); ++i) ins.push_back({input_slot_n((int)i), xs[i]});
  return add_layer(OpType::CONCAT, a, ins, name)[0];
}

std::vector<V> GraphBuilder::split(V x, const std::vector<int64_t> &sizes, int axis, const std::string &name) {
  Json a = Json::object();
  a["splits"] = Json::from_ints(sizes);
  a["axis"] = shape(x).norm_dim(axis);
  return add_layer(OpType::SPLIT, a, {{Slot::INPUT, x}}, name);
}

V GraphBuilder::flat(V x, int start_dim, int end_dim, const std::string &name) {
  Json a = Json::object();
  a["start_dim"] = shape(x).norm_dim(start_dim);
  a["end_dim"] = shape(x).norm_dim(end_dim);
  return add_layer(OpType::FLAT, a, {{Slot::INPUT, x}}, name)[0];
}

V GraphBuilder::transpose(V x, const std::vector<int> &perm, const std::string &name) {
  Json a = Json::object();
  a["permutation"] = Json::from_ints(perm);
  return add_layer(OpType::TRANSPOSE, a, {{Slot::INPUT, x}}, name)[0];
}

V GraphBuilder::reshape(V x, const std::vector<int64_t> &dims, const std::string &name) {
  std::vector<int64_t> d = dims;
  int64_t known = 1, total = shape(x).num_elements();
  int infer = -1;
  for (size_t i = 0; i < d.size(); ++i) {
    if (d[i] == -1) infer = (int)i;
    else known *= d[i];
  }
  if (infer >= 0) d[infer] = total / known;
  Json a = Json::object();
  a["shape"] = plain_shape_json(d, shape(x).dtype);
  return add_layer(OpType::RESHAPE, a, {{Slot::INPUT, x}}, name)[0];
}

V GraphBuilder::reverse(V x, int axis, const std::string &name) {
  Json a = Json::object();
  a["axis"] = shape(x).norm_dim(axis);
  return add_layer(OpType::REVERSE, a, {{Slot::INPUT, x}}, name)[0];
}

V GraphBuilder::gather(V x, V index, int dim, const std::string &name) {
  Json a = Json::object();
  a["dim"] = shape(x).norm_dim(dim);
  return add_layer(OpType::GATHER, a, {{Slot::INPUT, x}, {Slot::INDEX, index}}, name)[0];
}

std::vector<V> GraphBuilder::top_k(V x, int k, bool sorted, const std::string &name) {
  Json a = Json::object();
  a["k"] = k;
  a["sorted"] = sorted;
  return add_layer(OpType::TOPK, a, {{Slot::INPUT, x}}, name);
}

V GraphBuilder::reduce(OpType t, V x, const std::vector<int> &axes, bool keepdims, const std::string &name) {
  Json a = Json::object();
  std::vector<int> ax;
  for (int v : axes) ax.push_back(shape(x).norm_dim(v));
  a["axes"] = Json::from_ints(ax);
  a["op_type"] = to_string(t);
  a["keepdims"] = keepdims;
  return add_layer(t, a, {{Slot::INPUT, x}}, name)[0];
}

V GraphBuilder::broadcast(V x, const std::vector<int64_t> &target, const std::string &name) {
  Json a = Json::object();
  Json td = Json::object();
  td["ff_ordered"] = Json::from_ints(target);
  a["target_dims"] = td;
  return add_layer(OpType::BROADCAST, a, {{Slot::INPUT, x}}, name)[0];
}

V GraphBuilder::noop(V x, const std::string &name) { return add_layer(OpType::NOOP, Json::object(), {{Slot::INPUT, x}}, name)[0]; }

static void need_parallel(bool p, const char *what) {
  if (!p) throw Error(std::string(what) + " is only available in a parallel computation graph");
}
V GraphBuilder::parallel_partition(V x, int dim, int degree, const std::string &name) {
  need_parallel(parallel_, "parallel_partition");
  Json a = Json::object();
  a["repartition_dim"] = shape(x).norm_dim(dim);
  a["repartition_degree"] = degree;
  return add_layer(OpType::REPARTITION, a, {{Slot::INPUT, x}}, name)[0];
}
V GraphBuilder::parallel_combine(V x, int dim, int degree, const std::string &name) {
  need_parallel(parallel_, "parallel_combine");
  Json a = Json::object();
  a["combine_dim"] = shape(x).norm_dim(dim);
  a["combine_degree"] = degree;
  return add_layer(OpType::COMBINE, a, {{Slot::INPUT, x}}, name)[0];
}
V GraphBuilder::parallel_replicate(V x, int degree, const std::string &name) {
  need_parallel(parallel_, "parallel_replicate");
  Json a = Json::object();
  a["replicate_degree"] = degree;
  return add_layer(OpType::REPLICATE, a, {{Slot::INPUT, x}}, name)[0];
}
V GraphBuilder::parallel_reduce(V x, int degree, const std::string &name) {
  need_parallel(parallel_, "parallel_reduce");
  Json a = Json::object();
  a["reduction_degree"] = degree;
  return add_layer(OpType::REDUCTION, a, {{Slot::INPUT, x}}, name)[0];
}

Graph pcg_from_computation_graph(const Graph &cg) {
  for (auto &kv : cg.nodes()) {
    if (is_parallel_op(kv.second.type)) throw Error("computation graph already contains parallel operators");
    for (auto &o : kv.second.outputs)
      if (!o.shape.is_unparallel()) throw Error("computation graph has a parallel tensor");
  }
  return cg;
}

}  // namespace ff
