#include "ir.h"

#include <algorithm>
#include <queue>
#include <sstream>

namespace ff {

// ---------------------------------------------------------------- enums
std::string to_string(DataType d) {
  switch (d) {
#define X(n) case DataType::n: return #n;
    FF_DATATYPES(X)
#undef X
  }
  return "?";
}
DataType datatype_from_string(const std::string &s) {
#define X(n) if (s == #n) return DataType::n;
  FF_DATATYPES(X)
#undef X
  throw Error("unknown DataType '" + s + "'");
}
int dtype_bytes(DataType d) {
  switch (d) {
    case DataType::BOOL: return 1;
    case DataType::INT32: return 4;
    case DataType::INT64: return 8;
    case DataType::HALF: return 2;
    case DataType::FLOAT: return 4;
    case DataType::DOUBLE: return 8;
    case DataType::BFLOAT16: return 2;
  }
  return 4;
}

bool tensor_dims_has_dim(const std::vector<int64_t> &dims, int idx) { return idx >= 0 && idx < (int)dims.size(); }
bool tensor_dims_is_broadcastable_to(const std::vector<int64_t> &curr, const std::vector<int64_t> &goal) {
  if (goal.size() < curr.size()) return false;
  const size_t off = goal.size() - curr.size();
  for (size_t i = 0; i < curr.size(); ++i)
    if (curr[i] != goal[off + i] && curr[i] != 1) return false;
  return true;
}
std::optional<std::vector<int64_t>> get_broadcast_target_dims(const std::vector<std::vector<int64_t>> &inputs) {
  for (auto &goal : inputs) {
    bool all = true;
    for (auto &d : inputs) all = all && tensor_dims_is_broadcastable_to(d, goal);
    if (all) return goal;
  }
  return std::nullopt;
}
std::vector<std::vector<int64_t>> get_tensor_dims_coord_set(const std::vector<int64_t> &dims) {
  std::vector<std::vector<int64_t>> out = {{}};
  for (int64_t d : dims) {
    std::vector<std::vector<int64_t>> next;
    for (auto &prefix : out)
      for (int64_t c = 0; c < d; ++c) {
        auto p = prefix;
        p.push_back(c);
        next.push_back(std::move(p));
      }
    out = std::move(next);
  }
  return out;
}
std::vector<int64_t> tensor_dims_drop_dims(const std::vector<int64_t> &dims, const std::function<bool(int)> &should_drop) {
  std::vector<int64_t> out;
  for (int i = 0; i < (int)dims.size(); ++i)
    if (!should_drop(i)) out.push_back(dims[i]);
  return out;
}
std::string to_string(OpType t) {
  switch (t) {
#define X(n) case OpType::n: return #n;
    FF_OPTYPES(X)
#undef X
  }
  return "?";
}
OpType optype_from_string(const std::string &s) {
#define X(n) if (s == #n) return OpType::n;
  FF_OPTYPES(X)
#undef X
  throw Error("unknown OperatorType '" + s + "'");
}
bool is_parallel_op(OpType t) {
  return t == OpType::REPARTITION || t == OpType::COMBINE || t == OpType::REPLICATE || t == OpType::REDUCTION;
}
bool is_element_unary(OpType t) {
  switch (t) {
    case OpType::RELU: case OpType::IDENTITY: case OpType::SIGMOID: case OpType::TANH: case OpType::ELU:
    case OpType::GELU: case OpType::EXP: case OpType::RSQRT: case OpType::SIN: case OpType::COS:
    case OpType::SCALAR_MULTIPLY: case OpType::SCALAR_ADD: case OpType::SCALAR_SUB: case OpType::SCALAR_TRUE_DIV:
    case OpType::SCALAR_FLOOR_DIV: case OpType::POW: case OpType::LOG: case OpType::SQRT: case OpType::CEIL:
    case OpType::ROUND: case OpType::LOGICAL_NOT: case OpType::LEAKYRELU:
      return true;
    default: return false;
  }
}
bool is_element_binary(OpType t) {
  switch (t) {
    case OpType::EW_ADD: case OpType::EW_SUB: case OpType::EW_MUL: case OpType::EW_DIV: case OpType::EW_MAX:
    case OpType::EW_MIN: case OpType::EW_EQUAL: case OpType::EW_GREATER: case OpType::EW_LESS:
      return true;
    default: return false;
  }
}
static bool is_reduce(OpType t) {
  switch (t) {
    case OpType::REDUCE_SUM: case OpType::REDUCE_MEAN: case OpType::REDUCE_MAX: case OpType::REDUCE_MIN:
    case OpType::REDUCE_PROD: case OpType::REDUCE_ARGMAX: case OpType::REDUCE_ARGMIN: case OpType::MEAN:
      return true;
    default: return false;
  }
}
std::string attrs_variant_key(OpType t) {
  if (is_element_unary(t)) return "element_unary";
  if (is_element_binary(t)) return "element_binary";
  if (is_reduce(t)) return "reduce";
  switch (t) {
    case OpType::BATCHMATMUL: return "batch_matmul";
    case OpType::BATCHNORM: return "batch_norm";
    case OpType::BROADCAST: return "broadcast";
    case OpType::CAST: return "cast";
    case OpType::COMBINE: return "combine";
    case OpType::CONCAT: return "concat";
    case OpType::CONV2D: return "conv2d";
    case OpType::DROPOUT: return "dropout";
    case OpType::EMBEDDING: return "embedding";
    case OpType::FLAT: return "flat";
    case OpType::GATHER: return "gather";
    case OpType::INPUT: return "input";
    case OpType::LAYERNORM: return "layer_norm";
    case OpType::LINEAR: return "linear";
    case OpType::MULTIHEAD_ATTENTION: return "multi_head_attention";
    case OpType::NOOP: return "noop";
    case OpType::POOL2D: return "pool2d";
    case OpType::REDUCTION: return "reduction";
    case OpType::REPARTITION: return "repartition";
    case OpType::REPLICATE: return "replicate";
    case OpType::RESHAPE: return "reshape";
    case OpType::REVERSE: return "reverse";
    case OpType::SOFTMAX: return "softmax";
    case OpType::SPLIT: return "split";
    case OpType::TOPK: return "topk";
    case OpType::TRANSPOSE: return "transpose";
    case OpType::WEIGHT: return "weight";
    default: return "noop";
  }
}
static OpType optype_from_variant(const std::string &key, const Json &value) {
  if (key == "element_unary") return optype_from_string(value.at("op_type").as_string());
  if (key == "element_binary") return optype_from_string(value.at("type").as_string());
  if (key == "reduce") return optype_from_string(value.at("op_type").as_string());
  static const std::map<std::string, OpType> m = {
      {"batch_matmul", OpType::BATCHMATMUL}, {"batch_norm", OpType::BATCHNORM}, {"broadcast", OpType::BROADCAST},
      {"cast", OpType::CAST}, {"combine", OpType::COMBINE}, {"concat", OpType::CONCAT}, {"conv2d", OpType::CONV2D},
      {"dropout", OpType::DROPOUT}, {"embedding", OpType::EMBEDDING}, {"flat", OpType::FLAT},
      {"gather", OpType::GATHER}, {"input", OpType::INPUT}, {"layer_norm", OpType::LAYERNORM},
      {"linear", OpType::LINEAR}, {"multi_head_attention", OpType::MULTIHEAD_ATTENTION}, {"noop", OpType::NOOP},
      {"pool2d", OpType::POOL2D}, {"reduction", OpType::REDUCTION}, {"repartition", OpType::REPARTITION},
      {"replicate", OpType::REPLICATE}, {"reshape", OpType::RESHAPE}, {"reverse", OpType::REVERSE},
      {"softmax", OpType::SOFTMAX}, {"split", OpType::SPLIT}, {"topk", OpType::TOPK},
      {"transpose", OpType::TRANSPOSE}, {"weight", OpType::WEIGHT}};
  auto it = m.find(key);
  if (it == m.end()) throw Error("unknown op attrs variant '" + key + "'");
  return it->second;
}

std::string to_string(Slot s) {
  switch (s) {
#define X(n) case Slot::n: return #n;
    FF_SLOTS(X)
#undef X
  }
  return "?";
}
Slot slot_from_string(const std::string &s) {
#define X(n) if (s == #n) return Slot::n;
  FF_SLOTS(X)
#undef X
  throw Error("unknown TensorSlotName '" + s + "'");
}
Slot input_slot_n(int i) {
  if (i < 0 || i > 7) throw Error("at most 8 numbered inputs");
  return (Slot)((int)Slot::INPUT_0 + i);
}
Slot output_slot_n(int i) {
  if (i < 0 || i > 5) throw Error("at most 6 numbered outputs");
  return (Slot)((int)Slot::OUTPUT_0 + i);
}

// ---------------------------------------------------------------- PShape
PShape PShape::make(const std::vector<int64_t> &sizes, DataType dt) {
  PShape s;
  for (auto v : sizes) {
    if (v <= 0) throw Error("tensor dims must be positive");
    s.dims.push_back({v, 1});
  }
  s.dtype = dt;
  return s;
}
int PShape::norm_dim(int d) const {
  int n = ndim();
  if (d < 0) d += n;
  if (d < 0 || d >= n) throw Error("dim index out of range");
  return d;
}
std::vector<int64_t> PShape::sizes() const {
  std::vector<int64_t> r;
  for (auto &d : dims) r.push_back(d.size);
  return r;
}
std::vector<int> PShape::degrees() const {
  std::vector<int> r;
  for (auto &d : dims) r.push_back(d.degree);
  return r;
}
std::vector<int64_t> PShape::piece_sizes() const {
  std::vector<int64_t> r;
  for (auto &d : dims) {
    if (d.size % d.degree != 0) throw Error("shard degree does not divide dim size in " + str());
    r.push_back(d.size / d.degree);
  }
  return r;
}
int64_t PShape::num_elements() const {
  int64_t n = 1;
  for (auto &d : dims) n *= d.size;
  return n;
}
int64_t PShape::piece_elements() const {
  int64_t n = 1;
  for (auto &d : dims) n *= (d.size + d.degree - 1) / d.degree;
  return n;
}
int PShape::total_degree() const {
  int n = sum_degree * discard_copy_degree;
  for (auto &d : dims) n *= d.degree;
  return n;
}
PShape PShape::reduced() const {
  PShape s = *this;
  for (auto &d : s.dims) d.degree = 1;
  s.sum_degree = 1;
  s.discard_copy_degree = 1;
  return s;
}
std::string PShape::str() const {
  std::ostringstream o;
  o << to_string(dtype) << "[";
  for (size_t i = 0; i < dims.size(); ++i) {
    if (i) o << ",";
    o << dims[i].size;
    if (dims[i].degree != 1) o << "/" << dims[i].degree;
  }
  o << "]";
  if (sum_degree != 1) o << " sum=" << sum_degree;
  if (discard_copy_degree != 1) o << " copy=" << discard_copy_degree;
  return o.str();
}
Json PShape::to_json_parallel() const {
  Json shard = Json::array();
  for (auto &d : dims) {
    Json e = Json::object();
    e["size"] = (long long)d.size;
    e["degree"] = d.degree;
    shard.push_back(e);
  }
  Json rep = Json::object();
  rep["sum_degree"] = sum_degree;
  rep["discard_copy_degree"] = discard_copy_degree;
  Json pd = Json::object();
  pd["shard_dims"] = shard;
  pd["replica_dims"] = rep;
  Json j = Json::object();
  j["dims"] = pd;
  j["data_type"] = to_string(dtype);
  return j;
}
Json PShape::to_json_plain() const {
  Json td = Json::object();
  td["ff_ordered"] = Json::from_ints(sizes());
  Json j = Json::object();
  j["dims"] = td;
  j["data_type"] = to_string(dtype);
  return j;
}
PShape PShape::from_json(const Json &j) {
  PShape s;
  s.dtype = datatype_from_string(j.at("data_type").as_string());
  const Json &d = j.at("dims");
  if (d.contains("ff_ordered")) {
    for (auto v : d.at("ff_ordered").as_ints()) s.dims.push_back({v, 1});
  } else {
    for (auto &e : d.at("shard_dims").items())
      s.dims.push_back({e.at("size").as_int(), (int)e.at("degree").as_int()});
    const Json &r = d.at("replica_dims");
    s.sum_degree = (int)r.at("sum_degree").as_int();
    s.discard_copy_degree = (int)r.at("discard_copy_degree").as_int();
  }
  return s;
}

// ---------------------------------------------------------------- machine
Json MachineSpec::to_json() const {
  Json c = Json::object();
  c["num_nodes"] = num_nodes;
  c["num_cpus_per_node"] = num_cpus_per_node;
  c["num_gpus_per_node"] = num_gpus_per_node;
  Json i = Json::object();
  i["inter_node_bandwidth"] = inter_node_bandwidth;
  i["intra_node_bandwidth"] = intra_node_bandwidth;
  Json j = Json::object();
  j["compute_specification"] = c;
  j["interconnect_specification"] = i;
  return j;
}
MachineSpec MachineSpec::from_json(const Json &j) {
  MachineSpec m;
  const Json &c = j.contains("compute_specification") ? j.at("compute_specification") : j;
  m.num_nodes = (int)c.get_int("num_nodes", 1);
  m.num_cpus_per_node = (int)c.get_int("num_cpus_per_node", 1);
  m.num_gpus_per_node = (int)c.get_int("num_gpus_per_node", 1);
  const Json &i = j.contains("interconnect_specification") ? j.at("interconnect_specification") : j;
  m.inter_node_bandwidth = i.get_float("inter_node_bandwidth", m.inter_node_bandwidth);
  m.intra_node_bandwidth = i.get_float("intra_node_bandwidth", m.intra_node_bandwidth);
  return m;
}
Json MachineView::to_json() const {
  Json s = Json::object();
  s["node_idx"] = start_node;
  s["device_idx"] = start_device;
  s["device_type"] = "GPU";
  Json d = Json::array();
  for (auto &x : dims) {
    Json e = Json::object();
    e["stride"] = x.stride;
    e["projection"] = x.inter_node ? "INTER_NODE" : "INTRA_NODE";
    d.push_back(e);
  }
  Json j = Json::object();
  j["start"] = s;
  j["dimensions"] = d;
  return j;
}
MachineView MachineView::from_json(const Json &j) {
  MachineView v;
  v.start_node = (int)j.at("start").get_int("node_idx", 0);
  v.start_device = (int)j.at("start").get_int("device_idx", 0);
  for (auto &e : j.at("dimensions").items())
    v.dims.push_back({(int)e.at("stride").as_int(), e.at("projection").as_string() == "INTER_NODE"});
  return v;
}
std::string MachineView::str() const {
  std::ostringstream o;
  o << "@(" << start_node << "," << start_device << ")";
  for (auto &d : dims) o << (d.inter_node ? " N" : " D") << "x" << d.stride;
  return o.str();
}

// ---------------------------------------------------------------- Graph
const OutValue &Node::out(Slot s) const {
  for (auto &o : outputs) if (o.slot == s) return o;
  throw Error("node '" + name + "' (" + to_string(type) + ") has no output slot " + to_string(s));
}
const InEdge *Node::in(Slot s) const {
  for (auto &e : inputs) if (e.dst_slot == s) return &e;
  return nullptr;
}
NodeId Graph::add_node(OpType type, Json attrs, std::string name, std::vector<InEdge> inputs,
                       std::vector<OutValue> outputs) {
  for (auto &e : inputs) {
    if (!has_node(e.src.node)) throw Error("add_node: input refers to a node that does not exist");
    node(e.src.node).out(e.src.slot);  // validates the slot
  }
  NodeId id = next_id_++;
  Node n;
  n.type = type;
  n.attrs = attrs.is_null() ? Json::object() : std::move(attrs);
  n.name = std::move(name);
  n.inputs = std::move(inputs);
  n.outputs = std::move(outputs);
  nodes_.emplace(id, std::move(n));
  return id;
}
void Graph::remove_node(NodeId id) {
  for (auto &kv : nodes_)
    for (auto &e : kv.second.inputs)
      if (e.src.node == id && kv.first != id) throw Error("remove_node: node still has consumers");
  nodes_.erase(id);
}
const Node &Graph::node(NodeId n) const {
  auto it = nodes_.find(n);
  if (it == nodes_.end()) throw Error("no such node " + std::to_string(n));
  return it->second;
}
Node &Graph::node(NodeId n) {
  auto it = nodes_.find(n);
  if (it == nodes_.end()) throw Error("no such node " + std::to_string(n));
  return it->second;
}
std::vector<NodeId> Graph::node_ids() const {
  std::vector<NodeId> r;
  for (auto &kv : nodes_) r.push_back(kv.first);
  return r;
}
std::vector<NodeId> Graph::topological_order() const {
  std::map<NodeId, int> indeg;
  std::map<NodeId, std::vector<NodeId>> succ;
  for (auto &kv : nodes_) {
    std::set<NodeId> preds;
    for (auto &e : kv.second.inputs) preds.insert(e.src.node);
    indeg[kv.first] = (int)preds.size();
    for (auto p : preds) succ[p].push_back(kv.first);
  }
  // smallest-id-first keeps the order deterministic and close to construction order
  std::priority_queue<NodeId, std::vector<NodeId>, std::greater<NodeId>> ready;
  for (auto &kv : indeg) if (kv.second == 0) ready.push(kv.first);
  std::vector<NodeId> order;
  while (!ready.empty()) {
    NodeId n = ready.top();
    ready.pop();
    order.push_back(n);
    for (auto s : succ[n]) if (--indeg[s] == 0) ready.push(s);
  }
  if (order.size() != nodes_.size()) throw Error("graph has a cycle");
  return order;
}
std::vector<std::pair<NodeId, Slot>> Graph::consumers(const ValueRef &v) const {
  std::vector<std::pair<NodeId, Slot>> r;
  for (auto &kv : nodes_)
    for (auto &e : kv.second.inputs)
      if (e.src == v) r.push_back({kv.first, e.dst_slot});
  return r;
}
std::vector<NodeId> Graph::successors(NodeId n) const {
  std::set<NodeId> r;
  for (auto &kv : nodes_)
    for (auto &e : kv.second.inputs)
      if (e.src.node == n) r.insert(kv.first);
  return {r.begin(), r.end()};
}
std::vector<NodeId> Graph::predecessors(NodeId n) const {
  std::set<NodeId> r;
  for (auto &e : node(n).inputs) r.insert(e.src.node);
  return {r.begin(), r.end()};
}
std::vector<ValueRef> Graph::all_values() const {
  std::vector<ValueRef> r;
  for (auto &kv : nodes_)
    for (auto &o : kv.second.outputs) r.push_back({kv.first, o.slot});
  return r;
}
std::vector<ValueRef> Graph::sink_values() const {
  std::set<ValueRef> used;
  for (auto &kv : nodes_)
    for (auto &e : kv.second.inputs) used.insert(e.src);
  std::vector<ValueRef> r;
  for (auto &v : all_values()) if (!used.count(v)) r.push_back(v);
  return r;
}
void Graph::replace_uses(const ValueRef &from, const ValueRef &to) {
  for (auto &kv : nodes_)
    for (auto &e : kv.second.inputs)
      if (e.src == from) e.src = to;
}
bool Graph::is_mapped() const {
  for (auto &kv : nodes_) if (!kv.second.view) return false;
  return !nodes_.empty();
}
std::string Graph::signature() const {
  // Multiset of per-node labels, each extended with the labels of its producers:
  // invariant under renumbering, cheap, and distinguishes the graphs a search visits
  // (the reference dedupes on a layer-signature multiset hash,
  // lib/compiler/src/compiler/unity_algorithm/graph_optimize_state.cc).
  std::map<NodeId, std::string> label;
  for (auto n : topological_order()) {
    const Node &nd = node(n);
    std::string l = to_string(nd.type) + nd.attrs.canonical();
    for (auto &o : nd.outputs) l += "|" + o.shape.str();
    std::vector<std::string> ins;
    for (auto &e : nd.inputs) ins.push_back(to_string(e.dst_slot) + "<" + std::to_string(std::hash<std::string>{}(label[e.src.node])) + ":" + to_string(e.src.slot));
    std::sort(ins.begin(), ins.end());
    for (auto &s : ins) l += ";" + s;
    if (nd.view) l += nd.view->str();
    label[n] = l;
  }
  std::vector<size_t> hs;
  for (auto &kv : label) hs.push_back(std::hash<std::string>{}(kv.second));
  std::sort(hs.begin(), hs.end());
  std::string out;
  for (auto h : hs) out += std::to_string(h) + ",";
  return out;
}
std::string Graph::as_dot() const {
  std::ostringstream o;
  o << "digraph G {\n  node [shape=record, fontsize=10];\n";
  for (auto &kv : nodes_) {
    const Node &n = kv.second;
    o << "  n" << kv.first << " [label=\"{" << to_string(n.type);
    if (!n.name.empty()) o << "|" << n.name;
    for (auto &out : n.outputs) o << "|" << to_string(out.slot) << ": " << out.shape.str();
    if (n.view) o << "|" << n.view->str();
    o << "}\"";
    if (is_parallel_op(n.type)) o << ", style=filled, fillcolor=lightblue";
    o << "];\n";
  }
  for (auto &kv : nodes_)
    for (auto &e : kv.second.inputs)
      o << "  n" << e.src.node << " -> n" << kv.first << " [label=\"" << to_string(e.src.slot) << "->"
        << to_string(e.dst_slot) << "\", fontsize=8];\n";
  o << "}\n";
  return o.str();
}

// ---------------------------------------------------------------- v1 file format
Json graph_to_v1(const Graph &g, bool parallel) {
  Json node_labels = Json::array(), output_labels = Json::array(), nodes = Json::array(), edges = Json::array(),
       outputs = Json::array(), views = Json::array();
  bool any_view = false;
  for (auto &kv : g.nodes()) {
    const Node &n = kv.second;
    nodes.push_back(kv.first);
    Json op = Json::object();
    op["type"] = attrs_variant_key(n.type);
    op["value"] = n.attrs;
    Json layer = Json::object();
    layer["op_attrs"] = op;
    layer["name"] = n.name.empty() ? Json() : Json(n.name);
    Json pair = Json::array();
    pair.push_back(kv.first);
    pair.push_back(layer);
    node_labels.push_back(pair);
    for (auto &o : n.outputs) {
      Json ref = Json::object();
      ref["node"] = kv.first;
      ref["slot_name"] = to_string(o.slot);
      outputs.push_back(ref);
      Json ta = Json::object();
      ta["shape"] = parallel ? o.shape.to_json_parallel() : o.shape.to_json_plain();
      ta["create_grad"] = o.create_grad ? "YES" : "NO";
      Json p2 = Json::array();
      p2.push_back(ref);
      p2.push_back(ta);
      output_labels.push_back(p2);
    }
    for (auto &e : n.inputs) {
      Json ed = Json::object();
      ed["srcNode"] = e.src.node;
      ed["srcSlot"] = to_string(e.src.slot);
      ed["dstNode"] = kv.first;
      ed["dstSlot"] = to_string(e.dst_slot);
      edges.push_back(ed);
    }
    if (n.view) {
      any_view = true;
      Json p3 = Json::array();
      p3.push_back(kv.first);
      p3.push_back(n.view->to_json());
      views.push_back(p3);
    }
  }
  Json graph = Json::object();
  graph["nodes"] = nodes;
  graph["edges"] = edges;
  graph["outputs"] = outputs;
  Json raw = Json::object();
  raw["node_labels"] = node_labels;
  raw["output_labels"] = output_labels;
  raw["graph"] = graph;
  Json j = Json::object();
  j["raw_graph"] = raw;
  if (any_view) j["machine_views"] = views;
  return j;
}

Graph graph_from_v1(const Json &j) {
  const Json &raw = j.contains("raw_graph") ? j.at("raw_graph") : (j.contains("pcg") ? j.at("pcg").at("raw_graph") : j);
  struct Tmp {
    OpType type;
    Json attrs;
    std::string name;
    std::vector<std::pair<Slot, std::pair<int, Slot>>> ins;
    std::vector<OutValue> outs;
  };
  std::map<int, Tmp> tmp;
  for (auto &p : raw.at("node_labels").items()) {
    int id = (int)p[0].as_int();
    const Json &layer = p[1];
    const Json &op = layer.at("op_attrs");
    Tmp t;
    t.attrs = op.at("value");
    t.type = optype_from_variant(op.at("type").as_string(), t.attrs);
    if (layer.contains("name") && layer.at("name").is_string()) t.name = layer.at("name").as_string();
    tmp[id] = t;
  }
  for (auto &p : raw.at("output_labels").items()) {
    int id = (int)p[0].at("node").as_int();
    OutValue o;
    o.slot = slot_from_string(p[0].at("slot_name").as_string());
    o.shape = PShape::from_json(p[1].at("shape"));
    const Json &cg = p[1].at("create_grad");
    o.create_grad = cg.is_bool() ? cg.as_bool() : cg.as_string() == "YES";
    tmp.at(id).outs.push_back(o);
  }
  for (auto &e : raw.at("graph").at("edges").items()) {
    int dst = (int)e.at("dstNode").as_int();
    tmp.at(dst).ins.push_back({slot_from_string(e.at("dstSlot").as_string()),
                               {(int)e.at("srcNode").as_int(), slot_from_string(e.at("srcSlot").as_string())}});
  }
  // the file must be closed under its own references: every value an edge reads and every value the graph lists as an
  // output has a label (shape), and every endpoint is a labelled node
  auto has_output = [&](int node, Slot slot) {
    auto it = tmp.find(node);
    if (it == tmp.end()) return false;
    for (auto &o : it->second.outs)
      if (o.slot == slot) return true;
    return false;
  };
  for (auto &kv : tmp)
    for (auto &in : kv.second.ins)
      if (!has_output(in.second.first, in.second.second))
        throw Error("v1 graph: node " + std::to_string(kv.first) + " reads output " + to_string(in.second.second) + " of node " +
                    std::to_string(in.second.first) + ", which has no output label");
  if (raw.at("graph").contains("outputs"))
    for (auto &o : raw.at("graph").at("outputs").items())
      if (!has_output((int)o.at("node").as_int(), slot_from_string(o.at("slot_name").as_string())))
        throw Error("v1 graph: output " + o.at("slot_name").as_string() + " of node " + std::to_string((int)o.at("node").as_int()) +
                    " is listed by the graph but has no output label");
  // insert in dependency order, remembering the id translation
  std::map<int, NodeId> remap;
  Graph g;
  std::set<int> pending;
  for (auto &kv : tmp) pending.insert(kv.first);
  while (!pending.empty()) {
    bool progressed = false;
    for (auto it = pending.begin(); it != pending.end();) {
      Tmp &t = tmp[*it];
      bool ready = true;
      for (auto &in : t.ins) if (!remap.count(in.second.first)) ready = false;
      if (!ready) { ++it; continue; }
      std::vector<InEdge> ins;
      for (auto &in : t.ins) ins.push_back({in.first, {remap[in.second.first], in.second.second}});
      remap[*it] = g.add_node(t.type, t.attrs, t.name, ins, t.outs);
      it = pending.erase(it);
      progressed = true;
    }
    if (!progressed) throw Error("v1 graph has a cycle or a dangling edge");
  }
  if (j.contains("machine_views"))
    for (auto &p : j.at("machine_views").items())
      g.node(remap.at((int)p[0].as_int())).view = MachineView::from_json(p[1]);
  return g;
}

}  // namespace ff
