#include "substitutions.h"

#include <algorithm>
#include <functional>
#include <set>
#include <sstream>

#include "pyjson.h"

namespace ff {

// ---------------------------------------------------------------- constraint evaluation
static Json node_attribute(const Node &n, const std::string &key) {
  if (key == "op_type") return Json(to_string(n.type));
  if (n.attrs.contains(key)) return n.attrs.at(key);
  return Json();
}
static bool constraint_holds(const AttrConstraint &c, const Node &n) {
  Json v = node_attribute(n, c.key);
  if (c.kind == AttrConstraint::EQUAL) return v == c.value;
  if (!v.is_number() || !c.value.is_number()) return false;
  long long d = c.value.as_int();
  return d != 0 && v.as_int() % d == 0;
}
static bool tensor_constraint_holds(const TensorConstraint &c, const PShape &s) {
  auto dim_ok = [&](int d) { return (d >= 0 ? d : d + s.ndim()) >= 0 && (d >= 0 ? d : d + s.ndim()) < s.ndim(); };
  switch (c.kind) {
    case TensorConstraint::NUM_DIMS_AT_LEAST: return s.ndim() >= c.value;
    case TensorConstraint::DIM_DIVISIBLE_BY: {
      if (!dim_ok(c.dim)) return false;
      const ShardDim &d = s.dims[s.norm_dim(c.dim)];
      return (d.size / d.degree) % c.value == 0 && d.size % (d.degree * c.value) == 0;
    }
    case TensorConstraint::DIM_DEGREE_EQUAL:
      if (!dim_ok(c.dim)) return false;
      return s.dims[s.norm_dim(c.dim)].degree == c.value;
    case TensorConstraint::SUM_DEGREE_EQUAL: return s.sum_degree == c.value;
    case TensorConstraint::COPY_DEGREE_EQUAL: return s.discard_copy_degree == c.value;
  }
  return false;
}

// ---------------------------------------------------------------- validity
bool is_valid_substitution(const Substitution &s, std::string *why) {
  auto fail = [&](const std::string &m) { if (why) *why = m; return false; };
  if (s.pattern.nodes.empty()) return fail("empty pattern");
  for (size_t i = 0; i < s.pattern.nodes.size(); ++i)
    for (auto &in : s.pattern.nodes[i].inputs) {
      if (in.from_graph_input) { if (in.index < 0 || in.index >= s.pattern.num_inputs) return fail("pattern input index out of range"); }
      else if (in.index < 0 || in.index >= (int)s.pattern.nodes.size() || in.index == (int)i) return fail("pattern edge refers to a bad node");
    }
  for (size_t i = 0; i < s.out_nodes.size(); ++i) {
    auto &o = s.out_nodes[i];
    if (o.template_node && (*o.template_node < 0 || *o.template_node >= (int)s.pattern.nodes.size())) return fail("bad template node");
    for (auto &in : o.inputs) {
      if (in.from_graph_input) { if (in.index < 0 || in.index >= s.pattern.num_inputs) return fail("output graph uses an input the pattern lacks"); }
      else if (in.index < 0 || in.index >= (int)i) return fail("output graph nodes must be listed in dependency order");
    }
  }
  if (s.outputs.empty()) return fail("substitution has no interface outputs");
  for (auto &io : s.outputs) {
    if (io.pattern_node < 0 || io.pattern_node >= (int)s.pattern.nodes.size()) return fail("interface refers to a bad pattern node");
    if (io.out_node >= (int)s.out_nodes.size()) return fail("interface refers to a bad output node");
  }
  return true;
}

// ---------------------------------------------------------------- matching
std::vector<Match> find_pattern_matches(const Pattern &p, const Graph &g) {
  std::vector<Match> result;
  const int np = (int)p.nodes.size();
  // candidate graph nodes per pattern node (operator constraints only)
  std::vector<std::vector<NodeId>> cand(np);
  for (int i = 0; i < np; ++i)
    for (auto &kv : g.nodes()) {
      bool ok = true;
      for (auto &c : p.nodes[i].constraints) if (!constraint_holds(c, kv.second)) { ok = false; break; }
      if (ok) cand[i].push_back(kv.first);
    }
  // order pattern nodes so that each one after the first is adjacent to an earlier one when possible
  Match cur;
  cur.nodes.assign(np, -1);
  cur.inputs.assign(p.num_inputs, ValueRef{-1, Slot::OUTPUT});
  std::vector<bool> input_bound(p.num_inputs, false);

  std::function<bool(int, NodeId, std::vector<int> &)> bind_node = [&](int pi, NodeId gn, std::vector<int> &bound_inputs) {
    const Node &n = g.node(gn);
    const PatternNode &pn = p.nodes[pi];
    if (!pn.allow_extra_inputs && n.inputs.size() != pn.inputs.size()) return false;
    for (auto &in : pn.inputs) {
      const InEdge *e = n.in(in.slot);
      if (!e) return false;
      if (in.from_graph_input) {
        if (input_bound[in.index]) {
          if (!(cur.inputs[in.index] == e->src)) return false;
        } else {
          auto it = p.input_constraints.find(in.index);
          if (it != p.input_constraints.end())
            for (auto &tc : it->second) if (!tensor_constraint_holds(tc, g.shape(e->src))) return false;
          cur.inputs[in.index] = e->src;
          input_bound[in.index] = true;
          bound_inputs.push_back(in.index);
        }
      } else {
        NodeId want = cur.nodes[in.index];
        if (want >= 0) { if (e->src.node != want || e->src.slot != in.src_slot) return false; }
        else if (e->src.slot != in.src_slot) return false;
      }
    }
    return true;
  };

  std::function<void(int)> rec = [&](int pi) {
    if (pi == np) {
      // edges to later-bound nodes were only checked on slots; verify all internal edges now
      for (int i = 0; i < np; ++i)
        for (auto &in : p.nodes[i].inputs)
          if (!in.from_graph_input) {
            const InEdge *e = g.node(cur.nodes[i]).in(in.slot);
            if (!e || e->src.node != cur.nodes[in.index] || e->src.slot != in.src_slot) return;
          }
      // graph inputs must come from outside the match
      std::set<NodeId> matched(cur.nodes.begin(), cur.nodes.end());
      for (auto &v : cur.inputs) if (matched.count(v.node)) return;
      result.push_back(cur);
      return;
    }
    for (NodeId gn : cand[pi]) {
      bool used = false;
      for (int j = 0; j < pi; ++j) if (cur.nodes[j] == gn) used = true;
      if (used) continue;
      std::vector<int> bound;
      cur.nodes[pi] = gn;
      if (bind_node(pi, gn, bound)) rec(pi + 1);
      for (int b : bound) input_bound[b] = false;
      cur.nodes[pi] = -1;
    }
  };
  rec(0);
  return result;
}

// ---------------------------------------------------------------- application
std::optional<Graph> apply_substitution(const Graph &g, const Substitution &s, const Match &m, std::string *why) {
  auto fail = [&](const std::string &msg) -> std::optional<Graph> { if (why) *why = msg; return std::nullopt; };
  std::set<NodeId> matched(m.nodes.begin(), m.nodes.end());
  // interior values (not exported through the interface) must have no consumers outside the match
  std::set<ValueRef> exported;
  for (auto &io : s.outputs) exported.insert({m.nodes[io.pattern_node], io.pattern_slot});
  for (NodeId n : m.nodes)
    for (auto &o : g.node(n).outputs) {
      ValueRef v{n, o.slot};
      if (exported.count(v)) continue;
      for (auto &c : g.consumers(v)) if (!matched.count(c.first)) return fail("interior value is used outside the match");
    }
  Graph out = g;
  std::vector<NodeId> new_ids;
  try {
    for (size_t i = 0; i < s.out_nodes.size(); ++i) {
      const OutNode &on = s.out_nodes[i];
      OpType type = on.type;
      Json attrs = Json::object();
      std::string name;
      if (on.template_node) {
        const Node &t = g.node(m.nodes[*on.template_node]);
        type = t.type;
        attrs = t.attrs;
        name = t.name;
      }
      for (auto &kv : on.assigns) {
        Json v = kv.second.kind == AttrExpr::LITERAL ? kv.second.literal
                                                     : node_attribute(g.node(m.nodes[kv.second.pattern_node]), kv.second.key);
        if (kv.first == "op_type") type = optype_from_string(v.as_string());
        else attrs[kv.first] = v;
      }
      std::vector<InEdge> ins;
      SlotShapes data_shapes;
      for (auto &in : on.inputs) {
        ValueRef src = in.from_graph_input ? m.inputs[in.index] : ValueRef{new_ids[in.index], in.src_slot};
        ins.push_back({in.slot, src});
        if (!is_weight_slot(type, in.slot)) data_shapes.push_back({in.slot, out.shape(src)});
      }
      if (on.template_node && s.pattern.nodes[*on.template_node].allow_extra_inputs) {
        // inputs of the matched operator that the pattern did not name (an optional BIAS) carry over unchanged
        for (auto &e : g.node(m.nodes[*on.template_node]).inputs) {
          bool present = false;
          for (auto &x : ins) if (x.dst_slot == e.dst_slot) present = true;
          if (!present && !matched.count(e.src.node)) ins.push_back({e.dst_slot, e.src});
        }
      }
      Inferred inf = infer_shapes(type, attrs, data_shapes);
      // weight inputs must have the shard layout the operator expects (replication may be split between
      // sum and discard-copy degrees, see GraphBuilder::weight_for)
      for (auto &w : inf.weights) {
        const InEdge *e = nullptr;
        for (auto &x : ins) if (x.dst_slot == w.first) e = &x;
        if (!e) return fail("output operator lacks weight slot " + to_string(w.first));
        const PShape &have = out.shape(e->src);
        if (have.dims != w.second.dims ||
            have.sum_degree * have.discard_copy_degree != w.second.sum_degree * w.second.discard_copy_degree)
          return fail("weight slot " + to_string(w.first) + " has shape " + have.str() + ", expected " + w.second.str());
      }
      std::vector<OutValue> outs;
      for (auto &o : inf.outputs) outs.push_back({o.first, o.second, true});
      new_ids.push_back(out.add_node(type, attrs, name, ins, outs));
    }
  } catch (const std::exception &e) {
    return fail(e.what());
  }
  std::set<NodeId> keep_even_if_unused;  // new producers of values that were graph outputs before the rewrite
  for (auto &io : s.outputs) {
    ValueRef old_v{m.nodes[io.pattern_node], io.pattern_slot};
    ValueRef new_v = io.out_node < 0 ? m.inputs[-io.out_node - 1] : ValueRef{new_ids[io.out_node], io.out_slot};
    if (io.out_node >= 0 && g.consumers(old_v).empty()) keep_even_if_unused.insert(new_ids[io.out_node]);
    if (out.shape(old_v) != out.shape(new_v))
      return fail("interface shape changes from " + out.shape(old_v).str() + " to " + out.shape(new_v).str());
    out.replace_uses(old_v, new_v);
  }
  // remove the matched nodes, consumers first
  std::vector<NodeId> order = g.topological_order();
  for (auto it = order.rbegin(); it != order.rend(); ++it)
    if (matched.count(*it)) {
      try { out.remove_node(*it); } catch (const std::exception &e) { return fail(e.what()); }
    }
  // sweep parallel operators that the rewrite left without consumers
  bool swept = true;
  while (swept) {
    swept = false;
    for (NodeId n : new_ids) {  // only operators this rewrite created: a model output may legitimately end in a Combine
      if (!out.has_node(n) || keep_even_if_unused.count(n)) continue;
      const Node &nd = out.node(n);
      if (!is_parallel_op(nd.type)) continue;
      bool used = false;
      for (auto &o : nd.outputs) if (!out.consumers({n, o.slot}).empty()) used = true;
      if (!used) { out.remove_node(n); swept = true; }
    }
  }
  return out;
}

// ---------------------------------------------------------------- rule builders
namespace {
AttrConstraint op_is(OpType t) { return {AttrConstraint::EQUAL, "op_type", Json(to_string(t))}; }
AttrConstraint attr_eq(const std::string &k, Json v) { return {AttrConstraint::EQUAL, k, std::move(v)}; }
AttrConstraint attr_div(const std::string &k, long long d) { return {AttrConstraint::DIVISIBLE_BY, k, Json(d)}; }
PatternInput gin(Slot s, int idx) { return {s, true, idx, Slot::OUTPUT}; }
PatternInput nin(Slot s, int node, Slot src = Slot::OUTPUT) { return {s, false, node, src}; }
OutInput ogin(Slot s, int idx) { return {s, true, idx, Slot::OUTPUT}; }
OutInput onin(Slot s, int node, Slot src = Slot::OUTPUT) { return {s, false, node, src}; }
AttrExpr lit(Json v) { AttrExpr e; e.kind = AttrExpr::LITERAL; e.literal = std::move(v); return e; }

OutNode parallel_node(OpType t, std::map<std::string, AttrExpr> a, OutInput in) {
  OutNode n;
  n.type = t;
  n.assigns = std::move(a);
  n.inputs = {in};
  return n;
}
OutNode repartition(OutInput in, int dim, int degree) {
  return parallel_node(OpType::REPARTITION, {{"repartition_dim", lit(dim)}, {"repartition_degree", lit(degree)}}, in);
}
OutNode combine(OutInput in, int dim, int degree) {
  return parallel_node(OpType::COMBINE, {{"combine_dim", lit(dim)}, {"combine_degree", lit(degree)}}, in);
}
OutNode replicate(OutInput in, int degree) { return parallel_node(OpType::REPLICATE, {{"replicate_degree", lit(degree)}}, in); }
OutNode reduction(OutInput in, int degree) { return parallel_node(OpType::REDUCTION, {{"reduction_degree", lit(degree)}}, in); }
OutNode templated(int pattern_node, std::vector<OutInput> ins) {
  OutNode n;
  n.template_node = pattern_node;
  n.inputs = std::move(ins);
  return n;
}
std::string sfx(int a, int b = -1) { return "_" + std::to_string(a) + (b >= 0 ? "_" + std::to_string(b) : ""); }
}  // namespace

// Linear, column (out-channel) parallel: replicate the input, shard the weight's out dim, combine the
// output's last dim (unity_substitution_set.cc:186-267).
Substitution create_replicate_linear_combine(int degree, bool use_bias) {
  Substitution s;
  s.name = "replicate_linear_combine" + sfx(degree) + (use_bias ? "_bias" : "");
  PatternNode lin;
  lin.constraints = {op_is(OpType::LINEAR), attr_eq("use_bias", use_bias), attr_div("out_channels", degree)};
  lin.inputs = {gin(Slot::INPUT, 0), gin(Slot::WEIGHT, 1)};
  if (use_bias) lin.inputs.push_back(gin(Slot::BIAS, 2));
  s.pattern.nodes = {lin};
  s.pattern.num_inputs = use_bias ? 3 : 2;
  s.pattern.input_constraints[0] = {{TensorConstraint::COPY_DEGREE_EQUAL, 0, 1}, {TensorConstraint::SUM_DEGREE_EQUAL, 0, 1}};
  s.out_nodes.push_back(replicate(ogin(Slot::INPUT, 0), degree));                 // 0
  s.out_nodes.push_back(repartition(ogin(Slot::INPUT, 1), 0, degree));            // 1
  std::vector<OutInput> ins = {onin(Slot::INPUT, 0), onin(Slot::WEIGHT, 1)};
  if (use_bias) {
    s.out_nodes.push_back(repartition(ogin(Slot::INPUT, 2), 0, degree));          // 2
    ins.push_back(onin(Slot::BIAS, 2));
  }
  s.out_nodes.push_back(templated(0, ins));
  int lin_idx = (int)s.out_nodes.size() - 1;
  s.out_nodes.push_back(combine(onin(Slot::INPUT, lin_idx), -1, degree));
  s.outputs = {{0, Slot::OUTPUT, lin_idx + 1, Slot::OUTPUT}};
  return s;
}

// Linear, data parallel along a leading dim (unity_substitution_set.cc:269-356)
Substitution create_partition_linear_combine(int dim, int degree, bool use_bias) {
  Substitution s;
  s.name = "partition_linear_combine" + sfx(dim, degree) + (use_bias ? "_bias" : "");
  PatternNode lin;
  lin.constraints = {op_is(OpType::LINEAR), attr_eq("use_bias", use_bias)};
  lin.inputs = {gin(Slot::INPUT, 0), gin(Slot::WEIGHT, 1)};
  if (use_bias) lin.inputs.push_back(gin(Slot::BIAS, 2));
  s.pattern.nodes = {lin};
  s.pattern.num_inputs = use_bias ? 3 : 2;
  s.pattern.input_constraints[0] = {{TensorConstraint::NUM_DIMS_AT_LEAST, 0, dim + 2}, {TensorConstraint::DIM_DIVISIBLE_BY, dim, degree}, {TensorConstraint::DIM_DEGREE_EQUAL, dim, 1}};
  s.out_nodes.push_back(repartition(ogin(Slot::INPUT, 0), dim, degree));  // 0
  s.out_nodes.push_back(replicate(ogin(Slot::INPUT, 1), degree));         // 1
  std::vector<OutInput> ins = {onin(Slot::INPUT, 0), onin(Slot::WEIGHT, 1)};
  if (use_bias) {
    s.out_nodes.push_back(replicate(ogin(Slot::INPUT, 2), degree));
    ins.push_back(onin(Slot::BIAS, 2));
  }
  s.out_nodes.push_back(templated(0, ins));
  int li = (int)s.out_nodes.size() - 1;
  s.out_nodes.push_back(combine(onin(Slot::INPUT, li), dim, degree));
  s.outputs = {{0, Slot::OUTPUT, li + 1, Slot::OUTPUT}};
  return s;
}

// Linear, row (in-channel) parallel: shard the contracted dim, reduce the partial sums.  The algebra is in
// the reference (linear.cc:190-206) but no built-in rule emits it; it is the producer of GEMM -> Reduction.
Substitution create_partition_linear_reduce(int degree, bool use_bias) {
  Substitution s;
  s.name = "partition_linear_reduce" + sfx(degree) + (use_bias ? "_bias" : "");
  PatternNode lin;
  lin.constraints = {op_is(OpType::LINEAR), attr_eq("use_bias", use_bias)};
  lin.inputs = {gin(Slot::INPUT, 0), gin(Slot::WEIGHT, 1)};
  if (use_bias) lin.inputs.push_back(gin(Slot::BIAS, 2));
  s.pattern.nodes = {lin};
  s.pattern.num_inputs = use_bias ? 3 : 2;
  s.pattern.input_constraints[0] = {{TensorConstraint::DIM_DIVISIBLE_BY, -1, degree}, {TensorConstraint::DIM_DEGREE_EQUAL, -1, 1}, {TensorConstraint::COPY_DEGREE_EQUAL, 0, 1}};
  s.out_nodes.push_back(repartition(ogin(Slot::INPUT, 0), -1, degree));  // 0
  s.out_nodes.push_back(repartition(ogin(Slot::INPUT, 1), 1, degree));   // 1
  std::vector<OutInput> ins = {onin(Slot::INPUT, 0), onin(Slot::WEIGHT, 1)};
  if (use_bias) {
    s.out_nodes.push_back(replicate(ogin(Slot::INPUT, 2), degree));
    ins.push_back(onin(Slot::BIAS, 2));
  }
  s.out_nodes.push_back(templated(0, ins));
  int li = (int)s.out_nodes.size() - 1;
  s.out_nodes.push_back(reduction(onin(Slot::INPUT, li), degree));
  s.outputs = {{0, Slot::OUTPUT, li + 1, Slot::OUTPUT}};
  return s;
}

Substitution create_partition_conv2d_combine(int degree, bool use_bias) {
  Substitution s;
  s.name = "partition_conv2d_combine" + sfx(degree) + (use_bias ? "_bias" : "");
  PatternNode c;
  c.constraints = {op_is(OpType::CONV2D), attr_eq("use_bias", use_bias)};
  c.inputs = {gin(Slot::INPUT, 0), gin(Slot::FILTER, 1)};
  if (use_bias) c.inputs.push_back(gin(Slot::BIAS, 2));
  s.pattern.nodes = {c};
  s.pattern.num_inputs = use_bias ? 3 : 2;
  s.pattern.input_constraints[0] = {{TensorConstraint::DIM_DIVISIBLE_BY, 0, degree}, {TensorConstraint::DIM_DEGREE_EQUAL, 0, 1}};
  s.out_nodes.push_back(repartition(ogin(Slot::INPUT, 0), 0, degree));
  s.out_nodes.push_back(replicate(ogin(Slot::INPUT, 1), degree));
  std::vector<OutInput> ins = {onin(Slot::INPUT, 0), onin(Slot::FILTER, 1)};
  if (use_bias) {
    s.out_nodes.push_back(replicate(ogin(Slot::INPUT, 2), degree));
    ins.push_back(onin(Slot::BIAS, 2));
  }
  s.out_nodes.push_back(templated(0, ins));
  int li = (int)s.out_nodes.size() - 1;
  s.out_nodes.push_back(combine(onin(Slot::INPUT, li), 0, degree));
  s.outputs = {{0, Slot::OUTPUT, li + 1, Slot::OUTPUT}};
  return s;
}

static Substitution attention_rule(int degree, bool bias, bool head_parallel) {
  Substitution s;
  s.name = std::string(head_parallel ? "replicate_attention_reduce" : "partition_attention_combine") + sfx(degree) + (bias ? "_bias" : "");
  PatternNode a;
  a.constraints = {op_is(OpType::MULTIHEAD_ATTENTION), attr_eq("bias", bias)};
  if (head_parallel) a.constraints.push_back(attr_div("num_heads", degree));
  a.inputs = {gin(Slot::QUERY, 0), gin(Slot::KEY, 1), gin(Slot::VALUE, 2), gin(Slot::WEIGHT, 3)};
  if (bias) { a.inputs.push_back(gin(Slot::INPUT_BIAS, 4)); a.inputs.push_back(gin(Slot::OUTPUT_BIAS, 5)); }
  s.pattern.nodes = {a};
  s.pattern.num_inputs = bias ? 6 : 4;
  for (int i = 0; i < 3; ++i)
    s.pattern.input_constraints[i] = head_parallel ? std::vector<TensorConstraint>{{TensorConstraint::COPY_DEGREE_EQUAL, 0, 1}}
                                                   : std::vector<TensorConstraint>{{TensorConstraint::DIM_DIVISIBLE_BY, 0, degree}, {TensorConstraint::DIM_DEGREE_EQUAL, 0, 1}};
  // q, k and v may be one and the same value: three parallel ops are still emitted (they dedupe at execution)
  for (int i = 0; i < 3; ++i)
    s.out_nodes.push_back(head_parallel ? replicate(ogin(Slot::INPUT, i), degree) : repartition(ogin(Slot::INPUT, i), 0, degree));
  s.out_nodes.push_back(head_parallel ? repartition(ogin(Slot::INPUT, 3), 1, degree) : replicate(ogin(Slot::INPUT, 3), degree));  // 3
  std::vector<OutInput> ins = {onin(Slot::QUERY, 0), onin(Slot::KEY, 1), onin(Slot::VALUE, 2), onin(Slot::WEIGHT, 3)};
  if (bias) {
    s.out_nodes.push_back(head_parallel ? repartition(ogin(Slot::INPUT, 4), 0, degree) : replicate(ogin(Slot::INPUT, 4), degree));  // 4
    s.out_nodes.push_back(replicate(ogin(Slot::INPUT, 5), degree));                                                                 // 5
    ins.push_back(onin(Slot::INPUT_BIAS, 4));
    ins.push_back(onin(Slot::OUTPUT_BIAS, 5));
  }
  s.out_nodes.push_back(templated(0, ins));
  int ai = (int)s.out_nodes.size() - 1;
  s.out_nodes.push_back(head_parallel ? reduction(onin(Slot::INPUT, ai), degree) : combine(onin(Slot::INPUT, ai), 0, degree));
  s.outputs = {{0, Slot::OUTPUT, ai + 1, Slot::OUTPUT}};
  return s;
}
Substitution create_partition_attention_combine(int degree, bool bias) { return attention_rule(degree, bias, false); }
Substitution create_replicate_attention_reduce(int degree, bool bias) { return attention_rule(degree, bias, true); }

Substitution create_partition_unary_combine(OpType op, int dim, int degree) {
  Substitution s;
  s.name = "partition_" + to_string(op) + "_combine" + sfx(dim, degree);
  PatternNode n;
  n.constraints = {op_is(op)};
  n.inputs = {gin(Slot::INPUT, 0)};
  s.pattern.nodes = {n};
  s.pattern.num_inputs = 1;
  s.pattern.input_constraints[0] = {{TensorConstraint::NUM_DIMS_AT_LEAST, 0, dim + 1}, {TensorConstraint::DIM_DIVISIBLE_BY, dim, degree}, {TensorConstraint::DIM_DEGREE_EQUAL, dim, 1}};
  s.out_nodes = {repartition(ogin(Slot::INPUT, 0), dim, degree), templated(0, {onin(Slot::INPUT, 0)}), combine(onin(Slot::INPUT, 1), dim, degree)};
  s.outputs = {{0, Slot::OUTPUT, 2, Slot::OUTPUT}};
  return s;
}
Substitution create_partition_binary_combine(OpType op, int dim, int degree) {
  Substitution s;
  s.name = "partition_" + to_string(op) + "_combine" + sfx(dim, degree);
  PatternNode n;
  n.constraints = {op_is(op)};
  n.inputs = {gin(Slot::LHS_INPUT, 0), gin(Slot::RHS_INPUT, 1)};
  s.pattern.nodes = {n};
  s.pattern.num_inputs = 2;
  for (int i = 0; i < 2; ++i)
    s.pattern.input_constraints[i] = {{TensorConstraint::NUM_DIMS_AT_LEAST, 0, dim + 1}, {TensorConstraint::DIM_DIVISIBLE_BY, dim, degree}, {TensorConstraint::DIM_DEGREE_EQUAL, dim, 1}};
  s.out_nodes = {repartition(ogin(Slot::INPUT, 0), dim, degree), repartition(ogin(Slot::INPUT, 1), dim, degree),
                 templated(0, {onin(Slot::LHS_INPUT, 0), onin(Slot::RHS_INPUT, 1)}), combine(onin(Slot::INPUT, 2), dim, degree)};
  s.outputs = {{0, Slot::OUTPUT, 3, Slot::OUTPUT}};
  return s;
}
Substitution create_partition_softmax_combine(int softmax_dim, int dim, int degree) {
  Substitution s = create_partition_unary_combine(OpType::SOFTMAX, dim, degree);
  s.name = "partition_softmax_combine" + sfx(softmax_dim) + sfx(dim, degree);
  s.pattern.nodes[0].constraints.push_back(attr_eq("dim", softmax_dim));
  return s;
}
Substitution create_partition_layernorm_combine(int dim, int degree, bool affine) {
  Substitution s;
  s.name = "partition_layernorm_combine" + sfx(dim, degree) + (affine ? "_affine" : "");
  PatternNode n;
  n.constraints = {op_is(OpType::LAYERNORM), attr_eq("elementwise_affine", affine)};
  n.inputs = {gin(Slot::INPUT, 0)};
  if (affine) { n.inputs.push_back(gin(Slot::GAMMA, 1)); n.inputs.push_back(gin(Slot::BETA, 2)); }
  s.pattern.nodes = {n};
  s.pattern.num_inputs = affine ? 3 : 1;
  s.pattern.input_constraints[0] = {{TensorConstraint::NUM_DIMS_AT_LEAST, 0, dim + 2}, {TensorConstraint::DIM_DIVISIBLE_BY, dim, degree}, {TensorConstraint::DIM_DEGREE_EQUAL, dim, 1}};
  s.out_nodes.push_back(repartition(ogin(Slot::INPUT, 0), dim, degree));
  std::vector<OutInput> ins = {onin(Slot::INPUT, 0)};
  if (affine) {
    s.out_nodes.push_back(replicate(ogin(Slot::INPUT, 1), degree));
    s.out_nodes.push_back(replicate(ogin(Slot::INPUT, 2), degree));
    ins.push_back(onin(Slot::GAMMA, 1));
    ins.push_back(onin(Slot::BETA, 2));
  }
  s.out_nodes.push_back(templated(0, ins));
  int li = (int)s.out_nodes.size() - 1;
  s.out_nodes.push_back(combine(onin(Slot::INPUT, li), dim, degree));
  s.outputs = {{0, Slot::OUTPUT, li + 1, Slot::OUTPUT}};
  return s;
}
// BatchNorm over a partitioned sample dim: every shard normalises with the statistics of its own samples (the
// usual data-parallel batch norm); scale and shift are replicated.
Substitution create_partition_batchnorm_combine(int dim, int degree, bool affine) {
  Substitution s;
  s.name = "partition_batchnorm_combine" + sfx(dim, degree) + (affine ? "_affine" : "");
  PatternNode n;
  n.constraints = {op_is(OpType::BATCHNORM), attr_eq("affine", affine)};
  n.inputs = {gin(Slot::INPUT, 0)};
  if (affine) { n.inputs.push_back(gin(Slot::GAMMA, 1)); n.inputs.push_back(gin(Slot::BETA, 2)); }
  s.pattern.nodes = {n};
  s.pattern.num_inputs = affine ? 3 : 1;
  s.pattern.input_constraints[0] = {{TensorConstraint::NUM_DIMS_AT_LEAST, 0, dim + 2}, {TensorConstraint::DIM_DIVISIBLE_BY, dim, degree}, {TensorConstraint::DIM_DEGREE_EQUAL, dim, 1}};
  s.out_nodes.push_back(repartition(ogin(Slot::INPUT, 0), dim, degree));
  std::vector<OutInput> ins = {onin(Slot::INPUT, 0)};
  if (affine) {
    s.out_nodes.push_back(replicate(ogin(Slot::INPUT, 1), degree));
    s.out_nodes.push_back(replicate(ogin(Slot::INPUT, 2), degree));
    ins.push_back(onin(Slot::GAMMA, 1));
    ins.push_back(onin(Slot::BETA, 2));
  }
  s.out_nodes.push_back(templated(0, ins));
  int li = (int)s.out_nodes.size() - 1;
  s.out_nodes.push_back(combine(onin(Slot::INPUT, li), dim, degree));
  s.outputs = {{0, Slot::OUTPUT, li + 1, Slot::OUTPUT}};
  return s;
}
// Concat of `num_inputs` tensors along `axis`, all partitioned on another dim
Substitution create_partition_concat_combine(int num_inputs, int axis, int dim, int degree) {
  Substitution s;
  s.name = "partition_concat" + std::to_string(num_inputs) + "_axis" + std::to_string(axis) + "_combine" + sfx(dim, degree);
  PatternNode n;
  n.constraints = {op_is(OpType::CONCAT), attr_eq("axis", axis), attr_eq("num_inputs", num_inputs)};
  for (int i = 0; i < num_inputs; ++i) n.inputs.push_back(gin(input_slot_n(i), i));
  s.pattern.nodes = {n};
  s.pattern.num_inputs = num_inputs;
  std::vector<OutInput> ins;
  for (int i = 0; i < num_inputs; ++i) {
    s.pattern.input_constraints[i] = {{TensorConstraint::NUM_DIMS_AT_LEAST, 0, std::max(dim, axis) + 1}, {TensorConstraint::DIM_DIVISIBLE_BY, dim, degree}, {TensorConstraint::DIM_DEGREE_EQUAL, dim, 1}};
    s.out_nodes.push_back(repartition(ogin(Slot::INPUT, i), dim, degree));
    ins.push_back(onin(input_slot_n(i), i));
  }
  s.out_nodes.push_back(templated(0, ins));
  s.out_nodes.push_back(combine(onin(Slot::INPUT, num_inputs), dim, degree));
  s.outputs = {{0, Slot::OUTPUT, num_inputs + 1, Slot::OUTPUT}};
  return s;
}
Substitution create_partition_embedding_combine(int dim, int degree) {
  Substitution s;
  s.name = "partition_embedding_combine" + sfx(dim, degree);
  PatternNode n;
  n.constraints = {op_is(OpType::EMBEDDING)};
  n.inputs = {gin(Slot::INPUT, 0), gin(Slot::WEIGHT, 1)};
  s.pattern.nodes = {n};
  s.pattern.num_inputs = 2;
  s.pattern.input_constraints[0] = {{TensorConstraint::NUM_DIMS_AT_LEAST, 0, dim + 2}, {TensorConstraint::DIM_DIVISIBLE_BY, dim, degree}, {TensorConstraint::DIM_DEGREE_EQUAL, dim, 1}};
  s.out_nodes = {repartition(ogin(Slot::INPUT, 0), dim, degree), replicate(ogin(Slot::INPUT, 1), degree),
                 templated(0, {onin(Slot::INPUT, 0), onin(Slot::WEIGHT, 1)}), combine(onin(Slot::INPUT, 2), dim, degree)};
  s.outputs = {{0, Slot::OUTPUT, 3, Slot::OUTPUT}};
  return s;
}
// Linear(activation = none) -> act  ==>  Linear(activation = act)   (unity_substitution_set.cc:761)
Substitution create_fuse_linear_activation(const std::string &activation) {
  Substitution s;
  s.name = "fuse_linear_" + activation;
  PatternNode lin, act;
  lin.constraints = {op_is(OpType::LINEAR), attr_eq("activation", Json())};
  lin.inputs = {gin(Slot::INPUT, 0), gin(Slot::WEIGHT, 1)};
  lin.allow_extra_inputs = true;
  act.constraints = {op_is(optype_from_string(activation))};
  act.inputs = {nin(Slot::INPUT, 0)};
  s.pattern.nodes = {lin, act};
  s.pattern.num_inputs = 2;
  OutNode fused = templated(0, {ogin(Slot::INPUT, 0), ogin(Slot::WEIGHT, 1)});
  fused.assigns["activation"] = lit(Json(activation));
  s.out_nodes = {fused};
  s.outputs = {{1, Slot::OUTPUT, 0, Slot::OUTPUT}};
  return s;
}
// Combine(dim, k) immediately re-partitioned the same way is the identity (and vice versa): these two rules
// let neighbouring data-parallel operators share one partitioning instead of gathering in between.
static Substitution cancel_pair(OpType first, OpType second, const std::string &name) {
  Substitution s;
  s.name = name;
  PatternNode a, b;
  a.constraints = {op_is(first)};
  a.inputs = {gin(Slot::INPUT, 0)};
  b.constraints = {op_is(second)};
  b.inputs = {nin(Slot::INPUT, 0)};
  s.pattern.nodes = {a, b};
  s.pattern.num_inputs = 1;
  s.outputs = {{1, Slot::OUTPUT, -1, Slot::OUTPUT}};  // out_node -1 = pattern graph input 0
  return s;
}
// Same cancellation when the first operator has further consumers (a residual branch): the first operator
// is re-created for them and only this second operator disappears; a re-created operator that ends up
// without consumers is swept by apply_substitution's dead parallel-op removal.
static Substitution cancel_pair_shared(OpType first, OpType second, const std::string &name) {
  Substitution s = cancel_pair(first, second, name);
  s.out_nodes = {templated(0, {ogin(Slot::INPUT, 0)})};
  s.outputs = {{0, Slot::OUTPUT, 0, Slot::OUTPUT}, {1, Slot::OUTPUT, -1, Slot::OUTPUT}};
  return s;
}
// first -> second  ==>  second -> first, both re-created from the matched operators' own attributes.  Shape inference
// on the swapped pair decides whether the swap is legal at a match (the interface shape must come out unchanged).
// Used to bring a Combine next to the Repartition behind a Replicate / Reduction (hybrid data x tensor parallel
// graphs), after which the pair cancels.
static Substitution commute_pair(OpType first, OpType second, const std::string &name) {
  Substitution s = cancel_pair(first, second, name);
  s.out_nodes = {templated(1, {ogin(Slot::INPUT, 0)}), templated(0, {onin(Slot::INPUT, 0)})};
  s.outputs = {{1, Slot::OUTPUT, 1, Slot::OUTPUT}};
  return s;
}
std::vector<Substitution> get_commute_rules() {
  return {commute_pair(OpType::COMBINE, OpType::REPLICATE, "commute_combine_replicate"),
          commute_pair(OpType::COMBINE, OpType::REDUCTION, "commute_combine_reduction")};
}
Substitution create_cancel_combine_repartition() { return cancel_pair(OpType::COMBINE, OpType::REPARTITION, "cancel_combine_repartition"); }
Substitution create_cancel_repartition_combine() { return cancel_pair(OpType::REPARTITION, OpType::COMBINE, "cancel_repartition_combine"); }
Substitution create_cancel_replicate_reduction_free() { return cancel_pair(OpType::REPLICATE, OpType::NOOP, "cancel_replicate_noop"); }

std::vector<Substitution> get_substitution_set(const MachineSpec &m, int max_dims) {
  std::vector<Substitution> r;
  std::vector<int> degrees;
  for (int d = 2; d <= m.num_devices(); d *= 2) degrees.push_back(d);
  for (int d : degrees) {
    for (bool bias : {false, true}) {
      r.push_back(create_replicate_linear_combine(d, bias));
      r.push_back(create_partition_linear_reduce(d, bias));
      r.push_back(create_partition_conv2d_combine(d, bias));
      r.push_back(create_partition_attention_combine(d, bias));
      r.push_back(create_replicate_attention_reduce(d, bias));
      for (int dim = 0; dim < max_dims - 1; ++dim) r.push_back(create_partition_linear_combine(dim, d, bias));
    }
    for (int dim = 0; dim < max_dims; ++dim) {
      for (OpType u : {OpType::RELU, OpType::GELU, OpType::SIGMOID, OpType::TANH, OpType::DROPOUT, OpType::CAST})
        r.push_back(create_partition_unary_combine(u, dim, d));
      r.push_back(create_partition_binary_combine(OpType::EW_ADD, dim, d));
      r.push_back(create_partition_binary_combine(OpType::EW_MUL, dim, d));
      for (int sd = 0; sd < max_dims; ++sd)
        if (sd != dim) r.push_back(create_partition_softmax_combine(sd, dim, d));
      if (dim == 0) {  // sample-dim rules of the convolution-stack and shape operators
        for (OpType u : {OpType::POOL2D, OpType::FLAT, OpType::NOOP, OpType::ELU, OpType::EXP, OpType::SCALAR_MULTIPLY, OpType::SCALAR_ADD,
                         OpType::RESHAPE})  // (a Reshape that does not keep dim 0 fails shape inference and is skipped)
          r.push_back(create_partition_unary_combine(u, dim, d));
        // Transpose with the sample dim left in place
        for (int nd = 3; nd <= max_dims; ++nd) {
          std::vector<int> perm(nd);
          for (int i = 0; i < nd; ++i) perm[i] = i;
          do {
            Substitution t = create_partition_unary_combine(OpType::TRANSPOSE, dim, d);
            std::string tag;
            for (int v : perm) tag += std::to_string(v);
            t.name = "partition_TRANSPOSE" + tag + "_combine" + sfx(dim, d);
            t.pattern.nodes[0].constraints.push_back(attr_eq("permutation", Json::from_ints(std::vector<long long>(perm.begin(), perm.end()))));
            r.push_back(t);
          } while (std::next_permutation(perm.begin() + 1, perm.end()));
        }
        r.push_back(create_partition_binary_combine(OpType::EW_SUB, dim, d));
        r.push_back(create_partition_binary_combine(OpType::BATCHMATMUL, dim, d));
        r.push_back(create_partition_batchnorm_combine(dim, d, true));
        r.push_back(create_partition_batchnorm_combine(dim, d, false));
        for (int k = 2; k <= 8; ++k)
          for (int axis = 1; axis < max_dims; ++axis) r.push_back(create_partition_concat_combine(k, axis, dim, d));
      }
      if (dim < max_dims - 1) {
        r.push_back(create_partition_layernorm_combine(dim, d, true));
        r.push_back(create_partition_layernorm_combine(dim, d, false));
        r.push_back(create_partition_embedding_combine(dim, d));
      }
    }
  }
  for (const char *a : {"RELU", "SIGMOID", "TANH", "GELU"}) r.push_back(create_fuse_linear_activation(a));
  r.push_back(create_cancel_combine_repartition());
  r.push_back(create_cancel_repartition_combine());
  r.push_back(cancel_pair_shared(OpType::COMBINE, OpType::REPARTITION, "cancel_shared_combine_repartition"));
  return r;
}

// ---------------------------------------------------------------- legacy TASO rules
namespace {
struct LegacyOp {
  std::string type;
  std::vector<std::pair<int, int>> inputs;  // (opId, tsId); opId < 0 = external input
  std::map<std::string, long long> para;
};
LegacyOp parse_legacy_op(const Json &j) {
  LegacyOp o;
  o.type = j.at("type").as_string();
  for (auto &in : j.at("input").items()) o.inputs.push_back({(int)in.at("opId").as_int(), (int)in.at("tsId").as_int()});
  for (auto &p : j.at("para").items()) o.para[p.at("key").as_string()] = p.at("value").as_int();
  return o;
}
// legacy operator -> (pattern constraints | output node); false when the operator kind is not expressible
bool legacy_to_optype(const LegacyOp &o, OpType &t, std::map<std::string, Json> &attrs, std::vector<Slot> &in_slots) {
  auto P = [&](const char *k, long long d) { auto it = o.para.find(k); return it == o.para.end() ? d : it->second; };
  // legacy dims count from the innermost dim and include a replica dim; translate to negative indices
  auto dim = [&](long long legacy_dim) { return (int)(-1 - legacy_dim); };
  if (o.type == "OP_LINEAR") {
    t = OpType::LINEAR;
    static const char *acts[] = {nullptr, "SIGMOID", "RELU", "TANH", "GELU"};
    long long a = P("PM_ACTI", 0);
    attrs["activation"] = (a >= 1 && a <= 4) ? Json(acts[a]) : Json();
    in_slots = {Slot::INPUT, Slot::WEIGHT};
    return true;
  }
  if (o.type == "OP_RELU") { t = OpType::RELU; in_slots = {Slot::INPUT}; return true; }
  if (o.type == "OP_EW_ADD") { t = OpType::EW_ADD; in_slots = {Slot::LHS_INPUT, Slot::RHS_INPUT}; return true; }
  if (o.type == "OP_EW_MUL") { t = OpType::EW_MUL; in_slots = {Slot::LHS_INPUT, Slot::RHS_INPUT}; return true; }
  if (o.type == "OP_CONCAT") {
    t = OpType::CONCAT;
    long long n = P("PM_NUM_INPUTS", (long long)o.inputs.size());
    attrs["num_inputs"] = n;
    attrs["axis"] = dim(P("PM_AXIS", 0));
    for (int i = 0; i < n; ++i) in_slots.push_back(input_slot_n(i));
    return n <= 8;
  }
  if (o.type == "OP_PARTITION" || o.type == "OP_REPARTITION") {
    t = OpType::REPARTITION;
    attrs["repartition_dim"] = dim(P("PM_PARALLEL_DIM", 0));
    attrs["repartition_degree"] = P("PM_PARALLEL_DEGREE", 2);
    in_slots = {Slot::INPUT};
    return true;
  }
  if (o.type == "OP_COMBINE") {
    t = OpType::COMBINE;
    attrs["combine_dim"] = dim(P("PM_PARALLEL_DIM", 0));
    attrs["combine_degree"] = P("PM_PARALLEL_DEGREE", 2);
    in_slots = {Slot::INPUT};
    return true;
  }
  if (o.type == "OP_REPLICATE") {
    t = OpType::REPLICATE;
    attrs["replicate_degree"] = P("PM_PARALLEL_DEGREE", 2);
    in_slots = {Slot::INPUT};
    return true;
  }
  if (o.type == "OP_REDUCE" || o.type == "OP_REDUCTION") {
    t = OpType::REDUCTION;
    attrs["reduction_degree"] = P("PM_PARALLEL_DEGREE", 2);
    in_slots = {Slot::INPUT};
    return true;
  }
  return false;  // OP_SPLIT and others: multi-output legacy semantics are not converted
}
}  // namespace

std::vector<Substitution> load_legacy_rules(const Json &collection, LegacyRuleStats *stats) {
  std::vector<Substitution> out;
  LegacyRuleStats st;
  for (auto &rule : collection.at("rule").items()) {
    ++st.num_rules;
    std::vector<LegacyOp> src, dst;
    for (auto &o : rule.at("srcOp").items()) { src.push_back(parse_legacy_op(o)); st.op_histogram[src.back().type]++; }
    for (auto &o : rule.at("dstOp").items()) { dst.push_back(parse_legacy_op(o)); st.op_histogram[dst.back().type]++; }
    Substitution s;
    s.name = rule.get_string("name", "legacy_rule_" + std::to_string(st.num_rules));
    bool ok = true;
    std::map<std::pair<int, int>, int> ext_index;  // external (opId, tsId) -> pattern graph input
    auto ext = [&](int op, int ts) {
      auto key = std::make_pair(op, ts);
      auto it = ext_index.find(key);
      if (it == ext_index.end()) it = ext_index.emplace(key, (int)ext_index.size()).first;
      return it->second;
    };
    for (auto &o : src) {
      OpType t;
      std::map<std::string, Json> attrs;
      std::vector<Slot> slots;
      if (!legacy_to_optype(o, t, attrs, slots) || slots.size() != o.inputs.size()) { ok = false; break; }
      PatternNode pn;
      pn.constraints.push_back(op_is(t));
      for (auto &kv : attrs) pn.constraints.push_back(attr_eq(kv.first, kv.second));
      pn.allow_extra_inputs = (t == OpType::LINEAR);
      for (size_t i = 0; i < o.inputs.size(); ++i) {
        if (o.inputs[i].first < 0) pn.inputs.push_back(gin(slots[i], ext(o.inputs[i].first, o.inputs[i].second)));
        else pn.inputs.push_back(nin(slots[i], o.inputs[i].first));
      }
      s.pattern.nodes.push_back(pn);
    }
    if (ok)
      for (auto &o : dst) {
        OpType t;
        std::map<std::string, Json> attrs;
        std::vector<Slot> slots;
        if (!legacy_to_optype(o, t, attrs, slots) || slots.size() != o.inputs.size()) { ok = false; break; }
        OutNode on;
        on.type = t;
        for (auto &kv : attrs) on.assigns[kv.first] = lit(kv.second);
        if (t == OpType::LINEAR) {
          // out_channels / use_bias come from a source Linear when there is one
          for (size_t i = 0; i < src.size(); ++i)
            if (src[i].type == "OP_LINEAR") { on.template_node = (int)i; break; }
          if (!on.template_node) { ok = false; break; }
        }
        for (size_t i = 0; i < o.inputs.size(); ++i) {
          if (o.inputs[i].first < 0) {
            auto key = std::make_pair(o.inputs[i].first, o.inputs[i].second);
            if (!ext_index.count(key)) { ok = false; break; }
            on.inputs.push_back(ogin(slots[i], ext_index[key]));
          } else on.inputs.push_back(onin(slots[i], o.inputs[i].first));
        }
        s.out_nodes.push_back(on);
      }
    if (ok) {
      s.pattern.num_inputs = (int)ext_index.size();
      for (auto &mo : rule.at("mappedOutput").items())
        s.outputs.push_back({(int)mo.at("srcOpId").as_int(), Slot::OUTPUT, (int)mo.at("dstOpId").as_int(), Slot::OUTPUT});
      ok = is_valid_substitution(s);
    }
    if (ok) { out.push_back(s); ++st.num_converted; }
  }
  if (stats) *stats = st;
  return out;
}

// ---------------------------------------------------------------- rendering
Json Substitution::to_json() const {
  Json j = Json::object();
  j["name"] = name;
  Json pn = Json::array();
  for (auto &n : pattern.nodes) {
    Json e = Json::object();
    Json cs = Json::array();
    for (auto &c : n.constraints) {
      Json cj = Json::object();
      cj["kind"] = c.kind == AttrConstraint::EQUAL ? "EQUAL" : "DIVISIBLE_BY";
      cj["key"] = c.key;
      cj["value"] = c.value;
      cs.push_back(cj);
    }
    e["constraints"] = cs;
    Json ins = Json::array();
    for (auto &in : n.inputs) {
      Json ij = Json::object();
      ij["slot"] = to_string(in.slot);
      ij[in.from_graph_input ? "graph_input" : "node"] = in.index;
      ins.push_back(ij);
    }
    e["inputs"] = ins;
    pn.push_back(e);
  }
  j["pattern"] = pn;
  j["num_inputs"] = pattern.num_inputs;
  Json on = Json::array();
  for (auto &n : out_nodes) {
    Json e = Json::object();
    e["type"] = n.template_node ? Json("template:" + std::to_string(*n.template_node)) : Json(to_string(n.type));
    Json as = Json::object();
    for (auto &kv : n.assigns) as[kv.first] = kv.second.kind == AttrExpr::LITERAL ? kv.second.literal : Json("attr_of:" + std::to_string(kv.second.pattern_node) + "." + kv.second.key);
    e["assigns"] = as;
    Json ins = Json::array();
    for (auto &in : n.inputs) {
      Json ij = Json::object();
      ij["slot"] = to_string(in.slot);
      ij[in.from_graph_input ? "graph_input" : "node"] = in.index;
      ins.push_back(ij);
    }
    e["inputs"] = ins;
    on.push_back(e);
  }
  j["output_graph"] = on;
  return j;
}

std::string substitution_as_dot(const Substitution &s) {
  std::ostringstream o;
  o << "digraph substitution {\n  compound=true; node [shape=box, fontsize=10];\n";
  o << "  subgraph cluster_src { label=\"pattern: " << s.name << "\";\n";
  for (int i = 0; i < s.pattern.num_inputs; ++i) o << "    si" << i << " [label=\"input " << i << "\", shape=ellipse];\n";
  for (size_t i = 0; i < s.pattern.nodes.size(); ++i) {
    std::string label;
    for (auto &c : s.pattern.nodes[i].constraints) label += c.key + (c.kind == AttrConstraint::EQUAL ? "=" : "%") + c.value.dump() + "\\n";
    o << "    s" << i << " [label=\"" << label << "\"];\n";
    for (auto &in : s.pattern.nodes[i].inputs)
      o << "    " << (in.from_graph_input ? "si" : "s") << in.index << " -> s" << i << " [label=\"" << to_string(in.slot) << "\", fontsize=8];\n";
  }
  o << "  }\n  subgraph cluster_dst { label=\"output graph\";\n";
  for (int i = 0; i < s.pattern.num_inputs; ++i) o << "    di" << i << " [label=\"input " << i << "\", shape=ellipse];\n";
  for (size_t i = 0; i < s.out_nodes.size(); ++i) {
    auto &n = s.out_nodes[i];
    std::string label = n.template_node ? "copy of pattern node " + std::to_string(*n.template_node) : to_string(n.type);
    for (auto &kv : n.assigns) label += "\\n" + kv.first + "=" + (kv.second.kind == AttrExpr::LITERAL ? kv.second.literal.dump() : "attr");
    o << "    d" << i << " [label=\"" << label << "\"];\n";
    for (auto &in : n.inputs)
      o << "    " << (in.from_graph_input ? "di" : "d") << in.index << " -> d" << i << " [label=\"" << to_string(in.slot) << "\", fontsize=8];\n";
  }
  o << "  }\n}\n";
  return o.str();
}

std::string legacy_rule_as_dot(const Json &rule) {
  std::ostringstream o;
  o << "digraph rule {\n  node [shape=box, fontsize=10];\n";
  for (const char *side : {"srcOp", "dstOp"}) {
    std::string p = side[0] == 's' ? "s" : "d";
    o << "  subgraph cluster_" << p << " { label=\"" << side << "\";\n";
    int i = 0;
    for (auto &op : rule.at(side).items()) {
      std::string label = op.at("type").as_string();
      for (auto &pa : op.at("para").items()) label += "\\n" + pa.at("key").as_string() + "=" + std::to_string(pa.at("value").as_int());
      o << "    " << p << i << " [label=\"" << label << "\"];\n";
      for (auto &in : op.at("input").items()) {
        long long src = in.at("opId").as_int();
        if (src < 0) o << "    " << p << "x" << -src << "_" << in.at("tsId").as_int() << " [shape=ellipse, label=\"ext\"];\n    " << p << "x" << -src << "_" << in.at("tsId").as_int() << " -> " << p << i << ";\n";
        else o << "    " << p << src << " -> " << p << i << ";\n";
      }
      ++i;
    }
    o << "  }\n";
  }
  o << "}\n";
  return o.str();
}

// ---------------------------------------------------------------- python bindings
// Parallel operators with the same kind, attributes and input compute the same tensor: keep one of each and
// point every consumer at it (applying a rule once per input slot of an operator leaves such copies behind, e.g.
// three Replicates of the same tensor in front of self-attention).
Graph merge_duplicate_parallel_ops(const Graph &g_in) {
  Graph g = g_in;
  bool changed = true;
  while (changed) {
    changed = false;
    std::map<std::string, NodeId> seen;
    for (NodeId n : g.topological_order()) {
      const Node &nd = g.node(n);
      if (!is_parallel_op(nd.type) || nd.inputs.size() != 1 || nd.outputs.size() != 1) continue;
      std::string key = to_string(nd.type) + "|" + nd.attrs.dump() + "|" + std::to_string(nd.inputs[0].src.node) + ":" +
                        to_string(nd.inputs[0].src.slot);
      auto it = seen.find(key);
      if (it == seen.end()) {
        seen[key] = n;
        continue;
      }
      ValueRef from{n, nd.outputs[0].slot}, to{it->second, g.node(it->second).outputs[0].slot};
      g.replace_uses(from, to);
      g.remove_node(n);
      changed = true;
      break;
    }
  }
  return g;
}

void bind_substitutions(py::module &m) {
  m.def("merge_duplicate_parallel_ops", &merge_duplicate_parallel_ops);
  py::class_<Substitution>(m, "Substitution")
      .def_readonly("name", &Substitution::name)
      .def("to_json", [](const Substitution &s) { return json_to_py(s.to_json()); })
      .def("as_dot", &substitution_as_dot)
      .def("is_valid", [](const Substitution &s) { return is_valid_substitution(s); })
      .def("num_pattern_nodes", [](const Substitution &s) { return s.pattern.nodes.size(); });
  py::class_<Match>(m, "PatternMatch")
      .def_readonly("nodes", &Match::nodes)
      .def_property_readonly("inputs", [](const Match &mt) {
        py::list l;
        for (auto &v : mt.inputs) l.append(value_to_py(v));
        return l;
      });
  m.def("get_substitution_set", [](const MachineSpec &ms, int max_dims) { return get_substitution_set(ms, max_dims); }, py::arg("machine"),
        py::arg("max_dims") = 4);
  m.def("find_pattern_matches", [](const Substitution &s, const Graph &g) { return find_pattern_matches(s.pattern, g); });
  m.def("apply_substitution", [](const Graph &g, const Substitution &s, const Match &mt) -> py::object {
    std::string why;
    auto r = apply_substitution(g, s, mt, &why);
    if (!r) return py::none();
    return py::cast(*r);
  });
  m.def("why_not_applicable", [](const Graph &g, const Substitution &s, const Match &mt) {
    std::string why;
    auto r = apply_substitution(g, s, mt, &why);
    return r ? std::string() : why;
  });
  m.def("create_replicate_linear_combine", &create_replicate_linear_combine);
  m.def("create_partition_linear_combine", &create_partition_linear_combine);
  m.def("create_partition_linear_reduce", &create_partition_linear_reduce);
  m.def("create_partition_conv2d_combine", &create_partition_conv2d_combine);
  m.def("create_partition_attention_combine", &create_partition_attention_combine);
  m.def("create_replicate_attention_reduce", &create_replicate_attention_reduce);
  m.def("create_partition_unary_combine", [](const std::string &op, int dim, int deg) { return create_partition_unary_combine(optype_from_string(op), dim, deg); });
  m.def("create_partition_binary_combine", [](const std::string &op, int dim, int deg) { return create_partition_binary_combine(optype_from_string(op), dim, deg); });
  m.def("create_partition_softmax_combine", &create_partition_softmax_combine);
  m.def("create_partition_layernorm_combine", &create_partition_layernorm_combine);
  m.def("create_partition_embedding_combine", &create_partition_embedding_combine);
  m.def("create_fuse_linear_activation", &create_fuse_linear_activation);
  m.def("get_commute_rules", &get_commute_rules);
  m.def("create_cancel_combine_repartition", &create_cancel_combine_repartition);
  m.def("create_cancel_repartition_combine", &create_cancel_repartition_combine);
  m.def("load_legacy_rules", [](py::object collection) {
    Json j = py::isinstance<py::str>(collection) ? Json::parse(collection.cast<std::string>()) : json_from_py(collection);
    LegacyRuleStats st;
    auto rules = load_legacy_rules(j, &st);
    py::dict d;
    d["num_rules"] = st.num_rules;
    d["num_converted"] = st.num_converted;
    d["op_histogram"] = st.op_histogram;
    return py::make_tuple(rules, d);
  });
  m.def("legacy_rule_as_dot", [](py::object rule) { return legacy_rule_as_dot(json_from_py(rule)); });
}

}  // namespace ff
