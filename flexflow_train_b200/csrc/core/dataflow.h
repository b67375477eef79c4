// dataflow.h -- the dataflow graph family and the declarative command-line specification of the support library.
//
// Graph variants (lib/utils/include/utils/graph/index.dox): a DataflowGraph models a computation -- nodes are
// functions from an ordered tuple of inputs to an ordered tuple of outputs, edges are uses of values; it is acyclic by
// construction (a node can only be added after the producers of its inputs).  An OpenDataflowGraph additionally has
// graph inputs: values that come from outside, which is what a sub-graph cut out of a larger graph keeps of the edges
// that cross the cut.  KwargDataflowGraph names a node's inputs and outputs by slot instead of by position.  The
// Labelled variants attach a label to every node and every value.
//
// All of them are values with copy-on-write storage: copying a graph is cheap and shares the representation until one
// of the copies is modified; a *View type is the same storage without the mutating interface (a Graph converts to its
// View, never the other way round; `materialize` makes a fresh Graph from a View).
//
// Command lines (lib/utils/include/utils/cli/cli_spec.h, cli_parse.h, cli_get_help_message.h): a CLISpec lists flags
// and positional arguments (with an optional set of allowed values); cli_parse checks an argument vector against it.
#pragma once
#include <algorithm>
#include <map>
#include <memory>
#include <optional>
#include <set>
#include <sstream>
#include <stdexcept>
#include <string>
#include <variant>
#include <vector>

#include "graph_algos.h"

namespace ff {

// ---------------------------------------------------------------------------------------------- plain dataflow graph
struct DataflowOutput {
  int node, idx;
  bool operator<(const DataflowOutput &o) const { return std::tie(node, idx) < std::tie(o.node, o.idx); }
  bool operator==(const DataflowOutput &o) const { return node == o.node && idx == o.idx; }
};
struct DataflowInput {
  int node, idx;
  bool operator<(const DataflowInput &o) const { return std::tie(node, idx) < std::tie(o.node, o.idx); }
  bool operator==(const DataflowInput &o) const { return node == o.node && idx == o.idx; }
};
struct DataflowEdge {
  DataflowOutput src;
  DataflowInput dst;
  bool operator<(const DataflowEdge &o) const { return std::tie(src, dst) < std::tie(o.src, o.dst); }
  bool operator==(const DataflowEdge &o) const { return src == o.src && dst == o.dst; }
};
struct DataflowGraphInput {
  int idx;
  bool operator<(const DataflowGraphInput &o) const { return idx < o.idx; }
  bool operator==(const DataflowGraphInput &o) const { return idx == o.idx; }
};
// a value of an open graph: produced inside (an output of a node) or coming from outside (a graph input)
using OpenDataflowValue = std::variant<DataflowOutput, DataflowGraphInput>;

struct NodeAddedResult {
  int node;
  std::vector<DataflowOutput> outputs;
};

// query: an unset field matches everything (the reference's query_set with std::nullopt)
struct DataflowEdgeQuery {
  std::optional<std::set<int>> src_nodes, dst_nodes;
  std::optional<std::set<int>> src_idxs, dst_idxs;
};

namespace detail {
struct DataflowStorage {
  int next_node = 0, next_input = 0;
  std::vector<int> order;                                  // insertion (= a topological) order
  std::map<int, std::vector<OpenDataflowValue>> inputs;    // node -> ordered operands
  std::map<int, int> num_outputs;
  std::set<int> graph_inputs;
};
}  // namespace detail

class OpenDataflowGraphView {
public:
  OpenDataflowGraphView() : s_(std::make_shared<detail::DataflowStorage>()) {}
  std::vector<int> get_nodes() const { return s_->order; }
  std::set<int> query_nodes(const std::optional<std::set<int>> &q = std::nullopt) const {
    std::set<int> r;
    for (int n : s_->order)
      if (!q || q->count(n)) r.insert(n);
    return r;
  }
  bool has_node(int n) const { return s_->num_outputs.count(n) > 0; }
  std::vector<DataflowOutput> get_outputs(int node) const {
    std::vector<DataflowOutput> r;
    for (int i = 0; i < s_->num_outputs.at(node); ++i) r.push_back({node, i});
    return r;
  }
  const std::vector<OpenDataflowValue> &get_inputs(int node) const { return s_->inputs.at(node); }
  std::vector<DataflowGraphInput> get_graph_inputs() const {
    std::vector<DataflowGraphInput> r;
    for (int i : s_->graph_inputs) r.push_back({i});
    return r;
  }
  // edges between nodes of the graph
  std::set<DataflowEdge> query_edges(const DataflowEdgeQuery &q = DataflowEdgeQuery()) const {
    std::set<DataflowEdge> r;
    for (auto &kv : s_->inputs)
      for (size_t i = 0; i < kv.second.size(); ++i) {
        if (!std::holds_alternative<DataflowOutput>(kv.second[i])) continue;
        const DataflowOutput &src = std::get<DataflowOutput>(kv.second[i]);
        if (q.src_nodes && !q.src_nodes->count(src.node)) continue;
        if (q.dst_nodes && !q.dst_nodes->count(kv.first)) continue;
        if (q.src_idxs && !q.src_idxs->count(src.idx)) continue;
        if (q.dst_idxs && !q.dst_idxs->count((int)i)) continue;
        r.insert({src, {kv.first, (int)i}});
      }
    return r;
  }
  // uses of graph inputs: (graph input, consuming operand)
  std::vector<std::pair<DataflowGraphInput, DataflowInput>> get_input_edges() const {
    std::vector<std::pair<DataflowGraphInput, DataflowInput>> r;
    for (auto &kv : s_->inputs)
      for (size_t i = 0; i < kv.second.size(); ++i)
        if (std::holds_alternative<DataflowGraphInput>(kv.second[i])) r.push_back({std::get<DataflowGraphInput>(kv.second[i]), {kv.first, (int)i}});
    return r;
  }
  std::vector<DataflowInput> get_uses(const OpenDataflowValue &v) const {
    std::vector<DataflowInput> r;
    for (auto &kv : s_->inputs)
      for (size_t i = 0; i < kv.second.size(); ++i)
        if (kv.second[i] == v) r.push_back({kv.first, (int)i});
    return r;
  }
  // values nobody inside the graph uses
  std::vector<DataflowOutput> get_unused_outputs() const {
    std::set<DataflowOutput> used;
    for (auto &kv : s_->inputs)
      for (auto &v : kv.second)
        if (std::holds_alternative<DataflowOutput>(v)) used.insert(std::get<DataflowOutput>(v));
    std::vector<DataflowOutput> r;
    for (int n : s_->order)
      for (auto &o : get_outputs(n))
        if (!used.count(o)) r.push_back(o);
    return r;
  }
  std::vector<int> topological_ordering() const { return s_->order; }
  DiGraph as_digraph() const {
    DiGraph d;
    for (int n : s_->order) d.add_node(n);
    for (auto &e : query_edges()) d.add_edge(e.src.node, e.dst.node);
    return d;
  }
  bool is_closed() const { return s_->graph_inputs.empty(); }
  long use_count() const { return s_.use_count(); }  // how many graphs / views share this representation

protected:
  std::shared_ptr<detail::DataflowStorage> s_;
  detail::DataflowStorage &own() {  // copy on write
    if (s_.use_count() > 1) s_ = std::make_shared<detail::DataflowStorage>(*s_);
    return *s_;
  }
};

class OpenDataflowGraph : public OpenDataflowGraphView {
public:
  DataflowGraphInput add_input() {
    auto &s = own();
    int i = s.next_input++;
    s.graph_inputs.insert(i);
    return {i};
  }
  NodeAddedResult add_node(const std::vector<OpenDataflowValue> &inputs, int num_outputs) {
    for (auto &v : inputs) {
      if (std::holds_alternative<DataflowOutput>(v)) {
        const DataflowOutput &o = std::get<DataflowOutput>(v);
        auto it = s_->num_outputs.find(o.node);
        if (it == s_->num_outputs.end() || o.idx < 0 || o.idx >= it->second) throw std::invalid_argument("add_node: operand is not a value of this graph");
      } else if (!s_->graph_inputs.count(std::get<DataflowGraphInput>(v).idx)) {
        throw std::invalid_argument("add_node: operand is not an input of this graph");
      }
    }
    if (num_outputs < 0) throw std::invalid_argument("add_node: negative output count");
    auto &s = own();
    int n = s.next_node++;
    s.order.push_back(n);
    s.inputs[n] = inputs;
    s.num_outputs[n] = num_outputs;
    NodeAddedResult r{n, {}};
    for (int i = 0; i < num_outputs; ++i) r.outputs.push_back({n, i});
    return r;
  }
  static OpenDataflowGraph materialize(const OpenDataflowGraphView &v) {
    OpenDataflowGraph g;
    static_cast<OpenDataflowGraphView &>(g) = v;
    g.own();
    return g;
  }
};

// The sub-graph on `nodes`, as an open graph: every value produced outside the set and used inside becomes a graph
// input.  `input_of` says which value of the full graph each new input stands for; nodes are renumbered (`node_of`).
struct OpenSubgraphResult {
  OpenDataflowGraph graph;
  std::map<int, int> node_of;                                  // full-graph node -> sub-graph node
  std::vector<std::pair<DataflowGraphInput, OpenDataflowValue>> input_of;
};
inline OpenSubgraphResult get_open_subgraph(const OpenDataflowGraphView &g, const std::set<int> &nodes) {
  OpenSubgraphResult r;
  std::map<OpenDataflowValue, DataflowGraphInput> cut;
  for (int n : g.topological_ordering()) {
    if (!nodes.count(n)) continue;
    std::vector<OpenDataflowValue> ins;
    for (auto &v : g.get_inputs(n)) {
      bool inside = std::holds_alternative<DataflowOutput>(v) && nodes.count(std::get<DataflowOutput>(v).node);
      if (inside) {
        const DataflowOutput &o = std::get<DataflowOutput>(v);
        ins.push_back(DataflowOutput{r.node_of.at(o.node), o.idx});
      } else {
        auto it = cut.find(v);
        if (it == cut.end()) {
          DataflowGraphInput gi = r.graph.add_input();
          it = cut.emplace(v, gi).first;
          r.input_of.push_back({gi, v});
        }
        ins.push_back(it->second);
      }
    }
    r.node_of[n] = r.graph.add_node(ins, (int)g.get_outputs(n).size()).node;
  }
  return r;
}

// ---- algorithms over open dataflow graphs (lib/utils/include/utils/graph/{dataflow_graph,open_dataflow_graph}/algorithms/*.h)
// nodes all of whose operands are graph inputs (or that have none)
inline std::set<int> get_source_nodes(const OpenDataflowGraphView &g) {
  std::set<int> r;
  for (int n : g.get_nodes()) {
    bool src = true;
    for (auto &v : g.get_inputs(n)) src = src && std::holds_alternative<DataflowGraphInput>(v);
    if (src) r.insert(n);
  }
  return r;
}
inline std::set<DataflowGraphInput> get_unused_open_dataflow_graph_inputs(const OpenDataflowGraphView &g) {
  std::set<DataflowGraphInput> r;
  for (auto &gi : g.get_graph_inputs())
    if (g.get_uses(gi).empty()) r.insert(gi);
  return r;
}
inline std::set<DataflowEdge> get_dataflow_edges_from_node_to_node(const OpenDataflowGraphView &g, int src, int dst) {
  DataflowEdgeQuery q;
  q.src_nodes = std::set<int>{src};
  q.dst_nodes = std::set<int>{dst};
  return g.query_edges(q);
}
// the values a node set reads from outside itself: outputs of other nodes and graph inputs
inline std::set<OpenDataflowValue> get_subgraph_inputs(const OpenDataflowGraphView &g, const std::set<int> &nodes) {
  std::set<OpenDataflowValue> r;
  for (int n : nodes)
    for (auto &v : g.get_inputs(n))
      if (!(std::holds_alternative<DataflowOutput>(v) && nodes.count(std::get<DataflowOutput>(v).node))) r.insert(v);
  return r;
}
// edges from nodes outside the set to nodes inside it
inline std::set<DataflowEdge> get_subgraph_incoming_edges(const OpenDataflowGraphView &g, const std::set<int> &nodes) {
  std::set<DataflowEdge> r;
  for (auto &e : g.query_edges())
    if (nodes.count(e.dst.node) && !nodes.count(e.src.node)) r.insert(e);
  return r;
}
inline std::set<DataflowEdge> get_subgraph_outgoing_dataflow_edges(const OpenDataflowGraphView &g, const std::set<int> &nodes) {
  std::set<DataflowEdge> r;
  for (auto &e : g.query_edges())
    if (nodes.count(e.src.node) && !nodes.count(e.dst.node)) r.insert(e);
  return r;
}
// the same graph with nodes (inputs) renumbered; the maps must be injective and cover every node (input)
OpenDataflowGraph permute_node_ids(const OpenDataflowGraphView &g, const std::map<int, int> &new_of_old, std::map<int, int> *assigned = nullptr);
OpenDataflowGraph permute_input_ids(const OpenDataflowGraphView &g, const std::map<int, int> &new_of_old);
// does `node_map` (nodes of a -> nodes of b) together with `input_map` carry a onto b: same operands in the same order?
bool is_isomorphic_under(const OpenDataflowGraphView &a, const OpenDataflowGraphView &b, const std::map<int, int> &node_map,
                         const std::map<int, int> &input_map);
std::string open_dataflow_graph_as_dot(const OpenDataflowGraphView &g);

// closed graphs: the open graph without graph inputs
class DataflowGraphView : public OpenDataflowGraphView {};
class DataflowGraph : public OpenDataflowGraph {
public:
  NodeAddedResult add_node(const std::vector<DataflowOutput> &inputs, int num_outputs) {
    std::vector<OpenDataflowValue> v(inputs.begin(), inputs.end());
    return OpenDataflowGraph::add_node(v, num_outputs);
  }
};

// ---------------------------------------------------------------------------------------------- named slots
// Inputs and outputs of a node are named (SlotName = the operator slots of the IR, or any ordered key type).
template <typename Slot>
class KwargDataflowGraph {
public:
  struct Output {
    int node;
    Slot slot;
    bool operator<(const Output &o) const { return std::tie(node, slot) < std::tie(o.node, o.slot); }
    bool operator==(const Output &o) const { return node == o.node && slot == o.slot; }
  };
  struct Added {
    int node;
    std::map<Slot, Output> outputs;
  };
  Added add_node(const std::map<Slot, Output> &inputs, const std::vector<Slot> &output_slots) {
    std::vector<OpenDataflowValue> operands;
    std::vector<Slot> in_names;
    for (auto &kv : inputs) {
      auto it = out_index_.find(kv.second);
      if (it == out_index_.end()) throw std::invalid_argument("add_node: operand is not a value of this graph");
      operands.push_back(DataflowOutput{kv.second.node, it->second});
      in_names.push_back(kv.first);
    }
    if (std::set<Slot>(output_slots.begin(), output_slots.end()).size() != output_slots.size())
      throw std::invalid_argument("add_node: duplicate output slot");
    NodeAddedResult r = g_.add_node(operands, (int)output_slots.size());
    in_slots_[r.node] = in_names;
    out_slots_[r.node] = output_slots;
    Added a{r.node, {}};
    for (size_t i = 0; i < output_slots.size(); ++i) {
      Output o{r.node, output_slots[i]};
      out_index_[o] = (int)i;
      a.outputs[output_slots[i]] = o;
    }
    return a;
  }
  std::vector<int> get_nodes() const { return g_.get_nodes(); }
  std::map<Slot, Output> get_inputs(int node) const {
    std::map<Slot, Output> r;
    const auto &ops = g_.get_inputs(node);
    const auto &names = in_slots_.at(node);
    for (size_t i = 0; i < ops.size(); ++i) {
      const DataflowOutput &o = std::get<DataflowOutput>(ops[i]);
      r[names[i]] = Output{o.node, out_slots_.at(o.node)[(size_t)o.idx]};
    }
    return r;
  }
  std::vector<Slot> get_output_slots(int node) const { return out_slots_.at(node); }
  const OpenDataflowGraphView &positional() const { return g_; }  // the same graph with positions instead of names

private:
  OpenDataflowGraph g_;
  std::map<int, std::vector<Slot>> in_slots_, out_slots_;
  std::map<Output, int> out_index_;
};

// ---------------------------------------------------------------------------------------------- labels
template <typename NodeLabel, typename ValueLabel>
class LabelledOpenDataflowGraph {
public:
  DataflowGraphInput add_input(const ValueLabel &l) {
    DataflowGraphInput i = g_.add_input();
    input_labels_[i.idx] = l;
    return i;
  }
  NodeAddedResult add_node(const NodeLabel &label, const std::vector<OpenDataflowValue> &inputs, const std::vector<ValueLabel> &output_labels) {
    NodeAddedResult r = g_.add_node(inputs, (int)output_labels.size());
    node_labels_[r.node] = label;
    for (size_t i = 0; i < output_labels.size(); ++i) value_labels_[r.outputs[i]] = output_labels[i];
    return r;
  }
  const NodeLabel &at(int node) const { return node_labels_.at(node); }
  const ValueLabel &at(const OpenDataflowValue &v) const {
    if (std::holds_alternative<DataflowOutput>(v)) return value_labels_.at(std::get<DataflowOutput>(v));
    return input_labels_.at(std::get<DataflowGraphInput>(v).idx);
  }
  const OpenDataflowGraphView &raw() const { return g_; }
  // relabel without touching the topology (the reference's rewrite_node_labels / rewrite_value_labels)
  template <typename F>
  auto rewrite_node_labels(F f) const {
    using L2 = decltype(f(0, std::declval<NodeLabel>()));
    LabelledOpenDataflowGraph<L2, ValueLabel> out;
    out.adopt(g_, input_labels_, value_labels_);
    for (auto &kv : node_labels_) out.set_node_label(kv.first, f(kv.first, kv.second));
    return out;
  }
  void adopt(const OpenDataflowGraph &g, const std::map<int, ValueLabel> &il, const std::map<DataflowOutput, ValueLabel> &vl) {
    g_ = g;
    input_labels_ = il;
    value_labels_ = vl;
  }
  void set_node_label(int n, const NodeLabel &l) { node_labels_[n] = l; }

private:
  OpenDataflowGraph g_;
  std::map<int, NodeLabel> node_labels_;
  std::map<int, ValueLabel> input_labels_;
  std::map<DataflowOutput, ValueLabel> value_labels_;
};
template <typename NodeLabel, typename ValueLabel>
using LabelledDataflowGraph = LabelledOpenDataflowGraph<NodeLabel, ValueLabel>;  // closed = never given a graph input

// Are two (open) dataflow graphs the same up to a renaming of nodes and graph inputs?  Returns the node bijection.
// Backtracking over the topological order; meant for the small graphs of patterns and tests.
std::optional<std::map<int, int>> find_dataflow_isomorphism(const OpenDataflowGraphView &a, const OpenDataflowGraphView &b);

// ---------------------------------------------------------------------------------------------- command lines
struct CLIFlagSpec {
  std::string long_flag;
  std::optional<char> short_flag;
  std::optional<std::string> description;
};
struct CLIPositionalArgumentSpec {
  std::string name;
  std::optional<std::vector<std::string>> choices;
  std::optional<std::string> description;
};
struct CLIFlagKey { int raw_idx; bool operator<(const CLIFlagKey &o) const { return raw_idx < o.raw_idx; } };
struct CLIPositionalArgumentKey { int raw_idx; bool operator<(const CLIPositionalArgumentKey &o) const { return raw_idx < o.raw_idx; } };
using CLIArgumentKey = std::variant<CLIFlagKey, CLIPositionalArgumentKey>;
struct CLISpec {
  std::vector<CLIFlagSpec> flags;
  std::vector<CLIPositionalArgumentSpec> positional_arguments;
};
struct CLIParseResult {
  std::map<CLIFlagKey, bool> flags;
  std::map<CLIPositionalArgumentKey, std::string> positional_arguments;
};
struct CLIParseOutcome {  // a parse result or an error message (the reference returns tl::expected)
  std::optional<CLIParseResult> result;
  std::string error;
  bool ok() const { return result.has_value(); }
};

CLISpec empty_cli_spec();
CLIArgumentKey cli_add_help_flag(CLISpec &);
CLIArgumentKey cli_add_flag(CLISpec &, const CLIFlagSpec &);
CLIArgumentKey cli_add_positional_argument(CLISpec &, const CLIPositionalArgumentSpec &);
std::vector<CLIFlagKey> cli_get_flag_keys(const CLISpec &);
CLIParseOutcome cli_parse(const CLISpec &, const std::vector<std::string> &args);  // args[0] is the program name
bool cli_get_flag(const CLIParseResult &, const CLIArgumentKey &);
std::string cli_get_argument(const CLIParseResult &, const CLIArgumentKey &);
std::string cli_get_help_message(const std::string &program_name, const CLISpec &);

}  // namespace ff
