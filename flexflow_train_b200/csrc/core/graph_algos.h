// graph_algos.h -- directed-graph algorithms, series-parallel decomposition and SP-ization.
//
// Counterpart of lib/utils/include/utils/graph/digraph/algorithms/*.h,
// lib/utils/src/utils/graph/series_parallel/get_series_parallel_decomposition.cc:24-110 and
// lib/utils/include/utils/graph/series_parallel/sp_ization/*.
#pragma once
#include <functional>
#include <map>
#include <optional>
#include <set>
#include <string>
#include <vector>

#include "json.h"

namespace ff {

class DiGraph {
public:
  void add_node(int n) { succ_[n]; pred_[n]; }
  void add_edge(int a, int b) { add_node(a); add_node(b); succ_[a].insert(b); pred_[b].insert(a); }
  void remove_edge(int a, int b) { succ_[a].erase(b); pred_[b].erase(a); }
  bool has_edge(int a, int b) const { auto it = succ_.find(a); return it != succ_.end() && it->second.count(b); }
  bool has_node(int n) const { return succ_.count(n) > 0; }
  std::vector<int> nodes() const;
  std::vector<std::pair<int, int>> edges() const;
  const std::set<int> &successors(int n) const { return succ_.at(n); }
  const std::set<int> &predecessors(int n) const { return pred_.at(n); }
  size_t num_nodes() const { return succ_.size(); }
  size_t num_edges() const;
  std::vector<int> sources() const;
  std::vector<int> sinks() const;

private:
  std::map<int, std::set<int>> succ_, pred_;
};

bool is_acyclic(const DiGraph &g);
std::vector<int> topological_ordering(const DiGraph &g);  // throws on cycles
DiGraph transitive_closure(const DiGraph &g);
DiGraph transitive_reduction(const DiGraph &g);
std::map<int, std::set<int>> get_dominators(const DiGraph &g);       // node -> its dominators (incl. itself)
std::map<int, std::set<int>> get_post_dominators(const DiGraph &g);
std::optional<int> get_imm_dominator(const DiGraph &g, int n);
std::vector<std::set<int>> get_weakly_connected_components(const DiGraph &g);
std::map<int, int> get_longest_path_lengths_from_root(const DiGraph &g);  // unit weights, roots at 0... depth
std::map<int, double> get_weighted_longest_path_lengths(const DiGraph &g, const std::function<double(int)> &cost);
std::set<int> get_descendants(const DiGraph &g, int n);
std::set<int> get_ancestors(const DiGraph &g, int n);
std::optional<int> get_lowest_common_ancestor(const DiGraph &g, const std::set<int> &nodes);
bool is_2_terminal_dag(const DiGraph &g);
// more of lib/utils/include/utils/graph/digraph/algorithms/*.h
DiGraph flipped(const DiGraph &g);                                       // every edge reversed
std::map<int, std::set<int>> get_strict_dominators(const DiGraph &g);    // dominators without the node itself
std::map<int, std::optional<int>> get_imm_dominators_map(const DiGraph &g);
std::optional<int> get_imm_post_dominator(const DiGraph &g, int n);
std::map<int, std::optional<int>> get_imm_post_dominators_map(const DiGraph &g);
std::map<int, int> calculate_topo_rank(const DiGraph &g);                // position in the topological order
std::optional<int> get_node_with_greatest_topo_rank(const std::set<int> &nodes, const DiGraph &g);
std::vector<int> get_topological_ordering_from_starting_node(const DiGraph &g, int start);   // start and its descendants
std::vector<std::pair<int, int>> get_edge_topological_ordering(const DiGraph &g);           // by source in topological order
bool is_tree(const DiGraph &g);                                          // one root, connected, |E| = |V| - 1
std::set<std::pair<int, int>> get_edges_from_subgraph_to_subgraph(const DiGraph &g, const std::set<int> &src, const std::set<int> &dst);
std::set<std::pair<int, int>> get_subgraph_outgoing_edges(const DiGraph &g, const std::set<int> &sub);   // edges leaving the node set
std::set<int> get_subgraph_successors(const DiGraph &g, const std::set<int> &sub);                       // their heads
// Nodes merged along `into` (node -> node it is merged into, chains followed to their end); edges follow their endpoints,
// so an edge inside a merged group becomes a self loop.
DiGraph apply_contraction(const DiGraph &g, const std::map<int, int> &into);
DiGraph contract_node(const DiGraph &g, int from, int into);
// The graph without the nodes that `drop` picks: a -> b wherever there was a path from a to b through dropped nodes only
// (the auxiliary nodes of the SP-ization algorithms leave this way; sp_ization/node_role.h, contract_out_nodes_of_given_role).
DiGraph bridge_out_nodes(const DiGraph &g, const std::function<bool(int)> &drop);
bool is_complete_bipartite_digraph(const DiGraph &g);                    // every source has an edge to every sink and nothing else
std::string digraph_as_dot(const DiGraph &g);

// Series-parallel decomposition tree.  N-ary after normalisation; binary variants keep exactly two children.
struct SPTree {
  enum Kind { Leaf, Series, Parallel } kind = Leaf;
  int node = -1;
  std::vector<SPTree> children;
  static SPTree leaf(int n) { SPTree t; t.kind = Leaf; t.node = n; return t; }
  static SPTree series(std::vector<SPTree> c) { SPTree t; t.kind = Series; t.children = std::move(c); return t; }
  static SPTree parallel(std::vector<SPTree> c) { SPTree t; t.kind = Parallel; t.children = std::move(c); return t; }
  bool operator==(const SPTree &o) const;
  std::string str() const;
};
SPTree normalize_sp(const SPTree &t);                    // flatten nested same-kind nodes, drop single-child nodes
std::vector<int> sp_nodes(const SPTree &t);              // leaves in order (with multiplicity)
bool sp_is_binary(const SPTree &t);
SPTree left_associative_binary_sp_tree(const SPTree &nary);
SPTree right_associative_binary_sp_tree(const SPTree &nary);
SPTree balanced_binary_sp_tree(const SPTree &nary);      // balanced_binary_sp_tree_from_nary.h
double sp_work_cost(const SPTree &t, const std::function<double(int)> &cost);
double sp_critical_path_cost(const SPTree &t, const std::function<double(int)> &cost);
// Every node the tree orders before `node` (before any of its occurrences, if work was duplicated);
// lib/utils/include/utils/graph/series_parallel/get_ancestors.h
std::set<int> sp_ancestors(const SPTree &t, int node);
DiGraph digraph_from_sp(const SPTree &t);                // the dependencies the tree implies
Json sp_to_json(const SPTree &binary);                   // {"type": series|parallel|leaf, left_child, right_child, value}
SPTree sp_from_json(const Json &j);

// TTSP-reduction based decomposition; nullopt when the (transitively reduced) graph is not series-parallel.
std::optional<SPTree> get_series_parallel_decomposition(const DiGraph &g);

// SP-ization: produce an SP tree whose dependencies are a superset of the DAG's.
SPTree naive_stratum_sync_sp_ization(const DiGraph &g);
SPTree work_duplicating_sp_ization(const DiGraph &g, bool coalesce);
SPTree escribano_sp_ization(const DiGraph &g);
SPTree flexible_sp_ization(const DiGraph &g, const std::function<double(int)> &cost);
// true iff every dependency a->b of g is enforced by t (every occurrence of b comes after some occurrence of a)
bool sp_preserves_dependencies(const SPTree &t, const DiGraph &g);

}  // namespace ff
