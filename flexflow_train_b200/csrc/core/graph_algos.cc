#include "graph_algos.h"

#include <algorithm>
#include <queue>
#include <sstream>
#include <stdexcept>

namespace ff {

std::vector<int> DiGraph::nodes() const {
  std::vector<int> r;
  for (auto &kv : succ_) r.push_back(kv.first);
  return r;
}
std::vector<std::pair<int, int>> DiGraph::edges() const {
  std::vector<std::pair<int, int>> r;
  for (auto &kv : succ_) for (int b : kv.second) r.push_back({kv.first, b});
  return r;
}
size_t DiGraph::num_edges() const {
  size_t n = 0;
  for (auto &kv : succ_) n += kv.second.size();
  return n;
}
std::vector<int> DiGraph::sources() const {
  std::vector<int> r;
  for (auto &kv : pred_) if (kv.second.empty()) r.push_back(kv.first);
  return r;
}
std::vector<int> DiGraph::sinks() const {
  std::vector<int> r;
  for (auto &kv : succ_) if (kv.second.empty()) r.push_back(kv.first);
  return r;
}

static bool topo_impl(const DiGraph &g, std::vector<int> &order) {
  std::map<int, int> indeg;
  for (int n : g.nodes()) indeg[n] = (int)g.predecessors(n).size();
  std::priority_queue<int, std::vector<int>, std::greater<int>> ready;
  for (auto &kv : indeg) if (kv.second == 0) ready.push(kv.first);
  while (!ready.empty()) {
    int n = ready.top();
    ready.pop();
    order.push_back(n);
    for (int s : g.successors(n)) if (--indeg[s] == 0) ready.push(s);
  }
  return order.size() == g.num_nodes();
}
bool is_acyclic(const DiGraph &g) {
  std::vector<int> o;
  return topo_impl(g, o);
}
std::vector<int> topological_ordering(const DiGraph &g) {
  std::vector<int> o;
  if (!topo_impl(g, o)) throw std::runtime_error("topological_ordering: graph has a cycle");
  return o;
}
std::set<int> get_descendants(const DiGraph &g, int n) {
  std::set<int> seen;
  std::vector<int> stack(g.successors(n).begin(), g.successors(n).end());
  while (!stack.empty()) {
    int x = stack.back();
    stack.pop_back();
    if (!seen.insert(x).second) continue;
    for (int s : g.successors(x)) stack.push_back(s);
  }
  return seen;
}
std::set<int> get_ancestors(const DiGraph &g, int n) {
  std::set<int> seen;
  std::vector<int> stack(g.predecessors(n).begin(), g.predecessors(n).end());
  while (!stack.empty()) {
    int x = stack.back();
    stack.pop_back();
    if (!seen.insert(x).second) continue;
    for (int s : g.predecessors(x)) stack.push_back(s);
  }
  return seen;
}
DiGraph transitive_closure(const DiGraph &g) {
  DiGraph r;
  auto order = topological_ordering(g);
  std::map<int, std::set<int>> desc;
  for (auto it = order.rbegin(); it != order.rend(); ++it) {
    std::set<int> d;
    for (int s : g.successors(*it)) {
      d.insert(s);
      d.insert(desc[s].begin(), desc[s].end());
    }
    desc[*it] = d;
  }
  for (int n : order) {
    r.add_node(n);
    for (int d : desc[n]) r.add_edge(n, d);
  }
  return r;
}
DiGraph transitive_reduction(const DiGraph &g) {
  // an edge a->b is redundant iff b is reachable from another successor of a
  DiGraph r;
  auto order = topological_ordering(g);
  std::map<int, std::set<int>> desc;
  for (auto it = order.rbegin(); it != order.rend(); ++it) {
    std::set<int> d;
    for (int s : g.successors(*it)) {
      d.insert(s);
      d.insert(desc[s].begin(), desc[s].end());
    }
    desc[*it] = d;
  }
  for (int a : order) {
    r.add_node(a);
    for (int b : g.successors(a)) {
      bool redundant = false;
      for (int c : g.successors(a))
        if (c != b && desc[c].count(b)) { redundant = true; break; }
      if (!redundant) r.add_edge(a, b);
    }
  }
  return r;
}
static std::map<int, std::set<int>> dominators_impl(const DiGraph &g, bool post) {
  auto order = topological_ordering(g);
  if (post) std::reverse(order.begin(), order.end());
  std::map<int, std::set<int>> dom;
  for (int n : order) {
    const std::set<int> &ps = post ? g.successors(n) : g.predecessors(n);
    std::set<int> d;
    bool first = true;
    for (int p : ps) {
      if (first) { d = dom[p]; first = false; }
      else {
        std::set<int> t;
        std::set_intersection(d.begin(), d.end(), dom[p].begin(), dom[p].end(), std::inserter(t, t.begin()));
        d = t;
      }
    }
    d.insert(n);
    dom[n] = d;
  }
  return dom;
}
std::map<int, std::set<int>> get_dominators(const DiGraph &g) { return dominators_impl(g, false); }
std::map<int, std::set<int>> get_post_dominators(const DiGraph &g) { return dominators_impl(g, true); }
std::optional<int> get_imm_dominator(const DiGraph &g, int n) {
  auto dom = get_dominators(g);
  auto depth = get_longest_path_lengths_from_root(g);
  std::optional<int> best;
  for (int d : dom[n]) {
    if (d == n) continue;
    if (!best || depth[d] > depth[*best]) best = d;
  }
  return best;
}
std::vector<std::set<int>> get_weakly_connected_components(const DiGraph &g) {
  std::set<int> seen;
  std::vector<std::set<int>> comps;
  for (int n : g.nodes()) {
    if (seen.count(n)) continue;
    std::set<int> comp;
    std::vector<int> stack{n};
    while (!stack.empty()) {
      int x = stack.back();
      stack.pop_back();
      if (!comp.insert(x).second) continue;
      for (int s : g.successors(x)) stack.push_back(s);
      for (int p : g.predecessors(x)) stack.push_back(p);
    }
    seen.insert(comp.begin(), comp.end());
    comps.push_back(comp);
  }
  return comps;
}
std::map<int, int> get_longest_path_lengths_from_root(const DiGraph &g) {
  std::map<int, int> d;
  for (int n : topological_ordering(g)) {
    int v = 0;
    for (int p : g.predecessors(n)) v = std::max(v, d[p] + 1);
    d[n] = v;
  }
  return d;
}
std::map<int, double> get_weighted_longest_path_lengths(const DiGraph &g, const std::function<double(int)> &cost) {
  std::map<int, double> d;
  for (int n : topological_ordering(g)) {
    double v = 0;
    for (int p : g.predecessors(n)) v = std::max(v, d[p]);
    d[n] = v + cost(n);
  }
  return d;
}
std::optional<int> get_lowest_common_ancestor(const DiGraph &g, const std::set<int> &nodes) {
  if (nodes.empty()) return std::nullopt;
  std::set<int> common;
  bool first = true;
  for (int n : nodes) {
    std::set<int> a = get_ancestors(g, n);
    a.insert(n);
    if (first) { common = a; first = false; }
    else {
      std::set<int> t;
      std::set_intersection(common.begin(), common.end(), a.begin(), a.end(), std::inserter(t, t.begin()));
      common = t;
    }
  }
  if (common.empty()) return std::nullopt;
  auto depth = get_longest_path_lengths_from_root(g);
  int best = *common.begin();
  for (int c : common) if (depth[c] > depth[best]) best = c;
  return best;
}
bool is_2_terminal_dag(const DiGraph &g) { return is_acyclic(g) && g.sources().size() == 1 && g.sinks().size() == 1; }

// ---------------------------------------------------------------- SP trees
bool SPTree::operator==(const SPTree &o) const {
  if (kind != o.kind) return false;
  if (kind == Leaf) return node == o.node;
  if (children.size() != o.children.size()) return false;
  if (kind == Series) return children == o.children;
  // parallel children are unordered
  std::vector<bool> used(o.children.size(), false);
  for (auto &c : children) {
    bool found = false;
    for (size_t i = 0; i < o.children.size(); ++i)
      if (!used[i] && c == o.children[i]) { used[i] = true; found = true; break; }
    if (!found) return false;
  }
  return true;
}

DiGraph flipped(const DiGraph &g) {
  DiGraph r;
  for (int n : g.nodes()) r.add_node(n);
  for (auto &e : g.edges()) r.add_edge(e.second, e.first);
  return r;
}
std::map<int, std::set<int>> get_strict_dominators(const DiGraph &g) {
  auto d = get_dominators(g);
  for (auto &kv : d) kv.second.erase(kv.first);
  return d;
}
std::map<int, std::optional<int>> get_imm_dominators_map(const DiGraph &g) {
  std::map<int, std::optional<int>> out;
  for (int n : g.nodes()) out[n] = get_imm_dominator(g, n);
  return out;
}
std::optional<int> get_imm_post_dominator(const DiGraph &g, int n) { return get_imm_dominator(flipped(g), n); }
std::map<int, std::optional<int>> get_imm_post_dominators_map(const DiGraph &g) { return get_imm_dominators_map(flipped(g)); }
std::map<int, int> calculate_topo_rank(const DiGraph &g) {
  std::map<int, int> rank;
  int i = 0;
  for (int n : topological_ordering(g)) rank[n] = i++;
  return rank;
}
std::optional<int> get_node_with_greatest_topo_rank(const std::set<int> &nodes, const DiGraph &g) {
  auto rank = calculate_topo_rank(g);
  std::optional<int> best;
  for (int n : nodes)
    if (!best || rank.at(n) > rank.at(*best)) best = n;
  return best;
}
std::vector<int> get_topological_ordering_from_starting_node(const DiGraph &g, int start) {
  if (!is_acyclic(g)) throw std::runtime_error("topological ordering of a graph with a cycle");
  std::set<int> keep = get_descendants(g, start);
  keep.insert(start);
  std::vector<int> out;
  for (int n : topological_ordering(g))
    if (keep.count(n)) out.push_back(n);
  return out;
}
std::vector<std::pair<int, int>> get_edge_topological_ordering(const DiGraph &g) {
  std::vector<std::pair<int, int>> out;
  for (int n : topological_ordering(g))
    for (int s2 : g.successors(n)) out.push_back({n, s2});
  return out;
}
bool is_tree(const DiGraph &g) {
  if (g.num_nodes() == 0) throw std::runtime_error("is_tree of an empty graph");
  return g.sources().size() == 1 && get_weakly_connected_components(g).size() == 1 && g.num_edges() == g.num_nodes() - 1;
}
std::set<std::pair<int, int>> get_edges_from_subgraph_to_subgraph(const DiGraph &g, const std::set<int> &src, const std::set<int> &dst) {
  for (int n : src)
    if (dst.count(n)) throw std::runtime_error("the two node sets overlap");
  std::set<std::pair<int, int>> out;
  for (int a : src)
    if (g.has_node(a))
      for (int b : g.successors(a))
        if (dst.count(b)) out.insert({a, b});
  return out;
}
std::set<std::pair<int, int>> get_subgraph_outgoing_edges(const DiGraph &g, const std::set<int> &sub) {
  std::set<std::pair<int, int>> out;
  for (int a : sub)
    if (g.has_node(a))
      for (int b : g.successors(a))
        if (!sub.count(b)) out.insert({a, b});
  return out;
}
std::set<int> get_subgraph_successors(const DiGraph &g, const std::set<int> &sub) {
  std::set<int> out;
  for (auto &e : get_subgraph_outgoing_edges(g, sub)) out.insert(e.second);
  return out;
}
DiGraph apply_contraction(const DiGraph &g, const std::map<int, int> &into) {
  auto final_of = [&](int n) {
    std::set<int> seen;
    while (true) {
      auto it = into.find(n);
      if (it == into.end() || it->second == n) return n;
      if (!seen.insert(n).second) throw std::runtime_error("contraction map has a cycle");
      n = it->second;
    }
  };
  DiGraph r;
  for (int n : g.nodes()) r.add_node(final_of(n));
  for (auto &e : g.edges()) r.add_edge(final_of(e.first), final_of(e.second));
  return r;
}
DiGraph contract_node(const DiGraph &g, int from, int into) { return apply_contraction(g, {{from, into}}); }
bool is_complete_bipartite_digraph(const DiGraph &g) {
  auto src = g.sources(), snk = g.sinks();
  std::set<int> s(src.begin(), src.end()), t(snk.begin(), snk.end());
  if (s.size() + t.size() != g.num_nodes()) return false;
  for (int n : s)
    if (t.count(n)) return false;          // an isolated node is a source and a sink at once
  for (int a : s)
    for (int b : t)
      if (!g.has_edge(a, b)) return false;
  return g.num_edges() == s.size() * t.size();
}
std::string digraph_as_dot(const DiGraph &g) {
  std::string out = "digraph {\n";
  for (int n : g.nodes()) out += "  n" + std::to_string(n) + " [label=\"" + std::to_string(n) + "\"];\n";
  for (auto &e : g.edges()) out += "  n" + std::to_string(e.first) + " -> n" + std::to_string(e.second) + ";\n";
  return out + "}\n";
}
std::string SPTree::str() const {
  if (kind == Leaf) return std::to_string(node);
  std::string s = kind == Series ? "S(" : "P(";
  for (size_t i = 0; i < children.size(); ++i) s += (i ? " " : "") + children[i].str();
  return s + ")";
}
SPTree normalize_sp(const SPTree &t) {
  if (t.kind == SPTree::Leaf) return t;
  std::vector<SPTree> flat;
  for (auto &c : t.children) {
    SPTree n = normalize_sp(c);
    if (n.kind != SPTree::Leaf && n.children.empty()) continue;   // a split with nothing in it goes
    if (n.kind == t.kind) flat.insert(flat.end(), n.children.begin(), n.children.end());
    else flat.push_back(n);
  }
  if (flat.size() == 1) return flat[0];
  SPTree r;
  r.kind = t.kind;
  r.children = flat;
  return r;
}
std::vector<int> sp_nodes(const SPTree &t) {
  if (t.kind == SPTree::Leaf) return {t.node};
  std::vector<int> r;
  for (auto &c : t.children) {
    auto v = sp_nodes(c);
    r.insert(r.end(), v.begin(), v.end());
  }
  return r;
}
bool sp_is_binary(const SPTree &t) {
  if (t.kind == SPTree::Leaf) return true;
  if (t.children.size() != 2) return false;
  return sp_is_binary(t.children[0]) && sp_is_binary(t.children[1]);
}
static SPTree binarize(const SPTree &t, int mode);
static SPTree combine_range(SPTree::Kind k, const std::vector<SPTree> &c, size_t lo, size_t hi, int mode) {
  if (hi - lo == 1) return c[lo];
  SPTree r;
  r.kind = k;
  if (mode == 0) {  // left associative
    r.children = {combine_range(k, c, lo, hi - 1, mode), c[hi - 1]};
  } else if (mode == 1) {  // right associative
    r.children = {c[lo], combine_range(k, c, lo + 1, hi, mode)};
  } else {  // balanced
    size_t mid = lo + (hi - lo) / 2;
    r.children = {combine_range(k, c, lo, mid, mode), combine_range(k, c, mid, hi, mode)};
  }
  return r;
}
static SPTree binarize(const SPTree &t, int mode) {
  if (t.kind == SPTree::Leaf) return t;
  std::vector<SPTree> c;
  for (auto &x : t.children) c.push_back(binarize(x, mode));
  if (c.size() == 1) return c[0];
  return combine_range(t.kind, c, 0, c.size(), mode);
}
SPTree left_associative_binary_sp_tree(const SPTree &n) { return binarize(normalize_sp(n), 0); }
SPTree right_associative_binary_sp_tree(const SPTree &n) { return binarize(normalize_sp(n), 1); }
SPTree balanced_binary_sp_tree(const SPTree &n) { return binarize(normalize_sp(n), 2); }
double sp_work_cost(const SPTree &t, const std::function<double(int)> &cost) {
  if (t.kind == SPTree::Leaf) return cost(t.node);
  double s = 0;
  for (auto &c : t.children) s += sp_work_cost(c, cost);
  return s;
}
double sp_critical_path_cost(const SPTree &t, const std::function<double(int)> &cost) {
  if (t.kind == SPTree::Leaf) return cost(t.node);
  double s = 0;
  for (auto &c : t.children) {
    double v = sp_critical_path_cost(c, cost);
    s = t.kind == SPTree::Series ? s + v : std::max(s, v);
  }
  return s;
}
static void sp_ends(const SPTree &t, std::vector<int> &firsts, std::vector<int> &lasts) {
  if (t.kind == SPTree::Leaf) { firsts.push_back(t.node); lasts.push_back(t.node); return; }
  if (t.kind == SPTree::Parallel) {
    for (auto &c : t.children) sp_ends(c, firsts, lasts);
    return;
  }
  std::vector<int> dummy;
  sp_ends(t.children.front(), firsts, dummy);
  dummy.clear();
  sp_ends(t.children.back(), dummy, lasts);
}
static void sp_edges(const SPTree &t, DiGraph &g) {
  if (t.kind == SPTree::Leaf) { g.add_node(t.node); return; }
  for (auto &c : t.children) sp_edges(c, g);
  if (t.kind == SPTree::Series) {
    for (size_t i = 0; i + 1 < t.children.size(); ++i) {
      std::vector<int> f, l, f2, l2;
      sp_ends(t.children[i], f, l);
      sp_ends(t.children[i + 1], f2, l2);
      for (int a : l) for (int b : f2) g.add_edge(a, b);
    }
  }
}
DiGraph digraph_from_sp(const SPTree &t) {
  DiGraph g;
  sp_edges(t, g);
  return g;
}
Json sp_to_json(const SPTree &t) {
  Json j = Json::object();
  if (t.kind == SPTree::Leaf) {
    j["type"] = "leaf";
    j["value"] = t.node;
    return j;
  }
  if (t.children.size() != 2) throw std::runtime_error("sp_to_json: tree must be binary");
  j["type"] = t.kind == SPTree::Series ? "series" : "parallel";
  j["left_child"] = sp_to_json(t.children[0]);
  j["right_child"] = sp_to_json(t.children[1]);
  return j;
}
SPTree sp_from_json(const Json &j) {
  std::string ty = j.at("type").as_string();
  if (ty == "leaf") return SPTree::leaf((int)j.at("value").as_int());
  SPTree t;
  if (ty == "series") t.kind = SPTree::Series;
  else if (ty == "parallel") t.kind = SPTree::Parallel;
  else throw std::runtime_error("sp_from_json: unknown type '" + ty + "'");
  t.children = {sp_from_json(j.at("left_child")), sp_from_json(j.at("right_child"))};
  return t;
}

// ---------------------------------------------------------------- TTSP decomposition
// Build the inverse line graph of the transitively reduced DAG: every node becomes an edge between
// two "junction" vertices.  It exists iff nodes that share a successor share all successors and the
// members of that successor set share all predecessors (complete bipartite components).
std::optional<SPTree> get_series_parallel_decomposition(const DiGraph &g_in) {
  if (g_in.num_nodes() == 0) return std::nullopt;
  if (!is_acyclic(g_in)) return std::nullopt;
  DiGraph g = transitive_reduction(g_in);
  if (g.num_nodes() == 1) return SPTree::leaf(g.nodes()[0]);

  std::map<std::set<int>, int> junction_of_succset;
  const int SRC = 0, SNK = 1;
  int next_junction = 2;
  for (int n : g.nodes()) {
    const std::set<int> &s = g.successors(n);
    if (s.empty()) continue;
    if (!junction_of_succset.count(s)) junction_of_succset[s] = next_junction++;
  }
  // heads of each junction
  std::map<int, std::set<int>> heads;
  for (int n : g.nodes()) {
    const std::set<int> &s = g.successors(n);
    if (!s.empty()) heads[junction_of_succset[s]].insert(n);
  }
  // each tail of a junction must have exactly the junction's heads as predecessors
  for (auto &kv : junction_of_succset)
    for (int t : kv.first)
      if (g.predecessors(t) != heads[kv.second]) return std::nullopt;

  // Series and parallel reductions of the two-terminal multigraph, driven by a work list: a junction with one edge in and
  // one edge out is spliced away; two edges between the same pair of junctions merge into one.  Labels are moved, never
  // copied, so the whole reduction is near linear in the number of operators.
  struct Edge { int u, v; SPTree label; bool alive; };
  std::vector<Edge> edges;
  std::map<int, std::set<size_t>> in_e, out_e;
  std::map<std::pair<int, int>, size_t> between;  // the one alive edge between a pair of junctions
  std::vector<int> work;
  std::function<void(Edge)> add_edge = [&](Edge e) {
    auto key = std::make_pair(e.u, e.v);
    auto it = between.find(key);
    if (it != between.end()) {  // parallel reduction with the edge already there
      Edge &o = edges[it->second];
      std::vector<SPTree> cs;
      cs.push_back(std::move(o.label));
      cs.push_back(std::move(e.label));
      o.label = SPTree::parallel(std::move(cs));
      work.push_back(e.u);
      work.push_back(e.v);
      return;
    }
    const size_t id = edges.size();
    edges.push_back(std::move(e));
    between[key] = id;
    in_e[edges[id].v].insert(id);
    out_e[edges[id].u].insert(id);
    work.push_back(edges[id].u);
    work.push_back(edges[id].v);
  };
  for (int n : g.nodes()) {
    int u = g.predecessors(n).empty() ? SRC : junction_of_succset[g.successors(*g.predecessors(n).begin())];
    int v = g.successors(n).empty() ? SNK : junction_of_succset[g.successors(n)];
    add_edge({u, v, SPTree::leaf(n), true});
  }
  while (!work.empty()) {
    const int v = work.back();
    work.pop_back();
    if (v == SRC || v == SNK) continue;
    auto ii = in_e.find(v), oi = out_e.find(v);
    if (ii == in_e.end() || oi == out_e.end() || ii->second.size() != 1 || oi->second.size() != 1) continue;
    const size_t a = *ii->second.begin(), b = *oi->second.begin();
    if (a == b) continue;
    Edge ne{edges[a].u, edges[b].v, SPTree(), true};
    std::vector<SPTree> cs;
    cs.push_back(std::move(edges[a].label));
    cs.push_back(std::move(edges[b].label));
    ne.label = SPTree::series(std::move(cs));
    for (size_t dead : {a, b}) {
      edges[dead].alive = false;
      in_e[edges[dead].v].erase(dead);
      out_e[edges[dead].u].erase(dead);
      between.erase({edges[dead].u, edges[dead].v});
    }
    add_edge(std::move(ne));
  }
  std::vector<size_t> alive;
  for (size_t i = 0; i < edges.size(); ++i) if (edges[i].alive) alive.push_back(i);
  if (alive.size() != 1) return std::nullopt;
  return normalize_sp(edges[alive[0]].label);
}

// Walks down to `node`; on the way, a series split contributes all the children left of the one that holds the node.
static bool collect_sp_ancestors(const SPTree &t, int node, std::set<int> &out) {
  if (t.kind == SPTree::Leaf) return t.node == node;
  bool found = false;
  if (t.kind == SPTree::Parallel) {
    for (auto &c : t.children) found = collect_sp_ancestors(c, node, out) || found;
    return found;
  }
  std::set<int> before;
  for (auto &c : t.children) {
    std::set<int> inner;
    if (collect_sp_ancestors(c, node, inner)) {
      found = true;
      out.insert(before.begin(), before.end());
      out.insert(inner.begin(), inner.end());
    }
    for (int n : sp_nodes(c)) before.insert(n);
  }
  return found;
}
std::set<int> sp_ancestors(const SPTree &t, int node) {
  std::set<int> out;
  if (!collect_sp_ancestors(t, node, out)) throw std::runtime_error("sp_ancestors: node " + std::to_string(node) + " is not in the tree");
  return out;
}

// ---------------------------------------------------------------- SP-ization
SPTree naive_stratum_sync_sp_ization(const DiGraph &g) {
  auto depth = get_longest_path_lengths_from_root(g);
  std::map<int, std::vector<SPTree>> strata;
  for (auto &kv : depth) strata[kv.second].push_back(SPTree::leaf(kv.first));
  std::vector<SPTree> layers;
  for (auto &kv : strata) layers.push_back(SPTree::parallel(kv.second));
  return normalize_sp(SPTree::series(layers));
}

static SPTree coalesce_parallel(const SPTree &t) {
  // P(S(A, x), S(A, y), z) -> P(S(A, P(x, y)), z): factor a shared leading subtree out of parallel branches
  if (t.kind == SPTree::Leaf) return t;
  std::vector<SPTree> cs;
  for (auto &c : t.children) cs.push_back(coalesce_parallel(c));
  if (t.kind == SPTree::Series) return normalize_sp(SPTree::series(cs));
  bool merged = true;
  while (merged) {
    merged = false;
    for (size_t i = 0; i < cs.size() && !merged; ++i) {
      for (size_t j = i + 1; j < cs.size() && !merged; ++j) {
        auto head = [](const SPTree &s) -> const SPTree & { return s.kind == SPTree::Series ? s.children[0] : s; };
        auto rest = [](const SPTree &s) -> std::optional<SPTree> {
          if (s.kind != SPTree::Series) return std::nullopt;
          std::vector<SPTree> r(s.children.begin() + 1, s.children.end());
          return normalize_sp(SPTree::series(r));
        };
        if (head(cs[i]) == head(cs[j])) {
          std::vector<SPTree> tails;
          auto ri = rest(cs[i]), rj = rest(cs[j]);
          if (ri) tails.push_back(*ri);
          if (rj) tails.push_back(*rj);
          SPTree merged_t = tails.size() == 2 ? SPTree::series({head(cs[i]), coalesce_parallel(SPTree::parallel(tails))})
                            : tails.size() == 1 ? SPTree::series({head(cs[i]), tails[0]})
                                                : head(cs[i]);
          cs.erase(cs.begin() + j);
          cs[i] = normalize_sp(merged_t);
          merged = true;
        }
      }
    }
  }
  return normalize_sp(SPTree::parallel(cs));
}

SPTree work_duplicating_sp_ization(const DiGraph &g, bool coalesce) {
  // tree(n) = S(P(tree(p) for p in preds(n)), n); shared ancestors are duplicated.
  DiGraph r = transitive_reduction(g);
  std::map<int, SPTree> memo;
  for (int n : topological_ordering(r)) {
    std::vector<SPTree> ps;
    for (int p : r.predecessors(n)) ps.push_back(memo[p]);
    if (ps.empty()) memo[n] = SPTree::leaf(n);
    else memo[n] = normalize_sp(SPTree::series({SPTree::parallel(ps), SPTree::leaf(n)}));
  }
  std::vector<SPTree> roots;
  for (int s : r.sinks()) roots.push_back(memo[s]);
  SPTree t = normalize_sp(SPTree::parallel(roots));
  return coalesce ? coalesce_parallel(t) : t;
}

// Kept nodes of g with an edge a->b wherever g has a path from a to b whose inner nodes are all dropped.
DiGraph bridge_out_nodes(const DiGraph &g, const std::function<bool(int)> &drop) {
  DiGraph r;
  for (int n : g.nodes()) {
    if (drop(n)) continue;
    r.add_node(n);
    std::vector<int> stack(g.successors(n).begin(), g.successors(n).end());
    std::set<int> seen;
    while (!stack.empty()) {
      int x = stack.back();
      stack.pop_back();
      if (!seen.insert(x).second) continue;
      if (!drop(x)) { r.add_edge(n, x); continue; }
      for (int y : g.successors(x)) stack.push_back(y);
    }
  }
  return r;
}

static SPTree sp_without_leaves(const SPTree &t, const std::set<int> &gone) {
  if (t.kind == SPTree::Leaf) return t;
  SPTree r;
  r.kind = t.kind;
  for (auto &c : t.children) {
    if (c.kind == SPTree::Leaf && gone.count(c.node)) continue;
    SPTree k = sp_without_leaves(c, gone);
    if (k.kind != SPTree::Leaf && k.children.empty()) continue;
    r.children.push_back(k);
  }
  return r;
}

SPTree escribano_sp_ization(const DiGraph &g0) {
  // Local synchronisation of consecutive strata (after Escribano et al., "Mapping unstructured applications into
  // nested parallelism"): where the naive algorithm joins ALL nodes of one stratum with ALL nodes of the next, this
  // one joins only the nodes that the new dependencies actually tie together.
  //   1. every edge is made to span exactly one stratum by threading it through placeholder nodes;
  //   2. the series-parallel graph is grown one node at a time in breadth-first order.  The new node and its
  //      predecessors, together with whatever earlier joins between the last two strata they touch, form a class;
  //      the deepest common ancestor of the class is its handle, and every branch below the handle that reaches into
  //      the class is closed: all of those branches' nodes in the last stratum but one ("up") are joined to all of
  //      their nodes in the last stratum ("down") through one fresh join node;
  //   3. placeholders and join nodes are bridged out, and what is left is series-parallel by construction.
  // lib/utils/src/utils/graph/series_parallel/sp_ization/escribano_algo.cc:201-250 builds the same tree for
  // two-terminal graphs; here a graph with several sources or sinks first gets a common one, taken out again at the end.
  if (g0.num_nodes() == 0) return SPTree::parallel({});
  if (g0.num_nodes() == 1) return SPTree::leaf(g0.nodes()[0]);
  enum Role { Real, Placeholder, Join };
  std::map<int, Role> role;
  DiGraph g = g0;
  int next_id = 0;
  for (int n : g.nodes()) { role[n] = Real; next_id = std::max(next_id, n + 1); }
  std::set<int> added_terminals;
  if (g.sources().size() > 1) {
    int r = next_id++;
    for (int s : g.sources()) g.add_edge(r, s);
    role[r] = Real;
    added_terminals.insert(r);
  }
  if (g.sinks().size() > 1) {
    int t = next_id++;
    for (int s : g.sinks()) g.add_edge(s, t);
    role[t] = Real;
    added_terminals.insert(t);
  }
  std::map<int, int> depth = get_longest_path_lengths_from_root(g);
  for (auto &e : g.edges()) {
    int span = depth.at(e.second) - depth.at(e.first);
    if (span <= 1) continue;
    g.remove_edge(e.first, e.second);
    int prev = e.first;
    for (int i = 1; i < span; ++i) {
      int ph = next_id++;
      role[ph] = Placeholder;
      depth[ph] = depth.at(e.first) + i;
      g.add_edge(prev, ph);
      prev = ph;
    }
    g.add_edge(prev, e.second);
  }
  // strata in order; inside a stratum, nodes in id order (placeholders after the real nodes)
  std::map<int, std::vector<int>> strata;
  for (int n : g.nodes()) strata[depth.at(n)].push_back(n);

  // Once a stratum is closed every one of its nodes hangs below exactly one join, so the graph above the stratum
  // being worked on never changes again.  That makes ancestor sets of the previous stratum's nodes fixed bit rows,
  // and with bits numbered stratum by stratum (a stratum's joins before its nodes) the deepest common ancestor of a
  // class is the highest bit that all of its rows share.  Only the rows of the previous stratum are kept.
  std::map<int, size_t> bit, join_base;
  size_t total = 0;
  for (auto &layer : strata) {
    if (layer.first > 0) { join_base[layer.first] = total; total += layer.second.size(); }
    for (int n : layer.second) bit[n] = total++;
  }
  const size_t words = (total + 63) / 64;
  using Row = std::vector<uint64_t>;
  std::vector<int> node_at(total, -1);
  for (auto &kv : bit) node_at[kv.second] = kv.first;
  auto set_bit = [](Row &r, size_t i) { r[i >> 6] |= uint64_t(1) << (i & 63); };
  auto has_bit = [](const Row &r, size_t i) { return (r[i >> 6] >> (i & 63)) & 1; };

  DiGraph sp;
  std::map<int, Row> above_prev;  // ancestors-or-self of the previous stratum's nodes
  for (auto &layer : strata) {
    const int d = layer.first;
    if (d == 0) {
      for (int n : layer.second) { sp.add_node(n); Row r(words, 0); set_bit(r, bit.at(n)); above_prev[n] = r; }
      continue;
    }
    std::set<int> window;  // the last two strata and the joins between them
    for (auto &kv : above_prev) window.insert(kv.first);
    std::vector<int> arrived;
    size_t joins_made = 0;
    for (int node : layer.second) {
      sp.add_node(node);
      for (int p : g.predecessors(node)) sp.add_edge(p, node);
      window.insert(node);
      arrived.push_back(node);
      // the class of the new node: what it is tied to inside the window
      std::set<int> seen = {node};
      std::vector<int> stack = {node};
      while (!stack.empty()) {
        int x = stack.back();
        stack.pop_back();
        for (const std::set<int> *side : {&sp.successors(x), &sp.predecessors(x)})
          for (int y : *side) if (window.count(y) && seen.insert(y).second) stack.push_back(y);
      }
      std::vector<int> cls;
      Row common;
      for (int n : seen) {
        if (role.at(n) == Join) continue;
        cls.push_back(n);
        auto it = above_prev.find(n);
        if (it == above_prev.end()) continue;   // a node of this stratum adds nothing: its ancestors contain a member's
        if (common.empty()) common = it->second;
        else for (size_t w = 0; w < words; ++w) common[w] &= it->second[w];
      }
      int handle = -1;
      for (size_t w = words; w-- > 0 && handle < 0;)
        if (common[w]) handle = node_at[w * 64 + 63 - __builtin_clzll(common[w])];
      // The handle's branches sit in one block of bits, so only that word range of a row is ever looked at.
      // below: every branch bit that some member of the class has above it; those branches are the ones to close.
      const std::set<int> &branches = sp.successors(handle);
      size_t lo = words, hi = 0;
      for (int b : branches) { lo = std::min(lo, bit.at(b) >> 6); hi = std::max(hi, (bit.at(b) >> 6) + 1); }
      Row below(words, 0);
      auto add_row = [&](const Row &r) { for (size_t w = lo; w < hi; ++w) below[w] |= r[w]; };
      for (int m : cls) {
        auto it = above_prev.find(m);
        if (it != above_prev.end()) { add_row(it->second); continue; }
        set_bit(below, bit.at(m));
        for (int p : sp.predecessors(m)) {
          set_bit(below, bit.at(p));
          if (role.at(p) == Join && !above_prev.count(p)) { for (int q : sp.predecessors(p)) add_row(above_prev.at(q)); }
          else add_row(above_prev.at(p));
        }
      }
      Row closing(words, 0);
      std::set<int> touching;
      for (int b : branches) if (has_bit(below, bit.at(b))) { set_bit(closing, bit.at(b)); touching.insert(b); }
      auto meets = [&](const Row &r) { for (size_t w = lo; w < hi; ++w) if (r[w] & closing[w]) return true; return false; };
      std::set<int> up, down;
      for (auto &kv : above_prev) if (meets(kv.second)) up.insert(kv.first);
      for (int w : arrived) {
        bool in = touching.count(w) > 0;
        for (int p : sp.predecessors(w)) {
          if (in) break;
          if (touching.count(p) || up.count(p)) in = true;
          else if (role.at(p) == Join) for (int q : sp.predecessors(p)) if (up.count(q)) { in = true; break; }
        }
        if (in) down.insert(w);
      }
      if (role.at(handle) != Join && depth.at(handle) + 1 == d) up.insert(handle);
      for (int u : up) for (int x : std::set<int>(sp.successors(u))) sp.remove_edge(u, x);
      for (int w : down) for (int p : std::set<int>(sp.predecessors(w))) sp.remove_edge(p, w);
      int join = next_id++;
      role[join] = Join;
      bit[join] = join_base.at(d) + joins_made++;
      node_at[bit[join]] = join;
      sp.add_node(join);
      window.insert(join);
      for (int u : up) sp.add_edge(u, join);
      for (int w : down) sp.add_edge(join, w);
    }
    std::map<int, Row> above_cur, above_join;
    for (int n : layer.second) {
      Row r(words, 0);
      for (int p : sp.predecessors(n)) {
        if (role.at(p) != Join) { for (size_t w = 0; w < words; ++w) r[w] |= above_prev.at(p)[w]; continue; }
        auto it = above_join.find(p);
        if (it == above_join.end()) {
          Row jr(words, 0);
          set_bit(jr, bit.at(p));
          for (int u : sp.predecessors(p)) { const Row &ur = above_prev.at(u); for (size_t w = 0; w < words; ++w) jr[w] |= ur[w]; }
          it = above_join.emplace(p, std::move(jr)).first;
        }
        for (size_t w = 0; w < words; ++w) r[w] |= it->second[w];
      }
      set_bit(r, bit.at(n));
      above_cur[n] = std::move(r);
    }
    above_prev = std::move(above_cur);
  }
  DiGraph real = transitive_reduction(bridge_out_nodes(sp, [&](int n) { return role.at(n) != Real; }));
  std::optional<SPTree> tree = get_series_parallel_decomposition(real);
  if (!tree) throw std::runtime_error("escribano_sp_ization: result is not series-parallel");
  return normalize_sp(sp_without_leaves(*tree, added_terminals));
}

static DiGraph induced_subgraph(const DiGraph &g, const std::set<int> &keep) {
  DiGraph r;
  for (int n : keep) {
    r.add_node(n);
    for (int s : g.successors(n)) if (keep.count(s)) r.add_edge(n, s);
  }
  return r;
}

static double longest_weighted_path(const DiGraph &g, const std::function<double(int)> &cost) {
  double best = 0;
  for (auto &kv : get_weighted_longest_path_lengths(g, cost)) best = std::max(best, kv.second);
  return best;
}

SPTree flexible_sp_ization(const DiGraph &g0, const std::function<double(int)> &node_cost) {
  // Cost-aware generalisation of escribano_sp_ization.  The graph is again grown into a series-parallel one with
  // join nodes, but (a) nodes arrive in order of their earliest finish time instead of stratum by stratum (all ready
  // nodes that share the cheapest one's predecessor set arrive together), and (b) the region being closed is not cut
  // between its last two strata: every cut of the region into an upper and a lower part that keeps the new nodes
  // below and their ancestors above is a candidate, the candidates being the prefixes of the undecided nodes ordered
  // by finish time, and the cut with the smallest (longest path above + longest path below) wins; ties go to the
  // cheaper, then the smaller, lower part.  lib/utils/src/utils/graph/series_parallel/sp_ization/flexible_algo.cc:254-310
  // is the upstream statement of the algorithm (two-terminal graphs only; several sources or sinks get a common
  // zero-cost one here, which is taken out of the result).
  if (g0.num_nodes() == 0) return SPTree::parallel({});
  if (g0.num_nodes() == 1) return SPTree::leaf(g0.nodes()[0]);
  DiGraph g = transitive_reduction(g0);
  std::set<int> joins, added_terminals;
  int next_id = 0;
  for (int n : g.nodes()) next_id = std::max(next_id, n + 1);
  if (g.sources().size() > 1) {
    int r = next_id++;
    for (int s : g.sources()) g.add_edge(r, s);
    added_terminals.insert(r);
  }
  if (g.sinks().size() > 1) {
    int t = next_id++;
    for (int s : g.sinks()) g.add_edge(s, t);
    added_terminals.insert(t);
  }
  auto cost = [&](int n) { return joins.count(n) || added_terminals.count(n) ? 0.0 : node_cost(n); };
  auto is_join = [&](int n) { return joins.count(n) > 0; };

  DiGraph sp;
  sp.add_node(g.sources()[0]);
  while (sp.num_nodes() - joins.size() < g.num_nodes()) {
    // ---- the next batch of nodes
    std::map<int, double> finish = get_weighted_longest_path_lengths(sp, cost);
    std::vector<int> ready;
    for (int n : g.nodes()) {
      if (sp.has_node(n)) continue;
      bool ok = true;
      for (int p : g.predecessors(n)) ok = ok && sp.has_node(p);
      if (ok) ready.push_back(n);
    }
    int first = -1;
    double first_finish = 0;
    for (int n : ready) {
      double start = 0;
      for (int p : g.predecessors(n)) start = std::max(start, finish.at(p));
      double f = start + cost(n);
      if (first < 0 || f < first_finish) { first = n; first_finish = f; }
    }
    std::set<int> batch;
    for (int n : ready) if (g.predecessors(n) == g.predecessors(first)) batch.insert(n);
    for (int n : batch) for (int p : g.predecessors(n)) sp.add_edge(p, n);
    sp = transitive_reduction(sp);

    // ---- the region to close: what the batch's predecessors reach, and what else feeds into that
    std::set<int> region;
    for (int n : batch) for (int p : sp.predecessors(n)) region.insert(p);
    std::set<int> reached;
    for (int p : region) for (int x : get_descendants(sp, p)) reached.insert(x);
    for (int x : reached) { region.insert(x); for (int p : sp.predecessors(x)) region.insert(p); }
    int handle = *get_lowest_common_ancestor(sp, region);
    std::set<int> forest;
    for (int branch : sp.successors(handle)) {
      std::set<int> below = get_descendants(sp, branch);
      below.insert(branch);
      bool touches = false;
      for (int n : below) if (region.count(n)) { touches = true; break; }
      if (touches) for (int n : below) if (!is_join(n)) forest.insert(n);
    }
    if (!is_join(handle)) forest.insert(handle);

    // ---- choose the cut
    DiGraph pure = bridge_out_nodes(sp, is_join);
    std::set<int> fixed_up, undecided;
    for (int n : batch) for (int a : get_ancestors(pure, n)) if (forest.count(a)) fixed_up.insert(a);
    for (int n : forest) if (!fixed_up.count(n) && !batch.count(n)) undecided.insert(n);
    std::map<int, double> forest_finish = get_weighted_longest_path_lengths(induced_subgraph(pure, forest), cost);
    std::vector<std::optional<double>> limits = {std::nullopt};   // nothing undecided goes up / all up to this finish time
    for (int n : undecided) limits.push_back(forest_finish.at(n));
    bool have = false;
    std::set<int> best_up, best_down;
    std::tuple<double, double, size_t> best_key;
    for (auto &limit : limits) {
      std::set<int> up = fixed_up, down = batch;
      for (int n : undecided) (limit && forest_finish.at(n) <= *limit ? up : down).insert(n);
      bool valid = true;
      for (int d : down) for (int s : pure.successors(d)) if (up.count(s)) valid = false;
      if (!valid) continue;
      double cu = longest_weighted_path(induced_subgraph(pure, up), cost);
      double cd = longest_weighted_path(induced_subgraph(pure, down), cost);
      std::tuple<double, double, size_t> key{cu + cd, cd, down.size()};
      if (!have || key < best_key) { have = true; best_key = key; best_up = up; best_down = down; }
    }
    if (!have) throw std::runtime_error("flexible_sp_ization: no valid cut");

    // ---- replace what crosses the cut by one join
    for (int u : best_up) for (int s : std::set<int>(sp.successors(u))) if (best_down.count(s)) sp.remove_edge(u, s);
    for (int j : joins) {
      const std::set<int> ps = sp.predecessors(j), ss = sp.successors(j);
      bool inside = true;
      for (int p : ps) inside = inside && best_up.count(p);
      for (int x : ss) inside = inside && best_down.count(x);
      if (!inside) continue;
      for (int p : ps) sp.remove_edge(p, j);
      for (int x : ss) sp.remove_edge(j, x);
    }
    int join = next_id++;
    joins.insert(join);
    sp.add_node(join);
    for (int u : best_up) {
      bool last = true;
      for (int s : sp.successors(u)) if (best_up.count(s)) last = false;
      if (last) sp.add_edge(u, join);
    }
    for (int d : best_down) {
      bool head = true;
      for (int p : sp.predecessors(d)) if (best_down.count(p)) head = false;
      if (head) sp.add_edge(join, d);
    }
  }
  DiGraph real = transitive_reduction(bridge_out_nodes(transitive_reduction(sp), is_join));
  std::optional<SPTree> tree = get_series_parallel_decomposition(real);
  if (!tree) throw std::runtime_error("flexible_sp_ization: result is not series-parallel");
  return normalize_sp(sp_without_leaves(*tree, added_terminals));
}

bool sp_preserves_dependencies(const SPTree &t, const DiGraph &g) {
  // With duplicated work a node may occur several times; every occurrence of b must be preceded by an
  // occurrence of a.  Checked through the closure of the tree's own dependency graph, which for
  // duplicate-free trees is exact and for duplicated trees is checked per occurrence by relabelling.
  std::vector<int> occ = sp_nodes(t);
  // relabel occurrences uniquely
  int counter = 0;
  std::map<int, int> orig;  // unique id -> node
  std::function<SPTree(const SPTree &)> relabel = [&](const SPTree &s) {
    if (s.kind == SPTree::Leaf) { orig[counter] = s.node; return SPTree::leaf(counter++); }
    SPTree r;
    r.kind = s.kind;
    for (auto &c : s.children) r.children.push_back(relabel(c));
    return r;
  };
  SPTree u = relabel(t);
  DiGraph closure = transitive_closure(digraph_from_sp(u));
  std::map<int, std::vector<int>> ids_of;
  for (auto &kv : orig) ids_of[kv.second].push_back(kv.first);
  for (int n : g.nodes()) if (!ids_of.count(n)) return false;
  for (auto &e : g.edges()) {
    for (int b_id : ids_of[e.second]) {
      bool ok = false;
      for (int a_id : ids_of[e.first]) if (closure.has_edge(a_id, b_id)) { ok = true; break; }
      if (!ok) return false;
    }
  }
  return true;
}

}  // namespace ff
