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

SPTree escribano_sp_ization(const DiGraph &g) {
  // Layer-by-layer construction that synchronises only the components that a layer actually joins
  // (after Escribano et al.).  State: a forest of SP components, each with the set of DAG nodes it
  // contains.  For every stratum, the new nodes that (transitively through shared predecessors'
  // components) touch the same components are grouped; the touched components are closed under a
  // parallel node and followed by the parallel group of new nodes.
  auto depth = get_longest_path_lengths_from_root(g);
  std::map<int, std::vector<int>> strata;
  for (auto &kv : depth) strata[kv.second].push_back(kv.first);
  struct Comp { SPTree tree; std::set<int> members; };
  std::vector<Comp> comps;
  for (auto &kv : strata) {
    const std::vector<int> &layer = kv.second;
    // union-find over (components + new nodes)
    size_t nc = comps.size();
    std::vector<int> parent(nc + layer.size());
    for (size_t i = 0; i < parent.size(); ++i) parent[i] = (int)i;
    std::function<int(int)> find = [&](int x) { return parent[x] == x ? x : parent[x] = find(parent[x]); };
    for (size_t li = 0; li < layer.size(); ++li)
      for (int p : g.predecessors(layer[li]))
        for (size_t ci = 0; ci < nc; ++ci)
          if (comps[ci].members.count(p)) parent[find((int)(nc + li))] = find((int)ci);
    std::map<int, std::pair<std::vector<size_t>, std::vector<size_t>>> groups;  // root -> (comps, layer idx)
    for (size_t ci = 0; ci < nc; ++ci) groups[find((int)ci)].first.push_back(ci);
    for (size_t li = 0; li < layer.size(); ++li) groups[find((int)(nc + li))].second.push_back(li);
    std::vector<Comp> next;
    for (auto &gkv : groups) {
      auto &cidx = gkv.second.first;
      auto &lidx = gkv.second.second;
      if (lidx.empty()) {  // untouched components carry over
        for (size_t ci : cidx) next.push_back(comps[ci]);
        continue;
      }
      Comp c;
      std::vector<SPTree> olds, news;
      for (size_t ci : cidx) { olds.push_back(comps[ci].tree); c.members.insert(comps[ci].members.begin(), comps[ci].members.end()); }
      for (size_t li : lidx) { news.push_back(SPTree::leaf(layer[li])); c.members.insert(layer[li]); }
      if (olds.empty()) c.tree = normalize_sp(SPTree::parallel(news));
      else c.tree = normalize_sp(SPTree::series({SPTree::parallel(olds), SPTree::parallel(news)}));
      next.push_back(c);
    }
    comps = next;
  }
  std::vector<SPTree> all;
  for (auto &c : comps) all.push_back(c.tree);
  return normalize_sp(SPTree::parallel(all));
}

SPTree flexible_sp_ization(const DiGraph &g, const std::function<double(int)> &cost) {
  // Cost-aware choice: evaluate the candidate SP-izations under the given node costs and keep the one
  // with the smallest critical path, breaking ties on total work (duplication).
  std::vector<SPTree> cands = {escribano_sp_ization(g), naive_stratum_sync_sp_ization(g),
                               work_duplicating_sp_ization(g, true)};
  if (auto exact = get_series_parallel_decomposition(g)) return *exact;
  size_t best = 0;
  double best_cp = 0, best_w = 0;
  for (size_t i = 0; i < cands.size(); ++i) {
    double cp = sp_critical_path_cost(cands[i], cost), w = sp_work_cost(cands[i], cost);
    if (i == 0 || cp < best_cp - 1e-12 || (std::abs(cp - best_cp) <= 1e-12 && w < best_w)) {
      best = i; best_cp = cp; best_w = w;
    }
  }
  return cands[best];
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
