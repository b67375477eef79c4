// Python surface of utils.h (submodule `utils` of the core module): thin functions over builtins, so that the
// support types can be exercised from the test suite.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "flag_protocol.h"
#include "utils.h"

namespace py = pybind11;

namespace ff {
using namespace ff::utils;

namespace {
using Tree = FullBinaryTree<std::string, int>;
// nested tuples: an int is a leaf, (label, left, right) an inner node
Tree tree_from_py(const py::handle &h) {
  if (py::isinstance<py::int_>(h)) return Tree::make_leaf(h.cast<int>());
  py::tuple t = h.cast<py::tuple>();
  if (t.size() != 3) throw std::invalid_argument("an inner node is (label, left, right)");
  return Tree::make_parent(t[0].cast<std::string>(), tree_from_py(t[1]), tree_from_py(t[2]));
}
std::string path_str(const BinaryTreePath &p) {
  std::string s;
  for (Turn t : p) s += t == Turn::LEFT ? 'L' : 'R';
  return s;
}
BinaryTreePath path_from_str(const std::string &s) {
  BinaryTreePath p;
  for (char c : s) p.push_back(c == 'L' ? Turn::LEFT : Turn::RIGHT);
  return p;
}
}  // namespace

void bind_utils(py::module &root) {
  py::module m = root.def_submodule("utils", "support types of the compiler core");
  // ---- restricted ints and units
  m.def("nonnegative", [](long long v) { return nonnegative_int(v).value(); });
  m.def("positive", [](long long v) { return positive_int(v).value(); });
  m.def("ge_two", [](long long v) { return int_ge_two(v).value(); });
  m.def("positive_mul", [](long long a, long long b) { return (positive_int(a) * positive_int(b)).value(); });
  m.def("positive_add", [](long long a, long long b) { return (positive_int(a) + positive_int(b)).value(); });
  m.def("ceildiv", [](long long a, long long b) { return ceildiv(positive_int(a), positive_int(b)).value(); });
  m.def("transfer_ms", [](double bytes, double bytes_per_s) { return (num_bytes_t(bytes) / bytes_per_second_t(bytes_per_s)).v; });
  m.def("max_ms", [](double a, double b) { return max(milliseconds_t(a), milliseconds_t(b)).v; });
  // ---- containers
  m.def("cartesian_product", [](const std::vector<std::vector<int>> &l) { return cartesian_product(l); });
  m.def("get_all_assignments", [](const std::map<int, std::vector<int>> &o) { return get_all_assignments(o); });
  m.def("merge_maps_sum", [](const std::map<std::string, int> &a, const std::map<std::string, int> &b) {
    return merge_maps_with(a, b, [](int x, int y) { return x + y; });
  });
  m.def("group_by_mod", [](const std::vector<int> &v, int k) { return group_by(v, [k](int x) { return x % k; }); });
  m.def("get_all_permutations", [](const std::vector<int> &v) { return get_all_permutations(v); });
  m.def("transform_square", [](const std::vector<int> &v) { return transform(v, [](int x) { return x * x; }); });
  m.def("filter_even", [](const std::set<int> &s) { return filter(s, [](int x) { return x % 2 == 0; }); });
  m.def("zip", [](const std::vector<int> &a, const std::vector<std::string> &b) { return zip(a, b); });
  m.def("set_ops", [](const std::set<int> &a, const std::set<int> &b) {
    return py::make_tuple(set_union(a, b), intersection(a, b), is_subseteq_of(a, b));
  });
  m.def("product", [](const std::vector<long long> &v) { return product(v); });
  m.def("maximum", [](const std::vector<int> &v) { return maximum(v); });
  m.def("flatmap_concat", [](const std::vector<std::vector<int>> &v) { return flatmap_concat(v); });
  // ---- restricted maps
  m.def("bidict", [](const std::vector<std::pair<int, std::string>> &pairs) {
    bidict<int, std::string> b;
    for (auto &p : pairs) b.equate(p.first, p.second);
    return py::make_tuple(b.as_map(), b.reversed().as_map());
  });
  m.def("relational_join", [](const std::vector<std::pair<int, std::string>> &ab, const std::vector<std::pair<std::string, int>> &bc) {
    bidict<int, std::string> x;
    bidict<std::string, int> y;
    for (auto &p : ab) x.equate(p.first, p.second);
    for (auto &p : bc) y.equate(p.first, p.second);
    return exhaustive_relational_join(x, y).as_map();
  });
  m.def("one_to_many", [](const std::vector<std::pair<int, int>> &pairs) {
    OneToMany<int, int> o;
    for (auto &p : pairs) o.insert(p.first, p.second);
    std::map<int, std::set<int>> out;
    for (int l : o.left_values()) out[l] = o.at_l(l);
    return out;
  });
  m.def("many_to_one", [](const std::vector<std::pair<int, int>> &pairs, int query_right) {
    ManyToOne<int, int> o;
    for (auto &p : pairs) o.insert(p.first, p.second);
    return o.at_r(query_right);
  });
  // ---- union-find, queue, stack vector
  m.def("union_find_groups", [](const std::vector<std::pair<int, int>> &pairs) {
    disjoint_set<int> ds;
    for (auto &p : pairs) ds.unite(p.first, p.second);
    std::vector<std::set<int>> out;
    for (auto &g : ds.groups()) out.push_back(g.second);
    return out;
  });
  m.def("dedup_queue_order", [](const std::vector<int> &items) {
    DeduplicatedPriorityQueue<int> q;
    int accepted = 0;
    for (int x : items) accepted += q.push(x) ? 1 : 0;
    std::vector<int> order;
    while (!q.empty()) {
      order.push_back(q.top());
      q.pop();
    }
    return py::make_tuple(accepted, order);
  });
  m.def("stack_vector_fill", [](int n) {
    stack_vector<int, 8> v;
    for (int i = 0; i < n; ++i) v.push_back(i);
    int s = 0;
    for (int x : v) s += x;
    return py::make_tuple(v.size(), s);
  });
  // ---- full binary tree
  m.def("tree_info", [](py::object nested) {
    Tree t = tree_from_py(nested);
    std::vector<std::string> paths;
    for (auto &p : t.all_leaf_paths()) paths.push_back(path_str(p));
    return py::make_tuple(t.num_nodes(), t.leaves(), paths);
  });
  m.def("tree_leaves_at", [](py::object nested, const std::string &path) -> std::optional<std::vector<int>> {
    Tree t = tree_from_py(nested);
    const Tree *s = t.subtree_at(path_from_str(path));
    if (!s) return std::nullopt;
    return s->leaves();
  });
  // ---- orthotope
  m.def("orthotope_volume", [](const std::vector<long long> &d) { return Orthotope{d}.volume(); });
  m.def("orthotope_flatten", [](const std::vector<long long> &d, const std::vector<long long> &c) { return Orthotope{d}.flatten(c); });
  m.def("orthotope_unflatten", [](const std::vector<long long> &d, long long f) { return Orthotope{d}.unflatten(f); });
  m.def("orthotope_minimal", [](const std::vector<long long> &d) { return Orthotope{d}.minimal().dims; });
  m.def("project_domain", [](const std::vector<long long> &d, const std::vector<std::vector<int>> &g) {
    return DimProjection{g}.project_domain(Orthotope{d}).dims;
  });
  m.def("project_coord", [](const std::vector<long long> &d, const std::vector<std::vector<int>> &g, const std::vector<long long> &c) {
    return DimProjection{g}.project_coord(Orthotope{d}, c);
  });
  m.def("lift_coord", [](const std::vector<long long> &d, const std::vector<std::vector<int>> &g, const std::vector<long long> &c) {
    return DimProjection{g}.lift_coord(Orthotope{d}, c);
  });
  m.def("projection_is_bijection", [](const std::vector<long long> &d, const std::vector<std::vector<int>> &g) {
    return DimProjection{g}.is_bijection_on(Orthotope{d});
  });
  // ---- graphs
  m.def("connected_components", [](const std::vector<int> &nodes, const std::vector<std::pair<int, int>> &edges) {
    UndirectedGraph g;
    for (int n : nodes) g.add_node(n);
    for (auto &e : edges) g.add_edge(e.first, e.second);
    return py::make_tuple(g.connected_components(), g.num_edges());
  });
  m.def("multidigraph_counts", [](const std::vector<std::pair<int, int>> &edges, int a, int b) {
    MultiDiGraph g;
    std::vector<int> ids;
    for (auto &e : edges) ids.push_back(g.add_edge(e.first, e.second));
    size_t between = g.edges_between(a, b).size();
    if (!ids.empty()) g.remove_edge(ids.front());
    return py::make_tuple(g.nodes().size(), between, g.num_edges(), g.outgoing(a).size(), g.incoming(b).size());
  });
  // ---- flag protocol of the peer-memory kernels, with threads as ranks
  m.def("flag_protocol_rounds", [](int ranks, int epochs, int silent_rank, int silent_after, int limit_ms) {
    std::vector<flagproto::RankResult> res;
    {
      py::gil_scoped_release release;
      res = flagproto::run_rounds(ranks, epochs, silent_rank, silent_after, limit_ms);
    }
    py::list out;
    for (auto &r : res) {
      py::dict d;
      d["epochs_done"] = r.epochs_done;
      d["ok"] = r.report.ok;
      d["waiter"] = r.report.waiter;
      d["peer"] = r.report.peer;
      d["expected"] = r.report.expected;
      d["seen"] = r.report.seen;
      d["checksum"] = r.checksum;
      d["seconds"] = r.seconds;
      out.append(d);
    }
    return out;
  }, py::arg("ranks"), py::arg("epochs"), py::arg("silent_rank") = -1, py::arg("silent_after") = 0, py::arg("limit_ms") = 2000);
  // ---- formatters
  m.def("dot_text", [](const std::vector<std::string> &nodes, const std::vector<std::pair<std::string, std::string>> &edges) {
    DotFile d("g");
    d.begin_cluster("all");
    for (auto &n : nodes) d.add_node(n, {{"shape", "record"}});
    d.end_cluster();
    for (auto &e : edges) d.add_edge(e.first, e.second);
    return d.str();
  });
  m.def("record_text", [](const std::vector<std::string> &outer, const std::vector<std::string> &inner) {
    RecordFormatter in, out;
    for (auto &f : inner) in << f;
    for (auto &f : outer) out << f;
    out << in;
    return out.str();
  });
}

}  // namespace ff
