// utils.h -- the general-purpose support types of the compiler core, header-only.
//
// Counterparts of the reference's lib/utils: restricted integers and unit types
// (include/utils/{nonnegative_int,positive_int,int_ge_two,units}), the functional container helpers
// (include/utils/containers/*.h), the restricted maps (bidict, one_to_many, many_to_one), disjoint_set,
// DeduplicatedPriorityQueue, stack_vector, the full binary tree with paths (include/utils/full_binary_tree),
// the orthotope index-space algebra (include/utils/orthotope), undirected and multi-digraphs
// (include/utils/graph) and the dot / record formatters.  Everything is plain C++17 over the STL.
#pragma once
#include <algorithm>
#include <array>
#include <functional>
#include <map>
#include <optional>
#include <queue>
#include <set>
#include <sstream>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace ff {
namespace utils {

// ------------------------------------------------------------------ restricted integers
// An int that is known to be >= Min; arithmetic that could leave the range is checked.
template <long long Min>
class bounded_int {
public:
  bounded_int() : v_(Min) {}
  explicit bounded_int(long long v) : v_(v) {
    if (v < Min) throw std::invalid_argument("value " + std::to_string(v) + " is below the minimum " + std::to_string(Min));
  }
  long long value() const { return v_; }
  bounded_int operator+(bounded_int o) const { return bounded_int(checked_add(v_, o.v_)); }
  bounded_int operator*(bounded_int o) const { return bounded_int(checked_mul(v_, o.v_)); }
  // subtraction and division may leave the range: they return a plain integer
  long long operator-(bounded_int o) const { return v_ - o.v_; }
  long long operator/(bounded_int o) const {
    if (o.v_ == 0) throw std::domain_error("division by zero");
    return v_ / o.v_;
  }
  long long operator%(bounded_int o) const {
    if (o.v_ == 0) throw std::domain_error("modulo by zero");
    return v_ % o.v_;
  }
  bool operator==(bounded_int o) const { return v_ == o.v_; }
  bool operator!=(bounded_int o) const { return v_ != o.v_; }
  bool operator<(bounded_int o) const { return v_ < o.v_; }
  bool operator<=(bounded_int o) const { return v_ <= o.v_; }
  bool operator>(bounded_int o) const { return v_ > o.v_; }
  bool operator>=(bounded_int o) const { return v_ >= o.v_; }

private:
  static long long checked_add(long long a, long long b) {
    long long r;
    if (__builtin_add_overflow(a, b, &r)) throw std::overflow_error("integer overflow in addition");
    return r;
  }
  static long long checked_mul(long long a, long long b) {
    long long r;
    if (__builtin_mul_overflow(a, b, &r)) throw std::overflow_error("integer overflow in multiplication");
    return r;
  }
  long long v_;
};
using nonnegative_int = bounded_int<0>;
using positive_int = bounded_int<1>;
using int_ge_two = bounded_int<2>;

// ceil(a / b) on positive ints (utils/positive_int/ceildiv.h)
inline positive_int ceildiv(positive_int a, positive_int b) { return positive_int((a.value() + b.value() - 1) / b.value()); }

// ------------------------------------------------------------------ units
// Tagged floating-point quantities: only meaningful combinations compile.
template <typename Tag>
struct quantity {
  double v = 0;
  quantity() = default;
  explicit quantity(double x) : v(x) {
    if (x < 0) throw std::invalid_argument("a physical quantity cannot be negative");
  }
  quantity operator+(quantity o) const { return quantity(v + o.v); }
  quantity operator*(double s) const { return quantity(v * s); }
  bool operator<(quantity o) const { return v < o.v; }
  bool operator==(quantity o) const { return v == o.v; }
};
struct ms_tag {};
struct bytes_tag {};
struct bps_tag {};
using milliseconds_t = quantity<ms_tag>;
using num_bytes_t = quantity<bytes_tag>;
using bytes_per_second_t = quantity<bps_tag>;
inline milliseconds_t operator/(num_bytes_t b, bytes_per_second_t r) {
  if (r.v <= 0) throw std::domain_error("bandwidth must be positive");
  return milliseconds_t(b.v / r.v * 1e3);
}
inline milliseconds_t max(milliseconds_t a, milliseconds_t b) { return a < b ? b : a; }

// ------------------------------------------------------------------ container helpers
template <typename C, typename F>
auto transform(const C &c, F f) -> std::vector<decltype(f(*c.begin()))> {
  std::vector<decltype(f(*c.begin()))> out;
  for (auto &x : c) out.push_back(f(x));
  return out;
}
template <typename C, typename F>
C filter(const C &c, F pred) {
  C out;
  for (auto &x : c)
    if (pred(x)) out.insert(out.end(), x);
  return out;
}
template <typename A, typename B>
std::vector<std::pair<A, B>> zip(const std::vector<A> &a, const std::vector<B> &b) {
  std::vector<std::pair<A, B>> out;
  for (size_t i = 0; i < std::min(a.size(), b.size()); ++i) out.push_back({a[i], b[i]});
  return out;
}
template <typename T>
std::vector<std::vector<T>> cartesian_product(const std::vector<std::vector<T>> &lists) {
  std::vector<std::vector<T>> out = {{}};
  for (auto &l : lists) {
    std::vector<std::vector<T>> next;
    for (auto &prefix : out)
      for (auto &x : l) {
        auto p = prefix;
        p.push_back(x);
        next.push_back(p);
      }
    out = std::move(next);
  }
  return out;
}
// every way of assigning one of its options to each key (utils/containers/get_all_assignments.h)
template <typename K, typename V>
std::vector<std::map<K, V>> get_all_assignments(const std::map<K, std::vector<V>> &options) {
  std::vector<std::map<K, V>> out = {{}};
  for (auto &kv : options) {
    std::vector<std::map<K, V>> next;
    for (auto &partial : out)
      for (auto &v : kv.second) {
        auto m = partial;
        m[kv.first] = v;
        next.push_back(m);
      }
    out = std::move(next);
  }
  return out;
}
template <typename K, typename V, typename F>
std::map<K, V> merge_maps_with(const std::map<K, V> &a, const std::map<K, V> &b, F combine) {
  std::map<K, V> out = a;
  for (auto &kv : b) {
    auto it = out.find(kv.first);
    if (it == out.end()) out[kv.first] = kv.second;
    else it->second = combine(it->second, kv.second);
  }
  return out;
}
template <typename C, typename F>
auto group_by(const C &c, F key) -> std::map<decltype(key(*c.begin())), std::vector<typename C::value_type>> {
  std::map<decltype(key(*c.begin())), std::vector<typename C::value_type>> out;
  for (auto &x : c) out[key(x)].push_back(x);
  return out;
}
template <typename T>
std::set<T> set_union(const std::set<T> &a, const std::set<T> &b) {
  std::set<T> r = a;
  r.insert(b.begin(), b.end());
  return r;
}
template <typename T>
std::set<T> intersection(const std::set<T> &a, const std::set<T> &b) {
  std::set<T> r;
  for (auto &x : a)
    if (b.count(x)) r.insert(x);
  return r;
}
template <typename T>
bool is_subseteq_of(const std::set<T> &a, const std::set<T> &b) {
  return std::all_of(a.begin(), a.end(), [&](const T &x) { return b.count(x) > 0; });
}
template <typename K, typename V>
std::vector<K> keys(const std::map<K, V> &m) {
  std::vector<K> r;
  for (auto &kv : m) r.push_back(kv.first);
  return r;
}
template <typename T>
std::vector<T> flatmap_concat(const std::vector<std::vector<T>> &v) {
  std::vector<T> r;
  for (auto &x : v) r.insert(r.end(), x.begin(), x.end());
  return r;
}
template <typename T>
std::vector<std::vector<T>> get_all_permutations(std::vector<T> v) {
  std::sort(v.begin(), v.end());
  std::vector<std::vector<T>> out;
  do out.push_back(v);
  while (std::next_permutation(v.begin(), v.end()));
  return out;
}
template <typename T>
std::optional<T> maximum(const std::vector<T> &v) {
  if (v.empty()) return std::nullopt;
  return *std::max_element(v.begin(), v.end());
}
template <typename T>
T product(const std::vector<T> &v) {
  T r = 1;
  for (auto &x : v) r = r * x;
  return r;
}

// ------------------------------------------------------------------ restricted maps
// One-to-one map readable in both directions (utils/bidict).
template <typename L, typename R>
class bidict {
public:
  void equate(const L &l, const R &r) {
    erase_l(l);
    erase_r(r);
    fwd_[l] = r;
    bwd_[r] = l;
  }
  bool contains_l(const L &l) const { return fwd_.count(l) > 0; }
  bool contains_r(const R &r) const { return bwd_.count(r) > 0; }
  const R &at_l(const L &l) const { return fwd_.at(l); }
  const L &at_r(const R &r) const { return bwd_.at(r); }
  void erase_l(const L &l) {
    auto it = fwd_.find(l);
    if (it == fwd_.end()) return;
    bwd_.erase(it->second);
    fwd_.erase(it);
  }
  void erase_r(const R &r) {
    auto it = bwd_.find(r);
    if (it == bwd_.end()) return;
    fwd_.erase(it->second);
    bwd_.erase(it);
  }
  size_t size() const { return fwd_.size(); }
  bidict<R, L> reversed() const {
    bidict<R, L> out;
    for (auto &kv : fwd_) out.equate(kv.second, kv.first);
    return out;
  }
  const std::map<L, R> &as_map() const { return fwd_; }

private:
  std::map<L, R> fwd_;
  std::map<R, L> bwd_;
};
template <typename A, typename B, typename C>
bidict<A, C> exhaustive_relational_join(const bidict<A, B> &ab, const bidict<B, C> &bc) {
  bidict<A, C> out;
  if (ab.size() != bc.size()) throw std::invalid_argument("relational join: the two maps do not cover the same middle set");
  for (auto &kv : ab.as_map()) out.equate(kv.first, bc.at_l(kv.second));
  return out;
}

// Every right value belongs to exactly one left value (utils/one_to_many).
template <typename L, typename R>
class OneToMany {
public:
  void insert(const L &l, const R &r) {
    auto it = owner_.find(r);
    if (it != owner_.end() && !(it->second == l)) throw std::invalid_argument("OneToMany: the right value already has another owner");
    owner_[r] = l;
    members_[l].insert(r);
  }
  const std::set<R> &at_l(const L &l) const { return members_.at(l); }
  const L &at_r(const R &r) const { return owner_.at(r); }
  std::set<L> left_values() const {
    std::set<L> s;
    for (auto &kv : members_) s.insert(kv.first);
    return s;
  }
  std::set<R> right_values() const {
    std::set<R> s;
    for (auto &kv : owner_) s.insert(kv.first);
    return s;
  }
  size_t size() const { return owner_.size(); }

private:
  std::map<L, std::set<R>> members_;
  std::map<R, L> owner_;
};
// Every left value maps to exactly one right value (utils/many_to_one): the transpose of OneToMany.
template <typename L, typename R>
class ManyToOne {
public:
  void insert(const L &l, const R &r) { inv_.insert(r, l); }
  const R &at_l(const L &l) const { return inv_.at_r(l); }
  const std::set<L> &at_r(const R &r) const { return inv_.at_l(r); }
  size_t size() const { return inv_.size(); }

private:
  OneToMany<R, L> inv_;
};

// ------------------------------------------------------------------ disjoint sets (union-find with path halving)
template <typename T>
class disjoint_set {
public:
  const T &find(const T &x) {
    if (!parent_.count(x)) {
      parent_[x] = x;
      rank_[x] = 0;
    }
    T cur = x;
    while (!(parent_[cur] == cur)) {
      parent_[cur] = parent_[parent_[cur]];
      cur = parent_[cur];
    }
    return parent_.find(cur)->first;
  }
  void unite(const T &a, const T &b) {
    T ra = find(a), rb = find(b);
    if (ra == rb) return;
    if (rank_[ra] < rank_[rb]) std::swap(ra, rb);
    parent_[rb] = ra;
    if (rank_[ra] == rank_[rb]) ++rank_[ra];
  }
  bool same(const T &a, const T &b) { return find(a) == find(b); }
  std::map<T, std::set<T>> groups() {
    std::map<T, std::set<T>> out;
    for (auto &kv : parent_) out[find(kv.first)].insert(kv.first);
    return out;
  }

private:
  std::map<T, T> parent_;
  std::map<T, int> rank_;
};

// ------------------------------------------------------------------ priority queue that ignores repeated pushes
// (utils/deduplicated_priority_queue.h: the search never evaluates one state twice)
template <typename T, typename Compare = std::less<T>>
class DeduplicatedPriorityQueue {
public:
  bool push(const T &x) {
    if (!seen_.insert(x).second) return false;
    q_.push(x);
    return true;
  }
  const T &top() const { return q_.top(); }
  void pop() { q_.pop(); }
  bool empty() const { return q_.empty(); }
  size_t size() const { return q_.size(); }
  bool has_seen(const T &x) const { return seen_.count(x) > 0; }

private:
  std::priority_queue<T, std::vector<T>, Compare> q_;
  std::set<T> seen_;
};

// ------------------------------------------------------------------ fixed-capacity vector without heap allocation
template <typename T, size_t MAXSIZE>
class stack_vector {
public:
  void push_back(const T &x) {
    if (n_ == MAXSIZE) throw std::length_error("stack_vector is full (" + std::to_string(MAXSIZE) + ")");
    data_[n_++] = x;
  }
  void pop_back() {
    if (n_ == 0) throw std::out_of_range("pop_back on an empty stack_vector");
    --n_;
  }
  T &at(size_t i) {
    if (i >= n_) throw std::out_of_range("stack_vector index out of range");
    return data_[i];
  }
  const T &at(size_t i) const {
    if (i >= n_) throw std::out_of_range("stack_vector index out of range");
    return data_[i];
  }
  size_t size() const { return n_; }
  static constexpr size_t capacity() { return MAXSIZE; }
  const T *begin() const { return data_.data(); }
  const T *end() const { return data_.data() + n_; }
  T *begin() { return data_.data(); }
  T *end() { return data_.data() + n_; }
  T &operator[](size_t i) { return data_[i]; }
  const T &operator[](size_t i) const { return data_[i]; }
  T &back() { return at(n_ - 1); }

private:
  std::array<T, MAXSIZE> data_{};
  size_t n_ = 0;
};

// ------------------------------------------------------------------ full binary tree with paths
// A tree whose inner nodes have exactly two children; a BinaryTreePath (left/right turns from the root) names a
// subtree -- the keys of the machine-mapping recursion (utils/full_binary_tree/binary_tree_path.dtg.toml).
enum class Turn { LEFT, RIGHT };
using BinaryTreePath = std::vector<Turn>;
template <typename Parent, typename Leaf>
struct FullBinaryTree {
  std::optional<Leaf> leaf;       // set for leaves
  std::optional<Parent> label;    // set for inner nodes
  std::vector<FullBinaryTree> kids;  // empty or exactly two

  static FullBinaryTree make_leaf(const Leaf &l) {
    FullBinaryTree t;
    t.leaf = l;
    return t;
  }
  static FullBinaryTree make_parent(const Parent &p, FullBinaryTree l, FullBinaryTree r) {
    FullBinaryTree t;
    t.label = p;
    t.kids.push_back(std::move(l));
    t.kids.push_back(std::move(r));
    return t;
  }
  bool is_leaf() const { return leaf.has_value(); }
  int num_nodes() const { return is_leaf() ? 1 : 1 + kids[0].num_nodes() + kids[1].num_nodes(); }
  std::vector<Leaf> leaves() const {
    if (is_leaf()) return {*leaf};
    auto l = kids[0].leaves(), r = kids[1].leaves();
    l.insert(l.end(), r.begin(), r.end());
    return l;
  }
  const FullBinaryTree *subtree_at(const BinaryTreePath &p) const {
    const FullBinaryTree *cur = this;
    for (Turn t : p) {
      if (cur->is_leaf()) return nullptr;
      cur = &cur->kids[t == Turn::LEFT ? 0 : 1];
    }
    return cur;
  }
  std::vector<BinaryTreePath> all_leaf_paths() const {
    std::vector<BinaryTreePath> out;
    collect(BinaryTreePath{}, out);
    return out;
  }

private:
  void collect(BinaryTreePath here, std::vector<BinaryTreePath> &out) const {
    if (is_leaf()) {
      out.push_back(here);
      return;
    }
    auto l = here, r = here;
    l.push_back(Turn::LEFT);
    r.push_back(Turn::RIGHT);
    kids[0].collect(l, out);
    kids[1].collect(r, out);
  }
};

// ------------------------------------------------------------------ orthotope index-space algebra
// An N-d box of extents; coordinates flatten row-major (last dim fastest).  Projections say how the dims of one
// space are laid onto another: an operator's task space onto a tensor's shard space (utils/orthotope).
struct Orthotope {
  std::vector<long long> dims;
  long long volume() const {
    long long v = 1;
    for (auto d : dims) v *= d;
    return v;
  }
  bool contains(const std::vector<long long> &c) const {
    if (c.size() != dims.size()) return false;
    for (size_t i = 0; i < c.size(); ++i)
      if (c[i] < 0 || c[i] >= dims[i]) return false;
    return true;
  }
  long long flatten(const std::vector<long long> &c) const {
    if (!contains(c)) throw std::out_of_range("coordinate outside the orthotope");
    long long f = 0;
    for (size_t i = 0; i < c.size(); ++i) f = f * dims[i] + c[i];
    return f;
  }
  std::vector<long long> unflatten(long long f) const {
    if (f < 0 || f >= volume()) throw std::out_of_range("flat index outside the orthotope");
    std::vector<long long> c(dims.size());
    for (size_t i = dims.size(); i-- > 0;) {
      c[i] = f % dims[i];
      f /= dims[i];
    }
    return c;
  }
  std::vector<std::vector<long long>> all_coords() const {
    std::vector<std::vector<long long>> out;
    for (long long f = 0; f < volume(); ++f) out.push_back(unflatten(f));
    return out;
  }
  // the same box without its extent-1 dims (MinimalOrthotope)
  Orthotope minimal() const {
    Orthotope m;
    for (auto d : dims)
      if (d != 1) m.dims.push_back(d);
    return m;
  }
};
// dst dim j is fed by the (row-major flattened) group of src dims `groups[j]`; src dims in no group are dropped
// (a Down projection), a dst dim with several src dims merges them, and one src dim per dst dim is the Eq projection.
struct DimProjection {
  std::vector<std::vector<int>> groups;
  static DimProjection identity(int n) {
    DimProjection p;
    for (int i = 0; i < n; ++i) p.groups.push_back({i});
    return p;
  }
  Orthotope project_domain(const Orthotope &src) const {
    Orthotope d;
    for (auto &g : groups) {
      long long e = 1;
      for (int i : g) e *= src.dims.at(i);
      d.dims.push_back(e);
    }
    return d;
  }
  std::vector<long long> project_coord(const Orthotope &src, const std::vector<long long> &c) const {
    if (!src.contains(c)) throw std::out_of_range("coordinate outside the source orthotope");
    std::vector<long long> out;
    for (auto &g : groups) {
      long long f = 0;
      for (int i : g) f = f * src.dims.at(i) + c.at(i);
      out.push_back(f);
    }
    return out;
  }
  // an Up projection in the other direction: split dst coordinate j back into its group's src dims (dropped src dims get 0)
  std::vector<long long> lift_coord(const Orthotope &src, const std::vector<long long> &dst_coord) const {
    std::vector<long long> c(src.dims.size(), 0);
    for (size_t j = 0; j < groups.size(); ++j) {
      long long f = dst_coord.at(j);
      for (size_t k = groups[j].size(); k-- > 0;) {
        int i = groups[j][k];
        c[i] = f % src.dims.at(i);
        f /= src.dims.at(i);
      }
    }
    return c;
  }
  bool is_bijection_on(const Orthotope &src) const {
    std::set<int> used;
    for (auto &g : groups)
      for (int i : g)
        if (!used.insert(i).second) return false;
    for (size_t i = 0; i < src.dims.size(); ++i)
      if (!used.count((int)i) && src.dims[i] != 1) return false;
    return true;
  }
};

// ------------------------------------------------------------------ undirected and multi graphs
class UndirectedGraph {
public:
  void add_node(int n) { adj_[n]; }
  void add_edge(int a, int b) {
    adj_[a].insert(b);
    adj_[b].insert(a);
  }
  void remove_edge(int a, int b) {
    adj_[a].erase(b);
    adj_[b].erase(a);
  }
  bool has_edge(int a, int b) const {
    auto it = adj_.find(a);
    return it != adj_.end() && it->second.count(b);
  }
  std::set<int> nodes() const {
    std::set<int> s;
    for (auto &kv : adj_) s.insert(kv.first);
    return s;
  }
  const std::set<int> &neighbors(int n) const { return adj_.at(n); }
  size_t num_edges() const {
    size_t e = 0;
    for (auto &kv : adj_) e += kv.second.size();
    return e / 2;
  }
  std::vector<std::set<int>> connected_components() const {
    disjoint_set<int> ds;
    for (auto &kv : adj_) {
      ds.find(kv.first);
      for (int b : kv.second) ds.unite(kv.first, b);
    }
    std::vector<std::set<int>> out;
    for (auto &g : ds.groups()) out.push_back(g.second);
    return out;
  }

private:
  std::map<int, std::set<int>> adj_;
};
// Directed graph with parallel edges, each with its own id (utils/graph/multidigraph).
class MultiDiGraph {
public:
  struct Edge {
    int id, src, dst;
  };
  void add_node(int n) { nodes_.insert(n); }
  int add_edge(int src, int dst) {
    nodes_.insert(src);
    nodes_.insert(dst);
    edges_.push_back({next_++, src, dst});
    return edges_.back().id;
  }
  void remove_edge(int id) {
    edges_.erase(std::remove_if(edges_.begin(), edges_.end(), [&](const Edge &e) { return e.id == id; }), edges_.end());
  }
  std::vector<Edge> edges_between(int src, int dst) const {
    std::vector<Edge> r;
    for (auto &e : edges_)
      if (e.src == src && e.dst == dst) r.push_back(e);
    return r;
  }
  std::vector<Edge> outgoing(int n) const {
    std::vector<Edge> r;
    for (auto &e : edges_)
      if (e.src == n) r.push_back(e);
    return r;
  }
  std::vector<Edge> incoming(int n) const {
    std::vector<Edge> r;
    for (auto &e : edges_)
      if (e.dst == n) r.push_back(e);
    return r;
  }
  const std::set<int> &nodes() const { return nodes_; }
  size_t num_edges() const { return edges_.size(); }

private:
  std::set<int> nodes_;
  std::vector<Edge> edges_;
  int next_ = 0;
};

// ------------------------------------------------------------------ formatters
// Graphviz text: nodes (optionally record-shaped), edges, nested clusters.
class DotFile {
public:
  explicit DotFile(std::string name = "g") : name_(std::move(name)) {}
  void add_node(const std::string &id, const std::map<std::string, std::string> &attrs = {}) { lines_.push_back("  " + quote(id) + fmt(attrs) + ";"); }
  void add_edge(const std::string &a, const std::string &b, const std::map<std::string, std::string> &attrs = {}) {
    lines_.push_back("  " + quote(a) + " -> " + quote(b) + fmt(attrs) + ";");
  }
  void begin_cluster(const std::string &label) {
    lines_.push_back("  subgraph cluster_" + std::to_string(clusters_++) + " {");
    lines_.push_back("  label=" + quote(label) + ";");
  }
  void end_cluster() { lines_.push_back("  }"); }
  std::string str() const {
    std::ostringstream os;
    os << "digraph " << name_ << " {\n";
    for (auto &l : lines_) os << l << "\n";
    os << "}\n";
    return os.str();
  }

private:
  static std::string quote(const std::string &s) {
    std::string r = "\"";
    for (char c : s) {
      if (c == '"' || c == '\\') r += '\\';
      r += c;
    }
    return r + "\"";
  }
  static std::string fmt(const std::map<std::string, std::string> &attrs) {
    if (attrs.empty()) return "";
    std::string r = " [";
    bool first = true;
    for (auto &kv : attrs) {
      if (!first) r += ", ";
      first = false;
      r += kv.first + "=" + quote(kv.second);
    }
    return r + "]";
  }
  std::string name_;
  std::vector<std::string> lines_;
  int clusters_ = 0;
};
// Graphviz record labels: "{a|{b|c}}" (utils/record_formatter.h)
class RecordFormatter {
public:
  RecordFormatter &operator<<(const std::string &field) {
    parts_.push_back(escape(field));
    return *this;
  }
  RecordFormatter &operator<<(const RecordFormatter &nested) {
    parts_.push_back(nested.str());
    return *this;
  }
  std::string str() const {
    std::string r = "{";
    for (size_t i = 0; i < parts_.size(); ++i) r += (i ? "|" : "") + parts_[i];
    return r + "}";
  }

private:
  static std::string escape(const std::string &s) {
    std::string r;
    for (char c : s) {
      if (c == '{' || c == '}' || c == '|' || c == '<' || c == '>' || c == '"') r += '\\';
      r += c;
    }
    return r;
  }
  std::vector<std::string> parts_;
};

}  // namespace utils
}  // namespace ff
