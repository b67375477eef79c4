// Container helpers: the functional vocabulary the compiler-side code is written in (the role of the reference's
// lib/utils/include/utils/containers/*.h, one header per helper there).  They work on the ordered standard containers
// this code base uses (std::vector, std::set, std::multiset, std::map) and return new containers; failed requirements
// throw std::runtime_error / std::out_of_range.  The helpers of utils.h (transform, filter, zip, cartesian_product,
// get_all_assignments, merge_maps_with, group_by, set_union, intersection, is_subseteq_of, keys, flatmap_concat,
// get_all_permutations, maximum, product) are not repeated.
#pragma once
#include <algorithm>
#include <cctype>
#include <functional>
#include <map>
#include <memory>
#include <numeric>
#include <optional>
#include <set>
#include <stdexcept>
#include <string>
#include <tuple>
#include <type_traits>
#include <utility>
#include <vector>

#include "utils.h"

namespace ff {
namespace utils {

namespace detail {
template <typename T>
struct optional_value;
template <typename T>
struct optional_value<std::optional<T>> {
  using type = T;
};
template <typename T>
using optional_value_t = typename optional_value<std::decay_t<T>>::type;
inline void require(bool ok, const char *what) {
  if (!ok) throw std::runtime_error(what);
}
}  // namespace detail

// ------------------------------------------------------------------ predicates
template <typename C, typename F>
bool all_of(const C &c, F pred) {
  for (auto &&x : c)
    if (!pred(x)) return false;
  return true;
}
template <typename C, typename F>
bool any_of(const C &c, F pred) {
  for (auto &&x : c)
    if (pred(x)) return true;
  return false;
}
template <typename C>
bool all_are_true(const C &c) {
  return all_of(c, [](bool b) { return b; });
}
template <typename C>
bool contains(const C &c, const typename C::value_type &e) {
  return std::find(c.begin(), c.end(), e) != c.end();
}
template <typename K, typename V>
bool contains_key(const std::map<K, V> &m, const K &k) {
  return m.find(k) != m.end();
}
template <typename K, typename V>
bool contains_value(const std::map<K, V> &m, const V &v) {
  return any_of(m, [&](const std::pair<const K, V> &kv) { return kv.second == v; });
}
template <typename C>
bool are_all_distinct(const C &c) {
  std::set<typename C::value_type> seen(c.begin(), c.end());
  return seen.size() == (size_t)std::distance(c.begin(), c.end());
}
template <typename C>
bool contains_duplicates(const C &c) {
  return !are_all_distinct(c);
}
template <typename C>
bool are_all_same(const C &c) {
  if (c.begin() == c.end()) return true;
  auto &first = *c.begin();
  return all_of(c, [&](const typename C::value_type &x) { return x == first; });
}
template <typename T>
bool are_disjoint(const std::set<T> &a, const std::set<T> &b) {
  return intersection(a, b).empty();
}
template <typename T>
bool is_superseteq_of(const std::set<T> &a, const std::set<T> &b) {
  return is_subseteq_of(b, a);
}
// every entry of `sub` is an entry of `super`
template <typename K, typename V>
bool is_submapeq_of(const std::map<K, V> &sub, const std::map<K, V> &super) {
  return all_of(sub, [&](const std::pair<const K, V> &kv) {
    auto it = super.find(kv.first);
    return it != super.end() && it->second == kv.second;
  });
}

// ------------------------------------------------------------------ folds and scans
template <typename C, typename T, typename F>
T foldl(const C &c, T acc, F f) {  // f(acc, element), left to right
  for (auto &&x : c) acc = f(acc, x);
  return acc;
}
template <typename C, typename F>
typename C::value_type foldl1(const C &c, F f) {
  detail::require(c.begin() != c.end(), "foldl1 of an empty container");
  auto it = c.begin();
  typename C::value_type acc = *it;
  for (++it; it != c.end(); ++it) acc = f(acc, *it);
  return acc;
}
// Right fold, f(element, acc) from the last element to the first: the first entry of scanr.  (The reference's foldr.h
// walks left to right with f(acc, element) like its foldl; nothing there calls it.)
template <typename C, typename T, typename F>
T foldr(const C &c, T acc, F f) {
  for (auto it = c.rbegin(); it != c.rend(); ++it) acc = f(*it, acc);
  return acc;
}
// starts from the last element and combines f(acc, element) towards the first (containers/foldr1.h)
template <typename T, typename F>
T foldr1(const std::vector<T> &v, F f) {
  detail::require(!v.empty(), "foldr1 of an empty vector");
  auto it = v.rbegin();
  T acc = *it;
  for (++it; it != v.rend(); ++it) acc = f(acc, *it);
  return acc;
}
template <typename C, typename T, typename F>
std::vector<T> scanl(const C &c, T acc, F f) {  // {init, f(init, c0), f(f(init, c0), c1), ...}
  std::vector<T> out{acc};
  for (auto &&x : c) out.push_back(acc = f(acc, x));
  return out;
}
template <typename C, typename F>
std::vector<typename C::value_type> scanl1(const C &c, F f) {
  std::vector<typename C::value_type> out;
  for (auto &&x : c) out.push_back(out.empty() ? x : f(out.back(), x));
  return out;
}
template <typename C, typename T, typename F>
std::vector<T> scanr(const C &c, T acc, F f) {  // {..., f(c[n-2], f(c[n-1], init)), f(c[n-1], init), init}
  std::vector<T> out{acc};
  for (auto it = c.rbegin(); it != c.rend(); ++it) out.push_back(acc = f(*it, acc));
  std::reverse(out.begin(), out.end());
  return out;
}
template <typename C, typename F>
std::vector<typename C::value_type> scanr1(const C &c, F f) {
  std::vector<typename C::value_type> out;
  for (auto it = c.rbegin(); it != c.rend(); ++it) out.push_back(out.empty() ? *it : f(*it, out.back()));
  std::reverse(out.begin(), out.end());
  return out;
}
template <typename C>
typename C::value_type sum(const C &c) {
  typename C::value_type s{};
  for (auto &&x : c) s = s + x;
  return s;
}
template <typename C, typename F>
typename C::value_type sum_where(const C &c, F pred) {
  typename C::value_type s{};
  for (auto &&x : c)
    if (pred(x)) s = s + x;
  return s;
}
template <typename C, typename F>
typename C::value_type product_where(const C &c, F pred) {
  typename C::value_type p = 1;
  for (auto &&x : c)
    if (pred(x)) p = p * x;
  return p;
}
template <typename F, typename T>
T recurse_n(F f, int n, T x) {  // f applied n times
  detail::require(n >= 0, "recurse_n wants a non-negative count");
  for (int i = 0; i < n; ++i) x = f(x);
  return x;
}

// ------------------------------------------------------------------ selection
template <typename C>
std::optional<typename C::value_type> minimum(const C &c) {
  if (c.begin() == c.end()) return std::nullopt;
  return *std::min_element(c.begin(), c.end());
}
template <typename C, typename F>
typename C::value_type argmax(const C &c, F key) {  // the first element with the largest key
  using E = typename C::value_type;
  return foldl1(c, [&](const E &best, const E &x) { return key(best) < key(x) ? x : best; });
}
template <typename C, typename F>
typename C::value_type argmin(const C &c, F key) {
  using E = typename C::value_type;
  return foldl1(c, [&](const E &best, const E &x) { return key(x) < key(best) ? x : best; });
}
template <typename T>
T at_idx(const std::vector<T> &v, size_t i) {
  if (i >= v.size()) throw std::out_of_range("at_idx: index past the end");
  return v[i];
}
template <typename T>
std::optional<T> try_at_idx(const std::vector<T> &v, size_t i) {
  return i < v.size() ? std::optional<T>(v[i]) : std::nullopt;
}
template <typename K, typename V>
std::optional<V> try_at(const std::map<K, V> &m, const K &k) {
  auto it = m.find(k);
  return it == m.end() ? std::nullopt : std::optional<V>(it->second);
}
template <typename K, typename V>
std::function<V(const K &)> lookup_in_map(const std::map<K, V> &m) {
  return [m](const K &k) { return m.at(k); };
}
template <typename C>
std::optional<size_t> index_of(const C &c, const typename C::value_type &e) {
  auto it = std::find(c.begin(), c.end(), e);
  if (it == c.end()) return std::nullopt;
  return (size_t)std::distance(c.begin(), it);
}
template <typename C, typename F>
size_t count(const C &c, F pred) {
  return (size_t)std::count_if(c.begin(), c.end(), pred);
}
template <typename C>
typename C::value_type get_one_of(const C &c) {
  detail::require(c.begin() != c.end(), "get_one_of an empty container");
  return *c.begin();
}
template <typename C>
std::optional<typename C::value_type> try_get_one_of(const C &c) {
  if (c.begin() == c.end()) return std::nullopt;
  return *c.begin();
}
template <typename C>
typename C::value_type get_only(const C &c) {
  detail::require(std::distance(c.begin(), c.end()) == 1, "get_only wants exactly one element");
  return *c.begin();
}
template <typename C>
std::optional<typename C::value_type> maybe_get_only(const C &c) {
  if (std::distance(c.begin(), c.end()) != 1) return std::nullopt;
  return *c.begin();
}
template <typename C>
std::map<typename C::value_type, int> get_element_counts(const C &c) {
  std::map<typename C::value_type, int> out;
  for (auto &&x : c) ++out[x];
  return out;
}

// ------------------------------------------------------------------ requirements
template <typename T>
T require_same(const T &a, const T &b) {
  detail::require(a == b, "require_same: the two values differ");
  return a;
}
template <typename C>
std::optional<typename C::value_type> require_all_same(const C &c) {  // nullopt for an empty container
  if (c.begin() == c.end()) return std::nullopt;
  detail::require(are_all_same(c), "require_all_same: the elements differ");
  return *c.begin();
}
template <typename C>
typename C::value_type require_all_same1(const C &c) {
  detail::require(c.begin() != c.end(), "require_all_same1 of an empty container");
  detail::require(are_all_same(c), "require_all_same1: the elements differ");
  return *c.begin();
}
template <typename T>
std::set<T> require_no_duplicates(const std::vector<T> &v) {
  std::set<T> s(v.begin(), v.end());
  detail::require(s.size() == v.size(), "require_no_duplicates: an element repeats");
  return s;
}
template <typename K, typename V>
V require_only_key(const std::map<K, V> &m, const K &k) {
  detail::require(m.size() == 1 && m.count(k) == 1, "require_only_key: the map is not {key: value}");
  return m.at(k);
}
template <typename K, typename V>
std::pair<V, V> require_two_keys(const std::map<K, V> &m, const K &k1, const K &k2) {
  detail::require(!(k1 == k2) && m.size() == 2 && m.count(k1) && m.count(k2), "require_two_keys: the map does not have exactly these two keys");
  return {m.at(k1), m.at(k2)};
}

// ------------------------------------------------------------------ building sequences
inline std::vector<int> range(int start, int end, int step = 1) {  // python semantics; step may be negative
  detail::require(step != 0, "range with step 0");
  std::vector<int> out;
  if (step > 0)
    for (int i = start; i < end; i += step) out.push_back(i);
  else
    for (int i = start; i > end; i += step) out.push_back(i);
  return out;
}
inline std::vector<int> range(int end) { return range(0, end); }
template <typename F>
auto repeat(size_t n, F f) -> std::vector<decltype(f())> {  // n results of calling f
  std::vector<decltype(f())> out;
  for (size_t i = 0; i < n; ++i) out.push_back(f());
  return out;
}
template <typename T>
std::vector<T> repeat_element(size_t n, const T &x) {
  return std::vector<T>(n, x);
}
inline std::function<int()> make_counter_func(int start = 0) {
  auto next = std::make_shared<int>(start);
  return [next]() { return (*next)++; };
}
template <typename F>
auto generate_vector(size_t n, F f) -> std::vector<decltype(f((size_t)0))> {  // {f(0), ..., f(n-1)}
  std::vector<decltype(f((size_t)0))> out;
  for (size_t i = 0; i < n; ++i) out.push_back(f(i));
  return out;
}
template <typename C, typename F>
auto generate_map(const C &keys_, F f) -> std::map<typename C::value_type, decltype(f(*keys_.begin()))> {
  std::map<typename C::value_type, decltype(f(*keys_.begin()))> out;
  for (auto &k : keys_) {
    detail::require(out.count(k) == 0, "generate_map: a key repeats");
    out.emplace(k, f(k));
  }
  return out;
}
template <typename C>
std::vector<typename C::value_type> vector_of(const C &c) {
  return std::vector<typename C::value_type>(c.begin(), c.end());
}
template <typename C>
std::set<typename C::value_type> set_of(const C &c) {
  return std::set<typename C::value_type>(c.begin(), c.end());
}
template <typename C>
std::multiset<typename C::value_type> multiset_of(const C &c) {
  return std::multiset<typename C::value_type>(c.begin(), c.end());
}
template <typename C>
std::vector<typename C::value_type> sorted(const C &c) {
  std::vector<typename C::value_type> v(c.begin(), c.end());
  std::sort(v.begin(), v.end());
  return v;
}
template <typename C, typename F>
std::vector<typename C::value_type> sorted_by(const C &c, F less) {  // stable
  std::vector<typename C::value_type> v(c.begin(), c.end());
  std::stable_sort(v.begin(), v.end(), less);
  return v;
}
template <typename T, typename F>
std::function<bool(const T &, const T &)> compare_by(F key) {
  return [key](const T &a, const T &b) { return key(a) < key(b); };
}
template <typename T>
std::vector<T> reversed(std::vector<T> v) {
  std::reverse(v.begin(), v.end());
  return v;
}
template <typename T>
std::vector<T> concat_vectors(const std::vector<T> &a, const std::vector<T> &b) {
  std::vector<T> out = a;
  out.insert(out.end(), b.begin(), b.end());
  return out;
}
template <typename T>
std::vector<T> concat_vectors(const std::vector<std::vector<T>> &vs) {
  return flatmap_concat(vs);
}
template <typename T, typename C>
void extend(std::vector<T> &dst, const C &src) {
  dst.insert(dst.end(), src.begin(), src.end());
}
template <typename T, typename C>
void extend(std::set<T> &dst, const C &src) {
  dst.insert(src.begin(), src.end());
}
// python's v[start:end]: negative positions count from the end, an empty result when start >= end; a position outside
// [-size, size] is an error
template <typename T>
std::vector<T> slice(const std::vector<T> &v, int start, std::optional<int> end = std::nullopt) {
  const int n = (int)v.size();
  auto resolve = [&](int i) {
    const int j = i < 0 ? n + i : i;
    if (j < 0 || j > n) throw std::out_of_range("slice: position outside the vector");
    return j;
  };
  const int b = resolve(start), e = end ? resolve(*end) : n;
  if (b >= e) return {};
  return std::vector<T>(v.begin() + b, v.begin() + e);
}
template <typename T>
std::pair<std::vector<T>, std::vector<T>> vector_split(const std::vector<T> &v, int idx) {
  if (idx < 0 || idx > (int)v.size()) throw std::out_of_range("vector_split: index outside the vector");
  return {std::vector<T>(v.begin(), v.begin() + idx), std::vector<T>(v.begin() + idx, v.end())};
}
// {0: a, 1: b, ...} -> {a, b, ...}; nullopt unless the keys are exactly 0..n-1
template <typename T>
std::optional<std::vector<T>> vector_from_idx_map(const std::map<int, T> &m) {
  std::vector<T> out;
  for (auto &kv : m) {
    if (kv.first != (int)out.size()) return std::nullopt;
    out.push_back(kv.second);
  }
  return out;
}
template <typename T>
std::map<int, T> enumerate_vector(const std::vector<T> &v) {
  std::map<int, T> out;
  for (size_t i = 0; i < v.size(); ++i) out.emplace((int)i, v[i]);
  return out;
}
template <typename C>
std::map<int, typename C::value_type> enumerate(const C &c) {  // in iteration order
  std::map<int, typename C::value_type> out;
  int i = 0;
  for (auto &&x : c) out.emplace(i++, x);
  return out;
}
// the key-th permutation (lexicographic order of the positions, key taken modulo 10000) of v
template <typename T>
std::vector<T> permute_with_key(int key, const std::vector<T> &v) {
  std::vector<int> pos = range((int)v.size());
  for (int i = 0, n = key % 10000; i < n; ++i) std::next_permutation(pos.begin(), pos.end());
  std::vector<T> out;
  for (int p : pos) out.push_back(v[p]);
  return out;
}
// all length-n sequences over the elements of c (|c|^n of them; one empty sequence when n == 0 or c is empty)
template <typename C>
std::multiset<std::vector<typename C::value_type>> get_all_permutations_with_repetition(const C &c, size_t n) {
  using T = typename C::value_type;
  std::vector<T> elems(c.begin(), c.end());
  if (elems.empty() || n == 0) return {{}};
  std::multiset<std::vector<T>> out;
  std::vector<size_t> idx(n, 0);
  for (;;) {
    std::vector<T> seq;
    for (size_t i : idx) seq.push_back(elems[i]);
    out.insert(seq);
    size_t d = n;
    while (d > 0 && ++idx[d - 1] == elems.size()) idx[--d] = 0;
    if (d == 0) return out;
  }
}
template <typename A, typename B>
std::set<std::pair<A, B>> binary_cartesian_product(const std::set<A> &a, const std::set<B> &b) {
  std::set<std::pair<A, B>> out;
  for (auto &x : a)
    for (auto &y : b) out.insert({x, y});
  return out;
}

// ------------------------------------------------------------------ zips
template <typename A, typename B>
std::vector<std::pair<A, B>> zip_strict(const std::vector<A> &a, const std::vector<B> &b) {
  detail::require(a.size() == b.size(), "zip_strict: lengths differ");
  return zip(a, b);
}
template <typename A, typename B, typename F>
auto zip_with(const std::vector<A> &a, const std::vector<B> &b, F f) -> std::vector<decltype(f(a[0], b[0]))> {
  std::vector<decltype(f(a[0], b[0]))> out;
  for (size_t i = 0; i < std::min(a.size(), b.size()); ++i) out.push_back(f(a[i], b[i]));
  return out;
}
template <typename A, typename B, typename F>
auto zip_with_strict(const std::vector<A> &a, const std::vector<B> &b, F f) -> std::vector<decltype(f(a[0], b[0]))> {
  detail::require(a.size() == b.size(), "zip_with_strict: lengths differ");
  return zip_with(a, b, f);
}
template <typename A, typename B, typename C>
std::vector<std::tuple<A, B, C>> zip3(const std::vector<A> &a, const std::vector<B> &b, const std::vector<C> &c) {
  std::vector<std::tuple<A, B, C>> out;
  for (size_t i = 0; i < std::min({a.size(), b.size(), c.size()}); ++i) out.emplace_back(a[i], b[i], c[i]);
  return out;
}
template <typename A, typename B, typename C>
std::vector<std::tuple<A, B, C>> zip3_strict(const std::vector<A> &a, const std::vector<B> &b, const std::vector<C> &c) {
  detail::require(a.size() == b.size() && b.size() == c.size(), "zip3_strict: lengths differ");
  return zip3(a, b, c);
}
template <typename A, typename B, typename C, typename F>
auto zip3_with(const std::vector<A> &a, const std::vector<B> &b, const std::vector<C> &c, F f) -> std::vector<decltype(f(a[0], b[0], c[0]))> {
  std::vector<decltype(f(a[0], b[0], c[0]))> out;
  for (size_t i = 0; i < std::min({a.size(), b.size(), c.size()}); ++i) out.push_back(f(a[i], b[i], c[i]));
  return out;
}
template <typename A, typename B, typename C, typename F>
auto zip3_with_strict(const std::vector<A> &a, const std::vector<B> &b, const std::vector<C> &c, F f) -> std::vector<decltype(f(a[0], b[0], c[0]))> {
  detail::require(a.size() == b.size() && b.size() == c.size(), "zip3_with_strict: lengths differ");
  return zip3_with(a, b, c, f);
}
// two maps over the same key set -> key -> f(v1, v2)
template <typename K, typename V1, typename V2, typename F>
auto zip_values_strict_with(const std::map<K, V1> &a, const std::map<K, V2> &b, F f) -> std::map<K, decltype(f(a.begin()->second, b.begin()->second))> {
  detail::require(keys(a) == keys(b), "zip_values_strict: key sets differ");
  std::map<K, decltype(f(a.begin()->second, b.begin()->second))> out;
  for (auto &kv : a) out.emplace(kv.first, f(kv.second, b.at(kv.first)));
  return out;
}
template <typename K, typename V1, typename V2>
std::map<K, std::pair<V1, V2>> zip_values_strict(const std::map<K, V1> &a, const std::map<K, V2> &b) {
  return zip_values_strict_with(a, b, [](const V1 &x, const V2 &y) { return std::pair<V1, V2>(x, y); });
}
template <typename F>
auto uncurry(F f) {  // a two-argument function as a function of a pair
  return [f](const auto &p) { return f(p.first, p.second); };
}

// ------------------------------------------------------------------ element-wise transformations
template <typename T, typename F>
auto vector_transform(const std::vector<T> &v, F f) -> std::vector<decltype(f(v[0]))> {
  return transform(v, f);
}
template <typename T, typename F>
std::vector<T> filter_idxs(const std::vector<T> &v, F keep_index) {
  std::vector<T> out;
  for (size_t i = 0; i < v.size(); ++i)
    if (keep_index(i)) out.push_back(v[i]);
  return out;
}
template <typename C, typename F>
void inplace_filter(C &c, F pred) {
  for (auto it = c.begin(); it != c.end();) it = pred(*it) ? std::next(it) : c.erase(it);
}
// f returns an optional; the present results are kept
template <typename T, typename F>
auto filtrans(const std::vector<T> &v, F f) -> std::vector<detail::optional_value_t<decltype(f(v[0]))>> {
  std::vector<detail::optional_value_t<decltype(f(v[0]))>> out;
  for (auto &x : v)
    if (auto r = f(x)) out.push_back(*r);
  return out;
}
template <typename T, typename F>
auto filtrans(const std::set<T> &s, F f) -> std::set<detail::optional_value_t<decltype(f(*s.begin()))>> {
  std::set<detail::optional_value_t<decltype(f(*s.begin()))>> out;
  for (auto &x : s)
    if (auto r = f(x)) out.insert(*r);
  return out;
}
// results of f up to (not including) its first empty one
template <typename T, typename F>
auto transform_until(const std::vector<T> &v, F f) -> std::vector<detail::optional_value_t<decltype(f(v[0]))>> {
  std::vector<detail::optional_value_t<decltype(f(v[0]))>> out;
  for (auto &x : v) {
    auto r = f(x);
    if (!r) break;
    out.push_back(*r);
  }
  return out;
}
template <typename T, typename F>
auto flatmap(const std::vector<T> &v, F f) -> std::vector<typename decltype(f(v[0]))::value_type> {
  std::vector<typename decltype(f(v[0]))::value_type> out;
  for (auto &x : v) extend(out, f(x));
  return out;
}
template <typename T, typename F>
auto flatmap(const std::set<T> &s, F f) -> std::set<typename decltype(f(*s.begin()))::value_type> {
  std::set<typename decltype(f(*s.begin()))::value_type> out;
  for (auto &x : s) extend(out, f(x));
  return out;
}
template <typename T>
std::optional<T> collapse_optionals(const std::optional<std::optional<T>> &o) {
  return o ? *o : std::nullopt;
}
template <typename T>
std::vector<T> without_nullopts(const std::vector<std::optional<T>> &v) {
  std::vector<T> out;
  for (auto &x : v)
    if (x) out.push_back(*x);
  return out;
}
template <typename T>
std::vector<T> value_all(const std::vector<std::optional<T>> &v) {
  std::vector<T> out;
  for (auto &x : v) {
    detail::require(x.has_value(), "value_all: an element is empty");
    out.push_back(*x);
  }
  return out;
}
inline std::string to_uppercase(std::string s) {
  for (auto &ch : s) ch = (char)std::toupper((unsigned char)ch);
  return s;
}

// ------------------------------------------------------------------ maps
template <typename K, typename V>
std::vector<V> values(const std::map<K, V> &m) {  // in key order, repeats kept
  std::vector<V> out;
  for (auto &kv : m) out.push_back(kv.second);
  return out;
}
template <typename K, typename V>
std::vector<std::pair<K, V>> items(const std::map<K, V> &m) {
  return std::vector<std::pair<K, V>>(m.begin(), m.end());
}
template <typename C>
auto map_from_pairs(const C &pairs) -> std::map<typename C::value_type::first_type, typename C::value_type::second_type> {
  std::map<typename C::value_type::first_type, typename C::value_type::second_type> out;
  for (auto &p : pairs) detail::require(out.emplace(p.first, p.second).second, "map_from_pairs: a key repeats");
  return out;
}
template <typename K, typename V>
std::map<K, V> map_from_keys_and_values(const std::vector<K> &ks, const std::vector<V> &vs) {
  detail::require(ks.size() == vs.size(), "map_from_keys_and_values: lengths differ");
  return map_from_pairs(zip(ks, vs));
}
template <typename K, typename V, typename F>
std::map<K, V> filter_keys(const std::map<K, V> &m, F pred) {
  std::map<K, V> out;
  for (auto &kv : m)
    if (pred(kv.first)) out.insert(kv);
  return out;
}
template <typename K, typename V, typename F>
std::map<K, V> filter_values(const std::map<K, V> &m, F pred) {
  std::map<K, V> out;
  for (auto &kv : m)
    if (pred(kv.second)) out.insert(kv);
  return out;
}
template <typename K, typename V, typename F>
auto filtermap_keys(const std::map<K, V> &m, F f) -> std::map<detail::optional_value_t<decltype(f(m.begin()->first))>, V> {
  std::map<detail::optional_value_t<decltype(f(m.begin()->first))>, V> out;
  for (auto &kv : m)
    if (auto k2 = f(kv.first)) out.emplace(*k2, kv.second);
  return out;
}
template <typename K, typename V, typename F>
auto filtermap_values(const std::map<K, V> &m, F f) -> std::map<K, detail::optional_value_t<decltype(f(m.begin()->second))>> {
  std::map<K, detail::optional_value_t<decltype(f(m.begin()->second))>> out;
  for (auto &kv : m)
    if (auto v2 = f(kv.second)) out.emplace(kv.first, *v2);
  return out;
}
template <typename K, typename V, typename F>
auto map_keys(const std::map<K, V> &m, F f) -> std::map<decltype(f(m.begin()->first)), V> {  // f must keep the keys distinct
  std::map<decltype(f(m.begin()->first)), V> out;
  for (auto &kv : m) detail::require(out.emplace(f(kv.first), kv.second).second, "map_keys: two keys map to the same key");
  return out;
}
template <typename K, typename V, typename F>
auto map_keys2(const std::map<K, V> &m, F f) -> std::map<decltype(f(m.begin()->first, m.begin()->second)), V> {  // f(key, value)
  std::map<decltype(f(m.begin()->first, m.begin()->second)), V> out;
  for (auto &kv : m) detail::require(out.emplace(f(kv.first, kv.second), kv.second).second, "map_keys2: two keys map to the same key");
  return out;
}
template <typename K, typename V, typename F>
auto map_values(const std::map<K, V> &m, F f) -> std::map<K, decltype(f(m.begin()->second))> {
  std::map<K, decltype(f(m.begin()->second))> out;
  for (auto &kv : m) out.emplace(kv.first, f(kv.second));
  return out;
}
template <typename K, typename V, typename F>
auto map_values2(const std::map<K, V> &m, F f) -> std::map<K, decltype(f(m.begin()->first, m.begin()->second))> {  // f(key, value)
  std::map<K, decltype(f(m.begin()->first, m.begin()->second))> out;
  for (auto &kv : m) out.emplace(kv.first, f(kv.first, kv.second));
  return out;
}
template <typename K, typename V, typename FK, typename FV>
auto map_keys_and_values(const std::map<K, V> &m, FK fk, FV fv) -> std::map<decltype(fk(m.begin()->first)), decltype(fv(m.begin()->second))> {
  std::map<decltype(fk(m.begin()->first)), decltype(fv(m.begin()->second))> out;
  for (auto &kv : m) detail::require(out.emplace(fk(kv.first), fv(kv.second)).second, "map_keys_and_values: two keys map to the same key");
  return out;
}
// keys that collide after f have their values combined with merge(old, new), in key order
template <typename K, typename V, typename F, typename M>
auto map_keys_with_value_merging(const std::map<K, V> &m, F f, M merge) -> std::map<decltype(f(m.begin()->first)), V> {
  std::map<decltype(f(m.begin()->first)), V> out;
  for (auto &kv : m) {
    auto k2 = f(kv.first);
    auto it = out.find(k2);
    if (it == out.end()) out.emplace(k2, kv.second);
    else it->second = merge(it->second, kv.second);
  }
  return out;
}
template <typename K, typename V>
std::map<V, std::set<K>> invert_map(const std::map<K, V> &m) {  // value -> the keys that had it
  std::map<V, std::set<K>> out;
  for (auto &kv : m) out[kv.second].insert(kv.first);
  return out;
}
template <typename K, typename V>
std::map<K, V> restrict_keys(const std::map<K, V> &m, const std::set<K> &keep) {
  return filter_keys(m, [&](const K &k) { return keep.count(k) > 0; });
}
// all values present -> the map of values; all empty -> nullopt; a mixture (or an empty map) is an error
template <typename K, typename V>
std::optional<std::map<K, V>> lift_optional_through_map(const std::map<K, std::optional<V>> &m) {
  detail::require(!m.empty(), "lift_optional_through_map of an empty map");
  const size_t present = count(m, [](const std::pair<const K, std::optional<V>> &kv) { return kv.second.has_value(); });
  detail::require(present == 0 || present == m.size(), "lift_optional_through_map: some values are present and some are not");
  if (present == 0) return std::nullopt;
  return map_values(m, [](const std::optional<V> &v) { return *v; });
}
template <typename K, typename V>
void merge_in_map(const std::map<K, V> &src, std::map<K, V> &dst) {  // src's entries win
  for (auto &kv : src) dst[kv.first] = kv.second;
}
template <typename K, typename V>
std::map<K, V> binary_merge_disjoint_maps(const std::map<K, V> &a, const std::map<K, V> &b) {
  std::map<K, V> out = a;
  for (auto &kv : b) detail::require(out.insert(kv).second, "binary_merge_disjoint_maps: a key is in both maps");
  return out;
}
template <typename K, typename V>
std::map<K, V> binary_merge_maps_with_left_dominating(const std::map<K, V> &a, const std::map<K, V> &b) {
  return merge_maps_with(a, b, [](const V &l, const V &) { return l; });
}
template <typename K, typename V>
std::map<K, V> binary_merge_maps_with_right_dominating(const std::map<K, V> &a, const std::map<K, V> &b) {
  return merge_maps_with(a, b, [](const V &, const V &r) { return r; });
}
template <typename K, typename V>
std::map<K, V> merge_disjoint_maps(const std::vector<std::map<K, V>> &ms) {
  return foldl(ms, std::map<K, V>{}, [](const std::map<K, V> &a, const std::map<K, V> &b) { return binary_merge_disjoint_maps(a, b); });
}
template <typename K, typename V>
std::map<K, V> merge_maps_with_right_dominating(const std::vector<std::map<K, V>> &ms) {
  return foldl(ms, std::map<K, V>{}, [](const std::map<K, V> &a, const std::map<K, V> &b) { return binary_merge_maps_with_right_dominating(a, b); });
}
// the union of two maps that may share keys, provided they agree on them; nullopt when they do not
template <typename K, typename V>
std::optional<std::map<K, V>> try_merge_nondisjoint_maps(const std::map<K, V> &a, const std::map<K, V> &b) {
  std::map<K, V> out = a;
  for (auto &kv : b) {
    auto ins = out.insert(kv);
    if (!ins.second && !(ins.first->second == kv.second)) return std::nullopt;
  }
  return out;
}

// ------------------------------------------------------------------ sets
template <typename T>
std::set<T> set_minus(const std::set<T> &a, const std::set<T> &b) {
  std::set<T> out;
  for (auto &x : a)
    if (!b.count(x)) out.insert(x);
  return out;
}
template <typename T>
std::set<T> set_difference(const std::set<T> &a, const std::set<T> &b) {
  return set_minus(a, b);
}
template <typename T>
std::set<T> set_intersection(const std::set<T> &a, const std::set<T> &b) {
  return intersection(a, b);
}
template <typename T>
std::optional<std::set<T>> set_intersection(const std::vector<std::set<T>> &sets) {  // nullopt for no sets at all
  if (sets.empty()) return std::nullopt;
  return foldl1(sets, [](const std::set<T> &a, const std::set<T> &b) { return intersection(a, b); });
}
template <typename T>
std::set<T> set_union(const std::vector<std::set<T>> &sets) {
  return foldl(sets, std::set<T>{}, [](const std::set<T> &a, const std::set<T> &b) { return set_union(a, b); });
}
template <typename T>
std::multiset<T> multiset_union(const std::multiset<T> &a, const std::multiset<T> &b) {  // multiplicities add
  std::multiset<T> out = a;
  out.insert(b.begin(), b.end());
  return out;
}


// ------------------------------------------------------------------ strings
template <typename C, typename F>
std::string join_strings(const C &c, const std::string &delimiter, F f) {
  std::string out;
  bool first = true;
  for (auto &&x : c) {
    if (!first) out += delimiter;
    out += f(x);
    first = false;
  }
  return out;
}
template <typename C>
std::string join_strings(const C &c, const std::string &delimiter) {
  return join_strings(c, delimiter, [](const std::string &x) { return x; });
}
// every line, the first and an empty last one included, moved right by indent_size spaces
inline std::string indent(const std::string &text, int indent_size = 2) {
  const std::string pad((size_t)indent_size, ' ');
  std::string out = pad;
  for (char ch : text) {
    out += ch;
    if (ch == '\n') out += pad;
  }
  return out;
}

// ------------------------------------------------------------------ small value types
// an unordered pair: (a, b) == (b, a); ordered by (max, min)
template <typename T>
class commutative_pair {
public:
  commutative_pair(const T &a, const T &b) : hi_(a < b ? b : a), lo_(a < b ? a : b) {}
  const T &max() const { return hi_; }
  const T &min() const { return lo_; }
  bool operator==(const commutative_pair &o) const { return hi_ == o.hi_ && lo_ == o.lo_; }
  bool operator!=(const commutative_pair &o) const { return !(*this == o); }
  bool operator<(const commutative_pair &o) const { return std::tie(hi_, lo_) < std::tie(o.hi_, o.lo_); }

private:
  T hi_, lo_;
};
// a query over values: everything, nothing, or a set of allowed values (utils/graph/query_set.h)
template <typename T>
class query_set {
public:
  static query_set matchall() { return query_set(std::nullopt); }
  static query_set match_none() { return query_set(std::set<T>{}); }
  static query_set match_values_in(const std::set<T> &v) { return query_set(v); }
  static query_set match_single_value(const T &v) { return query_set(std::set<T>{v}); }
  bool is_matchall() const { return !allowed_.has_value(); }
  bool includes(const T &v) const { return !allowed_ || allowed_->count(v) > 0; }
  const std::set<T> &allowed_values() const {
    detail::require(allowed_.has_value(), "allowed_values of a match-all query");
    return *allowed_;
  }
  std::set<T> apply(const std::set<T> &universe) const { return allowed_ ? intersection(universe, *allowed_) : universe; }
  query_set intersect(const query_set &o) const {
    if (is_matchall()) return o;
    if (o.is_matchall()) return *this;
    return query_set(intersection(*allowed_, *o.allowed_));
  }
  bool operator==(const query_set &o) const { return allowed_ == o.allowed_; }

private:
  explicit query_set(std::optional<std::set<T>> a) : allowed_(std::move(a)) {}
  std::optional<std::set<T>> allowed_;
};
// fixed-capacity string and map without heap allocation (utils/stack_string.h, stack_map.h), over stack_vector
template <size_t MAXSIZE>
class stack_string {
public:
  stack_string() = default;
  stack_string(const char *s) {   // NOLINT: converting on purpose, like the reference's
    for (; *s; ++s) chars_.push_back(*s);
  }
  stack_string(const std::string &s) : stack_string(s.c_str()) {}   // NOLINT
  size_t size() const { return chars_.size(); }
  size_t length() const { return chars_.size(); }
  char operator[](size_t i) const { return chars_[i]; }
  void push_back(char ch) { chars_.push_back(ch); }
  operator std::string() const { return std::string(chars_.begin(), chars_.end()); }   // NOLINT
  bool operator==(const stack_string &o) const { return (std::string)*this == (std::string)o; }
  bool operator<(const stack_string &o) const { return (std::string)*this < (std::string)o; }

private:
  stack_vector<char, MAXSIZE> chars_;
};
template <typename K, typename V, size_t MAXSIZE>
class stack_map {
public:
  V &operator[](const K &k) {
    for (auto &kv : items_)
      if (kv.first == k) return kv.second;
    items_.push_back({k, V{}});
    return items_.back().second;
  }
  void insert(const K &k, const V &v) { (*this)[k] = v; }
  const V &at(const K &k) const {
    for (auto &kv : items_)
      if (kv.first == k) return kv.second;
    throw std::out_of_range("stack_map::at: no such key");
  }
  bool contains(const K &k) const {
    for (auto &kv : items_)
      if (kv.first == k) return true;
    return false;
  }
  size_t size() const { return items_.size(); }
  std::vector<std::pair<K, V>> sorted_items() const {   // in key order
    std::vector<std::pair<K, V>> out(items_.begin(), items_.end());
    std::sort(out.begin(), out.end(), [](const std::pair<K, V> &a, const std::pair<K, V> &b) { return a.first < b.first; });
    return out;
  }

private:
  stack_vector<std::pair<K, V>, MAXSIZE> items_;
};

}  // namespace utils
}  // namespace ff
