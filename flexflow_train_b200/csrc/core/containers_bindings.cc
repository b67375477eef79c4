// Python view of containers.h, instantiated on ints, strings and Python callables: `_ffcore.containers`.  It exists so
// that the helpers are exercised from the test-suite the way the reference tests its lib/utils/containers one by one.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "containers.h"

namespace py = pybind11;

namespace ff {
using namespace ff::utils;

using VI = std::vector<int>;
using SI = std::set<int>;
using MSI = std::map<std::string, int>;
using MII = std::map<int, int>;
using OI = std::optional<int>;
using F1 = std::function<int(int)>;
using F2 = std::function<int(int, int)>;
using P1 = std::function<bool(int)>;
using FO = std::function<OI(int)>;

void bind_containers(py::module &root) {
  py::module m = root.def_submodule("containers", "functional container helpers (csrc/core/containers.h) on ints and strings");
  // predicates
  m.def("all_of", [](const VI &v, P1 p) { return all_of(v, p); });
  m.def("any_of", [](const VI &v, P1 p) { return any_of(v, p); });
  m.def("all_are_true", [](const std::vector<bool> &v) { return all_are_true(v); });
  m.def("contains", [](const VI &v, int e) { return contains(v, e); });
  m.def("contains_key", [](const MSI &mp, const std::string &k) { return contains_key(mp, k); });
  m.def("contains_value", [](const MSI &mp, int v) { return contains_value(mp, v); });
  m.def("are_all_distinct", [](const VI &v) { return are_all_distinct(v); });
  m.def("contains_duplicates", [](const VI &v) { return contains_duplicates(v); });
  m.def("are_all_same", [](const VI &v) { return are_all_same(v); });
  m.def("are_disjoint", [](const SI &a, const SI &b) { return are_disjoint(a, b); });
  m.def("is_superseteq_of", [](const SI &a, const SI &b) { return is_superseteq_of(a, b); });
  m.def("is_submapeq_of", [](const MSI &a, const MSI &b) { return is_submapeq_of(a, b); });
  // folds
  m.def("foldl", [](const VI &v, int init, F2 f) { return foldl(v, init, f); });
  m.def("foldl1", [](const VI &v, F2 f) { return foldl1(v, f); });
  m.def("foldr", [](const VI &v, int init, F2 f) { return foldr(v, init, f); });
  m.def("foldr1", [](const VI &v, F2 f) { return foldr1(v, f); });
  m.def("scanl", [](const VI &v, int init, F2 f) { return scanl(v, init, f); });
  m.def("scanl1", [](const VI &v, F2 f) { return scanl1(v, f); });
  m.def("scanr", [](const VI &v, int init, F2 f) { return scanr(v, init, f); });
  m.def("scanr1", [](const VI &v, F2 f) { return scanr1(v, f); });
  m.def("sum", [](const VI &v) { return sum(v); });
  m.def("sum_where", [](const VI &v, P1 p) { return sum_where(v, p); });
  m.def("product_where", [](const VI &v, P1 p) { return product_where(v, p); });
  m.def("recurse_n", [](F1 f, int n, int x) { return recurse_n(f, n, x); });
  // selection
  m.def("minimum", [](const VI &v) { return minimum(v); });
  m.def("argmax", [](const VI &v, F1 key) { return argmax(v, key); });
  m.def("argmin", [](const VI &v, F1 key) { return argmin(v, key); });
  m.def("at_idx", [](const VI &v, size_t i) { return at_idx(v, i); });
  m.def("try_at_idx", [](const VI &v, size_t i) { return try_at_idx(v, i); });
  m.def("try_at", [](const MSI &mp, const std::string &k) { return try_at(mp, k); });
  m.def("lookup_in_map", [](const MSI &mp, const std::string &k) { return lookup_in_map(mp)(k); });
  m.def("index_of", [](const VI &v, int e) { return index_of(v, e); });
  m.def("count", [](const VI &v, P1 p) { return count(v, p); });
  m.def("get_one_of", [](const SI &s) { return get_one_of(s); });
  m.def("try_get_one_of", [](const SI &s) { return try_get_one_of(s); });
  m.def("get_only", [](const VI &v) { return get_only(v); });
  m.def("maybe_get_only", [](const VI &v) { return maybe_get_only(v); });
  m.def("get_element_counts", [](const VI &v) { return get_element_counts(v); });
  // requirements
  m.def("require_same", [](int a, int b) { return require_same(a, b); });
  m.def("require_all_same", [](const VI &v) { return require_all_same(v); });
  m.def("require_all_same1", [](const VI &v) { return require_all_same1(v); });
  m.def("require_no_duplicates", [](const VI &v) { return require_no_duplicates(v); });
  m.def("require_only_key", [](const MSI &mp, const std::string &k) { return require_only_key(mp, k); });
  m.def("require_two_keys", [](const MSI &mp, const std::string &a, const std::string &b) { return require_two_keys(mp, a, b); });
  // building
  m.def("range", [](int a, int b, int step) { return range(a, b, step); }, py::arg("start"), py::arg("end"), py::arg("step") = 1);
  m.def("repeat", [](size_t n, std::function<int()> f) { return repeat(n, f); });
  m.def("repeat_element", [](size_t n, int x) { return repeat_element(n, x); });
  m.def("counter_values", [](int start, int n) {
    auto next = make_counter_func(start);
    return repeat((size_t)n, next);
  });
  m.def("generate_vector", [](size_t n, std::function<int(size_t)> f) { return generate_vector(n, f); });
  m.def("generate_map", [](const VI &ks, F1 f) { return generate_map(ks, f); });
  m.def("vector_of", [](const SI &s) { return vector_of(s); });
  m.def("set_of", [](const VI &v) { return set_of(v); });
  m.def("multiset_of", [](const VI &v) { return vector_of(multiset_of(v)); });
  m.def("sorted", [](const VI &v) { return sorted(v); });
  m.def("sorted_by_key", [](const VI &v, F1 key) { return sorted_by(v, compare_by<int>(key)); });
  m.def("reversed", [](const VI &v) { return reversed(v); });
  m.def("concat_vectors", [](const VI &a, const VI &b) { return concat_vectors(a, b); });
  m.def("concat_all", [](const std::vector<VI> &vs) { return concat_vectors(vs); });
  m.def("extend", [](VI a, const SI &b) { extend(a, b); return a; });
  m.def("slice", [](const VI &v, int start, OI end) { return slice(v, start, end); }, py::arg("v"), py::arg("start"), py::arg("end") = py::none());
  m.def("vector_split", [](const VI &v, int i) { return vector_split(v, i); });
  m.def("vector_from_idx_map", [](const MII &mp) { return vector_from_idx_map(mp); });
  m.def("enumerate_vector", [](const VI &v) { return enumerate_vector(v); });
  m.def("enumerate", [](const SI &s) { return enumerate(s); });
  m.def("permute_with_key", [](int key, const VI &v) { return permute_with_key(key, v); });
  m.def("get_all_permutations_with_repetition", [](const VI &v, size_t n) { return vector_of(get_all_permutations_with_repetition(v, n)); });
  m.def("binary_cartesian_product", [](const SI &a, const SI &b) { return vector_of(binary_cartesian_product(a, b)); });
  // zips
  m.def("zip_strict", [](const VI &a, const VI &b) { return zip_strict(a, b); });
  m.def("zip_with", [](const VI &a, const VI &b, F2 f) { return zip_with(a, b, f); });
  m.def("zip_with_strict", [](const VI &a, const VI &b, F2 f) { return zip_with_strict(a, b, f); });
  m.def("zip3", [](const VI &a, const VI &b, const VI &c) { return zip3(a, b, c); });
  m.def("zip3_strict", [](const VI &a, const VI &b, const VI &c) { return zip3_strict(a, b, c); });
  m.def("zip3_with", [](const VI &a, const VI &b, const VI &c, std::function<int(int, int, int)> f) { return zip3_with(a, b, c, f); });
  m.def("zip3_with_strict", [](const VI &a, const VI &b, const VI &c, std::function<int(int, int, int)> f) { return zip3_with_strict(a, b, c, f); });
  m.def("zip_values_strict", [](const MSI &a, const MSI &b) { return zip_values_strict(a, b); });
  m.def("zip_values_strict_with", [](const MSI &a, const MSI &b, F2 f) { return zip_values_strict_with(a, b, f); });
  m.def("uncurry", [](F2 f, const std::pair<int, int> &p) { return uncurry(f)(p); });
  // transformations
  m.def("vector_transform", [](const VI &v, F1 f) { return vector_transform(v, f); });
  m.def("filter_idxs", [](const VI &v, std::function<bool(size_t)> p) { return filter_idxs(v, p); });
  m.def("inplace_filter", [](VI v, P1 p) { inplace_filter(v, p); return v; });
  m.def("inplace_filter_set", [](SI s, P1 p) { inplace_filter(s, p); return s; });
  m.def("filtrans", [](const VI &v, FO f) { return filtrans(v, f); });
  m.def("filtrans_set", [](const SI &s, FO f) { return filtrans(s, f); });
  m.def("transform_until", [](const VI &v, FO f) { return transform_until(v, f); });
  m.def("flatmap", [](const VI &v, std::function<VI(int)> f) { return flatmap(v, f); });
  m.def("flatmap_set", [](const SI &s, std::function<SI(int)> f) { return flatmap(s, f); });
  m.def("collapse_optionals", [](const std::optional<OI> &o) { return collapse_optionals(o); });
  m.def("without_nullopts", [](const std::vector<OI> &v) { return without_nullopts(v); });
  m.def("value_all", [](const std::vector<OI> &v) { return value_all(v); });
  m.def("to_uppercase", &to_uppercase);
  // maps
  m.def("values", [](const MSI &mp) { return values(mp); });
  m.def("items", [](const MSI &mp) { return items(mp); });
  m.def("map_from_pairs", [](const std::vector<std::pair<std::string, int>> &ps) { return map_from_pairs(ps); });
  m.def("map_from_keys_and_values", [](const std::vector<std::string> &ks, const VI &vs) { return map_from_keys_and_values(ks, vs); });
  m.def("filter_keys", [](const MII &mp, P1 p) { return filter_keys(mp, p); });
  m.def("filter_values", [](const MII &mp, P1 p) { return filter_values(mp, p); });
  m.def("filtermap_keys", [](const MII &mp, FO f) { return filtermap_keys(mp, f); });
  m.def("filtermap_values", [](const MII &mp, FO f) { return filtermap_values(mp, f); });
  m.def("map_keys", [](const MII &mp, F1 f) { return map_keys(mp, f); });
  m.def("map_keys2", [](const MII &mp, F2 f) { return map_keys2(mp, f); });
  m.def("map_values", [](const MII &mp, F1 f) { return map_values(mp, f); });
  m.def("map_values2", [](const MII &mp, F2 f) { return map_values2(mp, f); });
  m.def("map_keys_and_values", [](const MII &mp, F1 fk, F1 fv) { return map_keys_and_values(mp, fk, fv); });
  m.def("map_keys_with_value_merging", [](const MII &mp, F1 f, F2 merge) { return map_keys_with_value_merging(mp, f, merge); });
  m.def("invert_map", [](const MSI &mp) { return invert_map(mp); });
  m.def("restrict_keys", [](const MSI &mp, const std::set<std::string> &keep) { return restrict_keys(mp, keep); });
  m.def("lift_optional_through_map", [](const std::map<std::string, OI> &mp) { return lift_optional_through_map(mp); });
  m.def("merge_in_map", [](const MSI &src, MSI dst) { merge_in_map(src, dst); return dst; });
  m.def("binary_merge_disjoint_maps", [](const MSI &a, const MSI &b) { return binary_merge_disjoint_maps(a, b); });
  m.def("binary_merge_maps_with_left_dominating", [](const MSI &a, const MSI &b) { return binary_merge_maps_with_left_dominating(a, b); });
  m.def("binary_merge_maps_with_right_dominating", [](const MSI &a, const MSI &b) { return binary_merge_maps_with_right_dominating(a, b); });
  m.def("merge_disjoint_maps", [](const std::vector<MSI> &ms) { return merge_disjoint_maps(ms); });
  m.def("merge_maps_with_right_dominating", [](const std::vector<MSI> &ms) { return merge_maps_with_right_dominating(ms); });
  m.def("try_merge_nondisjoint_maps", [](const MSI &a, const MSI &b) { return try_merge_nondisjoint_maps(a, b); });
  // strings and small value types
  m.def("join_strings", [](const std::vector<std::string> &v, const std::string &d) { return join_strings(v, d); });
  m.def("join_ints", [](const VI &v, const std::string &d) { return join_strings(v, d, [](int x) { return std::to_string(x); }); });
  m.def("indent", &indent, py::arg("text"), py::arg("indent_size") = 2);
  m.def("commutative_pair", [](int a, int b) {
    commutative_pair<int> p(a, b);
    return std::make_pair(p.max(), p.min());
  });
  m.def("commutative_pair_compare", [](int a, int b, int c2, int d) {
    commutative_pair<int> p(a, b), q(c2, d);
    return py::make_tuple(p == q, p != q, p < q);
  });
  m.def("query_set_apply", [](std::optional<SI> allowed, const SI &universe) {
    auto q = allowed ? query_set<int>::match_values_in(*allowed) : query_set<int>::matchall();
    return q.apply(universe);
  }, py::arg("allowed"), py::arg("universe"), "None = match everything");
  m.def("query_set_intersect", [](std::optional<SI> a, std::optional<SI> b) -> std::optional<SI> {
    auto qa = a ? query_set<int>::match_values_in(*a) : query_set<int>::matchall();
    auto qb = b ? query_set<int>::match_values_in(*b) : query_set<int>::matchall();
    auto q = qa.intersect(qb);
    if (q.is_matchall()) return std::nullopt;
    return q.allowed_values();
  });
  m.def("query_set_includes", [](std::optional<SI> a, int v) {
    return (a ? query_set<int>::match_values_in(*a) : query_set<int>::matchall()).includes(v);
  });
  m.def("stack_string_roundtrip", [](const std::string &s2) {
    stack_string<16> t(s2);
    t.push_back('!');
    return py::make_tuple((std::string)t, t.size(), t.length());
  });
  m.def("stack_map_items", [](const std::vector<std::pair<int, int>> &writes) {
    stack_map<int, int, 4> mp;
    for (auto &kv : writes) mp[kv.first] = kv.second;
    return mp.sorted_items();
  });
  m.def("stack_map_at", [](const std::vector<std::pair<int, int>> &writes, int key) {
    stack_map<int, int, 4> mp;
    for (auto &kv : writes) mp.insert(kv.first, kv.second);
    return mp.at(key);
  });
  // sets
  m.def("set_minus", [](const SI &a, const SI &b) { return set_minus(a, b); });
  m.def("set_difference", [](const SI &a, const SI &b) { return set_difference(a, b); });
  m.def("set_intersection", [](const SI &a, const SI &b) { return set_intersection(a, b); });
  m.def("set_intersection_all", [](const std::vector<SI> &sets) { return set_intersection(sets); });
  m.def("set_union_all", [](const std::vector<SI> &sets) { return set_union(sets); });
  m.def("multiset_union", [](const VI &a, const VI &b) { return vector_of(multiset_union(multiset_of(a), multiset_of(b))); });
}

}  // namespace ff
