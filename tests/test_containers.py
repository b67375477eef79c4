"""The functional container helpers of the C++ core (csrc/core/containers.h), one case per helper, through the
`_ffcore.containers` test surface (the reference tests its lib/utils/containers the same way, one file per helper:
lib/utils/test/src/utils/containers/*.cc)."""
import operator

import pytest

from flexflow_train_b200 import _ffcore as core

C = core.containers
even = lambda x: x % 2 == 0  # noqa: E731


def test_predicates():
    assert C.all_of([2, 4], even) and not C.all_of([2, 3], even) and C.all_of([], even)
    assert C.any_of([1, 2], even) and not C.any_of([1, 3], even) and not C.any_of([], even)
    assert C.all_are_true([True, True]) and not C.all_are_true([True, False]) and C.all_are_true([])
    assert C.contains([1, 2, 3], 2) and not C.contains([1, 2, 3], 5)
    assert C.contains_key({"a": 1}, "a") and not C.contains_key({"a": 1}, "b")
    assert C.contains_value({"a": 1}, 1) and not C.contains_value({"a": 1}, 2)
    assert C.are_all_distinct([1, 2, 3]) and not C.are_all_distinct([1, 2, 1])
    assert C.contains_duplicates([1, 1]) and not C.contains_duplicates([])
    assert C.are_all_same([4, 4, 4]) and C.are_all_same([]) and not C.are_all_same([4, 5])
    assert C.are_disjoint({1, 2}, {3}) and not C.are_disjoint({1, 2}, {2, 3})
    assert C.is_superseteq_of({1, 2, 3}, {1, 3}) and not C.is_superseteq_of({1}, {1, 2})
    assert C.is_submapeq_of({"a": 1}, {"a": 1, "b": 2}) and not C.is_submapeq_of({"a": 2}, {"a": 1, "b": 2})
    assert C.is_submapeq_of({}, {"a": 1}) and not C.is_submapeq_of({"c": 1}, {"a": 1})


def test_folds_and_scans():
    sub = operator.sub
    assert C.foldl([1, 2, 3], 10, sub) == ((10 - 1) - 2) - 3
    assert C.foldl1([10, 1, 2], sub) == (10 - 1) - 2
    assert C.foldr([1, 2, 3], 10, sub) == 1 - (2 - (3 - 10))
    assert C.foldr1([1, 2, 10], sub) == (10 - 2) - 1
    assert C.scanl([1, 2, 3, 4], 0, operator.add) == [0, 1, 3, 6, 10]
    assert C.scanl1([1, 2, 3, 4], operator.add) == [1, 3, 6, 10] and C.scanl1([], operator.add) == []
    assert C.scanr([1, 2, 3, 4], 0, operator.add) == [10, 9, 7, 4, 0]
    assert C.scanr([1, 2, 3], 10, sub)[0] == C.foldr([1, 2, 3], 10, sub)
    assert C.scanr1([1, 2, 3, 4], operator.add) == [10, 9, 7, 4] and C.scanr1([], operator.add) == []
    assert C.sum([1, 2, 3]) == 6 and C.sum([]) == 0
    assert C.sum_where([1, 2, 3, 4], even) == 6 and C.product_where([1, 2, 3, 4], even) == 8 and C.product_where([], even) == 1
    assert C.recurse_n(lambda x: x + 3, 3, 5) == 14 and C.recurse_n(lambda x: x + 3, 0, 5) == 5
    with pytest.raises(RuntimeError):
        C.foldl1([], sub)
    with pytest.raises(RuntimeError):
        C.foldr1([], sub)
    with pytest.raises(RuntimeError):
        C.recurse_n(lambda x: x, -1, 0)


def test_selection():
    assert C.minimum([3, 1, 2]) == 1 and C.minimum([]) is None
    assert C.argmax([1, -5, 3], abs) == -5 and C.argmin([4, -1, 1], abs) == -1   # the first of equal keys wins
    assert C.at_idx([7, 8], 1) == 8 and C.try_at_idx([7, 8], 1) == 8 and C.try_at_idx([7, 8], 2) is None
    with pytest.raises(IndexError):
        C.at_idx([7, 8], 2)
    assert C.try_at({"a": 1}, "a") == 1 and C.try_at({"a": 1}, "b") is None
    assert C.lookup_in_map({"a": 1}, "a") == 1
    with pytest.raises(IndexError):
        C.lookup_in_map({"a": 1}, "b")
    assert C.index_of([5, 6, 6], 6) == 1 and C.index_of([5], 7) is None
    assert C.count([1, 2, 4], even) == 2
    assert C.get_one_of({3, 4}) in (3, 4) and C.try_get_one_of(set()) is None
    with pytest.raises(RuntimeError):
        C.get_one_of(set())
    assert C.get_only([9]) == 9 and C.maybe_get_only([9]) == 9 and C.maybe_get_only([9, 9]) is None and C.maybe_get_only([]) is None
    with pytest.raises(RuntimeError):
        C.get_only([1, 2])
    assert C.get_element_counts([1, 2, 1, 1]) == {1: 3, 2: 1}


def test_requirements():
    assert C.require_same(3, 3) == 3
    with pytest.raises(RuntimeError):
        C.require_same(3, 4)
    assert C.require_all_same([2, 2]) == 2 and C.require_all_same([]) is None
    with pytest.raises(RuntimeError):
        C.require_all_same([2, 3])
    assert C.require_all_same1([2, 2]) == 2
    with pytest.raises(RuntimeError):
        C.require_all_same1([])
    assert C.require_no_duplicates([3, 1, 2]) == {1, 2, 3}
    with pytest.raises(RuntimeError):
        C.require_no_duplicates([3, 1, 3])
    assert C.require_only_key({"a": 5}, "a") == 5
    for bad in ({"a": 5, "b": 6}, {"b": 5}, {}):
        with pytest.raises(RuntimeError):
            C.require_only_key(bad, "a")
    assert C.require_two_keys({"a": 1, "b": 2}, "b", "a") == (2, 1)
    for bad, k1, k2 in (({"a": 1, "b": 2, "c": 3}, "a", "b"), ({"a": 1, "b": 2}, "a", "a"), ({"a": 1, "c": 2}, "a", "b")):
        with pytest.raises(RuntimeError):
            C.require_two_keys(bad, k1, k2)


def test_building_sequences():
    assert C.range(0, 5) == [0, 1, 2, 3, 4] and C.range(2, 9, 3) == [2, 5, 8] and C.range(5, 0, -2) == [5, 3, 1] and C.range(3, 3) == []
    with pytest.raises(RuntimeError):
        C.range(0, 1, 0)
    it = iter([7, 8, 9])
    assert C.repeat(3, lambda: next(it)) == [7, 8, 9]
    assert C.repeat_element(3, 4) == [4, 4, 4] and C.repeat_element(0, 4) == []
    assert C.counter_values(5, 3) == [5, 6, 7]
    assert C.generate_vector(4, lambda i: i * i) == [0, 1, 4, 9]
    assert C.generate_map([1, 2, 3], lambda k: k * 10) == {1: 10, 2: 20, 3: 30}
    with pytest.raises(RuntimeError):
        C.generate_map([1, 1], lambda k: k)
    assert C.vector_of({3, 1, 2}) == [1, 2, 3] and C.set_of([1, 1, 2]) == {1, 2} and C.multiset_of([2, 1, 2]) == [1, 2, 2]
    assert C.sorted([3, 1, 2]) == [1, 2, 3]
    assert C.sorted_by_key([3, -1, -2, 1], abs) == [-1, 1, -2, 3]   # stable
    assert C.reversed([1, 2, 3]) == [3, 2, 1]
    assert C.concat_vectors([1], [2, 3]) == [1, 2, 3] and C.concat_all([[1], [], [2, 3]]) == [1, 2, 3]
    assert C.extend([1], {3, 2}) == [1, 2, 3]
    assert C.enumerate_vector([7, 8]) == {0: 7, 1: 8} and C.enumerate({5, 3}) == {0: 3, 1: 5}
    assert C.vector_from_idx_map({0: 7, 1: 8}) == [7, 8] and C.vector_from_idx_map({0: 7, 2: 8}) is None and C.vector_from_idx_map({}) == []


@pytest.mark.parametrize("start,end", [(0, None), (1, 3), (-2, None), (0, -1), (2, 2), (3, 1), (4, None), (-4, 4)])
def test_slice_follows_python(start, end):
    v = [10, 11, 12, 13]
    assert C.slice(v, start, end) == v[start:end]


def test_slice_and_split_reject_positions_outside_the_vector():
    for start, end in ((5, None), (-5, None), (0, 5), (0, -5)):
        with pytest.raises(IndexError):
            C.slice([1, 2, 3, 4], start, end)
    assert C.vector_split([1, 2, 3], 1) == ([1], [2, 3]) and C.vector_split([1, 2], 0) == ([], [1, 2]) and C.vector_split([1, 2], 2) == ([1, 2], [])
    for i in (-1, 3):
        with pytest.raises(IndexError):
            C.vector_split([1, 2], i)


def test_permutations_and_products():
    import itertools
    v = [4, 5, 6]
    perms = [list(p) for p in itertools.permutations(v)]
    for key in range(6):
        assert C.permute_with_key(key, v) == perms[key]
    assert C.permute_with_key(6, v) == perms[0]       # wraps around after the last permutation
    got = C.get_all_permutations_with_repetition([1, 2, 3], 2)
    assert sorted(got) == sorted(list(p) for p in itertools.product([1, 2, 3], repeat=2))
    assert C.get_all_permutations_with_repetition([1, 1], 2) == [[1, 1]] * 4     # a multiset: repeats are kept
    assert C.get_all_permutations_with_repetition([], 2) == [[]] and C.get_all_permutations_with_repetition([1], 0) == [[]]
    assert sorted(C.binary_cartesian_product({1, 2}, {3, 4})) == [(1, 3), (1, 4), (2, 3), (2, 4)]
    assert C.binary_cartesian_product(set(), {1}) == []


def test_zips():
    add = operator.add
    assert C.zip_strict([1, 2], [3, 4]) == [(1, 3), (2, 4)]
    with pytest.raises(RuntimeError):
        C.zip_strict([1], [3, 4])
    assert C.zip_with([1, 2, 3], [10, 20], add) == [11, 22]
    assert C.zip_with_strict([1, 2], [10, 20], add) == [11, 22]
    with pytest.raises(RuntimeError):
        C.zip_with_strict([1, 2, 3], [10, 20], add)
    assert C.zip3([1, 2], [3, 4, 5], [6, 7]) == [(1, 3, 6), (2, 4, 7)]
    assert C.zip3_strict([1], [2], [3]) == [(1, 2, 3)]
    with pytest.raises(RuntimeError):
        C.zip3_strict([1], [2, 2], [3])
    f3 = lambda a, b, c: a * b + c  # noqa: E731
    assert C.zip3_with([1, 2], [3, 4], [5, 6, 7], f3) == [8, 14] and C.zip3_with_strict([1], [2], [3], f3) == [5]
    with pytest.raises(RuntimeError):
        C.zip3_with_strict([1], [2], [3, 4], f3)
    assert C.zip_values_strict({"a": 1, "b": 2}, {"b": 20, "a": 10}) == {"a": (1, 10), "b": (2, 20)}
    assert C.zip_values_strict_with({"a": 1}, {"a": 10}, add) == {"a": 11}
    with pytest.raises(RuntimeError):
        C.zip_values_strict({"a": 1}, {"b": 1})
    assert C.uncurry(operator.sub, (5, 3)) == 2


def test_transformations():
    half = lambda x: x // 2 if x % 2 == 0 else None  # noqa: E731
    assert C.vector_transform([1, 2], lambda x: x + 1) == [2, 3]
    assert C.filter_idxs([5, 6, 7, 8], lambda i: i % 2 == 1) == [6, 8]
    assert C.inplace_filter([1, 2, 3, 4], even) == [2, 4] and C.inplace_filter_set({1, 2, 3, 4}, even) == {2, 4}
    assert C.filtrans([1, 2, 3, 4], half) == [1, 2] and C.filtrans_set({2, 4, 5}, half) == {1, 2}
    assert C.transform_until([2, 4, 5, 6], half) == [1, 2] and C.transform_until([1, 2], half) == []
    assert C.flatmap([1, 2], lambda x: [x] * x) == [1, 2, 2] and C.flatmap_set({1, 2}, lambda x: {x, x + 1}) == {1, 2, 3}
    assert C.collapse_optionals(None) is None and C.collapse_optionals(3) == 3
    assert C.without_nullopts([1, None, 3]) == [1, 3]
    assert C.value_all([1, 2]) == [1, 2]
    with pytest.raises(RuntimeError):
        C.value_all([1, None])
    assert C.to_uppercase("gelu_fast1") == "GELU_FAST1"


def test_maps():
    m = {1: 10, 2: 20, 3: 30}
    assert C.values({"b": 2, "a": 2}) == [2, 2] and C.items({"b": 2, "a": 1}) == [("a", 1), ("b", 2)]
    assert C.map_from_pairs([("a", 1), ("b", 2)]) == {"a": 1, "b": 2}
    with pytest.raises(RuntimeError):
        C.map_from_pairs([("a", 1), ("a", 2)])
    assert C.map_from_keys_and_values(["a", "b"], [1, 2]) == {"a": 1, "b": 2}
    with pytest.raises(RuntimeError):
        C.map_from_keys_and_values(["a"], [1, 2])
    assert C.filter_keys(m, even) == {2: 20} and C.filter_values(m, lambda v: v > 10) == {2: 20, 3: 30}
    half = lambda x: x // 2 if x % 2 == 0 else None  # noqa: E731
    assert C.filtermap_keys(m, half) == {1: 20} and C.filtermap_values(m, half) == {1: 5, 2: 10, 3: 15}
    assert C.map_keys(m, lambda k: k + 1) == {2: 10, 3: 20, 4: 30}
    with pytest.raises(RuntimeError):
        C.map_keys(m, lambda k: 0)
    assert C.map_keys2(m, lambda k, v: k + v) == {11: 10, 22: 20, 33: 30}
    assert C.map_values(m, lambda v: v + 1) == {1: 11, 2: 21, 3: 31}
    assert C.map_values2(m, lambda k, v: k * v) == {1: 10, 2: 40, 3: 90}
    assert C.map_keys_and_values(m, lambda k: -k, lambda v: v // 10) == {-1: 1, -2: 2, -3: 3}
    assert C.map_keys_with_value_merging(m, lambda k: k % 2, operator.add) == {1: 40, 0: 20}
    assert C.invert_map({"a": 1, "b": 1, "c": 2}) == {1: {"a", "b"}, 2: {"c"}}
    assert C.restrict_keys({"a": 1, "b": 2}, {"b", "z"}) == {"b": 2}
    assert C.lift_optional_through_map({"a": 1, "b": 2}) == {"a": 1, "b": 2} and C.lift_optional_through_map({"a": None, "b": None}) is None
    for bad in ({"a": 1, "b": None}, {}):
        with pytest.raises(RuntimeError):
            C.lift_optional_through_map(bad)


def test_map_merging():
    a, b = {"x": 1, "y": 2}, {"y": 3, "z": 4}
    assert C.merge_in_map(a, b) == {"x": 1, "y": 2, "z": 4}          # the source's entries win
    assert C.binary_merge_disjoint_maps({"x": 1}, {"z": 4}) == {"x": 1, "z": 4}
    with pytest.raises(RuntimeError):
        C.binary_merge_disjoint_maps(a, b)
    assert C.binary_merge_maps_with_left_dominating(a, b) == {"x": 1, "y": 2, "z": 4}
    assert C.binary_merge_maps_with_right_dominating(a, b) == {"x": 1, "y": 3, "z": 4}
    assert C.merge_disjoint_maps([{"a": 1}, {"b": 2}, {"c": 3}]) == {"a": 1, "b": 2, "c": 3} and C.merge_disjoint_maps([]) == {}
    with pytest.raises(RuntimeError):
        C.merge_disjoint_maps([{"a": 1}, {"b": 2}, {"a": 3}])
    assert C.merge_maps_with_right_dominating([{"a": 1}, {"a": 2, "b": 2}, {"b": 3}]) == {"a": 2, "b": 3}
    assert C.try_merge_nondisjoint_maps({"x": 1, "y": 2}, {"y": 2, "z": 4}) == {"x": 1, "y": 2, "z": 4}
    assert C.try_merge_nondisjoint_maps(a, b) is None


def test_sets():
    assert C.set_minus({1, 2, 3}, {2}) == {1, 3} and C.set_difference({1, 2}, {1, 2}) == set()
    assert C.set_intersection({1, 2, 3}, {2, 3, 4}) == {2, 3}
    assert C.set_intersection_all([{1, 2, 3}, {2, 3}, {3, 4}]) == {3} and C.set_intersection_all([]) is None
    assert C.set_union_all([{1}, {2}, {1, 3}]) == {1, 2, 3} and C.set_union_all([]) == set()
    assert C.multiset_union([1, 2, 2], [2, 3]) == [1, 2, 2, 2, 3]


# ------------------------------------------------------------------ properties against Python's own containers
from hypothesis import given, settings, strategies as st  # noqa: E402

ints = st.lists(st.integers(-50, 50), max_size=12)
small_sets = st.sets(st.integers(0, 15), max_size=8)


@settings(max_examples=150, deadline=None)
@given(ints, st.integers(-12, 12), st.one_of(st.none(), st.integers(-12, 12)))
def test_slice_property(v, start, end):
    inside = lambda i: -len(v) <= i <= len(v)  # noqa: E731
    if inside(start) and (end is None or inside(end)):
        assert C.slice(v, start, end) == v[start:end]
    else:
        with pytest.raises(IndexError):
            C.slice(v, start, end)


@settings(max_examples=100, deadline=None)
@given(ints, st.integers(-5, 5))
def test_scans_end_in_their_folds(v, init):
    f = lambda a, b: 2 * a - b  # noqa: E731   neither commutative nor associative
    assert C.scanl(v, init, f)[-1] == C.foldl(v, init, f) and len(C.scanl(v, init, f)) == len(v) + 1
    assert C.scanr(v, init, f)[0] == C.foldr(v, init, f) and C.scanr(v, init, f)[-1] == init
    if v:
        assert C.scanl1(v, f)[-1] == C.foldl1(v, f) and C.scanr1(v, f)[-1] == v[-1]
        assert C.foldr(v[:-1], v[-1], f) == C.scanr1(v, f)[0]


@settings(max_examples=100, deadline=None)
@given(small_sets, small_sets, small_sets)
def test_set_algebra_matches_python(a, b, c):
    assert C.set_minus(a, b) == a - b and C.set_intersection(a, b) == a & b
    assert C.set_union_all([a, b, c]) == a | b | c and C.set_intersection_all([a, b, c]) == a & b & c
    assert C.are_disjoint(a, b) == a.isdisjoint(b) and C.is_superseteq_of(a, b) == (a >= b)
    assert sorted(C.binary_cartesian_product(a, b)) == sorted((x, y) for x in a for y in b)


@settings(max_examples=100, deadline=None)
@given(st.dictionaries(st.sampled_from("abcdef"), st.integers(0, 3), max_size=5), st.dictionaries(st.sampled_from("abcdef"), st.integers(0, 3), max_size=5))
def test_map_merges_match_python(a, b):
    assert C.binary_merge_maps_with_right_dominating(a, b) == {**a, **b}
    assert C.binary_merge_maps_with_left_dominating(a, b) == {**b, **a}
    agree = all(a[k] == b[k] for k in a.keys() & b.keys())
    assert C.try_merge_nondisjoint_maps(a, b) == ({**a, **b} if agree else None)
    assert C.is_submapeq_of(a, {**b, **a}) and C.is_submapeq_of(a, b) == all(k in b and b[k] == v for k, v in a.items())
    inv = C.invert_map(a)
    assert sorted(k for ks in inv.values() for k in ks) == sorted(a) and all(a[k] == v for v, ks in inv.items() for k in ks)


# ------------------------------------------------------------------ strings and small value types
def test_join_strings_and_indent():
    assert C.join_strings(["a", "b", "c"], ", ") == "a, b, c" and C.join_strings([], ", ") == "" and C.join_strings(["x"], "-") == "x"
    assert C.join_ints([1, 2, 3], "x") == "1x2x3"
    # the reference's cases (lib/utils/test/src/utils/indent.cc)
    assert C.indent("") == "  "
    assert C.indent("hello world") == "  hello world"
    assert C.indent("\na b\nc d\ne f\ng\n") == "  \n  a b\n  c d\n  e f\n  g\n  "
    assert C.indent("   a b  \nc   d e\n     ") == "     a b  \n  c   d e\n       "
    assert C.indent("a\nb", 4) == "    a\n    b"


def test_commutative_pair():
    assert C.commutative_pair(1, 2) == (2, 1) == C.commutative_pair(2, 1)
    assert C.commutative_pair_compare(1, 2, 2, 1) == (True, False, False)
    assert C.commutative_pair_compare(1, 2, 1, 3) == (False, True, True)      # ordered by (max, min)
    assert C.commutative_pair_compare(1, 3, 2, 2) == (False, True, False)


@settings(max_examples=100, deadline=None)
@given(st.integers(-20, 20), st.integers(-20, 20), st.integers(-20, 20), st.integers(-20, 20))
def test_commutative_pair_properties(a, b, c2, d):
    hi, lo = C.commutative_pair(a, b)
    assert hi >= lo and {hi, lo} == {a, b}
    eq, ne, lt = C.commutative_pair_compare(a, b, c2, d)
    assert eq == (sorted((a, b)) == sorted((c2, d))) and ne == (not eq)
    assert lt == ((max(a, b), min(a, b)) < (max(c2, d), min(c2, d)))
    assert C.commutative_pair_compare(a, b, b, a) == (True, False, False)


def test_query_set():
    universe = {1, 2, 3, 4}
    assert C.query_set_apply(None, universe) == universe                   # match-all
    assert C.query_set_apply(set(), universe) == set()                     # match-none
    assert C.query_set_apply({2, 9}, universe) == {2}
    assert C.query_set_includes(None, 7) and C.query_set_includes({7}, 7) and not C.query_set_includes({1}, 7)
    assert C.query_set_intersect(None, None) is None
    assert C.query_set_intersect(None, {1, 2}) == {1, 2} == C.query_set_intersect({1, 2}, None)
    assert C.query_set_intersect({1, 2}, {2, 3}) == {2}


def test_stack_string_and_stack_map():
    assert C.stack_string_roundtrip("Hello") == ("Hello!", 6, 6) and C.stack_string_roundtrip("") == ("!", 1, 1)
    with pytest.raises(Exception):
        C.stack_string_roundtrip("x" * 16)                                  # capacity 16, one more character is pushed
    assert C.stack_map_items([(2, 20), (1, 10), (2, 21)]) == [(1, 10), (2, 21)]
    assert C.stack_map_at([(1, 10), (2, 20)], 2) == 20
    with pytest.raises(IndexError):
        C.stack_map_at([(1, 10)], 3)
    with pytest.raises(Exception):
        C.stack_map_items([(i, i) for i in range(5)])                       # capacity 4
