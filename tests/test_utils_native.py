"""The support types of the C++ core (csrc/core/utils.h) through their Python surface: restricted integers and
units, container helpers, restricted maps, union-find, the deduplicating priority queue, stack_vector, the full
binary tree with paths, the orthotope index-space algebra, undirected / multi graphs and the dot formatters.
The reference tests the same families in lib/utils/test/src/utils/**."""
import itertools

import pytest

from flexflow_train_b200 import _ffcore as core

U = core.utils


def test_restricted_integers_and_units():
    assert U.nonnegative(0) == 0 and U.positive(3) == 3 and U.ge_two(2) == 2
    for fn, bad in ((U.nonnegative, -1), (U.positive, 0), (U.ge_two, 1)):
        with pytest.raises(ValueError):
            fn(bad)
    assert U.positive_mul(6, 7) == 42 and U.positive_add(2, 3) == 5
    with pytest.raises(OverflowError):
        U.positive_mul(2 ** 62, 4)
    with pytest.raises(OverflowError):
        U.positive_add(2 ** 63 - 1, 1)
    assert U.ceildiv(10, 4) == 3 and U.ceildiv(8, 4) == 2
    assert U.transfer_ms(770e9, 770e9) == pytest.approx(1000.0)   # 770 GB at 770 GB/s
    with pytest.raises(ValueError):
        U.transfer_ms(1.0, 0.0)
    with pytest.raises(ValueError):
        U.transfer_ms(-1.0, 1.0)
    assert U.max_ms(1.5, 0.5) == 1.5


def test_container_helpers():
    assert U.cartesian_product([[1, 2], [3], [4, 5]]) == [list(t) for t in itertools.product([1, 2], [3], [4, 5])]
    assert U.cartesian_product([]) == [[]]
    a = U.get_all_assignments({1: [10, 11], 2: [20], 3: [30, 31]})
    assert len(a) == 4 and {1: 11, 2: 20, 3: 30} in a
    assert U.merge_maps_sum({"a": 1, "b": 2}, {"b": 5, "c": 7}) == {"a": 1, "b": 7, "c": 7}
    assert U.group_by_mod([1, 2, 3, 4, 5, 6, 7], 3) == {0: [3, 6], 1: [1, 4, 7], 2: [2, 5]}
    assert U.get_all_permutations([3, 1, 2]) == [list(p) for p in itertools.permutations([1, 2, 3])]
    assert U.transform_square([1, 2, 3]) == [1, 4, 9] and U.filter_even({1, 2, 3, 4}) == {2, 4}
    assert U.zip([1, 2, 3], ["a", "b"]) == [(1, "a"), (2, "b")]
    assert U.set_ops({1, 2}, {2, 3}) == ({1, 2, 3}, {2}, False) and U.set_ops({2}, {2, 3})[2]
    assert U.product([2, 3, 4]) == 24 and U.maximum([3, 9, 1]) == 9 and U.maximum([]) is None
    assert U.flatmap_concat([[1], [], [2, 3]]) == [1, 2, 3]


def test_restricted_maps():
    fwd, bwd = U.bidict([(1, "a"), (2, "b"), (3, "a")])   # re-using "a" evicts 1
    assert fwd == {2: "b", 3: "a"} and bwd == {"a": 3, "b": 2}
    assert U.relational_join([(1, "x"), (2, "y")], [("x", 10), ("y", 20)]) == {1: 10, 2: 20}
    with pytest.raises(ValueError):
        U.relational_join([(1, "x")], [("x", 10), ("y", 20)])
    assert U.one_to_many([(1, 10), (1, 11), (2, 20)]) == {1: {10, 11}, 2: {20}}
    with pytest.raises(ValueError):
        U.one_to_many([(1, 10), (2, 10)])              # a right value cannot have two owners
    assert U.many_to_one([(1, 7), (2, 7), (3, 8)], 7) == {1, 2}


def test_union_find_queue_and_stack_vector():
    groups = U.union_find_groups([(1, 2), (3, 4), (2, 3), (5, 5), (6, 7)])
    assert sorted(sorted(g) for g in groups) == [[1, 2, 3, 4], [5], [6, 7]]
    accepted, order = U.dedup_queue_order([5, 1, 5, 9, 1, 3])
    assert accepted == 4 and order == [9, 5, 3, 1]
    assert U.stack_vector_fill(8) == (8, 28)
    with pytest.raises(ValueError):
        U.stack_vector_fill(9)


def test_full_binary_tree_paths():
    tree = ("series", ("parallel", 1, 2), ("series", 3, ("parallel", 4, 5)))
    n, leaves, paths = U.tree_info(tree)
    assert n == 9 and leaves == [1, 2, 3, 4, 5] and paths == ["LL", "LR", "RL", "RRL", "RRR"]
    assert U.tree_leaves_at(tree, "RR") == [4, 5] and U.tree_leaves_at(tree, "") == leaves
    assert U.tree_leaves_at(tree, "LLL") is None
    with pytest.raises(ValueError):
        U.tree_info(("only", 1))


def test_orthotope_algebra():
    dims = [2, 3, 4]
    assert U.orthotope_volume(dims) == 24 and U.orthotope_minimal([1, 4, 1, 2]) == [4, 2]
    for f in range(24):
        c = U.orthotope_unflatten(dims, f)
        assert U.orthotope_flatten(dims, c) == f
    assert U.orthotope_flatten(dims, [1, 2, 3]) == 23
    with pytest.raises(IndexError):
        U.orthotope_flatten(dims, [2, 0, 0])
    with pytest.raises(IndexError):
        U.orthotope_unflatten(dims, 24)
    # task space (2, 3, 4) onto a tensor whose dim 0 is sharded by task dims 0 and 1 together and dim 1 by task dim 2
    groups = [[0, 1], [2]]
    assert U.project_domain(dims, groups) == [6, 4] and U.projection_is_bijection(dims, groups)
    seen = set()
    for f in range(24):
        c = U.orthotope_unflatten(dims, f)
        p = U.project_coord(dims, groups, c)
        assert U.lift_coord(dims, groups, p) == c
        seen.add(tuple(p))
    assert len(seen) == 24
    # dropping a task dim (replication over it) is not a bijection; lifting fills the dropped dim with 0
    assert not U.projection_is_bijection(dims, [[0], [2]])
    assert U.project_coord(dims, [[0], [2]], [1, 2, 3]) == [1, 3] and U.lift_coord(dims, [[0], [2]], [1, 3]) == [1, 0, 3]
    assert U.projection_is_bijection([2, 1, 4], [[0], [2]])        # a dropped dim of extent 1 loses nothing
    assert not U.projection_is_bijection(dims, [[0, 1], [1]])      # a task dim used twice


def test_graph_variants_and_formatters():
    comps, edges = U.connected_components([1, 2, 3, 4, 5], [(1, 2), (2, 3), (4, 5), (2, 1)])
    assert sorted(sorted(c) for c in comps) == [[1, 2, 3], [4, 5]] and edges == 3
    nodes, between, left, out_a, in_b = U.multidigraph_counts([(1, 2), (1, 2), (2, 3), (1, 3)], 1, 2)
    assert (nodes, between, left) == (3, 2, 3) and out_a == 2 and in_b == 1   # one of the parallel 1->2 edges was removed
    dot = U.dot_text(["a", 'b"q'], [("a", 'b"q')])
    assert dot.startswith("digraph g {") and "subgraph cluster_0" in dot and '"a" -> "b\\"q";' in dot and 'shape="record"' in dot
    assert U.record_text(["op", "x|y"], ["in", "out"]) == "{op|x\\|y|{in|out}}"


@pytest.mark.parametrize("ranks", [2, 4])
def test_flag_protocol_with_threads_as_ranks(ranks):
    """The epoch-flag protocol of the peer-memory kernels on host threads: publish, barrier, read, barrier for many
    epochs without ever resetting a flag; every rank sees every peer's value of the same epoch."""
    epochs = 300
    res = U.flag_protocol_rounds(ranks, epochs)
    want = sum(e * 1000 + p for e in range(1, epochs + 1) for p in range(ranks))
    for r in res:
        assert r["ok"] and r["epochs_done"] == epochs and r["checksum"] == want, r


def test_flag_protocol_bounded_wait_reports_a_silent_rank():
    """A rank that stops signalling (it left between steps) costs its peers one bounded wait; each reports who it
    waited for, the epoch it expected and the epoch it saw, and nobody spins on."""
    res = U.flag_protocol_rounds(3, 50, silent_rank=1, silent_after=7, limit_ms=300)
    assert res[1]["ok"] and res[1]["epochs_done"] == 7
    for r in (res[0], res[2]):
        assert not r["ok"] and r["epochs_done"] == 7
        assert (r["peer"], r["expected"], r["seen"]) == (1, 8, 7)
        assert 0.25 < r["seconds"] < 5.0
