"""Reader / writer dependency tracking over lowered training steps."""
from flexflow_train_b200 import _ffcore as core
from flexflow_train_b200.runtime import dependency as D
from flexflow_train_b200.runtime import lowering as L


def test_dependency_set_rules():
    ds = D.DependencySet()
    assert ds.add_writer("x", 0) == set()
    assert ds.add_reader("x", 1) == {0} and ds.add_reader("x", 2) == {0}      # read after write
    assert ds.add_writer("x", 3) == {0, 1, 2}                                  # write after read and after write
    assert ds.add_reader("x", 4) == {3}                                        # earlier readers are forgotten
    assert ds.add_writer("y", 5) == set() and ds.add_writer("y", 6) == {5}     # write after write


def _branches(n=3):
    b = core.GraphBuilder()
    x = b.create_input([8, 16], name="x")
    outs = [b.dense(x, 16, activation="RELU", name=f"branch{i}") for i in range(n)]
    t = outs[0]
    for o in outs[1:]:
        t = b.binary("EW_ADD", t, o)
    b.softmax(b.dense(t, 4, name="head"), name="prob")
    return b.graph


def test_lowered_step_order_is_valid_and_branches_share_a_level():
    g = _branches(3)
    inv = L.lower(g, optimizer={"kind": "sgd"})
    assert D.check_order(inv, range(len(inv))) == []
    # running everything backwards violates dependencies
    assert len(D.check_order(inv, reversed(range(len(inv))))) > 0
    deps = D.dependency_graph(inv)
    by = {(i["task"], i["name"]): k for k, i in enumerate(inv)}
    fwd_head, bwd_head = by[("FWD", "head")], by[("BWD", "head")]
    assert by[("FWD", "branch0")] in _closure(deps, fwd_head) and fwd_head in _closure(deps, bwd_head)
    upd = [k for k, i in enumerate(inv) if i["task"] == "UPD"]
    assert upd and all(any(inv[j]["task"] == "BWD" for j in deps[u]) for u in upd)   # an update waits for its gradient
    levels = D.schedule_levels(inv)
    where = {k: l for l, members in enumerate(levels) for k in members}
    assert len({where[by[("FWD", f"branch{i}")]] for i in range(3)}) == 1            # independent branches: one level
    assert len(levels) < len(inv)                                                    # so the step has parallel slack
    for l, members in enumerate(levels):
        for k in members:
            assert all(where[j] < l for j in deps[k])


def _closure(deps, i):
    seen, stack = set(), [i]
    while stack:
        for j in deps[stack.pop()]:
            if j not in seen:
                seen.add(j)
                stack.append(j)
    return seen
