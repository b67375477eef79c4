"""Allocators (owning, tracked) and tensor accessors with their copy / fill / compare / format helpers and the
naive reference matmul (the reference's lib/kernels/test/src/test_{accessor,copy_tensor_accessor,...}.cc on CPU)."""
import pytest
import torch

from flexflow_train_b200.runtime import allocator as A


def test_owning_and_tracked_allocators():
    with A.LocalCPUAllocator() as cpu:
        tr = A.TrackedAllocator(cpu)
        a = tr.allocate([4, 8], torch.float32)       # 128 bytes
        b = tr([16], torch.bfloat16)                 # 32 bytes, through the call signature task bodies use
        assert (tr.current_bytes, tr.peak_bytes, tr.total_allocated_bytes) == (160, 160, 160) and cpu.num_live == 2
        tr.deallocate(a)
        c = tr.allocate([2], torch.int64)            # 16 bytes
        assert (tr.current_bytes, tr.peak_bytes, tr.total_allocated_bytes) == (48, 160, 176)
        with pytest.raises(ValueError):
            cpu.deallocate(a)                        # already released
        with pytest.raises(ValueError):
            cpu.deallocate(torch.zeros(3))           # never handed out by this allocator
        assert b.dtype == torch.bfloat16 and c.shape == (2,)
    assert cpu.num_live == 0
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            A.LocalCudaAllocator()


def test_accessors_and_helpers():
    cpu = A.LocalCPUAllocator()
    src = A.TensorAccessor(torch.arange(12, dtype=torch.float32).reshape(3, 4))
    assert src.shape == [3, 4] and src.device_type == "CPU" and src.at(2, 1) == 9.0 and src.ptr == src.tensor.data_ptr()
    with pytest.raises(IndexError):
        src.at(1)
    with pytest.raises(PermissionError):
        src.set(1.0, 0, 0)
    cp = A.copy_tensor_accessor(src, cpu)
    assert cp.writable and A.accessors_are_equal(cp, src) and cp.ptr != src.ptr
    cp.set(-1.0, 0, 0)
    assert not A.accessors_are_equal(cp, src) and A.read_only(cp).writable is False
    A.copy_accessor_data_to_l_from_r(cp, src)
    assert A.accessors_are_equal(cp, src)
    with pytest.raises(ValueError):
        A.copy_accessor_data_to_l_from_r(cp, A.TensorAccessor(torch.zeros(4, 3)))
    with pytest.raises(PermissionError):
        A.copy_accessor_data_to_l_from_r(src, cp)
    A.fill_with_zeros(cp)
    assert float(cp.tensor.abs().sum()) == 0.0
    text = A.format_accessor_contents(src, max_elements=3)
    assert text == "<CPU float32 [3, 4]> [0.0, 1.0, 2.0, ... (9 more)]"


def test_reference_matmul_matches_torch():
    torch.manual_seed(0)
    a, b = torch.randn(5, 7), torch.randn(7, 3)
    out = A.tensor_accessor_matmul(A.TensorAccessor(a), A.TensorAccessor(b))
    assert out.shape == [5, 3] and torch.allclose(out.tensor, a @ b, atol=1e-5)
    with pytest.raises(ValueError):
        A.tensor_accessor_matmul(A.TensorAccessor(a), A.TensorAccessor(a))


def test_task_bodies_allocate_through_a_tracked_allocator():
    """A task body's scratch goes through TaskArgumentAccessor.new_tensor; with a tracked allocator behind it the
    executor (and the measured cost estimator) can read the bytes a task took."""
    from flexflow_train_b200.runtime.task_accessor import run_invocations

    tracked = A.TrackedAllocator(A.LocalCPUAllocator())
    inv = [{"task": "FWD", "node": 0, "op_type": "RELU", "name": "r", "inputs": [], "outputs": [], "shard": None, "device": None}]

    def body(acc):
        t = acc.new_tensor([8, 8], torch.float32)
        acc.tensors[(0, "OUTPUT", "FWD", None)] = t.zero_()

    table = run_invocations(inv, {("FWD", "*"): body}, allocate=tracked)
    assert tracked.peak_bytes == 256 and table[(0, "OUTPUT", "FWD", None)].shape == (8, 8)


def test_device_handle_folds_workspace_requests_and_counts_its_bytes():
    # the per-device handle (lib/kernels/include/kernels/ff_handle.h, managed_per_device_ff_handle.h): one workspace sized
    # by the largest request, allocated once through the tracked allocator; the CPU handle has no stream
    from flexflow_train_b200.runtime.device_handle import create_local_handle_for_device
    h = create_local_handle_for_device("cpu", workspace_bytes=64)
    assert not h.is_gpu and not h.stream().is_gpu and h.num_ranks == 1 and h.my_rank == 0
    h.reserve_workspace(1000)
    h.reserve_workspace(10)
    assert h.workspace_bytes == 1000 and h.workspace is None
    before = h.allocator.current_bytes
    ws = h.materialize_workspace()
    assert ws.dtype == torch.float32 and ws.numel() * 4 >= 1000 and h.materialize_workspace() is ws
    assert h.allocator.current_bytes - before == ws.numel() * 4
    h.reserve_workspace(500)       # fits: fine
    with pytest.raises(RuntimeError):
        h.reserve_workspace(1 << 20)   # the workspace is already allocated and too small
    assert "workspace 1000 bytes" in h.describe()


def test_cpu_executable_plans_its_workspace_through_the_handle():
    from flexflow_train_b200 import _ffcore as core
    from flexflow_train_b200.runtime.executor import ExecConfig, Executable
    g = core.build_model("mlp", {"batch_size": 8, "input_dim": 16, "hidden": [32], "num_classes": 4})
    ex = Executable(g, ExecConfig(device="cpu", compute_dtype="fp32"))
    assert ex.handle.allocator is ex.allocator and ex.handle.workspace is ex.scratch_f32() and ex.handle.workspace is not None


# ------------------------------------------------------------------ accessor utilities
# cases after lib/kernels/test/src/kernels/{map_tensor_accessors,compare_tensor_accessors,tensor_accessor_reductions,
# tensor_accessor_unary_ops,reduce_tensor_accessor,create_accessor_with_contents}.cc
def test_create_accessor_with_contents():
    a = A.create_accessor_with_contents([[1, 2, 3], [4, 5, 6]], torch.float32)
    assert a.shape == [2, 3] and a.at(1, 2) == 6.0 and a.writable
    r = A.create_accessor_with_contents([[[1], [2]]], torch.int32, writable=False)
    assert r.shape == [1, 2, 1] and r.dtype == torch.int32 and not r.writable
    alloc = A.TrackedAllocator(A.LocalCPUAllocator())
    A.create_accessor_with_contents([1.0, 2.0], allocator=alloc)
    assert alloc.current_bytes == 8
    with pytest.raises(ValueError):
        A.create_accessor_with_contents([[1, 2], [3]])


def test_map_tensor_accessors():
    a = A.create_accessor_with_contents([[1, 3, 2], [2, 1, 5]], torch.float32)
    assert A.map_tensor_accessor(a, lambda v: v + 1).tensor.tolist() == [[2, 4, 3], [3, 2, 6]]
    assert A.map_tensor_accessor(a, lambda v: v > 2, out_dtype=torch.bool).tensor.tolist() == [[False, True, False], [False, False, True]]
    b = A.create_accessor_with_contents([[0, 2, 5], [3, 3, 8]], torch.float32)
    assert A.map_tensor_accessors2(a, b, lambda x, y: x + 2 * y).tensor.tolist() == [[1, 7, 12], [8, 7, 21]]
    A.map_tensor_accessor_inplace(a, lambda v: v * v)
    assert a.tensor.tolist() == [[1, 9, 4], [4, 1, 25]]
    with pytest.raises(ValueError):
        A.map_tensor_accessors2(a, A.create_accessor_with_contents([1.0]), lambda x, y: x)
    with pytest.raises(PermissionError):
        A.map_tensor_accessor_inplace(A.read_only(a), lambda v: v)


def test_compare_tensor_accessors_and_reductions():
    lhs = A.create_accessor_with_contents([[1, 3, 2], [2, 1, 5]], torch.float32)
    rhs = A.create_accessor_with_contents([[2, 3, 1], [2, 0, 9]], torch.float32)
    assert A.compare_tensor_accessors_lt(lhs, rhs).tensor.tolist() == [[True, False, False], [False, False, True]]
    assert A.compare_tensor_accessors_le(lhs, rhs).tensor.tolist() == [[True, True, False], [True, False, True]]
    assert A.compare_tensor_accessors_gt(lhs, rhs).tensor.tolist() == [[False, False, True], [False, True, False]]
    assert A.compare_tensor_accessors_ge(lhs, rhs).tensor.tolist() == [[False, True, True], [True, True, False]]
    assert A.compare_tensor_accessors_eq(lhs, rhs).tensor.tolist() == [[False, True, False], [True, False, False]]
    ne = A.compare_tensor_accessors_ne(lhs, rhs)
    assert ne.dtype == torch.bool and A.tensor_accessor_any(ne) and not A.tensor_accessor_all(ne)
    assert A.tensor_accessor_all(A.compare_tensor_accessors_eq(lhs, lhs)) and not A.tensor_accessor_any(A.compare_tensor_accessors_ne(lhs, lhs))
    with pytest.raises(TypeError):
        A.tensor_accessor_all(lhs)
    with pytest.raises(ValueError):
        A.compare_tensor_accessors_lt(lhs, A.create_accessor_with_contents([[1, 2, 3]], torch.float32))


def test_tensor_accessor_unary_ops_and_reduce():
    a = A.create_accessor_with_contents([[1, -3, 2], [-2, 1, 5]], torch.float32)
    assert A.tensor_accessor_scale_by_constant(a, 2.0).tensor.tolist() == [[2, -6, 4], [-4, 2, 10]]
    assert A.tensor_accessor_relu(a).tensor.tolist() == [[1, 0, 2], [0, 1, 5]]
    assert A.tensor_accessor_transpose(a).tensor.tolist() == [[1, -2], [-3, 1], [2, 5]]
    assert A.tensor_accessor_broadcast(A.create_accessor_with_contents([[1], [2]], torch.float32), [3, 2, 2]).tensor.tolist() == [[[1, 1], [2, 2]]] * 3
    with pytest.raises(ValueError):
        A.tensor_accessor_broadcast(a, [2, 4])
    assert A.tensor_accessor_reduce(a, 0).tensor.tolist() == [-1, -2, 7] and A.tensor_accessor_reduce(a, 1).tensor.tolist() == [0, 4]
    t = A.create_accessor_with_contents([[[1, 2], [3, 4]], [[5, 6], [7, 8]]], torch.float32)
    assert A.reduce_tensor_accessor_in_dims(t, [0, 2], max).tensor.tolist() == [6, 8]
    assert A.reduce_tensor_accessor_in_dims(t, [1], lambda x, y: x - y).tensor.tolist() == [[-2, -2], [-2, -2]]
    with pytest.raises(ValueError):
        A.reduce_tensor_accessor_in_dims(t, [3], max)
    w = A.create_accessor_with_contents([1.0, 2.0])
    A.tensor_accessor_scale_by_constant_inplace(w, 3.0)
    assert w.tensor.tolist() == [3.0, 6.0]
    with pytest.raises(PermissionError):
        A.tensor_accessor_scale_by_constant_inplace(A.read_only(w), 3.0)
