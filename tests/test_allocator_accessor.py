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
