"""The allocation-free permutation plan (dice_permute_plan_static).

Some hosts of this library cannot allocate device memory while they run (a
serving loop with a memory pool frozen at start-up, a plug-in that only gets
its caller's buffers, an application with a hard memory budget), so they
cannot provide the scratch buffer that dice_permute_plan asks for.  This entry point keeps that scratch in a fixed
array inside the library.  The test calls it through the C ABI, twice in a row
on different inputs (the array is shared and keeps the previous call's
contents), and requires the very same outputs as the scratch-taking entry
point: the work is integer-only, so equality is exact.

Collected last on purpose: a failure here must not hide any other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(lib, flat, n_experts, dev):
    n = flat.numel()
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    for static in (False, True):
        pos = torch.full((max(n, 1),), -7, dtype=torch.int32, device=dev)
        order = torch.full((max(n, 1),), -7, dtype=torch.int32, device=dev)
        seg = torch.full((n_experts + 1,), -7, dtype=torch.int32, device=dev)
        if static:
            rc = lib.dice_permute_plan_static(flat.data_ptr(), n, n_experts, pos.data_ptr(), order.data_ptr(),
                                              seg.data_ptr(), stream)
        else:
            nbytes = lib.dice_permute_scratch_bytes(n, n_experts)
            scratch = torch.empty(max(nbytes // 4, 1), dtype=torch.int32, device=dev)
            rc = lib.dice_permute_plan(flat.data_ptr(), n, n_experts, scratch.data_ptr(), scratch.numel() * 4,
                                       pos.data_ptr(), order.data_ptr(), seg.data_ptr(), stream)
        assert rc == 0, lib.dice_strerror(rc)
        torch.cuda.synchronize()
        outs.append((pos[:n].cpu(), order[:n].cpu(), seg.cpu()))
    return outs


def test_static_plan_equals_scratch_plan_on_two_calls_in_a_row(cuda_device):
    from dice_b200 import _lib

    lib = _lib.load()
    g = torch.Generator().manual_seed(2024)
    # second call is smaller and uses other experts: stale cells of the first call stay in the array
    cases = [(40000, 16), (777, 8)]
    for n_rows, n_experts in cases:
        flat = torch.randint(0, n_experts, (n_rows,), generator=g).to(cuda_device)
        (pos_a, order_a, seg_a), (pos_b, order_b, seg_b) = _both(lib, flat, n_experts, cuda_device)
        assert torch.equal(pos_a, pos_b)
        assert torch.equal(order_a, order_b)
        assert torch.equal(seg_a, seg_b)
        # and both are the stable sort by expert
        want = flat.cpu().argsort(stable=True).to(torch.int32)
        assert torch.equal(order_b, want)
        assert int(seg_b[-1]) == n_rows


def test_static_plan_rejects_sizes_beyond_its_array(cuda_device):
    from dice_b200 import _lib

    lib = _lib.load()
    n_experts = 64
    too_many = (65536 // n_experts) * 256 + 1  # one chunk more than the array holds
    flat = torch.zeros(8, dtype=torch.int64, device=cuda_device)  # never read: the call must refuse first
    seg = torch.full((n_experts + 1,), -7, dtype=torch.int32, device=cuda_device)
    pos = torch.zeros(8, dtype=torch.int32, device=cuda_device)
    rc = lib.dice_permute_plan_static(flat.data_ptr(), too_many, n_experts, pos.data_ptr(), None, seg.data_ptr(),
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == -7 and b"maximum" in lib.dice_strerror(rc)
    torch.cuda.synchronize()
    assert bool((seg == -7).all())  # nothing was enqueued
    # the largest admissible size is accepted
    ok_rows = (65536 // n_experts) * 256
    flat = torch.randint(0, n_experts, (ok_rows,), device=cuda_device)
    pos = torch.empty(ok_rows, dtype=torch.int32, device=cuda_device)
    rc = lib.dice_permute_plan_static(flat.data_ptr(), ok_rows, n_experts, pos.data_ptr(), None, seg.data_ptr(),
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(seg[-1]) == ok_rows


def test_static_plan_allocates_nothing(cuda_device):
    """A warm call leaves the device's free memory and torch's allocator untouched: the scratch is the
    library's own fixed array, not something obtained per call."""
    from dice_b200 import _lib

    lib = _lib.load()
    n_rows, n_experts = 5000, 8
    flat = torch.randint(0, n_experts, (n_rows,), device=cuda_device)
    pos = torch.empty(n_rows, dtype=torch.int32, device=cuda_device)
    seg = torch.empty(n_experts + 1, dtype=torch.int32, device=cuda_device)
    stream = torch.cuda.current_stream().cuda_stream
    call = lambda: lib.dice_permute_plan_static(flat.data_ptr(), n_rows, n_experts, pos.data_ptr(), None, seg.data_ptr(), stream)
    assert call() == 0  # the first call on a device looks the array's address up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(cuda_device)
    torch_before = (torch.cuda.memory_allocated(cuda_device), torch.cuda.memory_reserved(cuda_device))
    for _ in range(3):
        assert call() == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(cuda_device)
    assert free_after >= free_before  # nothing was taken from the device
    assert (torch.cuda.memory_allocated(cuda_device), torch.cuda.memory_reserved(cuda_device)) == torch_before
    assert int(seg[-1]) == n_rows
