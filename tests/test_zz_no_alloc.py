"""The allocation-free AllReduce entry point, called through its exported C symbol.

Some callers of this library may not allocate device memory at all (code under an allocator lock,
processes whose memory belongs to a pool they cannot bypass, threads that are capturing a CUDA
graph).  `nano_nccl_all_reduce_local_noalloc` serves them with scratch memory that is part of the
library image.  This test checks it against the regular, allocating emulation entry point
(`nano_nccl_emu_all_reduce`) on two calls in a row: the second call reuses the scratch array with
the first call's leftovers in it.  The file name sorts last so that a failure here cannot hide
failures elsewhere when a run stops at the first error.
"""
import ctypes as C

import pytest
import torch

from nano_nccl_b200 import _native as N

pytestmark = pytest.mark.gpu

DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
TOL = {torch.float32: 1e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}


def _noalloc():
    lib = N.load_library()
    fn = lib.nano_nccl_all_reduce_local_noalloc
    fn.restype = C.c_int32
    fn.argtypes = [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int, C.c_size_t, C.c_int32, C.c_int32, C.c_void_p]
    return lib, fn


def _ptrs(ts):
    return (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])


def test_noalloc_matches_allocating_entry_point_twice_in_a_row():
    lib, fn = _noalloc()
    stream = torch.cuda.current_stream().cuda_stream
    emu = C.c_void_p()
    N.check(lib.nano_nccl_emu_create(torch.cuda.current_device(), 4, 5_000_000, C.byref(emu)))
    try:
        # call 1: bf16 sum, a size that needs several tiles; call 2: fp32 max with another size,
        # straight after, on the scratch that call 1 left behind
        # call 3 repeats call 2's variant: by then the driver has loaded that kernel, so the free device memory
        # must not move at all across the call (this also sees allocations that bypass torch's allocator)
        status_fn = lib.nano_nccl_all_reduce_local_noalloc_status
        status_fn.restype = C.c_int32
        status_fn.argtypes = [C.c_void_p, C.POINTER(C.c_uint32)]
        for call, (dtype, op, count, nranks) in enumerate([(torch.bfloat16, "sum", 300_003, 4),
                                                           (torch.float32, "max", 70_001, 4),
                                                           (torch.float32, "max", 65_537, 4)]):
            g = torch.Generator().manual_seed(17 + call)
            xs = [(torch.rand(count, generator=g) * 2 - 1).to(dtype).cuda() for _ in range(nranks)]
            got = [torch.full((count,), -9137.25, dtype=dtype, device="cuda") for _ in range(nranks)]
            want = [torch.empty(count, dtype=dtype, device="cuda") for _ in range(nranks)]
            torch.cuda.synchronize()
            before = torch.cuda.memory_allocated()
            free_before = torch.cuda.mem_get_info()[0]
            rc = fn(_ptrs(xs), _ptrs(got), nranks, count, DT[dtype], N.REDOPS[op], stream)
            assert rc == 0, lib.nano_nccl_get_last_error()
            words = (C.c_uint32 * 4)()
            assert status_fn(stream, words) == 0 and list(words) == [0, 0, 0, 0], (list(words), lib.nano_nccl_get_last_error())
            assert torch.cuda.memory_allocated() == before  # nothing taken from torch's allocator either
            if call == 2:
                assert torch.cuda.mem_get_info()[0] >= free_before, "device memory was allocated behind torch's back"
            N.check(lib.nano_nccl_emu_all_reduce(emu, _ptrs(xs), _ptrs(want), count, DT[dtype], N.REDOPS[op],
                                                 N.ALGOS["oneshot"], 8, stream))
            torch.cuda.synchronize()
            for r in range(nranks):
                err = (got[r].float() - want[r].float()).abs()
                bound = TOL[dtype] * want[r].float().abs().clamp(min=1.0)
                assert bool((err <= bound).all()), (call, r, err.max().item())
            # and against plain PyTorch in fp32
            acc = torch.stack([x.float() for x in xs])
            ref = (acc.sum(0) if op == "sum" else acc.max(0).values).to(dtype).float()
            assert bool(((got[0].float() - ref).abs() <= TOL[dtype] * ref.abs().clamp(min=1.0)).all())
    finally:
        lib.nano_nccl_emu_destroy(emu)


def test_noalloc_rejects_sizes_beyond_its_limits():
    lib, fn = _noalloc()
    a = torch.zeros(8, device="cuda")
    b = torch.zeros(8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    too_many = 4 * 1024 * 1024 + 1
    assert fn(_ptrs([a]), _ptrs([b]), 1, too_many, 0, 0, stream) == N.STATUS_INVALID_ARGUMENT
    assert b"NANO_NCCL_NOALLOC_MAX_COUNT" in lib.nano_nccl_get_last_error()
    assert fn(_ptrs([a] * 9), _ptrs([b] * 9), 9, 8, 0, 0, stream) == N.STATUS_INVALID_ARGUMENT
    assert b"MAX_RANKS" in lib.nano_nccl_get_last_error()
    assert fn(_ptrs([a]), _ptrs([a]), 1, 8, 0, 0, stream) == N.STATUS_INVALID_ARGUMENT
    torch.cuda.synchronize()
