"""The allocation-free C entry point `q38_moe_sort_static`, called through its exported symbol.

Some users of the library may not allocate device memory at the point where they route tokens (pre-planned arenas,
latency-critical threads that must not touch the allocator).  For them the library exports one C function whose scratch
is a static device array inside the shared object; the caller brings every input and output buffer.  This test calls it
via ctypes with raw device pointers, twice in a row (the second call reuses the scratch the first one dirtied, with a
different problem), and compares each result with the regular `moe_sort` operator.  The file name makes pytest collect
it last."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_sort_matches_operator():
    from q38 import ops
    lib_ops = ops.load()
    lib = ctypes.CDLL(ops.loaded_library())
    fn = lib.q38_moe_sort_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_int, ctypes.c_void_p]
    torch.manual_seed(21)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream(dev)
    for T, k, E in ((5000, 5, 64), (777, 2, 8)):
        idx = torch.stack([torch.randperm(E, device=dev)[:k] for _ in range(T)]).to(torch.int32).contiguous()
        P = T * k
        max_tiles = (P + 127) // 128 + E
        perm = torch.full((P,), -1, dtype=torch.int32, device=dev)
        inv = torch.full((P,), -1, dtype=torch.int32, device=dev)
        offsets = torch.full((E + 1,), -1, dtype=torch.int32, device=dev)
        sched = torch.full((1 + 3 * max_tiles,), -1, dtype=torch.int32, device=dev)
        code = fn(idx.data_ptr(), P, E, perm.data_ptr(), inv.data_ptr(), offsets.data_ptr(), sched.data_ptr(), max_tiles,
                  ctypes.c_void_p(stream.cuda_stream))
        assert code == 0
        torch.cuda.synchronize(dev)
        r_perm, r_inv, r_offsets, r_sched = lib_ops.moe_sort(idx, E)
        assert torch.equal(perm, r_perm) and torch.equal(inv, r_inv) and torch.equal(offsets, r_offsets)
        assert torch.equal(sched[:r_sched.numel()], r_sched)
    # expert ids outside [0, experts) are skipped: inv_perm -1, not counted, the remaining pairs sorted as usual
    T, k, E = 300, 2, 8
    idx = torch.stack([torch.randperm(E, device=dev)[:k] for _ in range(T)]).to(torch.int32).contiguous()
    bad = torch.tensor([3, 77, 410], device=dev)
    flat = idx.view(-1)
    flat[bad] = torch.tensor([-1, 64, 8], dtype=torch.int32, device=dev)
    P = T * k
    max_tiles = (P + 127) // 128 + E
    perm = torch.full((P,), -7, dtype=torch.int32, device=dev)
    inv = torch.full((P,), -7, dtype=torch.int32, device=dev)
    offsets = torch.full((E + 1,), -7, dtype=torch.int32, device=dev)
    sched = torch.full((1 + 3 * max_tiles,), -7, dtype=torch.int32, device=dev)
    assert fn(idx.data_ptr(), P, E, perm.data_ptr(), inv.data_ptr(), offsets.data_ptr(), sched.data_ptr(), max_tiles, ctypes.c_void_p(stream.cuda_stream)) == 0
    torch.cuda.synchronize(dev)
    good = torch.ones(P, dtype=torch.bool, device=dev)
    good[bad] = False
    assert int(offsets[E]) == P - 3 and torch.equal(inv[bad], torch.full((3,), -1, dtype=torch.int32, device=dev))
    order = torch.sort(flat[good].long(), stable=True).indices
    assert torch.equal(perm[:P - 3].long(), torch.nonzero(good).view(-1)[order])
    assert torch.equal(perm[P - 3:], torch.full((3,), -7, dtype=torch.int32, device=dev))
    # sizes beyond the static scratch are refused and nothing is launched
    big = 1024 * 1024 + 1
    assert fn(idx.data_ptr(), big, 64, perm.data_ptr(), inv.data_ptr(), offsets.data_ptr(), sched.data_ptr(), big, ctypes.c_void_p(stream.cuda_stream)) == 1
    assert fn(idx.data_ptr(), 100, 65, perm.data_ptr(), inv.data_ptr(), offsets.data_ptr(), sched.data_ptr(), 200, ctypes.c_void_p(stream.cuda_stream)) == 1
    assert fn(None, 100, 8, perm.data_ptr(), inv.data_ptr(), offsets.data_ptr(), sched.data_ptr(), 200, ctypes.c_void_p(stream.cuda_stream)) == 2
    ops.check_errors()
