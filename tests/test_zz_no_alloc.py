"""GPU: the sort entry point that allocates nothing (its scratch is a fixed array inside the
library) gives exactly what the ordinary entry point gives, on two calls in a row.

It exists for callers that cannot get device memory at call time, such as a server whose cache pool
already owns all free HBM, or a loop that cannot afford the device-wide synchronisation of
cudaMalloc/cudaFree.  This file is collected last on purpose, so that a run that stops at the first
failure has already run every other test."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _sort_both(cabi, ids_np, E):
    lib = cabi.lib
    dev = torch.cuda.current_device()
    stream = torch.cuda.current_stream().cuda_stream
    ids = torch.from_numpy(ids_np).cuda()
    P = ids.numel()

    def outputs():
        return (torch.full((P,), -7, dtype=torch.int32, device="cuda"),
                torch.full((P,), -7, dtype=torch.int32, device="cuda"),
                torch.full((E + 1,), -7, dtype=torch.int32, device="cuda"))

    s0, i0, o0 = outputs()
    scratch = torch.empty(max(int(lib.i4tc_moe_sort_scratch_bytes(P, E)), 4), dtype=torch.uint8, device="cuda")
    cabi.check(lib.i4tc_moe_sort(ids.data_ptr(), P, E, s0.data_ptr(), i0.data_ptr(), o0.data_ptr(),
                                 scratch.data_ptr(), scratch.numel(), dev, stream), "i4tc_moe_sort")
    s1, i1, o1 = outputs()
    cabi.check(lib.i4tc_moe_sort_noalloc(ids.data_ptr(), P, E, s1.data_ptr(), i1.data_ptr(), o1.data_ptr(),
                                         dev, stream), "i4tc_moe_sort_noalloc")
    torch.cuda.synchronize()
    return (s0, i0, o0), (s1, i1, o1)


def test_noalloc_sort_matches_on_two_calls_in_a_row():
    from fp8_inference_toolkit_b200 import _cabi

    # what a server does at start-up, while device memory is still free: resolve the array's address on this
    # device (which also loads the code module); nothing is launched
    _cabi.check(_cabi.lib.i4tc_moe_sort_noalloc_prepare(torch.cuda.current_device()), "i4tc_moe_sort_noalloc_prepare")
    rng = np.random.RandomState(11)
    # first a large problem that fills most of the built-in scratch, then a smaller one with a
    # different expert count, so stale contents of the shared array would show
    for P, E in [(60000, 256), (5000, 128)]:
        ids = rng.randint(0, E, size=P).astype(np.int32)
        ids[ids == 3] = 2  # leave one expert empty
        (s0, i0, o0), (s1, i1, o1) = _sort_both(_cabi, ids, E)
        assert torch.equal(o0, o1) and torch.equal(s0, s1) and torch.equal(i0, i1)
        order = np.argsort(ids, kind="stable")
        assert np.array_equal(s1.cpu().numpy(), order)
        assert int(o1[-1]) == P


def test_noalloc_sort_rejects_sizes_beyond_its_scratch():
    from fp8_inference_toolkit_b200 import _cabi

    lib = _cabi.lib
    cap = int(lib.i4tc_moe_sort_noalloc_max_scratch_ints())
    assert cap == 16384
    P, E = 1024 * 65, 256  # 65 chunks * 256 experts > 16384
    ids = torch.zeros(P, dtype=torch.int32, device="cuda")
    out = torch.empty(P, dtype=torch.int32, device="cuda")
    off = torch.empty(E + 1, dtype=torch.int32, device="cuda")
    rc = lib.i4tc_moe_sort_noalloc(ids.data_ptr(), P, E, out.data_ptr(), 0, off.data_ptr(),
                                   torch.cuda.current_device(), torch.cuda.current_stream().cuda_stream)
    assert rc == -1 and "exceeds the built-in scratch" in _cabi.last_error()
