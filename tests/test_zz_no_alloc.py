"""The workspace-free permutation-metadata entry point (b200moe_route_metadata_noalloc).

It exists for callers that cannot give the library scratch memory -- a process whose framework
owns all of device memory, a plug-in that only sees its inputs and outputs, a loop that must not
reach cudaMalloc -- and keeps its scratch in a fixed 1 MiB array inside the library.  The check
is against the regular entry point (b200moe_route_metadata), called through the same C ABI: the
two must agree bit for bit, also on a second call that finds the first call's leftovers in the
shared scratch.  This file sorts last so that a run that stops at the first failure has already
gone through every other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(N, ids, E):
    dev = ids.device
    n = ids.numel()
    lib = N.lib()
    st = torch.cuda.current_stream().cuda_stream

    def outs():
        return (torch.full((n,), -7, dtype=torch.int64, device=dev),
                torch.full((n,), -7, dtype=torch.int32, device=dev),
                torch.full((E + 1,), -7, dtype=torch.int64, device=dev))

    r0, s0, g0 = outs()
    ws = torch.empty(max(lib.b200moe_route_metadata_workspace_bytes(n, E), 16), dtype=torch.uint8, device=dev)
    N.check(lib.b200moe_route_metadata(ids.data_ptr(), n, E, r0.data_ptr(), s0.data_ptr(), g0.data_ptr(),
                                       ws.data_ptr(), ws.numel(), st))
    r1, s1, g1 = outs()
    N.check(lib.b200moe_route_metadata_noalloc(ids.data_ptr(), n, E, r1.data_ptr(), s1.data_ptr(),
                                               g1.data_ptr(), st))
    torch.cuda.synchronize()
    return (r0, s0, g0), (r1, s1, g1)


def test_noalloc_matches_workspace_entry_point_twice():
    import llm_kernels_b200._native as N
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(77)
    # first call: a large table (all 32 chunks x 256 experts written); second call: a smaller,
    # differently shaped problem that reuses the same array with the first call's contents in it
    for T, k, E in ((4096, 8, 256), (777, 3, 40)):
        ids = torch.rand(T, E, generator=g).topk(k, dim=-1)[1].to(dev).contiguous().view(-1)
        want, got = _both(N, ids, E)
        for a, b in zip(want, got):
            assert torch.equal(a, b)            # integer results: bit-exact
        assert int(got[2][-1]) == T * k
        # and both against the CPU oracle's stable sort (reference moe/group_gemm_kernel.py:48-78)
        from oracle import restate as R
        for a, b in zip(R.run_moe_ep_preproess(ids.cpu().view(T, k), E), got):
            assert torch.equal(a, b.cpu())


def test_noalloc_rejects_oversized_problem_and_handles_empty():
    import llm_kernels_b200._native as N
    lib = N.lib()
    dev = torch.device("cuda:0")
    dummy = torch.zeros(8, dtype=torch.int64, device=dev)
    # 1025 chunks x 256 experts > 262144 entries: refused before anything is launched
    rc = lib.b200moe_route_metadata_noalloc(dummy.data_ptr(), 1025 * 1024, 256, dummy.data_ptr(), dummy.data_ptr(),
                                            dummy.data_ptr(), None)
    assert rc == 1 and b"exceeds the built-in scratch" in lib.b200moe_last_error()
    seg = torch.full((5,), 9, dtype=torch.int64, device=dev)
    N.check(lib.b200moe_route_metadata_noalloc(None, 0, 4, None, None, seg.data_ptr(),
                                               torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.equal(seg.cpu(), torch.zeros(5, dtype=torch.int64))
