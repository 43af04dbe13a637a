"""The allocation-free grouping entry point (``fm_group_rows_static``) against ``fm_group_rows``.

Some hosts of this library are not allowed to allocate device memory (they work inside a fixed arena or
under a framework that forbids it at that point), so one entry point keeps its scratch in the library
image instead of taking a workspace.  It is called here straight through the C ABI, twice in a row with
different inputs, because the built-in scratch still holds the first call's counts when the second starts.
This file sorts last so that a run stopping at the first failure has already been through everything else.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _group_static(L, lib, hashes, total_buckets, seg_xb=None, seg_cb=None):
    n = hashes.numel()
    group_off = torch.empty(total_buckets + 1, dtype=torch.int32, device=DEV)
    perm = torch.empty(max(n, 1), dtype=torch.int32, device=DEV)
    n_seg = 1 if seg_xb is None else seg_xb.numel() - 1
    L.check(lib.fm_group_rows_static(L.ptr(hashes), n, total_buckets, n_seg, L.ptr(seg_xb), L.ptr(seg_cb),
                                     L.ptr(group_off), L.ptr(perm), L.stream_ptr(torch.device(DEV))),
            "fm_group_rows_static")
    return group_off, perm[:n]


def _same_grouping(a, b, hashes_global):
    """Offsets identical; inside a bucket the order is unspecified for both entry points, so the rows of
    every bucket are compared as sets (sort by (bucket, row))."""
    (off_a, perm_a), (off_b, perm_b) = a, b
    assert torch.equal(off_a, off_b)
    key = lambda perm: torch.sort(hashes_global[perm.long()].long() * (1 << 32) + perm.long()).values
    assert torch.equal(key(perm_a), key(perm_b))
    assert torch.equal(torch.sort(perm_a.long()).values, torch.arange(perm_a.numel(), device=DEV))


def test_static_scratch_grouping_matches_workspace_grouping_twice():
    import fast_memory_b200 as fm
    from fast_memory_b200 import _lib as L
    lib = L.lib()
    g = torch.Generator().manual_seed(123)
    # call 1: many buckets, every one populated; call 2: fewer rows over a different bucket count, with
    # segments, so stale counts from call 1 would show up as wrong offsets
    h1 = torch.randint(5000, (200000,), generator=g).int().to(DEV)
    got1 = _group_static(L, lib, h1, 5000)
    _same_grouping(got1, fm.group_rows(h1, 5000), h1)

    xb = torch.tensor([0, 300, 301, 1000], dtype=torch.int32, device=DEV)
    cb = torch.tensor([0, 7, 40, 300], dtype=torch.int32, device=DEV)
    local = torch.cat([torch.randint(7, (300,), generator=g), torch.randint(33, (1,), generator=g),
                       torch.randint(260, (699,), generator=g)]).int().to(DEV)
    group_off2 = torch.empty(301, dtype=torch.int32, device=DEV)
    perm2 = torch.empty(1000, dtype=torch.int32, device=DEV)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    L.check(lib.fm_group_rows_static(L.ptr(local), 1000, 300, 3, L.ptr(xb), L.ptr(cb), L.ptr(group_off2), L.ptr(perm2),
                                     L.stream_ptr(torch.device(DEV))), "fm_group_rows_static")
    torch.cuda.synchronize()
    # the claim itself: with the outputs made beforehand, the call leaves the device's free memory where it was
    assert torch.cuda.mem_get_info()[0] == free_before
    got2 = (group_off2, perm2)
    seg = torch.bucketize(torch.arange(1000, device=DEV), xb[1:].long(), right=True)
    _same_grouping(got2, fm.group_rows(local, 300, xb, cb), local + cb[seg])

    # sizes beyond the built-in scratch are refused with a clear message, before anything is launched
    limit = lib.fm_group_rows_static_max_buckets()
    assert limit == 65536
    rc = lib.fm_group_rows_static(L.ptr(h1), h1.numel(), limit + 1, 1, None, None, L.ptr(got1[0]), L.ptr(got1[1]),
                                  L.stream_ptr(torch.device(DEV)))
    assert rc == -2 and b"exceed the built-in scratch" in lib.fm_last_error()
