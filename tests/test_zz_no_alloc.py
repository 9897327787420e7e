"""fr_align_noalloc: the align stage for callers that cannot allocate device memory (a host
application that forbids cudaMalloc after start-up, an arena with nothing left to carve, a hot
path that must stay out of the allocator).  Its scratch lives in an array owned by the library.

The file name keeps this test last in collection order, so a run that stops at the first
failure has already run every other test.  It compares the new entry point with the existing
fr_align (given a workspace) through the C ABI, bit for bit, on two calls in a row."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _buffers(n, E, bs, dev):
    return (torch.empty(n + E * (bs - 1), dtype=torch.int32, device=dev),
            torch.empty(n + E, dtype=torch.int32, device=dev),
            torch.empty(1, dtype=torch.int32, device=dev),
            torch.empty(E, dtype=torch.int32, device=dev),
            torch.empty(n, dtype=torch.int32, device=dev))


def _call_pair(lib, _lib, ids, E, bs, dev):
    n = ids.numel()
    ref = _buffers(n, E, bs, dev)
    ws = torch.zeros(lib.fr_align_workspace_bytes(E), dtype=torch.uint8, device=dev)
    rc = lib.fr_align(_lib.ptr(ids), n, E, bs, _lib.ptr(ref[0]), ref[0].numel(), _lib.ptr(ref[1]), ref[1].numel(),
                      _lib.ptr(ref[2]), _lib.ptr(ref[3]), _lib.ptr(ref[4]), _lib.ptr(ws), ws.numel(),
                      _lib.stream_ptr(dev))
    assert rc == 0
    got = _buffers(n, E, bs, dev)
    rc = lib.fr_align_noalloc(_lib.ptr(ids), n, E, bs, _lib.ptr(got[0]), got[0].numel(), _lib.ptr(got[1]),
                              got[1].numel(), _lib.ptr(got[2]), _lib.ptr(got[3]), _lib.ptr(got[4]),
                              _lib.stream_ptr(dev))
    assert rc == 0
    torch.cuda.synchronize()
    for a, b in zip(ref, got):
        assert torch.equal(a, b)
    return got


def test_align_noalloc_matches_align_twice_in_a_row(dev, lib):
    import oracle
    from fast_route_b200 import _lib
    g = torch.Generator().manual_seed(123)
    # two calls in a row on different inputs and sizes: the second must not see leftovers of the first
    for (M, k, E, bs) in ((16384, 8, 128, 64), (5000, 2, 8, 128), (16384, 8, 128, 64), (7, 3, 200, 16)):
        ids = torch.randint(0, E, (M, k), generator=g, dtype=torch.int32)
        ids[ids == 1] = 0                       # an expert without tokens
        got = _call_pair(lib, _lib, ids.to(dev).contiguous(), E, bs, dev)
        os_, oe, on, oc = oracle.moe_align_block_size(ids, bs, E)
        assert np.array_equal(got[0].cpu().numpy(), os_) and int(got[2].item()) == int(on[0])
        assert np.array_equal(got[3].cpu().numpy(), oc)


def test_align_noalloc_at_its_limits(dev, lib):
    """The largest expert count and the largest batch the built-in array covers (8192 assignments per SM) still
    match fr_align; one assignment more is refused with a clear error."""
    import oracle
    from fast_route_b200 import _lib
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    E, bs = 256, 16
    n_max = 8192 * min(sms, 256)
    g = torch.Generator().manual_seed(9)
    ids = torch.randint(0, E, (n_max,), generator=g, dtype=torch.int32)
    got = _call_pair(lib, _lib, ids.to(dev), E, bs, dev)
    os_, _, on, oc = oracle.moe_align_block_size(ids.view(-1, 1), bs, E)
    assert np.array_equal(got[0].cpu().numpy(), os_) and int(got[2].item()) == int(on[0])
    ids1 = torch.zeros(n_max + 1, dtype=torch.int32, device=dev)
    s, e, npost, cnt, inv = _buffers(n_max + 1, E, bs, dev)
    rc = lib.fr_align_noalloc(_lib.ptr(ids1), n_max + 1, E, bs, _lib.ptr(s), s.numel(), _lib.ptr(e), e.numel(),
                              _lib.ptr(npost), _lib.ptr(cnt), _lib.ptr(inv), _lib.stream_ptr(dev))
    assert rc == -2 and b"not supported" in lib.fr_error_string(rc)


def test_align_noalloc_rejects_sizes_beyond_its_scratch(dev, lib):
    from fast_route_b200 import _lib
    E = 300                                     # more experts than the built-in array covers
    ids = torch.zeros(64, dtype=torch.int32, device=dev)
    s, e, npost, cnt, inv = _buffers(64, E, 16, dev)
    rc = lib.fr_align_noalloc(_lib.ptr(ids), 64, E, 16, _lib.ptr(s), s.numel(), _lib.ptr(e), e.numel(),
                              _lib.ptr(npost), _lib.ptr(cnt), _lib.ptr(inv), _lib.stream_ptr(dev))
    assert rc == -2
    assert b"not supported" in lib.fr_error_string(rc)
