"""The allocation-free prefix-sum entry point against the regular one, through the C-ABI.

Who needs it: hosts that may not call cudaMalloc where they need a scan — an allocator callback of a framework,
a latency-critical loop that must keep away from the driver's allocation lock, a plugin that is only handed input
and output buffers.  Its scratch is a fixed array inside the library (shared by all calls on a device), so the
test runs it twice in a row with different sizes: the second call must not be disturbed by what the first left
behind.  Collected last so that a failure here cannot hide the other tests' results.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

import hetuctr_b200 as hb  # noqa: E402


def _reference_scan(L, x):
    n = x.numel()
    out = torch.empty(n + 1, dtype=torch.int32, device=x.device)
    scratch = torch.empty(int(L.hctr_scan_scratch_words(n)) + 1, dtype=torch.int32, device=x.device)
    rc = L.hctr_scan_exclusive_u32(x.data_ptr(), out.data_ptr(), n, None, scratch.data_ptr(), None)
    assert rc == 0
    return out


_warmed = set()


def _noalloc_scan(L, x):
    """Runs the entry point and checks, with the driver's own figure for free device memory (which also sees
    allocations that bypass PyTorch's allocator), that a call which is not the first one on the device leaves
    that figure unchanged.  The first call on a device looks up the address of the built-in scratch, which may
    make the driver load the module's data lazily, so it is not held to that."""
    n = x.numel()
    out = torch.full((n + 1,), -1, dtype=torch.int32, device=x.device)
    if x.device.index not in _warmed:
        one = torch.zeros(2, dtype=torch.int32, device=x.device)
        assert L.hctr_scan_exclusive_u32_noalloc(one.data_ptr(), one.data_ptr(), 1, None) == 0
        torch.cuda.synchronize()
        _warmed.add(x.device.index)
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(x.device)
    rc = L.hctr_scan_exclusive_u32_noalloc(x.data_ptr(), out.data_ptr(), n, None)
    assert rc == 0, L.hctr_noalloc_last_error().decode()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(x.device)
    assert free_after == free_before, "the allocation-free entry point changed the amount of free device memory"
    return out


def test_noalloc_scan_matches_regular_scan_twice_in_a_row():
    L = hb.lib()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    # first a large input (hundreds of tiles of scratch), then a smaller one that reuses a prefix of the scratch
    # ... and sizes that end exactly on tile boundaries of the scan (4096 elements per tile)
    for n in (1_500_000, 70_001, 5, 0, 300_000, 4096, 4095, 4097, 8192, 4096 * 4096):
        x = torch.randint(0, 7, (max(n, 1),), dtype=torch.int32, device=dev, generator=g)[:n].contiguous()
        want = _reference_scan(L, x)
        got = _noalloc_scan(L, x)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"n={n}"
        host = np.concatenate([[0], np.cumsum(x.cpu().numpy().astype(np.int64))]).astype(np.int32)
        assert np.array_equal(got.cpu().numpy(), host), f"n={n}"


def test_noalloc_scan_in_place_and_size_limit():
    L = hb.lib()
    dev = torch.device("cuda:0")
    x = torch.ones(100_001, dtype=torch.int32, device=dev)
    assert L.hctr_scan_exclusive_u32_noalloc(x.data_ptr(), x.data_ptr(), 100_000, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(x, torch.arange(100_001, dtype=torch.int32, device=dev))
    # beyond the built-in scratch: refused with a message, nothing launched
    rc = L.hctr_scan_exclusive_u32_noalloc(x.data_ptr(), x.data_ptr(), (1 << 26) + 1, None)
    assert rc != 0
    assert "exceeds" in L.hctr_noalloc_last_error().decode()
    torch.cuda.synchronize()


def test_noalloc_scan_accepts_exactly_the_maximum():
    L = hb.lib()
    dev = torch.device("cuda:0")
    n = 1 << 26  # HCTR_NOALLOC_SCAN_MAX: the largest input the built-in scratch serves
    x = torch.ones(n, dtype=torch.int32, device=dev)
    got = _noalloc_scan(L, x)
    assert int(got[-1]) == n and int(got[n // 2]) == n // 2 and int(got[0]) == 0
    assert torch.equal(got[1:] - got[:-1], x)
