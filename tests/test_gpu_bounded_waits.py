"""Waits inside the exchange kernels are bounded: a peer that never publishes makes the waiting kernel give up
after its limit, set HCTR_ERR_TIMEOUT in the device error word and RETURN, so the context stays usable and the
host can report the failure.  Nothing here faults or hangs the GPU: the wait simply runs out, on a mailbox whose
sequence word nobody writes, with a limit of a few milliseconds.
"""
import ctypes
import time

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

import hetuctr_b200 as hb  # noqa: E402

HCTR_ERR_TIMEOUT = 8


from hetuctr_b200.owner_replay import Box, Ctx  # noqa: E402  (ctypes mirrors of hctr_p2p_box / hctr_p2p_ctx)


def _mailbox(nrank, timeout_ms):
    dev = torch.device("cuda:0")
    hdr = torch.zeros(nrank * 16, dtype=torch.int32, device=dev)
    boxes = (Box * nrank)()
    for b in boxes:
        b.hdr = hdr.data_ptr()  # only the headers are touched by a wait
    d_boxes = torch.frombuffer(bytearray(bytes(boxes)), dtype=torch.uint8).to(dev)
    cnt_in = torch.full((5 * nrank + 8,), 77, dtype=torch.int32, device=dev)
    err = torch.zeros(4, dtype=torch.int32, device=dev)
    ctx = Ctx(nrank, 0, 1000, 4, d_boxes.data_ptr(), cnt_in.data_ptr(), err.data_ptr(), int(timeout_ms * 1e6))
    return ctx, hdr, cnt_in, err, d_boxes


@pytest.mark.parametrize("phase", [0, 1])
def test_wait_for_a_silent_peer_gives_up_and_returns(phase):
    L = hb.lib()
    nrank = 4
    ctx, hdr, cnt_in, err, keep = _mailbox(nrank, timeout_ms=5)
    # sources 0 and 2 have published sequence number 9 with their counts; sources 1 and 3 stay silent
    h = hdr.view(nrank, 16)
    for s, (q, g, r) in {0: (11, 3, 5), 2: (7, 0, 2)}.items():
        h[s, 0], h[s, 1], h[s, 2] = 9, q, g
        h[s, 8], h[s, 9] = 9, r
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    assert L.hctr_p2p_wait(ctypes.byref(ctx), phase, 9, None) == 0
    torch.cuda.synchronize()  # returns: the kernel ended by itself
    assert time.perf_counter() - t0 < 2.0
    assert int(err[0]) & HCTR_ERR_TIMEOUT
    c = cnt_in.cpu().numpy()
    if phase == 0:
        assert list(c[:nrank]) == [11, 0, 7, 0] and list(c[nrank:2 * nrank]) == [3, 0, 0, 0]
        assert list(c[3 * nrank:4 * nrank + 1]) == [0, 11, 11, 18, 18]
    else:
        assert list(c[2 * nrank:3 * nrank]) == [5, 0, 2, 0]
    # the context is intact: the same wait succeeds once everybody has published
    h[:, 0] = 10
    h[:, 8] = 10
    h[:, 1] = 1
    h[:, 2] = 0
    h[:, 9] = 1
    err.zero_()
    torch.cuda.synchronize()
    assert L.hctr_p2p_wait(ctypes.byref(ctx), phase, 10, None) == 0
    torch.cuda.synchronize()
    assert int(err[0]) == 0


def test_announced_count_beyond_the_mailbox_is_refused():
    L = hb.lib()
    ctx, hdr, cnt_in, err, keep = _mailbox(2, timeout_ms=5)
    h = hdr.view(2, 16)
    h[:, 0] = 3
    h[0, 1] = 5
    h[1, 1] = 1001  # cap is 1000
    torch.cuda.synchronize()
    assert L.hctr_p2p_wait(ctypes.byref(ctx), 0, 3, None) == 0
    torch.cuda.synchronize()
    assert int(err[0]) == 4  # HCTR_ERR_CAPACITY, and no timeout
    assert list(cnt_in.cpu().numpy()[:2]) == [5, 0]


def test_timeout_setting_is_validated():
    import os
    import threading
    root = np.array([0, 1], dtype=np.uint8)
    for bad in ("soon", "0", "999999999"):
        os.environ["HCTR_EXCHANGE"], os.environ["HCTR_P2P_TIMEOUT_MS"] = "p2p", bad
        errs = []

        def make(r):
            try:
                hb.Table(r, 2, 0, "inproc", 9000 + len(bad), 2, 4, 0, 0, root, np.array([r]))
            except RuntimeError as e:
                errs.append(str(e))

        try:
            ts = [threading.Thread(target=make, args=(r,)) for r in range(2)]
            [t.start() for t in ts]
            [t.join() for t in ts]
        finally:
            del os.environ["HCTR_EXCHANGE"], os.environ["HCTR_P2P_TIMEOUT_MS"]
        assert len(errs) == 2 and all("HCTR_P2P_TIMEOUT_MS" in e for e in errs), (bad, errs)
