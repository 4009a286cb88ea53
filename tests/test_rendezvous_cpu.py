"""Host-side multi-process logic without a GPU: the TCP bootstrap that carries the NCCL unique id from rank 0 to
the other ranks.  World sizes 2 and 4 as separate processes on 127.0.0.1, plus the failure path: a rank that
never arrives must produce an error on the others (within the timeout), not a hang."""
import ctypes
import multiprocessing as mp
import os
import socket
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank(rank, nrank, port, timeout, q):
    sys.path.insert(0, ROOT)
    import hetuctr_b200 as hb
    L = hb.lib()
    buf = ctypes.create_string_buffer(128)
    if rank == 0:
        buf.raw = bytes(range(128))
    rc = L.hctr_rendezvous_broadcast(rank, nrank, b"127.0.0.1", port, buf, 128, timeout)
    q.put((rank, rc, bytes(buf.raw), L.hctr_last_error().decode() if rc else ""))


def _run(nrank, present, timeout):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, nrank, port, timeout, q)) for r in present]
    for p in procs:
        p.start()
    out = [q.get(timeout=60) for _ in procs]
    for p in procs:
        p.join(10)
    return {r: (rc, data, err) for r, rc, data, err in out}


@pytest.mark.parametrize("nrank", [2, 4])
def test_broadcast_reaches_every_rank(nrank):
    res = _run(nrank, range(nrank), 30.0)
    for r in range(nrank):
        rc, data, err = res[r]
        assert rc == 0, err
        assert data == bytes(range(128))


def test_missing_rank_times_out_with_an_error():
    res = _run(3, [0, 1], 2.0)  # rank 2 never starts
    assert res[0][0] == -1 and "ranks arrived" in res[0][2]
    assert res[1][0] == -1  # rank 1 was accepted but never receives the payload


def test_missing_root_times_out_with_an_error():
    res = _run(2, [1], 1.5)  # nobody listens
    assert res[1][0] == -1 and "not reachable" in res[1][2]
