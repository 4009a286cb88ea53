"""The config-5 style job on two CPU ranks (gloo): every rank computes the partitioned layout on its own and the
ranks must agree on owners, on who stores what and on the split of the click log, without exchanging anything but
the digests compared here."""
import hashlib
import multiprocessing as mp
import os
import socket
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from hetuctr_b200 import workloads as w
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    w.CONFIGS["cfg5_tiny"] = dict(w.CONFIGS["cfg5_sweep"], rows=200_000, samples=256)
    root, storage, mine, data = w.partitioned_job("cfg5_tiny", world, 20_000, 2000)
    h = hashlib.sha256()
    for a in [root, data, *storage, *mine]:
        h.update(np.ascontiguousarray(a).tobytes())
    digest = torch.tensor(list(h.digest()), dtype=torch.uint8)
    gathered = [torch.empty_like(digest) for _ in range(world)]
    dist.all_gather(gathered, digest)
    # this rank's share of the work: its samples and the rows they touch that it does not own
    keys = np.unique(data[mine[rank]])
    remote = torch.tensor([int((root[keys] != rank).sum()), int(keys.size), int(mine[rank].size)])
    totals = remote.clone()
    dist.all_reduce(totals)
    dist.destroy_process_group()
    q.put((rank, all(bool((g == digest).all()) for g in gathered), remote.tolist(), totals.tolist()))


def test_two_ranks_agree_on_the_partitioned_layout():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(30)
    assert [o[0] for o in out] == [0, 1]
    assert all(o[1] for o in out), "ranks computed different layouts"
    assert out[0][3] == out[1][3]
    assert out[0][3][2] == 20_000  # every sample belongs to exactly one rank
    # both ranks got a share, and most rows a rank's samples touch are its own
    for _, _, (remote, touched, samples), _ in out:
        assert samples > 5000 and remote < 0.5 * touched
