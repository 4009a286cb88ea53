"""Test helper: all ranks of a job on ONE GPU, driven in lockstep through the table-level C-ABI.

Mirrors the oracle's `World` API so a test can step both and compare.  With nrank > 1 the ranks are
threads of this process (ip="inproc") and there are two ways for them to exchange data:

  exchange="inproc"  the kernels of the NCCL path; bytes move between the ranks' buffers with cudaMemcpyAsync
  exchange="p2p"     the kernels of the peer-to-peer mailbox exchange, the default of a one-process-per-GPU job:
                     queries, pushed rows, flags and returned rows are stored straight into the destination rank's
                     mailbox.  The ranks share one CUDA context here, so a peer's mailbox is a plain pointer; the
                     table drains its stream and meets the other ranks at a host barrier between publishing and
                     consuming, so no kernel ever waits for another launch on the same GPU.
"""
import itertools
import os
import threading

import numpy as np
import torch

import hetuctr_b200 as hb

_job = itertools.count(1)


def _parallel(fns):
    errs = [None] * len(fns)

    def run(i):
        try:
            fns[i]()
        except BaseException as e:  # noqa: BLE001 - re-raised below
            errs[i] = e

    ts = [threading.Thread(target=run, args=(i,)) for i in range(len(fns))]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    for e in errs:
        if e is not None:
            raise e


class GpuWorld:
    def __init__(self, nrank, length, width, pull_bound, push_bound, learning_rate, root_arr, storage_arrs,
                 init=(hb.INIT_ZERO, 0.0, 0.0), device=0, keys_on_device=True, exchange="inproc",
                 buffers="device"):
        self.nrank, self.length, self.width = nrank, length, width
        self.exchange = exchange if nrank > 1 else "none"
        self.dev = torch.device("cuda", device)
        self.keys_on_device = keys_on_device
        self.buffers = buffers  # where gradients and pulled rows live: "device", "pinned" or "pageable" host memory
        self.tables = [None] * nrank
        port = next(_job)

        def make(r):
            self.tables[r] = hb.Table(r, nrank, device, "inproc" if nrank > 1 else "127.0.0.1", port, length, width,
                                      pull_bound, push_bound, root_arr, storage_arrs[r], init, learning_rate, 0)

        # the exchange flavour is read from the environment when a table is constructed
        saved = {k: os.environ.get(k) for k in ("HCTR_EXCHANGE", "HCTR_P2P_TIMEOUT_MS")}
        if exchange == "p2p":
            os.environ["HCTR_EXCHANGE"] = "p2p"
            os.environ["HCTR_P2P_TIMEOUT_MS"] = "2000"
        else:
            os.environ.pop("HCTR_EXCHANGE", None)
        try:
            _parallel([lambda r=r: make(r) for r in range(nrank)])
        finally:
            for k, v in saved.items():
                if v is None:
                    os.environ.pop(k, None)
                else:
                    os.environ[k] = v
        if nrank > 1:
            assert self.tables[0].exchange_name() == exchange
        self._batch = [0] * nrank
        self._keep = []

    def close(self):
        for t in self.tables:
            if t is not None:
                t.close()

    def set_embedding(self, rank, emb):
        self.tables[rank].set_embedding(emb)

    def preprocess(self, keys_per_rank):
        keys = [np.ascontiguousarray(k, dtype=np.int64) for k in keys_per_rank]
        if self.keys_on_device:
            bufs = [torch.from_numpy(k).to(self.dev) for k in keys]
        else:
            bufs = keys
        self._keep = bufs
        _parallel([lambda r=r: self.tables[r].preprocess(bufs[r], keys[r].size) for r in range(self.nrank)])
        self._batch = [k.size for k in keys]

    def push_pull(self, grads_per_rank):
        if self.buffers != "device":
            return self._push_pull_host(grads_per_rank)
        dsts = [torch.full((max(b, 1), self.width), float("nan"), device=self.dev) for b in self._batch]
        if grads_per_rank is None:
            grads = [None] * self.nrank
        else:
            grads = [torch.from_numpy(np.ascontiguousarray(g, dtype=np.float32)).to(self.dev) for g in grads_per_rank]
        torch.cuda.synchronize()
        _parallel([lambda r=r: self.tables[r].push_pull(grads[r], dsts[r]) for r in range(self.nrank)])
        return [d[:b].cpu().numpy() for d, b in zip(dsts, self._batch)]

    def _push_pull_host(self, grads_per_rank):
        pin = self.buffers == "pinned"
        dsts = [torch.full((max(b, 1), self.width), float("nan")) for b in self._batch]
        grads = [None] * self.nrank
        if grads_per_rank is not None:
            grads = [torch.from_numpy(np.array(g, dtype=np.float32, order="C")) for g in grads_per_rank]
        if pin:
            dsts = [d.pin_memory() for d in dsts]
            grads = [g.pin_memory() if g is not None else None for g in grads]
        _parallel([lambda r=r: self.tables[r].push_pull(grads[r], dsts[r]) for r in range(self.nrank)])
        return [d[:b].numpy().copy() for d, b in zip(dsts, self._batch)]

    def get_all(self, what, prev=False):
        """`what` of every rank, fetched by all ranks at the same time (some views are collective)."""
        out = [None] * self.nrank

        def one(r):
            out[r] = self.get(r, what, prev)

        _parallel([lambda r=r: one(r) for r in range(self.nrank)])
        return out

    def get(self, rank, what, prev=False):
        t = self.tables[rank]
        if what == "storage":
            return t.stats()["stored_rows"]
        if what == "nonlocal":
            return t.stats()["cached_rows"]
        if what == "unique_size":
            return len(t.dump("unique_idx", prev))
        return t.dump(what, prev)

    def get_f32(self, rank, what):
        return self.tables[rank].dump(what)


INDEX_ARRAYS = ("unique_idx", "idx_map", "sorted_arg", "run_length", "root", "offset", "shape", "shape_exchanged")


def assert_index_parity(gw, ow, ranks=None):
    """Bit-exact comparison of everything preprocess produces."""
    for name in INDEX_ARRAYS:
        # with the mailbox exchange the peers' counts only reach the host on demand, collectively
        every = gw.get_all(name) if name == "shape_exchanged" else None
        for r in ranks if ranks is not None else range(gw.nrank):
            g, o = every[r] if every else gw.get(r, name), ow.get(r, name)
            assert g.shape == o.shape and np.array_equal(g, o), f"rank {r}: {name} differs"


def assert_state_parity(gw, ow, exact=True, rtol=1e-5, atol=1e-6):
    for r in range(gw.nrank):
        assert np.array_equal(gw.get(r, "version"), ow.get(r, "version")), f"rank {r}: versions differ"
        assert np.array_equal(gw.get(r, "updates"), ow.get(r, "updates")), f"rank {r}: pending counts differ"
        for name in ("embedding", "gradient"):
            g, o = gw.get_f32(r, name), ow.get_f32(r, name)
            if exact:
                assert np.array_equal(g, o), f"rank {r}: {name} differs"
            else:
                np.testing.assert_allclose(g, o, rtol=rtol, atol=atol, err_msg=f"rank {r}: {name}")
