"""Replays the OWNER side of one step of the peer-to-peer exchange on a single GPU, from synthetic traffic.

  python -m hetuctr_b200.owner_replay [--sources 8] [--rows 4200000] [--width 128] [--pushed 68000]
                                      [--queries 77000] [--iters 20] [--check | --cap 212992]

In a job of several GPUs the owner-side kernels (source marking + versions, row apply, staleness test + row gather)
run once per step on what the peers stored into this rank's mailbox.  To time or profile them in isolation this
tool builds one rank's table shard and mailbox on one GPU, fills the mailbox the way `sources - 1` peers would
(key-sorted push lists drawn from a Zipf distribution over the rank's own rows, so hot rows are pushed by several
peers at once; key-sorted query lists with versions), and launches the kernels through the kernel-level C-ABI
(include/hctr_kernels.h).  The peers' mailboxes - where flags and returned rows are stored - are stand-ins in local
memory (one per peer), so NVLink is not part of what is measured: the figures are the kernels' HBM-side cost.
`--check` compares the table after one step with a numpy evaluation that applies the sources one after the other.
"""
import argparse
import ctypes
import json

import numpy as np

vp = ctypes.c_void_p


class Box(ctypes.Structure):  # hctr_p2p_box
    _fields_ = [(n, vp) for n in ("hdr", "qkey", "qver", "pkey", "pupd", "pval", "flag", "rver", "rval")]


class Ctx(ctypes.Structure):  # hctr_p2p_ctx
    _fields_ = [("nrank", ctypes.c_int), ("rank", ctypes.c_int), ("cap", ctypes.c_uint32), ("width", ctypes.c_size_t),
                ("box", vp), ("cnt_in", vp), ("err", vp), ("timeout_ns", ctypes.c_ulonglong)]


def cnt_words(n):
    return 5 * n + 8  # HCTR_P2P_CNT_WORDS


class OwnerReplay:
    def __init__(self, sources=8, rows=4_200_000, width=128, pushed=68_000, queries=77_000, alpha=1.05, seed=0,
                 device=0, cap=0, shared_peer=False):
        import torch

        import hetuctr_b200 as hb
        self.torch, self.L = torch, hb.lib()
        self.dev = dev = torch.device("cuda", device)
        torch.cuda.set_device(dev)
        n, S, W = sources, rows, width
        self.n, self.S, self.W, self.rank = n, S, W, 0
        rng = np.random.RandomState(seed)
        # this rank owns keys 0, n, 2n, ...; row of key k is a permutation of [0, S)
        self.length = n * S
        perm = rng.permutation(S).astype(np.int32)
        row_of = np.full(self.length, -1, dtype=np.int32)
        row_of[::n] = perm
        self.row_of_h = row_of
        self.row_of = torch.from_numpy(row_of).to(dev)
        self.emb = torch.randn(S, W, device=dev) * 0.1
        self.version = torch.randint(0, 50, (S,), dtype=torch.int64, device=dev)
        self.mask = torch.zeros(S, dtype=torch.int64, device=dev)
        self.head = torch.zeros(S, dtype=torch.int64, device=dev)

        # traffic of the peers: key-sorted unique keys per source, drawn from a bounded Zipf over this rank's rows
        def draw(m):
            m = min(m, S)
            ks = np.zeros(0, np.int64)
            while len(ks) < m:  # m distinct rows, the hot ones (low Zipf ranks) in nearly every source's list
                ranks = np.minimum(rng.zipf(alpha, size=2 * m) - 1, S - 1).astype(np.int64)
                ks = np.unique(np.concatenate([ks, ranks * 2654435761 % S]))
            if len(ks) > m:
                ks = np.sort(rng.choice(ks, m, replace=False))
            return ks * n  # this rank's keys

        per_push = max(pushed // max(n - 1, 1), 1)
        per_query = max(queries // n, 1)
        self.push_keys = [np.zeros(0, np.int64) if s == self.rank else draw(per_push) for s in range(n)]
        self.query_keys = [draw(per_query) for _ in range(n)]
        # rows per (mailbox, source) sub-region: a table uses its batch size, which also sizes the kernels' grids
        self.cap = cap = int(max(cap, max(len(k) for k in self.push_keys), max(len(k) for k in self.query_keys), 1))

        def z(shape, dt):
            return torch.zeros(shape, dtype=dt, device=dev)

        def region_set():
            return dict(hdr=z(n * 16, torch.int32), qkey=z(n * cap, torch.int64), qver=z(n * cap, torch.int64),
                        pkey=z(n * cap, torch.int64), pupd=z(n * cap, torch.int64), pval=z((n * cap, W), torch.float32),
                        flag=z(n * cap, torch.uint8), rver=z(n * cap, torch.int64), rval=z((n * cap, W), torch.float32))

        self.mine = region_set()
        # one stand-in mailbox per peer; `shared_peer` lets all peers share one (timing runs with a large cap)
        shared = region_set() if shared_peer else None
        self.peers = [self.mine if s == self.rank else (shared or region_set()) for s in range(n)]
        self.push_upd, self.push_val, self.query_ver = [], [], []
        for s in range(n):
            k = self.push_keys[s]
            upd = rng.randint(1, 5, size=len(k)).astype(np.int64)
            val = rng.normal(0, 0.01, size=(len(k), W)).astype(np.float32)
            self.push_upd.append(upd)
            self.push_val.append(val)
            self.mine["pkey"][s * cap:s * cap + len(k)] = torch.from_numpy(k).to(dev)
            self.mine["pupd"][s * cap:s * cap + len(k)] = torch.from_numpy(upd).to(dev)
            self.mine["pval"][s * cap:s * cap + len(k)] = torch.from_numpy(val).to(dev)
            q = self.query_keys[s]
            qv = rng.randint(0, 60, size=len(q)).astype(np.int64)
            qv[rng.rand(len(q)) < 0.2] = np.iinfo(np.int64).min
            self.query_ver.append(qv)
            self.mine["qkey"][s * cap:s * cap + len(q)] = torch.from_numpy(q).to(dev)
            self.mine["qver"][s * cap:s * cap + len(q)] = torch.from_numpy(qv).to(dev)
        boxes = (Box * n)()
        for s in range(n):
            src = self.peers[s]
            for f, _ in Box._fields_:
                setattr(boxes[s], f, src[f].data_ptr())
        self.mine_box = Box()
        for f, _ in Box._fields_:
            setattr(self.mine_box, f, self.mine[f].data_ptr())
        self.d_boxes = torch.frombuffer(bytearray(bytes(boxes)), dtype=torch.uint8).to(dev)
        self.cnt_in = z(cnt_words(n), torch.int32)
        self.err = z(4, torch.int32)
        self.ctx = Ctx(n, self.rank, cap, W, self.d_boxes.data_ptr(), self.cnt_in.data_ptr(), self.err.data_ptr(),
                       int(50e6))
        slots = n * cap
        self.ent_row = z(slots + 1, torch.int32)
        self.ent_next = z(slots + 1, torch.int32)
        self.seq = 0
        self.epoch = 0
        i64, u32, sz = ctypes.c_int64, ctypes.c_uint32, ctypes.c_size_t
        self.L.hctr_p2p_owner_mark.argtypes = [vp, vp, u32, vp, sz, sz, vp, vp, u32, vp, vp, vp, vp]
        self.L.hctr_p2p_owner_apply.argtypes = [vp, vp, sz, vp, vp, vp, vp, vp, vp]
        self.L.hctr_p2p_stale_gather.argtypes = [vp, u32, vp, sz, sz, vp, vp, i64, vp]

    def publish(self):
        """What the peers' last thread blocks do: counts + sequence number into this rank's headers."""
        self.seq += 1
        h = self.mine["hdr"].view(self.n, 16)
        for s in range(self.n):
            h[s, 1] = len(self.query_keys[s])
            h[s, 2] = len(self.push_keys[s])
        h[:, 0] = self.seq
        self.torch.cuda.synchronize()

    def step(self, pull_bound=0, events=None):
        """One owner-side step; with `events` (4 CUDA events) the three kernels are bracketed for timing."""
        L, c, mb = self.L, ctypes.byref(self.ctx), ctypes.byref(self.mine_box)
        rec = (lambda i: events[i].record()) if events else (lambda i: None)
        self.epoch += 2
        rec(0)
        rc = L.hctr_p2p_owner_mark(c, mb, self.seq, self.row_of.data_ptr(), self.length, 0, self.mask.data_ptr(),
                                   self.head.data_ptr(), self.epoch, self.ent_row.data_ptr(),
                                   self.ent_next.data_ptr(), self.version.data_ptr(), None)
        rec(1)
        rc |= L.hctr_p2p_owner_apply(c, mb, 0, self.ent_row.data_ptr(), self.mask.data_ptr(), self.head.data_ptr(),
                                     self.ent_next.data_ptr(), self.emb.data_ptr(), None)
        rec(2)
        rc |= L.hctr_p2p_stale_gather(c, self.seq, self.row_of.data_ptr(), self.length, 0, self.emb.data_ptr(),
                                      self.version.data_ptr(), pull_bound, None)
        rec(3)
        assert rc == 0, "launch failed"

    # -- numpy evaluation of the same step: sources one after the other (csrc/core/handle_query.cu:106-116, 7-40) --
    def expected(self, emb0, ver0, pull_bound=0):
        emb, ver = emb0.copy(), ver0.copy()
        for s in range(self.n):
            rows = self.row_of_h[self.push_keys[s]]
            ver[rows] += self.push_upd[s]
            emb[rows] += self.push_val[s]
        flags, ret_rows = [], []
        imin = np.iinfo(np.int64).min
        for s in range(self.n):
            rows = self.row_of_h[self.query_keys[s]]
            lv, gv = self.query_ver[s], ver[rows]
            with np.errstate(over="ignore"):
                stale = (lv == imin) | (lv + pull_bound < gv)
            f = stale & (s != self.rank)
            flags.append(f)
            ret_rows.append(rows[f])
        return emb, ver, flags, ret_rows

    def check(self):
        emb0, ver0 = self.emb.cpu().numpy(), self.version.cpu().numpy()
        self.publish()
        self.step()
        self.torch.cuda.synchronize()
        assert int(self.err[0]) == 0, f"device error word {int(self.err[0])}"
        emb, ver, flags, ret_rows = self.expected(emb0, ver0)
        assert np.array_equal(self.version.cpu().numpy(), ver), "versions differ"
        assert np.array_equal(self.emb.cpu().numpy(), emb), "rows differ (source order?)"
        cap, n = self.cap, self.n
        assert int(self.cnt_in[5 * n + 6]) == sum(len(r) for r in ret_rows), "number of returned rows differs"
        base = self.rank * cap
        for s in range(n):
            if s == self.rank:
                continue
            box = self.peers[s]
            q = len(self.query_keys[s])
            hdr = box["hdr"].cpu().numpy().reshape(n, 16)[self.rank]
            assert hdr[8] == self.seq, f"source {s}: phase-1 sequence number"
            f = flags[s]
            assert np.array_equal(box["flag"].cpu().numpy()[base:base + q], f.astype(np.uint8)), "flags"
            # the row for the j-th query sits at row j of this rank's sub-region, when the key was stale
            rows = self.row_of_h[self.query_keys[s]]
            assert np.array_equal(box["rval"].cpu().numpy()[base:base + q][f], emb[rows[f]]), "returned rows differ"
            assert np.array_equal(box["rver"].cpu().numpy()[base:base + q][f], ver[rows[f]]), "returned versions"
        return True

    def time(self, iters=20):
        torch = self.torch
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(iters)]
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.dev)
        for i in range(3):
            self.publish()
            self.step()
        for i in range(iters):
            self.publish()
            flush.fill_(i & 1)  # evict the 126 MB L2 between iterations
            torch.cuda.synchronize()
            self.step(events=ev[i])
        torch.cuda.synchronize()
        names = ["owner_mark", "owner_apply", "stale_gather"]
        us = {nm: 1e3 * float(np.median([ev[i][j].elapsed_time(ev[i][j + 1]) for i in range(iters)]))
              for j, nm in enumerate(names)}
        G = sum(len(k) for k in self.push_keys)
        Q = sum(len(k) for k in self.query_keys)
        R = int(self.cnt_in[5 * self.n + 6])
        D = 4 * self.W
        rows_touched = len(np.unique(np.concatenate(self.push_keys))) if G else 0
        alg = {"owner_mark": G * (8 + 8 + 4 + 4 + 16 + 16 + 12), "owner_apply": G * D + rows_touched * 2 * D + G * 16,
               "stale_gather": Q * (16 + 4 + 8 + 1) + R * (2 * D + 8)}
        return {"pushed_rows": G, "distinct_pushed_rows": rows_touched, "queries": Q, "returned_rows": R,
                "us": us, "algorithmic_bytes": alg,
                "gbs": {k: (alg[k] / (us[k] * 1e-6) / 1e9 if us[k] > 0 else 0.0) for k in names}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sources", type=int, default=8)
    ap.add_argument("--rows", type=int, default=4_200_000)
    ap.add_argument("--width", type=int, default=128)
    ap.add_argument("--pushed", type=int, default=68_000)
    ap.add_argument("--queries", type=int, default=77_000)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--cap", type=int, default=0,
                    help="rows per mailbox sub-region (a table uses its batch size; it sizes the grids); with a cap "
                         "the peers' stand-in mailboxes are one shared allocation and --check is not available")
    a = ap.parse_args()
    assert not (a.cap and a.check), "--check needs one stand-in mailbox per peer: leave --cap out"
    r = OwnerReplay(a.sources, a.rows, a.width, a.pushed, a.queries, cap=a.cap, shared_peer=a.cap > 0)
    if a.check:
        r.check()
        print("check ok: versions and rows equal a source-by-source numpy evaluation")
    print(json.dumps(r.time(a.iters)))


if __name__ == "__main__":
    main()
