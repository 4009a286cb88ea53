"""Replays the REQUESTER side of one step of the peer-to-peer exchange on a single GPU, from synthetic traffic.

  python -m hetuctr_b200.requester_replay [--ranks 8] [--batch 212992] [--unique 78000] [--width 128]
                                          [--owned-rows 500000] [--iters 20] [--check] [--cap 212992]

After the owners have answered, a rank of a multi-GPU job runs ONE kernel (hctr_p2p_refresh_expand): it waits for the
owners' sequence numbers, refreshes its cached rows from the returned ones and writes the pulled row of every batch
position.  To time or profile that kernel in isolation this tool builds one rank's state on one GPU - a table shard
(cached rows first, then owned rows), a batch whose unique keys are ordered (owner, key) with Zipf-distributed
duplicates, and a mailbox filled the way the owners would have filled it (a flag per query, returned row + version
where the flag is set) - and launches the kernel through the kernel-level C-ABI (include/hctr_kernels.h).
`--check` compares dst, the refreshed cache rows and their versions with a numpy evaluation of
update_cache_kernel + write_back_kernel (csrc/core/writeback.cu:8-71).  Everything is local memory: the figures are
the kernel's HBM-side cost.
"""
import argparse
import ctypes
import json

import numpy as np

from .owner_replay import Box, Ctx, cnt_words

vp = ctypes.c_void_p
META_WORDS = 4  # HCTR_META_WORDS: unique count, error word, long-run count, -, then the per-owner segment starts


class RequesterReplay:
    def __init__(self, ranks=8, batch=212_992, unique=78_000, width=128, owned_rows=500_000, cached_share=0.25,
                 flagged_share=0.7, alpha=1.05, seed=0, device=0, cap=0):
        import torch

        import hetuctr_b200 as hb
        self.torch, self.L = torch, hb.lib()
        self.dev = dev = torch.device("cuda", device)
        torch.cuda.set_device(dev)
        n, B, U, W = ranks, batch, unique, width
        self.n, self.B, self.U, self.W, self.rank = n, B, U, W, 0
        rng = np.random.RandomState(seed)
        # unique keys in (owner, key) order: only the owner of each matters here
        owner = np.sort(rng.randint(n, size=U)).astype(np.uint8)
        seg = np.searchsorted(owner, np.arange(n + 1)).astype(np.uint32)
        # popularity: bounded Zipf over a random order of the unique keys; every key occurs at least once
        weight = 1.0 / np.arange(1, U + 1) ** alpha
        weight = weight[rng.permutation(U)]
        idx_map = np.concatenate([np.arange(U), rng.choice(U, size=max(B - U, 0), p=weight / weight.sum())])[:B]
        idx_map = idx_map[rng.permutation(len(idx_map))].astype(np.int32)
        # the hottest keys other ranks own are cached here; this rank's own keys have owned rows; the rest is not stored
        mine = owner == self.rank
        other = np.where(~mine)[0]
        cached = other[np.argsort(-weight[other])[:int(len(other) * cached_share)]]
        C = len(cached)
        S = C + owned_rows
        uniq_row = np.full(U, -1, dtype=np.int32)
        uniq_row[cached] = rng.permutation(C).astype(np.int32)
        uniq_row[mine] = (C + rng.choice(owned_rows, size=int(mine.sum()), replace=False)).astype(np.int32)
        self.C, self.S = C, S
        per_owner = np.diff(seg.astype(np.int64))
        self.cap = cap = int(max(cap, per_owner.max(), 1))
        # what the owners answered: non-stored keys are always returned, cached keys when stale, own keys never
        slot = owner.astype(np.int64) * cap + (np.arange(U) - seg[owner])
        flag_u = np.zeros(U, dtype=bool)
        flag_u[(uniq_row < 0)] = True
        flag_u[cached] = rng.rand(C) < flagged_share
        self.h = dict(owner=owner, seg=seg, idx_map=idx_map, uniq_row=uniq_row, slot=slot, flag_u=flag_u,
                      pos_row=uniq_row[idx_map])

        def t(a):
            return torch.from_numpy(a).to(dev)

        self.uniq_owner, self.uniq_row, self.idx_map = t(owner), t(uniq_row), t(idx_map)
        self.pos_row = t(self.h["pos_row"])
        meta = np.zeros(META_WORDS + n + 1, dtype=np.uint32)
        meta[0] = U
        meta[META_WORDS:] = seg
        self.meta = t(meta)
        self.emb = torch.randn(S, W, device=dev) * 0.1
        self.pending = torch.randn(max(C, 1), W, device=dev) * 0.01
        self.version = torch.randint(0, 50, (S,), dtype=torch.int64, device=dev)
        slots = n * cap
        self.box = dict(hdr=torch.zeros(n * 16, dtype=torch.int32, device=dev),
                        flag=torch.zeros(slots, dtype=torch.uint8, device=dev),
                        rver=torch.zeros(slots, dtype=torch.int64, device=dev),
                        rval=torch.zeros(slots, W, device=dev))
        self.box["flag"][t(slot[flag_u])] = 1
        self.box["rver"][t(slot[flag_u])] = torch.randint(50, 90, (int(flag_u.sum()),), dtype=torch.int64, device=dev)
        self.box["rval"][t(slot[flag_u])] = torch.randn(int(flag_u.sum()), W, device=dev) * 0.1
        # slots the owners did not write keep whatever an earlier step left there: make sure nobody reads them
        self.box["rval"][t(slot[~flag_u])] = float("nan")
        b = Box()
        for f, _ in Box._fields_:
            setattr(b, f, self.box[f].data_ptr() if f in self.box else 0)
        boxes = (Box * n)(*([b] * n))
        self.d_boxes = torch.frombuffer(bytearray(bytes(boxes)), dtype=torch.uint8).to(dev)
        self.cnt_in = torch.zeros(cnt_words(n), dtype=torch.int32, device=dev)
        self.err = torch.zeros(4, dtype=torch.int32, device=dev)
        self.ctx = Ctx(n, self.rank, cap, W, self.d_boxes.data_ptr(), self.cnt_in.data_ptr(), self.err.data_ptr(),
                       int(50e6))
        self.dst = torch.full((B, W), float("nan"), device=dev)
        self.seq = 0
        u32, sz = ctypes.c_uint32, ctypes.c_size_t
        self.L.hctr_p2p_refresh_expand.argtypes = [vp, u32, vp, vp, vp, sz, vp, vp, vp, sz, vp, vp, vp, vp]

    def publish(self):
        """What the owners' last thread blocks do: returned-row count + sequence number into this rank's headers."""
        self.seq += 1
        h = self.box["hdr"].view(self.n, 16)
        h[:, 9] = 0
        h[:, 8] = self.seq
        self.cnt_in[2 * self.n] = 0  # the kernel that waits for the queries clears this statistics word in a real step
        self.torch.cuda.synchronize()

    def step(self):
        rc = self.L.hctr_p2p_refresh_expand(ctypes.byref(self.ctx), self.seq, self.meta.data_ptr(),
                                            self.uniq_owner.data_ptr(), self.uniq_row.data_ptr(), self.C,
                                            self.pending.data_ptr(), self.emb.data_ptr(), self.version.data_ptr(),
                                            self.B, self.pos_row.data_ptr(), self.idx_map.data_ptr(),
                                            self.dst.data_ptr(), None)
        assert rc == 0, "launch failed"

    def expected(self, emb0, ver0):
        h = self.h
        rval, rver = self.box["rval"].cpu().numpy(), self.box["rver"].cpu().numpy()
        pending = self.pending.cpu().numpy()
        row, slot, f = h["uniq_row"], h["slot"], h["flag_u"]
        emb, ver = emb0.copy(), ver0.copy()
        refresh = f & (row >= 0) & (row < self.C)
        emb[row[refresh]] = rval[slot[refresh]] + pending[row[refresh]]
        ver[row[refresh]] = rver[slot[refresh]]
        # pulled rows: table row (owned, or cached and not flagged), returned row (not stored), refreshed row
        u = h["idx_map"]
        dst = np.where((row[u] >= 0)[:, None], emb[np.maximum(row[u], 0)], rval[slot[u]])
        return emb, ver, dst, int(f.sum())

    def check(self):
        emb0, ver0 = self.emb.cpu().numpy(), self.version.cpu().numpy()
        self.publish()
        self.step()
        self.torch.cuda.synchronize()
        assert int(self.err[0]) == 0, f"device error word {int(self.err[0])}"
        emb, ver, dst, flagged = self.expected(emb0, ver0)
        assert np.array_equal(self.dst.cpu().numpy(), dst), "pulled rows differ"
        assert np.array_equal(self.emb.cpu().numpy(), emb), "refreshed cache rows differ"
        assert np.array_equal(self.version.cpu().numpy(), ver), "versions differ"
        assert int(self.cnt_in[2 * self.n]) == flagged, "number of flagged keys differs"
        return True

    def time(self, iters=20):
        torch = self.torch
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(iters)]
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.dev)
        for i in range(3):
            self.publish()
            self.step()
        for i in range(iters):
            self.publish()
            flush.fill_(i & 1)  # evict the 126 MB L2 between iterations
            torch.cuda.synchronize()
            ev[i][0].record()
            self.step()
            ev[i][1].record()
        torch.cuda.synchronize()
        us = 1e3 * float(np.median([a.elapsed_time(b) for a, b in ev]))
        h = self.h
        D = 4 * self.W
        refreshed = int((h["flag_u"] & (h["uniq_row"] >= 0) & (h["uniq_row"] < self.C)).sum())
        alg = 3 * D * refreshed + 14 * self.U + self.U * D + self.B * D + 8 * self.B
        pos = h["pos_row"]
        return {"batch": self.B, "unique": self.U, "cached_keys": self.C, "refreshed_rows": refreshed,
                "positions": {"owned": int((pos >= self.C).sum()), "cached": int(((pos >= 0) & (pos < self.C)).sum()),
                              "not_stored": int((pos < 0).sum())},
                "us": us, "algorithmic_bytes": alg, "gbs": alg / (us * 1e-6) / 1e9 if us > 0 else 0.0}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=8)
    ap.add_argument("--batch", type=int, default=212_992)
    ap.add_argument("--unique", type=int, default=78_000)
    ap.add_argument("--width", type=int, default=128)
    ap.add_argument("--owned-rows", type=int, default=500_000)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--cap", type=int, default=0, help="rows per mailbox sub-region (a table uses its batch size)")
    a = ap.parse_args()
    r = RequesterReplay(a.ranks, a.batch, a.unique, a.width, a.owned_rows, cap=a.cap)
    if a.check:
        r.check()
        print("check ok: pulled rows, refreshed cache rows and versions equal the numpy evaluation")
        r = RequesterReplay(a.ranks, a.batch, a.unique, a.width, a.owned_rows, cap=a.cap)
    print(json.dumps(r.time(a.iters)))


if __name__ == "__main__":
    main()
