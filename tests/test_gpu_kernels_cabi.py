"""Kernel-level C-ABI (include/hctr_kernels.h) called directly, without the table object: the dedupe launcher on
caller-owned buffers and a single stream (no side stream, no events), checked against numpy; repeated calls prove
that the persistent scratch comes back all-zero and that the epoch-tagged scratch needs no clearing."""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

import hetuctr_b200 as hb  # noqa: E402

vp, sz, u32 = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint32


class DedupeArgs(ctypes.Structure):  # field order of hctr_dedupe_args
    _fields_ = [("keys", vp), ("batch", sz), ("length", sz), ("length_pad", sz), ("nrank", ctypes.c_int),
                ("owner_of", vp), ("row_of", vp), ("bits", vp), ("blk_flag", vp), ("cnt", vp),
                ("chain_scratch", vp), ("scan_scratch", vp), ("epoch", u32), ("word_base", vp), ("sk", vp),
                ("rank_in_run", vp), ("uniq", vp), ("uniq_owner", vp), ("uniq_row", vp), ("run_start", vp),
                ("sorted_pos", vp), ("idx_map", vp), ("pos_row", vp), ("heavy_list", vp), ("meta", vp),
                ("side_stream", vp), ("fork_event", vp), ("join_event", vp), ("stride", u32)]


@pytest.mark.parametrize("stride", [0, 7, 26])
@pytest.mark.parametrize("nrank", [1, 3])
def test_dedupe_launcher_standalone(nrank, stride):
    L = hb.lib()
    L.hctr_dedupe_map.argtypes = [ctypes.POINTER(DedupeArgs), vp]
    L.hctr_scan_chained_scratch_words.restype = sz
    L.hctr_scan_chained_scratch_words.argtypes = [sz]
    dev = torch.device("cuda:0")
    N, B = 50_000, 30_000
    n_pad = (N + 4095) // 4096 * 4096
    words, blocks = nrank * n_pad // 64, nrank * n_pad // 4096
    rng = np.random.RandomState(nrank)
    owner = rng.randint(nrank, size=N).astype(np.uint8)
    row_of = rng.permutation(N).astype(np.int32)
    row_of[rng.rand(N) < 0.3] = -1

    def z(n, dt):
        return torch.zeros(max(int(n), 1), dtype=dt, device=dev)

    t = dict(owner_of=torch.from_numpy(owner).to(dev), row_of=torch.from_numpy(row_of).to(dev),
             bits=z(words, torch.int64), blk_flag=z(blocks + 1, torch.uint8), cnt=z(B + 1, torch.int32),
             chain_scratch=z(2 * (blocks // 8 + 2), torch.int32),
             scan_scratch=z(L.hctr_scan_chained_scratch_words(B + 1), torch.int32), word_base=z(words, torch.int32),
             sk=z(B, torch.int64), rank_in_run=z(B, torch.int32), uniq=z(B, torch.int64), uniq_owner=z(B, torch.uint8),
             uniq_row=z(B, torch.int32), run_start=z(B + 1, torch.int32), sorted_pos=z(B, torch.int32),
             idx_map=z(B, torch.int32), pos_row=z(B, torch.int32), heavy_list=z(B // 32 + 2, torch.int32),
             meta=z(4 + nrank + 1, torch.int32))
    for epoch in (1, 2, 3):
        keys = (rng.zipf(1.2, size=B) - 1 + rng.randint(N)) % N
        if epoch == 2:
            keys[: B // 3] = keys[0]  # one very long run
        kd = torch.from_numpy(keys.astype(np.int64)).to(dev)
        t["meta"].zero_()
        a = DedupeArgs(keys=kd.data_ptr(), batch=B, length=N, length_pad=n_pad, nrank=nrank, epoch=epoch,
                       side_stream=None, fork_event=None, join_event=None, stride=stride,
                       **{k: v.data_ptr() for k, v in t.items()})
        assert L.hctr_dedupe_map(ctypes.byref(a), None) == 0
        torch.cuda.synchronize()
        meta = t["meta"].cpu().numpy()
        U = int(meta[0])
        assert meta[1] == 0
        # expected: unique keys ordered by (owner, key)
        uk = np.unique(keys)
        order = np.lexsort((uk, owner[uk]))
        exp_uniq = uk[order]
        assert U == len(exp_uniq)
        uniq = t["uniq"].cpu().numpy()[:U]
        assert np.array_equal(uniq, exp_uniq)
        assert np.array_equal(t["uniq_owner"].cpu().numpy()[:U], owner[exp_uniq])
        assert np.array_equal(t["uniq_row"].cpu().numpy()[:U], row_of[exp_uniq])
        seg = meta[4:4 + nrank + 1]
        assert np.array_equal(seg, np.searchsorted(owner[exp_uniq], np.arange(nrank + 1)))
        idx_map = t["idx_map"].cpu().numpy()
        assert np.array_equal(uniq[idx_map], keys)
        assert np.array_equal(t["pos_row"].cpu().numpy(), row_of[keys])
        runs = t["run_start"].cpu().numpy()[:U + 1].astype(np.int64)
        pos = t["sorted_pos"].cpu().numpy().astype(np.int64)
        exp_pos = np.argsort(idx_map, kind="stable")  # grouped by unique, ascending positions inside a group
        assert np.array_equal(pos, exp_pos)
        assert np.array_equal(np.diff(runs), np.bincount(idx_map, minlength=U))
        assert int(meta[2]) == int(np.sum(np.diff(runs) > 32))
        # persistent scratch is all-zero again
        assert int(t["bits"].abs().sum()) == 0 and int(t["blk_flag"].sum()) == 0 and int(t["cnt"].abs().sum()) == 0


def _expand_inputs(rng, batch, width, n_rows, n_recv, dev):
    emb = rng.normal(size=(n_rows, width)).astype(np.float32)
    recv = rng.normal(size=(n_recv, width)).astype(np.float32)
    pos_row = rng.randint(n_rows, size=batch).astype(np.int32)
    idx_map = rng.randint(n_recv, size=batch).astype(np.int32)
    recv_slot = rng.permutation(n_recv).astype(np.uint32)
    remote = rng.rand(batch) < 0.3
    pos_row[remote] = -1
    bad = rng.rand(batch) < 0.02  # out-of-range keys: no row, no unique index -> zeros
    pos_row[bad] = -1
    idx_map[bad] = -1
    exp = np.where(pos_row[:, None] >= 0, emb[np.maximum(pos_row, 0)], recv[recv_slot[np.maximum(idx_map, 0)]])
    exp[bad] = 0
    t = [torch.from_numpy(x).to(dev) for x in (pos_row, idx_map, recv_slot.view(np.int32), recv, emb)]
    return t, exp.astype(np.float32)


@pytest.mark.parametrize("width", [32, 64, 128, 256, 1024])
@pytest.mark.parametrize("batch", [1, 37, 5000])
def test_expand_launchers_agree(width, batch):
    """Register kernel and bulk-copy kernel of the row expansion on caller-owned buffers, against numpy."""
    L = hb.lib()
    L.hctr_expand_rows.argtypes = [sz, sz, vp, vp, vp, vp, vp, vp, vp]
    L.hctr_expand_rows_bulk.argtypes = [sz, sz, vp, vp, vp, vp, vp, vp, vp, vp]
    dev = torch.device("cuda:0")
    rng = np.random.RandomState(width + batch)
    (pos_row, idx_map, recv_slot, recv, emb), exp = _expand_inputs(rng, batch, width, 3000, 700, dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    for bulk in (False, True):
        dst = torch.full((batch, width), float("nan"), device=dev)
        if bulk:
            rc = L.hctr_expand_rows_bulk(batch, width, pos_row.data_ptr(), idx_map.data_ptr(), recv_slot.data_ptr(),
                                         recv.data_ptr(), emb.data_ptr(), dst.data_ptr(), err.data_ptr(), None)
        else:
            rc = L.hctr_expand_rows(batch, width, pos_row.data_ptr(), idx_map.data_ptr(), recv_slot.data_ptr(),
                                    recv.data_ptr(), emb.data_ptr(), dst.data_ptr(), None)
        assert rc == 0
        torch.cuda.synchronize()
        assert int(err.item()) == 0
        assert np.array_equal(dst.cpu().numpy(), exp), f"bulk={bulk}"


@pytest.mark.parametrize("width", [128, 32, 6])
@pytest.mark.parametrize("in_host_memory", [False, True])
def test_expand_subset_halves_cover_every_position_once(width, in_host_memory):
    """hctr_expand_rows_subset: the positions whose key is / is not among the previous batch's unique keys.  Each half
    writes exactly its own rows (the others keep the fill value), together they equal the plain expansion; dst may
    be pinned host memory."""
    L = hb.lib()
    L.hctr_expand_rows_subset.argtypes = [sz, sz, vp, vp, vp, vp, ctypes.c_int, vp, vp, vp]
    dev = torch.device("cuda:0")
    rng = np.random.RandomState(width)
    n_rows, batch = 4000, 5000
    keys = rng.randint(n_rows, size=batch).astype(np.int64)
    prev_uniq = np.unique(rng.randint(n_rows, size=1500)).astype(np.int64)  # ascending
    pos_row = keys.astype(np.int32)  # single rank: row = key here
    pos_row[7] = -1  # a position without a row gets zeros from the half that owns it
    emb = rng.normal(size=(n_rows, width)).astype(np.float32)
    meta = np.zeros(8, dtype=np.uint32)
    meta[0] = len(prev_uniq)
    # more entries behind the announced count must be ignored
    padded = np.concatenate([prev_uniq, np.full(64, n_rows + 5, dtype=np.int64)])
    t = lambda a: torch.from_numpy(a).to(dev)  # noqa: E731
    d_keys, d_prev, d_pos, d_emb, d_meta = t(keys), t(padded), t(pos_row), t(emb), t(meta)
    in_prev = np.isin(keys, prev_uniq)
    want = emb[keys]
    want[7] = 0.0
    fill = np.float32(-7.5)
    outs = []
    for half in (0, 1):
        dst = torch.full((batch, width), float(fill))
        dst = dst.pin_memory() if in_host_memory else dst.to(dev)
        assert L.hctr_expand_rows_subset(batch, width, d_pos.data_ptr(), d_keys.data_ptr(), d_prev.data_ptr(),
                                         d_meta.data_ptr(), half, d_emb.data_ptr(), dst.data_ptr(), None) == 0
        torch.cuda.synchronize()
        got = dst.cpu().numpy()
        mine = in_prev == bool(half)
        assert np.array_equal(got[mine], want[mine])
        assert np.all(got[~mine] == fill)
        outs.append((mine, got))
    assert np.all(outs[0][0] ^ outs[1][0])


@pytest.mark.parametrize("ranks,width", [(4, 128), (2, 32), (8, 6), (3, 260)])
def test_requester_side_kernel_on_synthetic_mailbox(ranks, width):
    """hctr_p2p_refresh_expand on one rank's synthetic state (owned, cached and not-stored keys, a mailbox filled as
    the owners would): pulled rows, refreshed cache rows, versions and the flagged count against numpy."""
    from hetuctr_b200.requester_replay import RequesterReplay

    r = RequesterReplay(ranks=ranks, batch=6000, unique=2500, width=width, owned_rows=5000, seed=ranks + width)
    assert r.check()
    pos = r.h["pos_row"]
    assert (pos >= r.C).any() and ((pos >= 0) & (pos < r.C)).any() and (pos < 0).any()


def test_ingest_keys_and_deferred_ordering():
    """hctr_ingest_keys (copy + cleared meta in one launch) and the split pipeline: hctr_dedupe_map without the
    run ordering (fork event only), hctr_dedupe_order later on another stream."""
    L = hb.lib()
    L.hctr_ingest_keys.argtypes = [vp, vp, sz, vp, ctypes.c_uint, vp]
    L.hctr_dedupe_map.argtypes = [ctypes.POINTER(DedupeArgs), vp]
    L.hctr_dedupe_order.argtypes = [ctypes.POINTER(DedupeArgs), vp]
    L.hctr_scan_chained_scratch_words.restype = sz
    L.hctr_scan_chained_scratch_words.argtypes = [sz]
    dev = torch.device("cuda:0")
    N, B = 20_000, 9_000
    n_pad = (N + 4095) // 4096 * 4096
    words, blocks = n_pad // 64, n_pad // 4096
    rng = np.random.RandomState(3)
    keys = (rng.zipf(1.15, size=B) - 1) % N
    keys[:2000] = 77  # a long run
    user = torch.from_numpy(keys.astype(np.int64)).to(dev)

    def z(n, dt):
        return torch.zeros(max(int(n), 1), dtype=dt, device=dev)

    private = z(B, torch.int64)
    meta = torch.full((6,), 123, dtype=torch.int32, device=dev)
    assert L.hctr_ingest_keys(user.data_ptr(), private.data_ptr(), B, meta.data_ptr(), 6, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(private, user) and int(meta.abs().sum()) == 0

    t = dict(owner_of=z(N, torch.uint8), row_of=torch.arange(N, dtype=torch.int32, device=dev),
             bits=z(words, torch.int64), blk_flag=z(blocks + 1, torch.uint8), cnt=z(B + 1, torch.int32),
             chain_scratch=z(2 * (blocks // 8 + 2), torch.int32),
             scan_scratch=z(L.hctr_scan_chained_scratch_words(B + 1), torch.int32), word_base=z(words, torch.int32),
             sk=z(B, torch.int64), rank_in_run=z(B, torch.int32), uniq=z(B, torch.int64), uniq_owner=z(B, torch.uint8),
             uniq_row=z(B, torch.int32), run_start=z(B + 1, torch.int32), sorted_pos=z(B, torch.int32),
             idx_map=z(B, torch.int32), pos_row=z(B, torch.int32), heavy_list=z(B // 32 + 2, torch.int32), meta=meta)
    side = torch.cuda.Stream(device=dev)
    fork = torch.cuda.Event()
    fork.record()  # creates the underlying event handle
    a = DedupeArgs(keys=private.data_ptr(), batch=B, length=N, length_pad=n_pad, nrank=1, epoch=1,
                   side_stream=side.cuda_stream, fork_event=fork.cuda_event, join_event=None,
                   **{k: v.data_ptr() for k, v in t.items()})
    assert L.hctr_dedupe_map(ctypes.byref(a), None) == 0  # ordering NOT enqueued, fork event recorded
    side.wait_event(fork)
    assert L.hctr_dedupe_order(ctypes.byref(a), side.cuda_stream) == 0
    torch.cuda.synchronize()
    idx_map = t["idx_map"].cpu().numpy()
    assert np.array_equal(t["sorted_pos"].cpu().numpy().astype(np.int64), np.argsort(idx_map, kind="stable"))


@pytest.mark.parametrize("sources,width,rows", [(8, 128, 5000), (4, 32, 3000), (32, 8, 800), (3, 132, 2000), (2, 64, 1000)])
def test_owner_side_kernels_on_synthetic_mailbox(sources, width, rows):
    """hctr_p2p_owner_mark / _apply / _stale_scan / _gather on a mailbox filled the way `sources - 1` peers would
    fill it (hot rows pushed by many of them), against numpy applying the sources one after the other."""
    from hetuctr_b200.owner_replay import OwnerReplay
    r = OwnerReplay(sources, rows, width, pushed=rows * 2, queries=rows * 3, alpha=1.05, seed=sources)
    distinct = len(np.unique(np.concatenate(r.push_keys)))
    assert sources == 2 or sum(len(k) for k in r.push_keys) > distinct  # several pushers per row do occur
    assert r.check()
    assert r.check()  # a second step on the same scratch: epochs, tickets and sequence numbers move on
