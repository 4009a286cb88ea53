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
                ("side_stream", vp), ("fork_event", vp), ("join_event", vp)]


@pytest.mark.parametrize("nrank", [1, 3])
def test_dedupe_launcher_standalone(nrank):
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
                       side_stream=None, fork_event=None, join_event=None,
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
