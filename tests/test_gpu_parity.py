"""GPU parity: the CUDA path (through the C-ABI) against the CPU oracle on the same seeded inputs.

Index arrays (unique keys, owner/row maps, batch->unique map, position lists, per-owner counts), versions and
pending-update counts must be bit-exact.  Row values: the kernels sum duplicate gradients in batch order and
apply pushed rows source by source like the reference, so they are compared bit-exactly as well; the
tolerance the task allows (1e-5 relative) is only needed against the reference's own build.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

import hetuctr_b200 as hb  # noqa: E402
from gpu_world import GpuWorld, assert_index_parity, assert_state_parity  # noqa: E402


def make_worlds(oracle_mod, nrank, length, width, pull, push, lr, root, storage, seed=0, **kw):
    ow = oracle_mod.World(nrank, length, width, pull, push, lr, root, storage)
    gw = GpuWorld(nrank, length, width, pull, push, lr, root, storage, **kw)
    rng = np.random.RandomState(seed)
    for r in range(nrank):
        n = ow.get(r, "storage")
        emb = rng.normal(0, 0.01, size=(n, width)).astype(np.float32)
        ow.set_embedding(r, emb)
        gw.set_embedding(r, emb)
        assert np.array_equal(gw.get(r, "stored_keys"), ow.get(r, "stored_keys"))
        assert gw.get(r, "nonlocal") == ow.get(r, "nonlocal")
        assert np.array_equal(gw.get(r, "version"), ow.get(r, "version"))
    return gw, ow


def run_steps(gw, ow, batches, grads, exact=True):
    """batches[s][r] keys; grads[s][r] gradient for batches[s-1][r] (None => inference)."""
    for s, keys in enumerate(batches):
        gw.preprocess(keys)
        ow.preprocess(keys)
        assert_index_parity(gw, ow)
        dg = gw.push_pull(grads[s])
        do = ow.push_pull(grads[s])
        for r in range(gw.nrank):
            if exact:
                assert np.array_equal(dg[r], do[r]), f"step {s} rank {r}: pulled rows differ"
            else:
                np.testing.assert_allclose(dg[r], do[r], rtol=1e-5, atol=1e-6)
        assert_state_parity(gw, ow, exact=exact)


def test_config1_plumbing(oracle_mod):
    # BASELINE config 1: 1 rank, 100,000 x 16, batch 1024 x 26 uniform keys, N(0,0.01) grads, lr 0.1, 10 steps
    N, W, B = 100_000, 16, 1024 * 26
    root = np.zeros(N, dtype=np.uint8)
    gw, ow = make_worlds(oracle_mod, 1, N, W, 0, 0, 0.1, root, [np.arange(N)])
    rng = np.random.RandomState(1)
    batches = [[rng.randint(N, size=B)] for _ in range(10)]
    grads = [None] + [[rng.normal(0, 0.01, size=(B, W)).astype(np.float32)] for _ in range(9)]
    run_steps(gw, ow, batches, grads)
    gw.close()


@pytest.mark.parametrize("width", [1, 3, 4, 8, 20, 32, 64, 100, 128, 132, 256, 512, 516, 1024, 1100])
def test_single_rank_widths(oracle_mod, width):
    N, B = 5000, 3000
    root = np.zeros(N, dtype=np.uint8)
    perm = np.random.RandomState(5).permutation(N)  # storage order != key order
    gw, ow = make_worlds(oracle_mod, 1, N, width, 0, 0, 0.05, root, [perm])
    rng = np.random.RandomState(width)
    batches = [[(rng.zipf(1.3, size=B) - 1) % N] for _ in range(4)]
    grads = [None] + [[rng.normal(0, 1, size=(B, width)).astype(np.float32)] for _ in range(3)]
    run_steps(gw, ow, batches, grads)
    gw.close()


def test_heavy_duplicates_and_long_runs(oracle_mod):
    # few distinct keys => runs far longer than a warp; exercises the long-run ordering path
    N, W = 4096 * 3 + 17, 8
    root = np.zeros(N, dtype=np.uint8)
    gw, ow = make_worlds(oracle_mod, 1, N, W, 0, 0, 1.0, root, [np.arange(N)])
    rng = np.random.RandomState(2)
    b0 = rng.choice([3, N - 1, 4096, 4095, 700], size=20000)
    b1 = np.full(5000, 12345 % N)
    b2 = np.concatenate([rng.randint(N, size=3000), np.full(40, 9), np.full(33, 10), np.full(32, 11)])
    rng.shuffle(b2)
    batches = [[b0], [b1], [b2], [b0[:7]]]
    grads = [None] + [[rng.normal(0, 1, size=(len(b[0]), W)).astype(np.float32)] for b in batches[:-1]]
    run_steps(gw, ow, batches, grads)
    gw.close()


def test_batch_larger_than_one_ordering_window(oracle_mod):
    # > 2^20 positions with a hot key: the long-run path walks several shared-memory windows
    N, W, B = 50_000, 4, (1 << 20) + 4099
    root = np.zeros(N, dtype=np.uint8)
    gw, ow = make_worlds(oracle_mod, 1, N, W, 0, 0, 0.5, root, [np.arange(N)])
    rng = np.random.RandomState(3)
    keys = rng.randint(N, size=B)
    keys[rng.rand(B) < 0.05] = 77
    batches = [[keys], [keys[:10]]]
    grads = [None, [rng.normal(0, 1, size=(B, W)).astype(np.float32)]]
    run_steps(gw, ow, batches, grads)
    gw.close()


def test_edge_cases_empty_repeat_inference_host_keys(oracle_mod):
    N, W = 1000, 16
    root = np.zeros(N, dtype=np.uint8)
    gw, ow = make_worlds(oracle_mod, 1, N, W, 0, 0, 0.1, root, [np.arange(N)], keys_on_device=False)
    rng = np.random.RandomState(4)
    e = np.zeros(0, dtype=np.int64)
    k1, k2, k3 = rng.randint(N, size=10), rng.randint(N, size=500), rng.randint(N, size=300)
    g = lambda k: rng.normal(0, 1, size=(len(k), W)).astype(np.float32)  # noqa: E731
    # empty batch; preprocess twice in a row (older batch's gradient is never pushed); inference step
    for w in (gw, ow):
        w.preprocess([e])
    assert_index_parity(gw, ow)
    for w in (gw, ow):
        w.preprocess([k1])
        w.preprocess([k1])
    run_steps(gw, ow, [[k2], [k3], [e], [k1]], [[g(k1)], None, [g(k3)], [g(e)]])
    gw.close()


@pytest.mark.parametrize("buffers", ["pinned", "pageable"])
@pytest.mark.parametrize("width", [128, 16, 6])
def test_single_rank_host_gradients_and_rows(oracle_mod, buffers, width):
    # gradients and pulled rows in host memory.  With pinned memory the rows whose keys the previous batch did not
    # contain are written before the gradients are applied and the others after: consecutive batches here share
    # about half of their keys, contain duplicates, and one step is an inference step, one batch is empty.
    N, B = 5000, 3000
    root = np.zeros(N, dtype=np.uint8)
    gw, ow = make_worlds(oracle_mod, 1, N, width, 0, 0, 0.1, root, [np.arange(N)], buffers=buffers,
                         keys_on_device=False)
    rng = np.random.RandomState(21)
    hot = rng.randint(N, size=400)
    e = np.zeros(0, dtype=np.int64)

    def batch(n):
        k = rng.randint(N, size=n)
        m = rng.rand(n) < 0.5
        k[m] = hot[rng.randint(len(hot), size=int(m.sum()))]
        return k

    sizes = [B, B, 700, B, 0, B, B, 40, B]
    batches = [[batch(n) if n else e] for n in sizes]
    grads = [None] + [[rng.normal(0, 1, size=(sizes[i - 1], width)).astype(np.float32)] for i in range(1, len(sizes))]
    grads[4] = None  # inference step: batch 3's gradient is never applied
    run_steps(gw, ow, batches, grads)
    gw.close()


def test_out_of_range_key_raises_and_table_recovers(oracle_mod):
    N, W = 300, 4
    root = np.zeros(N, dtype=np.uint8)
    gw, ow = make_worlds(oracle_mod, 1, N, W, 0, 0, 0.1, root, [np.arange(N)])
    # the key ingest checks the range and preprocess reports it; the batch is dropped
    with pytest.raises(RuntimeError, match="outside"):
        gw.preprocess([[1, 2, N, 5]])
    gw.push_pull(None)
    with pytest.raises(RuntimeError, match="outside"):
        gw.preprocess([[-1]])
    gw.preprocess([[1]])
    gw.push_pull(None)
    rng = np.random.RandomState(6)
    batches = [[rng.randint(N, size=64)] for _ in range(3)]
    grads = [None] + [[rng.normal(0, 1, size=(64, W)).astype(np.float32)] for _ in range(2)]
    run_steps(gw, ow, batches, grads)
    gw.close()


def test_constructor_errors():
    root = np.zeros(10, dtype=np.uint8)
    with pytest.raises(RuntimeError):  # a rank must store the rows it owns
        hb.Table(0, 1, 0, "127.0.0.1", 1, 10, 4, 0, 0, root, np.arange(9))
    with pytest.raises(RuntimeError):  # duplicate storage key
        hb.Table(0, 1, 0, "127.0.0.1", 1, 10, 4, 0, 0, root, np.array([0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 9]))
    with pytest.raises(RuntimeError):  # key outside the table
        hb.Table(0, 1, 0, "127.0.0.1", 1, 10, 4, 0, 0, root, np.arange(11))
    with pytest.raises(RuntimeError):  # no such device
        hb.Table(0, 1, 1000, "127.0.0.1", 1, 10, 4, 0, 0, root, np.arange(10))


# ------------------------------------------------------------------------------------------------
# multi-rank: thread ranks on one GPU.  exchange="inproc" runs the kernels of the NCCL path (bytes moved by
# cudaMemcpyAsync), exchange="p2p" the kernels of the peer-to-peer mailbox exchange that one-process-per-GPU jobs
# use by default (see gpu_world.py).
# ------------------------------------------------------------------------------------------------
EXCHANGES = ["inproc", "p2p"]


def _hybrid_storage(root, nrank, rng, frac):
    return [np.where((root == r) | (rng.rand(len(root)) < frac))[0] for r in range(nrank)]


@pytest.mark.parametrize("nrank,pull,push,frac", [(2, 0, 0, 0.0), (2, 0, 0, 0.5), (4, 0, 0, 0.3), (4, 2, 3, 0.3),
                                                   (3, 10, 10, 1.0), (8, 1, 0, 0.1), (8, 0, 0, 0.6)])
@pytest.mark.parametrize("exchange", EXCHANGES)
def test_multi_rank_parity(oracle_mod, nrank, pull, push, frac, exchange):
    N, W, B = 3000, 16, 700
    rng = np.random.RandomState(nrank * 100 + pull)
    root = rng.randint(nrank, size=N).astype(np.uint8)
    storage = _hybrid_storage(root, nrank, rng, frac)
    gw, ow = make_worlds(oracle_mod, nrank, N, W, pull, push, 0.1, root, storage, exchange=exchange)
    batches = [[(rng.zipf(1.2, size=B) - 1) % N for _ in range(nrank)] for _ in range(8)]
    batches[4] = [np.zeros(0, dtype=np.int64)] * nrank
    grads = [None] + [[rng.normal(0, 1, size=(len(k), W)).astype(np.float32) for k in batches[s - 1]]
                      for s in range(1, 8)]
    grads[6] = None  # an inference step in the middle
    run_steps(gw, ow, batches, grads)
    gw.close()


@pytest.mark.parametrize("knob", ["HCTR_P2P_FUSED_EXPAND=0", "HCTR_EXPAND=bulk"])
def test_mailbox_exchange_with_refresh_and_expansion_as_two_launches(oracle_mod, monkeypatch, knob):
    # the requester side of the mailbox exchange is one launch by default; the two-launch form (flag / row-index
    # arrays, then the plain or the bulk-copy expansion) stays selectable and must give the same step
    name, value = knob.split("=")
    monkeypatch.setenv(name, value)
    nrank, N, W, B = 4, 3000, 32, 700
    rng = np.random.RandomState(77)
    root = rng.randint(nrank, size=N).astype(np.uint8)
    storage = _hybrid_storage(root, nrank, rng, 0.3)
    gw, ow = make_worlds(oracle_mod, nrank, N, W, 1, 2, 0.1, root, storage, exchange="p2p")
    batches = [[(rng.zipf(1.2, size=B) - 1) % N for _ in range(nrank)] for _ in range(5)]
    grads = [None] + [[rng.normal(0, 1, size=(len(k), W)).astype(np.float32) for k in batches[s - 1]]
                      for s in range(1, 5)]
    run_steps(gw, ow, batches, grads)
    gw.close()


@pytest.mark.parametrize("width", [128, 132, 256, 260, 512, 640])
@pytest.mark.parametrize("exchange", EXCHANGES)
def test_multi_rank_wide_rows(oracle_mod, width, exchange):
    # rows of 128..512 floats take the streaming reduction, wider ones the register kernel; with caches and
    # bounds every storage class (not stored / owned / cached push / cached hold) occurs
    nrank, N, B = 3, 2500, 900
    rng = np.random.RandomState(width)
    root = rng.randint(nrank, size=N).astype(np.uint8)
    storage = _hybrid_storage(root, nrank, rng, 0.4)
    gw, ow = make_worlds(oracle_mod, nrank, N, width, 2, 3, 0.1, root, storage, exchange=exchange)
    batches = [[(rng.zipf(1.15, size=B) - 1) % N for _ in range(nrank)] for _ in range(5)]
    grads = [None] + [[rng.normal(0, 1, size=(len(k), width)).astype(np.float32) for k in batches[s - 1]]
                      for s in range(1, 5)]
    run_steps(gw, ow, batches, grads)
    gw.close()


@pytest.mark.parametrize("exchange", EXCHANGES)
@pytest.mark.parametrize("nrank,width,push", [(2, 16, 2), (4, 128, 3), (5, 36, 0)])
def test_batch_size_grows_between_steps(oracle_mod, nrank, width, push, exchange):
    # The batch size changes from step to step, twice beyond everything reserved so far: all per-batch buffers (and,
    # with the mailbox exchange, the mailboxes themselves) are re-allocated between a batch's push decision - taken
    # at the end of its own push_pull - and the reduction that consumes the decision one step later.
    N = 4000
    rng = np.random.RandomState(17 * nrank + width)
    root = rng.randint(nrank, size=N).astype(np.uint8)
    storage = _hybrid_storage(root, nrank, rng, 0.5)
    gw, ow = make_worlds(oracle_mod, nrank, N, width, 1, push, 0.1, root, storage, exchange=exchange)
    sizes = [256, 700, 300, 5000, 64, 5000]
    batches = [[(rng.zipf(1.2, size=b) - 1) % N for _ in range(nrank)] for b in sizes]
    grads = [None] + [[rng.normal(0, 1, size=(len(k), width)).astype(np.float32) for k in batches[s - 1]]
                      for s in range(1, len(sizes))]
    run_steps(gw, ow, batches, grads)
    gw.close()


@pytest.mark.parametrize("exchange", EXCHANGES)
def test_many_pushers_per_row(oracle_mod, exchange):
    # 8 ranks, every rank caches every row and pushes each step (push bound 0), keys from a small hot set: most
    # owned rows receive pushes from several sources in one step, up to all seven peers - the case in which the
    # owner must add the contributions in ascending source order
    nrank, N, W, B = 8, 600, 128, 1500
    rng = np.random.RandomState(8)
    root = rng.randint(nrank, size=N).astype(np.uint8)
    storage = [np.arange(N)] * nrank
    gw, ow = make_worlds(oracle_mod, nrank, N, W, 0, 0, 0.1, root, storage, exchange=exchange)
    batches = [[(rng.zipf(1.1, size=B) - 1) % N for _ in range(nrank)] for _ in range(4)]
    grads = [None] + [[rng.normal(0, 1, size=(B, W)).astype(np.float32) for _ in range(nrank)] for _ in range(3)]
    run_steps(gw, ow, batches, grads)
    gw.close()


@pytest.mark.parametrize("exchange", EXCHANGES)
def test_reference_update_script_exact_counts(oracle_mod, exchange):
    # the reference's tests/test_update.py:17-43 through the CUDA path: 4 ranks, hybrid storage, lr=-1, grad=1
    nrank, W, N, B = 4, 128, 1024, 1024
    np.random.seed(0)
    root = np.random.randint(nrank, size=N)
    storage = [np.where(root <= r)[0] for r in range(nrank)]
    gw = GpuWorld(nrank, N, W, 0, 0, -1.0, root, storage, exchange=exchange)
    rngs = [np.random.RandomState(r) for r in range(nrank)]
    gw.preprocess([np.zeros(0, dtype=np.int64)] * nrank)
    ids = [np.zeros(0, dtype=np.int64)] * nrank
    store = np.zeros(N)
    grad = np.ones((B, W), dtype=np.float32)
    for _ in range(50):
        for r in range(nrank):
            np.add.at(store, ids[r], 1.0)
        ids = [rngs[r].randint(N, size=B).astype(np.int64) for r in range(nrank)]
        gw.preprocess(ids)
        dst = gw.push_pull([grad[: len(ids[r])] for r in range(nrank)])
    for r in range(nrank):
        assert np.array_equal(dst[r][:, 0], store[ids[r]].astype(np.float32))
    gw.close()
