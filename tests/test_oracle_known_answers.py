"""Pins the CPU oracle against the reference's own known-answer scripts.

The reference has no golden files; what it asserts is in three multi-process GPU scripts.  Each test
below replays one of them against the oracle with all ranks in one process:
  * tests/test_update.py:17-43  (exact occurrence counts, hybrid storage, bounds 0/0)
  * tests/test_update.py:45-70  (random gradients, max abs error < 1e-4)
  * tests/check.py:14-46        (bounds 10/10: equal keys <=> equal values inside a batch)
plus the hand-derived two-rank example of the index arrays.
"""
import numpy as np
import pytest

NRANK, WIDTH, LENGTH, BATCH = 4, 128, 1024, 1024


def _root():
    np.random.seed(0)
    return np.random.randint(NRANK, size=LENGTH)


@pytest.mark.parametrize("nrank", [1, 2, 4])
def test_update_exact_counts(oracle_mod, nrank):
    # tests/test_update.py:17-43 — lr=-1, grad=ones, Zero init => dst[:,0] == global occurrence count
    np.random.seed(0)
    root = np.random.randint(nrank, size=LENGTH)
    storage = [np.where(root <= r)[0] for r in range(nrank)]
    w = oracle_mod.World(nrank, LENGTH, WIDTH, 0, 0, -1.0, root, storage)
    rngs = [np.random.RandomState(r) for r in range(nrank)]
    w.preprocess([np.zeros(0, dtype=np.int64)] * nrank)
    ids = [np.zeros(0, dtype=np.int64)] * nrank
    store = np.zeros(LENGTH)
    grad = np.ones((BATCH, WIDTH), dtype=np.float32)
    for step in range(50):
        for r in range(nrank):
            np.add.at(store, ids[r], 1.0)
        ids = [rngs[r].randint(LENGTH, size=BATCH).astype(np.int64) for r in range(nrank)]
        w.preprocess(ids)
        dst = w.push_pull([grad[: len(ids[r])] for r in range(nrank)])
    for r in range(nrank):
        assert np.array_equal(dst[r][:, 0], store[ids[r]].astype(np.float32))
        assert np.array_equal(dst[r][:, 0], dst[r][:, WIDTH - 1])


def test_update_random_gradients(oracle_mod):
    # tests/test_update.py:45-70
    root = _root()
    storage = [np.where(root <= r)[0] for r in range(NRANK)]
    w = oracle_mod.World(NRANK, LENGTH, WIDTH, 0, 0, -1.0, root, storage)
    rngs = [np.random.RandomState(r) for r in range(NRANK)]
    ids = [np.zeros(0, dtype=np.int64)] * NRANK
    store = np.zeros(LENGTH)
    for step in range(50):
        grads = [rngs[r].rand(BATCH, WIDTH).astype(np.float32) for r in range(NRANK)]
        for r in range(NRANK):
            np.add.at(store, ids[r], grads[r][: len(ids[r]), 0].astype(np.float64))
        ids = [rngs[r].randint(LENGTH, size=BATCH).astype(np.int64) for r in range(NRANK)]
        w.preprocess(ids)
        dst = w.push_pull(grads)
    for r in range(NRANK):
        assert np.max(np.abs(dst[r][:, 0] - store[ids[r]])) < 1e-4


def _checkvalue(k, v):
    kv = {}
    for key, val in zip(k, v[:, 0]):
        if key in kv:
            assert kv[key] == val
        else:
            assert val not in kv.values()
            kv[key] = val


def test_check_consistency_with_bounds(oracle_mod):
    # tests/check.py:14-46 — owned-only storage, bounds 10/10, Normal(0,1) init, lr=1
    root = _root()
    storage = [np.where(root == r)[0] for r in range(NRANK)]
    w = oracle_mod.World(NRANK, LENGTH, WIDTH, 10, 10, 1.0, root, storage)
    rng = np.random.RandomState(7)
    for r in range(NRANK):
        w.set_embedding(r, rng.normal(0, 1, size=(len(storage[r]), WIDTH)))
    rngs = [np.random.RandomState(100 + r) for r in range(NRANK)]
    grads = [rngs[r].rand(BATCH, WIDTH).astype(np.float32) for r in range(NRANK)]
    w.preprocess([np.zeros(0, dtype=np.int64)] * NRANK)
    for step in range(5):
        ids = [rngs[r].randint(LENGTH, size=BATCH).astype(np.int64) for r in range(NRANK)]
        w.preprocess(ids)
        dst = w.push_pull(grads)
        for r in range(NRANK):
            _checkvalue(ids[r], dst[r])


def test_two_rank_worked_example(oracle_mod):
    root = np.array([0, 1, 0, 1, 1, 0, 1, 0])
    w = oracle_mod.World(2, 8, 2, 0, 0, 0.5, root, [[0, 1, 2, 5, 7], [1, 3, 4, 6]])
    assert w.get(0, "stored_keys").tolist() == [1, 0, 2, 5, 7] and w.get(0, "nonlocal") == 1
    assert w.get(1, "stored_keys").tolist() == [1, 3, 4, 6] and w.get(1, "nonlocal") == 0
    for r in range(2):
        k = w.get(r, "stored_keys").astype(np.float32)
        w.set_embedding(r, np.stack([k, k + 0.5], 1))
    keys = [[5, 1, 3, 5, 1, 0], [6, 6, 2, 4, 1, 2]]
    w.preprocess(keys)
    expect = {
        "sorted_arg": ([5, 0, 3, 1, 4, 2], [2, 5, 4, 3, 0, 1]),
        "unique_idx": ([0, 5, 1, 3], [2, 1, 4, 6]),
        "run_length": ([0, 1, 3, 5, 6], [0, 2, 3, 4, 6]),
        "root": ([0, 0, 1, 1], [0, 1, 1, 1]),
        "offset": ([1, 3, 0, -1], [-1, 0, 2, 3]),
        "idx_map": ([1, 2, 3, 1, 2, 0], [3, 3, 0, 2, 1, 0]),
        "shape": ([2, 2], [1, 3]),
        "shape_exchanged": ([2, 1], [2, 3]),
    }
    for name, vals in expect.items():
        for r in range(2):
            assert w.get(r, name).tolist() == vals[r], name
    dst = w.push_pull(None)
    for r in range(2):
        k = np.array(keys[r], dtype=np.float32)
        assert np.array_equal(dst[r], np.stack([k, k + 0.5], 1))
    w.preprocess([[0, 1], [1, 3]])
    dst = w.push_pull([np.arange(12).reshape(6, 2), np.ones((6, 2))])
    assert dst[0].tolist() == [[-5, -5], [-4.5, -5]]
    assert dst[1].tolist() == [[-4.5, -5], [1, 1]]
    assert w.get(0, "version").tolist() == [3, 1, 2, 2, 0]
    assert w.get(1, "version").tolist() == [3, 1, 1, 2]


def test_pending_count_never_exceeds_push_bound(oracle_mod):
    rng = np.random.RandomState(3)
    n, L, W = 3, 200, 4
    root = rng.randint(n, size=L)
    storage = [np.where((root == r) | (rng.rand(L) < 0.4))[0] for r in range(n)]
    w = oracle_mod.World(n, L, W, 2, 3, 0.1, root, storage)
    for step in range(20):
        ids = [rng.randint(L, size=64) for _ in range(n)]
        w.preprocess(ids)
        w.push_pull([rng.randn(64, W) for _ in range(n)] if step else None)
        for r in range(n):
            u = w.get(r, "updates")
            assert np.all(u >= 0) and np.all(u <= 3)


def test_out_of_range_key_raises(oracle_mod):
    w = oracle_mod.World(1, 10, 2, 0, 0, 0.1, np.zeros(10), [np.arange(10)])
    with pytest.raises(RuntimeError):
        w.preprocess([[3, 10]])
