"""Seeded inputs of the golden cases.  Shared by the script that records the reference's outputs
(make_reference_golden.py, run once on a GPU box with the reference's own build) and by the tests that replay
the same inputs through the CPU oracle and the CUDA path."""
import numpy as np

# name -> parameters.  Everything else (owners, storage sets, keys, gradients, initial rows) derives from `seed`.
CASES = {
    "r1_zipf": dict(nrank=1, length=2000, width=8, batch=512, steps=5, pull=0, push=0, lr=0.1, cache=0.0, seed=11),
    "r1_wide_dups": dict(nrank=1, length=300, width=32, batch=900, steps=4, pull=0, push=0, lr=0.5, cache=0.0, seed=12),
    "r2_owned_only": dict(nrank=2, length=1500, width=4, batch=300, steps=5, pull=0, push=0, lr=0.1, cache=0.0, seed=21),
    "r2_hybrid_bsp": dict(nrank=2, length=1500, width=8, batch=400, steps=6, pull=0, push=0, lr=0.05, cache=0.4, seed=22),
    "r2_hybrid_stale": dict(nrank=2, length=800, width=4, batch=400, steps=8, pull=2, push=3, lr=0.05, cache=0.5, seed=23),
    "r4_hybrid_stale": dict(nrank=4, length=1200, width=4, batch=256, steps=6, pull=1, push=2, lr=0.1, cache=0.3, seed=41),
    # rows of 128 / 256 floats (the shapes the benchmark configurations use); float arrays are recorded as
    # digests (see digest() below) to keep the fixtures small
    "r1_rows128": dict(nrank=1, length=1500, width=128, batch=1200, steps=4, pull=0, push=0, lr=0.1, cache=0.0,
                       seed=51, digest=True),
    "r2_rows256_stale": dict(nrank=2, length=1000, width=256, batch=700, steps=5, pull=2, push=3, lr=0.05,
                             cache=0.4, seed=52, digest=True),
}

# arrays recorded after every preprocess (per rank) and after the last step
INDEX_ARRAYS = ("unique_idx", "idx_map", "sorted_arg", "run_length", "root", "offset", "shape", "shape_exchanged")
STATE_ARRAYS = ("version", "updates", "embedding", "gradient")

# value initialisers recorded from the reference: (kind, a, b, seed, elements)
INIT_CASES = {
    "init_normal": (1, 0.0, 0.1, 0, 4096),
    "init_normal_seed7": (1, 0.5, 2.0, 7, 1000),
    "init_uniform": (2, -0.25, 0.75, 3, 4096),
    "init_truncated": (3, 0.0, 1.0, 5, 4096),
}


def digest(rows, width):
    """Compact stand-in for a [n, width] float array: per-row sum and sum of magnitudes (float64) plus six
    sampled columns.  Every row is still checked, at a fraction of the size."""
    rows = np.asarray(rows, dtype=np.float32).reshape(-1, width)
    cols = sorted({0, 1, width // 2 - 1, width // 2, width - 2, width - 1} & set(range(width)))
    r64 = rows.astype(np.float64)
    return {"rowsum": r64.sum(1), "rowabs": np.abs(r64).sum(1), "cols": rows[:, cols].copy()}


def make_inputs(name):
    c = CASES[name]
    rng = np.random.RandomState(c["seed"])
    n, N, W, B = c["nrank"], c["length"], c["width"], c["batch"]
    root = rng.randint(n, size=N).astype(np.uint8)
    storage = []
    for r in range(n):
        keep = (root == r) | (rng.rand(N) < c["cache"])
        keys = np.where(keep)[0].astype(np.int64)
        storage.append(rng.permutation(keys))  # storage order is the caller's choice; make it non-trivial
    emb = [rng.normal(0, 0.05, size=(len(storage[r]), W)).astype(np.float32) for r in range(n)]
    keys, grads = [], []
    for s in range(c["steps"]):
        ks = []
        for r in range(n):
            if s == 2:
                k = rng.randint(N, size=B)  # one uniform batch
            else:
                k = (rng.zipf(1.3, size=B) - 1 + rng.randint(N)) % N
            ks.append(k.astype(np.int64))
        keys.append(ks)
        grads.append(None if s == 0 else [rng.normal(0, 1, size=(B, W)).astype(np.float32) for _ in range(n)])
    return c, root, storage, emb, keys, grads


def layout_rows(root, storage_r, rank, emb_r):
    """Rows of `emb_r` (given per entry of storage_r) re-ordered to local-row order: keys owned by another rank
    first, then owned keys, each group in storage order (reference csrc/core/table_initialize.cu:76-91)."""
    storage_r = np.asarray(storage_r)
    cached = np.where(root[storage_r] != rank)[0]
    owned = np.where(root[storage_r] == rank)[0]
    idx = np.concatenate([cached, owned]).astype(np.int64)
    return emb_r[idx] if len(idx) else emb_r[:0]
