"""Seeded synthetic click logs for the partitioner fixtures (shared by the generator and the tests)."""
import numpy as np

CASES = {
    # name: samples, slots, ids per slot, clusters, parts, global batch, rounds, comm matrix kind
    "p2_small": dict(n_data=600, n_slot=4, per_slot=40, clusters=6, n_part=2, batch_size=32, rounds=3,
                     comm="uniform", seed=11),
    "p4_clustered": dict(n_data=4000, n_slot=8, per_slot=120, clusters=16, n_part=4, batch_size=128, rounds=4,
                         comm="uniform", seed=12),
    "p4_topology": dict(n_data=3000, n_slot=6, per_slot=90, clusters=12, n_part=4, batch_size=64, rounds=3,
                        comm="pairs", seed=13),
    "p8_sparse": dict(n_data=5000, n_slot=10, per_slot=400, clusters=40, n_part=8, batch_size=256, rounds=3,
                      comm="uniform", seed=14),
    # batch larger than the per-part sample count, ids with gaps (some embedding rows never used)
    "p3_gaps": dict(n_data=300, n_slot=3, per_slot=50, clusters=5, n_part=3, batch_size=512, rounds=2,
                    comm="uniform", seed=15, stride=3),
}


def make_case(cfg):
    """data [n_data, n_slot] int32: slot s draws from its own id range; a sample belongs to one of `clusters`
    groups and mostly (80%) uses that group's narrow window of the range, so that co-partitioning pays."""
    rng = np.random.RandomState(cfg["seed"])
    n, s, per, c = cfg["n_data"], cfg["n_slot"], cfg["per_slot"], cfg["clusters"]
    cluster = rng.randint(c, size=n)
    width = max(per // c, 1)
    local = (cluster[:, None] * width + rng.randint(width, size=(n, s))) % per
    anywhere = rng.randint(per, size=(n, s))
    ids = np.where(rng.rand(n, s) < 0.8, local, anywhere)
    data = (ids + np.arange(s)[None, :] * per) * cfg.get("stride", 1)
    p = cfg["n_part"]
    comm = np.ones((p, p), dtype=np.float32) - np.eye(p, dtype=np.float32)
    if cfg["comm"] == "pairs":  # ranks 2k and 2k+1 share a fast link
        for i in range(p):
            comm[i, i ^ 1] = 0.25
    return np.ascontiguousarray(data.astype(np.int32)), comm
