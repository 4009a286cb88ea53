"""Seeded synthetic CTR key batches and table partitions.

The reference measures on Criteo / Avazu click logs (reference tests/benchmark.py:26-31); only their SHAPE is
used here: a sample has one key per categorical field, fields have very different vocabulary sizes, keys inside
a field are power-law distributed.  Everything below is generated from seeds; no dataset record is reproduced.
"""
import numpy as np

# name -> (rows, width, samples per GPU, fields, zipf alpha or None for uniform, vocab ratio, cache fraction,
#          pull_bound, push_bound, lr, init stddev)
CONFIGS = {
    "cfg1_plumbing": dict(rows=100_000, width=16, samples=1024, fields=26, alpha=None, ratio=0.7, cache=0.0,
                          pull_bound=0, push_bound=0, lr=0.1, init_std=0.01),
    "cfg2_hybrid": dict(rows=33_762_577, width=128, samples=8192, fields=26, alpha=1.05, ratio=0.7, cache=0.10,
                        pull_bound=0, push_bound=0, lr=0.01, init_std=0.1),
    "cfg3_large": dict(rows=1_000_000_000, width=64, samples=16384, fields=39, alpha=1.2, ratio=0.8, cache=0.0,
                       pull_bound=0, push_bound=0, lr=0.01, init_std=0.1),
    "cfg4_stress": dict(rows=100_000_000, width=32, samples=32768, fields=26, alpha=None, ratio=0.7, cache=0.05,
                        pull_bound=10, push_bound=10, lr=0.05, init_std=0.1),
    "cfg5_sweep": dict(rows=50_000_000, width=256, samples=4096, fields=26, alpha=1.1, ratio=0.7, cache=0.0,
                       pull_bound=0, push_bound=0, lr=0.01, init_std=0.1),
}


def field_vocab(rows, fields, ratio):
    """Geometric split of `rows` over `fields` vocabularies: v_f ~ ratio**f, remainder to field 0."""
    w = ratio ** np.arange(fields)
    v = np.floor(rows * w / w.sum()).astype(np.int64)
    v = np.maximum(v, 1)
    v[0] += rows - v.sum()
    assert v.sum() == rows and v.min() >= 1
    return v


class KeySampler:
    """Draws [samples, fields] int64 key batches (flattened sample-major, like the reference's
    get_sample_data, tests/benchmark.py:20-24)."""

    def __init__(self, rows, fields, alpha, ratio, perm_seed=7):
        self.rows, self.fields, self.alpha = rows, fields, alpha
        self.vocab = field_vocab(rows, fields, ratio)
        self.base = np.concatenate([[0], np.cumsum(self.vocab)[:-1]])
        rng = np.random.RandomState(perm_seed)
        # per-field bijection rank -> id: (a*rank + b) mod v with gcd(a, v) = 1 spreads hot ranks over ids
        self.mul, self.add = [], []
        for v in self.vocab:
            a = int(rng.randint(1, max(int(v), 2)))
            while np.gcd(a, int(v)) != 1:
                a += 1
            self.mul.append(a)
            self.add.append(int(rng.randint(0, int(v))))
        self._cdf = None
        if alpha is not None:
            self._cdf = []
            for v in self.vocab:
                w = np.arange(1, int(v) + 1, dtype=np.float64) ** (-alpha)
                c = np.cumsum(w)
                self._cdf.append(c / c[-1])

    def field_rank_prob(self, f):
        """P(rank) for field f (rank 0 = hottest)."""
        v = int(self.vocab[f])
        if self.alpha is None:
            return np.full(v, 1.0 / v)
        c = self._cdf[f]
        return np.diff(np.concatenate([[0.0], c]))

    def key_of_rank(self, f, rank):
        v = int(self.vocab[f])
        return self.base[f] + (np.asarray(rank, dtype=np.int64) * self.mul[f] + self.add[f]) % v

    def batch(self, samples, rng):
        out = np.empty((samples, self.fields), dtype=np.int64)
        if self.alpha is None:
            # uniform over the whole table, as the reference's drivers draw keys (tests/driver.py:36)
            return rng.randint(self.rows, size=samples * self.fields).astype(np.int64)
        for f in range(self.fields):
            rank = np.searchsorted(self._cdf[f], rng.random_sample(samples), side="left")
            rank = np.minimum(rank, int(self.vocab[f]) - 1)
            out[:, f] = self.key_of_rank(f, rank)
        return out.reshape(-1)


def random_owners(rows, nrank, seed=0):
    """Owner of every key, as the reference's benchmark draws it (tests/benchmark.py:15-16)."""
    if nrank == 1:
        return np.zeros(rows, dtype=np.uint8)
    return np.random.RandomState(seed).randint(nrank, size=rows).astype(np.uint8)


def storage_with_cache(root, rank, sampler, cache_rows):
    """Keys stored by `rank`: the rows it owns plus the `cache_rows` non-owned keys with the highest expected
    access frequency (stand-in for the partitioner's priority list, reference csrc/partition/partition.cc:182-193)."""
    owned = np.where(root == rank)[0].astype(np.int64)
    if cache_rows <= 0:
        return owned
    cand_keys, cand_p = [], []
    per_field = max(1, int(cache_rows * 4 // sampler.fields) + 1)
    for f in range(sampler.fields):
        v = int(sampler.vocab[f])
        top = min(v, per_field)
        p = sampler.field_rank_prob(f)[:top]
        k = sampler.key_of_rank(f, np.arange(top))
        keep = root[k] != rank
        cand_keys.append(k[keep])
        cand_p.append(p[keep])
    keys = np.concatenate(cand_keys)
    prob = np.concatenate(cand_p)
    order = np.argsort(-prob, kind="stable")[:cache_rows]
    return np.concatenate([owned, np.sort(keys[order])])


class ClusteredSampler(KeySampler):
    """Click log with co-occurrence structure (config 5): every sample belongs to one of `clusters` seeded groups.
    In the large fields a sample draws, with probability `affinity`, from its group's own slice of the field's
    popularity ranking (the ranks congruent to the group id modulo `clusters`, power-law inside the slice) and
    otherwise from the whole field; small fields (fewer than 20 ranks per group) are always drawn globally.
    Samples of one group therefore share most of their rows, which is what a graph partitioner can exploit."""

    def __init__(self, rows, fields, alpha, ratio, clusters=1000, affinity=0.8, perm_seed=7):
        super().__init__(rows, fields, alpha, ratio, perm_seed)
        self.clusters, self.affinity = clusters, affinity
        self._slice_cdf = {}
        for f, v in enumerate(self.vocab):
            per = int(v) // clusters
            if per >= 20:
                w = np.arange(1, per + 1, dtype=np.float64) ** (-(alpha or 1.0))
                c = np.cumsum(w)
                self._slice_cdf[f] = c / c[-1]

    def log(self, samples, rng):
        """[samples, fields] int64 keys and the group of every sample."""
        group = rng.randint(self.clusters, size=samples)
        out = self.batch(samples, rng).reshape(samples, self.fields)  # global draws everywhere first
        for f, cdf in self._slice_cdf.items():
            own = rng.random_sample(samples) < self.affinity
            local = np.minimum(np.searchsorted(cdf, rng.random_sample(samples), side="left"), len(cdf) - 1)
            rank = local * self.clusters + group
            out[:, f] = np.where(own, self.key_of_rank(f, rank), out[:, f])
        return out, group


def partitioned_job(cfg, nrank, log_samples, cache_rows, seed=0, rounds=5, log=None):
    """Config-5 style job laid out by the offline partitioner: returns (root_arr, [storage_arr per rank],
    [sample indices per rank], click log).  Deterministic, so every rank of a job can compute it on its own."""
    from . import partition_tools as pt
    c = CONFIGS[cfg]
    sampler = ClusteredSampler(c["rows"], c["fields"], c["alpha"], c["ratio"])
    data, _ = sampler.log(log_samples, np.random.RandomState(1000 * int(cfg[3]) + 77))
    part = pt.direct_partition(data.astype(np.int32), nrank, nrank, c["samples"] * nrank, rounds, seed=seed, log=log)
    arrays = [pt.table_arrays(part, r, cache_rows, length=c["rows"]) for r in range(nrank)]
    mine = [np.where(part["data_partition"] == r)[0] for r in range(nrank)]
    return arrays[0][0], [a[1] for a in arrays], mine, data


def random_job(cfg, nrank, log_samples, cache_rows):
    """The same click log without the partitioner: random owners (the reference benchmark's choice), samples
    dealt to ranks regardless of content, every rank caches the globally most frequent rows of the log."""
    c = CONFIGS[cfg]
    sampler = ClusteredSampler(c["rows"], c["fields"], c["alpha"], c["ratio"])
    data, _ = sampler.log(log_samples, np.random.RandomState(1000 * int(cfg[3]) + 77))
    root = random_owners(c["rows"], nrank)
    freq = np.bincount(data.reshape(-1), minlength=c["rows"])
    order = np.argsort(-freq, kind="stable")
    storage = []
    for r in range(nrank):
        owned = np.where(root == r)[0].astype(np.int64)
        cand = order[root[order] != r][:cache_rows]
        cand = cand[freq[cand] > 0]
        storage.append(np.sort(np.concatenate([owned, cand.astype(np.int64)])))
    mine = [np.arange(r, log_samples, nrank) for r in range(nrank)]
    return root, storage, mine, data
