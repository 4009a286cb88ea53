"""From a click log to the arrays a HetuTable is built from.

Same flow and file format as the reference's experimental/partition.py: run the partitioner for a few refine
rounds, then store `embed_partition` (owner of every row), `data_partition` (rank of every sample) and, per
rank r under the key str(r), the non-owned rows ordered by caching priority, best first.  table_arrays() turns
that into the `root_arr` / `storage_arr` arguments of the table constructor (reference tests/benchmark.py:49-55).

  python -m hetuctr_b200.partition_tools --data sparse.npy -n 8 -g 8 -b 8192 -r 10 -o partition.npz
"""
import argparse
import time

import numpy as np


def get_comm_mat(nrank, ngpus):
    """Relative cost of fetching a row: 0 on the same rank, 0.1 inside a node of `ngpus` ranks, 1 across nodes
    (reference experimental/partition.py:20-30)."""
    r = np.arange(nrank)
    same_node = (r[:, None] // ngpus) == (r[None, :] // ngpus)
    mat = np.where(same_node, 0.1, 1.0)
    mat[r, r] = 0.0
    return mat.astype(np.float32)


def direct_partition(data, nparts, ngpus, batch_size, rerun, seed=0, log=None):
    """Returns the dict the reference script saves with np.savez.  `log`, if given, receives one line per round."""
    import hetuctr_b200
    part = hetuctr_b200.hetuCTR_partition
    data = np.ascontiguousarray(data, dtype=np.int32)
    mat = get_comm_mat(nparts, ngpus)
    p = part.partition(data, mat, nparts, batch_size, seed=seed)
    say = log or (lambda *_: None)
    say("Initial cost : {}".format(float((p.get_communication() * mat).sum())))
    for i in range(rerun):
        p.refine_data()
        p.refine_embed()
        cost = p.get_communication()
        say("Refine round {} : {}  data {} embed {}".format(i, float((cost * mat).sum()), p.get_data_cnt(),
                                                            p.get_embed_cnt()))
    item_partition, idx_partition = p.get_result()
    out = {"embed_partition": idx_partition, "data_partition": item_partition}
    priority = p.get_priority()
    for i in range(nparts):
        mine = idx_partition == i
        pr = priority[i].copy()
        pr[mine] = -1  # rows the rank owns need no cache slot
        # descending priority, row id ascending among equals (the reference's argsort leaves ties unordered).
        # Only rows some sample of the rank uses have a priority; the rest follow in id order without sorting.
        used = np.flatnonzero(pr > 0)
        used = used[np.lexsort((used, -pr[used]))]
        out[str(i)] = np.concatenate([used, np.flatnonzero(pr == 0)])
    return out


def table_arrays(partition, rank, cache_rows, length=None):
    """(root_arr uint8 [length], storage_arr int64 sorted): rows owned by `rank` plus its `cache_rows` best cache
    candidates.  Rows beyond the partitioned id range (never seen in the log) are dealt round-robin."""
    owner = np.asarray(partition["embed_partition"])
    n = owner.size if length is None else int(length)
    if n < owner.size:
        raise ValueError("length is smaller than the partitioned id range")
    root = np.empty(n, dtype=np.uint8)
    root[: owner.size] = owner
    nrank = int(owner.max()) + 1 if owner.size else 1
    nrank = max(nrank, len([k for k in partition if str(k).isdigit()]))
    root[owner.size:] = np.arange(owner.size, n) % nrank
    owned = np.where(root == rank)[0].astype(np.int64)
    cached = np.asarray(partition[str(rank)][: max(int(cache_rows), 0)], dtype=np.int64)
    return root, np.sort(np.concatenate([owned, cached]))


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--data", required=True, help=".npy int array [samples, slots] of embedding ids")
    ap.add_argument("--nrank", "-n", type=int, default=8)
    ap.add_argument("--batch_size", "-b", type=int, default=8192)
    ap.add_argument("--rerun", "-r", type=int, default=10)
    ap.add_argument("--ngpus", "-g", type=int, default=8)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--output", "-o", default="partition.npz")
    a = ap.parse_args(argv)
    t0 = time.time()
    out = direct_partition(np.load(a.data), a.nrank, a.ngpus, a.batch_size, a.rerun, a.seed, log=print)
    np.savez(a.output, **out)
    print("Partition Time : ", time.time() - t0)


if __name__ == "__main__":
    main()
