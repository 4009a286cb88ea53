"""End to end over the rows either side of the hot path: a click log is partitioned offline, the tables are
built from the partition (owners + cached rows), every rank then steps through its own samples.  The CUDA
tables must match the oracle exactly, and the partitioned job must move fewer rows between ranks than the
same job with randomly drawn owners and rank-agnostic sample placement."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from gpu_world import GpuWorld  # noqa: E402
from test_gpu_parity import make_worlds, run_steps  # noqa: E402

from hetuctr_b200 import partition_tools as pt  # noqa: E402
from tests.golden.partition_cases import make_case  # noqa: E402

CFG = dict(n_data=8000, n_slot=8, per_slot=300, clusters=16, n_part=4, batch_size=512, comm="uniform", seed=21)


def job_batches(data, data_part, nrank, per_rank, steps, rng):
    """Each rank draws `per_rank` of ITS samples per step; keys flattened sample-major."""
    mine = [np.where(data_part == r)[0] for r in range(nrank)]
    return [[data[rng.choice(mine[r], per_rank)].reshape(-1).astype(np.int64) for r in range(nrank)]
            for _ in range(steps)]


def moved_rows(gw):
    s = [t.stats() for t in gw.tables]
    return sum(x["pushed_rows"] + x["received_rows"] for x in s)


@pytest.mark.parametrize("bounds", [(0, 0), (3, 3)])
def test_partitioned_job_matches_oracle_and_moves_less(oracle_mod, bounds):
    nrank, width = CFG["n_part"], 16
    data, _ = make_case(CFG)
    length = int(data.max()) + 1
    part = pt.direct_partition(data, nrank, nrank, CFG["batch_size"], rerun=10)
    arrays = [pt.table_arrays(part, r, cache_rows=length // 20, length=length) for r in range(nrank)]
    root = arrays[0][0]
    assert all(np.array_equal(a[0], root) for a in arrays)
    gw, ow = make_worlds(oracle_mod, nrank, length, width, bounds[0], bounds[1], 0.05, root,
                         [a[1] for a in arrays])
    rng = np.random.RandomState(3)
    per_rank = CFG["batch_size"] // nrank
    batches = job_batches(data, part["data_partition"], nrank, per_rank, 6, rng)
    grads = [None] + [[rng.normal(0, 0.1, size=(b.size, width)).astype(np.float32) for b in batches[s - 1]]
                      for s in range(1, 6)]
    moved = 0
    for s in range(6):
        run_steps(gw, ow, [batches[s]], [grads[s]])
        moved += moved_rows(gw)
    gw.close()

    # the same job without the partitioner: random owners, samples dealt to ranks regardless of content
    rng = np.random.RandomState(3)
    root_rand = np.random.RandomState(9).randint(nrank, size=length).astype(np.uint8)
    storage = [np.where(root_rand == r)[0] for r in range(nrank)]
    gr = GpuWorld(nrank, length, width, bounds[0], bounds[1], 0.05, root_rand, storage)
    dealt = np.arange(len(data)) % nrank
    batches_r = job_batches(data, dealt, nrank, per_rank, 6, rng)
    moved_rand = 0
    for s in range(6):
        gr.preprocess(batches_r[s])
        gr.push_pull(None if s == 0 else [rng.normal(0, 0.1, size=(b.size, width)).astype(np.float32)
                                          for b in batches_r[s - 1]])
        moved_rand += moved_rows(gr)
    gr.close()
    assert moved < 0.75 * moved_rand, (moved, moved_rand)
