"""Offline partitioner (module hetuCTR_partition) against fixtures recorded from the reference's own module
(tests/golden/make_partition_golden.py): same starting assignment, same rounds, identical results."""
import os

import numpy as np
import pytest

import hetuctr_b200
from tests.golden.partition_cases import CASES, make_case

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def part():
    return hetuctr_b200.hetuCTR_partition


@pytest.mark.parametrize("name", sorted(CASES))
def test_replays_reference_rounds(part, name):
    cfg = CASES[name]
    g = np.load(os.path.join(GOLDEN, f"partition_{name}.npz"))
    data, comm = make_case(cfg)
    p = part.partition(data, comm, cfg["n_part"], cfg["batch_size"])
    p.set_result(g["init_data"], g["init_embed"])
    np.testing.assert_array_equal(p.get_communication(), g["init_comm"])
    np.testing.assert_array_equal(p.get_priority(), g["init_priority"])
    for r in range(cfg["rounds"]):
        p.refine_data()
        np.testing.assert_array_equal(p.get_result()[0], g[f"r{r}_data_after_data"])
        p.refine_embed()
        d, e = p.get_result()
        np.testing.assert_array_equal(d, g[f"r{r}_data"])
        np.testing.assert_array_equal(e, g[f"r{r}_embed"])
        np.testing.assert_array_equal(p.get_data_cnt(), g[f"r{r}_data_cnt"])
        np.testing.assert_array_equal(p.get_embed_cnt(), g[f"r{r}_embed_cnt"])
        np.testing.assert_array_equal(p.get_communication(), g[f"r{r}_comm"])
    np.testing.assert_array_equal(p.get_priority(), g["final_priority"])


def soft_count(n_data, n_part, batch):
    """numpy restatement of the expected-hit curve (csrc/partition/partition.cc:58-64), float64."""
    mx = n_data // n_part
    k = np.arange(n_data + 2, dtype=np.float64)
    s = (1 - (1 - k / mx) ** batch) * mx / batch
    s[mx:] = 1.0
    return s


def test_communication_matches_numpy_restatement(part):
    cfg = CASES["p4_topology"]
    data, comm = make_case(cfg)
    p = part.partition(data, comm, cfg["n_part"], cfg["batch_size"], seed=5)
    p.refine_data()
    d, e = p.get_result()
    n_embed = data.max() + 1
    cnt = np.zeros((cfg["n_part"], n_embed), dtype=np.int64)
    for k in range(cfg["n_part"]):
        np.add.at(cnt[k], data[d == k].ravel(), 1)
    soft = soft_count(len(data), cfg["n_part"], cfg["batch_size"])
    want = np.zeros((cfg["n_part"],) * 2)
    for k in range(cfg["n_part"]):
        np.add.at(want[k], e, soft[cnt[k]])
    want *= cfg["batch_size"] * cfg["n_part"] / len(data)
    np.testing.assert_allclose(p.get_communication(), want, rtol=2e-4)
    deg = cnt.sum(0)
    pr = np.where(cnt > 0, comm[np.arange(cfg["n_part"])[:, None], e[None, :]] * soft[cnt] ** 2
                  * (1.0 / np.maximum(deg, 1)[None, :] + 1.0 / np.maximum(cnt, 1)), 0.0)
    np.testing.assert_allclose(p.get_priority(), pr, rtol=2e-4)
    np.testing.assert_array_equal(p.get_data_cnt(), np.bincount(d, minlength=cfg["n_part"]))
    np.testing.assert_array_equal(p.get_embed_cnt(), np.bincount(e, minlength=cfg["n_part"]))


def test_seeded_and_improves(part):
    cfg = CASES["p4_clustered"]
    data, comm = make_case(cfg)
    a = part.partition(data, comm, cfg["n_part"], cfg["batch_size"], seed=3)
    b = part.partition(data, comm, cfg["n_part"], cfg["batch_size"], seed=3)
    c = part.partition(data, comm, cfg["n_part"], cfg["batch_size"], seed=4)
    assert all((x == y).all() for x, y in zip(a.get_result(), b.get_result()))
    assert not (a.get_result()[0] == c.get_result()[0]).all()
    cost0 = float((a.get_communication() * comm).sum())
    for _ in range(4):
        a.refine_data()
        a.refine_embed()
        b.refine_data()
        b.refine_embed()
    assert all((x == y).all() for x, y in zip(a.get_result(), b.get_result()))
    cost1 = float((a.get_communication() * comm).sum())
    assert cost1 < 0.5 * cost0
    # the balance terms keep every part populated
    assert a.get_data_cnt().min() > 0.5 * len(data) / cfg["n_part"]
    assert a.get_embed_cnt().min() > 0


def test_argument_errors(part):
    data, comm = make_case(CASES["p2_small"])
    with pytest.raises(RuntimeError, match="continuous"):
        part.partition(data[:, ::2], comm, 2, 32)
    with pytest.raises(RuntimeError, match="comm_mat"):
        part.partition(data, np.ones((3, 3), np.float32), 2, 32)
    bad = data.copy()
    bad[0, 0] = -1
    with pytest.raises(RuntimeError, match="negative"):
        part.partition(bad, comm, 2, 32)
    p = part.partition(data, comm, 2, 32)
    with pytest.raises(RuntimeError, match="out of range"):
        p.set_result(np.full(len(data), 2, np.int32), np.zeros(data.max() + 1, np.int32))


def test_glue_arrays(tmp_path):
    from hetuctr_b200 import partition_tools as pt
    cfg = CASES["p4_clustered"]
    data, _ = make_case(cfg)
    np.testing.assert_array_equal(pt.get_comm_mat(4, 2), np.array(
        [[0, .1, 1, 1], [.1, 0, 1, 1], [1, 1, 0, .1], [1, 1, .1, 0]], np.float32))
    lines = []
    out = pt.direct_partition(data, 4, 2, cfg["batch_size"], rerun=3, log=lines.append)
    assert len(lines) == 4 and lines[0].startswith("Initial cost")
    n_embed = data.max() + 1
    assert out["embed_partition"].shape == (n_embed,) and out["data_partition"].shape == (len(data),)
    for r in range(4):
        cand = out[str(r)]
        assert (out["embed_partition"][cand] != r).all()
        assert cand.size == n_embed - (out["embed_partition"] == r).sum()
        assert np.unique(cand).size == cand.size
    root, storage = pt.table_arrays(out, 1, cache_rows=50, length=n_embed + 10)
    assert root.dtype == np.uint8 and root.size == n_embed + 10
    assert (np.diff(storage) > 0).all()
    owned = np.where(root == 1)[0]
    assert np.isin(owned, storage).all() and storage.size == owned.size + 50
    assert set(storage) - set(owned) == set(out["1"][:50])
    # the command-line entry writes the reference's file layout
    np.save(tmp_path / "d.npy", data)
    pt.main(["--data", str(tmp_path / "d.npy"), "-n", "4", "-g", "2", "-b", "128", "-r", "1",
             "-o", str(tmp_path / "p.npz")])
    z = np.load(tmp_path / "p.npz")
    assert sorted(z.files) == sorted(["embed_partition", "data_partition", "0", "1", "2", "3"])


def test_clustered_job_layouts():
    """The config-5 style job builders: same click log for both layouts, the partitioned one needs far fewer
    remote rows per batch than random owners with samples dealt regardless of content."""
    from hetuctr_b200 import workloads as w
    w.CONFIGS["cfg5_tiny"] = dict(w.CONFIGS["cfg5_sweep"], rows=400_000, samples=512)
    try:
        root_g, storage_g, mine_g, data_g = w.partitioned_job("cfg5_tiny", 4, 40_000, 4000)
        root_r, storage_r, mine_r, data_r = w.random_job("cfg5_tiny", 4, 40_000, 4000)
    finally:
        del w.CONFIGS["cfg5_tiny"]
    assert np.array_equal(data_g, data_r) and data_g.shape == (40_000, 26)
    assert data_g.min() >= 0 and data_g.max() < 400_000
    for root, storage, mine in ((root_g, storage_g, mine_g), (root_r, storage_r, mine_r)):
        assert root.dtype == np.uint8 and root.size == 400_000 and root.max() == 3
        assert sorted(np.concatenate(mine).tolist()) == list(range(40_000))  # every sample on exactly one rank
        for r in range(4):
            assert (np.diff(storage[r]) > 0).all()
            assert np.isin(np.where(root == r)[0], storage[r]).all()

    def remote_rows(root, mine):
        rng = np.random.RandomState(0)
        return sum(int((root[np.unique(data_g[rng.choice(mine[r], 512)])] != r).sum()) for r in range(4))

    assert remote_rows(root_g, mine_g) < 0.8 * remote_rows(root_r, mine_r)
