"""Golden vectors recorded from the REFERENCE's own build (tests/golden/make_reference_golden.py, run on a GPU
box with oracle/_ref): internal index arrays after every preprocess, pulled rows after every push_pull, final
versions / pending counts / rows.  They pin the CPU oracle (CPU test) and the CUDA path (GPU tests).

Bit-exact for all integer arrays.  Row values: 1e-5 relative (the tolerance the task states) against the
reference's build, whose compiler is free to contract the reference's multiply-add; against the oracle the CUDA
path is bit-exact (tests/test_gpu_parity.py).
"""
import os
import subprocess
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = os.path.join(HERE, "golden")
sys.path.insert(0, GOLD)
import cases  # noqa: E402

RTOL, ATOL = 1e-5, 1e-7


def _gold(name):
    path = os.path.join(GOLD, name + ".npz")
    if not os.path.exists(path):
        pytest.skip(f"golden file {name}.npz has not been recorded")
    return np.load(path)


def _close(got, gold, key, width, digest, msg):
    """Row values against the recorded ones: whole arrays, or their digests for the wide-row cases."""
    if not digest:
        np.testing.assert_allclose(np.asarray(got).reshape(-1), gold[key].reshape(-1), rtol=RTOL, atol=ATOL,
                                   err_msg=msg)
        return
    d = cases.digest(got, width)
    assert d["cols"].shape == gold[key + ".cols"].shape, msg
    np.testing.assert_allclose(d["cols"], gold[key + ".cols"], rtol=RTOL, atol=ATOL, err_msg=msg)
    # a row sum moves by at most RTOL times the sum of magnitudes when every element moves by RTOL
    err = np.abs(d["rowsum"] - gold[key + ".rowsum"])
    assert (err <= RTOL * gold[key + ".rowabs"] + ATOL * width).all(), msg
    np.testing.assert_allclose(d["rowabs"], gold[key + ".rowabs"], rtol=RTOL, atol=ATOL * width, err_msg=msg)


def _check_world(world, gold, name, get_f32):
    c, root, storage, emb, keys, grads = cases.make_inputs(name)
    n = c["nrank"]
    for r in range(n):
        world.set_embedding(r, cases.layout_rows(root, storage[r], r, emb[r]))
    for s in range(c["steps"]):
        world.preprocess(keys[s])
        # with the mailbox exchange the peers' counts reach the host on demand only, all ranks asking together
        exchanged = world.get_all("shape_exchanged") if hasattr(world, "get_all") else None
        for r in range(n):
            for a in cases.INDEX_ARRAYS:
                got = exchanged[r] if exchanged and a == "shape_exchanged" else world.get(r, a)
                exp = gold[f"s{s}_r{r}_{a}"]
                assert got.shape == exp.shape and np.array_equal(got, exp), f"{name} step {s} rank {r}: {a}"
        dst = world.push_pull(grads[s])
        for r in range(n):
            _close(dst[r], gold, f"s{s}_r{r}_dst", c["width"], c.get("digest"),
                   f"{name} step {s} rank {r}: pulled rows")
    for r in range(n):
        assert np.array_equal(world.get(r, "version"), gold[f"final_r{r}_version"])
        assert np.array_equal(world.get(r, "updates"), gold[f"final_r{r}_updates"])
        for a in ("embedding", "gradient"):
            _close(get_f32(r, a), gold, f"final_r{r}_{a}", c["width"], c.get("digest"), f"{name} rank {r}: {a}")


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_oracle_matches_reference_build(oracle_mod, name):
    gold = _gold(name)
    c, root, storage, *_ = cases.make_inputs(name)
    w = oracle_mod.World(c["nrank"], c["length"], c["width"], c["pull"], c["push"], c["lr"], root, storage)
    _check_world(w, gold, name, w.get_f32)


@pytest.mark.gpu
@pytest.mark.parametrize("exchange", ["inproc", "p2p"])
@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_cuda_path_matches_reference_build(name, exchange):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from gpu_world import GpuWorld
    gold = _gold(name)
    c, root, storage, *_ = cases.make_inputs(name)
    if c["nrank"] == 1 and exchange == "p2p":
        pytest.skip("a single rank exchanges nothing")
    w = GpuWorld(c["nrank"], c["length"], c["width"], c["pull"], c["push"], c["lr"], root, storage,
                 exchange=exchange)
    try:
        _check_world(w, gold, name, w.get_f32)
    finally:
        w.close()


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(cases.INIT_CASES))
def test_initial_values_match_reference_build(name):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import hetuctr_b200 as hb
    gold = _gold("init_values")[name]
    kind, a, b, seed, n = cases.INIT_CASES[name]
    hb.lib().hctr_seed(seed)
    t = hb.Table(0, 1, 0, "127.0.0.1", 0, n, 1, 0, 0, np.zeros(n, dtype=np.uint8), np.arange(n), (kind, a, b), 0.0, 0)
    got = t.dump("embedding").reshape(-1)
    t.close()
    hb.lib().hctr_seed(0)
    assert np.array_equal(got, gold.reshape(-1)), f"{name}: initial values differ from the reference's"


@pytest.mark.gpu
@pytest.mark.parametrize("exchange", ["p2p", "nccl"])
@pytest.mark.parametrize("name", [n for n in sorted(cases.CASES) if cases.CASES[n]["nrank"] > 1])
def test_multi_process_matches_oracle(oracle_mod, name, exchange, tmp_path):
    """One process per GPU through the drop-in `hetuCTR` module (sync and async calls, host and device key buffers)
    against the oracle, with both exchange flavours: device-driven peer-to-peer mailboxes and NCCL groups.
    Needs as many GPUs as the case has ranks."""
    torch = pytest.importorskip("torch")
    c, root, storage, emb, keys, grads = cases.make_inputs(name)
    n = c["nrank"]
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    port = 25000 + (os.getpid() % 2000) + 10 * sorted(cases.CASES).index(name) + (5 if exchange == "p2p" else 0)
    outs = [str(tmp_path / f"r{r}.npz") for r in range(n)]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", HCTR_EXCHANGE=exchange)
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "mp_worker.py"), name, str(r), str(port), outs[r]],
                              env=env) for r in range(n)]
    for p in procs:
        assert p.wait(timeout=300) == 0
    w = oracle_mod.World(n, c["length"], c["width"], c["pull"], c["push"], c["lr"], root, storage)
    for r in range(n):
        w.set_embedding(r, cases.layout_rows(root, storage[r], r, emb[r]))
    got = [np.load(o) for o in outs]
    for s in range(c["steps"]):
        w.preprocess(keys[s])
        for r in range(n):
            for a in cases.INDEX_ARRAYS:
                assert np.array_equal(got[r][f"s{s}_r{r}_{a}"], w.get(r, a)), f"{name} step {s} rank {r}: {a}"
        dst = w.push_pull(grads[s])
        for r in range(n):
            assert np.array_equal(got[r][f"s{s}_r{r}_dst"], dst[r]), f"{name} step {s} rank {r}: pulled rows"
    for r in range(n):
        assert np.array_equal(got[r][f"final_r{r}_version"], w.get(r, "version"))
        assert np.array_equal(got[r][f"final_r{r}_updates"], w.get(r, "updates"))
        assert np.array_equal(got[r][f"final_r{r}_embedding"].reshape(-1), w.get_f32(r, "embedding").reshape(-1))
        st, nl = w.get(r, "storage"), w.get(r, "nonlocal")
        assert str(got[r]["repr"][0]) == f"<HetuTable root/store/all={st - nl}/{st}/{c['length']}>"
