"""Table state export/import: a job that is stopped, saved, rebuilt and loaded continues exactly like the job
that never stopped; damaged or foreign files are refused without touching the table."""
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from gpu_world import GpuWorld, assert_state_parity  # noqa: E402


def hybrid_layout(nrank, length, cache_every, seed):
    rng = np.random.RandomState(seed)
    root = rng.randint(nrank, size=length).astype(np.uint8)
    storage = []
    for r in range(nrank):
        owned = np.where(root == r)[0]
        other = np.where(root != r)[0]
        storage.append(np.sort(np.concatenate([owned, other[::cache_every]])) if nrank > 1 else owned)
    return root, storage


def drive(world, ow, batches, grads, first):
    """Steps `first`.. of the schedule on `world` (and the oracle, when given); returns pulled rows per step."""
    out = []
    for s in range(first, len(batches)):
        world.preprocess(batches[s])
        d = world.push_pull(grads[s])
        if ow is not None:
            ow.preprocess(batches[s])
            do = ow.push_pull(grads[s])
            for r in range(world.nrank):
                assert np.array_equal(d[r], do[r]), f"step {s} rank {r}"
        out.append(d)
    return out


@pytest.mark.parametrize("nrank,bounds", [(1, (0, 0)), (3, (0, 0)), (3, (4, 3))])
def test_resume_equals_uninterrupted(oracle_mod, tmp_path, nrank, bounds):
    length, width, B = 6000, 12, 1500
    root, storage = hybrid_layout(nrank, length, 5, 1)
    rng = np.random.RandomState(2)
    emb0 = [rng.normal(0, 0.1, size=(len(s), width)).astype(np.float32) for s in storage]
    # schedule: 3 steps, an empty batch that flushes the last gradient, then 3 more steps
    keysets = [[(rng.zipf(1.2, size=B) - 1) % length for _ in range(nrank)] for _ in range(3)]
    keysets.append([np.zeros(0, np.int64) for _ in range(nrank)])
    keysets += [[(rng.zipf(1.2, size=B) - 1) % length for _ in range(nrank)] for _ in range(3)]
    grads = [None] + [[rng.normal(0, 0.5, size=(k.size, width)).astype(np.float32) for k in keysets[s - 1]]
                      for s in range(1, len(keysets))]

    def fresh():
        w = GpuWorld(nrank, length, width, bounds[0], bounds[1], 0.1, root, storage)
        for r in range(nrank):
            w.set_embedding(r, emb0[r])
        return w

    ow = oracle_mod.World(nrank, length, width, bounds[0], bounds[1], 0.1, root, storage)
    for r in range(nrank):
        ow.set_embedding(r, emb0[r])
    a = fresh()
    pulled_a = drive(a, ow, keysets, grads, 0)

    b = fresh()
    drive(b, None, keysets[:4], grads[:4], 0)
    files = [str(tmp_path / f"rank{r}.hctr") for r in range(nrank)]
    for r in range(nrank):
        b.tables[r].export_state(files[r])
    b.close()
    c = GpuWorld(nrank, length, width, bounds[0], bounds[1], 0.1, root, storage)  # zero-initialised
    for r in range(nrank):
        c.tables[r].import_state(files[r])
    pulled_c = drive(c, None, keysets, grads, 4)
    for da, dc in zip(pulled_a[4:], pulled_c):
        for r in range(nrank):
            assert np.array_equal(da[r], dc[r])
    assert_state_parity(c, ow)
    assert_state_parity(a, ow)
    a.close()
    c.close()


def test_bad_files_are_refused(tmp_path):
    length, width = 3000, 8
    root, storage = hybrid_layout(1, length, 5, 1)
    w = GpuWorld(1, length, width, 0, 0, 0.1, root, storage)
    emb = np.random.RandomState(0).normal(size=(length, width)).astype(np.float32)
    w.set_embedding(0, emb)
    t = w.tables[0]
    good = str(tmp_path / "good.hctr")
    t.export_state(good)
    raw = open(good, "rb").read()
    assert len(raw) == 64 + length * (8 + 8 + 4 * width) + 8

    def refused(path, match):
        with pytest.raises(RuntimeError, match=match):
            t.import_state(path)
        assert np.array_equal(t.dump("embedding"), emb)  # nothing was overwritten

    bad = str(tmp_path / "bad.hctr")
    flipped = bytearray(raw)
    flipped[len(raw) // 2] ^= 0x10
    open(bad, "wb").write(flipped)
    refused(bad, "corrupt")
    open(bad, "wb").write(raw[: len(raw) // 2])
    refused(bad, "truncated")
    open(bad, "wb").write(b"not a table" * 20)
    refused(bad, "not a table state file")
    refused(str(tmp_path / "missing.hctr"), "cannot open")
    # a table of another width / other stored keys
    other = GpuWorld(1, length, width * 2, 0, 0, 0.1, root, storage)
    with pytest.raises(RuntimeError, match="another shape"):
        other.tables[0].import_state(good)
    other.close()
    perm = GpuWorld(1, length, width, 0, 0, 0.1, root, [storage[0][::-1].copy()])
    with pytest.raises(RuntimeError, match="other keys"):
        perm.tables[0].import_state(good)
    perm.close()
    # between preprocess and push_pull the table refuses to be replaced
    w.preprocess([np.arange(10)])
    with pytest.raises(RuntimeError, match="finish the step"):
        t.import_state(good)
    w.push_pull(None)
    t.import_state(good)
    assert np.array_equal(t.dump("embedding"), emb)
    w.close()
    assert os.path.getsize(good) == len(raw)
