"""Key ingestion pipeline: batches staged one step ahead give exactly the job that hands host keys to preprocess."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

import hetuctr_b200 as hb  # noqa: E402
from hetuctr_b200.ingest import KeyPipeline  # noqa: E402


def make_table(length, width, emb):
    t = hb.Table(0, 1, 0, "127.0.0.1", 0, length, width, 0, 0, np.zeros(length, np.uint8), np.arange(length),
                 (hb.INIT_ZERO, 0.0, 0.0), 0.1, 0)
    t.set_embedding(emb)
    return t


@pytest.mark.parametrize("depth", [2, 3])
def test_pipeline_equals_direct_calls(depth):
    length, width, steps = 5000, 16, 7
    rng = np.random.RandomState(depth)
    emb = rng.normal(size=(length, width)).astype(np.float32)
    sizes = [900, 1200, 0, 1200, 37, 1200, 600]  # ragged, one empty
    batches = [(rng.zipf(1.3, size=n) - 1) % length for n in sizes]
    grads = [None] + [torch.from_numpy(rng.normal(size=(n, width)).astype(np.float32)).cuda() for n in sizes[:-1]]
    dev = torch.device("cuda", 0)

    direct, out_direct = make_table(length, width, emb), []
    for s in range(steps):
        direct.preprocess(np.ascontiguousarray(batches[s], dtype=np.int64), sizes[s])  # host keys
        dst = torch.full((max(sizes[s], 1), width), float("nan"), device=dev)
        direct.push_pull(grads[s] if s and sizes[s - 1] else None, dst)
        out_direct.append(dst[:sizes[s]].cpu().numpy())

    piped, out_piped = make_table(length, width, emb), []
    pipe = KeyPipeline(piped, iter(batches), max_keys=max(sizes), depth=depth)
    for s, (keys, n) in enumerate(pipe):
        assert keys.is_cuda and n == sizes[s]
        piped.preprocess(keys, n)
        dst = torch.full((max(n, 1), width), float("nan"), device=dev)
        piped.push_pull(grads[s] if s and sizes[s - 1] else None, dst)
        out_piped.append(dst[:n].cpu().numpy())
    assert len(out_piped) == steps
    for a, b in zip(out_direct, out_piped):
        assert np.array_equal(a, b)
    assert np.array_equal(direct.dump("embedding"), piped.dump("embedding"))
    assert np.array_equal(direct.dump("version"), piped.dump("version"))
    direct.close()
    piped.close()


def test_pipeline_step_helper_and_limits():
    length, width = 300, 4
    t = make_table(length, width, np.zeros((length, width), np.float32))
    pipe = KeyPipeline(t, [np.arange(10), np.arange(5, 15)], max_keys=16)
    dst = torch.zeros(16, width, device="cuda")
    assert pipe.step(None, dst)
    assert pipe.step(torch.ones(10, width, device="cuda"), dst)
    assert not pipe.step(None, dst)
    with pytest.raises(ValueError, match="exceeds max_keys"):
        KeyPipeline(t, [np.arange(17)], max_keys=16)
    with pytest.raises(ValueError, match="depth"):
        KeyPipeline(t, [], max_keys=16, depth=1)
    t.close()
