"""BASELINE configurations at their FULL sizes on one GPU, checked through size-independent properties (the CPU
oracle cannot hold tables of this size in reasonable time): canonical order of the unique keys, the batch->unique
map composes back to the keys, position lists are ascending partitions of the batch, equal keys pull equal rows,
an inference step changes nothing, and one SGD step moves every sampled row by exactly -lr * sum of its gradients.

Single-rank versions of config 2 (33.76M x 128, Zipf 1.05, 8192 x 26), config 4 (1e8 x 32, uniform, 32768 x 26) and
config 5 (5e7 x 256, Zipf 1.1, 4096 x 26); config 3 (256 GB) does not fit one GPU and is covered at reduced length by
the multi-rank parity tests.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

import hetuctr_b200 as hb  # noqa: E402
from hetuctr_b200.workloads import CONFIGS, KeySampler  # noqa: E402


def _free_gb():
    free, _ = torch.cuda.mem_get_info()
    return free / 1e9


@pytest.mark.parametrize("cfg", ["cfg2_hybrid", "cfg4_stress", "cfg5_sweep"])
def test_full_size_properties(cfg):
    c = CONFIGS[cfg]
    N, W, B = c["rows"], c["width"], c["samples"] * c["fields"]
    need_gb = N * W * 4 / 1e9 + N * 6 / 1e9 + 4
    if _free_gb() < need_gb:
        pytest.skip(f"needs {need_gb:.0f} GB of device memory")
    dev = torch.device("cuda:0")
    sampler = KeySampler(N, c["fields"], c["alpha"], c["ratio"])
    rng = np.random.RandomState(17)
    root = np.zeros(N, dtype=np.uint8)
    hb.lib().hctr_seed(0)
    t = hb.Table(0, 1, 0, "127.0.0.1", 0, N, W, 0, 0, root, np.arange(N, dtype=np.int64),
                 (hb.INIT_NORMAL, 0.0, c["init_std"]), c["lr"], 0)
    lr = np.float32(c["lr"])
    dst = torch.empty(B, W, device=dev)
    keys0 = sampler.batch(c["samples"], rng)
    keys1 = keys0.copy()
    rng.shuffle(keys1)  # same multiset, other positions: every key of batch 0 is pulled again
    k0 = torch.from_numpy(keys0).to(dev)
    k1 = torch.from_numpy(keys1).to(dev)

    # ---- batch 0: index structure
    t.preprocess(k0, B)
    t.push_pull(None, dst)
    uniq, idx_map = t.dump("unique_idx"), t.dump("idx_map")
    runs, pos = t.dump("run_length"), t.dump("sorted_arg")
    assert np.all(np.diff(uniq) > 0), "unique keys must be strictly ascending (one owner)"
    assert np.array_equal(uniq, np.unique(keys0))
    assert np.array_equal(uniq[idx_map], keys0)
    assert runs[0] == 0 and runs[-1] == B and np.all(np.diff(runs) >= 1)
    assert np.array_equal(np.sort(pos), np.arange(B)), "position lists must partition the batch"
    assert np.array_equal(idx_map[pos], np.repeat(np.arange(len(uniq)), np.diff(runs))), "runs group equal keys"
    inside = np.ones(B, dtype=bool)
    inside[runs[:-1]] = False
    assert np.all(np.diff(pos)[inside[1:]] > 0), "positions ascend inside every run"
    rows0 = dst.cpu().numpy()
    first = pos[runs[:-1]]
    assert np.array_equal(rows0, rows0[first][idx_map]), "equal keys must pull equal rows"

    # ---- an inference step changes nothing
    t.preprocess(k0, B)
    t.push_pull(None, dst)
    assert np.array_equal(dst.cpu().numpy(), rows0)

    # ---- one SGD step: row_after = row_before - lr * (sum of the key's gradient rows, batch order)
    g = torch.Generator(device=dev)
    g.manual_seed(3)
    grad = torch.randn(B, W, device=dev, generator=g) * 0.01
    t.preprocess(k1, B)
    t.push_pull(grad, dst)  # gradient belongs to the previous batch (keys0), rows are pulled for keys1
    rows1 = dst.cpu().numpy()
    grad_h = grad.cpu().numpy()
    sample = rng.choice(len(uniq), size=min(3000, len(uniq)), replace=False)
    heavy = np.argsort(-np.diff(runs))[:20]  # the hottest keys too
    where1 = {int(k): i for i, k in enumerate(keys1)}
    for u in np.concatenate([sample, heavy]):
        ps = pos[runs[u]:runs[u + 1]]
        s = np.zeros(W, dtype=np.float32)
        for p in ps:  # sequential fp32 sum in batch order, then one multiply: the reference's order
            s = s + grad_h[p]
        expect = rows0[ps[0]] + s * (-lr)
        got = rows1[where1[int(uniq[u])]]
        assert np.array_equal(got, expect.astype(np.float32)), f"key {uniq[u]} ({len(ps)} occurrences)"
    t.close()
