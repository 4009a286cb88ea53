"""The drop-in `hetuCTR` module on ONE GPU, driven the way the reference's own driver script drives it
(tests/driver.py:16-39 of the reference): keyword-only construction, raw addresses for keys / gradients / output,
`preprocess` twice in a row before the first `push_pull`, then preprocess + push_pull per step, with the
synchronous and the `async_*` + `wait()` forms mixed.  Results are compared with the CPU oracle bit for bit.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

import hetuctr_b200 as hb  # noqa: E402


def test_reference_driver_call_pattern_single_rank(oracle_mod):
    hetuCTR = hb.hetuCTR
    length, width, batch_size, lr = 1024, 128, 1024, 0.5
    rng = np.random.RandomState(0)
    root_arr = np.zeros(length, dtype=np.int64)  # the reference's script passes int64; pybind converts
    storage_arr = np.where(root_arr == 0)[0]
    dest = torch.zeros([batch_size, width]).cuda()
    init = hetuCTR.Initializer(hetuCTR.InitType.Normal, 0, 1)
    hetuCTR.seed(7)
    table = hetuCTR.HetuTable(rank=0, nrank=1, device_id=0, ip="127.0.0.1", port=23456, pull_bound=0, push_bound=0,
                              init=init, learning_rate=lr, length=length, width=width, root_arr=root_arr,
                              storage_arr=storage_arr, verbose=0)
    hetuCTR.seed(0)
    assert repr(table) == f"<HetuTable root/store/all={length}/{length}/{length}>"
    assert "width=128" in table.debug()

    # the oracle starts from the rows the initialiser produced
    ow = oracle_mod.World(1, length, width, 0, 0, lr, root_arr.astype(np.uint8), [storage_arr])
    ow.set_embedding(0, table.dump("embedding").reshape(length, width))

    embed_id = np.arange(10, dtype=np.int64)
    table.preprocess(embed_id.ctypes.data, embed_id.shape[0])
    table.preprocess(embed_id.ctypes.data, embed_id.shape[0])  # the older batch's gradient is never pushed
    ow.preprocess([embed_id])
    ow.preprocess([embed_id])
    grad = torch.zeros([batch_size, width]).cuda()
    table.push_pull(grad.data_ptr(), dest.data_ptr())
    want = ow.push_pull([np.zeros((10, width), dtype=np.float32)])[0]
    assert np.array_equal(dest[:10].cpu().numpy(), want)

    prev_n = 10
    for i in range(12):
        n = batch_size if i % 4 else 37 + i  # ragged sizes in between
        embed_id = rng.randint(length, size=n).astype(np.int64)
        g = rng.normal(0, 1, size=(prev_n, width)).astype(np.float32)
        grad[:prev_n] = torch.from_numpy(g).cuda()
        if i % 2:
            table.async_preprocess(embed_id.ctypes.data, n).wait()
        else:
            keys_dev = torch.from_numpy(embed_id).cuda()  # device-resident keys are accepted too
            table.preprocess(keys_dev.data_ptr(), n)
        ow.preprocess([embed_id])
        if i % 3 == 0:
            table.async_push_pull(grad.data_ptr(), dest.data_ptr()).wait()
        else:
            table.push_pull(grad.data_ptr(), dest.data_ptr())
        want = ow.push_pull([g])[0]
        assert np.array_equal(dest[:n].cpu().numpy(), want), f"step {i}: pulled rows differ"
        for name in ("unique_idx", "idx_map", "sorted_arg", "run_length", "root", "offset"):
            assert np.array_equal(table.dump(name), ow.get(0, name)), f"step {i}: {name}"
        prev_n = n
    # an inference step: no gradient
    embed_id = rng.randint(length, size=batch_size).astype(np.int64)
    table.preprocess(embed_id.ctypes.data, batch_size)
    ow.preprocess([embed_id])
    table.push_pull(0, dest.data_ptr())
    assert np.array_equal(dest.cpu().numpy(), ow.push_pull(None)[0])
    assert np.array_equal(table.dump("embedding").reshape(-1), ow.get_f32(0, "embedding").reshape(-1))
    assert np.array_equal(table.dump("version"), ow.get(0, "version"))
