"""One rank of a multi-process job through the drop-in `hetuCTR` module (NCCL transport), one GPU per rank.
Replays a golden case and writes every observable array to an .npz for the parent test to compare.

  python tests/mp_worker.py <case> <rank> <port> <out.npz>
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.join(HERE, "golden"))


def main():
    name, rank, port, out_path = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
    import torch

    import cases
    import hetuctr_b200 as hb

    hetuCTR = hb.hetuCTR
    c, root, storage, emb, keys, grads = cases.make_inputs(name)
    n, W = c["nrank"], c["width"]
    torch.cuda.set_device(rank)
    init = hetuCTR.Initializer(hetuCTR.InitType.Zero, 0, 0)
    t = hetuCTR.HetuTable(rank=rank, nrank=n, device_id=rank, ip="127.0.0.1", port=port, length=c["length"], width=W,
                          pull_bound=c["pull"], push_bound=c["push"], root_arr=root, storage_arr=storage[rank],
                          init=init, learning_rate=c["lr"], verbose=0)
    t.set_embedding(cases.layout_rows(root, storage[rank], rank, emb[rank]))
    out = {}
    dst = torch.zeros(c["batch"], W, device="cuda")
    for s in range(c["steps"]):
        k = keys[s][rank]
        # alternate host / device key buffers and sync / async calls: all are part of the reference's API
        if s % 2 == 0:
            t.preprocess(k.ctypes.data, k.size)
        else:
            kd = torch.from_numpy(k).cuda()
            t.async_preprocess(kd.data_ptr(), k.size).wait()
        for a in cases.INDEX_ARRAYS:
            out[f"s{s}_r{rank}_{a}"] = t.dump(a)
        g = None if grads[s] is None else torch.from_numpy(grads[s][rank]).cuda()
        if s % 3 == 2:
            t.async_push_pull(0 if g is None else g.data_ptr(), dst.data_ptr()).wait()
        else:
            t.push_pull(0 if g is None else g.data_ptr(), dst.data_ptr())
        out[f"s{s}_r{rank}_dst"] = dst.cpu().numpy().copy()
    for a in cases.STATE_ARRAYS:
        out[f"final_r{rank}_{a}"] = t.dump(a)
    out["repr"] = np.array([repr(t), t.debug()])
    np.savez_compressed(out_path, **out)


if __name__ == "__main__":
    main()
