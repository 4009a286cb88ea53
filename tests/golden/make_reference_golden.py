"""Records the REFERENCE's outputs for the golden cases (run on a GPU box; needs oracle/_ref built and as many
GPUs as the largest case has ranks).  Writes tests/golden/<case>.npz and tests/golden/init_values.npz.

  python tests/golden/make_reference_golden.py [--out DIR] [case ...]

One process per rank, exactly as the reference is meant to run (reference tests/test_update.py:84-87); each rank
dumps the reference's internal arrays after every preprocess and its pulled rows after every push_pull.
"""
import multiprocessing as mp
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))
sys.path.insert(0, HERE)

import cases  # noqa: E402


def worker(name, rank, port, q):
    import hetuCTR_ref as ref

    c, root, storage, emb, keys, grads = cases.make_inputs(name)
    n, W = c["nrank"], c["width"]
    t = ref.HetuTable(rank=rank, nrank=n, device_id=rank, ip="127.0.0.1", port=port, length=c["length"], width=W,
                      pull_bound=c["pull"], push_bound=c["push"], root_arr=root, storage_arr=storage[rank],
                      init_kind=0, init_a=0.0, init_b=0.0, learning_rate=c["lr"], verbose=0)
    out = {}

    def put(key, rows):  # float rows: whole, or as a digest for the wide-row cases
        if c.get("digest"):
            for part, v in cases.digest(rows, W).items():
                out[f"{key}.{part}"] = v
        else:
            out[key] = rows

    t.set_embedding(cases.layout_rows(root, storage[rank], rank, emb[rank]))
    for s in range(c["steps"]):
        k = keys[s][rank]
        t.preprocess(k.ctypes.data, k.size)
        for a in cases.INDEX_ARRAYS:
            out[f"s{s}_r{rank}_{a}"] = t.dump(a)
        put(f"s{s}_r{rank}_dst", t.push_pull_np(None if grads[s] is None else grads[s][rank], k.size))
    for a in cases.STATE_ARRAYS:
        if a in ("embedding", "gradient"):
            put(f"final_r{rank}_{a}", t.dump(a))
        else:
            out[f"final_r{rank}_{a}"] = t.dump(a)
    q.put(out)


def record_case(name, outdir, port):
    c = cases.CASES[name]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(name, r, port, q)) for r in range(c["nrank"])]
    for p in procs:
        p.start()
    merged = {}
    for _ in procs:
        merged.update(q.get(timeout=300))
    for p in procs:
        p.join(60)
    np.savez_compressed(os.path.join(outdir, name + ".npz"), **merged)
    print("recorded", name, len(merged), "arrays")


def record_init(outdir):
    import hetuCTR_ref as ref
    out = {}
    for name, (kind, a, b, seed, n) in cases.INIT_CASES.items():
        ref.seed(seed)
        t = ref.HetuTable(rank=0, nrank=1, device_id=0, ip="127.0.0.1", port=23999, length=n, width=1, pull_bound=0,
                          push_bound=0, root_arr=np.zeros(n, dtype=np.uint8), storage_arr=np.arange(n),
                          init_kind=kind, init_a=a, init_b=b, learning_rate=0.0, verbose=0)
        out[name] = t.dump("embedding")
        del t
    np.savez_compressed(os.path.join(outdir, "init_values.npz"), **out)
    print("recorded init values")


def gpu_count():
    import subprocess
    try:
        return len(subprocess.run(["nvidia-smi", "-L"], stdout=subprocess.PIPE, text=True).stdout.strip().splitlines())
    except OSError:
        return 0


if __name__ == "__main__":
    args = sys.argv[1:]
    outdir = HERE
    if "--out" in args:
        i = args.index("--out")
        outdir = args[i + 1]
        del args[i:i + 2]
    os.makedirs(outdir, exist_ok=True)
    names = args or list(cases.CASES)
    ngpu = gpu_count()
    port = 24100
    for name in names:
        if cases.CASES[name]["nrank"] > ngpu:
            print("skipped", name, "(needs", cases.CASES[name]["nrank"], "GPUs)")
            continue
        port += 7
        record_case(name, outdir, port)
    mp.get_context("spawn").Process(target=record_init, args=(outdir,)).start()
