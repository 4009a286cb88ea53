"""Records what the reference's offline partitioner computes, as fixtures for tests/test_partition.py.

  python oracle/build_ref.py            # builds oracle/_ref/partition/hetuCTR_partition*.so (no OpenMP: sequential)
  python tests/golden/make_partition_golden.py

Each case draws a seeded synthetic click log (samples x slots of embedding ids with cluster structure), runs the
reference module's partition() and a few refine_data()/refine_embed() rounds, and stores the starting assignment
(the reference draws it with rand()) together with the assignment, counts, communication matrix and caching
priority after every round.  A test replays the same rounds from the same starting assignment.
"""
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from tests.golden.partition_cases import CASES, make_case  # noqa: E402


def load_reference():
    from oracle import build_ref
    path = build_ref.build_partition()
    spec = importlib.util.spec_from_file_location("hetuCTR_partition", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    ref = load_reference()
    for name, cfg in CASES.items():
        data, comm = make_case(cfg)
        p = ref.partition(data, comm, cfg["n_part"], cfg["batch_size"])
        out = {}
        d0, e0 = p.get_result()
        out["init_data"], out["init_embed"] = np.array(d0), np.array(e0)
        out["init_comm"] = np.array(p.get_communication())
        out["init_priority"] = np.array(p.get_priority())
        for r in range(cfg["rounds"]):
            p.refine_data()
            d, e = p.get_result()
            out[f"r{r}_data_after_data"] = np.array(d)
            p.refine_embed()
            d, e = p.get_result()
            out[f"r{r}_data"], out[f"r{r}_embed"] = np.array(d), np.array(e)
            out[f"r{r}_data_cnt"] = np.array(p.get_data_cnt())
            out[f"r{r}_embed_cnt"] = np.array(p.get_embed_cnt())
            out[f"r{r}_comm"] = np.array(p.get_communication())
        out["final_priority"] = np.array(p.get_priority())
        path = os.path.join(HERE, f"partition_{name}.npz")
        np.savez_compressed(path, **out)
        cost = lambda c: float((np.asarray(c) * comm).sum())
        print(name, "cost", cost(out["init_comm"]), "->", cost(out[f"r{cfg['rounds'] - 1}_comm"]),
              os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
