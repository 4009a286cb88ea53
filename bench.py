"""Benchmark of the HetuTable hot path: lookup+update keys/s (preprocess + push_pull with real gradients).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--config cfg2_hybrid] [--impl ours|reference]

One process per GPU (under torchrun for N > 1).  A step = preprocess(keys of batch k) then
push_pull(gradients of batch k-1, dst of batch k) on one batch of synthetic keys.  Prints ONE JSON line.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from hetuctr_b200.workloads import CONFIGS, KeySampler, random_owners, storage_with_cache  # noqa: E402

METRIC = "lookup+update keys/s"
UNIT = "keys/s"
N_BATCHES = 6  # distinct pre-generated batches / gradient buffers, cycled


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--config", default="cfg2_hybrid", choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=20)
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="CPU work in the cpu_baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--timeline", action="store_true",
                    help="after the run, time three more steps phase by phase and print where they ran (stderr)")
    ap.add_argument("--layout", default="benchmark", choices=["benchmark", "graph", "random"],
                    help="benchmark: the reference benchmark's layout (random owners, per-rank batch streams). "
                         "graph / random: batches drawn from one clustered click log that is laid out by the offline "
                         "partitioner or dealt at random (the config-5 comparison, N > 1)")
    ap.add_argument("--log-samples", type=int, default=0, help="click log size for --layout graph/random")
    ap.add_argument("--width", type=int, default=0, help="override the row width (small ncu captures only)")
    ap.add_argument("--rows", type=int, default=0,
                    help="override the table length (small ncu captures only; the line is then not a bench value)")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def bind_to_gpu_numa_node(gpu_index):
    """Pins this process to the CPU cores of the NUMA node its GPU hangs off, BEFORE any pinned host buffer is
    allocated, so that those buffers (first touch) and the threads that drive the copies are local to the GPU's PCIe
    root.  A launcher such as torchrun binds nothing; with eight ranks moving 220 MB per step each, buffers on the
    wrong socket make every copy cross the inter-socket link.  Used by both arms.  Returns a description."""
    try:
        bus = subprocess.run(["nvidia-smi", "--query-gpu=pci.bus_id", "--format=csv,noheader", "-i", str(gpu_index)],
                             stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True).stdout.strip().lower()
        if not bus:
            return {"numa_node": None}
        dom, rest = bus.split(":", 1)
        path = f"/sys/bus/pci/devices/{dom[-4:]}:{rest}/numa_node"
        node = int(open(path).read().strip())
        if node < 0:
            return {"numa_node": None}
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return {"numa_node": node, "cpus": 0}
        os.sched_setaffinity(0, cpus)
        return {"numa_node": node, "cpus": len(cpus)}
    except (OSError, ValueError):
        return {"numa_node": None}


def make_job_workload(cfg, nrank, rank, layout, log_samples):
    """Batches of one shared clustered click log; owners, caches and the rank of every sample either from the
    offline partitioner ("graph") or dealt at random ("random")."""
    from hetuctr_b200.workloads import partitioned_job, random_job
    c = dict(CONFIGS[cfg])
    log_samples = log_samples or 64 * c["samples"] * nrank
    cache_rows = max(int(c["rows"] * 0.02), 1)
    if layout == "graph":
        root, storage, mine, data = partitioned_job(cfg, nrank, log_samples, cache_rows,
                                                    log=(lambda m: print(m, file=sys.stderr)) if rank == 0 else None)
    else:
        root, storage, mine, data = random_job(cfg, nrank, log_samples, cache_rows)
    rng = np.random.RandomState(1000 * int(cfg[3]) + rank)
    batches = [data[rng.choice(mine[rank], c["samples"])].reshape(-1).astype(np.int64) for _ in range(N_BATCHES)]
    return c, root, storage[rank], batches


def make_workload(cfg, nrank, rank, rows=0, width=0):
    c = dict(CONFIGS[cfg])
    if rows:
        c["rows"] = rows
    if width:
        c["width"] = width
    sampler = KeySampler(c["rows"], c["fields"], c["alpha"], c["ratio"])
    root = random_owners(c["rows"], nrank)
    cache_rows = int(c["rows"] * c["cache"]) if nrank > 1 else 0
    storage = storage_with_cache(root, rank, sampler, cache_rows)
    cfg_id = int(cfg[3])
    rng = np.random.RandomState(1000 * cfg_id + rank)
    batches = [sampler.batch(c["samples"], rng) for _ in range(N_BATCHES)]
    return c, root, storage, batches


def algorithmic_bytes(c, st):
    """Algorithmic HBM bytes per step of each phase (D = 4*width bytes per row):
       dedupe            : 8B (keys) + B (owner lookups) + 4B (batch->unique map) + 17 per unique key
       reduce+apply+pack : B*D (gradients) + 2*D per locally stored unique row + (D+16) per pushed row
       owner update      : G*(D+16) (message) + G*2D (row read+write) + G*16 (version read+write)
       stale check+gather: Q*24 + R_s*(2D+8)
       expand            : D per unique row + B*D (dst) + 4*B (batch->unique map)"""
    D = 4 * c["width"]
    B, U = st["batch"], st["unique"]
    Bp, Up, P = st["prev_batch"], st["prev_unique"], st["pushed_rows"]
    G, Q, Rs = st["received_push_rows"], st["queried_keys"], st["returned_rows"]
    stored = max(Up - P, 0) + min(P, Up)  # every unique row is either applied locally, pushed, or both (cached)
    return {"dedupe": 13 * B + 17 * U, "reduce": Bp * D + stored * 2 * D + P * (D + 16),
            "owner_update": G * (3 * D + 32), "stale_gather": Q * 24 + Rs * (2 * D + 8),
            "expand": U * D + B * D + 4 * B}


def nvlink_bytes(c, st, world):
    """Algorithmic bytes ONE GPU stores into its peers' memory per step: queries (key + version, 16 B) for the keys
    other ranks own, pushed rows (row + key + count), one flag byte per remote query answered, returned rows
    (row + version).  Keys addressed to the rank itself stay local: with random owners that is 1/world of them."""
    D = 4 * c["width"]
    remote = (world - 1) / world
    return {"queries": 16 * st["unique"] * remote, "pushed_rows": st["pushed_rows"] * (D + 16),
            "flags": st["queried_keys"] * remote, "returned_rows": st["returned_rows"] * (D + 8)}


def run_ours(args):
    import torch
    import torch.distributed as dist

    import hetuctr_b200 as hb

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    all_cpus = os.sched_getaffinity(0)
    binding = bind_to_gpu_numa_node(local)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.layout == "benchmark":
        c, root, storage, batches = make_workload(args.config, world, rank, args.rows, args.width)
    else:
        c, root, storage, batches = make_job_workload(args.config, world, rank, args.layout, args.log_samples)
    W, B = c["width"], c["samples"] * c["fields"]
    addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ.get("MASTER_PORT", 29500)) + 101
    hb.lib().hctr_seed(0)
    table = hb.Table(rank, world, local, addr, port, c["rows"], W, c["pull_bound"], c["push_bound"], root, storage,
                     (hb.INIT_NORMAL, 0.0, c["init_std"]), c["lr"], 0)
    keys_dev = [torch.from_numpy(b).to(dev) for b in batches]
    g = torch.Generator(device=dev)
    g.manual_seed(1234 + rank)
    grads = [torch.randn(B, W, device=dev, generator=g) * 0.01 for _ in range(N_BATCHES)]
    dst = torch.empty(B, W, device=dev)
    stream = torch.cuda.ExternalStream(table.stream(), device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step(i, host=False):
        j = i % N_BATCHES
        if host:
            table.preprocess(keys_host[j], B)
            table.push_pull(grads_host[(j - 1) % N_BATCHES], dst_host)
        else:
            table.preprocess(keys_dev[j], B)
            table.push_pull(grads[(j - 1) % N_BATCHES], dst)

    # prime the pipeline (the first push_pull has no previous batch), then warm up
    table.preprocess(keys_dev[-1], B)
    table.push_pull(None, dst)
    clocks = ClockSampler(local)
    if rank == 0:
        # sampling covers warm-up, timed region and the end-to-end region, all under the same load; a short run
        # (the timed region of 20 steps lasts milliseconds) keeps stepping until the sampler has delivered
        clocks.start()
    for i in range(args.warmup):
        step(i)
    # every rank takes the same number of steps (a step is collective): rank 0 decides, the others follow
    t_wait, i = time.perf_counter(), 0
    while True:
        more = torch.tensor([1 if rank == 0 and len(clocks.lines) < 3 and time.perf_counter() - t_wait < 3.0 else 0],
                            device=dev)
        if world > 1:
            dist.broadcast(more, 0)
        if int(more.item()) == 0:
            break
        for _ in range(50):
            step(i)
            i += 1

    # phase timers on every 8th step: their events cost a timed step ~15 us, sampling keeps `value` honest
    PROFILE_EVERY = 8
    table.profile(PROFILE_EVERY)
    table.phase_times(reset=True)
    launches0 = hb.lib().hctr_launch_count()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    t0 = time.perf_counter()
    for i in range(args.steps):
        step(i)
    e1.record(stream)
    barrier()
    wall = time.perf_counter() - t0
    ms = e0.elapsed_time(e1)
    launches = hb.lib().hctr_launch_count() - launches0
    phases = table.phase_times(reset=True)
    table.profile(False)
    stats = table.stats()

    # end to end through the same calls with HOST buffers: keys, gradients and dst live in pinned host
    # memory; every step copies keys + gradients in and the pulled rows out
    keys_host = [torch.from_numpy(b).pin_memory().numpy() for b in batches]
    grads_host = [x.cpu().pin_memory() for x in grads[:3]] * 2
    dst_host = torch.empty(B, W).pin_memory()
    for i in range(3):
        step(i, host=True)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record(stream)
    for i in range(args.e2e_steps):
        step(i, host=True)
    f1.record(stream)
    barrier()
    e2e_ms = f0.elapsed_time(f1)
    clk = clocks.stop() if rank == 0 else None

    if args.timeline:
        table.profile(1)
        for i in range(3):
            step(i)
        barrier()
        spans = table.timeline()
        table.profile(0)
        if rank == 0 and spans:
            t_first = spans[0][1]
            for ph, a, b in spans:
                print(f"timeline {ph:13s} {1e3 * (a - t_first):8.1f} -> {1e3 * (b - t_first):8.1f} us ({1e3 * (b - a):6.1f})",
                      file=sys.stderr)
        # the same with host buffers: where the two transfers over the host link and the kernels between them lie
        table.profile(1)
        for i in range(3):
            step(i, host=True)
        barrier()
        spans = table.timeline()
        table.profile(0)
        if rank == 0 and spans:
            t_first = spans[0][1]
            for ph, a, b in spans:
                print(f"timeline(host buffers) {ph:13s} {1e3 * (a - t_first):8.1f} -> {1e3 * (b - t_first):8.1f} us "
                      f"({1e3 * (b - a):6.1f})", file=sys.stderr)

    t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()

    out = None
    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        peak = peaks.get("hbm_gbs", 6650.0)
        peak_src = "measured" if "hbm_gbs" in peaks else "fallback"
        alg = algorithmic_bytes(c, stats)
        per_phase = {p: (v[0] / v[1] if v[1] else 0.0) for p, v in phases.items()}
        timed_steps = (args.steps + PROFILE_EVERY - 1) // PROFILE_EVERY
        # the row-moving kernels; the dominant one (longest launch) is the line's `roofline`, all of them (and the
        # latency-bound dedupe pipeline, whose working set lives in L2) are listed under `roofline_phases`
        kernels = {"reduce": "grad_reduce_apply_pack", "expand": "expand_rows", "owner_update": "owner_mark + owner_apply",
                   "stale_gather": "p2p_stale_gather", "dedupe": "dedupe pipeline (5 launches)"}
        if world > 1 and per_phase.get("expand", 0.0) > 0 and per_phase.get("refresh", 0.0) == 0:
            # requester side of the mailbox exchange as one launch: the expansion plus the per-key flag look-ups of
            # the cache refresh (the refreshed rows themselves, 3D each, are not counted: their number stays on the
            # device)
            kernels["expand"] = "p2p_refresh_expand"
            alg["expand"] += 14 * stats["unique"]
        # the owner's row pass runs on a second stream next to the staleness scan: charge it to owner_update
        per_phase["owner_update"] = per_phase.get("owner_update", 0.0) + per_phase.get("owner_apply", 0.0)
        gather_only_ms = per_phase.get("stale_gather", 0.0)  # the peer-to-peer exchange times scan and gather apart
        per_phase["stale_gather"] = gather_only_ms + per_phase.get("stale_scan", 0.0)
        movers = [p for p in ("reduce", "expand", "owner_update", "stale_gather") if per_phase.get(p, 0.0) > 0]
        dom = max(movers, key=lambda p: per_phase[p])
        achieved = alg[dom] / (per_phase[dom] * 1e-3) / 1e9 if per_phase[dom] > 0 else 0.0
        roofline_phases = {p: {"kernel": kernels[p], "avg_launch_ms": per_phase[p], "algorithmic_bytes": alg[p],
                               "achieved_gbs": alg[p] / (per_phase[p] * 1e-3) / 1e9,
                               "frac": alg[p] / (per_phase[p] * 1e-3) / 1e9 / peak}
                           for p in movers + ["dedupe"] if per_phase.get(p, 0.0) > 0}
        traffic, traffic_note = None, None
        tfile = os.path.join(ROOT, "profiles", "traffic.json")
        if os.path.exists(tfile):
            tj = json.load(open(tfile))
            key = f"{args.config}:n{world}:{dom}"
            if key in tj:
                traffic = tj[key]["bytes_per_launch"]
                traffic_note = tj[key].get("source")
        nvlink = None
        if world > 1:
            nb = nvlink_bytes(c, stats, world)
            sent = sum(nb.values())
            store_ms = per_phase["reduce"] + per_phase.get("query", 0.0) + per_phase.get("stale_gather", 0.0)
            gather_ms = gather_only_ms if per_phase.get("stale_scan", 0.0) > 0 else per_phase.get("stale_gather", 0.0)
            nvlink = {"bytes_sent_per_gpu_per_step": sent, "parts": nb, "peak": 900.0, "unit": "GB/s per direction",
                      "step_gbs": sent / (ms / args.steps * 1e-3) / 1e9,
                      "step_frac": sent / (ms / args.steps * 1e-3) / 1e9 / 900.0,
                      "store_kernels_ms": store_ms,
                      "store_kernels_gbs": sent / (store_ms * 1e-3) / 1e9 if store_ms > 0 else 0.0,
                      "store_kernels_frac": sent / (store_ms * 1e-3) / 1e9 / 900.0 if store_ms > 0 else 0.0,
                      "gather_gbs": nb["returned_rows"] / (gather_ms * 1e-3) / 1e9 if gather_ms > 0 else 0.0,
                      "gather_frac": nb["returned_rows"] / (gather_ms * 1e-3) / 1e9 / 900.0 if gather_ms > 0 else 0.0,
                      "how": "algorithmic bytes this GPU stores into peer memory per step (counts of the last step) "
                             "over (a) the step, (b) the CUDA-event time of the kernels that issue the stores "
                             "(reduce: pushed rows; query: keys+versions; stale_gather: flags + returned rows), "
                             "(c) returned rows over the gather kernel alone",
                      "wait_for_peers_us": {"queries": stats["wait_queries_us"], "returned_rows": stats["wait_returns_us"]}}
        out = {
            "metric": METRIC, "value": world * B * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.config + (" (size overridden)" if args.rows or args.width else ""), "rows": c["rows"], "width": W, "keys_per_gpu_per_step": B,
                       "unique_per_gpu_per_step": stats["unique"], "key_distribution":
                       "uniform" if c["alpha"] is None else f"zipf({c['alpha']}) per field, {c['fields']} fields",
                       "cache_fraction": c["cache"] if world > 1 else 0.0, "pull_bound": c["pull_bound"],
                       "push_bound": c["push_bound"], "lr": c["lr"], "partition": {"benchmark": f"random owners x{world}",
                                     "graph": f"offline partitioner (5 rounds) x{world}, clustered click log",
                                     "random": f"random owners x{world}, clustered click log"}[args.layout],
                       "rows_moved_per_gpu_per_step": stats["pushed_rows"] + stats["received_rows"],
                       "l2": f"{N_BATCHES} rotating batches; >= {2 * B * 4 * W / 1e6:.0f} MB streamed per step exceeds the 126 MB L2"
                       if 2 * B * 4 * W > 126e6 else f"{N_BATCHES} rotating batches (per-step data smaller than L2)",
                       "transport": table.exchange_name()},
            "e2e": {"value": world * B * args.e2e_steps / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": B * 8 + B * W * 4, "d2h_bytes_per_step": B * W * 4,
                    "ms_per_step": e2e_ms / args.e2e_steps, "steps": args.e2e_steps,
                    "host_gbs_per_gpu": (B * 8 + 2 * B * W * 4) / (e2e_ms / args.e2e_steps * 1e-3) / 1e9,
                    "host_binding": binding},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "kernel": kernels[dom],
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_src, "algorithmic_bytes_per_launch": alg[dom],
                         "avg_launch_ms": per_phase[dom], "traffic": traffic, "traffic_source": traffic_note},
            "roofline_phases": roofline_phases,
            "phase_ms_per_step": {p: phases[p][0] / timed_steps for p in phases},
            "phase_timers": f"CUDA events on every {PROFILE_EVERY}th step of the timed region ({timed_steps} steps)",
            "wall_ms_per_step": wall * 1e3 / args.steps,
            "clocks": clk,
        }
        if nvlink:
            out["nvlink"] = nvlink
        # the CPU baseline is a single-GPU-run item (a multi-rank launcher also pins OpenMP to one thread)
        if not args.no_cpu_baseline and world == 1:
            os.sched_setaffinity(0, all_cpus)  # the CPU baseline uses every host core
            out["cpu_baseline"] = cpu_baseline(args, world)
    table.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return out


def cpu_baseline(args, world, seconds=None):
    """The CPU port of the same semantics (oracle, OpenMP build) on the host cores: all `world` logical ranks in
    one process, same table size and batches, a bounded number of steps."""
    from oracle import build as obuild
    from oracle.hetu_oracle import World

    obuild.build()
    seconds = seconds or args.cpu_seconds
    works = [make_workload(args.config, world, r) for r in range(world)]
    c = works[0][0]
    W, B = c["width"], c["samples"] * c["fields"]
    ow = World(world, c["rows"], W, c["pull_bound"], c["push_bound"], c["lr"], works[0][1], [w[2] for w in works],
               parallel=True)
    rng = np.random.RandomState(99)
    grad = (rng.standard_normal((B, W)) * 0.01).astype(np.float32)
    ow.preprocess([w[3][0] for w in works])
    ow.push_pull(None)
    t0 = time.perf_counter()
    steps = 0
    while steps < 3 or (time.perf_counter() - t0 < seconds and steps < 5000):
        ow.preprocess([w[3][(steps + 1) % N_BATCHES] for w in works])
        ow.push_pull([grad] * world)
        steps += 1
    dt = time.perf_counter() - t0
    return {"value": world * B * steps / dt, "unit": UNIT, "cores": ow.num_threads(), "kind": "port",
            "sample": f"{steps} steps of {args.config} ({world} logical rank(s) in one process, zero-initialised table, "
                      f"{dt:.1f} s)"}


def _ref_module():
    """The reference's own CUDA build (oracle/_ref), or None when it is not there / cannot load."""
    path = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.isdir(path):
        return None
    sys.path.insert(0, path)
    try:
        import hetuCTR_ref
        return hetuCTR_ref
    except Exception:  # noqa: BLE001 - fall back to the CPU port
        return None


def _gpu_present():
    try:
        return subprocess.run(["nvidia-smi", "-L"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL).returncode == 0
    except OSError:
        return False


def run_reference(args):
    """Reference arm.  The reference is GPU-only: when its own CUDA build (oracle/_ref, compiled from the reference's
    sources by oracle/build_ref.py) loads on this box it is what gets timed — same config, same synthetic batches,
    its own preprocess()/pushPull() — one process per GPU.  Otherwise the CPU port of its semantics (oracle/, all host
    threads) stands in.  No PyTorch in these processes: the reference build links its own CUDA runtime."""
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    c = CONFIGS[args.config]
    B = c["samples"] * c["fields"]
    ref = _ref_module() if _gpu_present() else None
    binding = bind_to_gpu_numa_node(local) if ref is not None else None
    if ref is None:
        if rank != 0:
            return None
        t0 = time.perf_counter()
        # --steps scales the sample: about 0.1 s of CPU work per requested step, 10-60 s in total
        cb = cpu_baseline(args, world, seconds=min(60.0, max(10.0, 0.1 * args.steps)))
        steps = int(cb["sample"].split(" steps")[0])
        return {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": world,
                "steps": steps, "warmup": 1, "ms_per_step": world * B / cb["value"] * 1e3, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": args.config, "rows": c["rows"], "width": c["width"],
                           "keys_per_gpu_per_step": B},
                "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "total_s": time.perf_counter() - t0}

    if args.layout == "benchmark":
        c, root, storage, batches = make_workload(args.config, world, rank, args.rows, args.width)
    else:
        c, root, storage, batches = make_job_workload(args.config, world, rank, args.layout, args.log_samples)
    W = c["width"]
    addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ.get("MASTER_PORT", 29500)) + 203
    ref.seed(0)
    table = ref.HetuTable(rank=rank, nrank=world, device_id=local, ip=addr, port=port, length=c["rows"], width=W,
                          pull_bound=c["pull_bound"], push_bound=c["push_bound"], root_arr=root, storage_arr=storage,
                          init_kind=1, init_a=0.0, init_b=c["init_std"], learning_rate=c["lr"], verbose=0)
    grad = (np.random.RandomState(1234 + rank).standard_normal((B, W)) * 0.01).astype(np.float32)
    steps, warmup = args.steps, max(args.warmup, 3)
    clocks = ClockSampler(local) if rank == 0 else None
    if clocks:
        clocks.start()
    ms = table.bench_loop(batches, grad, steps, warmup, False)
    e2e_steps = max(3, min(args.e2e_steps, steps))
    e2e_ms = table.bench_loop(batches, grad, e2e_steps, 2, True)
    clk = clocks.stop() if clocks else None
    del table
    # max over ranks through a scratch directory (no collective library in these processes)
    tag = os.environ.get("MASTER_PORT", "0")
    d = os.path.join("/tmp", f"hctr_ref_bench_{tag}")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, f"r{rank}.json.tmp"), "w") as f:
        json.dump({"ms": ms, "e2e_ms": e2e_ms}, f)
    os.replace(os.path.join(d, f"r{rank}.json.tmp"), os.path.join(d, f"r{rank}.json"))
    if rank != 0:
        return None
    times, t_wait = [], time.time()
    for r in range(world):
        fpath = os.path.join(d, f"r{r}.json")
        while not os.path.exists(fpath):
            if time.time() - t_wait > 600:
                raise RuntimeError("a rank of the reference arm did not finish")
            time.sleep(0.05)
        times.append(json.load(open(fpath)))
    for r in range(world):
        os.remove(os.path.join(d, f"r{r}.json"))
    ms = max(t["ms"] for t in times)
    e2e_ms = max(t["e2e_ms"] for t in times)
    value = world * B * steps / (ms * 1e-3)
    return {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.config + (" (size overridden)" if args.rows or args.width else ""),
                       "rows": c["rows"], "width": W, "keys_per_gpu_per_step": B, "partition": f"random owners x{world}",
                       "cache_fraction": c["cache"] if world > 1 else 0.0,
                       "what": "the reference's own CUDA/NCCL build (oracle/_ref), unmodified sources, "
                               "preprocess()+pushPull() per step, inputs resident on the device"},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": world, "kind": "reference",
                             "sample": f"{steps} steps of {args.config} by the reference's own GPU build "
                                       f"(one driving host thread per rank; the reference has no CPU path)"},
            "e2e": {"value": world * B * e2e_steps / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": B * 8 + B * W * 4, "d2h_bytes_per_step": B * W * 4,
                    "ms_per_step": e2e_ms / e2e_steps, "steps": e2e_steps, "host_binding": binding},
            "clocks": clk}


def main():
    args = parse_args()
    out = run_reference(args) if args.impl == "reference" else run_ours(args)
    if out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
