"""Builds the REFERENCE's own implementation as a checker (TEST INFRASTRUCTURE, never shipped).

  python oracle/build_ref.py [--reference DIR]      (DIR = checkout of the reference project; default: the
                                                     HCTR_REFERENCE_DIR environment variable, else a directory
                                                     named "reference" beside this repository)

Compiles the reference's sources where they lie (nothing is copied into this repository) for sm_100a and links
them with oracle/ref_binding.cu into oracle/_ref/hetuCTR_ref<ext>.so.  The reference's ZMQ rendezvous cannot be
built here (no zmq.h); oracle/ref_shim/utils/rendezvous.h, found first on the include path, substitutes this
repository's POSIX-socket TCPRendezvous, which has the same constructor and broadcast().  The reference also
launches empty grids, which the CUDA runtime of this image rejects: ref_empty_launch_shim.cc skips those at link
level.  -DNDEBUG turns the
reference's device-side asserts off so that a bad key cannot trap a shared GPU.
"""
import concurrent.futures
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT = os.path.join(HERE, "_ref")
MODULE = os.path.join(OUT, "hetuCTR_ref" + sysconfig.get_config_var("EXT_SUFFIX"))

REF_SOURCES = ["core/hetu_gpu_table.cu", "core/preprocess.cu", "core/preprocess_sturct.cu", "core/generate_query.cu",
               "core/handle_query.cu", "core/writeback.cu", "core/all2all.cu", "core/table_initialize.cu",
               "core/debug.cu", "utils/initializer.cu"]


def reference_dir():
    """Where the reference project's checkout is: HCTR_REFERENCE_DIR, else `reference` beside this repository."""
    return os.environ.get("HCTR_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")


def build(reference=None, force=False, verbose=False):
    reference = reference or reference_dir()
    csrc = os.path.join(reference, "csrc")
    if not os.path.isdir(csrc):
        raise RuntimeError(f"reference sources not found at {csrc}")
    if os.path.exists(MODULE) and not force:
        return MODULE
    import pybind11
    os.makedirs(os.path.join(OUT, "obj"), exist_ok=True)
    inc = ["-I", os.path.join(HERE, "ref_shim"), "-I", csrc, "-I", pybind11.get_include(),
           "-I", sysconfig.get_paths()["include"]]
    flags = ["-std=c++17", "-O3", "-w", "-DNDEBUG", "-gencode", "arch=compute_100a,code=sm_100a",
             "-Xcompiler", "-fPIC", *inc]
    jobs, objs = [], []
    for src in REF_SOURCES:
        obj = os.path.join(OUT, "obj", src.replace("/", "_") + ".o")
        objs.append(obj)
        jobs.append(["nvcc", *flags, "-c", os.path.join(csrc, src), "-o", obj])
    obj = os.path.join(OUT, "obj", "ref_binding.o")
    objs.append(obj)
    jobs.append(["nvcc", *flags, "-c", os.path.join(HERE, "ref_binding.cu"), "-o", obj])
    obj = os.path.join(OUT, "obj", "rendezvous.o")
    objs.append(obj)
    jobs.append(["g++", "-O2", "-std=c++17", "-fPIC", "-I", os.path.join(ROOT, "hetuctr_b200", "csrc"), "-c",
                 os.path.join(ROOT, "hetuctr_b200", "csrc", "utils", "rendezvous.cc"), "-o", obj])

    def run(cmd):
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError("reference build step failed:\n" + " ".join(cmd) + "\n" + r.stdout[-4000:])

    obj = os.path.join(OUT, "obj", "empty_launch_shim.o")
    objs.append(obj)
    jobs.append(["g++", "-O2", "-std=c++17", "-fPIC", "-I", "/usr/local/cuda/include", "-c",
                 os.path.join(HERE, "ref_empty_launch_shim.cc"), "-o", obj])

    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(run, jobs))
    # shared CUDA runtime + -Bsymbolic: the module's own launch hook (ref_empty_launch_shim.cc) is the one its
    # kernels' launch stubs call, and it forwards to the runtime library
    run(["nvcc", "-shared", "-cudart", "shared", "-o", MODULE, *objs, "-lnccl", "-ldl", "-Xlinker", "-Bsymbolic",
         "-Xlinker", "-rpath,/usr/local/cuda/lib64"])
    return MODULE


PARTITION_MODULE = os.path.join(OUT, "partition", "hetuCTR_partition" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_partition(reference=None, force=False, verbose=False):
    reference = reference or reference_dir()
    """The reference's offline partitioner (csrc/partition/), compiled WITHOUT OpenMP: its `omp parallel for`
    pragmas are then ignored, the sweeps run sequentially and the result is reproducible (its rand() starts from
    the C library's default seed in a fresh process)."""
    csrc = os.path.join(reference, "csrc")
    if not os.path.isdir(csrc):
        raise RuntimeError(f"reference sources not found at {csrc}")
    if os.path.exists(PARTITION_MODULE) and not force:
        return PARTITION_MODULE
    import pybind11
    os.makedirs(os.path.dirname(PARTITION_MODULE), exist_ok=True)
    cmd = ["g++", "-O2", "-std=c++17", "-w", "-fPIC", "-shared", "-fvisibility=hidden", "-I", csrc,
           "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
           os.path.join(csrc, "partition", "partition.cc"), os.path.join(csrc, "partition", "pybind.cc"),
           "-o", PARTITION_MODULE]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("reference partitioner build failed:\n" + r.stdout[-4000:])
    return PARTITION_MODULE


if __name__ == "__main__":
    ref = sys.argv[sys.argv.index("--reference") + 1] if "--reference" in sys.argv else reference_dir()
    print(build(ref, force="--force" in sys.argv, verbose=True))
    print(build_partition(ref, force="--force" in sys.argv, verbose=True))
