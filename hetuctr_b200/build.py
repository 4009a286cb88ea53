"""In-tree build of the native parts (sm_100a only).

  python -m hetuctr_b200.build [--force] [-v]

Produces, under hetuctr_b200/lib/:
  libhetuctr_b200.so                      kernels + C-ABI launchers (hctr_kernels.h) + HetuTable +
                                          table-level C-ABI (hctr_table.h)
  hetuCTR.cpython-*.so                    the drop-in Python module `hetuCTR`
"""
import concurrent.futures
import os
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "lib")
OBJ = os.path.join(LIB, "obj")
INCLUDE = os.path.join(ROOT, "include")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")

CU_SOURCES = ["kernels/scan.cu", "kernels/dedupe.cu", "kernels/update.cu", "kernels/query.cu", "kernels/table.cu",
              "kernels/p2p.cu", "kernels/p2p_pull.cu"]
CC_SOURCES = ["core/hetu_table.cc", "core/table_state.cc", "core/c_api.cc", "core/transport.cc", "core/p2p.cc", "utils/rendezvous.cc"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-I", INCLUDE, "-I", CSRC]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-I", INCLUDE, "-I", CSRC,
             "-I", os.path.join(CUDA_HOME, "include")]

LIB_NAME = "libhetuctr_b200.so"
MOD_NAME = "hetuCTR" + sysconfig.get_config_var("EXT_SUFFIX")
PART_NAME = "hetuCTR_partition" + sysconfig.get_config_var("EXT_SUFFIX")


def _headers():
    out = []
    for base in (CSRC, INCLUDE):
        for d, _, files in os.walk(base):
            out += [os.path.join(d, f) for f in files if f.endswith((".h", ".cuh"))]
    return out


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n" + " ".join(cmd) + "\n" + r.stdout)
    if verbose and r.stdout.strip():
        print(r.stdout)


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    hdrs = _headers()
    jobs, objs = [], []
    for src in CU_SOURCES + CC_SOURCES:
        path = os.path.join(CSRC, src)
        obj = os.path.join(OBJ, src.replace("/", "_") + ".o")
        objs.append(obj)
        if force or _stale(obj, [path] + hdrs):
            if src.endswith(".cu"):
                jobs.append([NVCC, *NVCC_FLAGS, "-c", path, "-o", obj])
            else:
                jobs.append(["g++", *CXX_FLAGS, "-c", path, "-o", obj])
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(lambda c: _run(c, verbose), jobs))
    lib = os.path.join(LIB, LIB_NAME)
    if force or jobs or _stale(lib, objs):
        _run([NVCC, "-shared", "-o", lib, *objs, "-lnccl", "-Xlinker", "-rpath,$ORIGIN"], verbose)
    mod = os.path.join(LIB, MOD_NAME)
    mod_src = os.path.join(CSRC, "pybind/module.cc")
    if force or _stale(mod, [mod_src, lib] + hdrs):
        import pybind11
        _run(["g++", *CXX_FLAGS, "-fvisibility=hidden", "-shared", "-I", pybind11.get_include(),
              "-I", sysconfig.get_paths()["include"], mod_src, "-o", mod,
              "-L", LIB, "-lhetuctr_b200", "-Wl,-rpath,$ORIGIN"], verbose)
    # the offline partitioner (CPU only): its own small module, `hetuCTR_partition`
    pmod = os.path.join(LIB, PART_NAME)
    psrc = [os.path.join(CSRC, "partition/partition.cc"), os.path.join(CSRC, "partition/module.cc")]
    if force or _stale(pmod, psrc + hdrs):
        import pybind11
        _run(["g++", *CXX_FLAGS, "-fopenmp", "-fvisibility=hidden", "-shared", "-I", pybind11.get_include(),
              "-I", sysconfig.get_paths()["include"], *psrc, "-o", pmod], verbose)
    return lib, mod


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
