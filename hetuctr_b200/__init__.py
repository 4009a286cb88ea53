"""hetuctr_b200 — B200-native implementation of HetuCTR's distributed embedding table hot path.

Two ways in, both backed by the same shared library (hetuctr_b200/lib/libhetuctr_b200.so):

  * `hetuctr_b200.hetuCTR`   the drop-in pybind module: `hetuCTR.HetuTable(...)`, `.preprocess()`,
                              `.push_pull()`, `hetuCTR.Initializer`, `hetuCTR.InitType`, `hetuCTR.seed`.
                              Putting hetuctr_b200/lib on PYTHONPATH makes plain `import hetuCTR` work.
  * `hetuctr_b200.Table`     a thin ctypes wrapper over the table-level C-ABI (include/hctr_table.h).

There is no CPU fallback: without the compiled library (run `python -m hetuctr_b200.build`) imports of the
native parts raise, and without a CUDA device table construction raises.
"""
import ctypes
import importlib.util
import os
import sysconfig

import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_DIR = os.path.join(_PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libhetuctr_b200.so")
MODULE_PATH = os.path.join(LIB_DIR, "hetuCTR" + sysconfig.get_config_var("EXT_SUFFIX"))

INIT_ZERO, INIT_NORMAL, INIT_UNIFORM, INIT_TRUNCATED_NORMAL = 0, 1, 2, 3
INVALID_VERSION = np.iinfo(np.int64).min

_lib = None
_mod = None


def _preload_nccl():
    """The library needs libnccl.so.2.  PyTorch wheels bundle their own (newer) copy under nvidia/nccl; if this
    library pulled in the system copy first, a later `import torch` in the same process would fail to resolve
    symbols of the newer one.  So when a bundled copy exists it is loaded first and both share it."""
    try:
        spec = importlib.util.find_spec("nvidia.nccl")
    except (ImportError, ValueError):
        spec = None
    if spec and spec.submodule_search_locations:
        for d in spec.submodule_search_locations:
            cand = os.path.join(d, "lib", "libnccl.so.2")
            if os.path.exists(cand):
                ctypes.CDLL(cand, mode=ctypes.RTLD_GLOBAL)
                return cand
    return None


def lib():
    """The C-ABI library as a ctypes.CDLL with argument types set."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m hetuctr_b200.build`")
    _preload_nccl()
    L = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
    c = ctypes
    vp, sz, i64, i32 = c.c_void_p, c.c_size_t, c.c_int64, c.c_int
    L.hctr_last_error.restype = c.c_char_p
    L.hctr_seed.argtypes = [c.c_ulong]
    L.hctr_table_create.restype = vp
    L.hctr_table_create.argtypes = [i32, i32, i32, c.c_char_p, i32, sz, sz, i64, i64, vp, vp, sz, i32, c.c_float,
                                    c.c_float, c.c_float, i32]
    L.hctr_table_destroy.argtypes = [vp]
    L.hctr_table_preprocess.argtypes = [vp, vp, sz]
    L.hctr_table_push_pull.argtypes = [vp, vp, vp]
    L.hctr_table_preprocess_async.restype = vp
    L.hctr_table_preprocess_async.argtypes = [vp, vp, sz]
    L.hctr_table_push_pull_async.restype = vp
    L.hctr_table_push_pull_async.argtypes = [vp, vp, vp]
    L.hctr_wait_finish.argtypes = [vp]
    L.hctr_table_repr.argtypes = [vp, i32, c.c_char_p, sz]
    L.hctr_table_dump.restype = c.c_longlong
    L.hctr_table_dump.argtypes = [vp, c.c_char_p, i32, vp]
    L.hctr_table_set_embedding.argtypes = [vp, vp]
    L.hctr_table_timeline.argtypes = [vp, vp, ctypes.c_int]
    L.hctr_table_export.argtypes = [vp, ctypes.c_char_p]
    L.hctr_table_import.argtypes = [vp, ctypes.c_char_p]
    L.hctr_table_stats.argtypes = [vp, vp]
    L.hctr_table_exchange_name.restype = c.c_char_p
    L.hctr_table_exchange_name.argtypes = [vp]
    L.hctr_table_stream.restype = vp
    L.hctr_table_stream.argtypes = [vp]
    L.hctr_rendezvous_broadcast.argtypes = [i32, i32, c.c_char_p, i32, vp, sz, c.c_double]
    L.hctr_table_profile.argtypes = [vp, i32]
    L.hctr_table_phase_times.argtypes = [vp, vp, vp, i32]
    L.hctr_launch_count.restype = c.c_ulonglong
    L.hctr_scan_exclusive_u32.argtypes = [vp, vp, sz, vp, vp, vp]
    L.hctr_scan_exclusive_u32_noalloc.argtypes = [vp, vp, sz, vp]
    L.hctr_noalloc_last_error.restype = c.c_char_p
    L.hctr_scan_scratch_words.restype = sz
    L.hctr_scan_scratch_words.argtypes = [sz]
    _lib = L
    return L


def _load_module():
    global _mod
    if _mod is None:
        if not os.path.exists(MODULE_PATH):
            raise ImportError(f"{MODULE_PATH} is missing: build it with `python -m hetuctr_b200.build`")
        lib()  # make sure the dependency resolves from this tree
        spec = importlib.util.spec_from_file_location("hetuCTR", MODULE_PATH)
        _mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(_mod)
    return _mod


_part = None


def _load_partition():
    global _part
    if _part is None:
        path = os.path.join(LIB_DIR, "hetuCTR_partition" + sysconfig.get_config_var("EXT_SUFFIX"))
        if not os.path.exists(path):
            raise ImportError(f"{path} is missing: build it with `python -m hetuctr_b200.build`")
        spec = importlib.util.spec_from_file_location("hetuCTR_partition", path)
        _part = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(_part)
    return _part


def __getattr__(name):
    if name == "hetuCTR":
        return _load_module()
    if name == "hetuCTR_partition":
        return _load_partition()
    raise AttributeError(name)


def _ptr(x):
    """Raw address of a numpy array / torch tensor / int / None."""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if isinstance(x, np.ndarray):
        return x.ctypes.data
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    raise TypeError(type(x))


class Table:
    """One rank of the table through the C-ABI.  Arguments as hetuCTR.HetuTable
    (reference csrc/pybind/pybind.cu:62-69); init is (kind, a, b)."""

    _STATS = ("batch", "unique", "prev_batch", "prev_unique", "pushed_rows", "received_push_rows", "queried_keys",
              "returned_rows", "received_rows", "stored_rows", "cached_rows", "wait_queries_us", "wait_returns_us")

    def __init__(self, rank, nrank, device_id, ip, port, length, width, pull_bound, push_bound, root_arr,
                 storage_arr, init=(INIT_ZERO, 0.0, 0.0), learning_rate=0.01, verbose=0):
        self._lib = lib()
        root = np.ascontiguousarray(root_arr, dtype=np.uint8)
        storage = np.ascontiguousarray(storage_arr, dtype=np.int64)
        if root.shape != (length,):
            raise RuntimeError("root_arr must have `length` entries")
        self.width, self.length, self.nrank, self.rank = width, length, nrank, rank
        self.device_id = device_id
        self._h = self._lib.hctr_table_create(rank, nrank, device_id, ip.encode(), port, length, width, pull_bound,
                                              push_bound, root.ctypes.data, storage.ctypes.data, storage.size,
                                              init[0], init[1], init[2], learning_rate, verbose)
        if not self._h:
            raise RuntimeError(self._lib.hctr_last_error().decode())

    def _check(self, rc):
        if rc != 0:
            raise RuntimeError(self._lib.hctr_last_error().decode())

    def close(self):
        if getattr(self, "_h", None):
            self._lib.hctr_table_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def preprocess(self, keys, n_keys=None):
        if n_keys is None:
            n_keys = keys.numel() if hasattr(keys, "numel") else keys.size
        self._check(self._lib.hctr_table_preprocess(self._h, _ptr(keys), n_keys))

    def push_pull(self, grad, dst):
        self._check(self._lib.hctr_table_push_pull(self._h, _ptr(grad), _ptr(dst)))

    def async_preprocess(self, keys, n_keys):
        return _Wait(self, self._lib.hctr_table_preprocess_async(self._h, _ptr(keys), n_keys))

    def async_push_pull(self, grad, dst):
        return _Wait(self, self._lib.hctr_table_push_pull_async(self._h, _ptr(grad), _ptr(dst)))

    def dump(self, what, prev=False):
        n = self._lib.hctr_table_dump(self._h, what.encode(), int(prev), None)
        if n < 0:
            raise RuntimeError(self._lib.hctr_last_error().decode())
        is_f = what in ("embedding", "gradient")
        out = np.zeros(n, dtype=np.float32 if is_f else np.int64)
        if self._lib.hctr_table_dump(self._h, what.encode(), int(prev), out.ctypes.data) < 0:
            raise RuntimeError(self._lib.hctr_last_error().decode())
        return out.reshape(-1, self.width) if is_f else out

    def set_embedding(self, rows):
        rows = np.ascontiguousarray(rows, dtype=np.float32)
        if rows.size != self.stats()["stored_rows"] * self.width:
            raise RuntimeError("set_embedding: expected stored_rows * width values")
        self._check(self._lib.hctr_table_set_embedding(self._h, rows.ctypes.data))

    def export_state(self, path):
        """Writes this rank's rows, versions and pending cached-row updates to `path`."""
        self._check(self._lib.hctr_table_export(self._h, str(path).encode()))

    def import_state(self, path):
        """Loads a file written by export_state() of a table built from the same arguments."""
        self._check(self._lib.hctr_table_import(self._h, str(path).encode()))

    def stats(self):
        out = (ctypes.c_longlong * len(self._STATS))()
        self._lib.hctr_table_stats(self._h, out)
        return dict(zip(self._STATS, list(out)))

    PHASES = ("dedupe", "push_decide", "reduce", "query", "exchange", "owner_update", "stale_gather", "refresh",
              "expand", "owner_apply")

    def profile(self, enable=True):
        """False/0: off; True/1: time every step; k > 1: time every k-th step."""
        self._lib.hctr_table_profile(self._h, int(enable))

    def phase_times(self, reset=True):
        """{phase: (total_ms, calls)} of the device time recorded while profiling was enabled."""
        ms = (ctypes.c_double * len(self.PHASES))()
        calls = (ctypes.c_longlong * len(self.PHASES))()
        self._lib.hctr_table_phase_times(self._h, ms, calls, int(reset))
        return {p: (ms[i], calls[i]) for i, p in enumerate(self.PHASES)}

    def timeline(self, max_spans=256):
        """[(phase, start_ms, end_ms)] of the most recent timed phases, oldest first."""
        out = (ctypes.c_double * (3 * max_spans))()
        n = self._lib.hctr_table_timeline(self._h, out, max_spans)
        return [(self.PHASES[int(out[3 * i])], out[3 * i + 1], out[3 * i + 2]) for i in range(n)]

    def exchange_name(self):
        return self._lib.hctr_table_exchange_name(self._h).decode()

    def stream(self):
        return self._lib.hctr_table_stream(self._h)

    def __repr__(self):
        buf = ctypes.create_string_buffer(1024)
        self._lib.hctr_table_repr(self._h, 0, buf, 1024)
        return buf.value.decode()

    def debug(self):
        buf = ctypes.create_string_buffer(1024)
        self._lib.hctr_table_repr(self._h, 1, buf, 1024)
        return buf.value.decode()


class _Wait:
    def __init__(self, table, handle):
        if not handle:
            raise RuntimeError(table._lib.hctr_last_error().decode())
        self._t, self._w = table, handle

    def wait(self):
        if self._w:
            w, self._w = self._w, None
            self._t._check(self._t._lib.hctr_wait_finish(w))
