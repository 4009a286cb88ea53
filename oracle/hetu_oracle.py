"""ctypes front end of the CPU oracle (TEST INFRASTRUCTURE, not part of the product).

`World` holds all ranks of one job in a single process and steps them in lockstep, mirroring the
call pattern of the reference's tests (tests/driver.py:31-38): preprocess(keys) then
push_pull(grad, dst) on every rank.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIBS = {}

INVALID_VERSION = np.iinfo(np.int64).min


def _load(parallel):
    name = "libhetu_oracle_mt.so" if parallel else "libhetu_oracle.so"
    if name in _LIBS:
        return _LIBS[name]
    path = os.path.join(_HERE, "_build", name)
    if not os.path.exists(path):
        from . import build as _b  # noqa: WPS433  (build on demand; g++ only)
        _b.build()
    lib = ctypes.CDLL(path)
    lib.ho_last_error.restype = ctypes.c_char_p
    lib.ho_world_create.restype = ctypes.c_void_p
    lib.ho_world_create.argtypes = [ctypes.c_int, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong,
                                    ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p]
    lib.ho_world_destroy.argtypes = [ctypes.c_void_p]
    lib.ho_set_storage.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_longlong]
    lib.ho_set_embedding.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    lib.ho_preprocess.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.ho_push_pull.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.ho_get_i64.restype = ctypes.c_longlong
    lib.ho_get_i64.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.c_void_p]
    lib.ho_get_f32.restype = ctypes.c_longlong
    lib.ho_get_f32.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_void_p]
    _LIBS[name] = lib
    return lib


class World:
    def __init__(self, nrank, length, width, pull_bound, push_bound, learning_rate, root_arr, storage_arrs,
                 parallel=False):
        self.lib = _load(parallel)
        self.nrank, self.length, self.width = nrank, length, width
        root = np.ascontiguousarray(root_arr, dtype=np.uint8)
        assert root.shape == (length,)
        self.h = self.lib.ho_world_create(nrank, length, width, pull_bound, push_bound, learning_rate,
                                          root.ctypes.data)
        assert len(storage_arrs) == nrank
        for r, st in enumerate(storage_arrs):
            st = np.ascontiguousarray(st, dtype=np.int64)
            self._check(self.lib.ho_set_storage(self.h, r, st.ctypes.data, st.size))
        self._batch = [0] * nrank

    def num_threads(self):
        return self.lib.ho_num_threads()

    def _check(self, rc):
        if rc != 0:
            raise RuntimeError(self.lib.ho_last_error().decode())

    def close(self):
        if self.h:
            self.lib.ho_world_destroy(self.h)
            self.h = None

    def __del__(self):
        self.close()

    def set_embedding(self, rank, emb):
        emb = np.ascontiguousarray(emb, dtype=np.float32)
        assert emb.size == self.get(rank, "storage") * self.width
        self._check(self.lib.ho_set_embedding(self.h, rank, emb.ctypes.data))

    def preprocess(self, keys_per_rank):
        keys = [np.ascontiguousarray(k, dtype=np.int64) for k in keys_per_rank]
        ptrs = (ctypes.c_void_p * self.nrank)(*[k.ctypes.data for k in keys])
        sizes = (ctypes.c_size_t * self.nrank)(*[k.size for k in keys])
        self._check(self.lib.ho_preprocess(self.h, ptrs, sizes))
        self._batch = [k.size for k in keys]

    def push_pull(self, grads_per_rank):
        """grads_per_rank: list of [n_prev, width] float32 arrays, or None for an inference step.
        Returns the list of [n_cur, width] pulled rows, one per rank."""
        dsts = [np.zeros((b, self.width), dtype=np.float32) for b in self._batch]
        dptr = (ctypes.c_void_p * self.nrank)(*[d.ctypes.data for d in dsts])
        if grads_per_rank is None:
            gptr = None
        else:
            grads = [np.ascontiguousarray(g, dtype=np.float32) for g in grads_per_rank]
            gptr = (ctypes.c_void_p * self.nrank)(*[g.ctypes.data for g in grads])
        self._check(self.lib.ho_push_pull(self.h, gptr, dptr))
        return dsts

    def get(self, rank, what, prev=False):
        n = self.lib.ho_get_i64(self.h, rank, what.encode(), int(prev), None)
        if n < 0:
            raise KeyError(what)
        out = np.zeros(n, dtype=np.int64)
        self.lib.ho_get_i64(self.h, rank, what.encode(), int(prev), out.ctypes.data)
        if what in ("storage", "nonlocal", "unique_size"):
            return int(out[0])
        return out

    def get_f32(self, rank, what):
        n = self.lib.ho_get_f32(self.h, rank, what.encode(), None)
        if n < 0:
            raise KeyError(what)
        out = np.zeros(n, dtype=np.float32)
        self.lib.ho_get_f32(self.h, rank, what.encode(), out.ctypes.data)
        if what in ("embedding", "gradient"):
            return out.reshape(-1, self.width)
        return out
