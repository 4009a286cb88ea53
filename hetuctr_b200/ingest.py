"""Key-batch ingestion in front of the table: host key batches reach the device one step ahead.

The reference hands `preprocess` a host pointer and pays the host-to-device copy (and the wait for it) inside the
step (csrc/core/preprocess.cu:98-99); its `async_preprocess` only moves that work to another host thread.  Here a
small ring of pinned host buffers and device buffers with its own copy stream keeps `depth` batches in flight, so
that `preprocess` always starts from keys that are already in device memory.

    pipe = KeyPipeline(table, batches, max_keys)        # batches: iterable of int64 numpy arrays
    for keys, n in pipe:                                 # device tensor + key count of the next batch
        table.preprocess(keys, n)
        table.push_pull(grad, dst)
"""
import numpy as np
import torch


class KeyPipeline:
    def __init__(self, table, batches, max_keys, depth=2, device=None):
        if depth < 2:
            raise ValueError("depth must be at least 2 (one batch in use, one in flight)")
        self.table = table
        self.device = torch.device("cuda", table.device_id if device is None else device)
        self._it = iter(batches)
        self._depth = depth
        self._host = [torch.empty(max_keys, dtype=torch.int64).pin_memory() for _ in range(depth)]
        self._dev = [torch.empty(max_keys, dtype=torch.int64, device=self.device) for _ in range(depth)]
        self._event = [torch.cuda.Event() for _ in range(depth)]
        self._count = [None] * depth  # key count of the batch sitting in each slot, None = slot empty
        self._stream = torch.cuda.Stream(device=self.device)
        self._next = 0      # slot handed out by the next __next__
        self._refill = None  # slot whose device buffer the table may still be reading until preprocess returns
        self._done = False
        for s in range(depth):
            self._fill(s)

    def _fill(self, slot):
        """Stage the next host batch into `slot` and start its copy."""
        self._count[slot] = None
        if self._done:
            return
        try:
            keys = next(self._it)
        except StopIteration:
            self._done = True
            return
        keys = np.ascontiguousarray(keys, dtype=np.int64).reshape(-1)
        n = keys.size
        if n > self._host[slot].numel():
            raise ValueError(f"batch of {n} keys exceeds max_keys={self._host[slot].numel()}")
        self._host[slot][:n].numpy()[:] = keys
        with torch.cuda.stream(self._stream):
            self._dev[slot][:n].copy_(self._host[slot][:n], non_blocking=True)
            self._event[slot].record(self._stream)
        self._count[slot] = n

    def __iter__(self):
        return self

    def __next__(self):
        # the slot handed out last time has been consumed: `preprocess` returns only after it has copied the keys
        if self._refill is not None:
            self._fill(self._refill)
            self._refill = None
        slot = self._next
        n = self._count[slot]
        if n is None:
            raise StopIteration
        self._event[slot].synchronize()  # normally long complete: the copy ran under the previous step
        self._refill = slot
        self._next = (slot + 1) % self._depth
        return self._dev[slot], n

    def step(self, grad, dst):
        """preprocess(next batch) + push_pull(grad of the previous batch, dst); False when the batches ran out."""
        try:
            keys, n = next(self)
        except StopIteration:
            return False
        self.table.preprocess(keys, n)
        self.table.push_pull(grad, dst)
        return True
