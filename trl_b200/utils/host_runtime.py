"""ctypes facade of ``libtrl_b200_host.so`` (C++ scheduler, block pool, BFD packer)."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_int, c_int32, c_int64, c_void_p

import numpy as np


class HostRuntime:
    def __init__(self, lib: ctypes.CDLL):
        self.lib = lib
        lib.trlb_sched_create.restype = c_void_p
        lib.trlb_sched_create.argtypes = [c_int, c_int, c_int, c_int]
        lib.trlb_sched_destroy.argtypes = [c_void_p]
        lib.trlb_sched_add.argtypes = [c_void_p, c_int64, c_int, c_int, c_int64]
        for fn in ("trlb_sched_num_waiting", "trlb_sched_num_running", "trlb_sched_num_free_blocks"):
            getattr(lib, fn).argtypes = [c_void_p]
            getattr(lib, fn).restype = c_int
        lib.trlb_sched_admit.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
        lib.trlb_sched_admit.restype = c_int
        lib.trlb_sched_retire.argtypes = [c_void_p, c_int, c_int64]
        lib.trlb_sched_retire.restype = c_int64
        lib.trlb_bfd_assign.argtypes = [c_void_p, c_int, c_int, c_void_p]
        lib.trlb_bfd_assign.restype = c_int

    def bfd_assign(self, lengths, seq_length: int) -> list[list[int]]:
        n = len(lengths)
        if n == 0:
            return []
        arr = np.ascontiguousarray(lengths, dtype=np.int32)
        out = np.empty(n, dtype=np.int32)
        nb = self.lib.trlb_bfd_assign(arr.ctypes.data, n, int(seq_length), out.ctypes.data)
        bins: list[list[int]] = [[] for _ in range(nb)]
        order = sorted(range(n), key=lambda i: -int(arr[i]))  # stable: matches the visiting order in C++
        for i in order:
            bins[int(out[i])].append(i)
        return bins

    def scheduler(self, max_slots: int, num_blocks: int, block_size: int, max_blocks_per_seq: int) -> "Scheduler":
        return Scheduler(self, max_slots, num_blocks, block_size, max_blocks_per_seq)


class Scheduler:
    """Continuous-batching scheduler handle.  ``block_table`` is a pinned int32 host tensor owned by the caller."""

    def __init__(self, rt: HostRuntime, max_slots, num_blocks, block_size, max_blocks_per_seq):
        self.rt, self.lib = rt, rt.lib
        self.h = self.lib.trlb_sched_create(max_slots, num_blocks, block_size, max_blocks_per_seq)
        self.max_slots, self.block_size, self.max_blocks_per_seq = max_slots, block_size, max_blocks_per_seq
        self._ids = np.empty(max_slots, dtype=np.int64)
        self._slots = np.empty(max_slots, dtype=np.int32)
        self._prefill = np.empty(max_slots, dtype=np.int32)
        self._copy = np.empty(max_slots, dtype=np.int32)

    def __del__(self):
        try:
            self.lib.trlb_sched_destroy(self.h)
        except Exception:
            pass

    def add(self, req_id: int, prompt_len: int, max_new: int, group: int):
        self.lib.trlb_sched_add(self.h, req_id, prompt_len, max_new, group)

    def admit(self, block_table_np: np.ndarray, max_admit: int | None = None):
        n = self.lib.trlb_sched_admit(self.h, max_admit or self.max_slots, self._ids.ctypes.data, self._slots.ctypes.data,
                                      self._prefill.ctypes.data, self._copy.ctypes.data, block_table_np.ctypes.data)
        return [(int(self._ids[i]), int(self._slots[i]), bool(self._prefill[i]), int(self._copy[i])) for i in range(n)]

    def retire(self, slot: int, group: int) -> int:
        return int(self.lib.trlb_sched_retire(self.h, slot, group))

    num_waiting = property(lambda s: s.lib.trlb_sched_num_waiting(s.h))
    num_running = property(lambda s: s.lib.trlb_sched_num_running(s.h))
    num_free_blocks = property(lambda s: s.lib.trlb_sched_num_free_blocks(s.h))
