"""The cache manager: pages, block tables and state slots.

Host bookkeeping is the C++ library ``host/cache_manager.cpp`` (pure integer
logic, usable without a GPU); this module wraps it and, on a device, owns the
page memory itself.

* A **cache group** is a set of layer caches with the same needs: all keys
  (``window=None``) or the last ``window`` keys.  Every group has its own page
  pool and its own block table per request.
* A **page** holds ``block_size`` tokens for every layer cache of its group.
* A **state slot** is an index per live request into arrays of per-request
  state of fixed size (mixers with a recurrent state, sampling state); it is
  handed out at admission and given back with the request.

Pages are given back when a request is released or when a group's window has
passed them (:meth:`advance`), and are used again (last freed, first reused).
The reference's counterparts are ``BlockPool`` (src/alofa/runtime/kv/pool.mojo:28-114),
``KvSpace`` (runtime/kv/space.mojo:52-532) and ``KvRoom``
(engine/kv_room.mojo:48-329)."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import numpy as np

from ..csrc.build import load_library
from ..errors import AlofaError

_lib = None


def _native():
    global _lib
    if _lib is None:
        lib = load_library("alofa_cache_manager", ["host/cache_manager.cpp"], cuda=False)
        I, P, L = ctypes.c_int, ctypes.c_void_p, ctypes.c_int64
        IP = ctypes.POINTER(ctypes.c_int)
        sigs = {
            "cm_create": (P, [I, IP, IP, IP, I, I]),
            "cm_destroy": (None, [P]),
            "cm_admit": (I, [P, L]),
            "cm_find": (I, [P, L]),
            "cm_pages_needed": (I, [P, I, I, IP]),
            "cm_reserve": (I, [P, I, I]),
            "cm_advance": (I, [P, I, I]),
            "cm_release": (I, [P, I]),
            "cm_share_prefix": (I, [P, I, I, I]),
            "cm_block_table": (I, [P, I, I, ctypes.c_void_p, I]),
            "cm_plan_step": (I, [P, I, P, P, P, P, P, P, I, P]),
            "cm_commit_step": (I, [P, I, P, P]),
            "cm_free_pages": (I, [P, I]),
            "cm_num_pages": (I, [P, I]),
            "cm_reserved_len": (I, [P, I]),
            "cm_computed_len": (I, [P, I]),
            "cm_live_requests": (I, [P]),
            "cm_counter": (L, [P, I, I]),
            "cm_defects": (I, [P]),
            "cm_digest": (L, [P]),
        }
        for name, (res, args) in sigs.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


@dataclass(frozen=True)
class GroupSpec:
    """What one cache group needs: ``window`` None keeps every key."""

    block_size: int
    num_pages: int
    window: Optional[int] = None


_ERRORS = {-1: ("capacity", "the cache has no page or slot left"), -2: ("invalid_argument", "bad slot, group or length"), -3: ("state", "request is unknown, already live or already freed")}


def _check(rc: int, what: str, detail: str = "") -> int:
    if rc < 0:
        code, text = _ERRORS.get(rc, ("state", "cache manager error"))
        raise AlofaError(code, f"{what}: {text}", detail)
    return rc


class CacheManager:
    """Host-side owner of pages, block tables and state slots."""

    def __init__(self, groups: list, max_requests: int, max_tokens: int):
        # no group at all is a model whose layers keep fixed-size state only: slots, no pages
        self.groups = list(groups)
        self.max_requests = max_requests
        self.max_blocks = max([(max_tokens + g.block_size - 1) // g.block_size for g in groups] + [1])
        n = len(groups)
        arr = lambda vals: (ctypes.c_int * n)(*vals)
        self._h = _native().cm_create(
            n,
            arr([g.block_size for g in groups]),
            arr([g.num_pages for g in groups]),
            arr([g.window or 0 for g in groups]),
            max_requests,
            self.max_blocks,
        )
        if not self._h:
            raise AlofaError("invalid_argument", "cache manager refused its configuration", f"groups={groups} max_requests={max_requests}")
        self._need = (ctypes.c_int * n)()

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and _lib is not None:
            _lib.cm_destroy(h)

    # -- requests ---------------------------------------------------------
    def admit(self, request_id: int) -> int:
        """A state slot for a new request; raises "capacity" when none is free."""
        return _check(_lib.cm_admit(self._h, request_id), "admit", f"request={request_id}")

    def try_admit(self, request_id: int) -> int:
        rc = _lib.cm_admit(self._h, request_id)
        if rc == -1:
            return -1
        return _check(rc, "admit", f"request={request_id}")

    def find(self, request_id: int) -> int:
        rc = _lib.cm_find(self._h, request_id)
        return rc if rc >= 0 else -1

    def pages_needed(self, slot: int, new_len: int) -> list:
        _check(_lib.cm_pages_needed(self._h, slot, new_len, self._need), "pages_needed", f"slot={slot}")
        return list(self._need)

    def try_reserve(self, slot: int, new_len: int) -> bool:
        """Reserve pages for ``new_len`` tokens in every group, or none."""
        rc = _lib.cm_reserve(self._h, slot, new_len)
        if rc == -1:
            return False
        _check(rc, "reserve", f"slot={slot} new_len={new_len}")
        return True

    def reserve(self, slot: int, new_len: int) -> None:
        if not self.try_reserve(slot, new_len):
            raise AlofaError("capacity", "the cache has too few free pages", f"slot={slot} new_len={new_len} free={self.free_pages()}")

    def advance(self, slot: int, new_len: int) -> int:
        """Entries up to ``new_len`` are written; frees pages behind windows."""
        return _check(_lib.cm_advance(self._h, slot, new_len), "advance", f"slot={slot} new_len={new_len}")

    def release(self, slot: int) -> int:
        return _check(_lib.cm_release(self._h, slot), "release", f"slot={slot}")

    def share_prefix(self, src: int, dst: int, n_tokens: int) -> None:
        _check(_lib.cm_share_prefix(self._h, src, dst, n_tokens), "share_prefix", f"src={src} dst={dst} n_tokens={n_tokens}")

    def block_table_into(self, slot: int, group: int, out: np.ndarray) -> int:
        """Write the table into ``out`` (int32, contiguous); returns its length."""
        return _check(_lib.cm_block_table(self._h, slot, group, out.ctypes.data, out.shape[0]), "block_table", f"slot={slot} group={group}")

    def block_table(self, slot: int, group: int) -> np.ndarray:
        out = np.empty(self.max_blocks, dtype=np.int32)
        n = self.block_table_into(slot, group, out)
        return out[:n].copy()

    def plan_step(self, slots, counts, want_counts, wants, meta_ptr: int, offsets, max_blocks: int):
        """Reserve pages for every entry and fill the step's metadata in one
        native call; returns (longest entry, most keys, total tokens).  The
        arrays are int32 numpy arrays; ``meta_ptr`` addresses the int32 buffer."""
        info = (ctypes.c_int * 3)()
        rc = _lib.cm_plan_step(self._h, len(slots), slots.ctypes.data, counts.ctypes.data, want_counts.ctypes.data, wants.ctypes.data,
                               meta_ptr, offsets.ctypes.data, max_blocks, info)
        if rc == -1:
            raise AlofaError("capacity", "the cache has too few free pages for this step", f"free={self.free_pages()}")
        _check(rc, "plan_step")
        return info[0], info[1], info[2]

    def commit_step(self, slots, counts) -> None:
        _check(_lib.cm_commit_step(self._h, len(slots), slots.ctypes.data, counts.ctypes.data), "commit_step")

    # -- books ------------------------------------------------------------
    def free_pages(self, group: Optional[int] = None):
        if group is None:
            return [_lib.cm_free_pages(self._h, g) for g in range(len(self.groups))]
        return _check(_lib.cm_free_pages(self._h, group), "free_pages")

    def used_pages(self, group: int = 0) -> int:
        return self.groups[group].num_pages - self.free_pages(group)

    def reserved_len(self, slot: int) -> int:
        return _check(_lib.cm_reserved_len(self._h, slot), "reserved_len", f"slot={slot}")

    def computed_len(self, slot: int) -> int:
        return _check(_lib.cm_computed_len(self._h, slot), "computed_len", f"slot={slot}")

    def live_requests(self) -> int:
        return _lib.cm_live_requests(self._h)

    def counters(self, group: int = 0) -> dict:
        return {"allocs": _lib.cm_counter(self._h, group, 0), "frees": _lib.cm_counter(self._h, group, 1)}

    def defects(self) -> int:
        """Disagreements between the books and a recount from the tables."""
        return _lib.cm_defects(self._h)

    def digest(self) -> int:
        return _lib.cm_digest(self._h)
