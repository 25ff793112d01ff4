"""The part of cupti-python's `cupti.cupti` module that kernel timing needs.

    activity_register_callbacks(buffer_requested, buffer_completed)
    activity_enable(kind) / activity_disable(kind)
    activity_flush_all(flag)
    ActivityKind.CONCURRENT_KERNEL / ActivityKind.KERNEL

`buffer_requested()` returns (buffer_bytes, max_records); `buffer_completed(activities)` receives a
list of records with the attributes of a kernel activity: kind, name (bytes), start, end
(nanoseconds), grid_x/y/z, block_x/y/z, cluster_x/y/z, dynamic_shared_memory,
static_shared_memory, registers_per_thread, local_memory_per_thread.  CUPTI completes buffers on
its own threads; the records are kept on the native side and delivered to `buffer_completed` from
the calling thread inside `activity_flush_all`.
"""

from __future__ import annotations

import ctypes
import enum
import pathlib
from types import SimpleNamespace

_LIB_PATH = pathlib.Path(__file__).resolve().parents[1] / "libmsc_cupti.so"
_lib = None
_callbacks = {"requested": None, "completed": None}


def _load():
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise ImportError(f"{_LIB_PATH} is missing: run `python -m mosaicist_b200.build`")
        lib = ctypes.CDLL(str(_LIB_PATH))
        lib.msc_cupti_last_error.restype = ctypes.c_char_p
        lib.msc_cupti_register.argtypes = [ctypes.c_size_t]
        lib.msc_cupti_enable.argtypes = lib.msc_cupti_disable.argtypes = lib.msc_cupti_flush.argtypes = [ctypes.c_uint32]
        lib.msc_cupti_count.restype = ctypes.c_size_t
        lib.msc_cupti_get.argtypes = [ctypes.c_size_t, ctypes.c_char_p, ctypes.c_size_t,
                                      ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_int32)]
        lib.msc_cupti_kind_concurrent_kernel.restype = ctypes.c_uint32
        lib.msc_cupti_kind_kernel.restype = ctypes.c_uint32
        _lib = lib
    return _lib


def _check(rc: int):
    if rc != 0:
        raise RuntimeError(_load().msc_cupti_last_error().decode() or "CUPTI call failed")


class _Kinds:
    """ActivityKind with the values of the CUPTI headers this library was built against."""

    def __getattr__(self, name):
        lib = _load()
        if name == "CONCURRENT_KERNEL":
            return lib.msc_cupti_kind_concurrent_kernel()
        if name == "KERNEL":
            return lib.msc_cupti_kind_kernel()
        raise AttributeError(name)


ActivityKind = _Kinds()


def activity_register_callbacks(buffer_requested, buffer_completed):
    _callbacks["requested"], _callbacks["completed"] = buffer_requested, buffer_completed
    size = 8 << 20
    try:
        size = int(buffer_requested()[0])
    except Exception:  # noqa: BLE001 - a callback that returns nothing usable keeps the default
        pass
    lib = _load()
    lib.msc_cupti_clear()
    _check(lib.msc_cupti_register(size))


def activity_enable(kind):
    _check(_load().msc_cupti_enable(int(kind)))


def activity_disable(kind):
    _check(_load().msc_cupti_disable(int(kind)))


def activity_flush_all(flag: int = 0):
    lib = _load()
    _check(lib.msc_cupti_flush(int(flag)))
    n = lib.msc_cupti_count()
    name = ctypes.create_string_buffer(1024)
    times = (ctypes.c_uint64 * 2)()
    ints = (ctypes.c_int32 * 13)()
    records = []
    for i in range(n):
        kind = lib.msc_cupti_get(i, name, len(name), times, ints)
        if kind < 0:
            break
        v = list(ints)
        records.append(SimpleNamespace(
            kind=kind, name=name.value, start=int(times[0]), end=int(times[1]),
            grid_x=v[0], grid_y=v[1], grid_z=v[2], block_x=v[3], block_y=v[4], block_z=v[5],
            cluster_x=v[6], cluster_y=v[7], cluster_z=v[8], dynamic_shared_memory=v[9],
            static_shared_memory=v[10], registers_per_thread=v[11], local_memory_per_thread=v[12]))
    lib.msc_cupti_clear()
    done = _callbacks["completed"]
    if records and done is not None:
        done(records)
