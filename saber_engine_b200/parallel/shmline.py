"""Python front of ShmLine (`csrc/exec/shmline.cpp`): small control / pick frames between two
processes of one host through POSIX shared memory, with torn-read detection."""
from __future__ import annotations

import ctypes as C

from ..ops import native as N


class TornRead(Exception):
    pass


class ShmLine:
    def __init__(self, name: str, create: bool, one_slot_control: bool = False):
        L = N.lib()
        L.saber_shmline_open.restype = C.c_void_p
        L.saber_shmline_open.argtypes = [C.c_char_p, C.c_int, C.c_int]
        L.saber_shmline_post.restype = C.c_int64
        L.saber_shmline_post.argtypes = [C.c_void_p, C.c_char_p, C.c_uint32, C.c_int]
        L.saber_shmline_take.restype = C.c_int32
        L.saber_shmline_take.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint32, C.c_uint64]
        L.saber_shmline_close.argtypes = [C.c_void_p]
        L.saber_shmline_posted.restype = C.c_uint64
        L.saber_shmline_posted.argtypes = [C.c_void_p]
        self._L = L
        self._h = L.saber_shmline_open(name.encode(), int(create), int(one_slot_control))
        if not self._h:
            raise OSError(f"cannot open shared-memory line {name}")

    def post(self, data: bytes, checked: bool = True) -> int:
        n = self._L.saber_shmline_post(self._h, data, len(data), int(checked))
        if n == -2:
            raise BlockingIOError("the reader has not taken the frame that occupies this slot")
        if n < 0:
            raise ValueError("frame too large")
        return n

    def take(self, n: int, timeout_s: float = 1.0) -> bytes:
        buf = C.create_string_buffer(4096)
        r = self._L.saber_shmline_take(self._h, n, buf, 4096, int(timeout_s * 1e9))
        if r == -3:
            raise TornRead(f"frame {n} was overwritten while it was read")
        if r < 0:
            raise TimeoutError(f"frame {n} did not arrive within {timeout_s} s")
        return buf.raw[:r]

    def close(self) -> None:
        if self._h:
            self._L.saber_shmline_close(self._h)
            self._h = None
