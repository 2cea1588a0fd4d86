"""Python front of the native streaming loader: verified O_DIRECT reads of pack records into host or
device memory (`csrc/pack/pack_stream.cpp`)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from ..ops import native as N
from . import format as PF


class PackStream:
    def __init__(self, path, chunk_bytes: int = PF.CHUNK_BYTES, ring_slots: int = 3, use_cuda: bool = False):
        L = N.lib()
        L.saber_pack_stream_open.restype = C.c_void_p
        L.saber_pack_stream_open.argtypes = [C.c_char_p, C.c_size_t, C.c_int, C.c_int]
        L.saber_pack_stream_record.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_void_p, C.c_int,
                                               C.c_void_p, C.c_void_p]
        L.saber_pack_stream_close.argtypes = [C.c_void_p]
        L.saber_pack_stream_bytes.restype = C.c_uint64
        L.saber_pack_stream_bytes.argtypes = [C.c_void_p]
        L.saber_pack_stream_verified.restype = C.c_uint64
        L.saber_pack_stream_verified.argtypes = [C.c_void_p]
        L.saber_pack_stream_is_direct.argtypes = [C.c_void_p]
        self._L = L
        self._h = L.saber_pack_stream_open(str(path).encode(), chunk_bytes, ring_slots, int(use_cuda))
        if not self._h:
            raise PF.PackError(f"cannot open {path} for streaming")
        self.reader = PF.PackReader(path)
        self.use_cuda = use_cuda

    def read_host(self, name: str) -> np.ndarray:
        r = self.reader.records[name]
        out = np.empty(r.length, dtype=np.uint8)
        dig = b"".join(r.chunks)
        code = self._L.saber_pack_stream_record(self._h, r.data_off, r.length, out.ctypes.data, 0, dig, None)
        self._check(code, name)
        return out

    def read_device(self, name: str, dst_ptr: int, stream: int = 0) -> None:
        r = self.reader.records[name]
        code = self._L.saber_pack_stream_record(self._h, r.data_off, r.length, dst_ptr, 1, b"".join(r.chunks), stream)
        self._check(code, name)

    @staticmethod
    def _check(code: int, name: str) -> None:
        if code < 0:
            raise PF.PackError(f"{name}: read error while streaming")
        if code > 0:
            raise PF.PackError(f"{name}: chunk {code - 1} digest mismatch (nothing was uploaded past it)")

    @property
    def stats(self) -> dict:
        return {"bytes": self._L.saber_pack_stream_bytes(self._h), "chunks_verified": self._L.saber_pack_stream_verified(self._h),
                "o_direct": bool(self._L.saber_pack_stream_is_direct(self._h))}

    def close(self) -> None:
        if self._h:
            self._L.saber_pack_stream_close(self._h)
            self._h = None
