"""Reader and writer for UBJSON (Universal Binary JSON, draft 12), the binary twin of XGBoost's JSON
model file (`Booster.save_model("model.ubj")`).

The reader covers the whole value grammar: null, no-op, booleans, the five integer widths, both
float widths, high-precision numbers, chars, strings, arrays and objects, including the optimised
containers (`$` type marker and `#` count) that XGBoost uses for its numeric arrays.  The writer
emits typed, counted arrays for homogeneous numeric lists, like XGBoost does, so files made here
exercise the same reader paths.  Written from the published specification; XGBoost is not
installed here, so only files produced by this module have been read.
"""
from __future__ import annotations

import struct
from typing import Any, Tuple

import numpy as np

_INT = {b"i": (">b", 1), b"U": (">B", 1), b"I": (">h", 2), b"l": (">i", 4), b"L": (">q", 8)}
_FLT = {b"d": (">f", 4), b"D": (">d", 8)}
_NP = {b"i": ">i1", b"U": ">u1", b"I": ">i2", b"l": ">i4", b"L": ">i8", b"d": ">f4", b"D": ">f8"}


class _Reader:
    def __init__(self, data: bytes):
        self.d = memoryview(data)
        self.p = 0

    def take(self, n: int) -> bytes:
        if self.p + n > len(self.d):
            raise ValueError("UBJSON: unexpected end of data")
        b = bytes(self.d[self.p:self.p + n])
        self.p += n
        return b

    def marker(self) -> bytes:
        m = self.take(1)
        while m == b"N":  # no-op
            m = self.take(1)
        return m

    def length(self) -> int:
        m = self.marker()
        if m not in _INT:
            raise ValueError(f"UBJSON: bad length marker {m!r}")
        n = self.scalar(m)
        if n < 0:
            raise ValueError("UBJSON: negative length")
        return n

    def scalar(self, m: bytes):
        if m in _INT:
            fmt, n = _INT[m]
            return struct.unpack(fmt, self.take(n))[0]
        if m in _FLT:
            fmt, n = _FLT[m]
            return struct.unpack(fmt, self.take(n))[0]
        raise ValueError(f"UBJSON: not a number marker {m!r}")

    def string(self) -> str:
        return self.take(self.length()).decode("utf-8")

    def value(self, m: bytes | None = None) -> Any:
        if m is None:
            m = self.marker()
        if m == b"Z":
            return None
        if m == b"T":
            return True
        if m == b"F":
            return False
        if m in _INT or m in _FLT:
            return self.scalar(m)
        if m == b"C":
            return self.take(1).decode("latin-1")
        if m == b"S":
            return self.string()
        if m == b"H":
            s = self.string()
            try:
                return int(s)
            except ValueError:
                return float(s)
        if m == b"[":
            return self.array()
        if m == b"{":
            return self.object()
        raise ValueError(f"UBJSON: unknown marker {m!r} at byte {self.p - 1}")

    def container_header(self) -> Tuple[bytes | None, int | None]:
        typ, count = None, None
        nxt = bytes(self.d[self.p:self.p + 1])
        if nxt == b"$":
            self.p += 1
            typ = self.take(1)
            if bytes(self.d[self.p:self.p + 1]) != b"#":
                raise ValueError("UBJSON: a typed container needs a count")
            nxt = b"#"
        if nxt == b"#":
            self.p += 1
            count = self.length()
        return typ, count

    def array(self):
        typ, count = self.container_header()
        if count is not None:
            if typ in _NP:  # homogeneous numbers: one bulk conversion
                width = np.dtype(_NP[typ]).itemsize
                arr = np.frombuffer(self.take(count * width), dtype=_NP[typ])
                return arr.tolist()
            if typ in (b"T", b"F", b"Z"):
                return [{b"T": True, b"F": False, b"Z": None}[typ]] * count
            return [self.value(typ) for _ in range(count)]
        out = []
        while True:
            m = self.marker()
            if m == b"]":
                return out
            out.append(self.value(m))

    def object(self):
        typ, count = self.container_header()
        out = {}
        if count is not None:
            for _ in range(count):
                k = self.string()
                out[k] = self.value(typ)
            return out
        while True:
            if bytes(self.d[self.p:self.p + 1]) == b"}":
                self.p += 1
                return out
            k = self.string()
            out[k] = self.value()


def loads(data: bytes) -> Any:
    """Decode one UBJSON value."""
    return _Reader(data).value()


def _w_int(n: int) -> bytes:
    if -128 <= n <= 127:
        return b"i" + struct.pack(">b", n)
    if 0 <= n <= 255:
        return b"U" + struct.pack(">B", n)
    if -32768 <= n <= 32767:
        return b"I" + struct.pack(">h", n)
    if -2 ** 31 <= n < 2 ** 31:
        return b"l" + struct.pack(">i", n)
    return b"L" + struct.pack(">q", n)


def _w_str(s: str) -> bytes:
    b = s.encode("utf-8")
    return _w_int(len(b)) + b


def dumps(obj: Any, float32: bool = True) -> bytes:
    """Encode a JSON-like value.  Lists of floats become typed arrays (`[$d#...`, or `$D` when
    `float32` is False), lists of ints typed int32 / int64 arrays."""
    if obj is None:
        return b"Z"
    if obj is True:
        return b"T"
    if obj is False:
        return b"F"
    if isinstance(obj, (int, np.integer)):
        return _w_int(int(obj))
    if isinstance(obj, (float, np.floating)):
        return (b"d" + struct.pack(">f", obj)) if float32 else (b"D" + struct.pack(">d", obj))
    if isinstance(obj, str):
        return b"S" + _w_str(obj)
    if isinstance(obj, dict):
        return b"{" + b"".join(_w_str(str(k)) + dumps(v, float32) for k, v in obj.items()) + b"}"
    if isinstance(obj, (list, tuple, np.ndarray)):
        seq = list(obj)
        if seq and all(isinstance(v, (float, np.floating)) for v in seq):
            dt, mk = (">f4", b"d") if float32 else (">f8", b"D")
            return b"[$" + mk + b"#" + _w_int(len(seq)) + np.asarray(seq, dt).tobytes()
        if seq and all(isinstance(v, (int, np.integer)) and not isinstance(v, bool) for v in seq):
            big = any(not (-2 ** 31 <= int(v) < 2 ** 31) for v in seq)
            dt, mk = (">i8", b"L") if big else (">i4", b"l")
            return b"[$" + mk + b"#" + _w_int(len(seq)) + np.asarray(seq, dt).tobytes()
        return b"[" + b"".join(dumps(v, float32) for v in seq) + b"]"
    raise TypeError(f"cannot encode {type(obj).__name__} as UBJSON")
