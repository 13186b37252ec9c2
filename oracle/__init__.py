"""TEST INFRASTRUCTURE — CPU checkers for the CUDA executor; never shipped.

Two executors with one Python face (`run(program, arena, rodata, ...)`):

* `RefExecutor`    — the reference's own CPU executor (oracle/_ref/libseeml_ref.so,
                     compiled from the reference's sources by oracle/Makefile).
* `OracleExecutor` — our C restatement of the same arithmetic
                     (oracle/libsee_oracle.so from oracle/see_oracle.c).

Only tests, the smoke check and the bench's CPU-baseline leg may import this
module.  The product package must never import it.
"""

from __future__ import annotations

import ctypes
import os
import struct
import subprocess
from typing import Optional, Sequence

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_LIB = os.path.join(HERE, "_ref", "libseeml_ref.so")
ORACLE_LIB = os.path.join(HERE, "libsee_oracle.so")


class StepParams(ctypes.Structure):
    _fields_ = [("lr", ctypes.c_float), ("beta1", ctypes.c_float),
                ("beta2", ctypes.c_float), ("eps", ctypes.c_float),
                ("weight_decay", ctypes.c_float), ("pad", ctypes.c_uint32),
                ("step", ctypes.c_uint64)]


def step_params(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, step=1):
    return StepParams(lr, beta1, beta2, eps, weight_decay, 0, step)


def build(target: str = "all") -> None:
    subprocess.run(["make", "-C", HERE, target], check=True, capture_output=True)


def _program_bytes(program) -> bytes:
    if isinstance(program, (bytes, bytearray, memoryview)):
        return bytes(program)
    return b"".join(i.pack() for i in program)


class _Executor:
    """Binds an arena (numpy uint8, mutated in place) and runs instruction words."""

    prefix = ""

    def __init__(self, lib_path: str):
        if not os.path.exists(lib_path):
            raise FileNotFoundError(lib_path)
        self.lib = ctypes.CDLL(lib_path)
        p = self.prefix
        self._create = getattr(self.lib, p + "create"); self._create.restype = ctypes.c_void_p
        self._destroy = getattr(self.lib, p + "destroy"); self._destroy.argtypes = [ctypes.c_void_p]
        self._bind = getattr(self.lib, p + "bind")
        self._bind.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64,
                               ctypes.c_void_p, ctypes.c_uint64]
        self._bind_source = getattr(self.lib, p + "bind_source")
        self._bind_source.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64]
        self._run = getattr(self.lib, p + "run")
        self._run.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64,
                              ctypes.c_uint64, ctypes.POINTER(StepParams)]
        self._run.restype = ctypes.c_int64
        self._err = getattr(self.lib, p + "last_error")
        self._err.argtypes = [ctypes.c_void_p]; self._err.restype = ctypes.c_char_p
        self.h = self._create()
        self._keep = []

    def close(self):
        if self.h:
            self._destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def bind(self, arena: np.ndarray, rodata: Optional[np.ndarray] = None,
             source: Optional[np.ndarray] = None):
        assert arena.dtype == np.uint8 and arena.flags.c_contiguous
        rodata = np.zeros(16, np.uint8) if rodata is None else np.ascontiguousarray(rodata)
        self._keep = [arena, rodata, source]
        if self._bind(self.h, arena.ctypes.data, arena.size, rodata.ctypes.data, rodata.size):
            raise RuntimeError(self._err(self.h).decode())
        if source is not None:
            self._bind_source(self.h, source.ctypes.data, source.size)

    def run(self, program, sp: Optional[StepParams] = None, begin: int = 0,
            end: Optional[int] = None):
        raw = _program_bytes(program)
        n = len(raw) // 64
        end = n if end is None else end
        buf = ctypes.create_string_buffer(raw, len(raw))
        sp = sp or step_params()
        rc = self._run(self.h, buf, begin, end, ctypes.byref(sp))
        if rc:
            raise RuntimeError(f"instruction {rc - 1}: {self._err(self.h).decode()}")


class RefExecutor(_Executor):
    prefix = "seeref_"

    def __init__(self):
        super().__init__(REF_LIB)
        self.lib.seeref_set_threads.argtypes = [ctypes.c_uint64]
        self.lib.seeref_threads.restype = ctypes.c_uint64

    def set_threads(self, n: int):
        self.lib.seeref_set_threads(n)

    def threads(self) -> int:
        return int(self.lib.seeref_threads())


class OracleExecutor(_Executor):
    prefix = "seeo_"

    def __init__(self):
        super().__init__(ORACLE_LIB)


def have_ref() -> bool:
    return os.path.exists(REF_LIB)


def have_oracle() -> bool:
    return os.path.exists(ORACLE_LIB)
