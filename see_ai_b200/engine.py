"""ctypes binding of the C++ UpdateEngine (see_engine_* in include/see_cuda.h):
the dispatcher that loads a sealed `.seeu` plan, owns the device slab and runs
the plan's programs (reference: runtime/dispatcher/update_engine.h:211-367).
"""

from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import numpy as np

from . import backend as B
from . import plan as P

ENGINE_SYMBOLS = [
    "see_engine_create", "see_engine_destroy", "see_engine_last_error", "see_engine_backend",
    "see_engine_load", "see_engine_bind_source", "see_engine_header", "see_engine_stage_batch",
    "see_engine_train_forward_backward", "see_engine_train_optimizer", "see_engine_step_program",
    "see_engine_read_loss", "see_engine_evaluate", "see_engine_evaluate_rows", "see_engine_run_merge",
    "see_engine_read_arena", "see_engine_write_arena", "see_engine_step", "see_engine_set_step",
    "see_engine_set_horizon", "see_engine_effective_lr", "see_engine_set_use_graphs",
    "see_engine_set_phase_timing", "see_engine_take_timings", "see_engine_gradient_block",
    "see_engine_snapshot_begin", "see_engine_snapshot_wait", "see_engine_restore",
    "see_cuda_exchange_id", "see_engine_attach_exchange", "see_engine_detach_exchange", "see_engine_exchange",
]

_configured = False


def make_exchange_id() -> bytes:
    """A fresh communicator id for Engine.attach_exchange (made on one rank, handed to all)."""
    lib = _lib()
    buf = (ctypes.c_uint8 * 128)()
    if lib.see_cuda_exchange_id(buf) != 0:
        raise RuntimeError(lib.see_cuda_create_error().decode())
    return bytes(buf)


class EvalResult(ctypes.Structure):
    """see_eval_result of include/see_cuda.h."""
    _fields_ = [("loss", ctypes.c_float), ("has_accuracy", ctypes.c_uint32), ("rows", ctypes.c_uint64),
                ("correct", ctypes.c_uint64), ("real_row_loss", ctypes.c_double),
                ("loss_rows", ctypes.c_uint64)]


def _lib() -> ctypes.CDLL:
    global _configured
    lib = B.load_library()
    if _configured:
        return lib
    vp, u64, i32 = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int
    lib.see_engine_create.argtypes = [i32, ctypes.POINTER(vp)]
    lib.see_engine_destroy.argtypes = [vp]
    lib.see_engine_destroy.restype = None
    lib.see_engine_last_error.argtypes = [vp]
    lib.see_engine_last_error.restype = ctypes.c_char_p
    lib.see_engine_backend.argtypes = [vp]
    lib.see_engine_backend.restype = vp
    lib.see_engine_load.argtypes = [vp, vp, u64]
    lib.see_engine_bind_source.argtypes = [vp, vp, u64]
    lib.see_engine_header.argtypes = [vp, vp]
    lib.see_engine_stage_batch.argtypes = [vp, vp, u64, vp, u64]
    lib.see_engine_train_forward_backward.argtypes = [vp, i32]
    lib.see_engine_train_optimizer.argtypes = [vp]
    lib.see_engine_step_program.argtypes = [vp]
    lib.see_engine_read_loss.argtypes = [vp, ctypes.POINTER(ctypes.c_float)]
    lib.see_engine_evaluate.argtypes = [vp, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(u64),
                                        ctypes.POINTER(u64)]
    lib.see_engine_evaluate_rows.argtypes = [vp, u64, ctypes.POINTER(EvalResult)]
    lib.see_engine_run_merge.argtypes = [vp, ctypes.POINTER(i32)]
    lib.see_engine_read_arena.argtypes = [vp, u64, u64, vp]
    lib.see_engine_write_arena.argtypes = [vp, u64, u64, vp]
    lib.see_engine_step.argtypes = [vp]
    lib.see_engine_step.restype = u64
    lib.see_engine_set_step.argtypes = [vp, u64]
    lib.see_engine_set_horizon.argtypes = [vp, u64]
    lib.see_engine_effective_lr.argtypes = [vp]
    lib.see_engine_effective_lr.restype = ctypes.c_float
    lib.see_engine_set_use_graphs.argtypes = [vp, i32]
    lib.see_engine_set_phase_timing.argtypes = [vp, i32]
    lib.see_engine_take_timings.argtypes = [vp] + [ctypes.POINTER(ctypes.c_float)] * 3 + \
        [ctypes.POINTER(u64)]
    lib.see_engine_gradient_block.argtypes = [vp, ctypes.POINTER(u64), ctypes.POINTER(u64)]
    lib.see_cuda_exchange_id.argtypes = [vp]
    lib.see_engine_attach_exchange.argtypes = [vp, ctypes.c_int, ctypes.c_int, vp]
    lib.see_engine_detach_exchange.argtypes = [vp]
    lib.see_engine_exchange.argtypes = [vp]
    lib.see_engine_snapshot_begin.argtypes = [vp]
    lib.see_engine_snapshot_wait.argtypes = [vp, vp, u64]
    lib.see_engine_restore.argtypes = [vp, vp, u64, u64]
    _configured = True
    return lib


class _BorrowedBackend(B.CudaBackend):
    """The engine's own backend, for the see_cuda_* knobs.  Not destroyed here."""

    def __init__(self, lib, handle):  # noqa: D401 - no create call
        self.lib = lib
        self.h = handle
        self._keep = []
        self._prog = None

    def close(self):
        self.h = None


class Engine:
    def __init__(self, device: int = 0):
        self.lib = _lib()
        h = ctypes.c_void_p()
        if self.lib.see_engine_create(device, ctypes.byref(h)) != B.SEE_OK:
            raise B.BackendError(self.lib.see_cuda_create_error().decode())
        self.h = h
        self.backend = _BorrowedBackend(self.lib, ctypes.c_void_p(self.lib.see_engine_backend(h)))
        self.header: dict = {}
        self._keep = None

    def close(self):
        if getattr(self, "h", None):
            self.lib.see_engine_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc == B.SEE_OK:
            return
        msg = self.lib.see_engine_last_error(self.h).decode()
        raise (B.Refusal if rc == B.SEE_REFUSED else B.BackendError)(msg)

    def load(self, blob: bytes):
        buf = np.frombuffer(blob, dtype=np.uint8)
        self._check(self.lib.see_engine_load(self.h, buf.ctypes.data, buf.size))
        raw = ctypes.create_string_buffer(P.HEADER_BYTES)
        self.lib.see_engine_header(self.h, raw)
        vals = P._HEADER.unpack_from(raw.raw, 0)
        self.header = {n: v for (n, _), v in zip(P._HEADER_FIELDS, vals)}
        train = P.Plan(blob).section("train")   # decodes the header and the instruction words only
        self.has_masked_loss = any(i.opcode in (P.Op.XENT_MASKED_FWD, P.Op.XENT_MASKED_BWD) for i in train)

    def bind_source(self, data: Optional[np.ndarray]):
        if data is None:
            self._check(self.lib.see_engine_bind_source(self.h, None, 0))
            return
        data = np.ascontiguousarray(data)
        self._check(self.lib.see_engine_bind_source(self.h, data.ctypes.data, data.size))

    def stage_batch(self, x: np.ndarray, y: Optional[np.ndarray]):
        x = np.ascontiguousarray(x)
        yb = np.ascontiguousarray(y) if y is not None else None
        self._check(self.lib.see_engine_stage_batch(
            self.h, x.ctypes.data, x.nbytes,
            yb.ctypes.data if yb is not None else None, yb.nbytes if yb is not None else 0))

    def train_forward_backward(self, advance: bool = True):
        self._check(self.lib.see_engine_train_forward_backward(self.h, int(advance)))

    def train_optimizer(self):
        self._check(self.lib.see_engine_train_optimizer(self.h))

    def step_program(self):
        self._check(self.lib.see_engine_step_program(self.h))

    def read_loss(self) -> float:
        v = ctypes.c_float()
        self._check(self.lib.see_engine_read_loss(self.h, ctypes.byref(v)))
        return float(np.float32(v.value))

    def train_step(self, x, y) -> float:
        """One optimizer step of a plan without gradient accumulation."""
        self.stage_batch(x, y)
        self.train_forward_backward(True)
        self.train_optimizer()
        return self.read_loss()

    def evaluate(self, x, y) -> Tuple[float, int, int]:
        self.stage_batch(x, y)
        loss, rows, correct = ctypes.c_float(), ctypes.c_uint64(), ctypes.c_uint64()
        self._check(self.lib.see_engine_evaluate(self.h, ctypes.byref(loss), ctypes.byref(rows),
                                                 ctypes.byref(correct)))
        return float(np.float32(loss.value)), int(rows.value), int(correct.value)

    def evaluate_rows(self, x, y, real_rows: int) -> EvalResult:
        """Evaluates one staged batch whose first `real_rows` rows are real (the
        rest wrapped duplicates): accuracy tallies and the real-row loss."""
        self.stage_batch(x, y)
        out = EvalResult()
        self._check(self.lib.see_engine_evaluate_rows(self.h, real_rows, ctypes.byref(out)))
        return out

    def run_merge(self) -> bool:
        ok = ctypes.c_int()
        self._check(self.lib.see_engine_run_merge(self.h, ctypes.byref(ok)))
        return bool(ok.value)

    def read_arena(self, offset: int, nbytes: int) -> np.ndarray:
        out = np.empty(nbytes, dtype=np.uint8)
        self._check(self.lib.see_engine_read_arena(self.h, offset, nbytes, out.ctypes.data))
        return out

    def write_arena(self, offset: int, data: np.ndarray):
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        self._check(self.lib.see_engine_write_arena(self.h, offset, data.size, data.ctypes.data))

    def read_persistent(self) -> np.ndarray:
        return self.read_arena(0, self.header["persistent_size"])

    @property
    def step(self) -> int:
        return int(self.lib.see_engine_step(self.h))

    def set_step(self, step: int):
        self._check(self.lib.see_engine_set_step(self.h, step))

    def set_horizon(self, steps: int):
        self._check(self.lib.see_engine_set_horizon(self.h, steps))

    def effective_lr(self) -> float:
        return float(self.lib.see_engine_effective_lr(self.h))

    def set_use_graphs(self, on: bool):
        self._check(self.lib.see_engine_set_use_graphs(self.h, int(on)))

    def set_phase_timing(self, on: bool):
        self._check(self.lib.see_engine_set_phase_timing(self.h, int(on)))

    def take_timings(self):
        f, b, o = ctypes.c_float(), ctypes.c_float(), ctypes.c_float()
        n = ctypes.c_uint64()
        self._check(self.lib.see_engine_take_timings(self.h, ctypes.byref(f), ctypes.byref(b),
                                                     ctypes.byref(o), ctypes.byref(n)))
        return dict(forward_ms=f.value, backward_ms=b.value, optimizer_ms=o.value, steps=n.value)

    def snapshot_begin(self):
        """Starts an asynchronous copy of the persistent prefix as it is now."""
        self._check(self.lib.see_engine_snapshot_begin(self.h))

    def snapshot_wait(self) -> np.ndarray:
        """Blocks until the snapshot begun last is on the host; returns its bytes."""
        out = np.empty(self.header["persistent_size"], dtype=np.uint8)
        self._check(self.lib.see_engine_snapshot_wait(self.h, out.ctypes.data_as(ctypes.c_void_p), out.size))
        return out

    def restore(self, persistent: np.ndarray, step: int):
        """Resume: the persistent prefix back into the arena, the timestep set."""
        data = np.ascontiguousarray(persistent, dtype=np.uint8)
        self._check(self.lib.see_engine_restore(self.h, data.ctypes.data_as(ctypes.c_void_p), data.size, step))

    def gradient_block(self) -> Tuple[int, int]:
        off, n = ctypes.c_uint64(), ctypes.c_uint64()
        self._check(self.lib.see_engine_gradient_block(self.h, ctypes.byref(off), ctypes.byref(n)))
        return int(off.value), int(n.value)

    # -- data parallelism: the NCCL all-gather of the gradient block inside the library --
    def attach_exchange(self, world: int, rank: int, comm_id: bytes):
        """Collective over the ranks (same 128-byte id everywhere); world <= 1 detaches."""
        buf = (ctypes.c_uint8 * 128).from_buffer_copy(comm_id) if comm_id else None
        self._check(self.lib.see_engine_attach_exchange(self.h, world, rank, buf))

    def detach_exchange(self):
        self._check(self.lib.see_engine_detach_exchange(self.h))

    def exchange(self):
        """Enqueues this step's all-gather now (otherwise the optimizer call does it)."""
        self._check(self.lib.see_engine_exchange(self.h))
