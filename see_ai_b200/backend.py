"""ctypes binding of libsee_cuda.so and a thin `CudaBackend` mirroring the
reference's backend seam (Bind / BindSource / Execute / BeginRange / EndRange /
Flush; reference: runtime/executor/backend.h:82-166).

The library is the product; this module adds nothing to the arithmetic.  If the
shared library is missing, importing `CudaBackend` still works but constructing
one raises — there is no CPU path here.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libsee_cuda.so")

SEE_OK, SEE_ERROR, SEE_REFUSED = 0, 1, 2
COHERENCE_STRICT, COHERENCE_LAZY = 0, 1

# Every symbol include/see_cuda.h declares.
EXPORTED_SYMBOLS = [
    "see_cuda_create", "see_cuda_create_error", "see_cuda_destroy", "see_cuda_name",
    "see_cuda_device", "see_cuda_last_error", "see_cuda_bind", "see_cuda_bind_source",
    "see_cuda_begin_range", "see_cuda_execute", "see_cuda_end_range", "see_cuda_flush",
    "see_cuda_run_range", "see_cuda_set_coherence", "see_cuda_host_wrote",
    "see_cuda_host_needs", "see_cuda_counters_get", "see_cuda_set_stream",
    "see_cuda_device_arena", "see_cuda_set_relaxed_allowed", "see_cuda_set_epilogue_fusion",
    "see_cuda_set_gradient_gather",
    "see_cuda_set_profiling", "see_cuda_take_profile",
    "see_cuda_xent_forward_static", "see_cuda_static_max_rows", "see_cuda_static_last_error",
    "see_cuda_quantize_columns", "see_cuda_set_lora_fold", "see_cuda_set_adapter_fma", "see_cuda_set_split_gemm", "see_cuda_set_cta_pairs", "see_cuda_set_adapter_tensor_backward", "see_cuda_set_attention_one_walk",
]


class StepParams(ctypes.Structure):
    _fields_ = [("lr", ctypes.c_float), ("beta1", ctypes.c_float), ("beta2", ctypes.c_float),
                ("eps", ctypes.c_float), ("weight_decay", ctypes.c_float),
                ("pad", ctypes.c_uint32), ("step", ctypes.c_uint64)]


class Counters(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint64) for n in
                ("relaxed_executions", "fused_dispatches", "kernel_launches", "h2d_bytes",
                 "d2h_bytes", "instructions", "split_executions")]


class ProfileRecord(ctypes.Structure):
    _fields_ = [("opcode", ctypes.c_uint16), ("absorbed", ctypes.c_uint16), ("index", ctypes.c_uint32),
                ("ms", ctypes.c_float), ("kernel_ms", ctypes.c_float), ("m", ctypes.c_uint64),
                ("n", ctypes.c_uint64), ("k", ctypes.c_uint64)]


class BackendError(RuntimeError):
    pass


class Refusal(BackendError):
    """The step was refused (non-finite gradient norm or a bad clip threshold)."""


_lib = None


def load_library() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise BackendError(
            f"{LIB_PATH} is missing: build it with `python -m see_ai_b200.build` "
            "(there is no CPU fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    vp, u64, i32 = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_int
    lib.see_cuda_create.argtypes = [i32, ctypes.POINTER(vp)]
    lib.see_cuda_create_error.restype = ctypes.c_char_p
    lib.see_cuda_destroy.argtypes = [vp]
    lib.see_cuda_destroy.restype = None
    for name in ("see_cuda_name", "see_cuda_device", "see_cuda_last_error"):
        getattr(lib, name).argtypes = [vp]
        getattr(lib, name).restype = ctypes.c_char_p
    lib.see_cuda_bind.argtypes = [vp, vp, u64, vp, u64]
    lib.see_cuda_bind_source.argtypes = [vp, vp, u64]
    lib.see_cuda_begin_range.argtypes = [vp, vp, u64, u64, u64]
    lib.see_cuda_execute.argtypes = [vp, vp, ctypes.POINTER(StepParams)]
    lib.see_cuda_end_range.argtypes = [vp]
    lib.see_cuda_flush.argtypes = [vp]
    lib.see_cuda_run_range.argtypes = [vp, vp, u64, u64, u64, ctypes.POINTER(StepParams),
                                       ctypes.POINTER(u64)]
    lib.see_cuda_set_coherence.argtypes = [vp, i32]
    lib.see_cuda_host_wrote.argtypes = [vp, u64, u64]
    lib.see_cuda_host_needs.argtypes = [vp, u64, u64]
    lib.see_cuda_counters_get.argtypes = [vp, ctypes.POINTER(Counters)]
    lib.see_cuda_set_stream.argtypes = [vp, vp]
    lib.see_cuda_device_arena.argtypes = [vp]
    lib.see_cuda_device_arena.restype = vp
    lib.see_cuda_set_relaxed_allowed.argtypes = [vp, i32]
    lib.see_cuda_set_epilogue_fusion.argtypes = [vp, i32]
    lib.see_cuda_set_gradient_gather.argtypes = [vp, i32, vp, u64, u64]
    lib.see_cuda_set_profiling.argtypes = [vp, i32]
    lib.see_cuda_take_profile.argtypes = [vp, ctypes.POINTER(ProfileRecord), u64]
    lib.see_cuda_take_profile.restype = ctypes.c_int64
    lib.see_cuda_quantize_columns.argtypes = [vp, vp, u64, u64, vp, vp]
    lib.see_cuda_set_lora_fold.argtypes = [vp, i32]
    lib.see_cuda_set_adapter_fma.argtypes = [vp, i32]
    lib.see_cuda_set_split_gemm.argtypes = [vp, i32]
    lib.see_cuda_set_cta_pairs.argtypes = [i32]
    lib.see_cuda_set_adapter_tensor_backward.argtypes = [i32]
    lib.see_cuda_set_attention_one_walk.argtypes = [vp, i32]
    lib.see_cuda_xent_forward_static.argtypes = [vp, vp, vp, vp, u64, u64, i32, vp]
    lib.see_cuda_static_max_rows.restype = u64
    lib.see_cuda_static_last_error.restype = ctypes.c_char_p
    _lib = lib
    return lib


def xent_forward_static(logits_ptr: int, labels_ptr: int, loss_ptr: int, probs_ptr: int,
                        rows: int, classes: int, masked: bool = False, stream: int = 0) -> None:
    """Softmax cross-entropy forward over DEVICE pointers with no allocation:
    the scratch is a fixed array inside the library (at most
    see_cuda_static_max_rows() rows).  For callers that may not call cudaMalloc."""
    lib = load_library()
    rc = lib.see_cuda_xent_forward_static(ctypes.c_void_p(logits_ptr), ctypes.c_void_p(labels_ptr),
                                          ctypes.c_void_p(loss_ptr), ctypes.c_void_p(probs_ptr),
                                          rows, classes, int(masked), ctypes.c_void_p(stream))
    if rc != SEE_OK:
        raise BackendError(lib.see_cuda_static_last_error().decode())


def program_bytes(program) -> bytes:
    if isinstance(program, (bytes, bytearray, memoryview)):
        return bytes(program)
    return b"".join(i.pack() for i in program)


class CudaBackend:
    """One handle per GPU.  `arena` passed to bind() is mutated in place by
    flush() (strict coherence) or host_needs() (lazy)."""

    def __init__(self, device: int = 0):
        self.lib = load_library()
        h = ctypes.c_void_p()
        if self.lib.see_cuda_create(device, ctypes.byref(h)) != SEE_OK:
            raise BackendError(self.lib.see_cuda_create_error().decode())
        self.h = h
        self._keep = []
        self._prog = None

    def close(self):
        if getattr(self, "h", None):
            self.lib.see_cuda_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc == SEE_OK:
            return
        msg = self.lib.see_cuda_last_error(self.h).decode()
        raise (Refusal if rc == SEE_REFUSED else BackendError)(msg)

    @property
    def name(self) -> str:
        return self.lib.see_cuda_name(self.h).decode()

    @property
    def device(self) -> str:
        return self.lib.see_cuda_device(self.h).decode()

    def bind(self, arena: np.ndarray, rodata: Optional[np.ndarray] = None):
        assert arena.dtype == np.uint8 and arena.flags.c_contiguous
        if rodata is not None:
            rodata = np.ascontiguousarray(rodata)
        self._keep = [arena, rodata]
        self._check(self.lib.see_cuda_bind(
            self.h, arena.ctypes.data, arena.size,
            rodata.ctypes.data if rodata is not None and rodata.size else None,
            rodata.size if rodata is not None else 0))

    def bind_source(self, data: Optional[np.ndarray]):
        if data is None:
            self._check(self.lib.see_cuda_bind_source(self.h, None, 0))
            return
        data = np.ascontiguousarray(data)
        self._check(self.lib.see_cuda_bind_source(self.h, data.ctypes.data, data.size))

    def set_program(self, program):
        raw = program_bytes(program)
        self._prog = (ctypes.create_string_buffer(raw, len(raw)), len(raw) // 64)

    def run(self, program=None, params: Optional[StepParams] = None, begin: int = 0,
            end: Optional[int] = None):
        """BeginRange, Execute each instruction of [begin, end), Flush, EndRange."""
        if program is not None:
            self.set_program(program)
        buf, n = self._prog
        end = n if end is None else end
        params = params or StepParams(1e-3, 0.9, 0.999, 1e-8, 0.01, 0, 1)
        failed = ctypes.c_uint64(0)
        self._check(self.lib.see_cuda_run_range(self.h, buf, n, begin, end, ctypes.byref(params),
                                                ctypes.byref(failed)))

    def begin_range(self, begin: int, end: int):
        buf, n = self._prog
        self._check(self.lib.see_cuda_begin_range(self.h, buf, n, begin, end))

    def execute(self, index: int, params: StepParams):
        buf, n = self._prog
        ptr = ctypes.cast(ctypes.addressof(buf) + 64 * index, ctypes.c_void_p)
        self._check(self.lib.see_cuda_execute(self.h, ptr, ctypes.byref(params)))

    def end_range(self):
        self._check(self.lib.see_cuda_end_range(self.h))

    def flush(self):
        self._check(self.lib.see_cuda_flush(self.h))

    def set_coherence(self, mode: int):
        self._check(self.lib.see_cuda_set_coherence(self.h, mode))

    def host_wrote(self, offset: int, nbytes: int):
        self._check(self.lib.see_cuda_host_wrote(self.h, offset, nbytes))

    def host_needs(self, offset: int, nbytes: int):
        self._check(self.lib.see_cuda_host_needs(self.h, offset, nbytes))

    def counters(self) -> Counters:
        c = Counters()
        self._check(self.lib.see_cuda_counters_get(self.h, ctypes.byref(c)))
        return c

    def set_stream(self, stream_handle: int):
        self._check(self.lib.see_cuda_set_stream(self.h, ctypes.c_void_p(stream_handle)))

    def device_arena(self) -> int:
        return int(self.lib.see_cuda_device_arena(self.h) or 0)

    def set_relaxed_allowed(self, allowed: bool):
        self._check(self.lib.see_cuda_set_relaxed_allowed(self.h, int(allowed)))

    def set_epilogue_fusion(self, enabled: bool):
        self._check(self.lib.see_cuda_set_epilogue_fusion(self.h, int(enabled)))

    def set_lora_fold(self, enabled: bool):
        self._check(self.lib.see_cuda_set_lora_fold(self.h, int(enabled)))

    def set_adapter_fma(self, enabled: bool):
        self._check(self.lib.see_cuda_set_adapter_fma(self.h, int(enabled)))

    def set_split_gemm(self, mode: int):
        """-1: exact f32 products on the tensor cores in lazy coherence only; 0 never; 1 always."""
        self._check(self.lib.see_cuda_set_split_gemm(self.h, mode))

    def set_attention_one_walk(self, enabled: bool):
        self._check(self.lib.see_cuda_set_attention_one_walk(self.h, int(enabled)))

    def set_cta_pairs(self, enabled: bool):
        """Process-wide: large tensor-core products on CTA pairs (default) or one CTA per tile."""
        self._check(self.lib.see_cuda_set_cta_pairs(int(enabled)))

    def set_adapter_tensor_backward(self, enabled: bool):
        """Process-wide: adapter backward sites on the tcgen05 tensor cores (default) or the legacy instruction."""
        self._check(self.lib.see_cuda_set_adapter_tensor_backward(int(enabled)))

    def set_gradient_gather(self, ranks: int, gathered_ptr: int, block_offset: int,
                            block_bytes: int):
        self._check(self.lib.see_cuda_set_gradient_gather(
            self.h, ranks, ctypes.c_void_p(gathered_ptr), block_offset, block_bytes))

    def quantize_columns(self, w_ptr: int, K: int, N: int, levels_ptr: int, scales_ptr: int):
        """Per-column int8 quantisation of W [K, N] over DEVICE pointers."""
        self._check(self.lib.see_cuda_quantize_columns(self.h, ctypes.c_void_p(w_ptr), K, N,
                                                       ctypes.c_void_p(levels_ptr), ctypes.c_void_p(scales_ptr)))

    def set_profiling(self, on: bool):
        self._check(self.lib.see_cuda_set_profiling(self.h, int(on)))

    def take_profile(self, capacity: int = 65536, with_absorbed: bool = False):
        """(opcode, index, ms, m, n, k, kernel_ms) per executed instruction; with
        `with_absorbed` an eighth field: how many following instructions the
        instruction also did (epilogue fusion)."""
        arr = (ProfileRecord * capacity)()
        n = self.lib.see_cuda_take_profile(self.h, arr, capacity)
        if with_absorbed:
            return [(r.opcode, r.index, r.ms, r.m, r.n, r.k, r.kernel_ms, r.absorbed) for r in arr[:n]]
        return [(r.opcode, r.index, r.ms, r.m, r.n, r.k, r.kernel_ms) for r in arr[:n]]
