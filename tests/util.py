"""Shared helpers for the parity tests: golden-case loading, the comparison
rule and the lockstep driver."""

from __future__ import annotations

import os

import numpy as np

from see_ai_b200 import plan as P

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = ["mlp_tiny", "mlp_unfused_clip", "mlp_global_clip", "mlp_sgd_accum",
         "gpt_tiny_cached", "gpt_tiny_tiled", "gpt_tiny_q8_relaxed", "llama_tiny_bf16"]

Op = P.Op

# Opcodes whose results are a fixed sequence of individually rounded f32 (or
# exact double) operations with no libm call and no reordered sum: identical
# bits to the reference CPU executor are required of them.
BIT_EXACT = {
    Op.NOP, Op.GEMM_NN, Op.GEMM_NT, Op.GEMM_TN, Op.GEMM_ACC_NN, Op.GEMM_NN_Q8, Op.GEMM_NT_Q8,
    Op.GEMM_NN_BF16, Op.GEMM_NT_BF16, Op.ADD_EW, Op.MUL_EW, Op.ADD_BIAS, Op.RELU_FWD,
    Op.RELU_BWD, Op.SCALE, Op.REDUCE_ROWS, Op.XENT_BWD, Op.XENT_MASKED_BWD, Op.FILL, Op.COPY,
    Op.ACCUMULATE, Op.EMBED_FWD, Op.SEGMENT_STARTS, Op.ATTN_DP, Op.ATTN_DV, Op.ATTN_DQ,
    Op.ATTN_DK, Op.MSE_BWD, Op.KL_BWD,
}
# GEMMs with a fused transcendental activation are exact only up to that call.
GEMM_OPS = {Op.GEMM_NN, Op.GEMM_NN_Q8, Op.GEMM_NN_BF16}


class Case:
    def __init__(self, name: str):
        z = np.load(os.path.join(GOLDEN, name + ".npz"))
        self.name = name
        self.z = z
        self.plan = P.Plan(z["plan"].tobytes())
        self.header = self.plan.header
        self.rodata = np.frombuffer(self.plan.rodata, dtype=np.uint8).copy()
        self.source = z["source_model"] if "source_model" in z else None
        self.lr = float(z["lr"])
        self.runs = []
        for i in range(int(z["n_runs"])):
            self.runs.append(dict(
                section=str(z[f"run{i}_section"]), step=int(z[f"run{i}_step"]),
                x=z[f"run{i}_x"] if f"run{i}_x" in z else None,
                y=z[f"run{i}_y"] if f"run{i}_y" in z else None,
                trace=P.read_trace(z[f"run{i}_trace"].tobytes())))
        self.final_arena = z["final_arena"]

    def stage_batch(self, arena: np.ndarray, run) -> list:
        """Writes the run's batch into the I/O slots; returns the written extents."""
        if run["x"] is None:
            return []
        h = self.header
        xb = np.ascontiguousarray(run["x"]).view(np.uint8).reshape(-1)
        yb = np.ascontiguousarray(run["y"]).view(np.uint8).reshape(-1)
        arena[h["input_ref"]:h["input_ref"] + xb.size] = xb
        arena[h["label_ref"]:h["label_ref"] + yb.size] = yb
        return [(h["input_ref"], xb.size), (h["label_ref"], yb.size)]

    def step_params(self, cls, step: int):
        h = self.header
        return cls(self.lr, h["beta1"], h["beta2"], h["eps"], h["weight_decay"], 0, step)


def is_i32_extent(op: int, ext_index: int) -> bool:
    return op == Op.SEGMENT_STARTS


def compare(got: bytes, want: bytes, rtol: float, atol: float):
    """The reference differ's rule, per written extent: |a-b| <= atol + rtol*max|b|
    (reference: tool/frontier_exec.py:49-55).  Returns (ok, worst error / bound)."""
    a = np.frombuffer(got, dtype=np.float32).astype(np.float64)
    b = np.frombuffer(want, dtype=np.float32).astype(np.float64)
    nan_a, nan_b = np.isnan(a), np.isnan(b)
    if not np.array_equal(nan_a, nan_b):
        return False, float("inf")
    fin = ~nan_b
    if not fin.any():
        return True, 0.0
    inf_b = np.isinf(b)
    if not np.array_equal(a[inf_b], b[inf_b]):
        return False, float("inf")
    fin &= ~inf_b
    if not fin.any():
        return True, 0.0
    bound = atol + rtol * np.max(np.abs(b[fin]))
    err = np.max(np.abs(a[fin] - b[fin]))
    return bool(err <= bound), float(err / bound) if bound > 0 else (0.0 if err == 0 else float("inf"))
