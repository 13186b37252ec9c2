"""The allocation-free softmax cross-entropy entry point.

Some users of this library cannot allocate device memory at the moment they
need a loss: a plugin living inside a host process whose own pool already owns
the GPU's memory, a control loop that forbids cudaMalloc after start-up (it can
stall the device and it can fail), or code the caller is recording into a CUDA
graph.  `see_cuda_xent_forward_static` serves them with a scratch array built
into the library.  This test calls it through the C ABI with device pointers
and holds it — on two calls in a row, which share that array — to the result
of the regular entry point (the backend's kSoftmaxXEntFwd instruction), bit
for bit: both run the same kernels, only the scratch's home differs.

Collected last on purpose (the file name sorts after every other test file).
"""

import numpy as np
import pytest

from see_ai_b200 import backend as B
from see_ai_b200 import plan as P

pytestmark = pytest.mark.gpu


def _regular(logits: np.ndarray, labels: np.ndarray, masked: bool):
    """The existing path: one kSoftmaxXEntFwd instruction through the backend."""
    n, c = logits.shape
    off_logits, off_labels = 0, 4 * n * c
    off_loss = off_labels + (4 * n + 63) // 64 * 64
    off_probs = off_loss + 64
    arena = np.zeros(off_probs + 4 * n * c, dtype=np.uint8)
    arena[off_logits:off_logits + 4 * n * c] = logits.view(np.uint8).reshape(-1)
    arena[off_labels:off_labels + 4 * n] = labels.view(np.uint8).reshape(-1)
    op = P.Op.XENT_MASKED_FWD if masked else P.Op.XENT_FWD
    be = B.CudaBackend(0)
    be.bind(arena, None)
    be.run([P.Instr(op, 0, 0, (off_logits, off_labels, off_loss, off_probs), (n, c, 0))])
    be.close()
    loss = arena[off_loss:off_loss + 4].view(np.float32)[0]
    probs = arena[off_probs:off_probs + 4 * n * c].view(np.float32).reshape(n, c).copy()
    return loss, probs


def _static(logits: np.ndarray, labels: np.ndarray, masked: bool):
    import torch
    n, c = logits.shape
    d_logits = torch.from_numpy(logits).cuda()
    d_labels = torch.from_numpy(labels).cuda()
    d_loss = torch.full((1,), -1.0, dtype=torch.float32, device="cuda")
    d_probs = torch.full((n, c), -1.0, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    B.xent_forward_static(d_logits.data_ptr(), d_labels.data_ptr(), d_loss.data_ptr(),
                          d_probs.data_ptr(), n, c, masked,
                          torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return d_loss.cpu().numpy()[0], d_probs.cpu().numpy()


def test_static_entry_matches_regular_entry_on_two_calls_in_a_row():
    rng = np.random.default_rng(42)
    # Two different batches back to back: the second reuses the array the first
    # left dirty (more rows first, fewer second, so stale entries sit behind it).
    # The third is the wide-row kernel (4096..32768 classes: rows held in registers,
    # first launch raises the kernel's shared-memory limit), masked.
    cases = [(777, 130, False), (300, 1029, True), (64, 4096, True)]
    for n, c, masked in cases:
        logits = (rng.standard_normal((n, c)) * 3).astype(np.float32)
        labels = rng.integers(0, c, size=n).astype(np.int32)
        if masked:
            labels[::4] = -1
        want_loss, want_probs = _regular(logits, labels, masked)
        got_loss, got_probs = _static(logits, labels, masked)
        assert np.isfinite(got_loss)
        assert got_loss.tobytes() == want_loss.tobytes(), (got_loss, want_loss)
        assert np.array_equal(got_probs, want_probs)


def test_static_entry_refuses_batches_beyond_its_scratch():
    import torch
    lib = B.load_library()
    limit = int(lib.see_cuda_static_max_rows())
    assert limit == 65536
    dummy = torch.zeros(16, dtype=torch.float32, device="cuda")
    with pytest.raises(B.BackendError) as e:
        B.xent_forward_static(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                              dummy.data_ptr(), limit + 1, 4)
    assert "exceed" in str(e.value) and str(limit) in str(e.value)
