"""The allocation-free entry point against the regular session path.

`accy_b200_mismatch_noalloc` exists for hosts that may not allocate device memory while they run
(their own pool owns the device, or they sit in a real-time loop or a fixed stream schedule): it
keeps the partial sums of the two-pass column-split reduction in an array built into the library
instead of a buffer allocated at load time.  This test calls it through the C ABI on buffers the
test owns, twice in a row (the array is shared between calls and keeps the previous call's
contents, so the second call must not be disturbed by the first), and compares each result with
what the session path computes for the same recorded program and with the CPU oracle (the
reference-order f32 fold and the f64 evaluation: two GPU paths could share a mistake, the oracle
shares none), to the f32 tolerance of the other parity tests (1e-5 relative).  The file sorts last so that a run that stops at the first failure
has already run everything else.
"""
import ctypes

import numpy as np
import pytest

from accy_b200 import configs, tensor
from accy_b200._native import lib
from oracle import oracle
from parity_checks import check_three_distances

pytestmark = pytest.mark.gpu


def rel_err(got, want):
    want = want.astype(np.float64)
    got = got.astype(np.float64)
    floor = max(np.abs(want).max() * 1e-6, 1e-30)
    return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), floor)))


def session_result(cfg, inputs, splits):
    session = tensor.Session(device=0, column_splits=splits)
    try:
        compiled = session.compile(cfg.program())
        out = np.empty(inputs[0].shape[0], np.float32)
        session.invoke(compiled, inputs, [out])
        return out
    finally:
        session.deinit()


def test_no_alloc_entry_point_matches_session_path_twice():
    import torch
    torch.cuda.set_device(0)
    error = ctypes.create_string_buffer(256)
    # two different problems back to back: the second must not see the first one's partials
    cases = [configs.mismatch(6, 200000, seed=11), configs.mismatch(3, 70001, seed=12)]
    for cfg in cases:
        inputs = cfg.make_inputs()
        guesses, points = inputs[0].shape[0], inputs[1].shape[0]
        expected = session_result(cfg, inputs, splits=16)
        device = [torch.from_numpy(a).cuda() for a in inputs]
        out = torch.full((guesses,), float("nan"), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        status = lib.accy_b200_mismatch_noalloc(device[0].data_ptr(), device[1].data_ptr(), device[2].data_ptr(),
                                                out.data_ptr(), guesses, points, 16, None, error, 256)
        assert status == 0, error.value
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        assert rel_err(got, expected) < 1e-5
        wire = cfg.program().wire
        check_three_distances("no-alloc mismatch %dx%d" % (guesses, points), got, oracle.run(wire, inputs)[0],
                              oracle.run(wire, inputs, mode="f64")[0], 1e-6)


def test_no_alloc_entry_point_refuses_oversized_calls():
    error = ctypes.create_string_buffer(256)
    status = lib.accy_b200_mismatch_noalloc(256, 256, 256, 256, 1 << 20, 1 << 20, 64, None, error, 256)
    assert status == 4  # invalid_buffer
    assert b"exceeds the built-in scratch" in error.value
