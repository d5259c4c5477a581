"""mlstm_forward_f16_static: the single-head fp16 forward whose scratch lives inside the library.

Some users of the C++ driver interface cannot give the library a workspace: they call from a
latency-critical loop where cudaMalloc is off limits, run under a fixed memory budget, or only have the
reference launcher's argument list (Q, K, V, F, I, H, S) to work with.  This entry point serves them
from a fixed device array.  The test calls it twice in a row, on different inputs and lengths, so
that the second call runs over the first call's leftovers in the shared array, and compares each
result with the workspace-taking entry point, which runs the same kernels on caller memory.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gc():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tests import gpu_cases
    return gpu_cases


def _inputs(S, D, seed, dev):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: (torch.rand(*s, generator=g) * 2 - 1).half().to(dev)  # the driver's U[-1, 1) recipe
    return mk(S, D), mk(S, D), mk(S, D), mk(S), mk(S)


def _with_workspace(gc, Q, K, V, F, I):
    L, dev = gc._lib.lib(), Q.device
    S, D = Q.shape
    H = torch.empty_like(Q)
    ws = gc._lib.workspace(L.mlstm_forward_f16_workspace(S, D), dev)
    rc = L.mlstm_forward_f16(Q.data_ptr(), K.data_ptr(), V.data_ptr(), F.data_ptr(), I.data_ptr(), H.data_ptr(), S, D,
                             ws.data_ptr(), ws.numel(), gc._lib.stream_ptr(dev))
    assert rc == 0
    gc._lib.read_status(ws, dev, "mlstm_forward_f16")
    return H


def _static(gc, Q, K, V, F, I):
    L, dev = gc._lib.lib(), Q.device
    S, D = Q.shape
    H = torch.full_like(Q, float("nan"))
    rc = L.mlstm_forward_f16_static(Q.data_ptr(), K.data_ptr(), V.data_ptr(), F.data_ptr(), I.data_ptr(), H.data_ptr(),
                                    S, D, gc._lib.stream_ptr(dev))
    assert rc == 0, L.mlstm_status_string(rc)
    torch.cuda.synchronize()
    return H


def test_static_scratch_forward_matches_workspace_forward_twice(gc):
    dev = torch.device("cuda", 0)
    # a longer call first, then a shorter, ragged one over its leftovers
    for S, D, seed in ((640, 128, 100), (200, 128, 101)):
        args = _inputs(S, D, seed, dev)
        want = _with_workspace(gc, *args)
        got = _static(gc, *args)
        assert bool(torch.isfinite(got).all())
        # the reference driver's own comparator: no element further than 0.01 away
        assert float((got.float() - want.float()).abs().max()) <= 0.01
        assert torch.equal(got, want)  # same kernels, same inputs: in fact identical


def test_static_scratch_matches_reference_golden(gc, golden_dir):
    """The reference driver's own inputs (srand(100) recipe) against the output of the reference's host
    forward, with the reference's comparator (no element further than 0.01 away)."""
    import numpy as np
    z = np.load(f"{golden_dir}/cpp_forward_seed100_s640_d128.npz")
    dev = torch.device("cuda", 0)
    args = [torch.from_numpy(z[k]).to(dev) for k in ("Q", "K", "V", "F", "I")]
    got = _static(gc, *args)
    diff = (got.float().cpu() - torch.from_numpy(z["H"]).float()).abs()
    assert int((diff > 0.01).sum()) == 0, float(diff.max())
    code = ctypes.c_int(-1)
    assert gc._lib.lib().mlstm_forward_f16_static_status(ctypes.byref(code), gc._lib.stream_ptr(dev)) == 0
    assert code.value == 0


def test_static_scratch_at_its_length_limit(gc):
    """S = MLSTM_STATIC_MAX_S must be served (the array is sized from the forward's real scratch layout);
    checked against the workspace entry on all rows and against the CPU oracle on a causal prefix."""
    from oracle import mlstm_oracle as orc
    dev = torch.device("cuda", 0)
    S, D = 16384, 128
    args = _inputs(S, D, 7, dev)
    got = _static(gc, *args)
    want = _with_workspace(gc, *args)
    assert torch.equal(got, want)
    P = 1024   # h[:P] depends on positions < P only
    ref = orc.mlstm_cpu_f16(*(a[:P].cpu() for a in args))
    diff = (got[:P].float().cpu() - ref.float()).abs()
    assert int((diff > 0.01).sum()) == 0, float(diff.max())
    code = ctypes.c_int(-1)
    assert gc._lib.lib().mlstm_forward_f16_static_status(ctypes.byref(code), gc._lib.stream_ptr(dev)) == 0
    assert code.value == 0


def test_static_scratch_rejects_long_sequences(gc):
    L = gc._lib.lib()
    dev = torch.device("cuda", 0)
    x = torch.zeros(16, dtype=torch.float16, device=dev)
    p = x.data_ptr()
    rc = L.mlstm_forward_f16_static(p, p, p, p, p, p, 16384 + 1, 128, None)
    assert rc == -8
    assert b"16384" in L.mlstm_status_string(rc)
