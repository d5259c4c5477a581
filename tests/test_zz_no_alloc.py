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


def test_static_scratch_rejects_long_sequences(gc):
    L = gc._lib.lib()
    dev = torch.device("cuda", 0)
    x = torch.zeros(16, dtype=torch.float16, device=dev)
    p = x.data_ptr()
    rc = L.mlstm_forward_f16_static(p, p, p, p, p, p, 16384 + 1, 128, None)
    assert rc == -8
    assert b"16384" in L.mlstm_status_string(rc)
