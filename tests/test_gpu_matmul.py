"""GPU parity tests of the parallel (matmul) path, through the C ABI, against the CPU oracle.

Tolerances (max |a-b| / max |b|): 1e-4 forward / 3e-4 gradients for fp32 inputs (the reference computes
IEEE fp32 dots; here the CUDA-core path and, at D = 64 and 128, the split tensor-core form), 1e-2 for
16-bit and tf32 tensor-core math (the reference's own check tolerance, utils.py:4).
"""
import numpy as np
import pytest
import torch

from oracle import mlstm_oracle as orc

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-4
TOL_16 = 1e-2


@pytest.fixture(scope="module")
def gc():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tests import gpu_cases
    return gpu_cases


@pytest.mark.parametrize("name", ["matmul_s128_d32_f0.npz", "matmul_s192_d64_f3.npz", "matmul_s768_d32_f1.npz"])
def test_fp32_against_reference_golden(gc, golden_dir, name):
    z = np.load(f"{golden_dir}/{name}")
    x = {k: torch.from_numpy(z[k]) for k in ("q", "k", "v", "f", "i", "dh")}
    h, m, b = gc.run_forward(x)
    assert orc.max_abs_rel(h, torch.from_numpy(z["h"])) < TOL_F32
    ok, frac = orc.check(h, torch.from_numpy(z["h"]))
    assert ok, frac
    grads = gc.run_backward(x, h, m, b)
    for key, g in zip(("dq", "dk", "dv", "df", "di"), grads):
        ref = torch.from_numpy(z[key]).clone()
        if key == "df":
            ref[..., 0] = 0.0
            assert float(g[..., 0].abs().max()) == 0.0
        assert orc.max_abs_rel(g, ref) < 2e-4, key


def test_bf16_against_reference_golden_long(gc, golden_dir):
    """S = 1024, D = 128, bf16: the tensor-core forward and backward against the reference's own PyTorch
    forward / backward on the same bf16 values (fixture made by tests/golden/make_golden.py)."""
    from tests.test_oracle import load_long_bf16
    x, ref = load_long_bf16(golden_dir)
    h, m, b = gc.run_forward(x, h_dtype=torch.bfloat16, flags=gc._lib.F_FORCE_TC)
    assert orc.max_abs_rel(h.float(), ref["h"]) < TOL_16
    grads = gc.run_backward(x, h, m, b, flags=gc._lib.F_FORCE_TC)
    for key, g in zip(("dq", "dk", "dv", "df", "di"), grads):
        r = ref[key].clone()
        if key == "df":
            r[..., 0] = 0.0
        assert orc.max_abs_rel(g.float(), r) < TOL_16, key


@pytest.mark.parametrize("B,NH,S,D,f_mean", [
    (1, 4, 2048, 64, 0.0),     # the reference demo / configuration 2
    (2, 3, 200, 40, 3.0),      # ragged S, D not a tile multiple
    (1, 2, 64, 8, -3.0),
    (1, 1, 3, 16, 0.0),        # three steps
])
def test_fp32_simt_forward_backward(gc, B, NH, S, D, f_mean):
    x = gc.make_inputs(B, NH, S, D, torch.float32, f_mean=f_mean, seed=S + D)
    flags = gc._lib.F_FORCE_SIMT
    h, m, b = gc.run_forward(x, flags=flags)
    ef = gc.errors_forward(x, h, m, b)
    assert ef["h"] < TOL_F32 and ef["m"] < 1e-5 and ef["b"] < TOL_F32, ef
    eb = gc.errors_backward(x, gc.run_backward(x, h, m, b, flags=flags), torch.float32)
    assert all(v < 3e-4 for v in eb.values()), eb


@pytest.mark.parametrize("B,NH,S,D,f_mean,scale", [
    (1, 4, 2048, 64, 0.0, 1.0),      # the reference demo / configuration 2, through the default path
    (1, 2, 328, 128, 1.0, 128 ** -0.5),
    (2, 2, 200, 64, 3.0, 1.0),       # ragged S
    (1, 2, 192, 128, -0.5, 1.0),     # strong decay, last 64-position block pure padding
    (1, 1, 1, 64, 0.0, 1.0),         # a single step (forward only, see test_single_step_sequence)
])
def test_fp32_split_tensor_core_forward_backward(gc, B, NH, S, D, f_mean, scale):
    """fp32 inputs at D = 64 / 128 take the tensor cores by default with operands split into two bf16 halves
    (three products per fp32 product): the fp32 tolerances apply, and the elementwise comparator must pass."""
    x = gc.make_inputs(B, NH, S, D, torch.float32, f_mean=f_mean, qkv_scale=scale, seed=S + D)
    assert gc._lib.lib().mlstm_mm_fwd_workspace(B, NH, S, D, 0, 0) > gc._lib.lib().mlstm_mm_fwd_workspace(B, NH, S, D, 0, 8)
    h, m, b = gc.run_forward(x, flags=gc._lib.F_FORCE_TC)
    ef = gc.errors_forward(x, h, m, b)
    assert ef["h"] < TOL_F32 and ef["m"] < 1e-5 and ef["b"] < TOL_F32, ef
    assert ef["h_check_frac"] == 0.0, ef
    if S > 1:
        eb = gc.errors_backward(x, gc.run_backward(x, h, m, b, flags=gc._lib.F_FORCE_TC), torch.float32)
        assert all(v < 3e-4 for k, v in eb.items() if k != "check_frac"), eb
        assert eb["check_frac"] == 0.0, eb


def test_single_step_sequence(gc):
    """S = 1.  Forward must match; the backward of a lone step is a difference of two terms that agree
    to about 1e-6 relative (dC/n + db = dC/n * (1 - |b|/n)), so only its structure is checked."""
    x = gc.make_inputs(1, 1, 1, 16, torch.float32, seed=17)
    h, m, b = gc.run_forward(x)
    ef = gc.errors_forward(x, h, m, b)
    assert ef["h"] < TOL_F32 and ef["b"] < TOL_F32, ef
    dq, dk, dv, df, di = gc.run_backward(x, h, m, b)
    assert all(bool(torch.isfinite(t).all()) for t in (dq, dk, dv, df, di))
    assert float(df.abs().max()) == 0.0
    assert orc.max_abs_rel(dv, gc.oracle_backward(x, torch.float32)[2]) < TOL_F32


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D", [64, 128, 256])
@pytest.mark.parametrize("S,f_mean", [(128, 0.0), (512, 3.0), (328, 0.0)])
def test_tensor_core_forward_backward(gc, dtype, D, S, f_mean):
    x = gc.make_inputs(1, 3, S, D, dtype, f_mean=f_mean, qkv_scale=D ** -0.5, seed=D + S)
    flags = gc._lib.F_FORCE_TC
    for h_dtype in (torch.float32, dtype):
        h, m, b = gc.run_forward(x, h_dtype=h_dtype, flags=flags)
        ef = gc.errors_forward(x, h, m, b)
        assert ef["h"] < TOL_16 and ef["m"] < 1e-5 and ef["b"] < TOL_16, (h_dtype, ef)
        assert ef["h_check_frac"] < gc.CHECK_FRAC_16 and ef["h_first_tile_row_rel"] < gc.ROW_REL_16, (h_dtype, ef)
        eb = gc.errors_backward(x, gc.run_backward(x, h, m, b, flags=flags), h_dtype)
        assert all(v < TOL_16 for v in eb.values()), (h_dtype, eb)


@pytest.mark.parametrize("dtype,D,S", [(torch.float16, 64, 192), (torch.bfloat16, 128, 192), (torch.float16, 256, 320),
                                       (torch.bfloat16, 256, 448)])
def test_strong_decay_with_a_fully_padded_column_block(gc, dtype, D, S):
    """Ragged S whose last 128-row tile ends in a 64-position block of pure padding, with forget gates around
    sigmoid(-0.5): the row term of the exponent alone reaches 2^140 for late keys, and the padded block has no
    reference to balance it.  Its columns weigh 0; the product must be 0, not NaN (regression)."""
    x = gc.make_inputs(1, 2, S, D, dtype, f_mean=-0.5, qkv_scale=D ** -0.5, seed=S + D)
    flags = gc._lib.F_FORCE_TC
    h, m, b = gc.run_forward(x, h_dtype=dtype, flags=flags)
    ef = gc.errors_forward(x, h, m, b)
    assert ef["h"] < TOL_16 and ef["b"] < TOL_16, ef
    assert ef["h_check_frac"] < gc.CHECK_FRAC_16 and ef["h_first_tile_row_rel"] < gc.ROW_REL_16, ef
    grads = gc.run_backward(x, h, m, b, flags=flags)
    assert all(bool(torch.isfinite(t.float()).all()) for t in grads)
    eb = gc.errors_backward(x, grads, dtype)
    assert all(v < TOL_16 for v in eb.values()), eb


@pytest.mark.parametrize("D", [64, 128, 256])
def test_tf32_tensor_core_forward_backward(gc, D):
    """fp32 inputs on the tensor cores (tf32 operands, fp32 accumulate), opt-in by flag."""
    x = gc.make_inputs(1, 2, 328, D, torch.float32, f_mean=1.0, qkv_scale=D ** -0.5, seed=D)
    flags = gc._lib.F_FORCE_TC | gc._lib.F_ALLOW_TF32
    h, m, b = gc.run_forward(x, flags=flags)
    ef = gc.errors_forward(x, h, m, b)
    # tf32 keeps 10 mantissa bits of every operand: about 1e-3 on h, 1e-3 .. 5e-3 on gradients (measured)
    assert ef["h"] < 3e-3 and ef["m"] < 1e-5 and ef["b"] < 3e-3, ef
    eb = gc.errors_backward(x, gc.run_backward(x, h, m, b, flags=flags), torch.float32)
    assert all(v < TOL_16 for v in eb.values()), eb


@pytest.mark.parametrize("dtype,D,S,f_mean", [
    (torch.bfloat16, 512, 400, 2.0),      # ragged: three full row tiles and a bit
    (torch.float16, 768, 128, 0.0),
    (torch.float32, 512, 300, 1.0),       # tf32 operands (by flag); an odd number of row tiles
    (torch.bfloat16, 512, 1300, 3.0),     # eleven row tiles
])
def test_head_dimensions_above_256_take_the_two_pass_form(gc, dtype, D, S, f_mean):
    """The parallel forward (float32 h) and backward at D = 512, 768: gated S x S matrices to scratch, then plain
    contractions, on the tensor cores; h, m, b and the five gradients against the oracle.  The workspace query
    says which form a call gets: the two-pass one needs room for the gated matrices."""
    x = gc.make_inputs(1, 2, S, D, dtype, f_mean=f_mean, qkv_scale=D ** -0.5, seed=D + S)
    flags = gc._lib.F_ALLOW_TF32 if dtype == torch.float32 else 0
    L = gc._lib.lib()
    dt = gc._lib.dtype_code(x["q"])
    Spad = (S + 127) // 128 * 128
    es = 4 if dtype == torch.float32 else 2
    assert L.mlstm_mm_fwd_workspace(1, 2, S, D, dt, flags) >= 2 * Spad * Spad * es
    assert L.mlstm_mm_fwd_workspace(1, 2, S, D, dt, flags | gc._lib.F_FORCE_SIMT) < Spad * Spad * es
    h, m, b = gc.run_forward(x, flags=flags)
    ef = gc.errors_forward(x, h, m, b)
    tol = 3e-3 if dtype == torch.float32 else TOL_16
    assert ef["h"] < tol and ef["m"] < 1e-5 and ef["b"] < tol, ef
    assert ef["h_check_frac"] < gc.CHECK_FRAC_16 and ef["h_first_tile_row_rel"] < gc.ROW_REL_16, ef
    # the same call on the CUDA cores agrees
    h2, m2, b2 = gc.run_forward(x, flags=gc._lib.F_FORCE_SIMT)
    assert orc.max_abs_rel(h, h2) < tol and orc.max_abs_rel(b, b2) < tol and torch.equal(m, m2)
    assert L.mlstm_mm_bwd_workspace(1, 2, S, D, dt, gc._lib.dtype_code(h), flags) >= 4 * Spad * Spad * es
    grads = gc.run_backward(x, h, m, b, flags=flags)
    eb = gc.errors_backward(x, grads, torch.float32)
    assert all(v < TOL_16 for v in eb.values()), eb
    # the CUDA-core backward of the same call agrees
    grads2 = gc.run_backward(x, h, m, b, flags=gc._lib.F_FORCE_SIMT)
    for name, g1, g2 in zip(("dq", "dk", "dv", "df", "di"), grads, grads2):
        assert orc.max_abs_rel(g1, g2) < TOL_16, name


def test_two_pass_form_in_slice_groups(gc):
    """Nine slices at S = 4096, D = 512: the backward keeps two gated matrices per slice (64 MB here), so it runs in
    two groups of slices (eight, then one) through the same scratch, the forward in one.  Slices of both groups agree
    with the same slice computed alone."""
    B, NH, S, D = 1, 9, 4096, 512
    x = gc.make_inputs(B, NH, S, D, torch.bfloat16, f_mean=3.0, qkv_scale=D ** -0.5, seed=99)
    L = gc._lib.lib()
    dt = gc._lib.dtype_code(x["q"])
    assert L.mlstm_mm_bwd_workspace(B, NH, S, D, dt, 0, 0) < 700 << 20     # two matrices of eight slices, not of nine
    h, m, b = gc.run_forward(x)
    grads = gc.run_backward(x, h, m, b)
    for hd in (0, 7, 8):
        one = {n: t[:, hd:hd + 1].contiguous() for n, t in x.items()}
        h1, m1, b1 = gc.run_forward(one)
        assert orc.max_abs_rel(h[:, hd:hd + 1], h1) < 1e-6 and orc.max_abs_rel(b[:, hd:hd + 1], b1) < 1e-6
        for name, g_all, g_one in zip(("dq", "dk", "dv", "df", "di"), grads, gc.run_backward(one, h1, m1, b1)):
            assert orc.max_abs_rel(g_all[:, hd:hd + 1], g_one) < 1e-6, (hd, name)
    # and one slice of the second group against the oracle
    one = {n: t[:, 8:9].contiguous() for n, t in x.items()}
    eb = gc.errors_backward(one, [g[:, 8:9] for g in grads], torch.float32)
    assert all(v < TOL_16 for v in eb.values()), eb


def test_calls_back_to_back_on_one_workspace(gc):
    """Forty forward + backward calls enqueued without a synchronize, alternating two input sets, all through the same
    cached workspace: a call's first kernel clears the status block and the passes are launched programmatically (they
    may start under the tail of the kernel before them), so this is where a missing dependency would show.  The
    results of the last two calls must equal those of the same calls made alone."""
    dev = torch.device("cuda", 0)
    sets = []
    for seed in (1, 2):
        x = gc.make_inputs(2, 3, 384, 128, torch.bfloat16, f_mean=2.0, qkv_scale=128 ** -0.5, seed=seed)
        sets.append({n: t.to(dev) for n, t in x.items()})
    def call(d):
        h, m, b = gc.PKG.mlstm_matmul_forward(d["q"], d["k"], d["v"], d["f"], d["i"])
        return (h, m, b) + tuple(gc.PKG.mlstm_matmul_backward(d["dh"], d["q"], d["k"], d["v"], d["f"], d["i"], h, m, b))
    alone = []
    for d in sets:
        out = call(d)
        torch.cuda.synchronize()
        alone.append([t.clone() for t in out])
    last = [None, None]
    for it in range(40):
        last[it & 1] = call(sets[it & 1])
    torch.cuda.synchronize()
    for k in range(2):
        for a, b in zip(last[k], alone[k]):
            assert torch.equal(a, b)


def test_tensor_core_matches_simt_on_device(gc):
    """Same 16-bit inputs through both kernel families."""
    x = gc.make_inputs(2, 2, 640, 128, torch.bfloat16, f_mean=3.0, qkv_scale=128 ** -0.5, seed=3)
    h1, m1, b1 = gc.run_forward(x, flags=gc._lib.F_FORCE_TC)
    h2, m2, b2 = gc.run_forward(x, flags=gc._lib.F_FORCE_SIMT)
    assert orc.max_abs_rel(h1, h2) < TOL_16
    assert torch.equal(m1, m2)
    g1 = gc.run_backward(x, h2, m2, b2, flags=gc._lib.F_FORCE_TC)
    g2 = gc.run_backward(x, h2, m2, b2, flags=gc._lib.F_FORCE_SIMT)
    for a, b_ in zip(g1, g2):
        assert orc.max_abs_rel(a.float(), b_.float()) < TOL_16


def test_autograd_function_matches_reference_api(gc):
    """Triton_mLSTM.apply(q,k,v,f,i,SB,NUM_WARPS) + h.backward(dh), as the reference demo does."""
    x = gc.make_inputs(1, 2, 256, 64, torch.float32, seed=11)
    dev = torch.device("cuda", 0)
    t = {n: x[n].to(dev).requires_grad_(True) for n in ("q", "k", "v", "f", "i")}
    h = gc.PKG.Triton_mLSTM.apply(t["q"], t["k"], t["v"], t["f"], t["i"], 32, 4)
    assert h.dtype == torch.float32
    h.backward(x["dh"].to(dev))
    ref = gc.oracle_backward(x, torch.float32)
    for n, r in zip(("q", "k", "v", "f", "i"), ref):
        assert t[n].grad.dtype == t[n].dtype
        assert orc.max_abs_rel(t[n].grad, r) < 3e-4, n
    h2 = gc.PKG.mlstm_matmul(*(t[n].detach() for n in ("q", "k", "v", "f", "i")), SB=32, num_warps=4)
    assert torch.equal(h2, h.detach())


@pytest.mark.parametrize("dtype,D", [(torch.float32, 64), (torch.bfloat16, 256)])
def test_autograd_function_with_output_gate(gc, dtype, D):
    """The optional eighth argument o of Triton_mLSTM.apply: h * silu(o), and gradients for all six inputs."""
    x = gc.make_inputs(1, 2, 256, D, dtype, f_mean=1.0, qkv_scale=D ** -0.5, seed=D + 5, with_o=True)
    dev = torch.device("cuda", 0)
    names = ("q", "k", "v", "f", "i", "o")
    t = {n: x[n].to(dev).requires_grad_(True) for n in names}
    h = gc.PKG.Triton_mLSTM.apply(t["q"], t["k"], t["v"], t["f"], t["i"], 32, 4, t["o"])
    assert h.dtype == torch.float32
    h.backward(x["dh"].to(dev))
    # reference: the oracle's forward and closed-form backward around the gate's own derivative
    od = x["o"].double()
    sig = torch.sigmoid(od)
    h_inner = orc.matmul_forward(x["q"], x["k"], x["v"], x["f"], x["i"], dtype=torch.float64)
    dhd = x["dh"].double()
    ref = dict(zip(("q", "k", "v", "f", "i"), orc.matmul_backward(dhd * od * sig, x["q"], x["k"], x["v"], x["f"], x["i"])))
    ref["o"] = dhd * h_inner * sig * (1 + od * (1 - sig))
    tol = 3e-4 if dtype == torch.float32 else TOL_16
    assert orc.max_abs_rel(h.detach(), h_inner * od * sig) < tol
    for n in names:
        assert t[n].grad.dtype == t[n].dtype
        assert orc.max_abs_rel(t[n].grad, ref[n]) < tol, n
    with pytest.raises(ValueError):
        gc.PKG.Triton_mLSTM.apply(t["q"], t["k"], t["v"], t["f"], t["i"], 32, 4, t["o"][..., :8])


@pytest.mark.parametrize("f_mean", [3.0, 0.0])
def test_model_scale_slice_properties(gc, f_mean):
    """Configuration-4 shape per slice (S=4096, D=256, bf16) on a few slices, with retention-biased gates
    (the configuration's own) and with N(0,1) gates: oracle parity on one slice, and slice independence
    (each slice equals the same slice run alone)."""
    x = gc.make_inputs(1, 3, 4096, 256, torch.bfloat16, f_mean=f_mean, qkv_scale=256 ** -0.5, seed=0)
    h, m, b = gc.run_forward(x, h_dtype=torch.bfloat16)
    grads = gc.run_backward(x, h, m, b)
    one = {k: v[:, 1:2].contiguous() for k, v in x.items()}
    h1, m1, b1 = gc.run_forward(one, h_dtype=torch.bfloat16)
    assert torch.equal(h1, h[:, 1:2])
    g1 = gc.run_backward(one, h1, m1, b1)
    for a, b_ in zip(g1, grads):
        assert torch.equal(a, b_[:, 1:2])
    ef = gc.errors_forward(one, h1, m1, b1)
    assert ef["h"] < TOL_16, ef
    assert ef["h_check_frac"] < gc.CHECK_FRAC_16, ef
    eb = gc.errors_backward(one, g1, torch.bfloat16)
    assert all(v < TOL_16 for v in eb.values()), eb


def test_bounded_wait_runs_out_and_the_device_stays_usable(gc):
    """The waits of every kernel are bounded; this makes one run out on purpose, the allowed way: a warp waits
    (limit: two million cycles, about a millisecond) on a barrier that nothing completes, then stores a code in the
    status word.  mlstm_read_status must report MLSTM_E_TIMEOUT with that code, and ordinary work must still pass."""
    import ctypes
    L = gc._lib.lib()
    dev = torch.device("cuda", 0)
    ws = torch.zeros(4096, dtype=torch.uint8, device=dev)
    stream = gc._lib.stream_ptr(dev)
    assert L.mlstm_selftest_wait_timeout(ws.data_ptr(), ws.numel(), 2_000_000, stream) == 0
    code = ctypes.c_int(0)
    assert L.mlstm_read_status(ws.data_ptr(), ctypes.byref(code), stream) == -7   # MLSTM_E_TIMEOUT
    assert code.value == 4000
    assert b"gave up" in L.mlstm_status_string(-7)
    assert L.mlstm_selftest_wait_timeout(ws.data_ptr(), 16, 2_000_000, stream) == -5
    assert L.mlstm_selftest_wait_timeout(ws.data_ptr(), ws.numel(), 0, stream) == -1
    # the context is intact: an ordinary call on the same device passes and reports a clean status
    x = gc.make_inputs(1, 2, 256, 64, torch.bfloat16, f_mean=1.0, qkv_scale=0.125, seed=2)
    h, m, b = gc.run_forward(x, flags=gc._lib.F_FORCE_TC)
    ef = gc.errors_forward(x, h, m, b)
    assert ef["h"] < TOL_16, ef


def test_argument_errors(gc):
    L = gc._lib.lib()
    assert L.mlstm_mm_fwd(None, None, None, None, None, None, None, None, None, 0, 1, 1, 8, 8, 0, 0, 0, None) == -1
    x = gc.make_inputs(1, 1, 64, 12, torch.float32)
    with pytest.raises(gc._lib.MlstmError):
        gc.run_forward(x)  # D not a multiple of 8
    x = gc.make_inputs(1, 1, 64, 32, torch.float32)
    with pytest.raises(gc._lib.MlstmError):
        gc.run_forward(x, flags=gc._lib.F_FORCE_TC)  # fp32 at D = 32 has no tensor-core path
