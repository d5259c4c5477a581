"""CPU tests: the oracle against the reference's golden vectors, and the kernel algebra."""
import ctypes
import os
import sys

import numpy as np
import pytest
import torch

from oracle import mlstm_oracle as orc
from tests import kernel_model as km

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
T = torch.from_numpy


def _load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name))
    return {k: T(z[k]) for k in z.files}


@pytest.mark.parametrize("name", ["matmul_s128_d32_f0.npz", "matmul_s192_d64_f3.npz", "matmul_s768_d32_f1.npz"])
def test_matmul_oracle_vs_reference_golden(golden_dir, name):
    z = _load(golden_dir, name)
    # the goldens are the reference's fp32 evaluation; its own rounding grows with S (about 3e-5 at S = 768)
    long_case = z["q"].shape[-2] > 256
    h = orc.matmul_forward(z["q"], z["k"], z["v"], z["f"], z["i"])
    assert orc.max_abs_rel(h, z["h"]) < (1e-4 if long_case else 2e-5)
    got = orc.matmul_backward(z["dh"], z["q"], z["k"], z["v"], z["f"], z["i"])
    for key, g in zip(("dq", "dk", "dv", "df", "di"), got):
        ref = z[key].clone()
        if key == "df":
            ref[..., 0] = 0.0  # the reference oracle wraps the (zero) total into slot 0
        assert orc.max_abs_rel(g, ref) < (2e-4 if long_case else 5e-5), key
    # fp32 evaluation of the oracle must also sit inside the reference's own tolerance
    ok, frac = orc.check(orc.matmul_forward(z["q"], z["k"], z["v"], z["f"], z["i"], dtype=torch.float32), z["h"])
    assert ok, frac


@pytest.mark.parametrize("name", ["scan_s96_d16_f0.npz", "scan_s64_d32_f3.npz", "scan_s512_d32_f1.npz"])
def test_scan_oracle_vs_reference_golden(golden_dir, name):
    z = _load(golden_dir, name)
    h = orc.scan_forward(z["q"], z["k"], z["v"], z["f"], z["i"], z["o"])
    assert orc.max_abs_rel(h, z["h"]) < (1e-4 if z["q"].shape[-2] > 256 else 2e-5)
    # recurrent form == parallel form times silu(o)
    hp = orc.matmul_forward(z["q"], z["k"], z["v"], z["f"], z["i"]) * torch.nn.functional.silu(z["o"].double())
    assert orc.max_abs_rel(h, hp) < 1e-5


def load_long_bf16(golden_dir, name="long_bf16_s1024_d128_f3.npz"):
    """The long 16-bit fixture: bf16 inputs (stored as bit patterns), reference outputs in fp16 / fp32."""
    z = np.load(os.path.join(golden_dir, name))
    x = {k: T(z[k].copy()).view(torch.bfloat16) for k in ("q", "k", "v", "f", "i", "dh")}
    ref = {k: T(z[k]).float() for k in ("h", "dq", "dk", "dv", "df", "di")}
    return x, ref


def test_oracle_vs_reference_golden_long_bf16(golden_dir):
    """S = 1024, D = 128 on bf16 values: the port against the reference's own forward and backward
    (stored in fp16, hence the 2e-3)."""
    x, ref = load_long_bf16(golden_dir)
    h = orc.matmul_forward(x["q"], x["k"], x["v"], x["f"], x["i"])
    assert orc.max_abs_rel(h, ref["h"]) < 2e-3
    grads = orc.matmul_backward(x["dh"], x["q"], x["k"], x["v"], x["f"], x["i"])
    for key, g in zip(("dq", "dk", "dv", "df", "di"), grads):
        r = ref[key].clone()
        if key == "df":
            r[..., 0] = 0.0
        assert orc.max_abs_rel(g, r) < 2e-3, key


def test_scan_oracle_segment_carry(golden_dir):
    z = _load(golden_dir, "scan_s96_d16_f0.npz")
    args = [z[k] for k in ("q", "k", "v", "f", "i", "o")]
    full = orc.scan_forward(*args)
    cut = 40
    first = [a[..., :cut, :] if a.dim() == 4 else a[..., :cut] for a in args]
    second = [a[..., cut:, :] if a.dim() == 4 else a[..., cut:] for a in args]
    h1, st = orc.scan_forward(*first, return_state=True)
    h2 = orc.scan_forward(*second, initial=st)
    assert orc.max_abs_rel(torch.cat([h1, h2], -2), full) < 1e-12


@pytest.mark.parametrize("name", ["cpp_forward_seed100_s640_d128.npz", "cpp_forward_seed100_s128_d128.npz"])
def test_cpp_oracle_vs_reference_golden(golden_dir, name):
    z = _load(golden_dir, name)
    h = orc.mlstm_cpu_f16(z["Q"], z["K"], z["V"], z["F"], z["I"])
    # the reference's own comparator for this path: |a - b| <= 0.01 on every element
    assert float((h.float() - z["H"].float()).abs().max()) <= 2e-3


def test_backward_oracle_vs_reference_golden_cpp_recipe(golden_dir):
    """The oracle's backward against the reference's PyTorch backward on the backward driver's input recipe
    (single head, fp16 values, srand(1678))."""
    z = _load(golden_dir, "cpp_backward_seed1678_s192_d128.npz")
    t = lambda k: z[k].float()[None, None]
    grads = orc.matmul_backward(t("dH"), t("Q"), t("K"), t("V"), t("F"), t("I"))
    for name, got in zip(("dQ", "dK", "dV", "dF", "dI"), grads):
        assert orc.max_abs_rel(got[0, 0], z[name].double()) < 1e-5, name


def _c_oracle():
    path = os.path.join(ROOT, "oracle", "libmlstm_oracle.so")
    if not os.path.exists(path):
        pytest.skip("oracle/libmlstm_oracle.so not built (python -c 'import __graft_entry__ as g; g.build()')")
    return ctypes.CDLL(path)


def test_c_restatement_vs_reference_golden(golden_dir):
    lib = _c_oracle()
    z = _load(golden_dir, "cpp_forward_seed100_s640_d128.npz")
    S, D = z["Q"].shape
    arrs = [np.ascontiguousarray(z[k].float().numpy()) for k in ("Q", "K", "V", "F", "I")]
    H = np.zeros((S, D), dtype=np.float32)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    rc = lib.mlstm_cpu_forward(*[p(a) for a in arrs], p(H), ctypes.c_uint(S), ctypes.c_uint(D), ctypes.c_int(1))
    assert rc == 0
    assert np.abs(H.astype(np.float16).astype(np.float32) - z["H"].float().numpy()).max() <= 2e-3


def test_c_restatement_vs_compiled_reference():
    """When the reference's own mlstmCpu has been compiled (oracle/_ref), compare directly."""
    ref_path = os.path.join(ROOT, "oracle", "_ref", "libmlstm_ref.so")
    if not os.path.exists(ref_path):
        pytest.skip("oracle/_ref not built")
    lib, ref = _c_oracle(), ctypes.CDLL(ref_path)
    S, D = 192, 64
    mk = lambda n: np.zeros(n, dtype=np.float16)
    Q, K, V, F, I, Href = mk(S * D), mk(S * D), mk(S * D), mk(S), mk(S), mk(S * D)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    ref.ref_fill(ctypes.c_uint(7), p(Q), p(K), p(V), p(F), p(I), ctypes.c_uint(S), ctypes.c_uint(D))
    ref.ref_mlstm_cpu(p(Q), p(K), p(V), p(F), p(I), p(Href), ctypes.c_uint(S), ctypes.c_uint(D))
    f32 = [a.astype(np.float32) for a in (Q, K, V, F, I)]
    H = np.zeros(S * D, dtype=np.float32)
    assert lib.mlstm_cpu_forward(*[p(a) for a in f32], p(H), ctypes.c_uint(S), ctypes.c_uint(D), ctypes.c_int(1)) == 0
    assert np.abs(H.astype(np.float16).astype(np.float32) - Href.astype(np.float32)).max() <= 2e-3


@pytest.mark.parametrize("f_mean", [0.0, 3.0, -3.0])
def test_kernel_algebra_matches_oracle(f_mean):
    g = torch.Generator().manual_seed(5)
    B, NH, S, D = 1, 2, 160, 32
    q, k, v, dh = (torch.randn(B, NH, S, D, generator=g) for _ in range(4))
    f = f_mean + torch.randn(B, NH, S, generator=g)
    i = torch.randn(B, NH, S, generator=g)
    h_ref, m_ref, b_ref, _ = orc.matmul_forward(q, k, v, f, i, return_state=True)
    h, m, b, n = km.forward(q, k, v, f, i)
    assert orc.max_abs_rel(h, h_ref) < 1e-10
    assert orc.max_abs_rel(m, m_ref) < 1e-10
    assert orc.max_abs_rel(b, b_ref) < 1e-9
    ref = orc.matmul_backward(dh, q, k, v, f, i)
    dQ, dK, dV, dF, dI, R, R_id = km.backward(dh, q, k, v, f, i, h, m, b)
    for got, want, name in zip((dQ, dK, dV, dF, dI), ref, "qkvfi"):
        assert orc.max_abs_rel(got, want) < 1e-8, name
    assert orc.max_abs_rel(R, R_id) < 1e-8


def test_kernel_algebra_with_bf16_tiles_is_inside_tolerance():
    """Rounding the gated tile to bf16 (what the tensor-core path does) stays within 1e-2."""
    g = torch.Generator().manual_seed(6)
    B, NH, S, D = 1, 1, 512, 64
    q, k, v = ((torch.randn(B, NH, S, D, generator=g) / 8).bfloat16() for _ in range(3))
    dh = torch.randn(B, NH, S, D, generator=g).bfloat16()
    f = (3.0 + torch.randn(B, NH, S, generator=g)).bfloat16()
    i = torch.randn(B, NH, S, generator=g).bfloat16()
    ref = orc.matmul_backward(dh, q, k, v, f, i)
    h, m, b, n = km.forward(q, k, v, f, i, round_w=torch.bfloat16)
    assert orc.max_abs_rel(h, orc.matmul_forward(q, k, v, f, i)) < 1e-2
    out = km.backward(dh, q, k, v, f, i, h, m, b, round_w=torch.bfloat16)
    for got, want, name in zip(out[:5], ref, "qkvfi"):
        assert orc.max_abs_rel(got, want) < 1e-2, name
