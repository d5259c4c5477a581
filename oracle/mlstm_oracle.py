"""CPU oracle for the mLSTM hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, with plain torch CPU tensor arithmetic, the algorithms of the
reference project's own CPU-capable mLSTM implementations.  It exists so that the CUDA
kernels can be checked; nothing in the shipped package may import it.  Only the tests,
the smoke entry and the benchmark's CPU-baseline leg use it.

Parity pin: every function below is checked against the reference's own functions
(imported from the reference checkout when it is present) and against the committed
golden vectors in ``tests/golden`` that were produced by those reference functions
(``tests/golden/make_golden.py``).

Reference locations restated here (paths inside the reference project):
  * parallel forward            mlstm_matmul.py:104-118  (``mlstm_matmul_pytorch``)
  * closed-form backward        mlstm_matmul.py:336-365  (``mlstm_matmul_backward_pytorch``)
  * recurrent scan forward      mlstm_scan.py:343-372    (``mlstm_scan_pytorch``)
  * pair algebra of the scan    mlstm_scan.py:15-26, 330-340
  * host C++ forward            cuda-src/cpu_utils.cuh:126-170 (``mlstmCpu``; the epsilon sits
                                inside the max there, see ``eps_inside_max``)
  * comparator                  utils.py:4-15 (``check``; atol = rtol = 1e-2)
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

REF_ATOL = 1e-2  # utils.py:4
REF_RTOL = 1e-2  # utils.py:4
EPS = 1e-6       # mlstm_matmul.py:95, 116; mlstm_scan.py:343


def _decay(f: torch.Tensor, i: torch.Tensor):
    """Return (d_tilde, m, d_prime) of the parallel form.

    mlstm_matmul.py:106-113.  d_tilde[.., r, c] = F_r - F_c + i_c for c <= r and -inf above
    the diagonal, with F the inclusive cumulative sum of logsigmoid(f); m is the row maximum;
    d_prime = exp(d_tilde - m).
    """
    S = f.shape[-1]
    fc = torch.cumsum(F.logsigmoid(f), -1)
    mask = torch.tril(torch.ones((S, S), dtype=torch.bool, device=f.device))
    d_tilde = fc[..., :, None] - fc[..., None, :]
    d_tilde = torch.where(mask, d_tilde, torch.full_like(d_tilde, -float("inf")))
    d_tilde = d_tilde + i[..., None, :]
    m = torch.max(d_tilde, -1)[0]
    d_prime = torch.exp(d_tilde - m[..., None])
    return d_tilde, m, d_prime


def matmul_forward(q, k, v, f, i, *, dtype=torch.float64, eps_inside_max=False, return_state=False):
    """Parallel (quadratic) mLSTM forward.  mlstm_matmul.py:104-118.

    q, k, v: [..., S, D]; f, i: [..., S].  Inputs are converted to ``dtype`` first, so a bf16
    or fp16 input is evaluated on its rounded values with wide accumulation.
    ``eps_inside_max`` selects the host C++ variant n = max(|b|, exp(-m) + eps)
    (cuda-src/cpu_utils.cuh:157) instead of n = max(|b|, exp(-m)) + eps.
    """
    q, k, v, f, i = (t.to(dtype) for t in (q, k, v, f, i))
    D = q.shape[-1]
    _, m, d_prime = _decay(f, i)
    c = (q @ (k.transpose(-2, -1) / math.sqrt(D))) * d_prime
    b = torch.sum(c, -1)
    if eps_inside_max:
        n = torch.maximum(torch.abs(b), torch.exp(-m) + EPS)
    else:
        n = torch.maximum(torch.abs(b), torch.exp(-m)) + EPS
    h = (c / n[..., None]) @ v
    if return_state:
        return h, m, b, n
    return h


def matmul_backward(dh, q, k, v, f, i, *, dtype=torch.float64):
    """Closed-form backward of the parallel form.  mlstm_matmul.py:336-365.

    Returns (dq, dk, dv, df, di).  The reference rolls the cumulative sum, so its df[..., 0]
    holds the (analytically zero) total; the kernels of this library and the reference's own
    GPU kernel (mlstm_matmul.py:316, 392) give exactly 0 there, so this oracle writes 0 too.
    """
    dh, q, k, v, f, i = (t.to(dtype) for t in (dh, q, k, v, f, i))
    D = q.shape[-1]
    _, m, d_prime = _decay(f, i)
    dC = dh @ v.transpose(-2, -1)
    s = q @ (k.transpose(-2, -1) / math.sqrt(D))
    c_tilde = s * d_prime
    b = torch.sum(c_tilde, -1)
    n = torch.maximum(torch.abs(b), torch.exp(-m)) + EPS
    dn = -torch.sum(c_tilde * dC, -1) / (n * n)
    db = torch.sign(b) * dn * (torch.abs(b) > torch.exp(-m)).to(dtype)
    c = c_tilde / n[..., None]
    dc_tilde = dC / n[..., None] + db[..., None]
    dD = s * d_prime * dc_tilde
    dQ = (dc_tilde * d_prime) @ (k / math.sqrt(D))
    dK = (dc_tilde * d_prime).transpose(-2, -1) @ (q / math.sqrt(D))
    dV = c.transpose(-2, -1) @ dh
    dI = torch.sum(dD, -2)
    G = torch.cumsum(dD.sum(-2) - dD.sum(-1), -1)
    dF = torch.zeros_like(f)
    dF[..., 1:] = torch.sigmoid(-f[..., 1:]) * G[..., :-1]
    return dQ, dK, dV, dF, dI


def stabilization_op(a, b):
    """(sum lf, m) o (sum lf', m') = (sum + sum', max(sum' + m, m')).  mlstm_scan.py:22-26, 336-340."""
    return b[0] + a[0], torch.maximum(b[0] + a[1], b[1])


def scan_forward(q, k, v, f, i, o, *, dtype=torch.float64, initial=None, return_state=False):
    """Recurrent mLSTM forward with output gate.  mlstm_scan.py:343-372.

    Same recurrence as the reference (one step per time index, state C[value, key], n, m with
    m_{-1} = 0), vectorised over the leading batch/head axes instead of Python loops over them.
    ``initial`` = (C, n, m) continues from an earlier segment (used for the long-sequence carry).
    """
    q, k, v, f, i, o = (t.to(dtype) for t in (q, k, v, f, i, o))
    lead = q.shape[:-2]
    S, D = q.shape[-2:]
    if initial is None:
        C = torch.zeros(*lead, D, D, dtype=dtype)
        n = torch.zeros(*lead, D, dtype=dtype)
        m = torch.zeros(*lead, dtype=dtype)
    else:
        C, n, m = (t.to(dtype).clone() for t in initial)
    lf = F.logsigmoid(f)
    hs = []
    for t in range(S):
        m_new = torch.maximum(lf[..., t] + m, i[..., t])           # :353-357
        i_st = torch.exp(i[..., t] - m_new)                        # :358
        f_st = torch.exp(lf[..., t] - m_new + m)                   # :359
        k_sc = k[..., t, :] / math.sqrt(D)                         # :360
        m = m_new
        C = f_st[..., None, None] * C + i_st[..., None, None] * (v[..., t, :, None] * k_sc[..., None, :])  # :363-365
        n = f_st[..., None] * n + i_st[..., None] * k_sc           # :364-366
        qt = q[..., t, :]
        normalizer = torch.maximum(torch.abs((n * qt).sum(-1)), torch.exp(-m)) + EPS  # :367-368
        hs.append(F.silu(o[..., t, :]) * (C @ qt[..., None])[..., 0] / normalizer[..., None])  # :369
    h = torch.stack(hs, -2)
    if return_state:
        return h, (C, n, m)
    return h


def mlstm_cpu_f16(q, k, v, f, i):
    """Host C++ forward for one head on fp16 data.  cuda-src/cpu_utils.cuh:126-170.

    fp32 arithmetic on the fp16 values, epsilon inside the max (:157), result rounded to fp16
    (``matmul`` stores into a half array, :69-79).
    """
    h = matmul_forward(q, k, v, f, i, dtype=torch.float32, eps_inside_max=True)
    return h.to(torch.float16)


def check(a: torch.Tensor, b: torch.Tensor, atol=REF_ATOL, rtol=REF_RTOL):
    """The reference comparator (utils.py:4-15) as a predicate plus the mismatch fraction."""
    a = a.detach().cpu().double()
    b = b.detach().cpu().double()
    close = torch.isclose(a, b, atol=atol, rtol=rtol)
    return bool(close.all()), float((~close).double().mean())


def max_abs_rel(a: torch.Tensor, b: torch.Tensor) -> float:
    """max |a - b| / max |b|: the error measure used for the stated tolerances."""
    a = a.detach().cpu().double()
    b = b.detach().cpu().double()
    denom = float(b.abs().max())
    return float((a - b).abs().max()) / (denom if denom > 0 else 1.0)
