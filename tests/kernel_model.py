"""Torch model of the decomposition the CUDA kernels use (host-side check of the algebra).

The kernels never build the S x S decay matrix from a running maximum.  They use
  a_t = i_t - F_t,  A_t = max_{s<=t} a_s,  m_t = F_t + A_t,  exp(d_tilde_rc - m_r) = exp(a_c - A_r)
and, in the backward, the row identities
  sum_c C~_rc dC_rc = n_r (dh_r . h_r),   dI_c = k_c . dK_c,   R_r = q_r . dQ_r.
This file evaluates exactly those formulas with dense torch ops so that the CPU tests can compare
them with the oracle; ``round_w`` rounds the gated tile to a 16-bit type before the second
contraction, as the tensor-core path does.
"""
import math

import torch
import torch.nn.functional as F


def gates(f, i):
    Fc = torch.cumsum(F.logsigmoid(f.double()), -1)
    a = i.double() - Fc
    A = torch.cummax(a, -1)[0]
    return Fc, a, A, Fc + A


def forward(q, k, v, f, i, round_w=None):
    dt = torch.float64
    q, k, v = q.to(dt), k.to(dt), v.to(dt)
    S, D = q.shape[-2:]
    _, a, A, m = gates(f, i)
    mask = torch.tril(torch.ones(S, S, dtype=torch.bool))
    e = torch.where(mask, torch.exp(a[..., None, :] - A[..., :, None]), torch.zeros((), dtype=dt))
    w = (q @ k.transpose(-1, -2)) / math.sqrt(D) * e
    b = w.sum(-1)
    if round_w is not None:
        w = w.to(round_w).to(dt)
    n = torch.maximum(b.abs(), torch.exp(-m)) + 1e-6
    return (w @ v) / n[..., None], m, b, n


def backward(dh, q, k, v, f, i, h, m, b, round_w=None):
    dt = torch.float64
    dh, q, k, v, h, m, b = (t.to(dt) for t in (dh, q, k, v, h, m, b))
    S, D = q.shape[-2:]
    sc = 1.0 / math.sqrt(D)
    _, a, A, _ = gates(f, i)
    mask = torch.tril(torch.ones(S, S, dtype=torch.bool))
    e = torch.where(mask, torch.exp(a[..., None, :] - A[..., :, None]), torch.zeros((), dtype=dt))
    n = torch.maximum(b.abs(), torch.exp(-m)) + 1e-6
    delta = (dh * h).sum(-1)
    db = torch.sign(b) * (-delta / n) * (b.abs() > torch.exp(-m)).to(dt)
    g = db * n
    rnd = (lambda x: x.to(round_w).to(dt)) if round_w is not None else (lambda x: x)
    dC = dh @ v.transpose(-1, -2)
    wq = rnd((dC + g[..., :, None]) * e * (sc / n)[..., :, None])      # dQ / dK tile
    wv = rnd((q @ k.transpose(-1, -2)) * e * (sc / n)[..., :, None])   # dV tile
    dQ = wq @ k
    dK = wq.transpose(-1, -2) @ q
    dV = wv.transpose(-1, -2) @ dh
    dI = (k * dK).sum(-1)
    R = (q * dQ).sum(-1)
    G = torch.cumsum(dI - R, -1)
    dF = torch.zeros_like(G)
    dF[..., 1:] = torch.sigmoid(-f.double()[..., 1:]) * G[..., :-1]
    R_identity = delta + db * b
    return dQ, dK, dV, dF, dI, R, R_identity
