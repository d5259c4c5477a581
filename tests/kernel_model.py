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


class ChunkSegmentModel:
    """Dense fp64 model of the chunkwise segment stages (same interface as the library's
    ChunkSegment: gate_summary / prepare / local_state / apply and sp_local / sp_apply), used to test
    the sequence-parallel protocol on CPU.  State convention as in the library: S[key, value] = sum_j exp(a_j - A_ref) k_j v_j^T,
    z[key] = sum_j exp(a_j - A_ref) k_j, with a = i - F in global terms and A its prefix maximum."""

    def __init__(self, q, k, v, f, i, chunk_size=256):
        self.q, self.k, self.v = (t.double().flatten(0, 1) for t in (q, k, v))   # [BH, S, D]
        self.f, self.i = f.double().flatten(0, 1), i.double().flatten(0, 1)      # [BH, S]
        self.shape = q.shape
        self.chunk = chunk_size

    def _gates(self, F_in, A_in):
        Fc = torch.cumsum(F.logsigmoid(self.f), -1) + F_in[:, None]
        a = self.i - Fc
        A = torch.maximum(torch.cummax(a, -1)[0], A_in[:, None])
        return Fc, a, A

    def gate_summary(self):
        BH = self.f.shape[0]
        Fc, a, A = self._gates(torch.zeros(BH, dtype=torch.float64), torch.full((BH,), -float("inf"), dtype=torch.float64))
        return torch.stack([Fc[:, -1], A[:, -1]], 1)

    def prepare(self, carry_in=None):
        BH = self.f.shape[0]
        if carry_in is None:
            carry_in = torch.stack([torch.zeros(BH, dtype=torch.float64),
                                    torch.full((BH,), -float("inf"), dtype=torch.float64)], 1)
        self.A_in = carry_in[:, 1].double()
        self.Fc, self.a, self.A = self._gates(carry_in[:, 0].double(), self.A_in)
        return torch.stack([self.Fc[:, -1], self.A[:, -1]], 1)

    def local_state(self):
        w = torch.exp(self.a - self.A[:, -1:])                                   # [BH, S]
        S = torch.einsum("bs,bsk,bsv->bkv", w, self.k, self.v)
        z = torch.einsum("bs,bsk->bk", w, self.k)
        return S.float(), z.float()

    def apply(self, state_in=None, h_dtype=torch.float32, return_state=False):
        B, NH, S, D = self.shape
        mask = torch.tril(torch.ones(S, S, dtype=torch.bool))
        e = torch.where(mask, torch.exp(self.a[:, None, :] - self.A[:, :, None]), torch.zeros((), dtype=torch.float64))
        w = (self.q @ self.k.transpose(-1, -2)) / math.sqrt(D) * e
        num = w @ self.v
        b = w.sum(-1)
        if state_in is not None:
            s_w = torch.exp(self.A_in[:, None] - self.A) / math.sqrt(D)          # [BH, S]
            num = num + s_w[..., None] * (self.q @ state_in[0].double())
            b = b + s_w * (self.q @ state_in[1].double()[..., None])[..., 0]
        m = self.Fc + self.A
        n = torch.maximum(b.abs(), torch.exp(-m)) + 1e-6
        return (num / n[..., None]).reshape(B, NH, S, D).to(h_dtype)

    # ---- the two stages of the one-exchange sequence-parallel protocol
    def sp_local(self):
        """Record per slice: S | z | {F_end, A_end} with no carry (the segment's own coordinates)."""
        summary = self.prepare(None)                                             # [BH, 2] float64
        S, z = self.local_state()
        BH, D = z.shape
        tail = summary.contiguous().view(torch.float32).reshape(BH, 4)
        return torch.cat([S.reshape(BH, D * D), z, tail], 1)

    def sp_apply(self, gathered, rank, h_dtype=torch.float32):
        import importlib
        mc = importlib.import_module("xlstm-triton-cuda-implementation_b200.mlstm_chunkwise")
        S_in, z_in, F_in, A_in = mc.fold_records(gathered, rank)
        self.prepare(torch.stack([F_in, A_in], 1))                               # gates again, now with the carry
        return self.apply((S_in, z_in) if rank > 0 else None, h_dtype=h_dtype)
