"""Chunkwise mLSTM forward for long sequences, on one GPU or sequence-parallel over several.

    h = mlstm_chunkwise(q, k, v, f, i, chunk_size=256)
    h_local = mlstm_chunkwise_sequence_parallel(q_seg, k_seg, v_seg, f_seg, i_seg, chunk_size=256, group=None)

The reference has no long-sequence entry point of its own; what this extends is the inter-block carry
of its scan path (mlstm_scan.py:143-195) with the carry algebra of its scan operators
(mlstm_scan.py:15-26).  Inputs are 16-bit, D = 128 or 256; h is float32 unless ``h_dtype`` says otherwise.

Sequence-parallel form: rank r of the group holds the r-th contiguous segment of every sequence
(all heads).  ONE all-gather connects the ranks and there is no other communication: every rank first
does all the work that needs no other rank (gates, per-block states, and the state its segment adds,
stabilised by its own prefix maximum with F counted from zero) and packs, per slice, one record
``S [D*D] | z [D] | {F_end, A_end}`` (0.53 MB per rank at 8 heads).  After the all-gather one kernel
folds the lower ranks' records into the inbound state and carry of this rank (``fold_records`` states
the same arithmetic in torch, for the CPU tests), and the output pass applies it.
``fold_gate_summaries`` / ``fold_states`` are the same combine on separate tensors, for callers that
move summaries and states themselves (state continuation across calls).
"""
import torch

from . import _lib

__all__ = ["mlstm_chunkwise", "mlstm_chunkwise_backward", "mlstm_chunkwise_sequence_parallel", "fold_gate_summaries", "fold_states",
           "fold_records", "ChunkSegment"]


class ChunkSegment:
    """One segment's pass through the four C-ABI stages, holding its workspace."""

    def __init__(self, q, k, v, f, i, chunk_size=256, shared_workspace=False, o=None):
        if q.dim() != 4 or k.shape != q.shape or v.shape != q.shape:
            raise ValueError("q, k, v must share the shape [B, NH, S, D]")
        if f.shape != q.shape[:3] or i.shape != q.shape[:3]:
            raise ValueError("f, i must have the shape [B, NH, S]")
        if not (k.dtype == v.dtype == f.dtype == i.dtype == q.dtype):
            raise TypeError("q, k, v, f, i must share one element type")
        self.dev = _lib.require_cuda(q, k, v, f, i)
        if o is not None:
            if o.shape != q.shape or o.dtype != q.dtype:
                raise ValueError("o must match q in shape and element type")
            _lib.require_cuda(q, o)
        self.q, self.k, self.v, self.f, self.i, self.o = q, k, v, f, i, o
        self.B, self.NH, self.S, self.D = q.shape
        self.dt = _lib.dtype_code(q)
        self.chunk = int(chunk_size)
        self.L = _lib.lib()
        nbytes = self.L.mlstm_chunk_workspace(self.B, self.NH, self.S, self.D, self.dt, self.chunk)
        if nbytes == 0:
            raise _lib.MlstmError(-4, "mlstm_chunk_workspace (needs float16/bfloat16, D = 128 or 256, chunk % 128 == 0)")
        # The workspace carries the gates and block states from stage to stage.  A private buffer is safe
        # however segments are interleaved; the per-stream shared one saves a large allocation per call
        # and is what the one-shot functions below use (they finish a segment before starting another).
        self.ws = (_lib.workspace(nbytes, self.dev) if shared_workspace
                   else torch.empty(nbytes, dtype=torch.uint8, device=self.dev))
        self.dims = (self.B, self.NH, self.S, self.D, self.dt, self.chunk)

    def _stream(self):
        return _lib.stream_ptr(self.dev)

    def gate_summary(self):
        """{F_end, A_end} of this segment alone (no carry): float64 [B*NH, 2]."""
        out = torch.empty((self.B * self.NH, 2), dtype=torch.float64, device=self.dev)
        with torch.cuda.device(self.dev):
            rc = self.L.mlstm_chunk_gate_summary(self.f.data_ptr(), self.i.data_ptr(), out.data_ptr(), self.ws.data_ptr(),
                                                 self.ws.numel(), *self.dims, self._stream())
        _lib.check(rc, "mlstm_chunk_gate_summary")
        return out

    def prepare(self, carry_in=None):
        """Gates (with the preceding segments' {F, A}, float64 [B*NH, 2], or None) and block states.
        Returns {F_end, A_end} including the carry."""
        if carry_in is not None:
            carry_in = carry_in.to(device=self.dev, dtype=torch.float64).contiguous()
        out = torch.empty((self.B * self.NH, 2), dtype=torch.float64, device=self.dev)
        with torch.cuda.device(self.dev):
            rc = self.L.mlstm_chunk_prepare(self.k.data_ptr(), self.v.data_ptr(), self.f.data_ptr(), self.i.data_ptr(),
                                            carry_in.data_ptr() if carry_in is not None else None, out.data_ptr(),
                                            self.ws.data_ptr(), self.ws.numel(), *self.dims, self._stream())
        _lib.check(rc, "mlstm_chunk_prepare")
        self._keep = carry_in
        return out

    def local_state(self):
        """The state this segment adds: S [B*NH, D, D] (key, value), z [B*NH, D], stabilised by A_end."""
        S = torch.empty((self.B * self.NH, self.D, self.D), dtype=torch.float32, device=self.dev)
        z = torch.empty((self.B * self.NH, self.D), dtype=torch.float32, device=self.dev)
        with torch.cuda.device(self.dev):
            rc = self.L.mlstm_chunk_local_state(self.ws.data_ptr(), self.ws.numel(), S.data_ptr(), z.data_ptr(),
                                                *self.dims, self._stream())
        _lib.check(rc, "mlstm_chunk_local_state")
        return S, z

    def apply(self, state_in=None, h_dtype=torch.float32, return_state=False):
        """h of the segment given the inbound (S, z) (stabilised by the carried-in A) or None."""
        h = torch.empty((self.B, self.NH, self.S, self.D), dtype=h_dtype, device=self.dev)
        S_in = z_in = None
        if state_in is not None:
            S_in = state_in[0].to(device=self.dev, dtype=torch.float32).contiguous()
            z_in = state_in[1].to(device=self.dev, dtype=torch.float32).contiguous()
        S_out = z_out = None
        if return_state:
            S_out = torch.empty((self.B * self.NH, self.D, self.D), dtype=torch.float32, device=self.dev)
            z_out = torch.empty((self.B * self.NH, self.D), dtype=torch.float32, device=self.dev)
        ptr = lambda t: t.data_ptr() if t is not None else None
        with torch.cuda.device(self.dev):
            rc = self.L.mlstm_chunk_apply(self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(), ptr(self.o), ptr(S_in),
                                          ptr(z_in), h.data_ptr(), _lib.dtype_code(h), ptr(S_out), ptr(z_out),
                                          self.ws.data_ptr(), self.ws.numel(), *self.dims, self._stream())
        _lib.check(rc, "mlstm_chunk_apply")
        _lib.maybe_read_status(self.ws, self.dev, "mlstm_chunk_apply")
        return (h, (S_out, z_out)) if return_state else h

    def read_mb(self):
        """After ``apply``: the stabiliser m and the row sums b [B, NH, S] float32 (the parallel forward's M, B)."""
        m = torch.empty((self.B, self.NH, self.S), dtype=torch.float32, device=self.dev)
        b = torch.empty_like(m)
        with torch.cuda.device(self.dev):
            rc = self.L.mlstm_chunk_read_mb(self.ws.data_ptr(), self.ws.numel(), m.data_ptr(), b.data_ptr(), *self.dims,
                                            self._stream())
        _lib.check(rc, "mlstm_chunk_read_mb")
        return m, b

    # ---- sequence-parallel stages (one exchange between them)
    def sp_local(self):
        """Everything that needs no other rank; returns this segment's record [B*NH, D*D + D + 4] float32
        (S | z | {F_end, A_end} as two float64 in four float32 words)."""
        rec = torch.empty((self.B * self.NH, self.L.mlstm_chunk_sp_record_floats(self.D)), dtype=torch.float32,
                          device=self.dev)
        with torch.cuda.device(self.dev):
            rc = self.L.mlstm_chunk_sp_local(self.k.data_ptr(), self.v.data_ptr(), self.f.data_ptr(), self.i.data_ptr(),
                                             rec.data_ptr(), self.ws.data_ptr(), self.ws.numel(), *self.dims, self._stream())
        _lib.check(rc, "mlstm_chunk_sp_local")
        return rec

    def sp_apply(self, gathered, rank, h_dtype=torch.float32):
        """h of the segment from the gathered records [G, B*NH, record] of all ranks (rank order = sequence order)."""
        gathered = gathered.contiguous()
        world = gathered.shape[0]
        h = torch.empty((self.B, self.NH, self.S, self.D), dtype=h_dtype, device=self.dev)
        with torch.cuda.device(self.dev):
            rc = self.L.mlstm_chunk_sp_apply(self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(),
                                             self.o.data_ptr() if self.o is not None else None, gathered.data_ptr(), world,
                                             int(rank), h.data_ptr(), _lib.dtype_code(h), None, self.ws.data_ptr(),
                                             self.ws.numel(), *self.dims, self._stream())
        _lib.check(rc, "mlstm_chunk_sp_apply")
        _lib.maybe_read_status(self.ws, self.dev, "mlstm_chunk_sp_apply")
        return h


def mlstm_chunkwise_backward(dh, q, k, v, f, i, h, m, b, chunk_size=256):
    """Gradients (dq, dk, dv, df, di) of the chunkwise forward without inbound state, in time linear in S."""
    dev = _lib.require_cuda(dh, q, k, v, f, i, h, m, b)
    B, NH, S, D = q.shape
    if dh.shape != q.shape or dh.dtype != h.dtype:
        raise ValueError("dh must match h in shape and element type")
    dt, hdt, chunk = _lib.dtype_code(q), _lib.dtype_code(h), int(chunk_size)
    L = _lib.lib()
    nbytes = L.mlstm_chunk_bwd_workspace(B, NH, S, D, dt, hdt, chunk)
    if nbytes == 0:
        raise _lib.MlstmError(-4, "mlstm_chunk_bwd_workspace (needs float16/bfloat16, D = 128 or 256, chunk % 128 == 0)")
    ws = _lib.workspace(nbytes, dev)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    df, di = torch.empty_like(f), torch.empty_like(i)
    with torch.cuda.device(dev):
        rc = L.mlstm_chunk_bwd(dh.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), f.data_ptr(), i.data_ptr(), h.data_ptr(),
                               m.data_ptr(), b.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), df.data_ptr(),
                               di.data_ptr(), ws.data_ptr(), ws.numel(), B, NH, S, D, dt, hdt, chunk, _lib.stream_ptr(dev))
    _lib.check(rc, "mlstm_chunk_bwd")
    _lib.maybe_read_status(ws, dev, "mlstm_chunk_bwd")
    return dq, dk, dv, df, di


class _ChunkwiseWithGrad(torch.autograd.Function):
    """Chunkwise forward and chunkwise backward (both linear in S); h is float32 like the parallel path's."""

    @staticmethod
    def forward(ctx, q, k, v, f, i, chunk_size):
        seg = ChunkSegment(q, k, v, f, i, chunk_size, shared_workspace=True)
        seg.prepare(None)
        h = seg.apply(None)
        m, b = seg.read_mb()
        ctx.save_for_backward(q, k, v, f, i, h, m, b)
        ctx.chunk = chunk_size
        return h

    @staticmethod
    def backward(ctx, dh):
        q, k, v, f, i, h, m, b = ctx.saved_tensors
        return mlstm_chunkwise_backward(dh.contiguous(), q, k, v, f, i, h, m, b, ctx.chunk) + (None,)


def mlstm_chunkwise(q, k, v, f, i, chunk_size=256, h_dtype=torch.float32, initial=None, return_state=False, o=None):
    """Chunkwise forward on one GPU (times silu(o) when the output-gate pre-activation ``o`` is given).
    Inputs that require gradients get them through the chunkwise backward (no ``initial`` / ``return_state``
    / ``o`` in that case; wrap the output gate around it, as ``mlstm_scan`` does).

    ``initial`` = (S, z, F, A) continues an earlier segment: S [B*NH, D, D] and z [B*NH, D] float32
    stabilised by A, and F, A float64 [B*NH] (the log-forget total and the prefix maximum of a = i - F
    at the end of that segment).  With ``return_state`` the same tuple for the end of this call is
    returned beside h.
    """
    if torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v, f, i)):
        if initial is not None or return_state or o is not None or h_dtype != torch.float32:
            raise ValueError("gradients are available for the plain call: no initial / return_state / o, float32 h")
        return _ChunkwiseWithGrad.apply(q, k, v, f, i, int(chunk_size))
    seg = ChunkSegment(q, k, v, f, i, chunk_size, shared_workspace=True, o=o)
    carry = None
    state_in = None
    if initial is not None:
        S0, z0, F0, A0 = initial
        carry = torch.stack([F0.double().reshape(-1), A0.double().reshape(-1)], dim=1)
        state_in = (S0, z0)
    summary = seg.prepare(carry)
    out = seg.apply(state_in, h_dtype=h_dtype, return_state=return_state)
    if return_state:
        h, (S1, z1) = out
        return h, (S1, z1, summary[:, 0].clone(), summary[:, 1].clone())
    return out


def fold_gate_summaries(local):
    """local: [G, BH, 2] = every segment's own {F_end, A_end} (no carry, float64).
    Returns carry_in [G, BH, 2]: {F, A} accumulated over the segments before each one (A of the first
    segment is -inf).  With F_in the log-forget total before segment g, a position's a = i - F shifts
    by -F_in, hence the segment's prefix maximum in global terms is A_local - F_in."""
    local = local.double()
    F_loc, A_loc = local[..., 0], local[..., 1]
    F_in = torch.cumsum(F_loc, 0) - F_loc                      # exclusive prefix sum over segments
    A_glob = A_loc - F_in
    A_in = torch.full_like(A_glob, -float("inf"))
    if A_glob.shape[0] > 1:
        A_in[1:] = torch.cummax(A_glob, 0).values[:-1]         # exclusive prefix maximum over segments
    return torch.stack([F_in, A_in], dim=-1)


def fold_states(S_all, z_all, A_end_all, rank):
    """Inbound state of segment ``rank`` from the states the lower segments add.

    S_all [G, BH, D, D], z_all [G, BH, D]: each segment's added state, stabilised by its own A_end
    (A_end_all [G, BH], float64, carries included, non-decreasing in g).  The result is stabilised by
    A_end of segment rank-1, i.e. by the carried-in A of segment ``rank``.  None for rank 0."""
    if rank == 0:
        return None
    A = A_end_all[:rank].double()
    w = torch.exp(A - A[rank - 1]).float()                      # [rank, BH], <= 1
    w = torch.nan_to_num(w, nan=0.0)                            # -inf - -inf (nothing seen yet): no contribution
    S = (w[:, :, None, None] * S_all[:rank].float()).sum(0)
    z = (w[:, :, None] * z_all[:rank].float()).sum(0)
    return S, z


def fold_records(gathered, rank):
    """The arithmetic of the fold kernel in torch: gathered [G, BH, D*D + D + 4] float32 records (see
    ``ChunkSegment.sp_local``) -> (S_in [BH, D, D], z_in [BH, D], F_in [BH], A_in [BH]) of segment ``rank``.
    Segment g's state is stabilised by its own prefix maximum A_g with F counted from zero, i.e. by
    A_g - F_in(g) in global terms; A_in is the maximum of those over g < rank."""
    G, BH, R = gathered.shape
    D = int(round((-1 + (1 + 4 * (R - 4)) ** 0.5) / 2))
    tail = gathered[:, :, D * D + D:].contiguous().view(torch.float64).reshape(G, BH, 2)
    F_loc, A_loc = tail[..., 0], tail[..., 1]
    F_before = torch.cumsum(F_loc, 0) - F_loc                   # [G, BH] log-forget total before each segment
    A_hat = A_loc - F_before
    S_in = torch.zeros((BH, D, D), dtype=torch.float32, device=gathered.device)
    z_in = torch.zeros((BH, D), dtype=torch.float32, device=gathered.device)
    A_in = torch.full((BH,), -float("inf"), dtype=torch.float64, device=gathered.device)
    if rank > 0:
        A_in = A_hat[:rank].max(0).values
        w = torch.exp(A_hat[:rank] - A_in).float()              # [rank, BH], <= 1
        S_in = (w[:, :, None] * gathered[:rank, :, :D * D]).sum(0).reshape(BH, D, D)
        z_in = (w[:, :, None] * gathered[:rank, :, D * D:D * D + D]).sum(0)
    return S_in, z_in, F_before[rank], A_in


def _all_gather(t, group):
    import torch.distributed as dist
    t = t.contiguous()
    G = dist.get_world_size(group)
    out = torch.empty((G * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)   # concatenated along dim 0
    dist.all_gather_into_tensor(out, t, group=group)
    return out.view((G,) + tuple(t.shape))


def sequence_parallel_forward(segment, group=None, h_dtype=torch.float32):
    """The sequence-parallel protocol over any object with the ``sp_local`` / ``sp_apply`` stages of
    ChunkSegment: local work, one all-gather of the per-slice records, fold + output."""
    import torch.distributed as dist
    rank = dist.get_rank(group)
    record = segment.sp_local()                                      # [BH, D*D + D + 4]
    gathered = _all_gather(record, group)                            # [G, BH, D*D + D + 4]
    return segment.sp_apply(gathered, rank, h_dtype=h_dtype)


def mlstm_chunkwise_sequence_parallel(q, k, v, f, i, chunk_size=256, group=None, h_dtype=torch.float32, o=None):
    """Every rank passes its contiguous segment [B, NH, S/G, D] (rank order = sequence order) and gets
    the outputs of that segment (times silu(o) when the output-gate pre-activation ``o`` is given).
    Needs an initialised torch.distributed process group (NCCL)."""
    return sequence_parallel_forward(ChunkSegment(q, k, v, f, i, chunk_size, shared_workspace=True, o=o), group=group,
                                     h_dtype=h_dtype)
