"""GPU parity tests of the chunkwise forward (single GPU and sequence-parallel over NCCL)."""
import importlib
import os
import socket

import pytest
import torch

from oracle import mlstm_oracle as orc
from tests import kernel_model as km

pytestmark = pytest.mark.gpu
PKG = "xlstm-triton-cuda-implementation_b200"
TOL_16 = 1e-2


@pytest.fixture(scope="module")
def gc():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from tests import gpu_cases
    return gpu_cases


def _dev(x, names=("q", "k", "v", "f", "i")):
    return [x[n].cuda() for n in names]


@pytest.mark.parametrize("dtype,S,chunk,f_mean", [
    (torch.bfloat16, 1024, 256, 3.0),
    (torch.bfloat16, 1000, 256, 0.0),     # ragged last block
    (torch.float16, 768, 128, 3.0),
    (torch.bfloat16, 256, 256, -2.0),     # a single block: no inbound state anywhere
    (torch.bfloat16, 2048, 512, 5.0),
    (torch.bfloat16, 9000, 256, 3.0),     # long enough for the segmented gate scan, ragged
])
def test_chunkwise_against_oracle(gc, dtype, S, chunk, f_mean):
    x = gc.make_inputs(1, 2, S, 128, dtype, f_mean=f_mean, qkv_scale=128 ** -0.5, seed=S + chunk)
    h = gc.PKG.mlstm_chunkwise(*_dev(x), chunk_size=chunk)
    torch.cuda.synchronize()
    assert h.dtype == torch.float32
    assert orc.max_abs_rel(h, orc.matmul_forward(x["q"], x["k"], x["v"], x["f"], x["i"])) < TOL_16


def test_chunkwise_matches_quadratic_kernel_at_4096(gc):
    x = gc.make_inputs(2, 2, 4096, 128, torch.bfloat16, f_mean=3.0, qkv_scale=128 ** -0.5, seed=9)
    d = _dev(x)
    h1 = gc.PKG.mlstm_chunkwise(*d, chunk_size=256)
    h2 = gc.PKG.mlstm_matmul(*d)
    assert orc.max_abs_rel(h1, h2) < TOL_16


def test_segment_stages_against_model(gc):
    """gate summary, carried gates and the segment's added state against the dense fp64 model."""
    x = gc.make_inputs(1, 2, 512, 128, torch.bfloat16, f_mean=2.0, qkv_scale=128 ** -0.5, seed=4)
    host = [x[n] for n in ("q", "k", "v", "f", "i")]
    mc = importlib.import_module(PKG + ".mlstm_chunkwise")
    seg = mc.ChunkSegment(*_dev(x), chunk_size=256)
    model = km.ChunkSegmentModel(*host, chunk_size=256)
    # log-sigmoid is evaluated in fp32 (1e-7 relative per term) and summed in double
    assert orc.max_abs_rel(seg.gate_summary().cpu(), model.gate_summary()) < 1e-6
    carry = torch.tensor([[-3.0, 1.5], [-1.0, -0.25]], dtype=torch.float64)
    assert orc.max_abs_rel(seg.prepare(carry).cpu(), model.prepare(carry)) < 1e-6
    S_g, z_g = seg.local_state()
    S_m, z_m = model.local_state()
    assert orc.max_abs_rel(S_g.cpu(), S_m) < TOL_16
    assert orc.max_abs_rel(z_g.cpu(), z_m) < TOL_16


def test_state_continuation_equals_one_call(gc):
    """Two calls with the state carried through `initial` / `return_state` against the unsplit oracle."""
    x = gc.make_inputs(1, 2, 1536, 128, torch.bfloat16, f_mean=3.0, qkv_scale=128 ** -0.5, seed=5)
    cut = 512
    first = [t[:, :, :cut].contiguous() for t in _dev(x)]
    second = [t[:, :, cut:].contiguous() for t in _dev(x)]
    h1, st = gc.PKG.mlstm_chunkwise(*first, chunk_size=256, return_state=True)
    h2 = gc.PKG.mlstm_chunkwise(*second, chunk_size=256, initial=st)
    ref = orc.matmul_forward(x["q"], x["k"], x["v"], x["f"], x["i"])
    assert orc.max_abs_rel(torch.cat([h1, h2], 2), ref) < TOL_16


@pytest.mark.parametrize("cuts,f_mean", [((1024,), 3.0), ((512, 1536, 2560), 0.0), ((256, 512, 768, 1024, 1280, 1536, 3584), 4.0)])
def test_sequence_parallel_stages_on_one_gpu(gc, cuts, f_mean):
    """The one-exchange protocol with the ranks emulated one after the other on one GPU: every segment's
    record with no carry (sp_local), the records stacked as the all-gather would, then fold + output per
    segment (sp_apply).  Checks the fold kernel against its torch statement and h against the unsplit oracle."""
    mc = importlib.import_module(PKG + ".mlstm_chunkwise")
    S = 4096
    x = gc.make_inputs(1, 2, S, 128, torch.bfloat16, f_mean=f_mean, qkv_scale=128 ** -0.5, seed=len(cuts), with_o=True)
    edges = (0,) + tuple(cuts) + (S,)
    segs = []
    for a, b in zip(edges[:-1], edges[1:]):
        part = [x[n][:, :, a:b].contiguous().cuda() for n in ("q", "k", "v", "f", "i")]
        segs.append(mc.ChunkSegment(*part, chunk_size=256, o=x["o"][:, :, a:b].contiguous().cuda()))
    gathered = torch.stack([s.sp_local() for s in segs])
    h = torch.cat([s.sp_apply(gathered, g) for g, s in enumerate(segs)], 2)
    torch.cuda.synchronize()
    ref = orc.matmul_forward(x["q"], x["k"], x["v"], x["f"], x["i"]) * torch.nn.functional.silu(x["o"].double())
    assert orc.max_abs_rel(h, ref) < TOL_16
    # the fold kernel against its torch statement, for the last segment
    g = len(segs) - 1
    S_in, z_in, F_in, A_in = mc.fold_records(gathered, g)
    L = gc._lib.lib()
    carry = torch.empty((2, 2), dtype=torch.float64, device="cuda")
    seg = segs[g]
    hbuf = torch.empty((1, 2, seg.S, 128), dtype=torch.float32, device="cuda")
    rc = L.mlstm_chunk_sp_apply(seg.q.data_ptr(), seg.k.data_ptr(), seg.v.data_ptr(), None, gathered.data_ptr(), len(segs), g,
                                hbuf.data_ptr(), 0, carry.data_ptr(), seg.ws.data_ptr(), seg.ws.numel(), *seg.dims, seg._stream())
    assert rc == 0
    torch.cuda.synchronize()
    assert orc.max_abs_rel(carry[:, 0].cpu(), F_in.cpu()) < 1e-12
    assert orc.max_abs_rel(carry[:, 1].cpu(), A_in.cpu()) < 1e-12


@pytest.mark.parametrize("dtype,S,chunk,f_mean", [
    (torch.bfloat16, 1024, 256, 3.0),
    (torch.float16, 900, 256, 0.0),       # ragged last block
    (torch.bfloat16, 2048, 512, 1.0),     # four-tile blocks
    (torch.bfloat16, 256, 256, -2.0),     # a single block
    (torch.bfloat16, 640, 128, 2.0),      # one-tile blocks: every row tile has a state step only plus its own tile
])
def test_chunkwise_at_head_dimension_256(gc, dtype, S, chunk, f_mean):
    """D = 256: a block's state is written in two halves of 128 key rows and applied in two state steps; the
    forward against the oracle, with the output gate, in two calls with the state carried, and split over three
    segments through the sequence-parallel stages; then the chunkwise backward (its state steps are split the same
    way) against the closed-form backward of the oracle."""
    D = 256
    mc = importlib.import_module(PKG + ".mlstm_chunkwise")
    x = gc.make_inputs(1, 2, S, D, dtype, f_mean=f_mean, qkv_scale=D ** -0.5, seed=S + chunk + 2, with_o=True)
    ref = orc.matmul_forward(x["q"], x["k"], x["v"], x["f"], x["i"])
    h = gc.PKG.mlstm_chunkwise(*_dev(x), chunk_size=chunk)
    torch.cuda.synchronize()
    assert h.dtype == torch.float32 and orc.max_abs_rel(h, ref) < TOL_16
    ref_o = ref * torch.nn.functional.silu(x["o"].double())
    ho = gc.PKG.mlstm_chunkwise(*_dev(x), chunk_size=chunk, o=x["o"].cuda())
    assert orc.max_abs_rel(ho, ref_o) < TOL_16
    if S >= 2 * chunk:
        cut = chunk
        first = [t[:, :, :cut].contiguous() for t in _dev(x)]
        second = [t[:, :, cut:].contiguous() for t in _dev(x)]
        h1, st = gc.PKG.mlstm_chunkwise(*first, chunk_size=chunk, return_state=True)
        h2 = gc.PKG.mlstm_chunkwise(*second, chunk_size=chunk, initial=st)
        assert orc.max_abs_rel(torch.cat([h1, h2], 2), ref) < TOL_16
    if S >= 3 * chunk:
        edges = (0, chunk, 2 * chunk, S)
        segs = []
        for a, b in zip(edges[:-1], edges[1:]):
            part = [x[n][:, :, a:b].contiguous().cuda() for n in ("q", "k", "v", "f", "i")]
            segs.append(mc.ChunkSegment(*part, chunk_size=chunk, o=x["o"][:, :, a:b].contiguous().cuda()))
        gathered = torch.stack([sg.sp_local() for sg in segs])
        hs = torch.cat([sg.sp_apply(gathered, g) for g, sg in enumerate(segs)], 2)
        assert orc.max_abs_rel(hs, ref_o) < TOL_16
    names = ("q", "k", "v", "f", "i")
    t = {n: x[n].cuda().requires_grad_(True) for n in names}
    hg = gc.PKG.mlstm_chunkwise(*(t[n] for n in names), chunk_size=chunk)
    hg.backward(x["dh"].cuda())
    torch.cuda.synchronize()
    for n, r in zip(names, gc.oracle_backward(x, torch.float32)):
        assert t[n].grad.dtype == dtype
        assert orc.max_abs_rel(t[n].grad, r) < TOL_16, n


def test_scan_entry_takes_the_chunkwise_form_at_256(gc):
    """mlstm_scan on a long 16-bit sequence at D = 256 (S > 2 D): routed to the chunkwise form by the library; against
    the oracle and against the parallel kernel forced by hand."""
    S, D = 2304, 256
    x = gc.make_inputs(1, 2, S, D, torch.bfloat16, f_mean=3.0, qkv_scale=D ** -0.5, seed=77, with_o=True)
    d = [x[n].cuda() for n in ("q", "k", "v", "f", "i", "o")]
    L = gc._lib.lib()
    dt = gc._lib.dtype_code(x["q"])
    assert L.mlstm_scan_fwd_workspace(1, 2, S, D, dt, 0) == L.mlstm_chunk_workspace(1, 2, S, D, dt, 256)
    h = gc.PKG.mlstm_scan(*d)
    ref = orc.matmul_forward(x["q"], x["k"], x["v"], x["f"], x["i"]) * torch.nn.functional.silu(x["o"].double())
    assert orc.max_abs_rel(h, ref) < TOL_16
    h2 = gc.PKG.mlstm_matmul(*d[:5]) * torch.nn.functional.silu(d[5].float())
    assert orc.max_abs_rel(h, h2) < TOL_16


def test_long_carry_at_head_dimension_256(gc):
    """S = 16 384 at D = 256 (64 blocks of carried state, two state steps each) on one head against the recurrent
    oracle (one step per time index), on the first block, one in the middle and the last."""
    S, D = 16384, 256
    x = gc.make_inputs(1, 1, S, D, torch.bfloat16, f_mean=3.0, qkv_scale=D ** -0.5, seed=66)
    h = gc.PKG.mlstm_chunkwise(*_dev(x), chunk_size=256).cpu()
    ref = orc.scan_forward(x["q"], x["k"], x["v"], x["f"], x["i"], torch.zeros_like(x["q"]).float() + 1.2784645,
                           dtype=torch.float64)   # silu(1.2784645...) = 1: the gate drops out
    ref = ref / torch.nn.functional.silu(torch.tensor(1.2784645, dtype=torch.float64))
    for lo in (0, 31 * 256, S - 256):
        err = orc.max_abs_rel(h[:, :, lo:lo + 256], ref[:, :, lo:lo + 256])
        assert err < TOL_16, (lo, err)


def test_chunkwise_calls_back_to_back(gc):
    """Twenty chunkwise forward + backward calls without a synchronize in between, alternating two sequences on one
    workspace size: equal to the same calls made alone."""
    dev = torch.device("cuda", 0)
    mc = importlib.import_module(PKG + ".mlstm_chunkwise")
    sets = []
    for seed in (3, 4):
        x = gc.make_inputs(1, 2, 1024, 128, torch.bfloat16, f_mean=3.0, qkv_scale=128 ** -0.5, seed=seed)
        sets.append({n: t.to(dev) for n, t in x.items()})
    def call(d):
        seg = mc.ChunkSegment(d["q"], d["k"], d["v"], d["f"], d["i"], 256, shared_workspace=True)
        seg.prepare(None)
        h = seg.apply(None)
        m, b = seg.read_mb()
        return (h,) + tuple(mc.mlstm_chunkwise_backward(d["dh"], d["q"], d["k"], d["v"], d["f"], d["i"], h, m, b, chunk_size=256))
    alone = []
    for d in sets:
        out = call(d)
        torch.cuda.synchronize()
        alone.append([t.clone() for t in out])
    last = [None, None]
    for it in range(20):
        last[it & 1] = call(sets[it & 1])
    torch.cuda.synchronize()
    for k in range(2):
        for a, b in zip(last[k], alone[k]):
            assert torch.equal(a, b)


def test_long_context_configuration_at_its_own_size(gc):
    """Configuration 5 (S = 65 536, D = 128, bf16, chunk 256: 256 blocks of carry) on one head against the
    recurrent oracle (one step per time index), compared on the first block, two blocks in the middle and
    the last block."""
    S, D = 65536, 128
    x = gc.make_inputs(1, 1, S, D, torch.bfloat16, f_mean=3.0, qkv_scale=D ** -0.5, seed=65)
    h = gc.PKG.mlstm_chunkwise(*_dev(x), chunk_size=256).cpu()
    ref = orc.scan_forward(x["q"], x["k"], x["v"], x["f"], x["i"], torch.zeros_like(x["q"]).float() + 1.2784645,
                           dtype=torch.float64)   # silu(1.2784645...) = 1: the gate drops out
    ref = ref / torch.nn.functional.silu(torch.tensor(1.2784645, dtype=torch.float64))
    for lo in (0, 20 * 256, 133 * 256, S - 256):
        err = orc.max_abs_rel(h[:, :, lo:lo + 256], ref[:, :, lo:lo + 256])
        assert err < TOL_16, (lo, err)


@pytest.mark.parametrize("dtype,S,chunk,f_mean", [
    (torch.bfloat16, 1024, 256, 3.0),
    (torch.bfloat16, 1000, 256, 0.0),     # ragged last block
    (torch.float16, 768, 128, 1.0),
    (torch.bfloat16, 256, 256, 0.0),      # a single block: nothing is carried
    (torch.bfloat16, 2304, 512, -1.0),    # strong decay, four-tile blocks and a ragged last one
])
def test_chunkwise_backward_against_oracle(gc, dtype, S, chunk, f_mean):
    """Chunkwise forward + chunkwise backward (states carried forward for dQ, back for dK and dV) against the
    closed-form backward of the parallel oracle, and against the parallel backward kernels on the device."""
    x = gc.make_inputs(1, 2, S, 128, dtype, f_mean=f_mean, qkv_scale=128 ** -0.5, seed=S + chunk + 1)
    names = ("q", "k", "v", "f", "i")
    t = {n: x[n].cuda().requires_grad_(True) for n in names}
    h = gc.PKG.mlstm_chunkwise(*(t[n] for n in names), chunk_size=chunk)
    h.backward(x["dh"].cuda())
    torch.cuda.synchronize()
    ref = gc.oracle_backward(x, torch.float32)
    for n, r in zip(names, ref):
        g = t[n].grad
        assert g.dtype == dtype and bool(torch.isfinite(g.float()).all()), n
        assert orc.max_abs_rel(g.float(), r) < TOL_16, (n, orc.max_abs_rel(g.float(), r))
    assert float(t["f"].grad[..., 0].abs().max()) == 0.0
    # the quadratic kernels on the same h, m, b
    d = [x[n].cuda() for n in names]
    hq, m, b = gc.PKG.mlstm_matmul_forward(*d)
    gq = gc.PKG.mlstm_matmul_backward(x["dh"].cuda(), *d, hq, m, b)
    for n, a in zip(names, gq):
        assert orc.max_abs_rel(t[n].grad.float(), a.float()) < TOL_16, n


def test_chunkwise_forward_backward_against_reference_golden(gc, golden_dir):
    """S = 1024, D = 128, bf16, chunk 256: chunkwise forward and backward against the reference's own PyTorch
    forward / backward on the same bf16 values."""
    from tests.test_oracle import load_long_bf16
    x, ref = load_long_bf16(golden_dir)
    names = ("q", "k", "v", "f", "i")
    t = {n: x[n].cuda().requires_grad_(True) for n in names}
    h = gc.PKG.mlstm_chunkwise(*(t[n] for n in names), chunk_size=256)
    h.backward(x["dh"].float().cuda())
    assert orc.max_abs_rel(h.detach(), ref["h"]) < TOL_16
    for n in names:
        r = ref["d" + n].clone()
        if n == "f":
            r[..., 0] = 0.0
        assert orc.max_abs_rel(t[n].grad.float(), r) < TOL_16, n


def test_chunkwise_backward_of_a_long_slice(gc):
    """S = 8448 (three 4096-position segments of the gate scan and of the dF scan, 33 blocks of carried state in each
    direction): the chunkwise backward against the parallel backward kernels on the same inputs."""
    S, D = 8448, 128
    x = gc.make_inputs(1, 2, S, D, torch.bfloat16, f_mean=3.0, qkv_scale=D ** -0.5, seed=84)
    d = _dev(x)
    h, m, b = gc.PKG.mlstm_matmul_forward(*d)
    dh = x["dh"].cuda()
    ref = gc.PKG.mlstm_matmul_backward(dh, *d, h, m, b)
    mc = importlib.import_module(PKG + ".mlstm_chunkwise")
    got = mc.mlstm_chunkwise_backward(dh, *d, h, m, b, chunk_size=256)
    torch.cuda.synchronize()
    for name, g1, g2 in zip(("dq", "dk", "dv", "df", "di"), got, ref):
        assert orc.max_abs_rel(g1, g2) < TOL_16, name


def test_chunkwise_backward_with_16_bit_h(gc):
    """The backward through the C ABI with h and dh in the input type (no fp32 copy of h anywhere)."""
    mc = importlib.import_module(PKG + ".mlstm_chunkwise")
    x = gc.make_inputs(2, 2, 1280, 128, torch.bfloat16, f_mean=3.0, qkv_scale=128 ** -0.5, seed=12)
    d = _dev(x)
    seg = mc.ChunkSegment(*d, chunk_size=256)
    seg.prepare(None)
    h = seg.apply(None, h_dtype=torch.bfloat16)
    m, b = seg.read_mb()
    dh = x["dh"].bfloat16().cuda()
    grads = mc.mlstm_chunkwise_backward(dh, *d, h, m, b, chunk_size=256)
    torch.cuda.synchronize()
    ref = gc.oracle_backward(x, torch.bfloat16)
    for n, g, r in zip(("dq", "dk", "dv", "df", "di"), grads, ref):
        assert orc.max_abs_rel(g.float(), r) < TOL_16, (n, orc.max_abs_rel(g.float(), r))
    # m and b are what the parallel forward returns
    hq, mq, bq = gc.PKG.mlstm_matmul_forward(*d, h_dtype=torch.bfloat16)
    assert orc.max_abs_rel(m, mq) < 1e-5 and orc.max_abs_rel(b, bq) < TOL_16


def test_scan_gradients_take_the_chunkwise_backward(gc):
    """mlstm_scan on a long 16-bit sequence with inputs that require gradients: chunkwise forward and backward
    behind the output gate, against autograd of the fp64 oracle."""
    x = gc.make_inputs(1, 2, 1536, 128, torch.bfloat16, f_mean=2.0, qkv_scale=128 ** -0.5, seed=77, with_o=True)
    names = ("q", "k", "v", "f", "i", "o")
    t = {n: x[n].cuda().requires_grad_(True) for n in names}
    h = gc.PKG.mlstm_scan(*(t[n] for n in names))
    h.backward(x["dh"].cuda())
    r = {n: x[n].double().requires_grad_(True) for n in names}
    href = orc.matmul_forward(r["q"], r["k"], r["v"], r["f"], r["i"]) * torch.nn.functional.silu(r["o"])
    href.backward(x["dh"].double())
    assert orc.max_abs_rel(h.detach(), href.detach()) < TOL_16
    for n in names:
        assert orc.max_abs_rel(t[n].grad.float(), r[n].grad) < TOL_16, n


def test_chunkwise_rejects_unsupported_cases(gc):
    x = gc.make_inputs(1, 1, 256, 64, torch.bfloat16)
    with pytest.raises(gc._lib.MlstmError):
        gc.PKG.mlstm_chunkwise(*_dev(x))              # D != 128
    x = gc.make_inputs(1, 1, 256, 128, torch.bfloat16)
    with pytest.raises(gc._lib.MlstmError):
        gc.PKG.mlstm_chunkwise(*_dev(x), chunk_size=200)   # chunk not a multiple of 128


def _sp_worker(rank, world, port, x, out):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        pkg = importlib.import_module(PKG)
        S = x["q"].shape[2]
        a, b = rank * S // world, (rank + 1) * S // world
        seg = [x[n][:, :, a:b].contiguous().cuda() for n in ("q", "k", "v", "f", "i")]
        h = pkg.mlstm_chunkwise_sequence_parallel(*seg, chunk_size=256)
        torch.cuda.synchronize()
        ref = orc.matmul_forward(x["q"], x["k"], x["v"], x["f"], x["i"])[:, :, a:b]
        out[rank] = orc.max_abs_rel(h, ref)
    finally:
        dist.destroy_process_group()


def test_sequence_parallel_over_nccl(gc):
    """Contiguous segments on 2 (or 4) GPUs, carry over one NCCL all-gather, against the unsplit oracle."""
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    x = gc.make_inputs(1, 2, 4096, 128, torch.bfloat16, f_mean=3.0, qkv_scale=128 ** -0.5, seed=6)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = mp.Manager().dict()
    mp.spawn(_sp_worker, args=(world, port, x, out), nprocs=world, join=True)
    assert len(out) == world and all(e < TOL_16 for e in out.values()), dict(out)
