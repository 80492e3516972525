"""GPU parity tests of the individual kernels, called through the C ABI (via mok.ops / mok._lib)
and checked against the CPU oracle and the committed golden vectors."""
import os

import numpy as np
import pytest
import torch

from oracle import mok_oracle as O
from tests.golden import make_golden as MG
from tests.helpers import bf16_from_u16, rel_l2, to_bytes

pytestmark = pytest.mark.gpu


def _mok():
    import mok
    return mok


# ----------------------------------------------------------------------------------------
# scheduler: bit-exact
# ----------------------------------------------------------------------------------------
def _run_schedule(topk_all, El, cap, rank, dev):
    mok = _mok()
    out = mok.ops.schedule(topk_all.to(dev), El, cap, rank)
    torch.cuda.synchronize()
    return [t.cpu().numpy() for t in out]


def test_schedule_matches_golden(cuda_device, golden_dir):
    z = np.load(os.path.join(golden_dir, "schedule.npz"))
    for i, (W, T, K, El, fac, kind) in enumerate(MG.SCHEDULE_CASES):
        topk = MG.schedule_topk(W, T, K, El, kind)
        for rank in range(W):
            got = _run_schedule(topk, El, T * K * fac, rank, cuda_device)
            for name, g in zip(("peer_rank", "peer_token_idx", "num_tokens", "tokens_per_expert"), got):
                assert np.array_equal(z[f"{i}/{rank}/{name}"], g), (i, rank, name)
    assert _mok().last_status(cuda_device)[0] == 0


@pytest.mark.parametrize("W,T,K,El", [(1, 2048, 8, 128), (8, 1024, 8, 32), (4, 768, 5, 3), (2, 512, 1, 1),
                                       (1, 512, 7, 512), (8, 1792, 6, 8)])
def test_schedule_matches_oracle(cuda_device, W, T, K, El):
    g = torch.Generator().manual_seed(W * 31 + K)
    topk = torch.topk(torch.randn(W, T, W * El, generator=g), K, dim=2).indices.to(torch.int32)
    cap = T * K * max(2, W) + El * 256
    cap = (cap + 255) // 256 * 256
    for rank in sorted({0, W - 1}):
        ref = O.schedule_tables(topk.numpy(), El, cap, rank)
        got = _run_schedule(topk, El, cap, rank, cuda_device)
        for r, g_ in zip(ref, got):
            assert np.array_equal(r, g_)


def test_schedule_skewed_and_ragged(cuda_device):
    """Zipf-like skew: a few experts take most routes, many experts are empty."""
    W, T, K, El = 4, 1024, 4, 16
    g = torch.Generator().manual_seed(9)
    logits = torch.randn(W, T, W * El, generator=g) - 1.2 * torch.log(torch.arange(1, W * El + 1).float())
    logits[..., 5] = -1e9   # an expert nobody picks
    topk = torch.topk(logits, K, dim=2).indices.to(torch.int32)
    cap = T * K * W + El * 256
    for rank in range(W):
        ref = O.schedule_tables(topk.numpy(), El, cap, rank)
        got = _run_schedule(topk, El, cap, rank, cuda_device)
        for r, g_ in zip(ref, got):
            assert np.array_equal(r, g_)


def test_schedule_overflow_sets_status_not_trap(cuda_device):
    mok = _mok()
    W, T, K, El = 1, 512, 1, 8          # 512 routes over 8 experts -> 8 * 256 padded rows > capacity 1024
    topk = (torch.arange(T) % El).to(torch.int32).view(1, T, 1)
    mok.last_status(cuda_device, clear=True)
    pr, pt, nt, tpe = mok.ops.schedule(topk.to(cuda_device), El, 1024, 0)
    torch.cuda.synchronize()
    code, detail, _ = mok.last_status(cuda_device, clear=True)
    assert code == 1 and detail == 2048 and int(nt.item()) == 2048
    ref = O.schedule_tables(topk.numpy(), El, 1024, 0)
    assert np.array_equal(ref[0], pr.cpu().numpy())   # in-range slots are still exact


def test_schedule_full_size_properties(cuda_device):
    """EP=8 x 16384 tokens x top-8 (the MXFP8 benchmark shape): every route of every peer that
    targets this rank appears exactly once, experts are 256-padded, rows past num_tokens are -1."""
    W, T, K, El = 8, 16384, 8, 32
    g = torch.Generator().manual_seed(1)
    topk = torch.topk(torch.rand(W, T, W * El, generator=g), K, dim=2).indices.to(torch.int32)
    cap = T * K * 4
    rank = 3
    pr, pt, nt, tpe = _run_schedule(topk, El, cap, rank, cuda_device)
    n = int(nt[0])
    assert n == int(tpe.sum()) and (tpe % 256 == 0).all() and (pr[n:] == -1).all() and (pt[n:] == -1).all()
    valid = pr >= 0
    flat = topk.numpy().reshape(W, -1)
    owners = flat[pr[valid], pt[valid]]
    assert ((owners // El) == rank).all()
    assert valid.sum() == ((flat // El) == rank).sum()
    assert len(np.unique(pr[valid].astype(np.int64) * (T * K) + pt[valid])) == valid.sum()
    # rows of one expert are contiguous and sorted by expert
    starts = np.concatenate([[0], np.cumsum(tpe)])
    row_expert = np.searchsorted(starts, np.nonzero(valid)[0], side="right") - 1
    assert np.array_equal(owners - rank * El, row_expert)


# ----------------------------------------------------------------------------------------
# MXFP8 quantiser: bit-exact bytes
# ----------------------------------------------------------------------------------------
def test_quantize_matches_golden(cuda_device, golden_dir):
    mok = _mok()
    z = np.load(os.path.join(golden_dir, "quantize.npz"))
    for tag in ("x3", "x2"):
        x = bf16_from_u16(z[f"{tag}/in"]).to(cuda_device)
        got = mok.ops.mxfp8_quantize(x, True, True)
        for name, g in zip(("fp8", "sc", "fp8_t", "sc_t"), got):
            assert np.array_equal(z[f"{tag}/{name}"], to_bytes(g).reshape(z[f"{tag}/{name}"].shape)), (tag, name)


@pytest.mark.parametrize("shape,normal,transposed", [((256, 384), True, True), ((3, 128, 256), True, False),
                                                       ((2, 384, 128), False, True), ((1024, 2048), True, True)])
def test_quantize_matches_oracle(cuda_device, shape, normal, transposed):
    mok = _mok()
    g = torch.Generator().manual_seed(5678)
    x = (torch.randn(*shape, generator=g) * torch.exp(2.0 * torch.randn(*shape[:-1], 1, generator=g))).to(torch.bfloat16)
    x.view(-1)[:64] = 0       # an all-zero block (padding rows look like this)
    ref = O.mxfp8_quantize(x, normal, transposed)
    got = mok.ops.mxfp8_quantize(x.to(cuda_device), normal, transposed)
    for r, g_ in zip(ref, got):
        if r is None:
            assert g_ is None
        else:
            assert np.array_equal(r, to_bytes(g_).reshape(r.shape))


# ----------------------------------------------------------------------------------------
# epilogues
# ----------------------------------------------------------------------------------------
def test_epilogues_match_golden(cuda_device, golden_dir):
    mok = _mok()
    z = np.load(os.path.join(golden_dir, "elementwise.npz"))
    ys, cb = bf16_from_u16(z["ys"]).to(cuda_device), bf16_from_u16(z["cb"]).to(cuda_device)
    w = torch.from_numpy(z["w"]).to(cuda_device)
    out = mok.ops.fwd_epilogue(ys, cb, w)
    assert rel_l2(bf16_from_u16(z["fwd_epilogue"]).float(), out.float()) < 2e-3
    assert torch.equal(O.fwd_epilogue(ys.cpu(), cb.cpu(), w.cpu()), out.cpu())   # same fp32 order as the oracle
    dx = mok.ops.bwd_epilogue(ys, cb)
    assert torch.equal(bf16_from_u16(z["bwd_epilogue"]), dx.cpu())


def test_epilogue_constants_and_many_tokens(cuda_device):
    """Closed-form case from the reference tests: constants give exactly 1.5 and 3.0, with more
    than 2 * 65535 tokens."""
    mok = _mok()
    T, H, K = 131584, 256, 2
    ys = torch.full((T, H), 0.5, dtype=torch.bfloat16, device=cuda_device)
    cb = torch.full((T * K, H), 1.0, dtype=torch.bfloat16, device=cuda_device)
    w = torch.full((T, K), 0.5, dtype=torch.float32, device=cuda_device)
    assert bool((mok.ops.fwd_epilogue(ys, cb, w) == 1.5).all())
    ys.fill_(1.0)
    assert bool((mok.ops.bwd_epilogue(ys, cb) == 3.0).all())


# ----------------------------------------------------------------------------------------
# tcgen05 GEMM building block, all operand layouts
# ----------------------------------------------------------------------------------------
@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1)])
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (256, 512, 256), (1024, 768, 2048), (768, 256, 4160)])
def test_gemm_bf16_layouts(cuda_device, a_mn, b_mn, m, n, k):
    mok = _mok()
    L = mok._lib
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(cuda_device)
    b = torch.randn(n, k, generator=g).to(torch.bfloat16).to(cuda_device)
    ref = a.float() @ b.float().T
    a_arg = a.T.contiguous() if a_mn else a           # [K, M] when M-major
    b_arg = b.T.contiguous() if b_mn else b           # [K, N] when N-major
    c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=cuda_device)
    mok.last_status(cuda_device, clear=True)
    L.check(L.mok_gemm_bf16(a_arg.data_ptr(), b_arg.data_ptr(), c.data_ptr(), m, n, k, a_mn, b_mn,
                            L.status_tensor(cuda_device).data_ptr(), L.stream_ptr(cuda_device)), "gemm")
    torch.cuda.synchronize()
    assert mok.last_status(cuda_device)[0] == 0
    assert torch.isfinite(c.float()).all()
    assert rel_l2(ref, c.float()) < 4e-3


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (256, 512, 512), (1024, 768, 2048), (384, 256, 7168)])
def test_gemm_mxfp8(cuda_device, m, n, k):
    """Block-scaled tcgen05 GEMM: operands quantised by ops.mxfp8_quantize (bit-exact, tested above),
    result compared with an fp32 matmul of the dequantised operands."""
    mok = _mok()
    L = mok._lib
    g = torch.Generator().manual_seed(m + n + k)
    a = (torch.randn(m, k, generator=g) * torch.exp(torch.randn(m, 1, generator=g))).to(torch.bfloat16)
    b = (torch.randn(n, k, generator=g) * torch.exp(torch.randn(n, 1, generator=g))).to(torch.bfloat16)
    aq, asc, _, _ = mok.ops.mxfp8_quantize(a.to(cuda_device), True, False)
    bq, bsc, _, _ = mok.ops.mxfp8_quantize(b.to(cuda_device), True, False)
    a_dq = torch.from_numpy(O.mxfp8_dequantize(to_bytes(aq).reshape(m, k), asc.cpu().numpy()))
    b_dq = torch.from_numpy(O.mxfp8_dequantize(to_bytes(bq).reshape(n, k), bsc.cpu().numpy()))
    ref = a_dq @ b_dq.T
    c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=cuda_device)
    mok.last_status(cuda_device, clear=True)
    L.check(L.mok_gemm_mxfp8(aq.data_ptr(), asc.data_ptr(), bq.data_ptr(), bsc.data_ptr(), c.data_ptr(), m, n, k,
                             L.status_tensor(cuda_device).data_ptr(), L.stream_ptr(cuda_device)), "gemm_mxfp8")
    torch.cuda.synchronize()
    assert mok.last_status(cuda_device)[0] == 0
    assert torch.isfinite(c.float()).all()
    assert rel_l2(ref, c.float()) < 4e-3


# ----------------------------------------------------------------------------------------
# device barrier: the bounded wait runs out, reports it and returns
# ----------------------------------------------------------------------------------------
def test_barrier_wait_runs_out_and_recovers(cuda_device):
    """A two-rank barrier whose second "rank" never arrives: the peer list is {own counter, a scratch word}, so
    the own counter reaches 1 of the 2 arrivals it waits for.  With a 2 ms limit the kernel must give up, write
    MOK_STATUS_BARRIER_TIMEOUT (detail = the counter value it saw) and return; the context stays usable and a
    one-rank barrier on a fresh counter completes.  (The reference spins without limit here,
    csrc/utils.cuh:291-293.)"""
    import time
    mok = _mok()
    L = mok._lib
    dev = cuda_device
    mok.last_status(dev, clear=True)
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    scratch = torch.zeros(1, dtype=torch.int32, device=dev)
    target = torch.zeros(1, dtype=torch.int32, device=dev)
    status = L.status_tensor(dev)
    t0 = time.perf_counter()
    L.check(L.mok_barrier_all(counter.data_ptr(), L.ptr_array([counter.data_ptr(), scratch.data_ptr()]), 2,
                              target.data_ptr(), status.data_ptr(), 2_000_000, L.stream_ptr(dev)), "barrier_all")
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 2.0                       # it gave up after milliseconds, not the default minutes
    code, detail, _block = mok.last_status(dev, clear=True)
    assert code == 2 and detail == 1, (code, detail)
    assert int(target.item()) == 2 and int(counter.item()) == 1 and int(scratch.item()) == 1
    # a one-rank barrier on fresh state passes
    fresh, fresh_target = torch.zeros(1, dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev)
    L.check(L.mok_barrier_all(fresh.data_ptr(), L.ptr_array([fresh.data_ptr()]), 1, fresh_target.data_ptr(),
                              status.data_ptr(), 2_000_000, L.stream_ptr(dev)), "barrier_all")
    torch.cuda.synchronize()
    assert mok.last_status(dev)[0] == 0
    assert int(fresh.item()) == 1 and int(fresh_target.item()) == 1
    status.copy_(torch.tensor([2, 1, 0, 0], dtype=torch.int32))     # what a caller sees at its step boundary
    with pytest.raises(mok._lib.MokNativeError):
        mok.raise_for_status(dev)
    mok.last_status(dev, clear=True)
