"""GPU: the scheduler entry point that allocates nothing (`mok_schedule_static`).

Some callers of the library may not allocate device memory at all — a serving process whose
memory plan is fixed at start-up, or a loop that cannot afford the device-wide synchronisation a
cudaMalloc implies.  For them the scheduler's scratch sits in a fixed array inside the library.
This test drives that entry point through the C ABI, twice in a row on different routings (the
array keeps the previous call's contents, so the second call proves nothing stale is read), and
requires bit-identical tables to the caller-scratch entry point `mok_schedule` and to the CPU
oracle.  It also checks that a problem beyond the fixed limit is refused without launching, and
that the limit sits exactly where the header says (ep_size * num_local_experts <= 4080).

The file name keeps it last in collection order, so a run that stops at the first failure has
already run every other test.
"""
import numpy as np
import pytest
import torch

from oracle import mok_oracle as O

pytestmark = pytest.mark.gpu


def _tables(dev, cap, El):
    i32 = dict(dtype=torch.int32, device=dev)
    return (torch.full((cap,), 7, **i32), torch.full((cap,), 7, **i32), torch.full((1,), 7, **i32),
            torch.full((El,), 7, **i32))


def _call_both(L, dev, topk, W, T, K, El, cap, rank):
    status = L.status_tensor(dev)
    stream = L.stream_ptr(dev)
    ref = _tables(dev, cap, El)
    nbytes = L.mok_schedule_scratch_bytes(W, El)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    L.check(L.mok_schedule(topk.data_ptr(), W, T, K, El, cap, rank, *[t.data_ptr() for t in ref],
                           scratch.data_ptr(), nbytes, status.data_ptr(), stream), "mok_schedule")
    got = _tables(dev, cap, El)
    L.check(L.mok_schedule_static(topk.data_ptr(), W, T, K, El, cap, rank, *[t.data_ptr() for t in got],
                                  status.data_ptr(), stream), "mok_schedule_static")
    torch.cuda.synchronize()
    return ref, got


def test_static_scratch_scheduler_matches_twice(cuda_device):
    import mok
    L = mok._lib
    dev = cuda_device
    mok.last_status(dev, clear=True)
    cases = [(4, 1024, 8, 16, 3), (8, 768, 6, 4, 0)]          # (W, T, K, El, rank); second call reuses the array
    for seed, (W, T, K, El, rank) in enumerate(cases):
        g = torch.Generator().manual_seed(100 + seed)
        topk = torch.topk(torch.randn(W, T, W * El, generator=g), K, dim=2).indices.to(torch.int32).to(dev)
        cap = T * K * W
        ref, got = _call_both(L, dev, topk, W, T, K, El, cap, rank)
        want = O.schedule_tables(topk.cpu().numpy(), El, cap, rank)
        for name, r, g_, w in zip(("peer_rank", "peer_token_idx", "num_tokens", "tokens_per_expert"), ref, got, want):
            assert torch.equal(r, g_), (seed, name)
            if name == "peer_token_idx":                      # slots without a route are undefined in the oracle's table
                live = want[0] >= 0
                assert np.array_equal(w[live], g_.cpu().numpy()[live]), (seed, name)
            else:
                assert np.array_equal(w, g_.cpu().numpy()), (seed, name)
        assert int(got[2].item()) > 0
    assert mok.last_status(dev)[0] == 0


def test_static_scratch_scheduler_rejects_oversized(cuda_device):
    import mok
    L = mok._lib
    dev = cuda_device
    W, T, K, El = 8, 512, 1, 1024                             # needs ~8 MiB of scratch, the array holds 4 MiB
    assert L.mok_schedule_scratch_bytes(W, El) > L.mok_schedule_static_max_scratch_bytes()
    topk = torch.zeros(W, T, K, dtype=torch.int32, device=dev)
    out = _tables(dev, T * K * W, El)
    rc = L.mok_schedule_static(topk.data_ptr(), W, T, K, El, T * K * W, 0, *[t.data_ptr() for t in out],
                               L.status_tensor(dev).data_ptr(), L.stream_ptr(dev))
    assert rc == -4 and L.mok_error_string(rc) == b"problem exceeds the fixed size limit of this entry point"
    torch.cuda.synchronize()
    assert bool((out[0] == 7).all())                          # nothing was launched


def test_static_scratch_limit_is_where_the_header_says(cuda_device):
    """ep_size * num_local_experts = 4080 is served (and matches mok_schedule), 4081 is refused."""
    import mok
    L = mok._lib
    dev = cuda_device
    W, T, K, El = 8, 512, 2, 510
    assert W * El == 4080 and L.mok_schedule_scratch_bytes(W, El) <= L.mok_schedule_static_max_scratch_bytes()
    g = torch.Generator().manual_seed(5)
    topk = torch.topk(torch.randn(W, T, W * El, generator=g), K, dim=2).indices.to(torch.int32).to(dev)
    cap = (T * K * W + El * 256 + 255) // 256 * 256
    ref, got = _call_both(L, dev, topk, W, T, K, El, cap, 5)
    for r, g_ in zip(ref, got):
        assert torch.equal(r, g_)
    W, El = 7, 583
    assert W * El == 4081 and L.mok_schedule_scratch_bytes(W, El) > L.mok_schedule_static_max_scratch_bytes()
    topk = torch.zeros(W, T, K, dtype=torch.int32, device=dev)
    out = _tables(dev, cap, El)
    rc = L.mok_schedule_static(topk.data_ptr(), W, T, K, El, cap, 0, *[t.data_ptr() for t in out],
                               L.status_tensor(dev).data_ptr(), L.stream_ptr(dev))
    assert rc == -4
    torch.cuda.synchronize()
    assert mok.last_status(dev)[0] == 0
