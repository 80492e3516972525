"""GPU parity tests of the router kernel (top-K experts + renormalised weights, and its gradient) against the
CPU oracle on the golden logits taken from the reference's input generator, and of route_and_schedule against
build_schedule."""
import os

import numpy as np
import pytest
import torch

from oracle import mok_oracle as O

pytestmark = pytest.mark.gpu

WEIGHT_ATOL = 2e-6       # f32 exp/divide on the device against float64 on the host


@pytest.mark.parametrize("case", [0, 1, 2])
def test_router_matches_golden(cuda_device, golden_dir, case):
    import mok
    g = np.load(os.path.join(golden_dir, "router.npz"))
    logits, experts, weights = g[f"{case}/logits"], g[f"{case}/topk_experts"], g[f"{case}/router_weights"]
    e, w = mok.ops.router_topk(torch.from_numpy(logits).to(cuda_device), experts.shape[1])
    assert e.dtype == torch.int64 and w.dtype == torch.float32
    assert (e.cpu().numpy() == experts).all()
    assert np.abs(w.cpu().numpy() - weights).max() < WEIGHT_ATOL


@pytest.mark.parametrize("T,E,K", [(512, 100, 7), (300, 1000, 32), (1024, 33, 1), (512, 5, 5)])
def test_router_shapes_against_oracle(cuda_device, T, E, K):
    import mok
    logits = np.random.default_rng(T + E).standard_normal((T, E)).astype(np.float32) * 3.0
    ref_e, ref_w = O.router_topk(logits, K)
    e, w = mok.ops.router_topk(torch.from_numpy(logits).to(cuda_device), K)
    assert (e.cpu().numpy() == ref_e).all()
    assert np.abs(w.cpu().numpy() - ref_w).max() < WEIGHT_ATOL
    dw = np.random.default_rng(1).standard_normal((T, K)).astype(np.float32)
    got = mok.ops.router_topk_bwd(e, w, torch.from_numpy(dw).to(cuda_device), E).cpu().numpy()
    ref = O.router_topk_bwd(ref_e, ref_w, dw, E)
    assert np.abs(got - ref).max() < 1e-5


def test_router_ties_take_the_lower_expert(cuda_device):
    import mok
    logits = torch.zeros(512, 64, device=cuda_device)
    logits[:, 40] = 1.0
    e, w = mok.ops.router_topk(logits, 4)
    assert (e.cpu() == torch.tensor([40, 0, 1, 2])).all()
    ref = torch.softmax(torch.tensor([1.0, 0.0, 0.0, 0.0]), 0)
    assert (w.cpu() - ref).abs().max() < 1e-6


def test_router_autograd(cuda_device):
    import mok
    logits = torch.randn(512, 64, device=cuda_device, requires_grad=True)
    e, w = mok.functional.route(logits, 6)
    dw = torch.randn_like(w)
    (w * dw).sum().backward()
    ref_logits = logits.detach().clone().requires_grad_(True)
    (torch.softmax(torch.gather(ref_logits, 1, e), dim=-1) * dw).sum().backward()
    assert (logits.grad - ref_logits.grad).abs().max() < 1e-5


def test_route_and_schedule_equals_build_schedule(cuda_device, single_rank_group):
    import mok
    F = mok.functional
    T, E, K = 1024, 16, 4
    cfg = F.MoKConfig(minibatch_size=256, macrobatch_size=8192, schedule_capacity_multiplier=4.0,
                      all_gather_top_experts_chunk_bytes=16)
    ws = F.get_workspace(cfg, single_rank_group, device=cuda_device, num_local_tokens=T, hidden_size=256, topk=K)
    logits = torch.randn(T, E, device=cuda_device)
    sched, experts, weights = F.route_and_schedule(ws, cfg, logits, num_local_experts=E)
    ref = F.build_schedule(ws, cfg, experts, num_local_experts=E)
    n = int(ref.num_tokens.item())
    assert torch.equal(sched.num_tokens, ref.num_tokens) and torch.equal(sched.tokens_per_expert, ref.tokens_per_expert)
    assert torch.equal(sched.peer_rank[:n], ref.peer_rank[:n])
    valid = ref.peer_rank[:n] >= 0
    assert torch.equal(sched.peer_token_idx[:n][valid], ref.peer_token_idx[:n][valid])
    e2, w2 = F.route(logits, K)
    assert torch.equal(e2, experts) and torch.equal(w2, weights)
    assert torch.equal(ws.all_gather_top_experts_buffer[0], experts.to(torch.int32))
