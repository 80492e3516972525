"""The plain-PyTorch GPU baseline of bench.py (all_to_all_single + torch._grouped_mm + autograd) and this
library's kernels compute the same layer: an independent GPU-side cross-check, on one rank."""
import pytest
import torch

from oracle import mok_oracle as O
from tests.helpers import BF16_REL_L2, rel_l2
from tests.test_gpu_layer import GRAD_NAMES, run_layer

pytestmark = pytest.mark.gpu


def test_torch_baseline_agrees_with_the_kernels(cuda_device, single_rank_group):
    import bench
    cfg = dict(T=1024, H=512, I=512, E=8, W=1, K=4)
    inp = O.make_rank_inputs(0, seed=41, **cfg)
    got = run_layer(cuda_device, single_rank_group, inp)
    d = lambda t: t.to(cuda_device).requires_grad_(True)       # noqa: E731
    x, rw = d(inp.x), d(inp.router_weights)
    w = [d(v) for v in (inp.w_shared_gate, inp.w_shared_up, inp.w_shared_down, inp.w_routed_gate, inp.w_routed_up,
                        inp.w_routed_down)]
    moe = bench.TorchMoE(w, cfg["K"], 1)
    out = moe.forward(x, inp.topk_experts.to(cuda_device), rw)
    grads = torch.autograd.grad(out, [x, rw] + w, inp.d_output.to(cuda_device))
    assert rel_l2(out.float(), got["output"].float()) < BF16_REL_L2
    names = ("d_x", "d_router_weights", "d_w_shared_gate", "d_w_shared_up", "d_w_shared_down", "d_w_routed_gate",
             "d_w_routed_up", "d_w_routed_down")
    assert set(names) == set(GRAD_NAMES)
    for name, g in zip(names, grads):
        assert rel_l2(g.float(), got[name].float()) < 2 * BF16_REL_L2, name
