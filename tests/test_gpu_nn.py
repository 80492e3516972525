"""GPU tests of the trainer-facing wrappers: the autograd function and MoKLayer against the CPU oracle, the
complete path traced by torch.compile(fullgraph=True), and CUDA-graph capture of schedule -> forward -> backward."""
import pytest
import torch

from oracle import mok_oracle as O
from tests.helpers import BF16_REL_L2, MXFP8_REL_L2, rel_l2

pytestmark = pytest.mark.gpu

CFG = dict(T=1024, H=512, I=512, E=8, W=1, K=4)


def make_layer(dev, group, inp, *, mxfp8=False):
    import mok
    cfg = mok.functional.MoKConfig(minibatch_size=256, macrobatch_size=131072, schedule_capacity_multiplier=2.0,
                                   all_gather_top_experts_chunk_bytes=16)
    layer = mok.nn.MoKLayer(CFG["H"], CFG["I"], CFG["E"], CFG["K"], group=group, config=cfg, mxfp8=mxfp8, device=dev, seed=3)
    with torch.no_grad():
        for name in ("shared_gate", "shared_up", "shared_down", "routed_gate", "routed_up", "routed_down"):
            getattr(layer, name).copy_(getattr(inp, "w_" + name))
    return layer


@pytest.mark.parametrize("mxfp8", [False, True])
def test_layer_module_gradients_match_oracle(cuda_device, single_rank_group, mxfp8):
    inp = O.make_rank_inputs(0, seed=31, **CFG)
    ref = O.layer_forward_backward([inp], device_rounding=True, mxfp8=mxfp8)[0]
    layer = make_layer(cuda_device, single_rank_group, inp, mxfp8=mxfp8)
    x = inp.x.to(cuda_device).requires_grad_(True)
    rw = inp.router_weights.to(cuda_device).requires_grad_(True)
    out = layer(x, inp.topk_experts.to(cuda_device), rw)
    out.backward(inp.d_output.to(cuda_device))
    tol = MXFP8_REL_L2 if mxfp8 else BF16_REL_L2
    assert rel_l2(ref["output"].float(), out.float()) < tol
    assert rel_l2(ref["d_x"].float(), x.grad.float()) < tol
    assert rel_l2(ref["d_router_weights"].float(), rw.grad.float()) < tol
    for name in ("shared_gate", "shared_up", "shared_down", "routed_gate", "routed_up", "routed_down"):
        assert rel_l2(ref["d_w_" + name].float(), getattr(layer, name).grad.float()) < tol, name


def test_layer_module_with_its_own_router(cuda_device, single_rank_group):
    """layer(x) = router GEMM -> router kernel -> schedule -> experts; the router weight receives the gradient the
    chain rule gives from d_router_weights."""
    import mok
    inp = O.make_rank_inputs(0, seed=32, **CFG)
    layer = make_layer(cuda_device, single_rank_group, inp)
    x = inp.x.to(cuda_device)
    d_out = inp.d_output.to(cuda_device)
    out = layer(x)
    out.backward(d_out)
    logits = torch.nn.functional.linear(x, layer.router_weight.detach().to(x.dtype)).float()
    experts, weights = mok.functional.route(logits, CFG["K"])
    x2 = x.clone().requires_grad_(True)
    w2 = weights.clone().requires_grad_(True)
    layer.zero_grad()
    out2 = layer(x2, experts, w2)
    assert torch.equal(out, out2)
    router_grad = None
    out2.backward(d_out)
    d_logits = mok.ops.router_topk_bwd(experts, weights, w2.grad, CFG["E"])
    expect = (d_logits.to(x.dtype).float().t() @ x.float())
    layer.zero_grad()
    layer(x).backward(d_out)
    router_grad = layer.router_weight.grad
    assert rel_l2(expect, router_grad.float()) < 2e-2


def test_quantised_weights_follow_the_masters(cuda_device, single_rank_group):
    inp = O.make_rank_inputs(0, seed=33, **CFG)
    layer = make_layer(cuda_device, single_rank_group, inp, mxfp8=True)
    q1 = layer.quantised()
    assert layer.quantised() is q1
    with torch.no_grad():
        layer.routed_up.mul_(0.5)
    q2 = layer.quantised()
    assert q2 is not q1 and not torch.equal(q1.fwd[1][1], q2.fwd[1][1])


def _fake_workspace(F, dev, T, H, K, ep_size, cap):
    ptrs = list(range(1, ep_size + 1))
    t = lambda shape, dtype: torch.empty(shape, device=dev, dtype=dtype)    # noqa: E731
    return F.MoKWorkspace(
        group_name="fake", ep_rank=0, ep_size=ep_size, device=dev, num_local_tokens=T, hidden_size=H, topk=K,
        schedule_capacity=cap,
        x_buffer=t((T, H), torch.bfloat16), x_buffer_handle=None, x_buffer_ptrs=ptrs,
        combine_buffer=t((T * K, H), torch.bfloat16), combine_buffer_handle=None, combine_buffer_ptrs=ptrs,
        d_y_buffer=t((T, H), torch.bfloat16), d_y_buffer_handle=None, d_y_buffer_ptrs=ptrs,
        d_x_routed_buffer=t((T * K, H), torch.bfloat16), d_x_routed_buffer_handle=None, d_x_routed_buffer_ptrs=ptrs,
        router_weight_buffer=t((T, K), torch.float32), router_weight_buffer_handle=None, router_weight_buffer_ptrs=ptrs,
        d_router_weight_buffer=t((T, K), torch.float32), d_router_weight_buffer_handle=None,
        d_router_weight_buffer_ptrs=ptrs,
        all_gather_top_experts_buffer=t((ep_size, T, K), torch.int32), all_gather_top_experts_buffer_handle=None,
        all_gather_top_experts_buffer_multicast_ptr=0,
        barrier_buffer=t((1,), torch.int32), barrier_buffer_handle=None, barrier_buffer_ptrs=ptrs,
        barrier_buffer_multicast_ptr=0, barrier_target=t((1,), torch.int32))


@pytest.mark.parametrize("ep_size", [1, 4])
@pytest.mark.parametrize("precision", ["bf16", "mxfp8"])
def test_compile_fullgraph_traces_the_complete_path(cuda_device, ep_size, precision):
    """build_schedule -> forward -> backward is one graph of opaque operators under torch.compile(fullgraph=True),
    traced on fake tensors (nothing is launched), as the reference's tests/test_misc.py:1046-1305 requires."""
    import mok
    from torch._subclasses.fake_tensor import FakeTensorMode
    F, ops = mok.functional, mok.ops
    T, H, I, El, K = 512, 1024, 256, 4, 2
    cfg = F.MoKConfig(minibatch_size=256, macrobatch_size=512 if ep_size > 1 else 4096)
    graphs = []

    def backend(gm, _inputs):
        graphs.append(gm)
        return gm.forward

    with FakeTensorMode():
        t = lambda shape, dtype=torch.bfloat16: torch.empty(shape, device=cuda_device, dtype=dtype)   # noqa: E731
        ws = _fake_workspace(F, cuda_device, T, H, K, ep_size, 4096)

        def complete_path(x, top_experts, rw, d_out, sg, su, sd, rg, ru, rd):
            sched = F.build_schedule(ws, cfg, top_experts, num_local_experts=El)
            if precision == "bf16":
                fw = bw = (rg, ru, rd)
            else:
                qg, qu, qd = (ops.mxfp8_quantize(w, True, True) for w in (rg, ru, rd))
                fw = ((qg[0], qg[1]), (qu[0], qu[1]), (qd[0], qd[1]))
                bw = (tuple(qg), tuple(qu), (qd[2], qd[3]))
            out, ctx = F.forward(cfg, ws, sched, x, rw, sg, su, sd, *fw)
            return (out, *F.backward(cfg, ws, sched, ctx, d_out, x, rw, sg, su, sd, *bw))

        res = torch.compile(complete_path, fullgraph=True, backend=backend)(
            t((T, H)), t((T, K), torch.int64), t((T, K), torch.float32), t((T, H)),
            t((I, H)), t((I, H)), t((H, I)), t((El, I, H)), t((El, I, H)), t((El, H, I)))
    assert len(graphs) == 1
    shapes = [tuple(r.shape) for r in res]
    assert shapes == [(T, H), (T, H), (T, K), (El, I, H), (El, I, H), (El, H, I), (I, H), (I, H), (H, I)]
    names = {n.target.__name__ if hasattr(n.target, "__name__") else str(n.target) for n in graphs[0].graph.nodes
             if n.op == "call_function"}
    assert any("dispatch_mlp_swiglu_combine_fwd" in s for s in map(str, names))


def test_cuda_graph_replay_is_bit_identical(cuda_device, single_rank_group):
    """schedule -> forward -> backward captured once in a CUDA graph gives, on replay, the bytes of the eager call."""
    import mok
    F = mok.functional
    inp = O.make_rank_inputs(0, seed=34, **CFG)
    cfg = F.MoKConfig(minibatch_size=256, macrobatch_size=131072, schedule_capacity_multiplier=2.0,
                      all_gather_top_experts_chunk_bytes=16)
    ws = F.get_workspace(cfg, single_rank_group, device=cuda_device, num_local_tokens=CFG["T"], hidden_size=CFG["H"],
                         topk=CFG["K"])
    d = lambda v: v.to(cuda_device)          # noqa: E731
    x, rw, top, d_out = d(inp.x), d(inp.router_weights), d(inp.topk_experts), d(inp.d_output)
    w = [d(v) for v in (inp.w_shared_gate, inp.w_shared_up, inp.w_shared_down, inp.w_routed_gate, inp.w_routed_up,
                        inp.w_routed_down)]

    def step():
        sched = F.build_schedule(ws, cfg, top, num_local_experts=CFG["E"])
        out, ctx = F.forward(cfg, ws, sched, x, rw, *w)
        return (out, *F.backward(cfg, ws, sched, ctx, d_out, x, rw, *w))

    eager = [v.clone() for v in step()]
    side = torch.cuda.Stream(cuda_device)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = step()
    for v in captured:
        v.zero_()
    graph.replay()
    torch.cuda.synchronize()
    for a, b in zip(eager, captured):
        assert torch.equal(a, b)
    assert mok.last_status(cuda_device)[0] == 0
