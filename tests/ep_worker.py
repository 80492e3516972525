"""Multi-rank parity worker (one process per GPU, launched by torch.distributed.run).

Every rank rebuilds the seeded inputs of ALL ranks on the CPU, runs the oracle over the W virtual
ranks, then runs the real layer (build_schedule -> forward -> backward through mok.functional over
symmetric memory) and compares its own rank's results with the oracle's.  Exit code 0 = parity.
"""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "mixture-of-kittens_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

GRADS = ("d_x", "d_router_weights", "d_w_routed_gate", "d_w_routed_up", "d_w_routed_down",
         "d_w_shared_gate", "d_w_shared_up", "d_w_shared_down")


def rel(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    n = a.norm().item()
    return (a - b).norm().item() / (n if n > 0 else 1.0)


def main():
    import mok
    from oracle import mok_oracle as O
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    F = mok.functional
    cases = [dict(T=512, H=256, I=256, E=2 * world, K=2, limit=None, macro=131072, zipf=None, mx=False),
             dict(T=1024, H=512, I=512, E=4 * world, K=4, limit=1.0, macro=131072, zipf=None, mx=False),
             dict(T=512, H=256, I=256, E=2 * world, K=2, limit=None, macro=512, zipf=1.2, mx=False),
             dict(T=512, H=256, I=512, E=2 * world, K=2, limit=None, macro=131072, zipf=None, mx=True),
             dict(T=512, H=512, I=256, E=2 * world, K=3, limit=None, macro=512, zipf=1.2, mx=True)]
    worst, failures = 0.0, []
    for ci, c in enumerate(cases):
        shape = dict(T=c["T"], H=c["H"], I=c["I"], E=c["E"], W=world, K=c["K"], seed=40 + ci, zipf_s=c["zipf"])
        ranks = [O.make_rank_inputs(r, **shape) for r in range(world)]
        mult = 1.0                                # capacity = T*K*max(2, W): nothing can overflow
        cap = c["T"] * c["K"] * max(2, world)
        ref = O.layer_forward_backward(ranks, swiglu_limit=c["limit"], device_rounding=True, capacity=cap,
                                       mxfp8=c["mx"])[rank]
        tol = 3e-2 if c["mx"] else 1e-2
        cfg = F.MoKConfig(minibatch_size=256, macrobatch_size=c["macro"], schedule_capacity_multiplier=mult,
                          all_gather_top_experts_chunk_bytes=16)
        ws = F.get_workspace(cfg, dist.group.WORLD, device=dev, num_local_tokens=c["T"], hidden_size=c["H"], topk=c["K"])
        me = ranks[rank]
        d = lambda t: t.to(dev)  # noqa: E731
        w = [d(t) for t in (me.w_shared_gate, me.w_shared_up, me.w_shared_down, me.w_routed_gate, me.w_routed_up,
                            me.w_routed_down)]
        x, rw = d(me.x), d(me.router_weights)
        fw = bw = w
        if c["mx"]:
            qg, qu, qd = (mok.ops.mxfp8_quantize(t, True, True) for t in w[3:])
            fw = w[:3] + [(qg[0], qg[1]), (qu[0], qu[1]), (qd[0], qd[1])]
            bw = w[:3] + [tuple(qg), tuple(qu), (qd[2], qd[3])]
        outs = []
        for rep in range(2):                      # second pass: bit-identical
            sched = F.build_schedule(ws, cfg, d(me.topk_experts), num_local_experts=c["E"] // world)
            out, ctx = F.forward(cfg, ws, sched, x, rw, *fw, swiglu_limit=c["limit"])
            grads = F.backward(cfg, ws, sched, ctx, d(me.d_output), x, rw, *bw, swiglu_limit=c["limit"])
            torch.cuda.synchronize()
            outs.append((out, grads))
        code = mok.last_status(dev)[0]
        if code != 0:
            failures.append(f"case {ci}: status {mok.last_status(dev)}")
        for name, r_, g_ in zip(("peer_rank", "peer_token_idx", "num_tokens", "tokens_per_expert"),
                                (ref["peer_rank"], ref["peer_token_idx"], ref["num_tokens"], ref["tokens_per_expert"]),
                                (sched.peer_rank, sched.peer_token_idx, sched.num_tokens, sched.tokens_per_expert)):
            if not np.array_equal(r_, g_.cpu().numpy()):
                failures.append(f"case {ci}: schedule table {name} differs")
        e = rel(ref["output"].float(), outs[1][0].float())
        worst = max(worst, e)
        if e > tol:
            failures.append(f"case {ci}: output rel-L2 {e:.3e}")
        for name, g_ in zip(GRADS, outs[1][1]):
            e = rel(ref[name].float(), g_.float())
            worst = max(worst, e)
            if e > tol:
                failures.append(f"case {ci}: {name} rel-L2 {e:.3e}")
        if not torch.equal(outs[0][0], outs[1][0]) or any(not torch.equal(a, b) for a, b in zip(outs[0][1], outs[1][1])):
            failures.append(f"case {ci}: two runs differ bitwise")
    # router kernel writing the routes straight into every rank's all-gather buffer == cast + all-gather, and the
    # plain-PyTorch baseline (all_to_all_single + grouped_mm) computes the same layer as the kernels
    import bench
    c = cases[1]
    El = c["E"] // world
    me = O.make_rank_inputs(rank, T=c["T"], H=c["H"], I=c["I"], E=c["E"], W=world, K=c["K"], seed=77)
    cfg = F.MoKConfig(minibatch_size=256, macrobatch_size=c["macro"], schedule_capacity_multiplier=1.0,
                      all_gather_top_experts_chunk_bytes=16)
    ws = F.get_workspace(cfg, dist.group.WORLD, device=dev, num_local_tokens=c["T"], hidden_size=c["H"], topk=c["K"])
    w = [t.to(dev) for t in (me.w_shared_gate, me.w_shared_up, me.w_shared_down, me.w_routed_gate, me.w_routed_up,
                             me.w_routed_down)]
    x = me.x.to(dev)
    logits = torch.randn(c["T"], c["E"], generator=torch.Generator().manual_seed(900 + rank)).to(dev)
    sched_a, experts, weights = F.route_and_schedule(ws, cfg, logits, num_local_experts=El)
    sched_b = F.build_schedule(ws, cfg, experts, num_local_experts=El)
    n = int(sched_b.num_tokens.item())
    valid = sched_b.peer_rank[:n] >= 0
    same = (torch.equal(sched_a.num_tokens, sched_b.num_tokens) and torch.equal(sched_a.tokens_per_expert, sched_b.tokens_per_expert)
            and torch.equal(sched_a.peer_rank[:n], sched_b.peer_rank[:n])
            and torch.equal(sched_a.peer_token_idx[:n][valid], sched_b.peer_token_idx[:n][valid]))
    if not same:
        failures.append("route_and_schedule tables differ from build_schedule")
    out, _ = F.forward(cfg, ws, sched_b, x, weights, *w)
    # the nn.Module wrapper (backward runs on the autograd engine's worker thread of this rank's device) gives the
    # bytes of the functional calls
    d_out = me.d_output.to(dev)
    out, ctx = F.forward(cfg, ws, sched_b, x, weights, *w)
    ref_grads = F.backward(cfg, ws, sched_b, ctx, d_out, x, weights, *w)
    layer = mok.nn.MoKLayer(c["H"], c["I"], c["E"], c["K"], group=dist.group.WORLD, config=cfg, device=dev, seed=rank)
    with torch.no_grad():
        for name, t in zip(("shared_gate", "shared_up", "shared_down", "routed_gate", "routed_up", "routed_down"), w):
            getattr(layer, name).copy_(t)
    xg, wg = x.clone().requires_grad_(True), weights.clone().requires_grad_(True)
    out_l = layer(xg, experts, wg)
    out_l.backward(d_out)
    torch.cuda.synchronize()
    if not (torch.equal(out_l, out) and torch.equal(xg.grad, ref_grads[0]) and torch.equal(wg.grad, ref_grads[1])
            and torch.equal(layer.routed_down.grad, ref_grads[4]) and torch.equal(layer.shared_gate.grad, ref_grads[5])):
        failures.append("MoKLayer forward/backward differs from the functional calls")
    # inputs built directly in the rank-visible buffers: no staging copy, same bytes out
    ws.x_buffer.copy_(x)
    ws.router_weight_buffer.copy_(weights)
    out_zc, _ = F.forward(cfg, ws, sched_b, ws.x_buffer, ws.router_weight_buffer, *w)
    if not torch.equal(out, out_zc):
        failures.append("forward on the workspace buffers differs from forward on copies")
    out_t = bench.TorchMoE(w, c["K"], world).forward(x, experts, weights)
    e = rel(out_t.float(), out.float())
    worst = max(worst, e)
    if e > 1e-2:
        failures.append(f"torch baseline vs kernels: output rel-L2 {e:.3e}")
    if mok.last_status(dev)[0] != 0:
        failures.append(f"router/baseline section: status {mok.last_status(dev)}")
    F.clear_workspace_cache()
    # Two cases with the hidden / intermediate sizes, expert counts and top-k of the full-size training workloads
    # (BF16: H=4096, I=1536, 64 experts, top-6; MXFP8: H=7168, I=2048, 32 experts per rank, top-8) on fewer
    # tokens, windows cut into chunks with SMs set aside for the row movers.  The CPU oracle would take minutes at
    # these sizes, so sampled tokens are recomputed in fp32 on the device (bench.sampled_parity, itself pinned to
    # the oracle by a CPU test); every routed row of a sampled token comes back from the rank that owns its expert.
    shaped = [("bf16 H=4096", dict(T=1024, H=4096, I=1536, E=64, K=6, router="uniform", backward=True, minibatch=256,
                                   macrobatch=131072, multiplier=1.0), 24, 1e-2),
              ("mxfp8 H=7168", dict(T=512, H=7168, I=2048, E=32 * world, K=8, router="linear", backward=True, mxfp8=True,
                                    minibatch=256, macrobatch=131072, multiplier=1.0), 8, 3e-2)]
    for label, wl, samples, tol in shaped:
        run = bench.LayerRun(label, wl, rank, world, local, dist.group.WORLD)
        results = {}
        for n_sms in (None, 4, 52):                  # the configuration's default, the smallest and the largest swept
            if n_sms is not None:
                run.set_comm_sms(n_sms)
            out, grads, sched_s, ctx_s = run.step(keep=True)
            torch.cuda.synchronize()
            if n_sms is None:
                par = bench.sampled_parity(wl, rank, world, dev, run.dev_in, out, grads, sched_s, ctx_s, samples)
                for name, e in par.items():
                    worst = max(worst, e)
                    if not e < tol:
                        failures.append(f"{label}: {name} rel-L2 {e:.3e}")
            results[n_sms] = (out, grads)
            del sched_s, ctx_s
        for n_sms in (4, 52):
            same = torch.equal(results[None][0], results[n_sms][0]) and all(
                torch.equal(a, b) for a, b in zip(results[None][1], results[n_sms][1]))
            if not same:
                failures.append(f"{label}: results with {n_sms} communication SMs differ bitwise from the default")
        if mok.last_status(dev)[0] != 0:
            failures.append(f"{label}: status {mok.last_status(dev)}")
        del results
        run.release()
        F.clear_workspace_cache()
    flag = torch.tensor([len(failures)], device=dev)
    dist.all_reduce(flag)
    print(json.dumps({"rank": rank, "world": world, "worst_rel_l2": worst, "failures": failures}), flush=True)
    F.clear_workspace_cache()
    dist.destroy_process_group()
    sys.exit(1 if flag.item() else 0)


if __name__ == "__main__":
    main()
