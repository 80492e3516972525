"""Benchmark of the MoE-layer hot path (schedule -> dispatch -> grouped SwiGLU FFN -> combine).

    python bench.py --gpus N --steps K --warmup W [--impl reference]

N = 1   workload "C2": BF16 forward, EP=1, T=16384 tokens, hidden 2048, 128 experts, top-8,
        intermediate 768 (router: x @ W_r^T, W_r ~ N(0, 0.02), softmax, top-8, renormalise).
        A step = build_schedule + forward, as the reference times its forward
        (benchmarks/bench_mok.py:56-57 in Mixture-of-Kittens).
N > 1   workload "C3": BF16 forward + backward, EP=N, 16384 tokens per rank, hidden 4096,
        64 experts split over the ranks, top-6, intermediate 1536, uniform-random router logits,
        minibatch 4096, macrobatch 131072.  Launched by torchrun, one rank per GPU; NCCL only
        bootstraps the process group and the symmetric-memory rendezvous.

One JSON line is printed by rank 0.  `value` is TFLOP/s summed over the N GPUs with inputs
resident in HBM, FLOPs counted as the reference does (6*(T + T*K)*H*I forward, 3x that for
forward+backward, padding and replay not counted).  `e2e` is the same metric through
mok.functional with the step's inputs copied from pinned host memory and its results copied back
inside the timed region.  `roofline` describes the dominant kernel (the routed gate|up grouped
GEMM with fused SwiGLU) from CUDA events recorded around its launches inside the timed region.
`cpu_baseline` / `--impl reference` time the CPU oracle (a port of the reference's pure-PyTorch
test oracle) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "mixture-of-kittens_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

METRIC = "MoE layer TFLOP/s (reference FLOP convention), BF16"
UNIT = "TFLOP/s"

WORKLOADS = {
    "C2": dict(T=16384, H=2048, I=768, E=128, K=8, router="linear", backward=False,
               minibatch=4096, macrobatch=262144, multiplier=0.5,
               desc="BF16 forward, EP=1, T=16384, H=2048, E=128, top-8, I=768"),
    "C3": dict(T=16384, H=4096, I=1536, E=64, K=6, router="uniform", backward=True,
               minibatch=4096, macrobatch=131072, multiplier=0.5,
               desc="BF16 fwd+bwd, 16384 tokens/rank, H=4096, 64 experts, top-6, I=1536"),
    # MXFP8 shapes of BASELINE config 4 (EP=8: 256 experts, 32 per GPU).  "C4x1" keeps one GPU's share
    # (32 local experts, all 16384*8 routes local) so the per-GPU work of C4 can be measured on one GPU.
    "C4": dict(T=16384, H=7168, I=2048, E=256, K=8, router="linear", backward=True, mxfp8=True,
               minibatch=4096, macrobatch=131072, multiplier=0.5,
               desc="MXFP8 fwd+bwd, 16384 tokens/rank, H=7168, 256 experts, top-8, I=2048"),
    # skewed-routing stress (BASELINE config 5): C4 shapes, expert popularity ~ Zipf(1.2) laid out so that one rank
    # receives about 35 % of the routes, schedule_capacity_multiplier 1.0
    "C5": dict(T=16384, H=7168, I=2048, E=256, K=8, router="linear", backward=True, mxfp8=True, zipf=1.2,
               minibatch=4096, macrobatch=131072, multiplier=1.0,
               desc="MXFP8 fwd+bwd, C4 shapes, Zipf(1.2) expert popularity, capacity multiplier 1.0"),
    "C5-bf16": dict(T=16384, H=7168, I=2048, E=256, K=8, router="linear", backward=True, zipf=1.2,
                    minibatch=4096, macrobatch=131072, multiplier=1.0,
                    desc="BF16 fwd+bwd, C4 shapes, Zipf(1.2) expert popularity, capacity multiplier 1.0"),
    "C4x1": dict(T=16384, H=7168, I=2048, E=32, K=8, router="linear", backward=True, mxfp8=True,
                 minibatch=4096, macrobatch=131072, multiplier=0.5,
                 desc="MXFP8 fwd+bwd, one GPU's share of C4: 16384 tokens, H=7168, 32 local experts, top-8, I=2048"),
    "C4x1-bf16": dict(T=16384, H=7168, I=2048, E=32, K=8, router="linear", backward=True,
                      minibatch=4096, macrobatch=131072, multiplier=0.5,
                      desc="BF16 fwd+bwd at the C4x1 shapes"),
}
# DRAM bytes per launch of the dominant kernel from the ncu capture summarised under profiles/
# (filled in per workload once captured; None = not captured)
# C2: routed gate|up GEMM captured at 2048 tokens (951 MB read + 137 MB written, of which 805 MB are the weights,
# read once whatever the row count) and scaled by rows to the full launch: 0.805e9 + 147456 rows * 8640 B
NCU_TRAFFIC_BYTES = {"C2": 2.08e9, "C3": None}


def layer_flops(T, K, H, I, backward):
    f = 6.0 * (T + T * K) * H * I
    return 3.0 * f if backward else f


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            d = json.load(fh)
        return dict(tflops=float(d["bf16_tflops_sustained"]), burst=float(d["bf16_tflops"]),
                    hbm=float(d["hbm_gbs"]), source="measured")
    except Exception:
        return dict(tflops=1400.0, burst=1590.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples during the timed region (reading only)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc = index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [s for s in sm if s > 0.5 * max(sm)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def make_inputs(wl, rank, world, dev):
    """Seeded synthetic inputs: per-step tensors in pinned host memory, parameters on the device."""
    T, H, I, E, K = wl["T"], wl["H"], wl["I"], wl["E"], wl["K"]
    El = E // world
    g = torch.Generator(device=dev).manual_seed(1000 * 0 + rank)           # seed 0, offset by rank
    x = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
    if wl["router"] == "linear":
        w_r = torch.randn(E, H, generator=g, device=dev) * 0.02
        logits = x.float() @ w_r.T
    else:
        logits = torch.rand(T, E, generator=g, device=dev)
    if wl.get("zipf"):
        # expert -> popularity rank: the four most popular experts sit on rank 0 and the others are dealt round-robin
        # over the ranks, which puts about 35 % of all routes on rank 0 at EP=8 (36.6 % measured for these shapes)
        hot = min(4, El)
        rest = sorted(range(hot, E), key=lambda i: ((i % El) if i >= El else (i - hot) + 0.5, i // El))
        zipf_rank = torch.empty(E, dtype=torch.long)
        zipf_rank[:hot] = torch.arange(1, hot + 1)
        zipf_rank[torch.tensor(rest)] = torch.arange(hot + 1, E + 1)
        p = zipf_rank.to(dev).float() ** (-wl["zipf"])
        logits = logits + torch.log(p / p.sum())
    vals, idx = torch.topk(torch.softmax(logits, dim=-1), K, dim=-1)
    rw = (vals / vals.sum(-1, keepdim=True)).float()
    d_out = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
    mk = lambda *s, fan: (torch.randn(*s, generator=g, device=dev) * fan ** -0.5).to(torch.bfloat16)  # noqa: E731
    params = [mk(I, H, fan=H), mk(I, H, fan=H), mk(H, I, fan=I),
              mk(El, I, H, fan=H), mk(El, I, H, fan=H), mk(El, H, I, fan=I)]
    host = {k: v.cpu().pin_memory() for k, v in dict(x=x, topk=idx.to(torch.int64), rw=rw, d_out=d_out).items()}
    return host, params


def run_ours(args, rank, world, local_rank):
    import mok
    F, L = mok.functional, mok._lib
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if not dist.is_initialized():
        if world > 1:
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        else:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29560")
            dist.init_process_group("gloo", rank=0, world_size=1)
    name = args.workload if args.workload != "auto" else ("C2" if world == 1 else "C3")
    wl = dict(WORKLOADS[name])
    if args.tokens:                      # smaller copy of the workload (profiler captures); never a bench value
        wl["T"] = args.tokens
        wl["desc"] += f" [reduced to {args.tokens} tokens per rank]"
    T, H, I, E, K = wl["T"], wl["H"], wl["I"], wl["E"], wl["K"]
    El = E // world
    cfg = F.MoKConfig(minibatch_size=wl["minibatch"], macrobatch_size=wl["macrobatch"],
                      schedule_capacity_multiplier=wl["multiplier"])
    ws = F.get_workspace(cfg, dist.group.WORLD, device=dev, num_local_tokens=T, hidden_size=H, topk=K)
    host, params = make_inputs(wl, rank, world, dev)
    dev_in = {k: v.to(dev) for k, v in host.items()}
    # share of all routes that lands on the busiest rank (1/world when balanced)
    dest = torch.bincount((dev_in["topk"] // El).flatten(), minlength=world).double()
    if world > 1:
        dist.all_reduce(dest)
    max_rank_share = (dest.max() / dest.sum()).item()
    out_host = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()
    dx_host = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()
    drw_host = torch.empty(T, K, dtype=torch.float32).pin_memory()

    fwd_params = bwd_params = params
    if wl.get("mxfp8"):                  # routed weights quantised once, outside the timed region (as the reference does)
        qg, qu, qd = (mok.ops.mxfp8_quantize(w, True, True) for w in params[3:])
        fwd_params = params[:3] + [(qg[0], qg[1]), (qu[0], qu[1]), (qd[0], qd[1])]
        bwd_params = params[:3] + [tuple(qg), tuple(qu), (qd[2], qd[3])]
        params[3:] = []                  # the bf16 masters are not needed any more

    def step(inp):
        sched = F.build_schedule(ws, cfg, inp["topk"], num_local_experts=El)
        out, ctx = F.forward(cfg, ws, sched, inp["x"], inp["rw"], *fwd_params)
        if wl["backward"]:
            grads = F.backward(cfg, ws, sched, ctx, inp["d_out"], inp["x"], inp["rw"], *bwd_params)
            return out, grads
        return out, None

    # End-to-end step: inputs start in pinned host memory and results end there, every step.  The copies
    # are double-buffered on their own streams: the inputs of step i+1 are uploaded while step i computes
    # and the results of step i are downloaded while step i+1 computes; the host reads a step's results
    # one step later (it synchronises on that step's download).
    e2e_keys = [k for k in host if k != "d_out" or wl["backward"]]
    h2d_stream, d2h_stream = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    slots = [{k: torch.empty_like(host[k], device=dev) for k in e2e_keys} for _ in range(2)]
    uploaded = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    downloaded = [torch.cuda.Event() for _ in range(2)]
    state = {"i": 0, "primed": False}

    def upload(slot):
        with torch.cuda.stream(h2d_stream):
            h2d_stream.wait_event(consumed[slot])          # the previous user of this slot has finished
            for k in e2e_keys:
                slots[slot][k].copy_(host[k], non_blocking=True)
            uploaded[slot].record(h2d_stream)

    def step_e2e():
        i = state["i"]
        slot = i & 1
        main = torch.cuda.current_stream()
        if not state["primed"]:
            consumed[0].record(main); consumed[1].record(main)
            upload(slot)
            state["primed"] = True
        upload(slot ^ 1)                                   # prefetch the next step's inputs
        main.wait_event(uploaded[slot])
        out, grads = step(slots[slot])
        consumed[slot].record(main)
        with torch.cuda.stream(d2h_stream):
            d2h_stream.wait_event(consumed[slot])
            out_host.copy_(out, non_blocking=True)
            out.record_stream(d2h_stream)
            if grads is not None:
                dx_host.copy_(grads[0], non_blocking=True)
                drw_host.copy_(grads[1], non_blocking=True)
                grads[0].record_stream(d2h_stream); grads[1].record_stream(d2h_stream)
            downloaded[slot].record(d2h_stream)
        if i > 0:
            downloaded[slot ^ 1].synchronize()             # the caller reads the previous step's results
        state["i"] = i + 1

    def drain_e2e():
        i = state["i"]
        if i > 0:
            torch.cuda.current_stream().wait_event(downloaded[(i - 1) & 1])
            torch.cuda.current_stream().wait_event(uploaded[i & 1])

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize()

    def timed(fn, steps, finish=None):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        if finish is not None:
            finish()
        b.record()
        barrier()
        ms = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() / steps

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(max(args.warmup, 3)):
        step(dev_in)
    torch.cuda.synchronize()
    mok.raise_for_status(dev)
    launches0 = L.mok_launch_count()
    ms_step = timed(lambda: step(dev_in), args.steps)
    launches = L.mok_launch_count() - launches0
    # the same K steps again with a CUDA-event pair around every launch: the per-kernel split behind `roofline`
    # (the event records cost a little, so `value` comes from the region above)
    L.mok_profile_enable(1)
    L.profile_collect()
    ms_step_events = timed(lambda: step(dev_in), args.steps)
    prof = L.profile_collect()
    L.mok_profile_enable(0)
    ms_graph = None
    if args.graph and world == 1:        # the same step captured once and replayed as a CUDA graph
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step(dev_in)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            graph_out = step(dev_in)
        graph.replay()
        torch.cuda.synchronize()
        eager_out = step(dev_in)
        assert torch.equal(graph_out[0], eager_out[0]), "graph replay differs from the eager step"
        ms_graph = timed(graph.replay, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    # rows this rank's schedule holds against the routes it received (expert groups are padded to 256 rows)
    sched0 = F.build_schedule(ws, cfg, dev_in["topk"], num_local_experts=El)
    n_rows = int(sched0.num_tokens.item())
    n_routes = int((sched0.peer_rank[:min(n_rows, sched0.peer_rank.numel())] >= 0).sum().item())
    out_a, _ = step(dev_in)
    out_b, _ = step(dev_in)
    rerun_identical = bool(torch.equal(out_a, out_b))

    for _ in range(3):
        step_e2e()
    drain_e2e()
    ms_e2e = timed(step_e2e, args.steps, finish=drain_e2e)
    mok.raise_for_status(dev)

    flops = layer_flops(T, K, H, I, wl["backward"])
    peaks = measured_peaks()
    if wl.get("mxfp8"):                  # no measured MXFP8 peak on file: twice the measured bf16 figures
        peaks = dict(peaks, tflops=2 * peaks["tflops"], burst=2 * peaks["burst"], source=peaks["source"] + " x2 for fp8")
    dom = "gemm_gate_up_swiglu_routed"
    dom_ms, dom_cnt = prof.get(dom, (0.0, 0))
    dom_ms_step = dom_ms / args.steps if dom_cnt else None
    dom_flops = 4.0 * T * K * H * I      # gate + up GEMMs over the T*K routed rows (padding not counted)
    achieved = dom_flops / (dom_ms_step * 1e-3) / 1e12 if dom_ms_step else None
    if rank != 0:
        return
    h2d = sum(v.numel() * v.element_size() for k, v in host.items() if k != "d_out" or wl["backward"])
    d2h = out_host.numel() * 2 + ((dx_host.numel() * 2 + drw_host.numel() * 4) if wl["backward"] else 0)
    line = {
        "metric": METRIC, "value": world * flops / (ms_step * 1e-3) / 1e12, "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "mxfp8 (e4m3 x e8m0, fp32 accumulate)" if wl.get("mxfp8") else "bf16", "data": "synthetic",
        "config": {"workload": f"{name}: {wl['desc']}", "ep_size": world, "tokens_per_rank": T, "hidden": H,
                   "intermediate": I, "experts": E, "topk": K, "minibatch_size": wl["minibatch"],
                   "macrobatch_size": wl["macrobatch"], "capacity_multiplier": wl["multiplier"],
                   "busiest_rank_share_of_routes": max_rank_share, "pass": "fwd+bwd" if wl["backward"] else "fwd (incl. build_schedule)",
                   "rank0_schedule_rows": n_rows, "rank0_routes": n_routes,
                   "padding_overhead": (n_rows / n_routes - 1.0) if n_routes else None,
                   "rerun_bit_identical": rerun_identical,
                   "ms_per_step_with_kernel_events": ms_step_events,
                   "l2": "inputs larger than L2 (no flush needed)", "per_gpu_tflops": flops / (ms_step * 1e-3) / 1e12,
                   "pct_of_measured_bf16_peak": 100.0 * flops / (ms_step * 1e-3) / 1e12 / peaks["tflops"]},
        "e2e": {"value": world * flops / (ms_e2e * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": {"kernel": dom, "bound": "tensor", "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s",
                     "frac": (achieved / peaks["tflops"]) if achieved else None, "traffic": NCU_TRAFFIC_BYTES.get(name),
                     "peak_source": f"{peaks['source']}: bf16_tflops_sustained (kernel timed inside a long step); burst {peaks['burst']}",
                     "launches_per_step": dom_cnt / args.steps if dom_cnt else 0,
                     "ms_per_step": dom_ms_step},
        "kernel_ms_per_step": {k: v[0] / args.steps for k, v in sorted(prof.items())},
    }
    if ms_graph is not None:
        line["cuda_graph"] = {"ms_per_step": ms_graph, "value": flops / (ms_graph * 1e-3) / 1e12, "unit": UNIT,
                              "note": "the same step captured once with torch.cuda.graph and replayed"}
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(name, steps=1)
    print(json.dumps(line), flush=True)


def cpu_baseline(name, steps=1, sample_tokens=None):
    """The CPU oracle on a bounded sample of the workload: same H, I, E, K and router law, fewer
    tokens per rank, single process, all host threads."""
    from oracle import mok_oracle as O
    wl = WORKLOADS[name]
    W = 1
    T = sample_tokens or (min(wl["T"], 16384) if not wl["backward"] else 4096)   # about 3-10 s of CPU work per step
    cfgs = dict(T=T, H=wl["H"], I=wl["I"], E=wl["E"], W=W, K=wl["K"], seed=0, router=wl["router"],
                with_grad=wl["backward"])
    ranks = [O.make_rank_inputs(r, **cfgs) for r in range(W)]
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        O.layer_forward_backward(ranks, device_rounding=True, backward=wl["backward"])
        times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    fl = W * layer_flops(T, wl["K"], wl["H"], wl["I"], wl["backward"])
    return {"value": fl / sec / 1e12, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{T} tokens (of {wl['T']}) on one virtual rank, all {wl['E']} experts local, "
                      f"{'fwd+bwd' if wl['backward'] else 'fwd'}, {sec:.2f} s per step", "seconds_per_step": sec}


class TorchMoE:
    """GPU-side library baseline for the same layer: routes sorted by expert, NCCL all_to_all_single for dispatch and
    combine, torch._grouped_mm for the expert GEMMs, autograd for the backward (BF16 only).  What a user would write
    in plain PyTorch; the counterpart of the reference's benchmarks/bench_nccl_torch.py.  Its splits need one host
    synchronisation per step (all_to_all_single takes Python lists)."""

    def __init__(self, params, topk, world):
        self.sg, self.su, self.sd, self.rg, self.ru, self.rd = params
        self.K, self.W, self.El = topk, world, params[3].shape[0]

    def _a2a(self, rows, out_splits, in_splits):
        if self.W == 1:
            return rows
        import torch.distributed.nn.functional as dnn
        out = rows.new_empty(sum(out_splits), rows.shape[1])
        return dnn.all_to_all_single(out, rows, out_splits, in_splits)

    def forward(self, x, top_experts, router_weights):
        T, H = x.shape
        K, W, El = self.K, self.W, self.El
        flat = top_experts.flatten()
        order = torch.argsort(flat, stable=True)                     # routes by expert, hence by destination rank
        counts = torch.bincount(flat, minlength=W * El)
        recv_counts = counts
        if W > 1:
            recv_counts = torch.empty_like(counts)
            dist.all_to_all_single(recv_counts, counts)               # [src rank, local expert]
        send_splits = counts.view(W, El).sum(1).tolist()
        recv_splits = recv_counts.view(W, El).sum(1).tolist()
        recv = self._a2a(x[order // K], recv_splits, send_splits)
        # rows arrive ordered by (source rank, expert): regroup them expert-major for the grouped GEMM
        ids = torch.repeat_interleave(torch.arange(El, device=x.device).repeat(W), recv_counts)
        perm = torch.argsort(ids, stable=True)
        offs = torch.cumsum(recv_counts.view(W, El).sum(0), 0).to(torch.int32)
        grouped = recv[perm]
        gate = torch._grouped_mm(grouped, self.rg.transpose(1, 2), offs=offs)
        up = torch._grouped_mm(grouped, self.ru.transpose(1, 2), offs=offs)
        y = torch._grouped_mm(torch.nn.functional.silu(gate) * up, self.rd.transpose(1, 2), offs=offs)
        back = torch.empty_like(y).index_copy(0, perm, y)
        ret = self._a2a(back, send_splits, recv_splits)
        flat_out = torch.empty_like(ret).index_copy(0, order, ret)
        shared = (torch.nn.functional.silu(x @ self.sg.T) * (x @ self.su.T)) @ self.sd.T
        routed = (router_weights.unsqueeze(-1) * flat_out.view(T, K, H).float()).sum(1)
        return (shared.float() + routed).to(torch.bfloat16)


def run_torch(args, rank, world, local_rank):
    """--impl torch: the TorchMoE baseline on the GPUs, same workload, inputs and timing rules as the product arm."""
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    name = args.workload if args.workload != "auto" else ("C2" if world == 1 else "C3")
    wl = dict(WORKLOADS[name])
    if wl.get("mxfp8"):
        if rank == 0:
            print(json.dumps({"impl": "torch", "unavailable": "the PyTorch baseline is BF16 only"}), flush=True)
        return
    if args.tokens:
        wl["T"] = args.tokens
    T, H, I, K = wl["T"], wl["H"], wl["I"], wl["K"]
    host, params = make_inputs(wl, rank, world, dev)
    inp = {k: v.to(dev) for k, v in host.items()}
    leaves = [p.requires_grad_(wl["backward"]) for p in params]
    x = inp["x"].requires_grad_(wl["backward"])
    rw = inp["rw"].requires_grad_(wl["backward"])
    moe = TorchMoE(leaves, K, world)

    def step():
        out = moe.forward(x, inp["topk"], rw)
        if wl["backward"]:
            return out, torch.autograd.grad(out, [x, rw] + leaves, inp["d_out"])
        return out, None

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize()

    steps = args.steps
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        step()
    b.record()
    barrier()
    ms = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_step = ms.item() / steps
    if rank == 0:
        flops = layer_flops(T, K, H, I, wl["backward"])
        print(json.dumps({
            "impl": "torch", "metric": METRIC, "value": world * flops / (ms_step * 1e-3) / 1e12, "unit": UNIT,
            "n_gpus": world, "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{name}: {wl['desc']}", "ep_size": world,
                       "note": "library baseline: NCCL all_to_all_single + torch._grouped_mm + autograd; "
                               "none of this repository's kernels"},
            "gpu_launches": 0}), flush=True)


def run_reference(args, rank, world):
    """The reference arm: the reference's CPU implementation of the path (its pure-PyTorch test
    oracle, restated in oracle/) on the host cores, on a bounded sample per step."""
    if rank != 0:
        return
    name = args.workload if args.workload != "auto" else ("C2" if world == 1 else "C3")
    wl = WORKLOADS[name]
    steps = max(1, min(args.steps, 3))
    base = cpu_baseline(name, steps=steps)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": world,
        "steps": steps, "warmup": 0, "ms_per_step": base["seconds_per_step"] * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{name}: {wl['desc']}", "note": "CPU port of the reference's PyTorch oracle; "
                   "the reference's own sm_100 build needs ThunderKittens and CUDA 13, neither available offline"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"])
    ap.add_argument("--workload", default="auto", choices=["auto"] + sorted(WORKLOADS))
    ap.add_argument("--tokens", type=int, default=0, help="override tokens per rank (profiling a reduced case)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--graph", action="store_true", help="also time the step replayed as one CUDA graph (1 GPU)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("--gpus N with N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.impl == "torch":
        try:
            run_torch(args, rank, world, local_rank)
        finally:
            if dist.is_initialized():
                dist.destroy_process_group()
        return
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if dist.is_initialized():
            try:
                import mok
                mok.functional.clear_workspace_cache()
            except Exception:
                pass
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
