"""Benchmark of the MoE-layer hot path (schedule -> dispatch -> grouped SwiGLU FFN -> combine).

    python bench.py --gpus N --steps K --warmup W [--impl reference|torch] [--workload NAME]

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
forward+backward, padding and replay not counted): K steps between two barriers, max over ranks.
The same region also carries one CUDA event per step, so the line adds the reference's own
statistic (benchmarks/utils.py:66-110 there: per-iteration maximum over ranks, then the median).
`e2e` is the same metric through mok.functional with the step's inputs copied from pinned host memory
and its results copied back inside the timed region.  `roofline` describes the dominant kernel (the
routed gate|up grouped GEMM with fused SwiGLU) from CUDA events recorded around its launches inside a
second pass over the same K steps.  `config.parity_rel_l2` is a check, made after the timed regions, of
sampled tokens of this very run against an fp32 recomputation with the device's rounding points (the
routed rows of those tokens live on other ranks when N > 1); the run exits non-zero when it fails.
`cpu_baseline` / `--impl reference` time the CPU oracle (a port of the reference's pure-PyTorch
test oracle) on a bounded sample of the same workload.  `--workload C1` times the small CPU
configuration (fp32 forward + backward, T=256, H=512, 8 experts, top-2, I=1024) on the host alone.
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
    "C1": dict(T=256, H=512, I=1024, E=8, K=2, router="linear", backward=True, cpu_only=True,
               minibatch=256, macrobatch=131072, multiplier=2.0,
               desc="fp32 fwd+bwd on the host CPU, one rank, T=256, H=512, 8 experts, top-2, I=1024"),
    "C2": dict(T=16384, H=2048, I=768, E=128, K=8, router="linear", backward=False,
               minibatch=4096, macrobatch=262144, multiplier=0.5,
               desc="BF16 forward, EP=1, T=16384, H=2048, E=128, top-8, I=768"),
    "C3": dict(T=16384, H=4096, I=1536, E=64, K=6, router="uniform", backward=True,
               minibatch=4096, macrobatch=131072, multiplier=0.5,
               desc="BF16 fwd+bwd, 16384 tokens/rank, H=4096, 64 experts, top-6, I=1536"),
    # one GPU's share of C3 at eight ranks with every row local (8 local experts): the per-GPU work of the
    # eight-rank run without any traffic between GPUs
    "C3x1": dict(T=16384, H=4096, I=1536, E=8, K=6, router="uniform", backward=True,
                 minibatch=4096, macrobatch=131072, multiplier=0.5,
                 desc="BF16 fwd+bwd, one GPU's share of C3 at EP=8: 16384 tokens, H=4096, 8 local experts, top-6, I=1536"),
    # MXFP8 training shapes at eight ranks: 256 experts, 32 per GPU.  "C4x1" keeps one GPU's share
    # (32 local experts, all 16384*8 routes local) so the per-GPU work of C4 can be measured on one GPU.
    "C4": dict(T=16384, H=7168, I=2048, E=256, K=8, router="linear", backward=True, mxfp8=True,
               minibatch=4096, macrobatch=131072, multiplier=0.5,
               desc="MXFP8 fwd+bwd, 16384 tokens/rank, H=7168, 256 experts, top-8, I=2048"),
    # skewed-routing stress: C4 shapes, expert popularity ~ Zipf(1.2) laid out so that one rank
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
# DRAM traffic of the dominant kernel: fixed bytes per local expert (its gate and up weights, read once per launch
# whatever the row count) and bytes per schedule row, from ncu captures of reduced cases
TRAFFIC_MODEL = os.path.join(ROOT, "profiles", "dominant_kernel_traffic.json")

BF16_REL_L2 = 1e-2     # parity bound for the BF16 path (output and gradients against the fp32 recomputation)
MXFP8_REL_L2 = 3e-2    # the same for the MXFP8 path, against the recomputation with block-quantised operands


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


def dominant_traffic(name, local_experts, rows):
    """Bytes one launch of the dominant kernel moves to and from DRAM, scaled from the reduced capture."""
    try:
        with open(TRAFFIC_MODEL) as fh:
            m = json.load(fh).get(name.replace("x1", ""))
    except Exception:
        return None
    if not m or rows is None:
        return None
    return m["fixed_bytes_per_local_expert"] * local_experts + m["bytes_per_schedule_row"] * rows


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


def bind_to_gpu_numa_node(local_rank: int):
    """Best effort, host side only (nothing is set on the GPU): run this rank's host thread on the CPUs next to its GPU
    and prefer that NUMA node for the memory it allocates from now on, so that the pinned buffers of the end-to-end
    step and their copies do not cross the socket link.  The GPU's node comes from sysfs (its PCI device) and the
    CPU list from NVML; a container whose CPU set excludes those CPUs keeps its affinity and only gets the memory
    preference.  Returns a short description of what was done."""
    done = {}
    try:
        import pynvml
        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
        bus = pynvml.nvmlDeviceGetPciInfo(handle).busId
        bus = (bus.decode() if isinstance(bus, bytes) else bus).lower()
        if len(bus.split(":")[0]) == 8:                     # NVML prints an 8-digit domain, sysfs a 4-digit one
            bus = bus[4:]
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as fh:
            node = int(fh.read().strip())
        done["gpu_numa_node"] = node
        try:
            words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
            cpus = {64 * i + b for i, w in enumerate(words) for b in range(64) if (w >> b) & 1} & os.sched_getaffinity(0)
            if cpus:
                os.sched_setaffinity(0, cpus)
                done["cpus_bound"] = len(cpus)
        except Exception:
            pass
        if node >= 0:
            import ctypes
            libc = ctypes.CDLL(None, use_errno=True)
            mask = ctypes.c_ulong(1 << node)
            MPOL_PREFERRED, SYS_set_mempolicy = 1, 238     # x86-64
            rc = libc.syscall(SYS_set_mempolicy, MPOL_PREFERRED, ctypes.byref(mask), ctypes.c_ulong(64))
            done["memory_preferred_node"] = node if rc == 0 else f"refused (errno {ctypes.get_errno()})"
    except Exception as e:                                  # no NVML, no sysfs entry, another architecture
        done["skipped"] = type(e).__name__
    return done


def make_inputs(wl, rank, world, dev, pinned=True):
    """Seeded synthetic inputs of one rank: per-step tensors (in pinned host memory, or on the device with
    pinned=False) and the parameters on the device."""
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
    step_in = dict(x=x, topk=idx.to(torch.int64), rw=rw, d_out=d_out)
    if pinned:
        step_in = {k: v.cpu().pin_memory() for k, v in step_in.items()}
    return step_in, params


# ----------------------------------------------------------------------------------------------------------
# parity of sampled tokens: fp32 recomputation on the device with the rounding points of the kernels
# ----------------------------------------------------------------------------------------------------------
def mx_quant_dequant(t: torch.Tensor, axis: int) -> torch.Tensor:
    """What an MXFP8 operand contributes numerically: fp32 values that are bf16-representable, quantised in
    blocks of 32 along `axis` (amax * (1/448) floored at 1e-12, rounded up to a power of two; E4M3 round to
    nearest even) and dequantised again.  Same law as the CPU oracle's block quantiser."""
    if axis == 0:
        return mx_quant_dequant(t.T.contiguous(), 1).T.contiguous()
    shape = t.shape
    b = t.reshape(*shape[:-1], shape[-1] // 32, 32).float()
    amax = b.abs().amax(-1, keepdim=True)
    scale = torch.clamp(amax * 0.002232142857, min=1e-12)
    mant, expo = torch.frexp(scale)                                   # scale = mant * 2^expo, mant in [0.5, 1)
    p2 = torch.ldexp(torch.ones_like(mant), torch.where(mant == 0.5, expo - 1, expo))
    q = (b / p2).to(torch.float8_e4m3fn).float()
    return (q * p2).reshape(shape)


def _silu_fwd(g, u, limit):
    if limit is not None:
        g, u = g.clamp(max=limit), u.clamp(min=-limit, max=limit)
    return g / (1.0 + torch.exp(-g)) * u


def _silu_bwd(g, u, dh, limit):
    gm = um = None
    if limit is not None:
        gm, um = g <= limit, (u >= -limit) & (u <= limit)
        g, u = g.clamp(max=limit), u.clamp(min=-limit, max=limit)
    sig = 1.0 / (1.0 + torch.exp(-g))
    silu = g * sig
    dg, du = ((1.0 - silu) * sig + silu) * u * dh, silu * dh
    if limit is not None:
        dg, du = torch.where(gm, dg, torch.zeros_like(dg)), torch.where(um, du, torch.zeros_like(du))
    return dg, du, silu * u


def _rel_l2(ref, got):
    ref, got = ref.double(), got.double()
    n = ref.norm().item()
    return (ref - got).norm().item() / (n if n > 0 else 1.0)


def sampled_parity(wl, rank, world, dev, inp, out, grads, sched, ctx, samples):
    """Recomputes `samples` of this rank's tokens in fp32 with the device's bf16 rounding points (and, for MXFP8,
    block-quantised operands): output and, with a backward pass, d_x and d_router_weights — every routed row of
    those tokens was computed on the rank that owns its expert, so with several ranks this checks dispatch and
    combine end to end — plus eight rows of one routed expert's down-projection weight gradient (BF16 workloads),
    contracted over the rows that expert received from all ranks (their hidden activations recomputed here too).  Every rank's seeded inputs are regenerated
    here; nothing is read from another rank.  Returns {name: rel-L2}."""
    T, H, I, E, K = wl["T"], wl["H"], wl["I"], wl["E"], wl["K"]
    El = E // world
    mx = bool(wl.get("mxfp8"))
    rd = lambda t: t.to(torch.bfloat16).float()  # noqa: E731
    qd = (lambda t, axis: mx_quant_dequant(t, axis)) if mx else (lambda t, axis: t)
    idx = torch.arange(0, T, T // samples, device=dev)[:samples]
    experts = inp["topk"][idx]                                         # [S, K] global expert ids
    needed = torch.unique(experts).tolist()
    weights = {}                                                       # expert -> (wg [I,H], wu [I,H], wd [H,I]) bf16
    shared = None
    # schedule rows of the first local expert, for the weight-gradient rows
    n_rows0 = int(sched.tokens_per_expert[0].item())
    pr0 = sched.peer_rank[:n_rows0].long()
    pt0 = sched.peer_token_idx[:n_rows0].long()
    h_rows = torch.arange(0, H, H // 8, device=dev)[:8]
    d_y_rows = torch.zeros(n_rows0, len(h_rows), device=dev)
    x_rows0 = torch.zeros(n_rows0, H, device=dev) if (wl["backward"] and not mx) else None   # what expert 0 received
    for p in range(world):
        step_p, params_p = make_inputs(wl, p, world, dev, pinned=False)
        for e in needed:
            if e // El == p:
                weights[e] = tuple(w[e - p * El].clone() for w in params_p[3:])
        if p == rank:
            shared = [w.float() for w in params_p[:3]]
        if wl["backward"] and not mx and n_rows0:
            sel = pr0 == p
            tok, kk = pt0[sel] // K, pt0[sel] % K
            d_y_rows[sel] = rd(step_p["d_out"][tok][:, h_rows].float() * step_p["rw"][tok, kk][:, None])
            x_rows0[sel] = step_p["x"][tok].float()
            if p == rank:
                w0 = tuple(w[0].float() for w in params_p[3:])       # this rank's first local expert
        del step_p, params_p
    x = inp["x"][idx].float()
    rw = inp["rw"][idx]
    sg, su, sd = shared
    g_s, u_s = rd(x @ sg.T), rd(x @ su.T)
    acc = rd(rd(_silu_fwd(g_s, u_s, None)) @ sd.T)
    if wl["backward"]:
        d_out = inp["d_out"][idx].float()
        d_h = rd(d_out @ sd)
        d_g, d_u, _ = _silu_bwd(g_s, u_s, d_h, None)
        d_x = rd(rd(d_g) @ sg + rd(d_u) @ su)
        d_rw = torch.zeros(samples, K, device=dev)
    for k in range(K):
        for s in range(samples):                                       # one (token, route) at a time: little memory
            wg, wu, wd = (w.float() for w in weights[int(experts[s, k])])
            xs = x[s:s + 1]
            ge, ue = rd(qd(xs, 1) @ qd(wg, 1).T), rd(qd(xs, 1) @ qd(wu, 1).T)
            he = rd(_silu_fwd(ge, ue, None))
            ye = rd(qd(he, 1) @ qd(wd, 1).T)
            acc[s] = acc[s] + (ye * rw[s, k])[0]
            if wl["backward"]:
                w_route = rw[s, k]
                d_y = rd(d_out[s:s + 1] * w_route)
                d_he = rd(qd(d_y, 1) @ qd(wd, 0))
                d_ge, d_ue, hid_f = _silu_bwd(qd(ge, 1), qd(ue, 1), d_he, None)
                inv_w = 1.0 / w_route if w_route > 0 else torch.zeros((), device=dev)
                d_rw[s, k] = (d_he * inv_w * hid_f).sum()
                d_x[s] = d_x[s] + rd(qd(rd(d_ge), 1) @ qd(wg, 0) + qd(rd(d_ue), 1) @ qd(wu, 0))[0]
    res = {"output": _rel_l2(rd(acc), out[idx].float())}
    if wl["backward"]:
        res["d_x"] = _rel_l2(rd(d_x), grads[0][idx].float())
        res["d_router_weights"] = _rel_l2(d_rw, grads[1][idx])
        if not mx and n_rows0:
            # hidden of the rows the first local expert received, recomputed from the senders' tokens (the saved
            # activations are not used: a backward over several windows overwrites them with its replay)
            hid0 = rd(_silu_fwd(rd(x_rows0 @ w0[0].T), rd(x_rows0 @ w0[1].T), None))
            ref_rows = d_y_rows.T @ hid0                                       # [8, I]
            res["d_w_routed_down_rows"] = _rel_l2(ref_rows, grads[4][0][h_rows].float())
    return res


# ----------------------------------------------------------------------------------------------------------
# one workload on this rank's GPU
# ----------------------------------------------------------------------------------------------------------
class LayerRun:
    """Workspace, inputs, and the step functions (device-resident and end-to-end) of one workload."""

    def __init__(self, name, wl, rank, world, local_rank, group, comm_sms=None):
        import mok
        self.mok, self.F, self.L = mok, mok.functional, mok._lib
        self.name, self.wl, self.rank, self.world, self.local_rank, self.group = name, wl, rank, world, local_rank, group
        self.dev = torch.device("cuda", local_rank)
        F = self.F
        T, H, E, K = wl["T"], wl["H"], wl["E"], wl["K"]
        self.El = E // world
        knobs = {}
        if comm_sms is not None:
            knobs = dict(fwd_num_comm_sms=comm_sms, bwd_num_comm_sms=comm_sms)
        self.cfg = F.MoKConfig(minibatch_size=wl["minibatch"], macrobatch_size=wl["macrobatch"],
                               schedule_capacity_multiplier=wl["multiplier"], **knobs)
        self.ws = F.get_workspace(self.cfg, group, device=self.dev, num_local_tokens=T, hidden_size=H, topk=K)
        self.host, params = make_inputs(wl, rank, world, self.dev)
        self.dev_in = {k: v.to(self.dev) for k, v in self.host.items()}
        if world > 1:
            # the device-resident step finds its inputs where a producer running on this GPU would have written
            # them: in the workspace's rank-visible buffers, which mok.functional then uses in place (no staging copy)
            self.dev_in["x"] = self.ws.x_buffer.copy_(self.dev_in["x"])
            self.dev_in["rw"] = self.ws.router_weight_buffer.copy_(self.dev_in["rw"])
            if wl["backward"]:
                self.dev_in["d_out"] = self.ws.d_y_buffer.copy_(self.dev_in["d_out"])
        # share of all routes that lands on the busiest rank (1/world when balanced)
        dest = torch.bincount((self.dev_in["topk"] // self.El).flatten(), minlength=world).double()
        if world > 1:
            dist.all_reduce(dest, group=group)
        self.max_rank_share = (dest.max() / dest.sum()).item()
        self.fwd_params = self.bwd_params = params
        if wl.get("mxfp8"):              # routed weights quantised once, outside the timed region (as the reference does)
            qg, qu, qd = (mok.ops.mxfp8_quantize(w, True, True) for w in params[3:])
            self.fwd_params = params[:3] + [(qg[0], qg[1]), (qu[0], qu[1]), (qd[0], qd[1])]
            self.bwd_params = params[:3] + [tuple(qg), tuple(qu), (qd[2], qd[3])]
            params[3:] = []              # the bf16 masters are not needed any more
        self._e2e = None

    def set_comm_sms(self, n):
        """The same run with another number of SMs set aside for row movement (the workspace does not depend on it)."""
        self.cfg = self.F.MoKConfig(minibatch_size=self.wl["minibatch"], macrobatch_size=self.wl["macrobatch"],
                                    schedule_capacity_multiplier=self.wl["multiplier"], fwd_num_comm_sms=n,
                                    bwd_num_comm_sms=n)

    def step(self, inp=None, keep=False):
        F, wl = self.F, self.wl
        inp = inp or self.dev_in
        sched = F.build_schedule(self.ws, self.cfg, inp["topk"], num_local_experts=self.El)
        out, ctx = F.forward(self.cfg, self.ws, sched, inp["x"], inp["rw"], *self.fwd_params)
        grads = None
        if wl["backward"]:
            grads = F.backward(self.cfg, self.ws, sched, ctx, inp["d_out"], inp["x"], inp["rw"], *self.bwd_params)
        if keep:
            return out, grads, sched, ctx
        return out, grads

    # End-to-end step: inputs start in pinned host memory and results end there, every step.  The copies
    # are double-buffered on their own streams: the inputs of step i+1 are uploaded while step i computes
    # and the results of step i are downloaded while step i+1 computes; the host reads a step's results
    # one step later (it synchronises on that step's download).
    def _e2e_state(self):
        if self._e2e is None:
            wl, dev, host = self.wl, self.dev, self.host
            T, H, K = wl["T"], wl["H"], wl["K"]
            keys = [k for k in host if k != "d_out" or wl["backward"]]
            self._e2e = dict(
                keys=keys, h2d=torch.cuda.Stream(dev), d2h=torch.cuda.Stream(dev),
                slots=[{k: torch.empty_like(host[k], device=dev) for k in keys} for _ in range(2)],
                uploaded=[torch.cuda.Event() for _ in range(2)], consumed=[torch.cuda.Event() for _ in range(2)],
                downloaded=[torch.cuda.Event() for _ in range(2)], i=0, primed=False,
                out_host=torch.empty(T, H, dtype=torch.bfloat16).pin_memory(),
                dx_host=torch.empty(T, H, dtype=torch.bfloat16).pin_memory(),
                drw_host=torch.empty(T, K, dtype=torch.float32).pin_memory(),
                metric_host=torch.empty(3, dtype=torch.float32).pin_memory())
        return self._e2e

    def _upload(self, s, slot):
        with torch.cuda.stream(s["h2d"]):
            s["h2d"].wait_event(s["consumed"][slot])       # the previous user of this slot has finished
            for k in s["keys"]:
                s["slots"][slot][k].copy_(self.host[k], non_blocking=True)
            s["uploaded"][slot].record(s["h2d"])

    def step_e2e_metric(self):
        """The end-to-end step with a scalar result: the same uploads, but what goes back to the host is one number
        per result tensor (its mean square, reduced on the device inside the timed region), as a trainer would read a
        loss, instead of the tensors themselves."""
        return self.step_e2e(metric_only=True)

    def step_e2e(self, metric_only=False):
        s = self._e2e_state()
        i = s["i"]
        slot = i & 1
        main = torch.cuda.current_stream()
        if not s["primed"]:
            s["consumed"][0].record(main); s["consumed"][1].record(main)
            self._upload(s, slot)
            s["primed"] = True
        self._upload(s, slot ^ 1)                          # prefetch the next step's inputs
        main.wait_event(s["uploaded"][slot])
        out, grads = self.step(s["slots"][slot])
        metric = None
        if metric_only:
            parts = [out.float().square().mean()]
            if grads is not None:
                parts += [grads[0].float().square().mean(), grads[1].square().mean()]
            metric = torch.stack(parts)
        s["consumed"][slot].record(main)
        with torch.cuda.stream(s["d2h"]):
            s["d2h"].wait_event(s["consumed"][slot])
            if metric is not None:
                s["metric_host"][:metric.numel()].copy_(metric, non_blocking=True)
                metric.record_stream(s["d2h"])
            else:
                s["out_host"].copy_(out, non_blocking=True)
                out.record_stream(s["d2h"])
                if grads is not None:
                    s["dx_host"].copy_(grads[0], non_blocking=True)
                    s["drw_host"].copy_(grads[1], non_blocking=True)
                    grads[0].record_stream(s["d2h"]); grads[1].record_stream(s["d2h"])
            s["downloaded"][slot].record(s["d2h"])
        if i > 0:
            s["downloaded"][slot ^ 1].synchronize()        # the caller reads the previous step's results
        s["i"] = i + 1

    def drain_e2e(self):
        s = self._e2e_state()
        i = s["i"]
        if i > 0:
            torch.cuda.current_stream().wait_event(s["downloaded"][(i - 1) & 1])
            torch.cuda.current_stream().wait_event(s["uploaded"][i & 1])

    def copy_only_step(self):
        """The host<->device copies of one end-to-end step and nothing else (same pinned buffers, same two copy
        streams, the downloads reading device tensors of the results' sizes): what the host side alone can sustain."""
        s = self._e2e_state()
        if "fake" not in s:
            s["fake"] = (torch.empty_like(s["out_host"], device=self.dev), torch.empty_like(s["dx_host"], device=self.dev),
                         torch.empty_like(s["drw_host"], device=self.dev))
        with torch.cuda.stream(s["h2d"]):
            for k in s["keys"]:
                s["slots"][0][k].copy_(self.host[k], non_blocking=True)
        with torch.cuda.stream(s["d2h"]):
            s["out_host"].copy_(s["fake"][0], non_blocking=True)
            if self.wl["backward"]:
                s["dx_host"].copy_(s["fake"][1], non_blocking=True)
                s["drw_host"].copy_(s["fake"][2], non_blocking=True)

    def copy_only_finish(self):
        s = self._e2e_state()
        torch.cuda.current_stream().wait_stream(s["h2d"])
        torch.cuda.current_stream().wait_stream(s["d2h"])

    def e2e_bytes(self):
        wl, s = self.wl, self._e2e_state()
        h2d = sum(v.numel() * v.element_size() for k, v in self.host.items() if k != "d_out" or wl["backward"])
        d2h = s["out_host"].numel() * 2 + ((s["dx_host"].numel() * 2 + s["drw_host"].numel() * 4) if wl["backward"] else 0)
        return h2d, d2h

    # ---- timing -------------------------------------------------------------------------------------------
    def barrier(self):
        if self.world > 1:
            dist.barrier(group=self.group, device_ids=[self.local_rank])
        torch.cuda.synchronize()

    def timed(self, fn, steps, finish=None):
        """K steps between two barriers; returns (ms per step from the whole region, max over ranks; median over the
        steps of the per-step maximum over ranks)."""
        self.barrier()
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        marks[0].record()
        for i in range(steps):
            fn()
            if i + 1 < steps:
                marks[i + 1].record()
        if finish is not None:
            finish()
        marks[steps].record()
        self.barrier()
        per = torch.tensor([marks[i].elapsed_time(marks[i + 1]) for i in range(steps)] + [marks[0].elapsed_time(marks[steps])],
                           dtype=torch.float64, device=self.dev)
        if self.world > 1:
            dist.all_reduce(per, op=dist.ReduceOp.MAX, group=self.group)
        per = per.tolist()
        return per[-1] / steps, statistics.median(per[:-1])

    def measure(self, steps, warmup, e2e=True, kernel_events=True, parity_samples=0):
        wl, L, mok, dev = self.wl, self.L, self.mok, self.dev
        T, H, I, K = wl["T"], wl["H"], wl["I"], wl["K"]
        for _ in range(warmup):
            self.step()
        torch.cuda.synchronize()
        mok.raise_for_status(dev)
        launches0 = L.mok_launch_count()
        ms_step, ms_median = self.timed(self.step, steps)
        launches = L.mok_launch_count() - launches0
        res = dict(ms_step=ms_step, ms_median=ms_median, launches=int(launches), flops=layer_flops(T, K, H, I, wl["backward"]))
        if kernel_events:
            # the same K steps again with a CUDA-event pair around every launch: the per-kernel split behind
            # `roofline` (the event records cost a little, so `value` comes from the region above)
            L.mok_profile_enable(1)
            L.profile_collect()
            res["ms_step_events"], _ = self.timed(self.step, steps)
            res["prof"] = L.profile_collect()
            L.mok_profile_enable(0)
        # rows this rank's schedule holds against the routes it received (expert groups are padded to 256 rows)
        out_a, grads_a, sched, ctx = self.step(keep=True)
        n_rows = int(sched.num_tokens.item())
        n_routes = int((sched.peer_rank[:min(n_rows, sched.peer_rank.numel())] >= 0).sum().item())
        res.update(n_rows=n_rows, n_routes=n_routes)
        if parity_samples:
            par = sampled_parity(wl, self.rank, self.world, dev, self.dev_in, out_a, grads_a, sched, ctx, parity_samples)
            worst = torch.tensor([max(par.values())], dtype=torch.float64, device=dev)
            if self.world > 1:
                dist.all_reduce(worst, op=dist.ReduceOp.MAX, group=self.group)
            res["parity"] = dict(worst_over_ranks=worst.item(), rank0=par, samples_per_rank=parity_samples,
                                 bound=MXFP8_REL_L2 if wl.get("mxfp8") else BF16_REL_L2)
        del sched, ctx
        out_b, grads_b = self.step()
        same = torch.equal(out_a, out_b)
        if grads_a is not None:
            same = same and all(torch.equal(a, b) for a, b in zip(grads_a, grads_b))
        flag = torch.tensor([0 if same else 1], device=dev)
        if self.world > 1:
            dist.all_reduce(flag, group=self.group)
        res["rerun_identical"] = flag.item() == 0
        del out_a, out_b, grads_a, grads_b
        if e2e:
            for _ in range(3):
                self.step_e2e()
            self.drain_e2e()
            res["ms_e2e"], _ = self.timed(self.step_e2e, steps, finish=self.drain_e2e)
            res["h2d"], res["d2h"] = self.e2e_bytes()
            torch.cuda.synchronize()
            res["ms_copy_only"], _ = self.timed(self.copy_only_step, min(steps, 20), finish=self.copy_only_finish)
            for _ in range(2):
                self.step_e2e_metric()
            self.drain_e2e()
            res["ms_e2e_metric"], _ = self.timed(self.step_e2e_metric, min(steps, 50), finish=self.drain_e2e)
        mok.raise_for_status(dev)
        return res

    def release(self):
        """Drops this run's tensors (the cached workspace stays with mok.functional until the cache is cleared)."""
        self.host = self.dev_in = self.fwd_params = self.bwd_params = self._e2e = None
        torch.cuda.empty_cache()


def roofline_record(name, wl, res, steps, world):
    """The routed gate|up GEMM launches of the event-timed pass against the measured tensor peak."""
    T, H, I, E, K = wl["T"], wl["H"], wl["I"], wl["E"], wl["K"]
    peaks = measured_peaks()
    scale = 2.0 if wl.get("mxfp8") else 1.0      # no measured MXFP8 peak on file: twice the measured bf16 figures
    dom = "gemm_gate_up_swiglu_routed"
    dom_ms, dom_cnt = res.get("prof", {}).get(dom, (0.0, 0))
    dom_ms_step = dom_ms / steps if dom_cnt else None
    dom_flops = 4.0 * T * K * H * I              # gate + up GEMMs over the T*K routed rows (padding not counted)
    achieved = dom_flops / (dom_ms_step * 1e-3) / 1e12 if dom_ms_step else None
    burst, sustained = scale * peaks["burst"], scale * peaks["tflops"]
    return dict(kernel=dom, bound="tensor", achieved=achieved, unit="TFLOP/s",
                frac_vs_burst=(achieved / burst) if achieved else None,
                frac_vs_sustained=(achieved / sustained) if achieved else None,
                burst_peak=burst, sustained_peak=sustained,
                peak_source=peaks["source"] + (" bf16 figures x2 for fp8" if scale == 2.0 else ""),
                traffic=dominant_traffic(name, E // world, res.get("n_rows")),
                traffic_scope="one step: the launches_per_step launches of this kernel together cover the step's rows "
                              "once and read each local expert's weights once; achieved is over the same launches",
                launches_per_step=dom_cnt / steps if dom_cnt else 0, ms_per_step=dom_ms_step)


def finish_roofline(roof, region_seconds, clocks):
    """`frac` and `peak` against the burst figure when the event-timed region was short and no cap was seen in the
    clock samples, else against the sustained figure."""
    capped = bool(clocks and "sw_power_cap" in (clocks.get("reasons") or []))
    burst = region_seconds < 1.0 and not capped
    roof["peak"] = roof["burst_peak"] if burst else roof["sustained_peak"]
    roof["frac"] = roof["frac_vs_burst"] if burst else roof["frac_vs_sustained"]
    roof["peak_kind"] = ("burst (timed region %.2f s, no power cap sampled)" if burst else
                         "sustained (timed region %.2f s%s)") % ((region_seconds,) if burst else
                                                                  (region_seconds, ", power cap sampled" if capped else ""))
    return roof


def sub_record(run: LayerRun, steps, warmup, parity_samples):
    """A second workload measured inside the same job (its own workspace and inputs): a compact record."""
    wl = run.wl
    res = run.measure(steps, warmup, e2e=False, kernel_events=True, parity_samples=parity_samples)
    roof = roofline_record(run.name, wl, res, steps, run.world)
    per_gpu = res["flops"] / (res["ms_step"] * 1e-3) / 1e12
    rec = {"workload": f"{run.name}: {wl['desc']}", "dtype": "mxfp8" if wl.get("mxfp8") else "bf16", "steps": steps,
           "warmup": warmup, "ms_per_step": res["ms_step"], "ms_per_step_median_of_per_step_max": res["ms_median"],
           "per_gpu_tflops": per_gpu, "value": run.world * per_gpu, "unit": UNIT,
           "busiest_rank_share_of_routes": run.max_rank_share, "rank0_schedule_rows": res["n_rows"],
           "rank0_routes": res["n_routes"],
           "padding_overhead": (res["n_rows"] / res["n_routes"] - 1.0) if res["n_routes"] else None,
           "rerun_bit_identical": res["rerun_identical"],
           "roofline": {k: roof[k] for k in ("kernel", "achieved", "unit", "frac_vs_burst", "frac_vs_sustained",
                                             "burst_peak", "sustained_peak", "peak_source", "ms_per_step")},
           "kernel_ms_per_step": {k: v[0] / steps for k, v in sorted(res["prof"].items())}}
    if "parity" in res:
        rec["parity_rel_l2"] = res["parity"]["worst_over_ranks"]
        rec["parity"] = res["parity"]
    return rec, res


def run_ours(args, rank, world, local_rank):
    numa_cpus = bind_to_gpu_numa_node(local_rank) if world > 1 else None
    import mok
    F = mok.functional
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
    steps, warmup = args.steps, max(args.warmup, 3)
    extras = not args.tokens and not args.no_extras
    # one-rank groups for the single-GPU share of the workload measured beside a multi-rank run
    solo = None
    if world > 1:
        for r in range(world):
            g = dist.new_group([r])
            if r == rank:
                solo = g

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    run = LayerRun(name, wl, rank, world, local_rank, dist.group.WORLD,
                   comm_sms=args.comm_sms if args.comm_sms >= 0 else None)
    parity_samples = 0 if args.no_parity else (8 if wl.get("mxfp8") else 24)
    res = run.measure(steps, warmup, e2e=True, kernel_events=True, parity_samples=parity_samples)
    ms_graph = None
    if args.graph and world == 1:        # the same step captured once and replayed as a CUDA graph
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            run.step()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            graph_out = run.step()
        graph.replay()
        torch.cuda.synchronize()
        eager_out = run.step()
        assert torch.equal(graph_out[0], eager_out[0]), "graph replay differs from the eager step"
        ms_graph, _ = run.timed(graph.replay, steps)
    clocks = sampler.stop() if rank == 0 else None
    comm_sms_used = (run.cfg.fwd_num_comm_sms, run.cfg.bwd_num_comm_sms)
    sweep = None
    if args.sweep_comm_sms and world > 1:      # the same workload with other numbers of SMs set aside for row movement
        sweep = []
        for n in [int(v) for v in args.sweep_comm_sms.split(",")]:
            run.set_comm_sms(n)
            for _ in range(2):
                run.step()
            ms, med = run.timed(run.step, max(5, steps // 2))
            sweep.append({"num_comm_sms": n, "ms_per_step": ms, "ms_per_step_median_of_per_step_max": med})
        mok.raise_for_status(dev)
    run.release()

    flops = res["flops"]
    ms_step, ms_e2e = res["ms_step"], res["ms_e2e"]
    roof = finish_roofline(roofline_record(name, wl, res, steps, world), res["ms_step_events"] * steps * 1e-3, clocks)
    peaks = measured_peaks()
    sustained = (2.0 if wl.get("mxfp8") else 1.0) * peaks["tflops"]
    per_gpu = flops / (ms_step * 1e-3) / 1e12
    config = {"workload": f"{name}: {wl['desc']}", "ep_size": world, "tokens_per_rank": T, "hidden": H,
              "intermediate": I, "experts": E, "topk": K, "minibatch_size": wl["minibatch"],
              "macrobatch_size": wl["macrobatch"], "capacity_multiplier": wl["multiplier"],
              "fwd_num_comm_sms": comm_sms_used[0], "bwd_num_comm_sms": comm_sms_used[1],
              "comm_sms_form": "dedicated SMs" if os.environ.get("MOK_B200_DEDICATED_COMM_SMS", "0") not in ("", "0")
              else "16 thin mover CTAs per budgeted SM beside the GEMM CTAs",
              "busiest_rank_share_of_routes": run.max_rank_share,
              "pass": "fwd+bwd" if wl["backward"] else "fwd (incl. build_schedule)",
              "rank0_schedule_rows": res["n_rows"], "rank0_routes": res["n_routes"],
              "padding_overhead": (res["n_rows"] / res["n_routes"] - 1.0) if res["n_routes"] else None,
              "rerun_bit_identical": res["rerun_identical"],
              "ms_per_step_median_of_per_step_max": res["ms_median"],
              "ms_per_step_with_kernel_events": res["ms_step_events"],
              "l2": "inputs larger than L2 (no flush needed)", "per_gpu_tflops": per_gpu,
              "pct_of_measured_bf16_peak": 100.0 * per_gpu / sustained,
              "pct_of_measured_burst_peak": 100.0 * per_gpu / ((2.0 if wl.get("mxfp8") else 1.0) * peaks["burst"]),
              "host_numa_placement": numa_cpus}
    if "parity" in res:
        config["parity_rel_l2"] = res["parity"]["worst_over_ranks"]
        config["parity"] = res["parity"]
    gemm_ms = sum(v[0] for k, v in res["prof"].items() if k.startswith("gemm_")) / steps
    config["gemm_launches_ms_per_step"] = gemm_ms
    config["not_covered_by_gemm_launches"] = (ms_step - gemm_ms) / ms_step
    if sweep is not None:
        config["num_comm_sms_sweep"] = sweep

    # the same per-GPU work with every row local, on every GPU at once (one-rank workspaces): what the step costs
    # without any traffic between GPUs.  With one GPU: the single-GPU share of the eight-rank training workload,
    # so that the N = 1 record also carries a point of the curve the N > 1 records lie on.
    failed = []
    if extras and (world > 1 or name == "C2"):
        share = "C3x1" if name in ("C2", "C3") else ("C4x1" if name in ("C4", "C5") else None)
        if share:
            wl1 = dict(WORKLOADS[share])
            if world > 1:
                wl1["E"] = max(1, wl["E"] // world)
                wl1["desc"] = f"one GPU's share of {name} at EP={world} with every row local ({wl1['E']} local experts)"
            solo_run = LayerRun(share, wl1, 0, 1, local_rank, solo if world > 1 else dist.group.WORLD)
            r1 = solo_run.measure(min(steps, 20), 3, e2e=False, kernel_events=False, parity_samples=0)
            solo_run.release()
            ms1 = torch.tensor([r1["ms_step"]], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(ms1, op=dist.ReduceOp.MAX)
            config["same_workload_n1_tflops"] = r1["flops"] / (ms1.item() * 1e-3) / 1e12
            config["same_workload_n1"] = {"workload": f"{share}: {wl1['desc']}", "ms_per_step": ms1.item(),
                                          "steps": min(steps, 20), "note": "all GPUs of the job run it at the same time"}
    line = {
        "metric": METRIC, "value": world * per_gpu, "unit": UNIT,
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "mxfp8 (e4m3 x e8m0, fp32 accumulate)" if wl.get("mxfp8") else "bf16", "data": "synthetic",
        "config": config,
        "e2e": {"value": world * flops / (ms_e2e * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": res["h2d"], "d2h_bytes_per_step": res["d2h"],
                "copies_alone_ms_per_step": res["ms_copy_only"],
                "copies_alone_gb_per_s_per_gpu_each_way": (res["h2d"] + res["d2h"]) / 2 / (res["ms_copy_only"] * 1e-3) / 1e9,
                "note": "copies_alone = the step's uploads and downloads with no compute, all ranks at once (max over ranks)",
                "scalar_result": {"value": world * flops / (res["ms_e2e_metric"] * 1e-3) / 1e12, "unit": UNIT,
                                  "ms_per_step": res["ms_e2e_metric"], "h2d_bytes_per_step": res["h2d"],
                                  "d2h_bytes_per_step": 12 if wl["backward"] else 4,
                                  "note": "same uploads; the host reads one mean-square per result tensor (reduced on the "
                                          "device inside the timed region) instead of the tensors"}},
        "gpu_launches": res["launches"],
        "clocks": clocks,
        "roofline": roof,
        "kernel_ms_per_step": {k: v[0] / steps for k, v in sorted(res["prof"].items())},
    }
    if ms_graph is not None:
        line["cuda_graph"] = {"ms_per_step": ms_graph, "value": flops / (ms_graph * 1e-3) / 1e12, "unit": UNIT,
                              "note": "the same step captured once with torch.cuda.graph and replayed"}
    # eight ranks: the MXFP8 half of the metric and the skewed-routing stress, each a short run of its own
    if (extras and world == 8 and name == "C3") or (args.sub_records and world > 1):
        F.clear_workspace_cache()
        torch.cuda.empty_cache()
        for key, sub, n_steps in (("mxfp8", "C4", 20), ("skew", "C5", 8)):
            sub_run = LayerRun(sub, dict(WORKLOADS[sub]), rank, world, local_rank, dist.group.WORLD,
                               comm_sms=args.comm_sms if args.comm_sms >= 0 else None)
            rec, _ = sub_record(sub_run, n_steps, 3, 0 if args.no_parity else 8)
            sub_run.release()
            F.clear_workspace_cache()
            torch.cuda.empty_cache()
            line[key] = rec
            if rec.get("parity_rel_l2") is not None and rec["parity_rel_l2"] > rec["parity"]["bound"]:
                failed.append(f"{sub} parity {rec['parity_rel_l2']:.3e}")
    if "parity" in res and res["parity"]["worst_over_ranks"] > res["parity"]["bound"]:
        failed.append(f"{name} parity {res['parity']['worst_over_ranks']:.3e}")
    if rank != 0:
        if failed:
            raise SystemExit(3)
        return
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(name, steps=1)
        if extras:
            line["cpu_baseline_c1"] = cpu_c1(repeats=10)
    print(json.dumps(line), flush=True)
    if failed:
        raise SystemExit("parity check failed: " + "; ".join(failed))


def use_all_host_threads():
    """The CPU arms use every hardware thread this process may run on.  (A launcher that starts one rank per GPU
    exports OMP_NUM_THREADS=1 to each of them, which would leave the CPU baseline on a single thread.)"""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    if n > torch.get_num_threads():
        torch.set_num_threads(n)
    return torch.get_num_threads()


def cpu_baseline(name, steps=1, warmup=0, sample_tokens=None, budget_s=None):
    """The CPU oracle on a bounded sample of the workload: same H, I, E, K and router law, fewer
    tokens per rank, single process, all host threads.  With `budget_s` the loop stops early once that much
    wall time is spent (the record says how many steps ran)."""
    from oracle import mok_oracle as O
    use_all_host_threads()
    wl = WORKLOADS[name]
    W = 1
    T = sample_tokens or (min(wl["T"], 16384) if not wl["backward"] else 4096)   # about 3-10 s of CPU work per step
    cfgs = dict(T=T, H=wl["H"], I=wl["I"], E=wl["E"], W=W, K=wl["K"], seed=0, router=wl["router"],
                with_grad=wl["backward"])
    ranks = [O.make_rank_inputs(r, **cfgs) for r in range(W)]
    times = []
    t_begin = time.perf_counter()
    ran_warmup = 0
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        O.layer_forward_backward(ranks, device_rounding=True, backward=wl["backward"])
        t1 = time.perf_counter()
        if i >= warmup:
            times.append(t1 - t0)
        else:
            ran_warmup += 1
        if budget_s is not None and t1 - t_begin > budget_s and times:
            break
    sec = statistics.median(times)
    fl = W * layer_flops(T, wl["K"], wl["H"], wl["I"], wl["backward"])
    return {"value": fl / sec / 1e12, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{T} tokens (of {wl['T']}) on one virtual rank, all {wl['E']} experts local, "
                      f"{'fwd+bwd' if wl['backward'] else 'fwd'}, {sec:.2f} s per step (median of {len(times)})",
            "seconds_per_step": sec, "steps_run": len(times), "warmup_run": ran_warmup}


def cpu_c1(repeats=10):
    """The small CPU configuration: fp32 forward + backward of the layer (T=256, H=512, 8 experts, top-2, I=1024,
    seed 0) through the CPU oracle without the device's rounding points; median of `repeats` runs."""
    from oracle import mok_oracle as O
    use_all_host_threads()
    wl = WORKLOADS["C1"]
    inp = [O.make_rank_inputs(0, T=wl["T"], H=wl["H"], I=wl["I"], E=wl["E"], W=1, K=wl["K"], seed=0)]
    O.layer_forward_backward(inp, device_rounding=False)
    times = []
    for _ in range(max(repeats, 10)):
        t0 = time.perf_counter()
        O.layer_forward_backward(inp, device_rounding=False)
        times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    fl = layer_flops(wl["T"], wl["K"], wl["H"], wl["I"], True)
    return {"value": fl / sec / 1e9, "unit": "GFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"C1: {wl['desc']}; median of {len(times)} runs, {sec * 1e3:.1f} ms each",
            "seconds_per_step": sec}


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
    oracle, restated in oracle/) on the host cores, one CPU process whatever N is, on a bounded sample per step.
    --warmup W and --steps K are honoured up to a wall-time budget of about two minutes; the record says how
    many steps ran."""
    if rank != 0:
        return
    name = args.workload if args.workload != "auto" else ("C2" if world == 1 else "C3")
    wl = WORKLOADS[name]
    if wl.get("cpu_only"):
        base = cpu_c1(repeats=max(args.steps, 10))
        print(json.dumps({"impl": "reference", "metric": "MoE layer fwd+bwd GFLOP/s (reference FLOP convention), fp32, host CPU",
                          "value": base["value"], "unit": base["unit"], "n_gpus": 0, "steps": max(args.steps, 10),
                          "warmup": 1, "ms_per_step": base["seconds_per_step"] * 1e3, "higher_is_better": True,
                          "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                          "config": {"workload": f"C1: {wl['desc']}"}, "cpu_baseline": base}), flush=True)
        return
    base = cpu_baseline(name, steps=max(1, args.steps), warmup=max(0, args.warmup), budget_s=120.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": world,
        "steps": base["steps_run"], "warmup": base["warmup_run"], "steps_requested": args.steps,
        "warmup_requested": args.warmup, "ms_per_step": base["seconds_per_step"] * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "ran_on": f"one CPU process with {base['cores']} threads, one virtual rank, no GPU: {base['sample']}; "
                  f"n_gpus only echoes how the arm was launched",
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
    ap.add_argument("--no-parity", action="store_true", help="skip the sampled-token parity check after the timed regions")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the single-GPU share of the workload and, at eight ranks, the MXFP8 and skew sub-records")
    ap.add_argument("--sub-records", action="store_true",
                    help="add the MXFP8 and skew sub-records at any rank count above one (they are automatic at eight)")
    ap.add_argument("--comm-sms", type=int, default=-1,
                    help="fwd/bwd_num_comm_sms of the MoKConfig (default: the configuration's own defaults)")
    ap.add_argument("--sweep-comm-sms", default="", help="comma-separated num_comm_sms values to time after the main run")
    ap.add_argument("--graph", action="store_true", help="also time the step replayed as one CUDA graph (1 GPU)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("--gpus N with N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    if args.workload == "C1" or args.impl == "reference":
        if args.workload == "C1" and args.impl == "ours":
            args.impl = "reference"      # C1 is the host-CPU configuration: there is nothing else to run
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
