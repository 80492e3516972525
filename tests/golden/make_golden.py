"""Generates the golden vectors under tests/golden/ by RUNNING THE REFERENCE's own
pure-PyTorch test oracles (reference `tests/utils.py`) on the CPU.

Usage (only where the reference tree is mounted):
    python tests/golden/make_golden.py /path/to/reference [router]     (a second word limits the run to that file)

What is stored
  schedule.npz   slot tables from `run_schedule_reference` for a handful of seeded routings,
                 including the adversarial `arange(T) % W` pattern at minimum capacity.
  quantize.npz   bytes and scale bytes from `run_mxfp8_quantize_reference` (2-D and 3-D).
  layer_w2.npz   the nine results of `run_reference_bf16` on two ranks (gloo), with and
                 without the SwiGLU clamp; inputs come from oracle.make_rank_inputs (seeded),
                 and an input checksum is stored so a drifting RNG is reported as such.
  router.npz     logits, top-k experts and router weights from the reference's `generate_inputs`
                 (torch.topk on the logits, softmax over the selected values), two shapes.
  layer_c1.npz   the same for the single-rank CPU configuration T=256, H=512, 8 experts,
                 top-2, I=1024 (seed 0), stored as a strided subsample (every 97th element; arrays of at most 8192
                 elements in full) plus norms.

The reference oracle needs a process group.  It is run under gloo; gloo has no
`all_gather_into_tensor` for 2-D outputs, so that one call is served by an equivalent
list all-gather (same values, no arithmetic involved).
"""
from __future__ import annotations

import importlib.util
import os
import sys
import zlib

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import mok_oracle as O  # noqa: E402

SCHEDULE_CASES = [  # (W, T, K, El, capacity factor, kind)
    (4, 512, 1, 1, 1, "arange"),
    (1, 512, 2, 8, 2, "randn"),
    (2, 512, 3, 5, 2, "randn"),
    (4, 1024, 8, 4, 4, "randn"),
    (8, 768, 6, 2, 8, "randn"),
    (4, 512, 4, 4, 4, "first_k"),
]
LAYER_W2 = dict(T=512, H=256, I=256, E=4, W=2, K=2, seed=11)
LAYER_C1 = dict(T=256, H=512, I=1024, E=8, W=1, K=2, seed=0)
RESULT_NAMES = ("output", "d_x", "d_router_weights", "d_w_routed_gate", "d_w_routed_up",
                "d_w_routed_down", "d_w_shared_gate", "d_w_shared_up", "d_w_shared_down")


def load_reference(ref_root: str):
    spec = importlib.util.spec_from_file_location("reference_test_utils",
                                                  os.path.join(ref_root, "tests", "utils.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def schedule_topk(W, T, K, El, kind):
    if kind == "arange":
        return (torch.arange(T) % W).to(torch.int32).view(1, T, 1).repeat(W, 1, 1)
    if kind == "first_k":
        return torch.arange(K, dtype=torch.int32).view(1, 1, K).repeat(W, T, 1)
    g = torch.Generator().manual_seed(W * 1000 + T + K)
    return torch.topk(torch.randn(W, T, W * El, generator=g), K, dim=2).indices.to(torch.int32)


def to_u(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def input_checksum(inp: O.RankInputs) -> int:
    c = 0
    for t in (inp.x, inp.topk_experts, inp.router_weights, inp.w_shared_gate, inp.w_routed_down,
              inp.d_output):
        c = zlib.crc32(to_u(t.contiguous()).tobytes(), c)
    return c


def _layer_worker(rank, W, ref_root, cfg, limits, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=W)
    ref = load_reference(ref_root)

    def all_gather_2d(out, inp, group=None):
        parts = [torch.empty_like(inp) for _ in range(W)]
        dist.all_gather(parts, inp)
        out.copy_(torch.stack(parts).view_as(out))
    dist.all_gather_into_tensor = all_gather_2d

    inp = O.make_rank_inputs(rank, **cfg)
    store = {"checksum": np.array([input_checksum(inp)], dtype=np.int64)}
    for tag, limit in limits:
        res = ref.run_reference_bf16(
            inp.x, inp.topk_experts, inp.router_weights, inp.w_shared_gate, inp.w_shared_up,
            inp.w_shared_down, inp.w_routed_gate, inp.w_routed_up, inp.w_routed_down,
            inp.d_output, limit)
        for name, t in zip(RESULT_NAMES, res):
            store[f"{tag}/{name}"] = to_u(t.detach().contiguous())
    np.savez(out_path + f".rank{rank}.npz", **store)
    dist.barrier()
    dist.destroy_process_group()


def run_layer(ref_root, cfg, limits, port):
    W = cfg["W"]
    tmp = os.path.join(HERE, "_tmp_layer")
    mp.spawn(_layer_worker, args=(W, ref_root, cfg, limits, port, tmp), nprocs=W)
    merged = {}
    for r in range(W):
        path = tmp + f".rank{r}.npz"
        with np.load(path) as z:
            for k in z.files:
                merged[f"rank{r}/{k}"] = z[k]
        os.remove(path)
    return merged


ROUTER_CASES = [dict(T=512, E=64, K=6), dict(T=768, E=256, K=8), dict(T=512, E=8, K=2)]


def router_golden(ref) -> None:
    store = {}
    for i, c in enumerate(ROUTER_CASES):
        rank = i
        out = ref.generate_inputs(rank, torch.device("cpu"), c["E"], c["E"], c["K"], c["T"], 256, 256)
        # the logits are the generator's first draw (reference tests/utils.py:80-82)
        g = torch.Generator().manual_seed(1234 + rank)
        logits = torch.randn(c["T"], c["E"], generator=g)
        assert torch.equal(torch.topk(logits, c["K"], dim=1).indices, out[1])
        store[f"{i}/logits"] = logits.numpy()
        store[f"{i}/topk_experts"] = out[1].numpy()
        store[f"{i}/router_weights"] = out[2].numpy()
    np.savez_compressed(os.path.join(HERE, "router.npz"), **store)


def main(ref_root: str, only: str | None = None):
    ref = load_reference(ref_root)
    torch.manual_seed(0)
    router_golden(ref)
    if only == "router":
        print("router golden vectors written to", HERE)
        return

    # ---- scheduler
    store = {}
    for i, (W, T, K, El, fac, kind) in enumerate(SCHEDULE_CASES):
        topk = schedule_topk(W, T, K, El, kind)
        cap = T * K * fac
        for rank in range(W):
            pr, pt, nt, tpe = ref.run_schedule_reference(topk, El, cap, rank)
            store[f"{i}/{rank}/peer_rank"] = pr.numpy()
            store[f"{i}/{rank}/peer_token_idx"] = pt.numpy()
            store[f"{i}/{rank}/num_tokens"] = nt.numpy()
            store[f"{i}/{rank}/tokens_per_expert"] = tpe.numpy()
    np.savez_compressed(os.path.join(HERE, "schedule.npz"), **store)

    # ---- quantiser
    store = {}
    g = torch.Generator().manual_seed(5678)
    x3 = (torch.randn(2, 128, 256, generator=g) * torch.exp(2.0 * torch.randn(2, 128, 1, generator=g))).to(torch.bfloat16)
    x2 = torch.randn(256, 128, generator=g).to(torch.bfloat16)
    for tag, x in (("x3", x3), ("x2", x2)):
        store[f"{tag}/in"] = to_u(x)
        for name, t in zip(("fp8", "sc", "fp8_t", "sc_t"), ref.run_mxfp8_quantize_reference(x, True, True)):
            store[f"{tag}/{name}"] = to_u(t.contiguous())
    np.savez_compressed(os.path.join(HERE, "quantize.npz"), **store)

    # ---- SwiGLU and epilogues (small closed cases)
    store = {}
    gate = torch.randn(128, 256, generator=g).to(torch.bfloat16)
    up = torch.randn(128, 256, generator=g).to(torch.bfloat16)
    store["gate"], store["up"] = to_u(gate), to_u(up)
    store["hidden"] = to_u(ref.run_swiglu_reference(gate, up, None))
    store["hidden_clamped"] = to_u(ref.run_swiglu_reference(gate, up, 1.0))
    ys = torch.randn(512, 256, generator=g).to(torch.bfloat16)
    cb = torch.randn(512 * 3, 256, generator=g).to(torch.bfloat16)
    w = torch.rand(512, 3, generator=g)
    store["ys"], store["cb"], store["w"] = to_u(ys), to_u(cb), w.numpy()
    store["fwd_epilogue"] = to_u(ref.run_fwd_epilogue_reference(ys, cb, w))
    store["bwd_epilogue"] = to_u(ref.run_bwd_epilogue_reference(ys, cb))
    np.savez_compressed(os.path.join(HERE, "elementwise.npz"), **store)

    # ---- whole layer, two ranks
    merged = run_layer(ref_root, LAYER_W2, (("plain", None), ("clamped", 1.0)), 29541)
    np.savez_compressed(os.path.join(HERE, "layer_w2.npz"), **merged)

    # ---- whole layer, single-rank CPU configuration: subsample + norms
    merged = run_layer(ref_root, LAYER_C1, (("plain", None),), 29542)
    small = {}
    for k, v in merged.items():
        if k.endswith("checksum"):
            small[k] = v
            continue
        f = (torch.from_numpy(v.view(np.int16)).view(torch.bfloat16).float().numpy()
             if v.dtype == np.uint16 else v.astype(np.float32))
        small[k + "/sample"] = f.reshape(-1)[::(97 if f.size > 8192 else 1)].copy()
        small[k + "/abs_sum"] = np.array([np.abs(f.astype(np.float64)).sum()])
        small[k + "/sq_sum"] = np.array([(f.astype(np.float64) ** 2).sum()])
    np.savez_compressed(os.path.join(HERE, "layer_c1.npz"), **small)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    main(sys.argv[1], sys.argv[2] if len(sys.argv) > 2 else None)
