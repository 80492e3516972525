"""CPU oracle for the Mixture-of-Kittens MoE hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, on the CPU, the arithmetic of the reference's path
schedule -> dispatch -> grouped SwiGLU expert FFN -> combine (forward and
backward).  Only the test-suite, the smoke check and the CPU-baseline leg of the
benchmark may import it; the product path never does.

Parity status: PINNED.  Every function below is checked against the reference's
own pure-PyTorch test oracles (reference `tests/utils.py`), which were imported
and run in the build container; the resulting vectors are stored under
`tests/golden/` together with the script that generated them
(`tests/golden/make_golden.py`), and `tests/test_oracle.py` replays them.

Reference anchors (paths are relative to the reference project root):
  schedule tables          csrc/scheduler.cuh:35-147, tests/utils.py:122-176
  MXFP8 quantiser          csrc/mxfp8.cuh:45-72,184, tests/utils.py:179-221
  SwiGLU (+clamp), grads   csrc/mok_megakernel.cuh:612-647,746-776, tests/utils.py:224-235
  epilogues                csrc/utils.cuh:65-117,158-194, tests/utils.py:299-317
  router (top-K, weights)  tests/utils.py:82-84 (torch.topk on the logits, softmax over the K values)
  layer forward/backward   tests/utils.py:238-296,320-430 and the device rounding
                           points csrc/mok_megakernel.cuh:464-467,776,958,1002,1135
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

EXPERT_PADDING = 256        # csrc/scheduler.cuh:14
SCHEDULE_THREADS = 1024     # csrc/scheduler.cuh:16
MX_BLOCK = 32               # csrc/mxfp8.cuh:104


# --------------------------------------------------------------------------------------
# Scheduler
# --------------------------------------------------------------------------------------
def route_order(num_routes: int) -> np.ndarray:
    """Thread-major visiting order of one rank's routes.

    The reference scheduler gives route r to thread r % 1024 and each thread walks
    its routes in increasing r (csrc/scheduler.cuh:106,130); slots inside one
    (expert, peer) list are therefore ordered by (r % 1024, r // 1024).
    """
    r = np.arange(num_routes, dtype=np.int64)
    return r[np.lexsort((r // SCHEDULE_THREADS, r % SCHEDULE_THREADS))]


def schedule_tables(topk_all: np.ndarray, num_local_experts: int, capacity: int, rank: int):
    """Slot tables of rank `rank` (csrc/scheduler.cuh:35-147).

    topk_all: int32 [W, T, K].  Returns (peer_rank[capacity], peer_token_idx[capacity],
    num_tokens[1], tokens_per_expert[El]) as int32 arrays; unwritten slots hold -1 in
    both tables.  Destination row of the j-th route of peer p for expert e is
    base_e + sum_r min(cnt_r, j) + [r < p and cnt_r > j]   (scheduler.cuh:134-139).
    """
    topk_all = np.asarray(topk_all)
    W, T, K = topk_all.shape
    R = T * K
    flat = topk_all.reshape(W, R)
    order = route_order(R)
    first = rank * num_local_experts
    peer_rank = np.full(capacity, -1, dtype=np.int32)
    peer_tok = np.full(capacity, -1, dtype=np.int32)
    tokens_per_expert = np.zeros(num_local_experts, dtype=np.int32)
    base = 0
    overflow = False
    for e in range(num_local_experts):
        lists = [order[flat[p, order] == first + e] for p in range(W)]
        cnt = np.array([len(l) for l in lists], dtype=np.int64)
        total = int(cnt.sum())
        padded = (total + EXPERT_PADDING - 1) // EXPERT_PADDING * EXPERT_PADDING
        tokens_per_expert[e] = padded
        for p in range(W):
            if cnt[p] == 0:
                continue
            j = np.arange(cnt[p], dtype=np.int64)
            dst = base + np.minimum(cnt[None, :], j[:, None]).sum(1)
            dst += ((np.arange(W)[None, :] < p) & (cnt[None, :] > j[:, None])).sum(1)
            ok = dst < capacity
            overflow |= not ok.all()
            peer_rank[dst[ok]] = p
            peer_tok[dst[ok]] = lists[p][ok].astype(np.int32)
        base += padded
    num_tokens = np.array([base], dtype=np.int32)
    return peer_rank, peer_tok, num_tokens, tokens_per_expert


# --------------------------------------------------------------------------------------
# MXFP8 quantiser (bit level)
# --------------------------------------------------------------------------------------
def _f32_bits(x: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest-even bfloat16, returned as float32."""
    b = _f32_bits(x).astype(np.uint64)
    nan = np.isnan(x)
    rounded = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16 << 16).astype(np.uint32)
    out = rounded.view(np.float32).copy()
    out[nan] = np.nan
    return out


def e8m0_round_up(scale: np.ndarray) -> np.ndarray:
    """cvt.rp.satfinite.ue8m0x2.f32: round a positive float up to a power of two, biased
    exponent byte (csrc/mxfp8.cuh:58)."""
    b = _f32_bits(scale)
    e = (b >> 23) & 0xFF
    mant = b & 0x7FFFFF
    e = e + (mant != 0)
    # subnormal inputs (e == 0 before the bump) round up to 2^-126 -> byte 1, or 0 if zero
    e = np.where(((b >> 23) & 0xFF) == 0, (mant != 0).astype(np.uint32), e)
    return np.minimum(e, 254).astype(np.uint8)


def e4m3_rn_satfinite(x: np.ndarray) -> np.ndarray:
    """cvt.rn.satfinite.e4m3x2.f32 for finite inputs: nearest-even to E4M3 (bias 7, 3
    mantissa bits, max 448, subnormal step 2^-9), saturating; returns the byte."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    a = np.abs(x).astype(np.float64)
    a = np.minimum(a, 448.0)
    # exponent of the quantisation step
    with np.errstate(divide="ignore"):
        ex = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    ex = np.maximum(ex, -6.0)                      # subnormal range shares the 2^-6 binade
    step = np.exp2(ex - 3.0)
    q = np.rint(a / step) * step                   # rint = round-half-even
    q = np.minimum(q, 448.0)
    # encode
    with np.errstate(divide="ignore"):
        qe = np.floor(np.log2(np.where(q > 0, q, 1.0)))
    qe = np.maximum(qe, -6.0)
    is_sub = q < 2.0 ** -6
    mant = np.where(is_sub, q / 2.0 ** -9, (q / np.exp2(qe) - 1.0) * 8.0)
    expo = np.where(is_sub, 0.0, qe + 7.0)
    byte = (expo.astype(np.uint8) << 3) | mant.astype(np.uint8)
    byte = np.where(np.isnan(x), np.uint8(0x7F), byte)
    return (byte | sign).astype(np.uint8)


def e4m3_decode(byte: np.ndarray) -> np.ndarray:
    b = np.asarray(byte, dtype=np.uint8)
    s = np.where(b & 0x80, -1.0, 1.0)
    e = ((b >> 3) & 0xF).astype(np.int32)
    m = (b & 7).astype(np.float64)
    v = np.where(e == 0, m * 2.0 ** -9, (1.0 + m / 8.0) * np.exp2(e - 7.0))
    return (s * v).astype(np.float32)


def mx_block_quantize(x_bf16_as_f32: np.ndarray):
    """Quantise along the last axis in blocks of 32 (csrc/mxfp8.cuh:45-72).

    Input holds bf16-representable float32 values, last dim % 32 == 0.  Returns
    (fp8 bytes with the input shape, scale bytes with last dim // 32).
    """
    x = np.ascontiguousarray(x_bf16_as_f32, dtype=np.float32)
    blocks = x.reshape(*x.shape[:-1], x.shape[-1] // MX_BLOCK, MX_BLOCK)
    amax = np.abs(blocks).max(-1)
    scale = np.maximum(amax * np.float32(0.002232142857), np.float32(1e-12)).astype(np.float32)
    sbyte = e8m0_round_up(scale)
    inv = ((np.uint32(254) - sbyte.astype(np.uint32)) << 23).view(np.float32)
    q = e4m3_rn_satfinite((blocks * inv[..., None]).astype(np.float32))
    return q.reshape(x.shape), sbyte


def scale_tile_layout(sbyte: np.ndarray) -> np.ndarray:
    """[rows, cols/32] scale bytes -> [rows/128, cols/128, 32, 16] tcgen05 block-scale
    layout: byte of (row r, k-block kb) of a 128x128 tile sits at (r%32)*16 + (r//32)*4 + kb
    (csrc/mxfp8.cuh:184; tests/utils.py:198-200)."""
    rows, kblocks = sbyte.shape
    t = sbyte.reshape(rows // 128, 4, 32, kblocks // 4, 4)        # [rt, r//32, r%32, ct, kb]
    t = t.transpose(0, 3, 2, 1, 4)                                # [rt, ct, r%32, r//32, kb]
    return np.ascontiguousarray(t).reshape(rows // 128, kblocks // 4, 32, 16)


def scale_tile_unlayout(sc: np.ndarray) -> np.ndarray:
    rt, ct = sc.shape[:2]
    t = sc.reshape(rt, ct, 32, 4, 4).transpose(0, 3, 2, 1, 4)
    return np.ascontiguousarray(t).reshape(rt * 128, ct * 4)


def mxfp8_quantize(x_bf16: torch.Tensor, return_normal: bool, return_transposed: bool):
    """CPU restatement of ops.mxfp8_quantize (csrc/mxfp8.cuh:188-278).  Returns uint8
    numpy arrays (fp8 bytes, scale bytes, transposed fp8 bytes, transposed scale bytes)."""
    x = x_bf16.float().numpy()
    x3 = x[None] if x.ndim == 2 else x
    E, M, N = x3.shape
    out = [None, None, None, None]
    if return_normal:
        q, s = mx_block_quantize(x3.reshape(E * M, N))
        out[0] = q.reshape(x.shape)
        out[1] = scale_tile_layout(s)
    if return_transposed:
        xt = np.ascontiguousarray(x3.transpose(0, 2, 1))
        q, s = mx_block_quantize(xt.reshape(E * N, M))
        out[2] = q.reshape((E, N, M) if x.ndim == 3 else (N, M))
        out[3] = scale_tile_layout(s)
    return tuple(out)


def mxfp8_dequantize(q: np.ndarray, sc_layout: np.ndarray) -> np.ndarray:
    """Inverse view used by the MXFP8 layer oracle: bytes + laid-out scales -> float32."""
    rows = int(np.prod(q.shape[:-1]))
    cols = q.shape[-1]
    s = scale_tile_unlayout(sc_layout).reshape(rows, cols // 32)
    scale = (s.astype(np.uint32) << 23).view(np.float32)
    v = e4m3_decode(q.reshape(rows, cols)).reshape(rows, cols // 32, 32) * scale[..., None]
    return v.reshape(q.shape).astype(np.float32)


# --------------------------------------------------------------------------------------
# SwiGLU and epilogues (torch, fp32)
# --------------------------------------------------------------------------------------
def router_topk(logits: np.ndarray, topk: int):
    """Routes of every token: the K largest logits in descending order (lower expert index first
    among equal values) and the softmax over those K values, in float64 then rounded to float32.
    Follows tests/utils.py:82-84."""
    logits = np.asarray(logits, dtype=np.float32)
    order = np.argsort(-logits.astype(np.float64), axis=1, kind="stable")[:, :topk]
    vals = np.take_along_axis(logits, order, axis=1).astype(np.float64)
    ex = np.exp(vals - vals[:, :1])
    return order.astype(np.int64), (ex / ex.sum(axis=1, keepdims=True)).astype(np.float32)


def router_topk_bwd(experts: np.ndarray, weights: np.ndarray, d_weights: np.ndarray, num_experts: int) -> np.ndarray:
    """Gradient of router_topk's weights with respect to the logits (softmax Jacobian on the
    selected experts, zero elsewhere)."""
    w = weights.astype(np.float64)
    dw = d_weights.astype(np.float64)
    inner = (w * dw).sum(axis=1, keepdims=True)
    d_logits = np.zeros((experts.shape[0], num_experts), dtype=np.float64)
    np.put_along_axis(d_logits, experts.astype(np.int64), w * (dw - inner), axis=1)
    return d_logits.astype(np.float32)


def swiglu_fwd(gate: torch.Tensor, up: torch.Tensor, limit: float | None) -> torch.Tensor:
    g, u = gate.float(), up.float()
    if limit is not None:
        g = g.clamp(max=limit)
        u = u.clamp(min=-limit, max=limit)
    return g / (1.0 + torch.exp(-g)) * u


def swiglu_bwd(gate: torch.Tensor, up: torch.Tensor, d_hidden: torch.Tensor, limit: float | None):
    """(d_gate, d_up, hidden) in fp32 following csrc/mok_megakernel.cuh:612-647."""
    g, u, dh = gate.float(), up.float(), d_hidden.float()
    gmask = umask = None
    if limit is not None:
        gmask = g <= limit
        umask = (u >= -limit) & (u <= limit)
        g = g.clamp(max=limit)
        u = u.clamp(min=-limit, max=limit)
    sig = 1.0 / (1.0 + torch.exp(-g))
    silu = g * sig
    dsilu = (1.0 - silu) * sig + silu
    d_gate = dsilu * u * dh
    d_up = silu * dh
    if limit is not None:
        d_gate = torch.where(gmask, d_gate, torch.zeros_like(d_gate))
        d_up = torch.where(umask, d_up, torch.zeros_like(d_up))
    return d_gate, d_up, silu * u


def fwd_epilogue(y_shared, combine_buffer, topk_weights):
    T, H = y_shared.shape
    K = topk_weights.shape[1]
    acc = y_shared.float().clone()
    routed = combine_buffer.view(T, K, H).float()
    for k in range(K):                                   # fixed k order, csrc/utils.cuh:107-111
        acc += routed[:, k] * topk_weights[:, k:k + 1]
    return acc.to(torch.bfloat16)


def bwd_epilogue(d_x_shared, d_x_routed_buffer):
    T, H = d_x_shared.shape
    K = d_x_routed_buffer.shape[0] // T
    acc = d_x_shared.float().clone()
    routed = d_x_routed_buffer.view(T, K, H).float()
    for k in range(K):
        acc += routed[:, k]
    return acc.to(torch.bfloat16)


# --------------------------------------------------------------------------------------
# Whole layer, W virtual ranks in one process
# --------------------------------------------------------------------------------------
@dataclass
class RankInputs:
    x: torch.Tensor                # [T, H]
    topk_experts: torch.Tensor     # [T, K] int64
    router_weights: torch.Tensor   # [T, K] f32
    w_shared_gate: torch.Tensor    # [I, H]
    w_shared_up: torch.Tensor      # [I, H]
    w_shared_down: torch.Tensor    # [H, I]
    w_routed_gate: torch.Tensor    # [El, I, H]
    w_routed_up: torch.Tensor      # [El, I, H]
    w_routed_down: torch.Tensor    # [El, H, I]
    d_output: torch.Tensor | None  # [T, H]


def _rd(t: torch.Tensor, device_rounding: bool) -> torch.Tensor:
    """Round to bf16 where the device path stores bf16; identity in ideal-fp32 mode."""
    return t.to(torch.bfloat16).float() if device_rounding else t


def _mx(t: torch.Tensor, axis: int) -> torch.Tensor:
    """Quantise-dequantise a 2-D fp32 tensor (already bf16-rounded) in 1x32 blocks along
    `axis` — what an MXFP8 GEMM operand contributes numerically."""
    a = t.numpy()
    if axis == 0:
        a = np.ascontiguousarray(a.T)
    q, s = mx_block_quantize(a)
    scale = (s.astype(np.uint32) << 23).view(np.float32)
    v = (e4m3_decode(q).reshape(*s.shape, 32) * scale[..., None]).reshape(a.shape)
    if axis == 0:
        v = np.ascontiguousarray(v.T)
    return torch.from_numpy(v.astype(np.float32))


def layer_forward_backward(ranks: list[RankInputs], *, swiglu_limit: float | None = None,
                           device_rounding: bool = True, mxfp8: bool = False,
                           capacity: int | None = None, backward: bool = True):
    """Forward (+ backward) of the expert-parallel MoE layer over len(ranks) virtual ranks.

    The all-to-alls of the reference oracle (tests/utils.py:274,287,400,408) become index
    shuffles through the slot tables of `schedule_tables`.  `device_rounding` inserts the
    bf16 rounding points of the device path: GEMM outputs (mok_megakernel.cuh:1499), hidden
    (:776), w*d_y (:464-467), SwiGLU grads (:634-644).  `mxfp8` additionally passes every
    routed GEMM operand through the 1x32 block quantiser along its contraction axis and the
    saved gate/up through quantise-dequantise (:992-995).  fp32 accumulation everywhere.

    Returns a list (one per rank) of dicts holding `output` and, when `backward`, the eight
    gradients of functional.backward plus the slot tables.
    """
    W = len(ranks)
    T, H = ranks[0].x.shape
    K = ranks[0].topk_experts.shape[1]
    El, I, _ = ranks[0].w_routed_gate.shape
    R = T * K
    cap = capacity if capacity is not None else R * W + El * EXPERT_PADDING   # never overflows
    topk_all = np.stack([r.topk_experts.numpy().astype(np.int32) for r in ranks])
    rd = lambda t: _rd(t, device_rounding)  # noqa: E731
    results = [dict() for _ in range(W)]
    combine = [torch.zeros(R, H) for _ in range(W)]
    d_x_routed_buf = [torch.zeros(R, H) for _ in range(W)]
    d_rw = [torch.zeros(T, K) for _ in range(W)]

    for dst in range(W):
        me = ranks[dst]
        pr, pt, ntok, tpe = schedule_tables(topk_all, El, cap, dst)
        n = int(ntok[0])
        results[dst].update(peer_rank=pr, peer_token_idx=pt, num_tokens=ntok, tokens_per_expert=tpe)
        valid = pr[:n] >= 0
        rows = np.nonzero(valid)[0]
        src_rank = pr[:n][valid]
        src_tok = pt[:n][valid]
        x_routed = torch.zeros(n, H)
        for p in range(W):
            sel = src_rank == p
            x_routed[rows[sel]] = ranks[p].x.float()[src_tok[sel] // K]
        # ---- routed forward, expert by expert
        y_routed = torch.zeros(n, H)
        gate_all = torch.zeros(n, I); up_all = torch.zeros(n, I); hid_all = torch.zeros(n, I)
        base = 0
        spans = []
        for e in range(El):
            sl = slice(base, base + int(tpe[e])); spans.append(sl); base += int(tpe[e])
            if sl.stop == sl.start:
                continue
            wg, wu, wd = me.w_routed_gate[e].float(), me.w_routed_up[e].float(), me.w_routed_down[e].float()
            xe = x_routed[sl]
            if mxfp8:
                xe_q, wg_q, wu_q, wd_q = _mx(xe, 1), _mx(wg, 1), _mx(wu, 1), _mx(wd, 1)
            else:
                xe_q, wg_q, wu_q, wd_q = xe, wg, wu, wd
            gate = rd(xe_q @ wg_q.T); up = rd(xe_q @ wu_q.T)
            hid = rd(swiglu_fwd(gate, up, swiglu_limit))
            gate_all[sl], up_all[sl], hid_all[sl] = gate, up, hid
            y_routed[sl] = rd((_mx(hid, 1) if mxfp8 else hid) @ wd_q.T)
        for p in range(W):
            sel = src_rank == p
            combine[p][src_tok[sel]] = y_routed[rows[sel]]
        results[dst]["_saved"] = (x_routed, gate_all, up_all, hid_all, spans, rows, src_rank, src_tok, n)

    # ---- shared expert + forward epilogue
    for r in range(W):
        me = ranks[r]
        xs = me.x.float()
        g = rd(xs @ me.w_shared_gate.float().T); u = rd(xs @ me.w_shared_up.float().T)
        h = rd(swiglu_fwd(g, u, swiglu_limit))
        y_sh = rd(h @ me.w_shared_down.float().T)
        results[r]["_shared"] = (g, u, h)
        results[r]["combine_buffer"] = combine[r].to(torch.bfloat16)
        results[r]["output"] = fwd_epilogue(y_sh.to(torch.bfloat16), combine[r].to(torch.bfloat16),
                                            me.router_weights)
    if not backward:
        for r in results:
            r.pop("_saved"); r.pop("_shared")
        return results

    # ---- routed backward
    for dst in range(W):
        me = ranks[dst]
        x_routed, gate_all, up_all, hid_all, spans, rows, src_rank, src_tok, n = results[dst].pop("_saved")
        w_row = torch.zeros(n)
        d_y = torch.zeros(n, H)
        for p in range(W):
            sel = src_rank == p
            w_row[rows[sel]] = ranks[p].router_weights.reshape(-1)[src_tok[sel]]
            d_y[rows[sel]] = ranks[p].d_output.float()[src_tok[sel] // K]
        d_y = rd(d_y * w_row[:, None])                       # mok_megakernel.cuh:464-467
        inv_w = torch.where(w_row > 0, 1.0 / w_row, torch.zeros_like(w_row))   # :958
        d_x_routed = torch.zeros(n, H)
        d_rw_row = torch.zeros(n)
        dwg = torch.zeros(El, I, H); dwu = torch.zeros(El, I, H); dwd = torch.zeros(El, H, I)
        for e, sl in enumerate(spans):
            if sl.stop == sl.start:
                continue
            wg, wu, wd = me.w_routed_gate[e].float(), me.w_routed_up[e].float(), me.w_routed_down[e].float()
            dy, xe, hid = d_y[sl], x_routed[sl], hid_all[sl]
            gate, up = gate_all[sl], up_all[sl]
            if mxfp8:
                gate, up = _mx(gate, 1), _mx(up, 1)          # saved as fp8, :992-995
                d_hidden = rd(_mx(dy, 1) @ _mx(wd, 0))
            else:
                d_hidden = rd(dy @ wd)
            dg, du, hid_f = swiglu_bwd(gate, up, d_hidden, swiglu_limit)
            d_rw_row[sl] = (d_hidden * inv_w[sl, None] * hid_f).sum(1)       # :1002,1135
            dg, du = rd(dg), rd(du)
            if mxfp8:
                d_x_routed[sl] = rd(_mx(dg, 1) @ _mx(wg, 0) + _mx(du, 1) @ _mx(wu, 0))
                dwd[e] = _mx(dy, 0).T @ _mx(hid, 0)
                dwg[e] = _mx(dg, 0).T @ _mx(xe, 0)
                dwu[e] = _mx(du, 0).T @ _mx(xe, 0)
            else:
                d_x_routed[sl] = rd(dg @ wg + du @ wu)
                dwd[e] = dy.T @ hid
                dwg[e] = dg.T @ xe
                dwu[e] = du.T @ xe
        for p in range(W):
            sel = src_rank == p
            d_x_routed_buf[p][src_tok[sel]] = d_x_routed[rows[sel]]
            d_rw[p].reshape(-1)[src_tok[sel]] = d_rw_row[rows[sel]]
        results[dst]["d_w_routed_gate"] = dwg.to(torch.bfloat16)
        results[dst]["d_w_routed_up"] = dwu.to(torch.bfloat16)
        results[dst]["d_w_routed_down"] = dwd.to(torch.bfloat16)

    # ---- shared backward + backward epilogue
    for r in range(W):
        me = ranks[r]
        g, u, h = results[r].pop("_shared")
        dy = me.d_output.float()
        xs = me.x.float()
        d_h = rd(dy @ me.w_shared_down.float())
        dg, du, _ = swiglu_bwd(g, u, d_h, swiglu_limit)
        dg, du = rd(dg), rd(du)
        d_x_sh = rd(dg @ me.w_shared_gate.float() + du @ me.w_shared_up.float())
        results[r]["d_w_shared_down"] = (dy.T @ h).to(torch.bfloat16)
        results[r]["d_w_shared_gate"] = (dg.T @ xs).to(torch.bfloat16)
        results[r]["d_w_shared_up"] = (du.T @ xs).to(torch.bfloat16)
        results[r]["d_x"] = bwd_epilogue(d_x_sh.to(torch.bfloat16), d_x_routed_buf[r].to(torch.bfloat16))
        results[r]["d_router_weights"] = d_rw[r]
    return results


# --------------------------------------------------------------------------------------
# Synthetic inputs (the configurations the benchmark and the parity tests share)
# --------------------------------------------------------------------------------------
def make_rank_inputs(rank: int, *, T: int, H: int, I: int, E: int, W: int, K: int, seed: int = 0,
                     router: str = "linear", zipf_s: float | None = None,
                     with_grad: bool = True) -> RankInputs:
    """Seeded CPU inputs: x~N(0,1) bf16, router W_r~N(0,0.02) -> softmax -> top-K ->
    renormalise (or uniform-random logits with router="uniform"), expert weights
    ~N(0, 1/sqrt(fan_in)) bf16, upstream grad ~N(0,1) bf16.  `zipf_s` adds log p_e with
    p_e ∝ (e+1)^-s to the logits (skewed-routing stress)."""
    g = torch.Generator().manual_seed(seed * 1000003 + rank)
    El = E // W
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    if router == "linear":
        w_r = torch.randn(E, H, generator=g) * 0.02
        logits = x.float() @ w_r.T
    else:
        logits = torch.rand(T, E, generator=g)
    if zipf_s is not None:
        p = (torch.arange(E, dtype=torch.float32) + 1.0) ** (-zipf_s)
        logits = logits + torch.log(p / p.sum())
    probs = torch.softmax(logits, dim=-1)
    vals, idx = torch.topk(probs, K, dim=-1)
    weights = (vals / vals.sum(-1, keepdim=True)).float()
    gw = torch.Generator().manual_seed(seed * 1000003 + 7919 + rank)
    mk = lambda *s, fan: (torch.randn(*s, generator=gw) * fan ** -0.5).to(torch.bfloat16)  # noqa: E731
    d_out = torch.randn(T, H, generator=g).to(torch.bfloat16) if with_grad else None
    return RankInputs(
        x=x, topk_experts=idx.to(torch.int64), router_weights=weights,
        w_shared_gate=mk(I, H, fan=H), w_shared_up=mk(I, H, fan=H), w_shared_down=mk(H, I, fan=I),
        w_routed_gate=mk(El, I, H, fan=H), w_routed_up=mk(El, I, H, fan=H),
        w_routed_down=mk(El, H, I, fan=I), d_output=d_out)


def layer_flops(T: int, K: int, H: int, I: int, backward: bool) -> float:
    """Reference FLOP convention (benchmarks/utils.py:19-23): 6*(T + T*K)*H*I forward,
    twice that again for backward; padding rows and replay are not counted."""
    f = 6.0 * (T + T * K) * H * I
    return f * 3.0 if backward else f
