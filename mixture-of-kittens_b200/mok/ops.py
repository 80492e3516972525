"""The ten `mok::*` operators, same names, argument order and validation behaviour as
Mixture-of-Kittens' `mok/ops.py` (reference lines cited per operator), implemented on top of
the C ABI of libmok_b200.so.  Outputs are allocated here with torch (stream-ordered caching
allocator); the native side only receives raw device pointers.

Deliberate differences from the reference:
  * expert-parallel sizes 1, 2, 4 and 8 are accepted (the reference accepts 4..64); one NVSwitch
    box holds at most eight ranks;
  * the top-k all-gather uses per-peer stores, so the multicast pointer may be 0 when the
    workspace registered the peer addresses of its buffer (see `_lib.register_all_gather_peers`).
"""
from __future__ import annotations

import torch

from . import _lib

Tensor = torch.Tensor
_EP_SIZES = (1, 2, 4, 8)
_EP_TEXT = "1, 2, 4, 8"


# ------------------------------------------------------------------------------------------
# shared validators (exception classes follow the reference's negative-argument tables)
# ------------------------------------------------------------------------------------------
def _need(cond: bool, message: str, exc=ValueError) -> None:
    if not cond:
        raise exc(message)


def _token_hidden(t: Tensor, what: str) -> tuple[int, int]:
    _need(t.ndim == 2, f"{what} must have shape (num_local_tokens, hidden_size)")
    tokens, hidden = t.shape
    _need(tokens >= 512 and tokens % 256 == 0, "num_local_tokens must be at least 512 and divisible by 256")
    _need(hidden > 0 and hidden % 256 == 0, "hidden_size must be positive and divisible by 256")
    return tokens, hidden


def _layer_scalars(topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size) -> None:
    _need(type(topk) is int and 0 < topk <= 255, "topk must be an integer in [1, 255]")
    _need(swiglu_limit is None or (type(swiglu_limit) in (int, float) and swiglu_limit >= 0),
          "swiglu_limit must be None or a non-negative number")
    _need(type(num_comm_sms) is int and num_comm_sms > 0 and num_comm_sms % 2 == 0,
          "num_comm_sms must be a positive even integer")
    _need(type(minibatch_size) is int and minibatch_size > 0 and minibatch_size % 256 == 0,
          "minibatch_size must be positive and divisible by 256")
    _need(type(macrobatch_size) is int and macrobatch_size > 0 and macrobatch_size % minibatch_size == 0,
          "macrobatch_size must be a positive multiple of minibatch_size")


# A pointer list equal to SELF_PTRS stands for "one rank: the address of the tensor passed beside it".  It keeps
# data_ptr() calls out of the caller, so the single-rank path stays traceable by torch.compile.
SELF_PTRS = [-1]


def _self_ptrs(local: Tensor, ptrs: list[int]) -> list[int]:
    return [local.data_ptr()] if list(ptrs) == SELF_PTRS else ptrs


def _pointer_lists(named: dict[str, list[int]], lead: str) -> int:
    for name, ptrs in named.items():
        ok = isinstance(ptrs, list) and all(type(p) is int and p > 0 for p in ptrs)
        _need(ok, f"{name} must be a list of positive integers", TypeError)
    ep_size = len(named[lead])
    _need(ep_size in _EP_SIZES, f"{lead} length must be one of {_EP_TEXT}")
    for name, ptrs in named.items():
        _need(len(ptrs) == ep_size, f"{name} length must match {lead}")
    return ep_size


def _intermediate(w_shared_gate: Tensor, hidden: int, strict_cols: bool) -> int:
    ok = w_shared_gate.ndim == 2 and (not strict_cols or w_shared_gate.shape[1] == hidden)
    _need(ok, "w_shared_gate must have shape (intermediate_size, hidden_size)")
    inter = w_shared_gate.shape[0]
    _need(inter > 0 and inter % 256 == 0, "intermediate_size must be positive and divisible by 256")
    return inter


def _local_experts(w_routed_gate: Tensor) -> int:
    _need(w_routed_gate.ndim == 3 and w_routed_gate.shape[0] > 0,
          "w_routed_gate must have shape (num_local_experts, intermediate_size, hidden_size)")
    return w_routed_gate.shape[0]


def _shapes_and_devices(device, expected: list[tuple[str, Tensor, tuple]], extra: list[tuple[str, Tensor]] = ()) -> None:
    for name, t, shape in expected:
        _need(tuple(t.shape) == tuple(shape), f"{name} must have shape {tuple(shape)}")
    for name, t, _ in expected:
        _need(t.device == device, f"{name} must be on {device}")
    for name, t in extra:
        _need(t.device == device, f"{name} must be on {device}")


def _schedule_capacity(schedule_peer_rank: Tensor) -> int:
    _need(schedule_peer_rank.ndim == 1 and schedule_peer_rank.numel() > 0,
          "schedule_peer_rank must be a nonempty 1D tensor")
    cap = schedule_peer_rank.numel()
    _need(cap % 256 == 0, "schedule_capacity must be divisible by 256")
    return cap


def _vp(t: Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _common(x: Tensor, ep_size: int, inter: int, n_experts: int, topk: int, cap: int, macro: int, mini: int,
            comm_sms: int, limit, sched, defer_combine: bool = False) -> _lib.LayerCommon:
    peer_rank, peer_tok, num_tokens, tokens_per_expert = sched
    for name, t in (("schedule_peer_rank", peer_rank), ("schedule_peer_token_idx", peer_tok),
                    ("num_tokens", num_tokens), ("tokens_per_expert", tokens_per_expert)):
        _need(t.dtype == torch.int32 and t.is_contiguous(), f"{name} must be contiguous int32", TypeError)
    c = _lib.LayerCommon()
    c.ep_size = ep_size
    c.ep_rank = -1
    c.num_local_tokens, c.hidden = x.shape
    c.intermediate, c.num_local_experts, c.topk = inter, n_experts, topk
    c.schedule_capacity, c.macrobatch_size, c.minibatch_size, c.num_comm_sms = cap, macro, mini, comm_sms
    c.has_swiglu_limit = 0 if limit is None else 1
    c.swiglu_limit = 0.0 if limit is None else float(limit)
    if defer_combine:
        _need(ep_size == 1 and cap <= macro,
              "defer_combine needs a single rank and a schedule capacity within one macrobatch")
    c.defer_combine = 1 if defer_combine else 0
    c.schedule_peer_rank, c.schedule_peer_token_idx = peer_rank.data_ptr(), peer_tok.data_ptr()
    c.num_tokens, c.tokens_per_expert = num_tokens.data_ptr(), tokens_per_expert.data_ptr()
    c.status = _lib.status_tensor(x.device).data_ptr()
    return c


def _own_rank(local: Tensor, ptrs: list[int], name: str) -> int:
    try:
        return ptrs.index(local.data_ptr())
    except ValueError:
        raise ValueError(f"{name} must contain the address of the local buffer") from None


def _bf16(named: dict[str, Tensor]) -> None:
    for name, t in named.items():
        _need(t.dtype == torch.bfloat16 and t.is_contiguous(), f"{name} must be contiguous bfloat16", TypeError)


# ------------------------------------------------------------------------------------------
# all_gather_top_experts  (reference mok/ops.py:6-58)
# ------------------------------------------------------------------------------------------
@torch.library.custom_op("mok::all_gather_top_experts", mutates_args=("all_gather_top_experts_buffer",))
def all_gather_top_experts(top_experts: Tensor, all_gather_top_experts_buffer: Tensor,
                           all_gather_top_experts_buffer_multicast_ptr: int, rank: int, chunk_bytes: int) -> None:
    buf = all_gather_top_experts_buffer
    _need(top_experts.is_cuda and top_experts.dtype == torch.int32 and top_experts.is_contiguous()
          and top_experts.ndim == 2, "top_experts must be contiguous CUDA int32 [num_local_tokens, topk]")
    _need(buf.is_cuda, "all_gather_top_experts_buffer must be a CUDA tensor")
    _need(buf.dtype == torch.int32, "all_gather_top_experts_buffer must have dtype torch.int32", TypeError)
    _need(buf.is_contiguous(), "all_gather_top_experts_buffer must be contiguous")
    _need(buf.ndim == 3, "all_gather_top_experts_buffer must have shape (ep_size, num_local_tokens, topk)")
    _need(all(s > 0 for s in top_experts.shape), "top_experts dimensions must be positive")
    _need(all(s > 0 for s in buf.shape), "all_gather_top_experts_buffer dimensions must be positive")
    ep_size = buf.shape[0]
    _need(ep_size in _EP_SIZES, f"all_gather_top_experts_buffer ep_size must be one of {_EP_TEXT}")
    _need(buf.device == top_experts.device and tuple(buf.shape[1:]) == tuple(top_experts.shape),
          "all_gather_top_experts_buffer must match top_experts shape and device")
    mc = all_gather_top_experts_buffer_multicast_ptr
    _need(type(mc) is int and mc >= 0, "all_gather_top_experts_buffer_multicast_ptr must be a non-negative integer",
          TypeError)
    _need(type(rank) is int and 0 <= rank < ep_size, "rank must be an integer in [0, ep_size)")
    _need(type(chunk_bytes) is int and chunk_bytes > 0, "chunk_bytes must be a positive integer")
    _need(chunk_bytes % 16 == 0, "chunk_bytes must be divisible by 16")
    _need((top_experts.numel() * 4) % chunk_bytes == 0, "chunk_bytes must divide one rank's route-buffer bytes")

    peers = _lib.all_gather_peers(buf.data_ptr())
    if peers is None:
        _need(ep_size == 1, "all_gather_top_experts_buffer has no registered peer addresses; create it through "
                            "mok.functional.create_workspace", RuntimeError)
        peers = [buf.data_ptr()]
    _lib.check(_lib.mok_all_gather_top_experts(top_experts.data_ptr(), top_experts.numel(), _lib.ptr_array(peers),
                                               ep_size, rank, _lib.stream_ptr(buf.device)), "all_gather_top_experts")


# ------------------------------------------------------------------------------------------
# barrier_all  (reference mok/ops.py:61-100)
# ------------------------------------------------------------------------------------------
@torch.library.custom_op("mok::barrier_all", mutates_args=("barrier_buffer", "target"))
def barrier_all(barrier_buffer: Tensor, barrier_buffer_ptrs: list[int], barrier_buffer_multicast_ptr: int,
                target: Tensor) -> None:
    _need(barrier_buffer.is_cuda, "barrier_buffer must be a CUDA tensor")
    _need(barrier_buffer.dtype == torch.int32, "barrier_buffer must have dtype torch.int32", TypeError)
    _need(barrier_buffer.is_contiguous(), "barrier_buffer must be contiguous")
    _need(tuple(barrier_buffer.shape) == (1,), "barrier_buffer must have shape (1,)")
    ok = isinstance(barrier_buffer_ptrs, list) and all(type(p) is int and p > 0 for p in barrier_buffer_ptrs)
    _need(ok, "barrier_buffer_ptrs must be a list of positive integers", TypeError)
    ep_size = len(barrier_buffer_ptrs)
    _need(ep_size in _EP_SIZES, f"barrier_buffer_ptrs length must be one of {_EP_TEXT}")
    mc = barrier_buffer_multicast_ptr
    _need(type(mc) is int and mc >= 0, "barrier_buffer_multicast_ptr must be a non-negative integer", TypeError)
    _need(target.is_cuda and target.device == barrier_buffer.device and target.dtype == torch.int32
          and target.is_contiguous() and tuple(target.shape) == (1,),
          "target must be contiguous int32 [1] on the barrier CUDA device")
    dev = barrier_buffer.device
    _lib.check(_lib.mok_barrier_all(barrier_buffer.data_ptr(), _lib.ptr_array(barrier_buffer_ptrs), ep_size,
                                    target.data_ptr(), _lib.status_tensor(dev).data_ptr(), 0, _lib.stream_ptr(dev)),
               "barrier_all")


# ------------------------------------------------------------------------------------------
# schedule  (reference mok/ops.py:103-150)
# ------------------------------------------------------------------------------------------
@torch.library.custom_op("mok::schedule", mutates_args=())
def schedule(topk_all: Tensor, num_local_experts: int, schedule_capacity: int,
             rank: int) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    _need(topk_all.ndim == 3, "topk_all must have shape (ep_size, num_local_tokens, topk)")
    ep_size, tokens, topk = topk_all.shape
    _need(ep_size in _EP_SIZES, f"topk_all ep_size must be one of {_EP_TEXT}")
    _need(tokens >= 512 and tokens % 256 == 0, "topk_all num_local_tokens must be at least 512 and divisible by 256")
    _need(0 < topk <= 255, "topk_all topk must be in [1, 255]")
    _need(type(num_local_experts) is int and num_local_experts > 0, "num_local_experts must be a positive integer")
    _need(type(schedule_capacity) is int and schedule_capacity > 0 and schedule_capacity % 256 == 0,
          "schedule_capacity must be positive and divisible by 256")
    _need(schedule_capacity >= tokens * topk, "schedule_capacity must hold at least one rank's routed tokens")
    _need(type(rank) is int and 0 <= rank < ep_size, "rank must be an integer in [0, ep_size)")
    _need(topk_all.is_cuda and topk_all.dtype == torch.int32 and topk_all.is_contiguous(),
          "topk_all must be a contiguous CUDA int32 tensor", TypeError)
    _need(num_local_experts <= _lib.MAX_LOCAL_EXPERTS, "num_local_experts exceeds this build's limit of 1024",
          NotImplementedError)

    dev = topk_all.device
    i32 = dict(dtype=torch.int32, device=dev)
    peer_rank = torch.empty(schedule_capacity, **i32)
    peer_tok = torch.empty(schedule_capacity, **i32)
    num_tokens = torch.empty(1, **i32)
    tokens_per_expert = torch.empty(num_local_experts, **i32)
    scratch_bytes = _lib.mok_schedule_scratch_bytes(ep_size, num_local_experts)
    scratch = torch.empty(scratch_bytes, dtype=torch.uint8, device=dev)
    _lib.check(_lib.mok_schedule(topk_all.data_ptr(), ep_size, tokens, topk, num_local_experts, schedule_capacity, rank,
                                 peer_rank.data_ptr(), peer_tok.data_ptr(), num_tokens.data_ptr(),
                                 tokens_per_expert.data_ptr(), scratch.data_ptr(), scratch_bytes,
                                 _lib.status_tensor(dev).data_ptr(), _lib.stream_ptr(dev)), "schedule")
    return peer_rank, peer_tok, num_tokens, tokens_per_expert


# ------------------------------------------------------------------------------------------
# mxfp8_quantize  (reference mok/ops.py:153-191)
# ------------------------------------------------------------------------------------------
@torch.library.custom_op(
    "mok::mxfp8_quantize", mutates_args=(),
    schema="(Tensor x_bf16, bool return_normal, bool return_transposed) -> (Tensor?, Tensor?, Tensor?, Tensor?)")
def mxfp8_quantize(x_bf16: Tensor, return_normal: bool,
                   return_transposed: bool) -> tuple[Tensor | None, Tensor | None, Tensor | None, Tensor | None]:
    _need(x_bf16.ndim in (2, 3), "x_bf16 must have shape (M, N) or (E, M, N)")
    _need(all(s > 0 for s in x_bf16.shape), "x_bf16 dimensions must be positive")
    _need(x_bf16.shape[-2] % 128 == 0 and x_bf16.shape[-1] % 128 == 0,
          "x_bf16 M and N dimensions must be divisible by 128")
    _need(type(return_normal) is bool and type(return_transposed) is bool,
          "return_normal and return_transposed must be booleans", TypeError)
    _need(return_normal or return_transposed, "at least one quantized layout must be requested")
    _need(x_bf16.is_cuda and x_bf16.dtype == torch.bfloat16 and x_bf16.is_contiguous(),
          "x_bf16 must be a contiguous CUDA bfloat16 tensor", TypeError)

    n_mat = x_bf16.shape[0] if x_bf16.ndim == 3 else 1
    rows, cols = x_bf16.shape[-2:]
    dev = x_bf16.device
    q = sc = qt = sct = None
    if return_normal:
        q = torch.empty(x_bf16.shape, dtype=torch.float8_e4m3fn, device=dev)
        sc = torch.empty(n_mat * rows // 128, cols // 128, 32, 16, dtype=torch.uint8, device=dev)
    if return_transposed:
        t_shape = (n_mat, cols, rows) if x_bf16.ndim == 3 else (cols, rows)
        qt = torch.empty(t_shape, dtype=torch.float8_e4m3fn, device=dev)
        sct = torch.empty(n_mat * cols // 128, rows // 128, 32, 16, dtype=torch.uint8, device=dev)
    _lib.check(_lib.mok_mxfp8_quantize(x_bf16.data_ptr(), n_mat, rows, cols, _vp(q), _vp(sc), _vp(qt), _vp(sct),
                                       _lib.stream_ptr(dev)), "mxfp8_quantize")
    return q, sc, qt, sct


# ------------------------------------------------------------------------------------------
# forward, BF16 routed experts  (reference mok/ops.py:371-514)
# ------------------------------------------------------------------------------------------
@torch.library.custom_op("mok::dispatch_mlp_swiglu_combine_fwd_bf16", mutates_args=("combine_buffer",))
def dispatch_mlp_swiglu_combine_fwd_bf16(
    x: Tensor, x_ptrs: list[int], combine_buffer: Tensor, combine_buffer_ptrs: list[int],
    w_shared_gate: Tensor, w_routed_gate: Tensor, w_shared_up: Tensor, w_routed_up: Tensor,
    w_shared_down: Tensor, w_routed_down: Tensor,
    schedule_peer_rank: Tensor, schedule_peer_token_idx: Tensor, num_tokens: Tensor, tokens_per_expert: Tensor,
    topk: int, swiglu_limit: float | None, num_comm_sms: int, macrobatch_size: int, minibatch_size: int,
    defer_combine: bool = False,
) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    x_ptrs = _self_ptrs(x, x_ptrs)
    T, H = _token_hidden(x, "x")
    I = _intermediate(w_shared_gate, H, strict_cols=True)
    El = _local_experts(w_routed_gate)
    _layer_scalars(topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size)
    ep_size = _pointer_lists({"x_ptrs": x_ptrs, "combine_buffer_ptrs": combine_buffer_ptrs}, "x_ptrs")
    cap = _schedule_capacity(schedule_peer_rank)
    _shapes_and_devices(x.device, [
        ("combine_buffer", combine_buffer, (T * topk, H)),
        ("w_shared_gate", w_shared_gate, (I, H)), ("w_routed_gate", w_routed_gate, (El, I, H)),
        ("w_shared_up", w_shared_up, (I, H)), ("w_routed_up", w_routed_up, (El, I, H)),
        ("w_shared_down", w_shared_down, (H, I)), ("w_routed_down", w_routed_down, (El, H, I)),
        ("schedule_peer_token_idx", schedule_peer_token_idx, (cap,)),
        ("num_tokens", num_tokens, (1,)), ("tokens_per_expert", tokens_per_expert, (El,)),
    ], [("schedule_peer_rank", schedule_peer_rank)])
    _bf16({"x": x, "combine_buffer": combine_buffer, "w_shared_gate": w_shared_gate, "w_routed_gate": w_routed_gate,
           "w_shared_up": w_shared_up, "w_routed_up": w_routed_up, "w_shared_down": w_shared_down,
           "w_routed_down": w_routed_down})

    bf = dict(dtype=torch.bfloat16, device=x.device)
    MB = macrobatch_size
    x_routed = torch.empty(MB, H, **bf)
    gate_shared, up_shared, hidden_shared = (torch.empty(T, I, **bf) for _ in range(3))
    gate_routed, up_routed, hidden_routed = (torch.empty(MB, I, **bf) for _ in range(3))
    y_shared = torch.empty(T, H, **bf)
    y_routed = torch.empty(MB, H, **bf)

    a = _lib.FwdBf16Args()
    a.c = _common(x, ep_size, I, El, topk, cap, MB, minibatch_size, num_comm_sms, swiglu_limit,
                  (schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert), defer_combine)
    a.c.ep_rank = _own_rank(x, x_ptrs, "x_ptrs")
    xp, cp = _lib.ptr_array(x_ptrs), _lib.ptr_array(combine_buffer_ptrs)
    a.x_ptrs, a.combine_buffer_ptrs = xp, cp
    a.w_shared_gate, a.w_shared_up, a.w_shared_down = (t.data_ptr() for t in (w_shared_gate, w_shared_up, w_shared_down))
    a.w_routed_gate, a.w_routed_up, a.w_routed_down = (t.data_ptr() for t in (w_routed_gate, w_routed_up, w_routed_down))
    a.x_routed = x_routed.data_ptr()
    a.gate_shared, a.up_shared, a.hidden_shared = (t.data_ptr() for t in (gate_shared, up_shared, hidden_shared))
    a.gate_routed, a.up_routed, a.hidden_routed = (t.data_ptr() for t in (gate_routed, up_routed, hidden_routed))
    a.y_shared, a.y_routed = y_shared.data_ptr(), y_routed.data_ptr()
    _lib.check(_lib.mok_fwd_bf16(a, _lib.stream_ptr(x.device)), "dispatch_mlp_swiglu_combine_fwd_bf16")
    return (x_routed, gate_shared, gate_routed, up_shared, up_routed, hidden_shared, hidden_routed, y_shared, y_routed)


# ------------------------------------------------------------------------------------------
# backward, BF16 routed experts  (reference mok/ops.py:811-1008)
# ------------------------------------------------------------------------------------------
@torch.library.custom_op(
    "mok::dispatch_mlp_swiglu_combine_bwd_bf16",
    mutates_args=("d_x_routed_buffer", "d_router_weight_buffer", "x_routed", "gate_routed", "up_routed", "hidden_routed"))
def dispatch_mlp_swiglu_combine_bwd_bf16(
    d_y_buffer: Tensor, d_y_buffer_ptrs: list[int], d_x_routed_buffer: Tensor, d_x_routed_buffer_ptrs: list[int],
    router_weight_buffer: Tensor, router_weight_buffer_ptrs: list[int],
    d_router_weight_buffer: Tensor, d_router_weight_buffer_ptrs: list[int],
    w_shared_gate: Tensor, w_routed_gate: Tensor, w_shared_up: Tensor, w_routed_up: Tensor,
    w_shared_down: Tensor, w_routed_down: Tensor,
    x_routed: Tensor, gate_shared: Tensor, gate_routed: Tensor, up_shared: Tensor, up_routed: Tensor,
    hidden_shared: Tensor, hidden_routed: Tensor, x: Tensor, x_ptrs: list[int],
    schedule_peer_rank: Tensor, schedule_peer_token_idx: Tensor, num_tokens: Tensor, tokens_per_expert: Tensor,
    topk: int, swiglu_limit: float | None, num_comm_sms: int, macrobatch_size: int, minibatch_size: int,
    defer_combine: bool = False,
) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor,
           Tensor, Tensor]:
    x_ptrs, d_y_buffer_ptrs = _self_ptrs(x, x_ptrs), _self_ptrs(d_y_buffer, d_y_buffer_ptrs)
    router_weight_buffer_ptrs = _self_ptrs(router_weight_buffer, router_weight_buffer_ptrs)
    T, H = _token_hidden(x, "x")
    I = _intermediate(w_shared_gate, H, strict_cols=True)
    El = _local_experts(w_routed_gate)
    _layer_scalars(topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size)
    ep_size = _pointer_lists({"x_ptrs": x_ptrs, "d_y_buffer_ptrs": d_y_buffer_ptrs,
                              "d_x_routed_buffer_ptrs": d_x_routed_buffer_ptrs,
                              "router_weight_buffer_ptrs": router_weight_buffer_ptrs,
                              "d_router_weight_buffer_ptrs": d_router_weight_buffer_ptrs}, "x_ptrs")
    cap = _schedule_capacity(schedule_peer_rank)
    MB = macrobatch_size
    _shapes_and_devices(x.device, [
        ("d_y_buffer", d_y_buffer, (T, H)), ("d_x_routed_buffer", d_x_routed_buffer, (T * topk, H)),
        ("router_weight_buffer", router_weight_buffer, (T, topk)),
        ("d_router_weight_buffer", d_router_weight_buffer, (T, topk)),
        ("w_shared_gate", w_shared_gate, (I, H)), ("w_routed_gate", w_routed_gate, (El, I, H)),
        ("w_shared_up", w_shared_up, (I, H)), ("w_routed_up", w_routed_up, (El, I, H)),
        ("w_shared_down", w_shared_down, (H, I)), ("w_routed_down", w_routed_down, (El, H, I)),
        ("x_routed", x_routed, (MB, H)),
        ("gate_shared", gate_shared, (T, I)), ("gate_routed", gate_routed, (MB, I)),
        ("up_shared", up_shared, (T, I)), ("up_routed", up_routed, (MB, I)),
        ("hidden_shared", hidden_shared, (T, I)), ("hidden_routed", hidden_routed, (MB, I)),
        ("schedule_peer_token_idx", schedule_peer_token_idx, (cap,)),
        ("num_tokens", num_tokens, (1,)), ("tokens_per_expert", tokens_per_expert, (El,)),
    ], [("schedule_peer_rank", schedule_peer_rank)])
    _bf16({"x": x, "d_y_buffer": d_y_buffer, "d_x_routed_buffer": d_x_routed_buffer,
           "w_shared_gate": w_shared_gate, "w_routed_gate": w_routed_gate, "w_shared_up": w_shared_up,
           "w_routed_up": w_routed_up, "w_shared_down": w_shared_down, "w_routed_down": w_routed_down,
           "x_routed": x_routed, "gate_shared": gate_shared, "gate_routed": gate_routed, "up_shared": up_shared,
           "up_routed": up_routed, "hidden_shared": hidden_shared, "hidden_routed": hidden_routed})
    for name, t in (("router_weight_buffer", router_weight_buffer), ("d_router_weight_buffer", d_router_weight_buffer)):
        _need(t.dtype == torch.float32 and t.is_contiguous(), f"{name} must be contiguous float32", TypeError)

    dev = x.device
    bf = dict(dtype=torch.bfloat16, device=dev)
    d_x_shared = torch.empty(T, H, **bf)
    d_x_routed = torch.empty(MB, H, **bf)
    d_gate_shared, d_up_shared, d_hidden_shared = (torch.empty(T, I, **bf) for _ in range(3))
    d_gate_routed, d_up_routed, d_hidden_routed = (torch.empty(MB, I, **bf) for _ in range(3))
    d_y_routed = torch.empty(MB, H, **bf)
    d_w_shared_gate, d_w_shared_up = torch.empty(I, H, **bf), torch.empty(I, H, **bf)
    d_w_shared_down = torch.empty(H, I, **bf)
    d_w_routed_gate, d_w_routed_up = torch.empty(El, I, H, **bf), torch.empty(El, I, H, **bf)
    d_w_routed_down = torch.empty(El, H, I, **bf)
    row_weights = torch.empty(MB, dtype=torch.float32, device=dev)
    partials = torch.empty(MB, I // 128, dtype=torch.float32, device=dev)

    a = _lib.BwdBf16Args()
    a.c = _common(x, ep_size, I, El, topk, cap, MB, minibatch_size, num_comm_sms, swiglu_limit,
                  (schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert), defer_combine)
    a.c.ep_rank = _own_rank(x, x_ptrs, "x_ptrs")
    keep = [_lib.ptr_array(p) for p in (d_y_buffer_ptrs, d_x_routed_buffer_ptrs, router_weight_buffer_ptrs,
                                        d_router_weight_buffer_ptrs, x_ptrs)]
    a.d_y_ptrs, a.d_x_routed_buffer_ptrs, a.router_weight_ptrs, a.d_router_weight_ptrs, a.x_ptrs = keep
    a.w_shared_gate, a.w_shared_up, a.w_shared_down = (t.data_ptr() for t in (w_shared_gate, w_shared_up, w_shared_down))
    a.w_routed_gate, a.w_routed_up, a.w_routed_down = (t.data_ptr() for t in (w_routed_gate, w_routed_up, w_routed_down))
    a.x_routed, a.gate_routed, a.up_routed, a.hidden_routed = (t.data_ptr() for t in (x_routed, gate_routed, up_routed, hidden_routed))
    a.gate_shared, a.up_shared, a.hidden_shared = (t.data_ptr() for t in (gate_shared, up_shared, hidden_shared))
    a.d_x_shared, a.d_x_routed = d_x_shared.data_ptr(), d_x_routed.data_ptr()
    a.d_gate_shared, a.d_up_shared, a.d_hidden_shared = (t.data_ptr() for t in (d_gate_shared, d_up_shared, d_hidden_shared))
    a.d_gate_routed, a.d_up_routed, a.d_hidden_routed = (t.data_ptr() for t in (d_gate_routed, d_up_routed, d_hidden_routed))
    a.d_y_routed = d_y_routed.data_ptr()
    a.d_w_shared_gate, a.d_w_shared_up, a.d_w_shared_down = (t.data_ptr() for t in (d_w_shared_gate, d_w_shared_up, d_w_shared_down))
    a.d_w_routed_gate, a.d_w_routed_up, a.d_w_routed_down = (t.data_ptr() for t in (d_w_routed_gate, d_w_routed_up, d_w_routed_down))
    a.router_weights_routed, a.d_router_weight_partials = row_weights.data_ptr(), partials.data_ptr()
    _lib.check(_lib.mok_bwd_bf16(a, _lib.stream_ptr(dev)), "dispatch_mlp_swiglu_combine_bwd_bf16")
    if defer_combine:      # no combine ran: gather the rows here; d_x_shared becomes d_x, the router gradients land in the buffer
        route_row = torch.empty(T * topk, dtype=torch.int32, device=dev)
        _lib.check(_lib.mok_bwd_epilogue_rows(
            d_x_shared.data_ptr(), d_x_routed.data_ptr(), partials.data_ptr(), partials.shape[1], schedule_peer_rank.data_ptr(),
            schedule_peer_token_idx.data_ptr(), num_tokens.data_ptr(), route_row.data_ptr(), d_x_shared.data_ptr(),
            d_router_weight_buffer.data_ptr(), T, H, topk, MB, _lib.stream_ptr(dev)), "bwd_epilogue_rows")
    return (d_x_shared, d_x_routed, d_gate_shared, d_gate_routed, d_up_shared, d_up_routed, d_hidden_shared,
            d_hidden_routed, d_y_routed, d_w_shared_gate, d_w_routed_gate, d_w_shared_up, d_w_routed_up,
            d_w_shared_down, d_w_routed_down)


# ------------------------------------------------------------------------------------------
# epilogues  (reference mok/ops.py:1011-1081)
# ------------------------------------------------------------------------------------------
@torch.library.custom_op("mok::fwd_epilogue", mutates_args=())
def fwd_epilogue(y_shared: Tensor, combine_buffer: Tensor, topk_weights: Tensor) -> Tensor:
    T, H = _token_hidden(y_shared, "y_shared")
    _need(topk_weights.device == y_shared.device and combine_buffer.device == y_shared.device,
          "all tensors must be on the same CUDA device")
    _need(topk_weights.ndim == 2 and topk_weights.shape[0] == T, "topk_weights must have shape (num_local_tokens, topk)")
    topk = topk_weights.shape[1]
    _need(0 < topk <= 255, "topk must be in [1, 255]")
    _need(tuple(combine_buffer.shape) == (T * topk, H), "combine_buffer must have shape (num_local_tokens * topk, hidden_size)")
    _bf16({"y_shared": y_shared, "combine_buffer": combine_buffer})
    _need(topk_weights.dtype == torch.float32 and topk_weights.is_contiguous(),
          "topk_weights must be contiguous float32", TypeError)
    out = torch.empty_like(y_shared)
    _lib.check(_lib.mok_fwd_epilogue(y_shared.data_ptr(), combine_buffer.data_ptr(), topk_weights.data_ptr(),
                                     out.data_ptr(), T, H, topk, _lib.stream_ptr(y_shared.device)), "fwd_epilogue")
    return out


@torch.library.custom_op("mok::fwd_epilogue_rows", mutates_args=())
def fwd_epilogue_rows(y_shared: Tensor, y_routed: Tensor, schedule_peer_rank: Tensor, schedule_peer_token_idx: Tensor,
                      num_tokens: Tensor, topk_weights: Tensor) -> Tensor:
    """Single-rank forward epilogue that reads the routed rows where the down GEMM left them.

    Follows a forward op called with ``defer_combine=True``; gives the bytes ``fwd_epilogue`` gives after a
    combine.  No reference counterpart (the reference always goes through the combine buffer,
    mok/functional.py:569-571)."""
    T, H = _token_hidden(y_shared, "y_shared")
    _need(topk_weights.ndim == 2 and topk_weights.shape[0] == T, "topk_weights must have shape (num_local_tokens, topk)")
    topk = topk_weights.shape[1]
    _need(0 < topk <= 255, "topk must be in [1, 255]")
    _need(y_routed.ndim == 2 and y_routed.shape[1] == H and y_routed.shape[0] > 0,
          "y_routed must have shape (macrobatch_size, hidden_size)")
    for name, t in (("y_routed", y_routed), ("schedule_peer_rank", schedule_peer_rank),
                    ("schedule_peer_token_idx", schedule_peer_token_idx), ("num_tokens", num_tokens),
                    ("topk_weights", topk_weights)):
        _need(t.device == y_shared.device, f"{name} must be on the same CUDA device as y_shared")
    _bf16({"y_shared": y_shared, "y_routed": y_routed})
    _need(topk_weights.dtype == torch.float32 and topk_weights.is_contiguous(),
          "topk_weights must be contiguous float32", TypeError)
    for name, t in (("schedule_peer_rank", schedule_peer_rank), ("schedule_peer_token_idx", schedule_peer_token_idx),
                    ("num_tokens", num_tokens)):
        _need(t.dtype == torch.int32 and t.is_contiguous(), f"{name} must be contiguous int32", TypeError)
    _need(schedule_peer_rank.numel() == schedule_peer_token_idx.numel() and schedule_peer_rank.numel() <= y_routed.shape[0],
          "the schedule must fit in y_routed")
    out = torch.empty_like(y_shared)
    route_row = torch.empty(T * topk, dtype=torch.int32, device=y_shared.device)
    _lib.check(_lib.mok_fwd_epilogue_rows(
        y_shared.data_ptr(), y_routed.data_ptr(), schedule_peer_rank.data_ptr(), schedule_peer_token_idx.data_ptr(),
        num_tokens.data_ptr(), topk_weights.data_ptr(), route_row.data_ptr(), out.data_ptr(), T, H, topk,
        schedule_peer_rank.numel(), _lib.stream_ptr(y_shared.device)), "fwd_epilogue_rows")
    return out


@torch.library.custom_op("mok::bwd_epilogue", mutates_args=())
def bwd_epilogue(d_x_shared: Tensor, d_x_routed_buffer: Tensor) -> Tensor:
    T, H = _token_hidden(d_x_shared, "d_x_shared")
    _need(d_x_routed_buffer.device == d_x_shared.device, "d_x_routed_buffer must be on the same CUDA device")
    shape_msg = "d_x_routed_buffer must have shape (num_local_tokens * topk, hidden_size)"
    _need(d_x_routed_buffer.ndim == 2, shape_msg)
    rows = d_x_routed_buffer.shape[0]
    _need(d_x_routed_buffer.shape[1] == H and rows % T == 0 and rows != 0 and rows <= T * 255, shape_msg)
    _bf16({"d_x_shared": d_x_shared, "d_x_routed_buffer": d_x_routed_buffer})
    out = torch.empty_like(d_x_shared)
    _lib.check(_lib.mok_bwd_epilogue(d_x_shared.data_ptr(), d_x_routed_buffer.data_ptr(), out.data_ptr(), T, H,
                                     rows // T, _lib.stream_ptr(d_x_shared.device)), "bwd_epilogue")
    return out


# ------------------------------------------------------------------------------------------
# MXFP8 routed experts  (reference mok/ops.py:194-368 forward, :517-808 backward)
# ------------------------------------------------------------------------------------------
def _sc_shape(rows: int, cols: int) -> tuple[int, int, int, int]:
    return (rows // 128, cols // 128, 32, 16)


def _fp8_and_scales(named: dict[str, Tensor]) -> None:
    for name, t in named.items():
        want = torch.uint8 if name.endswith("_sc") else torch.float8_e4m3fn
        _need(t.dtype == want and t.is_contiguous(), f"{name} must be contiguous {want}", TypeError)


@torch.library.custom_op("mok::dispatch_mlp_swiglu_combine_fwd_mxfp8", mutates_args=("combine_buffer",))
def dispatch_mlp_swiglu_combine_fwd_mxfp8(
    x: Tensor, x_ptrs: list[int], combine_buffer: Tensor, combine_buffer_ptrs: list[int],
    w_shared_gate: Tensor, w_routed_gate: Tensor, w_routed_gate_sc: Tensor,
    w_shared_up: Tensor, w_routed_up: Tensor, w_routed_up_sc: Tensor,
    w_shared_down: Tensor, w_routed_down: Tensor, w_routed_down_sc: Tensor,
    schedule_peer_rank: Tensor, schedule_peer_token_idx: Tensor, num_tokens: Tensor, tokens_per_expert: Tensor,
    topk: int, swiglu_limit: float | None, num_comm_sms: int, macrobatch_size: int, minibatch_size: int,
    defer_combine: bool = False,
) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    x_ptrs = _self_ptrs(x, x_ptrs)
    T, H = _token_hidden(x, "x")
    _layer_scalars(topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size)
    ep_size = _pointer_lists({"x_ptrs": x_ptrs, "combine_buffer_ptrs": combine_buffer_ptrs}, "x_ptrs")
    I = _intermediate(w_shared_gate, H, strict_cols=False)
    El = _local_experts(w_routed_gate)
    MB = macrobatch_size
    cap_probe = schedule_peer_rank.numel() if schedule_peer_rank.ndim == 1 else 0
    _shapes_and_devices(x.device, [
        ("combine_buffer", combine_buffer, (T * topk, H)),
        ("w_shared_gate", w_shared_gate, (I, H)), ("w_routed_gate", w_routed_gate, (El, I, H)),
        ("w_routed_gate_sc", w_routed_gate_sc, _sc_shape(El * I, H)),
        ("w_shared_up", w_shared_up, (I, H)), ("w_routed_up", w_routed_up, (El, I, H)),
        ("w_routed_up_sc", w_routed_up_sc, _sc_shape(El * I, H)),
        ("w_shared_down", w_shared_down, (H, I)), ("w_routed_down", w_routed_down, (El, H, I)),
        ("w_routed_down_sc", w_routed_down_sc, _sc_shape(El * H, I)),
    ], [("schedule_peer_rank", schedule_peer_rank), ("schedule_peer_token_idx", schedule_peer_token_idx),
        ("num_tokens", num_tokens), ("tokens_per_expert", tokens_per_expert)])
    cap = _schedule_capacity(schedule_peer_rank)
    _need(tuple(schedule_peer_token_idx.shape) == (cap,), "schedule_peer_token_idx must have shape (schedule_capacity,)")
    _need(tuple(num_tokens.shape) == (1,), "num_tokens must have shape (1,)")
    _need(tuple(tokens_per_expert.shape) == (El,), "tokens_per_expert must have shape (num_local_experts,)")
    _bf16({"x": x, "combine_buffer": combine_buffer, "w_shared_gate": w_shared_gate, "w_shared_up": w_shared_up,
           "w_shared_down": w_shared_down})
    _fp8_and_scales({"w_routed_gate": w_routed_gate, "w_routed_gate_sc": w_routed_gate_sc, "w_routed_up": w_routed_up,
                     "w_routed_up_sc": w_routed_up_sc, "w_routed_down": w_routed_down,
                     "w_routed_down_sc": w_routed_down_sc})

    dev = x.device
    bf = dict(dtype=torch.bfloat16, device=dev)
    f8 = dict(dtype=torch.float8_e4m3fn, device=dev)
    u8 = dict(dtype=torch.uint8, device=dev)
    x_qt, x_sct = torch.empty(H, MB, **f8), torch.empty(_sc_shape(H, MB), **u8)
    gate_shared, up_shared, hidden_shared = (torch.empty(T, I, **bf) for _ in range(3))
    gate_q, gate_sc = torch.empty(MB, I, **f8), torch.empty(_sc_shape(MB, I), **u8)
    up_q, up_sc = torch.empty(MB, I, **f8), torch.empty(_sc_shape(MB, I), **u8)
    hid_qt, hid_sct = torch.empty(I, MB, **f8), torch.empty(_sc_shape(I, MB), **u8)
    y_shared, y_routed = torch.empty(T, H, **bf), torch.empty(MB, H, **bf)
    work = [torch.empty(MB, H, **f8), torch.empty(_sc_shape(MB, H), **u8),
            torch.empty(MB, I, **f8), torch.empty(_sc_shape(MB, I), **u8)]

    a = _lib.FwdMxfp8Args()
    a.c = _common(x, ep_size, I, El, topk, cap, MB, minibatch_size, num_comm_sms, swiglu_limit,
                  (schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert), defer_combine)
    a.c.ep_rank = _own_rank(x, x_ptrs, "x_ptrs")
    keep = (_lib.ptr_array(x_ptrs), _lib.ptr_array(combine_buffer_ptrs))
    a.x_ptrs, a.combine_buffer_ptrs = keep
    fields = dict(
        w_shared_gate=w_shared_gate, w_shared_up=w_shared_up, w_shared_down=w_shared_down,
        w_routed_gate_q=w_routed_gate, w_routed_gate_sc=w_routed_gate_sc, w_routed_up_q=w_routed_up,
        w_routed_up_sc=w_routed_up_sc, w_routed_down_q=w_routed_down, w_routed_down_sc=w_routed_down_sc,
        x_qt=x_qt, x_sct=x_sct, gate_shared=gate_shared, up_shared=up_shared, hidden_shared=hidden_shared,
        gate_q=gate_q, gate_sc=gate_sc, up_q=up_q, up_sc=up_sc, hidden_qt=hid_qt, hidden_sct=hid_sct,
        y_shared=y_shared, y_routed=y_routed, work_x_q=work[0], work_x_sc=work[1], work_hidden_q=work[2],
        work_hidden_sc=work[3])
    for k, t in fields.items():
        setattr(a, k, t.data_ptr())
    _lib.check(_lib.mok_fwd_mxfp8(a, _lib.stream_ptr(dev)), "dispatch_mlp_swiglu_combine_fwd_mxfp8")
    return (x_qt, x_sct, gate_shared, gate_q, gate_sc, up_shared, up_q, up_sc, hidden_shared, hid_qt, hid_sct,
            y_shared, y_routed)


@torch.library.custom_op(
    "mok::dispatch_mlp_swiglu_combine_bwd_mxfp8",
    mutates_args=("d_x_routed_buffer", "d_router_weight_buffer", "x_fp8_t_routed", "x_sc_t_routed",
                  "gate_fp8_routed", "gate_sc_routed", "up_fp8_routed", "up_sc_routed",
                  "hidden_fp8_t_routed", "hidden_sc_t_routed"))
def dispatch_mlp_swiglu_combine_bwd_mxfp8(
    d_y_buffer: Tensor, d_y_buffer_ptrs: list[int], d_x_routed_buffer: Tensor, d_x_routed_buffer_ptrs: list[int],
    router_weight_buffer: Tensor, router_weight_buffer_ptrs: list[int],
    d_router_weight_buffer: Tensor, d_router_weight_buffer_ptrs: list[int],
    w_shared_gate: Tensor, w_routed_gate_T: Tensor, w_routed_gate_T_sc: Tensor,
    w_shared_up: Tensor, w_routed_up_T: Tensor, w_routed_up_T_sc: Tensor,
    w_shared_down: Tensor, w_routed_down_T: Tensor, w_routed_down_T_sc: Tensor,
    x_fp8_t_routed: Tensor, x_sc_t_routed: Tensor,
    gate_shared: Tensor, gate_fp8_routed: Tensor, gate_sc_routed: Tensor,
    up_shared: Tensor, up_fp8_routed: Tensor, up_sc_routed: Tensor,
    hidden_shared: Tensor, hidden_fp8_t_routed: Tensor, hidden_sc_t_routed: Tensor,
    x: Tensor, x_ptrs: list[int],
    w_routed_gate: Tensor, w_routed_gate_sc: Tensor, w_routed_up: Tensor, w_routed_up_sc: Tensor,
    schedule_peer_rank: Tensor, schedule_peer_token_idx: Tensor, num_tokens: Tensor, tokens_per_expert: Tensor,
    topk: int, swiglu_limit: float | None, num_comm_sms: int, macrobatch_size: int, minibatch_size: int,
    defer_combine: bool = False,
) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor,
           Tensor, Tensor, Tensor, Tensor, Tensor]:
    x_ptrs, d_y_buffer_ptrs = _self_ptrs(x, x_ptrs), _self_ptrs(d_y_buffer, d_y_buffer_ptrs)
    router_weight_buffer_ptrs = _self_ptrs(router_weight_buffer, router_weight_buffer_ptrs)
    T, H = _token_hidden(x, "x")
    _layer_scalars(topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size)
    ep_size = _pointer_lists({"x_ptrs": x_ptrs, "d_y_buffer_ptrs": d_y_buffer_ptrs,
                              "d_x_routed_buffer_ptrs": d_x_routed_buffer_ptrs,
                              "router_weight_buffer_ptrs": router_weight_buffer_ptrs,
                              "d_router_weight_buffer_ptrs": d_router_weight_buffer_ptrs}, "x_ptrs")
    I = _intermediate(w_shared_gate, H, strict_cols=True)
    El = _local_experts(w_routed_gate)
    MB = macrobatch_size
    _shapes_and_devices(x.device, [
        ("d_y_buffer", d_y_buffer, (T, H)), ("d_x_routed_buffer", d_x_routed_buffer, (T * topk, H)),
        ("router_weight_buffer", router_weight_buffer, (T, topk)),
        ("d_router_weight_buffer", d_router_weight_buffer, (T, topk)),
        ("w_shared_gate", w_shared_gate, (I, H)),
        ("w_routed_gate_T", w_routed_gate_T, (El, H, I)), ("w_routed_gate_T_sc", w_routed_gate_T_sc, _sc_shape(El * H, I)),
        ("w_shared_up", w_shared_up, (I, H)),
        ("w_routed_up_T", w_routed_up_T, (El, H, I)), ("w_routed_up_T_sc", w_routed_up_T_sc, _sc_shape(El * H, I)),
        ("w_shared_down", w_shared_down, (H, I)),
        ("w_routed_down_T", w_routed_down_T, (El, I, H)), ("w_routed_down_T_sc", w_routed_down_T_sc, _sc_shape(El * I, H)),
        ("x_fp8_t_routed", x_fp8_t_routed, (H, MB)), ("x_sc_t_routed", x_sc_t_routed, _sc_shape(H, MB)),
        ("gate_shared", gate_shared, (T, I)),
        ("gate_fp8_routed", gate_fp8_routed, (MB, I)), ("gate_sc_routed", gate_sc_routed, _sc_shape(MB, I)),
        ("up_shared", up_shared, (T, I)),
        ("up_fp8_routed", up_fp8_routed, (MB, I)), ("up_sc_routed", up_sc_routed, _sc_shape(MB, I)),
        ("hidden_shared", hidden_shared, (T, I)),
        ("hidden_fp8_t_routed", hidden_fp8_t_routed, (I, MB)), ("hidden_sc_t_routed", hidden_sc_t_routed, _sc_shape(I, MB)),
        ("w_routed_gate", w_routed_gate, (El, I, H)), ("w_routed_gate_sc", w_routed_gate_sc, _sc_shape(El * I, H)),
        ("w_routed_up", w_routed_up, (El, I, H)), ("w_routed_up_sc", w_routed_up_sc, _sc_shape(El * I, H)),
    ], [("schedule_peer_rank", schedule_peer_rank), ("schedule_peer_token_idx", schedule_peer_token_idx),
        ("num_tokens", num_tokens), ("tokens_per_expert", tokens_per_expert)])
    cap = _schedule_capacity(schedule_peer_rank)
    _need(tuple(schedule_peer_token_idx.shape) == (cap,), "schedule_peer_token_idx must have shape (schedule_capacity,)")
    _need(tuple(num_tokens.shape) == (1,), "num_tokens must have shape (1,)")
    _need(tuple(tokens_per_expert.shape) == (El,), "tokens_per_expert must have shape (num_local_experts,)")
    _bf16({"x": x, "d_y_buffer": d_y_buffer, "d_x_routed_buffer": d_x_routed_buffer, "w_shared_gate": w_shared_gate,
           "w_shared_up": w_shared_up, "w_shared_down": w_shared_down, "gate_shared": gate_shared,
           "up_shared": up_shared, "hidden_shared": hidden_shared})
    _fp8_and_scales({"w_routed_gate_T": w_routed_gate_T, "w_routed_gate_T_sc": w_routed_gate_T_sc,
                     "w_routed_up_T": w_routed_up_T, "w_routed_up_T_sc": w_routed_up_T_sc,
                     "w_routed_down_T": w_routed_down_T, "w_routed_down_T_sc": w_routed_down_T_sc,
                     "x_fp8_t_routed": x_fp8_t_routed, "x_sc_t_routed_sc": x_sc_t_routed,
                     "gate_fp8_routed": gate_fp8_routed, "gate_sc_routed_sc": gate_sc_routed,
                     "up_fp8_routed": up_fp8_routed, "up_sc_routed_sc": up_sc_routed,
                     "hidden_fp8_t_routed": hidden_fp8_t_routed, "hidden_sc_t_routed_sc": hidden_sc_t_routed,
                     "w_routed_gate": w_routed_gate, "w_routed_gate_sc": w_routed_gate_sc,
                     "w_routed_up": w_routed_up, "w_routed_up_sc": w_routed_up_sc})
    for name, t in (("router_weight_buffer", router_weight_buffer), ("d_router_weight_buffer", d_router_weight_buffer)):
        _need(t.dtype == torch.float32 and t.is_contiguous(), f"{name} must be contiguous float32", TypeError)

    dev = x.device
    bf = dict(dtype=torch.bfloat16, device=dev)
    f8 = dict(dtype=torch.float8_e4m3fn, device=dev)
    u8 = dict(dtype=torch.uint8, device=dev)
    d_x_shared, d_x_routed = torch.empty(T, H, **bf), torch.empty(MB, H, **bf)
    d_gate_shared, d_up_shared, d_hidden_shared = (torch.empty(T, I, **bf) for _ in range(3))
    d_gate_q, d_gate_sc = torch.empty(MB, I, **f8), torch.empty(_sc_shape(MB, I), **u8)
    d_up_q, d_up_sc = torch.empty(MB, I, **f8), torch.empty(_sc_shape(MB, I), **u8)
    d_hidden_routed = torch.empty(MB, I, **bf)
    d_y_q, d_y_sc = torch.empty(MB, H, **f8), torch.empty(_sc_shape(MB, H), **u8)
    d_w_shared_gate, d_w_shared_up, d_w_shared_down = torch.empty(I, H, **bf), torch.empty(I, H, **bf), torch.empty(H, I, **bf)
    d_w_routed_gate, d_w_routed_up = torch.empty(El, I, H, **bf), torch.empty(El, I, H, **bf)
    d_w_routed_down = torch.empty(El, H, I, **bf)
    work = dict(
        work_x_q=torch.empty(MB, H, **f8), work_x_sc=torch.empty(_sc_shape(MB, H), **u8),
        work_hidden_q=torch.empty(MB, I, **f8), work_hidden_sc=torch.empty(_sc_shape(MB, I), **u8),
        work_d_y_qt=torch.empty(H, MB, **f8), work_d_y_sct=torch.empty(_sc_shape(H, MB), **u8),
        work_d_gate_qt=torch.empty(I, MB, **f8), work_d_gate_sct=torch.empty(_sc_shape(I, MB), **u8),
        work_d_up_qt=torch.empty(I, MB, **f8), work_d_up_sct=torch.empty(_sc_shape(I, MB), **u8),
        router_weights_routed=torch.empty(MB, dtype=torch.float32, device=dev),
        d_router_weight_partials=torch.empty(MB, I // 64, dtype=torch.float32, device=dev))

    a = _lib.BwdMxfp8Args()
    a.c = _common(x, ep_size, I, El, topk, cap, MB, minibatch_size, num_comm_sms, swiglu_limit,
                  (schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert), defer_combine)
    a.c.ep_rank = _own_rank(x, x_ptrs, "x_ptrs")
    keep = [_lib.ptr_array(p) for p in (d_y_buffer_ptrs, d_x_routed_buffer_ptrs, router_weight_buffer_ptrs,
                                        d_router_weight_buffer_ptrs, x_ptrs)]
    a.d_y_ptrs, a.d_x_routed_buffer_ptrs, a.router_weight_ptrs, a.d_router_weight_ptrs, a.x_ptrs = keep
    fields = dict(
        w_shared_gate=w_shared_gate, w_shared_up=w_shared_up, w_shared_down=w_shared_down,
        w_routed_gate_T_q=w_routed_gate_T, w_routed_gate_T_sc=w_routed_gate_T_sc,
        w_routed_up_T_q=w_routed_up_T, w_routed_up_T_sc=w_routed_up_T_sc,
        w_routed_down_T_q=w_routed_down_T, w_routed_down_T_sc=w_routed_down_T_sc,
        w_routed_gate_q=w_routed_gate, w_routed_gate_sc=w_routed_gate_sc,
        w_routed_up_q=w_routed_up, w_routed_up_sc=w_routed_up_sc,
        x_qt=x_fp8_t_routed, x_sct=x_sc_t_routed, gate_q=gate_fp8_routed, gate_sc=gate_sc_routed,
        up_q=up_fp8_routed, up_sc=up_sc_routed, hidden_qt=hidden_fp8_t_routed, hidden_sct=hidden_sc_t_routed,
        gate_shared=gate_shared, up_shared=up_shared, hidden_shared=hidden_shared,
        d_x_shared=d_x_shared, d_x_routed=d_x_routed, d_gate_shared=d_gate_shared, d_gate_q=d_gate_q,
        d_gate_sc=d_gate_sc, d_up_shared=d_up_shared, d_up_q=d_up_q, d_up_sc=d_up_sc,
        d_hidden_shared=d_hidden_shared, d_hidden_routed=d_hidden_routed, d_y_q=d_y_q, d_y_sc=d_y_sc,
        d_w_shared_gate=d_w_shared_gate, d_w_shared_up=d_w_shared_up, d_w_shared_down=d_w_shared_down,
        d_w_routed_gate=d_w_routed_gate, d_w_routed_up=d_w_routed_up, d_w_routed_down=d_w_routed_down, **work)
    for k, t in fields.items():
        setattr(a, k, t.data_ptr())
    _lib.check(_lib.mok_bwd_mxfp8(a, _lib.stream_ptr(dev)), "dispatch_mlp_swiglu_combine_bwd_mxfp8")
    if defer_combine:      # no combine ran: gather the rows here; d_x_shared becomes d_x, the router gradients land in the buffer
        route_row = torch.empty(T * topk, dtype=torch.int32, device=dev)
        _lib.check(_lib.mok_bwd_epilogue_rows(
            d_x_shared.data_ptr(), d_x_routed.data_ptr(), work["d_router_weight_partials"].data_ptr(), work["d_router_weight_partials"].shape[1], schedule_peer_rank.data_ptr(),
            schedule_peer_token_idx.data_ptr(), num_tokens.data_ptr(), route_row.data_ptr(), d_x_shared.data_ptr(),
            d_router_weight_buffer.data_ptr(), T, H, topk, MB, _lib.stream_ptr(dev)), "bwd_epilogue_rows")
    return (d_x_shared, d_x_routed, d_gate_shared, d_gate_q, d_gate_sc, d_up_shared, d_up_q, d_up_sc,
            d_hidden_shared, d_hidden_routed, d_y_q, d_y_sc, d_w_shared_gate, d_w_routed_gate, d_w_shared_up,
            d_w_routed_up, d_w_shared_down, d_w_routed_down)



# ------------------------------------------------------------------------------------------
# router in front of the layer (no reference op: the reference takes finished routes; the law is the
# one its tests use, torch.topk on the logits + softmax over the K values, tests/utils.py:82-84)
# ------------------------------------------------------------------------------------------
def _router_args(logits: Tensor, topk: int) -> tuple[int, int]:
    _need(logits.is_cuda and logits.ndim == 2 and logits.is_contiguous(),
          "logits must be a contiguous CUDA tensor of shape (num_local_tokens, num_experts)")
    _need(logits.dtype == torch.float32, "logits must have dtype torch.float32", TypeError)
    T, E = logits.shape
    _need(T > 0 and 0 < E <= 1024, "num_experts must be in [1, 1024]")
    _need(type(topk) is int and 0 < topk <= min(32, E), "topk must be in [1, min(32, num_experts)]")
    return T, E


@torch.library.custom_op("mok::router_topk", mutates_args=())
def router_topk(logits: Tensor, topk: int) -> tuple[Tensor, Tensor]:
    """(top_experts int64 [T, K], router_weights f32 [T, K]): the K largest logits of every token in
    descending order and the softmax over them."""
    T, E = _router_args(logits, topk)
    experts = torch.empty(T, topk, dtype=torch.int64, device=logits.device)
    weights = torch.empty(T, topk, dtype=torch.float32, device=logits.device)
    _lib.check(_lib.mok_router_topk(logits.data_ptr(), T, E, topk, None, experts.data_ptr(), weights.data_ptr(), None, 0, 0,
                                    _lib.stream_ptr(logits.device)), "router_topk")
    return experts, weights


@torch.library.custom_op("mok::router_topk_gather", mutates_args=("all_gather_top_experts_buffer",))
def router_topk_gather(logits: Tensor, topk: int, all_gather_top_experts_buffer: Tensor, rank: int) -> tuple[Tensor, Tensor]:
    """router_topk that also writes the int32 routes into slot `rank` of every rank's all-gather buffer
    (what the cast + all_gather_top_experts of build_schedule would do)."""
    T, E = _router_args(logits, topk)
    buf = all_gather_top_experts_buffer
    _need(buf.is_cuda and buf.dtype == torch.int32 and buf.is_contiguous() and buf.ndim == 3 and buf.device == logits.device,
          "all_gather_top_experts_buffer must be a contiguous CUDA int32 tensor (ep_size, num_local_tokens, topk)")
    ep_size = buf.shape[0]
    _need(ep_size in _EP_SIZES, f"all_gather_top_experts_buffer ep_size must be one of {_EP_TEXT}")
    _need(tuple(buf.shape[1:]) == (T, topk), "all_gather_top_experts_buffer must match (num_local_tokens, topk)")
    _need(type(rank) is int and 0 <= rank < ep_size, "rank must be an integer in [0, ep_size)")
    peers = _lib.all_gather_peers(buf.data_ptr())
    if peers is None:
        _need(ep_size == 1, "all_gather_top_experts_buffer has no registered peer addresses; create it through "
                            "mok.functional.create_workspace", RuntimeError)
        peers = [buf.data_ptr()]
    experts = torch.empty(T, topk, dtype=torch.int64, device=logits.device)
    weights = torch.empty(T, topk, dtype=torch.float32, device=logits.device)
    _lib.check(_lib.mok_router_topk(logits.data_ptr(), T, E, topk, None, experts.data_ptr(), weights.data_ptr(),
                                    _lib.ptr_array(peers), ep_size, rank, _lib.stream_ptr(logits.device)), "router_topk_gather")
    return experts, weights


@torch.library.custom_op("mok::router_topk_bwd", mutates_args=())
def router_topk_bwd(top_experts: Tensor, router_weights: Tensor, d_router_weights: Tensor, num_experts: int) -> Tensor:
    """d_logits f32 [T, num_experts] from the gradient of the router weights."""
    _need(top_experts.is_cuda and top_experts.ndim == 2 and top_experts.dtype in (torch.int64, torch.int32),
          "top_experts must be a CUDA integer tensor of shape (num_local_tokens, topk)")
    T, K = top_experts.shape
    for name, t in (("router_weights", router_weights), ("d_router_weights", d_router_weights)):
        _need(t.device == top_experts.device and tuple(t.shape) == (T, K), f"{name} must match top_experts")
        _need(t.dtype == torch.float32, f"{name} must have dtype torch.float32", TypeError)
    _need(type(num_experts) is int and K <= num_experts <= 1024 and K <= 32, "num_experts must be in [topk, 1024]")
    idx = top_experts.to(torch.int32).contiguous()
    rw, d_rw = router_weights.contiguous(), d_router_weights.contiguous()     # kept alive until the launch is enqueued
    d_logits = torch.empty(T, num_experts, dtype=torch.float32, device=top_experts.device)
    _lib.check(_lib.mok_router_topk_bwd(idx.data_ptr(), rw.data_ptr(), d_rw.data_ptr(), d_logits.data_ptr(), T,
                                        num_experts, K, _lib.stream_ptr(top_experts.device)), "router_topk_bwd")
    return d_logits


def _router_setup(ctx, inputs, output):
    ctx.num_experts = inputs[0].shape[1]
    ctx.save_for_backward(output[0], output[1])
    ctx.set_materialize_grads(False)


def _router_backward(ctx, _d_experts, d_weights):
    experts, weights = ctx.saved_tensors
    d_logits = None if d_weights is None else router_topk_bwd(experts, weights, d_weights.contiguous(), ctx.num_experts)
    return (d_logits,) + (None,) * (len(ctx.needs_input_grad) - 1)


torch.library.register_autograd("mok::router_topk", _router_backward, setup_context=_router_setup)
