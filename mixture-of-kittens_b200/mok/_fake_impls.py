"""Shape/dtype propagation ("fake" kernels) for the `mok::*` operators, so the layer can be traced
by torch.compile and FakeTensorMode without touching a GPU.  Output shapes mirror the operator
docstrings of Mixture-of-Kittens' `mok/ops.py` (shape tables at :259-272, :426-435, :635-653,
:901-916) and its `mok/_fake_impls.py`.
"""
from __future__ import annotations

import torch

from . import ops as _ops  # noqa: F401  (registers the operators)

_fake = torch.library.register_fake
_BF16, _FP8, _U8 = torch.bfloat16, torch.float8_e4m3fn, torch.uint8


def _new(like: torch.Tensor, shape, dtype) -> torch.Tensor:
    return like.new_empty(tuple(shape), dtype=dtype)


def _sc(rows: int, cols: int) -> tuple[int, int, int, int]:
    return (rows // 128, cols // 128, 32, 16)


@_fake("mok::all_gather_top_experts")
def _(top_experts, all_gather_top_experts_buffer, all_gather_top_experts_buffer_multicast_ptr, rank, chunk_bytes):
    return None


@_fake("mok::barrier_all")
def _(barrier_buffer, barrier_buffer_ptrs, barrier_buffer_multicast_ptr, target):
    return None


@_fake("mok::schedule")
def _(topk_all, num_local_experts, schedule_capacity, rank):
    i32 = torch.int32
    return (_new(topk_all, (schedule_capacity,), i32), _new(topk_all, (schedule_capacity,), i32),
            _new(topk_all, (1,), i32), _new(topk_all, (num_local_experts,), i32))


@_fake("mok::mxfp8_quantize")
def _(x_bf16, return_normal, return_transposed):
    n = x_bf16.shape[0] if x_bf16.ndim == 3 else 1
    rows, cols = x_bf16.shape[-2], x_bf16.shape[-1]
    t_shape = (n, cols, rows) if x_bf16.ndim == 3 else (cols, rows)
    return (_new(x_bf16, x_bf16.shape, _FP8) if return_normal else None,
            _new(x_bf16, _sc(n * rows, cols), _U8) if return_normal else None,
            _new(x_bf16, t_shape, _FP8) if return_transposed else None,
            _new(x_bf16, _sc(n * cols, rows), _U8) if return_transposed else None)


@_fake("mok::dispatch_mlp_swiglu_combine_fwd_bf16")
def _(x, x_ptrs, combine_buffer, combine_buffer_ptrs, w_shared_gate, w_routed_gate, w_shared_up, w_routed_up,
      w_shared_down, w_routed_down, schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert,
      topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size, defer_combine=False):
    T, H = x.shape
    I, MB = w_shared_gate.shape[0], macrobatch_size
    shapes = ((MB, H), (T, I), (MB, I), (T, I), (MB, I), (T, I), (MB, I), (T, H), (MB, H))
    return tuple(_new(x, s, _BF16) for s in shapes)


@_fake("mok::dispatch_mlp_swiglu_combine_bwd_bf16")
def _(d_y_buffer, d_y_buffer_ptrs, d_x_routed_buffer, d_x_routed_buffer_ptrs, router_weight_buffer,
      router_weight_buffer_ptrs, d_router_weight_buffer, d_router_weight_buffer_ptrs, w_shared_gate, w_routed_gate,
      w_shared_up, w_routed_up, w_shared_down, w_routed_down, x_routed, gate_shared, gate_routed, up_shared, up_routed,
      hidden_shared, hidden_routed, x, x_ptrs, schedule_peer_rank, schedule_peer_token_idx, num_tokens,
      tokens_per_expert, topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size, defer_combine=False):
    T, H = x.shape
    I, El, MB = w_shared_gate.shape[0], w_routed_gate.shape[0], macrobatch_size
    shapes = ((T, H), (MB, H), (T, I), (MB, I), (T, I), (MB, I), (T, I), (MB, I), (MB, H),
              (I, H), (El, I, H), (I, H), (El, I, H), (H, I), (El, H, I))
    return tuple(_new(x, s, _BF16) for s in shapes)


@_fake("mok::fwd_epilogue")
def _(y_shared, combine_buffer, topk_weights):
    return torch.empty_like(y_shared)


@_fake("mok::fwd_epilogue_rows")
def _(y_shared, y_routed, schedule_peer_rank, schedule_peer_token_idx, num_tokens, topk_weights):
    return torch.empty_like(y_shared)


@_fake("mok::bwd_epilogue")
def _(d_x_shared, d_x_routed_buffer):
    return torch.empty_like(d_x_shared)


@_fake("mok::dispatch_mlp_swiglu_combine_fwd_mxfp8")
def _(x, x_ptrs, combine_buffer, combine_buffer_ptrs, w_shared_gate, w_routed_gate, w_routed_gate_sc, w_shared_up,
      w_routed_up, w_routed_up_sc, w_shared_down, w_routed_down, w_routed_down_sc, schedule_peer_rank,
      schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit, num_comm_sms, macrobatch_size,
      minibatch_size, defer_combine=False):
    T, H = x.shape
    I, MB = w_shared_gate.shape[0], macrobatch_size
    spec = (((H, MB), _FP8), (_sc(H, MB), _U8), ((T, I), _BF16), ((MB, I), _FP8), (_sc(MB, I), _U8), ((T, I), _BF16),
            ((MB, I), _FP8), (_sc(MB, I), _U8), ((T, I), _BF16), ((I, MB), _FP8), (_sc(I, MB), _U8), ((T, H), _BF16),
            ((MB, H), _BF16))
    return tuple(_new(x, s, dt) for s, dt in spec)


@_fake("mok::dispatch_mlp_swiglu_combine_bwd_mxfp8")
def _(d_y_buffer, d_y_buffer_ptrs, d_x_routed_buffer, d_x_routed_buffer_ptrs, router_weight_buffer,
      router_weight_buffer_ptrs, d_router_weight_buffer, d_router_weight_buffer_ptrs, w_shared_gate, w_routed_gate_T,
      w_routed_gate_T_sc, w_shared_up, w_routed_up_T, w_routed_up_T_sc, w_shared_down, w_routed_down_T,
      w_routed_down_T_sc, x_fp8_t_routed, x_sc_t_routed, gate_shared, gate_fp8_routed, gate_sc_routed, up_shared,
      up_fp8_routed, up_sc_routed, hidden_shared, hidden_fp8_t_routed, hidden_sc_t_routed, x, x_ptrs, w_routed_gate,
      w_routed_gate_sc, w_routed_up, w_routed_up_sc, schedule_peer_rank, schedule_peer_token_idx, num_tokens,
      tokens_per_expert, topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size, defer_combine=False):
    T, H = x.shape
    I, El, MB = w_shared_gate.shape[0], w_routed_gate.shape[0], macrobatch_size
    spec = (((T, H), _BF16), ((MB, H), _BF16), ((T, I), _BF16), ((MB, I), _FP8), (_sc(MB, I), _U8), ((T, I), _BF16),
            ((MB, I), _FP8), (_sc(MB, I), _U8), ((T, I), _BF16), ((MB, I), _BF16), ((MB, H), _FP8), (_sc(MB, H), _U8),
            ((I, H), _BF16), ((El, I, H), _BF16), ((I, H), _BF16), ((El, I, H), _BF16), ((H, I), _BF16),
            ((El, H, I), _BF16))
    return tuple(_new(x, s, dt) for s, dt in spec)


@_fake("mok::router_topk")
def _(logits, topk):
    T = logits.shape[0]
    return _new(logits, (T, topk), torch.int64), _new(logits, (T, topk), torch.float32)


@_fake("mok::router_topk_gather")
def _(logits, topk, all_gather_top_experts_buffer, rank):
    T = logits.shape[0]
    return _new(logits, (T, topk), torch.int64), _new(logits, (T, topk), torch.float32)


@_fake("mok::router_topk_bwd")
def _(top_experts, router_weights, d_router_weights, num_experts):
    return _new(router_weights, (top_experts.shape[0], num_experts), torch.float32)
