"""Functional layer of the B200 MoE path: configuration, symmetric-memory workspace, schedule
construction, forward and backward.  Names, signatures and argument meaning follow
Mixture-of-Kittens' `mok/functional.py` (MoKConfig :22-29, MoKSchedule :32-37,
MoKForwardContext :40-48, MoKWorkspace :51-86, create/get_workspace :160-335,
build_schedule :354-430, forward :474-572, backward :575-703) so the module is a drop-in.

Differences a caller can observe:
  * EP sizes 1, 2, 4, 8 are accepted; with a single rank the workspace lives in ordinary
    device memory and no symmetric-memory rendezvous happens;
  * cross-rank traffic is unicast peer loads/stores; the NVLS multicast pointers kept in the
    workspace for signature compatibility may be 0 and are not used;
  * `schedule` is exported as an alias of `build_schedule`;
  * device-detected problems (capacity overflow, a peer that never reaches a barrier) land in
    a status word readable through `mok.last_status()`, never in a trap or an endless wait.
"""
from __future__ import annotations

import os
import math
from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist

from . import _lib
from . import ops

_SUPPORTED_EP_SIZES = (1, 2, 4, 8)

# With one rank no peer reads this rank's buffers: skip the staging copies, the barriers and, when one macrobatch
# holds the whole schedule, the combine pass.  MOK_B200_LOCAL_FAST_PATH=0 keeps the multi-rank sequence (tests
# compare the two bit for bit).
SINGLE_RANK_FAST_PATH = os.environ.get("MOK_B200_LOCAL_FAST_PATH", "1") != "0"


@dataclass(frozen=True, slots=True)
class MoKConfig:
    fwd_num_comm_sms: int = 40
    bwd_num_comm_sms: int = 28
    minibatch_size: int = 4096
    macrobatch_size: int = 131072
    schedule_capacity_multiplier: float = 0.5
    all_gather_top_experts_chunk_bytes: int = 2048


@dataclass(frozen=True, slots=True)
class MoKSchedule:
    peer_rank: torch.Tensor          # int32 [schedule_capacity]
    peer_token_idx: torch.Tensor     # int32 [schedule_capacity], token * topk + k
    num_tokens: torch.Tensor         # int32 [1]
    tokens_per_expert: torch.Tensor  # int32 [num_local_experts], padded to 256


@dataclass(frozen=True, slots=True)
class MoKForwardContext:
    x_routed: torch.Tensor | tuple[torch.Tensor, torch.Tensor]
    gate_shared: torch.Tensor
    gate_routed: torch.Tensor | tuple[torch.Tensor, torch.Tensor]
    up_shared: torch.Tensor
    up_routed: torch.Tensor | tuple[torch.Tensor, torch.Tensor]
    hidden_shared: torch.Tensor
    hidden_routed: torch.Tensor | tuple[torch.Tensor, torch.Tensor]


@dataclass(slots=True)
class MoKWorkspace:
    group_name: str
    ep_rank: int
    ep_size: int
    device: torch.device
    num_local_tokens: int
    hidden_size: int
    topk: int
    schedule_capacity: int
    x_buffer: torch.Tensor                            # bf16 [T, H]
    x_buffer_handle: Any
    x_buffer_ptrs: list[int]
    combine_buffer: torch.Tensor                      # bf16 [T*K, H]
    combine_buffer_handle: Any
    combine_buffer_ptrs: list[int]
    d_y_buffer: torch.Tensor                          # bf16 [T, H]
    d_y_buffer_handle: Any
    d_y_buffer_ptrs: list[int]
    d_x_routed_buffer: torch.Tensor                   # bf16 [T*K, H]
    d_x_routed_buffer_handle: Any
    d_x_routed_buffer_ptrs: list[int]
    router_weight_buffer: torch.Tensor                # f32 [T, K]
    router_weight_buffer_handle: Any
    router_weight_buffer_ptrs: list[int]
    d_router_weight_buffer: torch.Tensor              # f32 [T, K]
    d_router_weight_buffer_handle: Any
    d_router_weight_buffer_ptrs: list[int]
    all_gather_top_experts_buffer: torch.Tensor       # i32 [W, T, K]
    all_gather_top_experts_buffer_handle: Any
    all_gather_top_experts_buffer_multicast_ptr: int
    barrier_buffer: torch.Tensor                      # i32 [1]
    barrier_buffer_handle: Any
    barrier_buffer_ptrs: list[int]
    barrier_buffer_multicast_ptr: int
    barrier_target: torch.Tensor                      # i32 [1]


_WORKSPACE_CACHE: dict[tuple[str, int, int, int, int, int], MoKWorkspace] = {}


def _device_index(device: torch.device) -> int:
    return device.index if device.index is not None else torch.cuda.current_device()


def _capacity_factor(config: MoKConfig, ep_size: int) -> int:
    return max(2, math.ceil(ep_size * config.schedule_capacity_multiplier))


def validate_workspace_args(config: MoKConfig, group: dist.ProcessGroup, *, device: torch.device,
                            num_local_tokens: int, hidden_size: int, topk: int) -> None:
    """Raises on arguments `create_workspace` / `get_workspace` cannot serve."""
    mult = config.schedule_capacity_multiplier
    if type(mult) not in (int, float) or not math.isfinite(mult) or mult <= 0:
        raise ValueError("schedule_capacity_multiplier must be a positive finite number")
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed must be initialized")
    if not isinstance(group, dist.ProcessGroup):
        raise TypeError("group must be a torch.distributed.ProcessGroup")
    if not isinstance(device, torch.device):
        raise TypeError("device must be a torch.device")
    if device.type != "cuda":
        raise ValueError("device must be a CUDA device")
    index = _device_index(device)
    if index != torch.cuda.current_device():
        raise ValueError("MoK workspace device must be the current CUDA device")
    if torch.cuda.get_device_capability(index) not in ((10, 0), (10, 3)):
        raise NotImplementedError("MoK currently requires an SM100 or SM103 GPU")
    if type(num_local_tokens) is not int or num_local_tokens < 512:
        raise ValueError("num_local_tokens must be an integer at least 512")
    if num_local_tokens % 256 != 0:
        raise ValueError("num_local_tokens must be divisible by 256")
    if type(hidden_size) is not int or hidden_size <= 0:
        raise ValueError("hidden_size must be a positive integer")
    if hidden_size % 256 != 0:
        raise ValueError("hidden_size must be divisible by 256")
    if type(topk) is not int or not 0 < topk <= 255:
        raise ValueError("topk must be an integer in [1, 255]")
    name = group.group_name
    if not isinstance(name, str) or not name:
        raise RuntimeError("process group must have a nonempty group_name")
    ep_rank, ep_size = dist.get_rank(group=group), dist.get_world_size(group=group)
    if ep_size not in _SUPPORTED_EP_SIZES:
        raise ValueError("MoK EP size must be one of 1, 2, 4, 8")
    if not 0 <= ep_rank < ep_size:
        raise RuntimeError("current process is not a member of the EP process group")


def _symmetric(shape: tuple[int, ...], dtype: torch.dtype, device: torch.device, group_name: str, ep_size: int,
               zero: bool = False):
    """One buffer visible to every rank: (tensor, handle, per-rank addresses, multicast address)."""
    if ep_size == 1:
        t = torch.zeros(shape, dtype=dtype, device=device) if zero else torch.empty(shape, dtype=dtype, device=device)
        return t, None, [t.data_ptr()], 0
    import torch.distributed._symmetric_memory as symm_mem
    t = symm_mem.empty(*shape, dtype=dtype, device=device)
    if zero:
        t.zero_()
    handle = symm_mem.rendezvous(t, group_name)
    ptrs = [int(handle.buffer_ptrs[r]) for r in range(ep_size)]
    try:
        multicast = int(handle.multicast_ptr)
    except Exception:   # no NVLS multicast object on this system; unicast is all this build needs
        multicast = 0
    return t, handle, ptrs, multicast


def create_workspace(config: MoKConfig, group: dist.ProcessGroup, *, device: torch.device, num_local_tokens: int,
                     hidden_size: int, topk: int) -> MoKWorkspace:
    """Allocates a caller-owned workspace: eight rank-visible buffers plus the barrier state."""
    validate_workspace_args(config, group, device=device, num_local_tokens=num_local_tokens,
                            hidden_size=hidden_size, topk=topk)
    device = torch.device("cuda", _device_index(device))
    group_name = group.group_name
    ep_rank, ep_size = dist.get_rank(group=group), dist.get_world_size(group=group)
    T, H, K = num_local_tokens, hidden_size, topk

    if ep_size > 1:
        mine = torch.tensor([T, H, K], dtype=torch.int64, device=device)
        everyone = torch.empty(ep_size * 3, dtype=torch.int64, device=device)
        dist.all_gather_into_tensor(everyone, mine, group=group)
        if not bool((everyone.view(ep_size, 3) == mine).all().item()):   # one-time set-up: a host sync is fine here
            raise ValueError("MoK requires identical token, hidden, and top-k shapes on every EP rank")
        import torch.distributed._symmetric_memory as symm_mem
        symm_mem.enable_symm_mem_for_group(group_name)

    capacity = T * K * _capacity_factor(config, ep_size)
    mk = lambda shape, dtype, zero=False: _symmetric(shape, dtype, device, group_name, ep_size, zero)  # noqa: E731
    x_buf, x_h, x_p, _ = mk((T, H), torch.bfloat16)
    cb_buf, cb_h, cb_p, _ = mk((T * K, H), torch.bfloat16)
    dy_buf, dy_h, dy_p, _ = mk((T, H), torch.bfloat16)
    dxr_buf, dxr_h, dxr_p, _ = mk((T * K, H), torch.bfloat16)
    rw_buf, rw_h, rw_p, _ = mk((T, K), torch.float32)
    drw_buf, drw_h, drw_p, _ = mk((T, K), torch.float32)
    ag_buf, ag_h, ag_p, ag_mc = mk((ep_size, T, K), torch.int32)
    bar_buf, bar_h, bar_p, bar_mc = mk((1,), torch.int32, True)
    _lib.register_all_gather_peers(ag_buf.data_ptr(), ag_p)
    barrier_target = torch.zeros(1, dtype=torch.int32, device=device)

    if ep_size > 1:
        dist.barrier(group=group, async_op=True, device_ids=[device.index]).block_current_stream()

    return MoKWorkspace(
        group_name=group_name, ep_rank=ep_rank, ep_size=ep_size, device=device,
        num_local_tokens=T, hidden_size=H, topk=K, schedule_capacity=capacity,
        x_buffer=x_buf, x_buffer_handle=x_h, x_buffer_ptrs=x_p,
        combine_buffer=cb_buf, combine_buffer_handle=cb_h, combine_buffer_ptrs=cb_p,
        d_y_buffer=dy_buf, d_y_buffer_handle=dy_h, d_y_buffer_ptrs=dy_p,
        d_x_routed_buffer=dxr_buf, d_x_routed_buffer_handle=dxr_h, d_x_routed_buffer_ptrs=dxr_p,
        router_weight_buffer=rw_buf, router_weight_buffer_handle=rw_h, router_weight_buffer_ptrs=rw_p,
        d_router_weight_buffer=drw_buf, d_router_weight_buffer_handle=drw_h, d_router_weight_buffer_ptrs=drw_p,
        all_gather_top_experts_buffer=ag_buf, all_gather_top_experts_buffer_handle=ag_h,
        all_gather_top_experts_buffer_multicast_ptr=ag_mc,
        barrier_buffer=bar_buf, barrier_buffer_handle=bar_h, barrier_buffer_ptrs=bar_p,
        barrier_buffer_multicast_ptr=bar_mc, barrier_target=barrier_target,
    )


def get_workspace(config: MoKConfig, group: dist.ProcessGroup, *, device: torch.device, num_local_tokens: int,
                  hidden_size: int, topk: int) -> MoKWorkspace:
    """Cached `create_workspace`; the key is (group, device, T, H, K, capacity factor)."""
    validate_workspace_args(config, group, device=device, num_local_tokens=num_local_tokens,
                            hidden_size=hidden_size, topk=topk)
    index = _device_index(device)
    key = (group.group_name, index, num_local_tokens, hidden_size, topk,
           _capacity_factor(config, dist.get_world_size(group=group)))
    ws = _WORKSPACE_CACHE.get(key)
    if ws is None:
        ws = create_workspace(config, group, device=torch.device("cuda", index), num_local_tokens=num_local_tokens,
                              hidden_size=hidden_size, topk=topk)
        _WORKSPACE_CACHE[key] = ws
    return ws


def _barrier(ws: MoKWorkspace) -> None:
    ops.barrier_all(ws.barrier_buffer, ws.barrier_buffer_ptrs, ws.barrier_buffer_multicast_ptr, ws.barrier_target)


def clear_workspace_cache() -> None:
    """Drops every cached workspace after all ranks passed a device barrier on it."""
    for ws in _WORKSPACE_CACHE.values():
        _barrier(ws)
        torch.cuda.synchronize(ws.device)
        _lib.unregister_all_gather_peers(ws.all_gather_top_experts_buffer.data_ptr())
    _WORKSPACE_CACHE.clear()


def _validate_config(config: MoKConfig, ws: MoKWorkspace) -> None:
    props = torch.cuda.get_device_properties(ws.device)
    for label, value in (("fwd_num_comm_sms", config.fwd_num_comm_sms), ("bwd_num_comm_sms", config.bwd_num_comm_sms)):
        if type(value) is not int or value <= 0:
            raise ValueError(f"{label} must be a positive integer")
        if value % 2 != 0:
            raise ValueError(f"{label} must be even")
    if max(config.fwd_num_comm_sms, config.bwd_num_comm_sms) >= props.multi_processor_count:
        raise ValueError("communication-SM counts must leave at least one compute SM")
    mini, macro = config.minibatch_size, config.macrobatch_size
    if type(mini) is not int or mini <= 0 or mini % 256 != 0:
        raise ValueError("minibatch_size must be positive and divisible by 256")
    if type(macro) is not int or macro <= 0 or macro % mini != 0:
        raise ValueError("macrobatch_size must be a positive multiple of minibatch_size")
    chunk = config.all_gather_top_experts_chunk_bytes
    if type(chunk) is not int or chunk <= 0 or chunk % 16 != 0:
        raise ValueError("all_gather_top_experts_chunk_bytes must be a positive multiple of 16")
    if chunk + 1024 > props.shared_memory_per_block_optin:
        raise ValueError("all_gather_top_experts_chunk_bytes exceeds device dynamic shared-memory capacity")
    if (ws.num_local_tokens * ws.topk * 4) % chunk != 0:
        raise ValueError("all_gather_top_experts_chunk_bytes must divide one rank's route-buffer bytes")


def build_schedule(workspace: MoKWorkspace, config: MoKConfig, top_experts: torch.Tensor, *,
                   num_local_experts: int) -> MoKSchedule:
    """All-gathers the routing choices and builds this rank's padded slot tables.

    top_experts: int64 [num_local_tokens, topk].  No host synchronisation.
    """
    if not isinstance(workspace, MoKWorkspace):
        raise TypeError("workspace must be a MoKWorkspace")
    if not isinstance(config, MoKConfig):
        raise TypeError("config must be a MoKConfig")
    _validate_config(config, workspace)
    if not top_experts.is_cuda or top_experts.device != workspace.device:
        raise ValueError("top_experts must be on the workspace CUDA device")
    if top_experts.dtype != torch.int64:
        raise TypeError("top_experts must have dtype torch.int64")
    if not top_experts.is_contiguous():
        raise ValueError("top_experts must be contiguous")
    if tuple(top_experts.shape) != (workspace.num_local_tokens, workspace.topk):
        raise ValueError("top_experts must have shape (num_local_tokens, topk)")
    if type(num_local_experts) is not int or num_local_experts <= 0:
        raise ValueError("num_local_experts must be a positive integer")

    if workspace.ep_size == 1 and SINGLE_RANK_FAST_PATH:           # nothing to gather: the scheduler reads the routes where the cast put them
        topk_all = top_experts.to(torch.int32).unsqueeze(0)
    else:
        ops.all_gather_top_experts(top_experts.to(torch.int32), workspace.all_gather_top_experts_buffer,
                                   workspace.all_gather_top_experts_buffer_multicast_ptr, workspace.ep_rank,
                                   config.all_gather_top_experts_chunk_bytes)
        _barrier(workspace)
        topk_all = workspace.all_gather_top_experts_buffer
    peer_rank, peer_token_idx, num_tokens, tokens_per_expert = ops.schedule(
        topk_all, num_local_experts, workspace.schedule_capacity, workspace.ep_rank)
    return MoKSchedule(peer_rank=peer_rank, peer_token_idx=peer_token_idx, num_tokens=num_tokens,
                       tokens_per_expert=tokens_per_expert)


schedule = build_schedule


def route(logits: torch.Tensor, topk: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Router in front of the layer: (top_experts int64 [T, K], router_weights f32 [T, K]) from f32 logits
    [T, num_experts] — the K largest logits per token, descending, and the softmax over them (softmax over all
    experts, top-K, renormalise).  Differentiable with respect to the logits."""
    return ops.router_topk(logits, topk)


class _RouteGather(torch.autograd.Function):
    """router_topk_gather on the autograd tape (an operator that writes into a buffer cannot carry a registered
    gradient formula, so the formula sits here)."""

    @staticmethod
    def forward(ctx, logits, topk, buffer, rank):
        experts, weights = ops.router_topk_gather(logits, topk, buffer, rank)
        ctx.save_for_backward(experts, weights)
        ctx.num_experts = logits.shape[1]
        ctx.mark_non_differentiable(experts)
        return experts, weights

    @staticmethod
    def backward(ctx, _d_experts, d_weights):
        experts, weights = ctx.saved_tensors
        return ops.router_topk_bwd(experts, weights, d_weights.contiguous(), ctx.num_experts), None, None, None


def route_and_schedule(workspace: MoKWorkspace, config: MoKConfig, logits: torch.Tensor, *,
                       num_local_experts: int) -> tuple[MoKSchedule, torch.Tensor, torch.Tensor]:
    """route() + build_schedule() with the int32 routes written straight into every rank's all-gather buffer by the
    router kernel (no cast, no separate all-gather launch).  Returns (schedule, top_experts, router_weights)."""
    if not isinstance(workspace, MoKWorkspace):
        raise TypeError("workspace must be a MoKWorkspace")
    if not isinstance(config, MoKConfig):
        raise TypeError("config must be a MoKConfig")
    _validate_config(config, workspace)
    if type(num_local_experts) is not int or num_local_experts <= 0:
        raise ValueError("num_local_experts must be a positive integer")
    if logits.ndim != 2 or logits.shape[0] != workspace.num_local_tokens:
        raise ValueError("logits must have shape (num_local_tokens, num_experts)")
    if logits.shape[1] != num_local_experts * workspace.ep_size:
        raise ValueError("logits must have num_local_experts * ep_size columns")
    top_experts, router_weights = _RouteGather.apply(logits, workspace.topk, workspace.all_gather_top_experts_buffer,
                                                     workspace.ep_rank)
    if workspace.ep_size > 1:
        _barrier(workspace)
    peer_rank, peer_token_idx, num_tokens, tokens_per_expert = ops.schedule(
        workspace.all_gather_top_experts_buffer, num_local_experts, workspace.schedule_capacity, workspace.ep_rank)
    sched = MoKSchedule(peer_rank=peer_rank, peer_token_idx=peer_token_idx, num_tokens=num_tokens,
                        tokens_per_expert=tokens_per_expert)
    return sched, top_experts, router_weights


def validate_inputs(config: MoKConfig, workspace: MoKWorkspace, schedule: MoKSchedule, x: torch.Tensor,
                    router_weights: torch.Tensor, grad_output: torch.Tensor | None = None) -> None:
    if not isinstance(config, MoKConfig):
        raise TypeError("config must be a MoKConfig")
    if not isinstance(workspace, MoKWorkspace):
        raise TypeError("workspace must be a MoKWorkspace")
    if not isinstance(schedule, MoKSchedule):
        raise TypeError("schedule must be a MoKSchedule")
    act = (workspace.num_local_tokens, workspace.hidden_size)
    wanted = [("x", x, torch.bfloat16, act)]
    if grad_output is not None:
        wanted.append(("grad_output", grad_output, torch.bfloat16, act))
    wanted.append(("router_weights", router_weights, torch.float32, (workspace.num_local_tokens, workspace.topk)))
    for name, t, dtype, shape in wanted:
        if not t.is_cuda or t.device != workspace.device or t.dtype != dtype or not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous {dtype} on the workspace CUDA device")
        if tuple(t.shape) != shape:
            raise ValueError(f"{name} shape does not match the workspace")
    if schedule.peer_rank.numel() != workspace.schedule_capacity:
        raise ValueError("schedule capacity does not match the workspace")


def _stage(buffer: torch.Tensor, value: torch.Tensor) -> None:
    """Copies a per-step input into its rank-visible buffer, unless the caller built it there: passing
    ``workspace.x_buffer`` / ``d_y_buffer`` / ``router_weight_buffer`` themselves as x / grad_output /
    router_weights skips the copy (the reference marks these copies as removable, mok/functional.py:513)."""
    if value is not buffer:
        buffer.copy_(value)


def forward(config: MoKConfig, workspace: MoKWorkspace, schedule: MoKSchedule, x: torch.Tensor,
            router_weights: torch.Tensor, shared_gate_weights: torch.Tensor, shared_up_weights: torch.Tensor,
            shared_down_weights: torch.Tensor,
            routed_gate_weights: torch.Tensor | tuple[torch.Tensor, torch.Tensor],
            routed_up_weights: torch.Tensor | tuple[torch.Tensor, torch.Tensor],
            routed_down_weights: torch.Tensor | tuple[torch.Tensor, torch.Tensor],
            swiglu_limit: float | None = None) -> tuple[torch.Tensor, MoKForwardContext]:
    """MoE forward.  Routed weights are bf16 tensors, or (fp8, scales) pairs for MXFP8.

    Returns (output bf16 [T, H], context holding the activations backward needs).
    """
    validate_inputs(config, workspace, schedule, x, router_weights)
    ws = workspace
    # Single rank: no peer reads this rank's buffers, so the kernels work on the caller's tensors (no staging
    # copies, no barriers), and when one macrobatch holds the whole schedule the routed rows are summed straight
    # from the down-GEMM output instead of going through the combine buffer.
    local = ws.ep_size == 1 and SINGLE_RANK_FAST_PATH
    defer = local and ws.schedule_capacity <= config.macrobatch_size
    if local:
        x_buf, x_ptrs, rw_buf = x, ops.SELF_PTRS, router_weights
    else:
        _stage(ws.x_buffer, x)
        _stage(ws.router_weight_buffer, router_weights)
        _barrier(ws)
        x_buf, x_ptrs, rw_buf = ws.x_buffer, ws.x_buffer_ptrs, ws.router_weight_buffer
    sched = (schedule.peer_rank, schedule.peer_token_idx, schedule.num_tokens, schedule.tokens_per_expert)
    knobs = (ws.topk, swiglu_limit, config.fwd_num_comm_sms, config.macrobatch_size, config.minibatch_size, defer)

    if isinstance(routed_gate_weights, tuple):
        (g_q, g_s), (u_q, u_s), (d_q, d_s) = routed_gate_weights, routed_up_weights, routed_down_weights
        (x_t_q, x_t_s, gate_sh, gate_q, gate_s, up_sh, up_q, up_s, hid_sh, hid_t_q, hid_t_s,
         y_shared, y_routed) = ops.dispatch_mlp_swiglu_combine_fwd_mxfp8(
            x_buf, x_ptrs, ws.combine_buffer, ws.combine_buffer_ptrs,
            shared_gate_weights, g_q, g_s, shared_up_weights, u_q, u_s, shared_down_weights, d_q, d_s,
            *sched, *knobs)
        ctx = MoKForwardContext(x_routed=(x_t_q, x_t_s), gate_shared=gate_sh, gate_routed=(gate_q, gate_s),
                                up_shared=up_sh, up_routed=(up_q, up_s), hidden_shared=hid_sh,
                                hidden_routed=(hid_t_q, hid_t_s))
    else:
        (x_routed, gate_sh, gate_r, up_sh, up_r, hid_sh, hid_r,
         y_shared, y_routed) = ops.dispatch_mlp_swiglu_combine_fwd_bf16(
            x_buf, x_ptrs, ws.combine_buffer, ws.combine_buffer_ptrs,
            shared_gate_weights, routed_gate_weights, shared_up_weights, routed_up_weights,
            shared_down_weights, routed_down_weights, *sched, *knobs)
        ctx = MoKForwardContext(x_routed=x_routed, gate_shared=gate_sh, gate_routed=gate_r, up_shared=up_sh,
                                up_routed=up_r, hidden_shared=hid_sh, hidden_routed=hid_r)

    if defer:
        output = ops.fwd_epilogue_rows(y_shared, y_routed, schedule.peer_rank, schedule.peer_token_idx,
                                       schedule.num_tokens, rw_buf)
    else:
        if not local:
            _barrier(ws)
        output = ops.fwd_epilogue(y_shared, ws.combine_buffer, rw_buf)
    return output, ctx


def backward(config: MoKConfig, workspace: MoKWorkspace, schedule: MoKSchedule, forward_context: MoKForwardContext,
             grad_output: torch.Tensor, x: torch.Tensor, router_weights: torch.Tensor,
             shared_gate_weights: torch.Tensor, shared_up_weights: torch.Tensor, shared_down_weights: torch.Tensor,
             routed_gate_weights: torch.Tensor | tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor],
             routed_up_weights: torch.Tensor | tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor],
             routed_down_weights: torch.Tensor | tuple[torch.Tensor, torch.Tensor],
             swiglu_limit: float | None = None):
    """MoE backward.  Returns (d_x, d_router_weights, d_routed_gate, d_routed_up, d_routed_down,
    d_shared_gate, d_shared_up, d_shared_down).  MXFP8 routed weights come as
    (fp8, sc, fp8_t, sc_t) for gate and up and (down_t_fp8, down_t_sc) for down."""
    validate_inputs(config, workspace, schedule, x, router_weights, grad_output)
    if not isinstance(forward_context, MoKForwardContext):
        raise TypeError("forward_context must be a MoKForwardContext")
    ws, ctx = workspace, forward_context
    local = ws.ep_size == 1 and SINGLE_RANK_FAST_PATH              # see forward
    defer = local and ws.schedule_capacity <= config.macrobatch_size
    if local:
        d_y_buf, d_y_ptrs, x_buf, x_ptrs = grad_output, ops.SELF_PTRS, x, ops.SELF_PTRS
        rw_buf, rw_ptrs = router_weights, ops.SELF_PTRS
    else:
        _stage(ws.d_y_buffer, grad_output)
        _stage(ws.x_buffer, x)
        _stage(ws.router_weight_buffer, router_weights)
        _barrier(ws)
        d_y_buf, d_y_ptrs, x_buf, x_ptrs = ws.d_y_buffer, ws.d_y_buffer_ptrs, ws.x_buffer, ws.x_buffer_ptrs
        rw_buf, rw_ptrs = ws.router_weight_buffer, ws.router_weight_buffer_ptrs
    sched = (schedule.peer_rank, schedule.peer_token_idx, schedule.num_tokens, schedule.tokens_per_expert)
    knobs = (ws.topk, swiglu_limit, config.bwd_num_comm_sms, config.macrobatch_size, config.minibatch_size, defer)
    buffers = (d_y_buf, d_y_ptrs, ws.d_x_routed_buffer, ws.d_x_routed_buffer_ptrs, rw_buf, rw_ptrs,
               ws.d_router_weight_buffer, ws.d_router_weight_buffer_ptrs)

    if isinstance(routed_gate_weights, tuple):
        g_q, g_s, g_t_q, g_t_s = routed_gate_weights
        u_q, u_s, u_t_q, u_t_s = routed_up_weights
        d_t_q, d_t_s = routed_down_weights
        res = ops.dispatch_mlp_swiglu_combine_bwd_mxfp8(
            *buffers,
            shared_gate_weights, g_t_q, g_t_s, shared_up_weights, u_t_q, u_t_s, shared_down_weights, d_t_q, d_t_s,
            *ctx.x_routed, ctx.gate_shared, *ctx.gate_routed, ctx.up_shared, *ctx.up_routed,
            ctx.hidden_shared, *ctx.hidden_routed,
            x_buf, x_ptrs, g_q, g_s, u_q, u_s, *sched, *knobs)
        d_x_shared = res[0]
        d_w_sh_gate, d_w_r_gate, d_w_sh_up, d_w_r_up, d_w_sh_down, d_w_r_down = res[12:18]
    else:
        res = ops.dispatch_mlp_swiglu_combine_bwd_bf16(
            *buffers,
            shared_gate_weights, routed_gate_weights, shared_up_weights, routed_up_weights,
            shared_down_weights, routed_down_weights,
            ctx.x_routed, ctx.gate_shared, ctx.gate_routed, ctx.up_shared, ctx.up_routed,
            ctx.hidden_shared, ctx.hidden_routed, x_buf, x_ptrs, *sched, *knobs)
        d_x_shared = res[0]
        d_w_sh_gate, d_w_r_gate, d_w_sh_up, d_w_r_up, d_w_sh_down, d_w_r_down = res[9:15]

    if defer:                            # the op summed the routed rows in place: its first output is d_x already
        d_x = d_x_shared
    else:
        if not local:
            _barrier(ws)
        d_x = ops.bwd_epilogue(d_x_shared, ws.d_x_routed_buffer)
    d_router_weights = ws.d_router_weight_buffer.clone()
    return (d_x, d_router_weights, d_w_r_gate, d_w_r_up, d_w_r_down, d_w_sh_gate, d_w_sh_up, d_w_sh_down)
