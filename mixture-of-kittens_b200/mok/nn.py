"""What a trainer calls: the layer as a ``torch.autograd.Function`` and as an ``nn.Module``.

The reference stops at ``mok.functional`` (explicit ``forward`` / ``backward`` calls, README.md:116-228);
these wrappers sit directly on top of it and add nothing to the arithmetic:

  * ``moe_experts(...)``  — ``functional.forward`` recorded on the autograd tape, ``functional.backward`` as its
    gradient (x, router weights and all six weight tensors receive gradients);
  * ``MoKLayer``          — parameters of one expert-parallel rank (router, shared expert, local routed experts),
    ``forward(x)`` = router GEMM -> fused top-K router kernel -> schedule -> experts.  With ``mxfp8=True`` the
    routed bf16 master weights are quantised with ``ops.mxfp8_quantize`` whenever they changed, and their
    gradients come back in bf16.

One workspace per (tokens, hidden, top-k) is shared by all layers of a model, as in the reference.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import functional as F
from . import ops


class _Quantised:
    """MXFP8 copies of the routed weights in the layouts forward and backward take."""

    def __init__(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor):
        qg, qu, qd = (ops.mxfp8_quantize(w, True, True) for w in (gate, up, down))
        self.fwd = ((qg[0], qg[1]), (qu[0], qu[1]), (qd[0], qd[1]))
        self.bwd = (tuple(qg), tuple(qu), (qd[2], qd[3]))


class _ExpertsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, router_weights, shared_gate, shared_up, shared_down, routed_gate, routed_up, routed_down,
                config, workspace, schedule, swiglu_limit, quantised):
        routed = (routed_gate, routed_up, routed_down) if quantised is None else quantised.fwd
        out, fctx = F.forward(config, workspace, schedule, x, router_weights, shared_gate, shared_up, shared_down,
                              *routed, swiglu_limit=swiglu_limit)
        ctx.save_for_backward(x, router_weights, shared_gate, shared_up, shared_down, routed_gate, routed_up, routed_down)
        ctx.call = (config, workspace, schedule, fctx, swiglu_limit, quantised)
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, d_out):
        x, router_weights, shared_gate, shared_up, shared_down, routed_gate, routed_up, routed_down = ctx.saved_tensors
        config, workspace, schedule, fctx, swiglu_limit, quantised = ctx.call
        routed = (routed_gate, routed_up, routed_down) if quantised is None else quantised.bwd
        (d_x, d_rw, d_routed_gate, d_routed_up, d_routed_down, d_shared_gate, d_shared_up, d_shared_down) = F.backward(
            config, workspace, schedule, fctx, d_out.contiguous(), x, router_weights, shared_gate, shared_up, shared_down,
            *routed, swiglu_limit=swiglu_limit)
        return (d_x, d_rw, d_shared_gate, d_shared_up, d_shared_down, d_routed_gate, d_routed_up, d_routed_down,
                None, None, None, None, None)


def moe_experts(config: F.MoKConfig, workspace: F.MoKWorkspace, schedule: F.MoKSchedule, x: torch.Tensor,
                router_weights: torch.Tensor, shared_gate: torch.Tensor, shared_up: torch.Tensor,
                shared_down: torch.Tensor, routed_gate: torch.Tensor, routed_up: torch.Tensor, routed_down: torch.Tensor,
                swiglu_limit: float | None = None, quantised: _Quantised | None = None) -> torch.Tensor:
    """Differentiable ``functional.forward``: returns the layer output [T, H]; ``.backward()`` runs
    ``functional.backward`` and fills the gradients of x, router_weights and the six bf16 weight tensors."""
    return _ExpertsFn.apply(x, router_weights, shared_gate, shared_up, shared_down, routed_gate, routed_up, routed_down,
                            config, workspace, schedule, swiglu_limit, quantised)


class MoKLayer(torch.nn.Module):
    """Router + shared expert + this rank's routed experts of one MoE layer.

    ``forward(x)`` routes with the layer's own router; ``forward(x, top_experts, router_weights)`` takes finished
    routes (int64 [T, K], f32 [T, K]) as ``functional.build_schedule`` / ``functional.forward`` do.
    """

    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, topk: int, *,
                 group: dist.ProcessGroup | None = None, config: F.MoKConfig | None = None, mxfp8: bool = False,
                 swiglu_limit: float | None = None, device: torch.device | str | None = None, seed: int | None = None):
        super().__init__()
        self.group = group if group is not None else dist.group.WORLD
        ep_size = dist.get_world_size(self.group)
        if num_experts % ep_size != 0:
            raise ValueError("num_experts must be divisible by the expert-parallel size")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.num_experts, self.num_local_experts, self.topk = num_experts, num_experts // ep_size, topk
        self.config = config if config is not None else F.MoKConfig()
        self.mxfp8, self.swiglu_limit = mxfp8, swiglu_limit
        dev = torch.device(device if device is not None else "cuda")
        gen = None
        if seed is not None:
            gen = torch.Generator(device=dev).manual_seed(seed)

        def param(*shape, fan_in, dtype=torch.bfloat16):
            w = torch.randn(*shape, generator=gen, device=dev, dtype=torch.float32) * fan_in ** -0.5
            return torch.nn.Parameter(w.to(dtype))

        H, I, El = hidden_size, intermediate_size, self.num_local_experts
        self.router_weight = torch.nn.Parameter(torch.randn(num_experts, H, generator=gen, device=dev) * 0.02)
        self.shared_gate, self.shared_up = param(I, H, fan_in=H), param(I, H, fan_in=H)
        self.shared_down = param(H, I, fan_in=I)
        self.routed_gate, self.routed_up = param(El, I, H, fan_in=H), param(El, I, H, fan_in=H)
        self.routed_down = param(El, H, I, fan_in=I)
        self._quantised: _Quantised | None = None
        self._quantised_key: tuple | None = None

    def quantised(self) -> _Quantised | None:
        """MXFP8 copies of the routed weights, refreshed when a master weight was written since the last call."""
        if not self.mxfp8:
            return None
        masters = (self.routed_gate, self.routed_up, self.routed_down)
        key = tuple((w.data_ptr(), w._version) for w in masters)
        if self._quantised is None or key != self._quantised_key:
            with torch.no_grad():
                self._quantised = _Quantised(*(w.detach() for w in masters))
            self._quantised_key = key
        return self._quantised

    def forward(self, x: torch.Tensor, top_experts: torch.Tensor | None = None,
                router_weights: torch.Tensor | None = None) -> torch.Tensor:
        if (top_experts is None) != (router_weights is None):
            raise ValueError("pass both top_experts and router_weights, or neither")
        ws = F.get_workspace(self.config, self.group, device=x.device, num_local_tokens=x.shape[0],
                             hidden_size=self.hidden_size, topk=self.topk)
        if top_experts is None:
            logits = torch.nn.functional.linear(x, self.router_weight.to(x.dtype)).float()
            schedule, top_experts, router_weights = F.route_and_schedule(ws, self.config, logits,
                                                                         num_local_experts=self.num_local_experts)
        else:
            schedule = F.build_schedule(ws, self.config, top_experts, num_local_experts=self.num_local_experts)
        return moe_experts(self.config, ws, schedule, x, router_weights, self.shared_gate, self.shared_up, self.shared_down,
                           self.routed_gate, self.routed_up, self.routed_down, self.swiglu_limit, self.quantised())
