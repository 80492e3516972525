"""ctypes binding of libmok_b200.so (the C ABI declared in include/mok_b200.h).

This is the counterpart of the reference's pybind11 module `mok._C` (csrc/bindings.cu:6-78 in
Mixture-of-Kittens): the same ten operations, but behind plain C entry points that take raw
device pointers.  There is no fallback: if the shared library is missing, importing `mok` fails.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.environ.get("MOK_B200_LIB", os.path.join(_PKG_DIR, "lib", "libmok_b200.so"))

MAX_PEERS = 8
MAX_LOCAL_EXPERTS = 1024

STATUS_NAMES = {0: "ok", 1: "schedule capacity exceeded", 2: "device barrier timed out",
                3: "kernel pipeline wait timed out"}


class MokNativeError(RuntimeError):
    pass


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"libmok_b200.so not found at {LIB_PATH}. Build it with "
            "`python mixture-of-kittens_b200/csrc/build.py` (needs nvcc with sm_100a support); "
            "there is no CPU or PyTorch fallback for the MoE kernels.")
    return C.CDLL(LIB_PATH)


lib = _load()

u64p = C.POINTER(C.c_uint64)
vp = C.c_void_p


class LayerCommon(C.Structure):
    _fields_ = [
        ("ep_size", C.c_int), ("ep_rank", C.c_int),
        ("num_local_tokens", C.c_int), ("hidden", C.c_int), ("intermediate", C.c_int),
        ("num_local_experts", C.c_int), ("topk", C.c_int),
        ("schedule_capacity", C.c_int), ("macrobatch_size", C.c_int), ("minibatch_size", C.c_int),
        ("num_comm_sms", C.c_int),
        ("has_swiglu_limit", C.c_int), ("swiglu_limit", C.c_float), ("defer_combine", C.c_int),
        ("schedule_peer_rank", vp), ("schedule_peer_token_idx", vp),
        ("num_tokens", vp), ("tokens_per_expert", vp), ("status", vp),
    ]


class FwdBf16Args(C.Structure):
    _fields_ = [
        ("c", LayerCommon),
        ("x_ptrs", u64p), ("combine_buffer_ptrs", u64p),
        ("w_shared_gate", vp), ("w_shared_up", vp), ("w_shared_down", vp),
        ("w_routed_gate", vp), ("w_routed_up", vp), ("w_routed_down", vp),
        ("x_routed", vp),
        ("gate_shared", vp), ("up_shared", vp), ("hidden_shared", vp),
        ("gate_routed", vp), ("up_routed", vp), ("hidden_routed", vp),
        ("y_shared", vp), ("y_routed", vp),
    ]


class BwdBf16Args(C.Structure):
    _fields_ = [
        ("c", LayerCommon),
        ("d_y_ptrs", u64p), ("d_x_routed_buffer_ptrs", u64p),
        ("router_weight_ptrs", u64p), ("d_router_weight_ptrs", u64p), ("x_ptrs", u64p),
        ("w_shared_gate", vp), ("w_shared_up", vp), ("w_shared_down", vp),
        ("w_routed_gate", vp), ("w_routed_up", vp), ("w_routed_down", vp),
        ("x_routed", vp), ("gate_routed", vp), ("up_routed", vp), ("hidden_routed", vp),
        ("gate_shared", vp), ("up_shared", vp), ("hidden_shared", vp),
        ("d_x_shared", vp), ("d_x_routed", vp),
        ("d_gate_shared", vp), ("d_up_shared", vp), ("d_hidden_shared", vp),
        ("d_gate_routed", vp), ("d_up_routed", vp), ("d_hidden_routed", vp),
        ("d_y_routed", vp),
        ("d_w_shared_gate", vp), ("d_w_shared_up", vp), ("d_w_shared_down", vp),
        ("d_w_routed_gate", vp), ("d_w_routed_up", vp), ("d_w_routed_down", vp),
        ("router_weights_routed", vp), ("d_router_weight_partials", vp),
    ]


def _ptr_struct(name: str, fields: str, ptr_arrays: str) -> type:
    """A ctypes Structure of `c` (LayerCommon), some uint64* arrays and then plain pointers, in order."""
    f = [("c", LayerCommon)] + [(n, u64p) for n in ptr_arrays.split()] + [(n, vp) for n in fields.split()]
    return type(name, (C.Structure,), {"_fields_": f})


FwdMxfp8Args = _ptr_struct(
    "FwdMxfp8Args",
    "w_shared_gate w_shared_up w_shared_down w_routed_gate_q w_routed_gate_sc w_routed_up_q w_routed_up_sc "
    "w_routed_down_q w_routed_down_sc x_qt x_sct gate_shared up_shared hidden_shared gate_q gate_sc up_q up_sc "
    "hidden_qt hidden_sct y_shared y_routed work_x_q work_x_sc work_hidden_q work_hidden_sc",
    "x_ptrs combine_buffer_ptrs")

BwdMxfp8Args = _ptr_struct(
    "BwdMxfp8Args",
    "w_shared_gate w_shared_up w_shared_down w_routed_gate_T_q w_routed_gate_T_sc w_routed_up_T_q w_routed_up_T_sc "
    "w_routed_down_T_q w_routed_down_T_sc w_routed_gate_q w_routed_gate_sc w_routed_up_q w_routed_up_sc "
    "x_qt x_sct gate_q gate_sc up_q up_sc hidden_qt hidden_sct gate_shared up_shared hidden_shared "
    "d_x_shared d_x_routed d_gate_shared d_gate_q d_gate_sc d_up_shared d_up_q d_up_sc d_hidden_shared d_hidden_routed "
    "d_y_q d_y_sc d_w_shared_gate d_w_shared_up d_w_shared_down d_w_routed_gate d_w_routed_up d_w_routed_down "
    "work_x_q work_x_sc work_hidden_q work_hidden_sc work_d_y_qt work_d_y_sct work_d_gate_qt work_d_gate_sct "
    "work_d_up_qt work_d_up_sct router_weights_routed d_router_weight_partials",
    "d_y_ptrs d_x_routed_buffer_ptrs router_weight_ptrs d_router_weight_ptrs x_ptrs")


def _sig(name, restype, argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = argtypes
    return fn


mok_version = _sig("mok_version", C.c_int, [])
mok_error_string = _sig("mok_error_string", C.c_char_p, [C.c_int])
mok_last_cuda_error = _sig("mok_last_cuda_error", C.c_char_p, [])
mok_all_gather_top_experts = _sig("mok_all_gather_top_experts", C.c_int, [vp, C.c_int64, u64p, C.c_int, C.c_int, vp])
mok_barrier_all = _sig("mok_barrier_all", C.c_int, [vp, u64p, C.c_int, vp, vp, C.c_uint64, vp])
mok_schedule_scratch_bytes = _sig("mok_schedule_scratch_bytes", C.c_size_t, [C.c_int, C.c_int])
mok_schedule = _sig("mok_schedule", C.c_int, [vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                              vp, vp, vp, vp, vp, C.c_size_t, vp, vp])
mok_schedule_static_max_scratch_bytes = _sig("mok_schedule_static_max_scratch_bytes", C.c_size_t, [])
mok_schedule_static = _sig("mok_schedule_static", C.c_int, [vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                                            vp, vp, vp, vp, vp, vp])
mok_mxfp8_quantize = _sig("mok_mxfp8_quantize", C.c_int, [vp, C.c_int, C.c_int, C.c_int, vp, vp, vp, vp, vp])
mok_fwd_epilogue = _sig("mok_fwd_epilogue", C.c_int, [vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, vp])
mok_bwd_epilogue = _sig("mok_bwd_epilogue", C.c_int, [vp, vp, vp, C.c_int, C.c_int, C.c_int, vp])
mok_router_topk = _sig("mok_router_topk", C.c_int, [vp, C.c_int, C.c_int, C.c_int, vp, vp, vp, u64p, C.c_int, C.c_int, vp])
mok_router_topk_bwd = _sig("mok_router_topk_bwd", C.c_int, [vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, vp])
mok_fwd_epilogue_rows = _sig("mok_fwd_epilogue_rows", C.c_int,
                             [vp, vp, vp, vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, vp])
mok_bwd_epilogue_rows = _sig("mok_bwd_epilogue_rows", C.c_int,
                             [vp, vp, vp, C.c_int, vp, vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, vp])
mok_fwd_bf16 = _sig("mok_fwd_bf16", C.c_int, [C.POINTER(FwdBf16Args), vp])
mok_bwd_bf16 = _sig("mok_bwd_bf16", C.c_int, [C.POINTER(BwdBf16Args), vp])
mok_fwd_mxfp8 = _sig("mok_fwd_mxfp8", C.c_int, [C.POINTER(FwdMxfp8Args), vp])
mok_bwd_mxfp8 = _sig("mok_bwd_mxfp8", C.c_int, [C.POINTER(BwdMxfp8Args), vp])
mok_gemm_mxfp8 = _sig("mok_gemm_mxfp8", C.c_int, [vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, vp, vp])
mok_launch_count = _sig("mok_launch_count", C.c_longlong, [])
mok_profile_enable = _sig("mok_profile_enable", C.c_int, [C.c_int])
mok_profile_num_slots = _sig("mok_profile_num_slots", C.c_int, [])
mok_profile_slot_name = _sig("mok_profile_slot_name", C.c_char_p, [C.c_int])
mok_profile_collect = _sig("mok_profile_collect", C.c_int, [C.POINTER(C.c_double), C.POINTER(C.c_longlong)])
mok_gemm_bf16 = _sig("mok_gemm_bf16", C.c_int, [vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp, vp])


class WorkspaceBytes(C.Structure):
    _fields_ = [("schedule_capacity", C.c_int64)] + [(n, C.c_size_t) for n in (
        "x_buffer combine_buffer d_y_buffer d_x_routed_buffer router_weight_buffer d_router_weight_buffer "
        "all_gather_top_experts_buffer barrier_buffer barrier_target status_word schedule_tables schedule_scratch").split()]


mok_query_workspace_bytes = _sig("mok_query_workspace_bytes", C.c_int,
                                 [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_double, C.POINTER(WorkspaceBytes)])
mok_last_status = _sig("mok_last_status", C.c_int, [vp, C.POINTER(C.c_int32), C.c_int, vp])


def check(rc: int, what: str) -> None:
    """Turns a negative return code of the C ABI into a Python exception."""
    if rc == 0:
        return
    msg = mok_error_string(rc).decode()
    if rc == -1:
        raise ValueError(f"{what}: {msg}")
    if rc == -3:
        raise NotImplementedError(f"{what}: {msg}")
    if rc == -4:
        raise ValueError(f"{what}: {msg}")
    if rc == -2:
        detail = mok_last_cuda_error().decode()
        raise MokNativeError(f"{what}: {msg}: {detail}")
    raise MokNativeError(f"{what}: {msg}")


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr_array(ptrs) -> C.Array:
    return (C.c_uint64 * len(ptrs))(*[int(p) for p in ptrs])


# ---- per-device status word (device-detected errors) ------------------------------------------
_STATUS: dict[int, torch.Tensor] = {}


def status_tensor(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _STATUS.get(idx)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", idx))
        _STATUS[idx] = t
    return t


def last_status(device: torch.device | None = None, clear: bool = False) -> tuple[int, int, int]:
    """Reads the status word of `device` (synchronises).  Returns (code, detail, block)."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    t = status_tensor(device)
    out = (C.c_int32 * 4)()
    with torch.cuda.device(device):
        check(mok_last_status(t.data_ptr(), out, 1 if clear else 0, stream_ptr(device)), "last_status")
    return int(out[0]), int(out[1]), int(out[2])


def raise_for_status(device: torch.device | None = None) -> None:
    code, detail, block = last_status(device)
    if code != 0:
        raise MokNativeError(f"device status {code} ({STATUS_NAMES.get(code, '?')}), detail={detail}, block={block}")


# ---- peer pointers of the top-k all-gather buffers --------------------------------------------
# The reference op signature carries only an NVLS multicast pointer for this buffer.  This build
# uses plain peer stores, so workspaces register the per-rank addresses of their buffer here,
# keyed by the local buffer address.
_ALL_GATHER_PEERS: dict[int, list[int]] = {}


def register_all_gather_peers(local_ptr: int, peer_ptrs: list[int]) -> None:
    _ALL_GATHER_PEERS[int(local_ptr)] = [int(p) for p in peer_ptrs]


def unregister_all_gather_peers(local_ptr: int) -> None:
    _ALL_GATHER_PEERS.pop(int(local_ptr), None)


def all_gather_peers(local_ptr: int) -> list[int] | None:
    return _ALL_GATHER_PEERS.get(int(local_ptr))


def profile_collect() -> dict[str, tuple[float, int]]:
    """Device milliseconds and launch counts per slot recorded since the last call (synchronises)."""
    n = mok_profile_num_slots()
    ms = (C.c_double * n)()
    cnt = (C.c_longlong * n)()
    check(mok_profile_collect(ms, cnt), "profile_collect")
    return {mok_profile_slot_name(i).decode(): (ms[i], cnt[i]) for i in range(n) if cnt[i]}
