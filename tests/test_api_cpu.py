"""CPU: the Python boundary mirrors the reference's operator/functional interface — names, defaults,
exception classes raised before any launch, FakeTensor shape propagation, mutation schemas
(reference: mok/functional.py:22-48, mok/ops.py validation blocks, tests/test_misc.py:582-1043)."""
import dataclasses
import os

import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode


def test_config_defaults_and_dataclasses():
    import mok
    F = mok.functional
    cfg = F.MoKConfig()
    assert dataclasses.asdict(cfg) == dict(fwd_num_comm_sms=40, bwd_num_comm_sms=28, minibatch_size=4096,
                                           macrobatch_size=131072, schedule_capacity_multiplier=0.5,
                                           all_gather_top_experts_chunk_bytes=2048)
    with pytest.raises(dataclasses.FrozenInstanceError):
        cfg.minibatch_size = 1
    assert [f.name for f in dataclasses.fields(F.MoKSchedule)] == ["peer_rank", "peer_token_idx", "num_tokens",
                                                                   "tokens_per_expert"]
    assert [f.name for f in dataclasses.fields(F.MoKForwardContext)] == [
        "x_routed", "gate_shared", "gate_routed", "up_shared", "up_routed", "hidden_shared", "hidden_routed"]
    assert len(dataclasses.fields(F.MoKWorkspace)) == 34
    assert F.schedule is F.build_schedule
    assert mok.__version__ == "0.1.0"


def test_ten_operators_are_registered():
    import mok  # noqa: F401
    names = ["all_gather_top_experts", "barrier_all", "schedule", "mxfp8_quantize",
             "dispatch_mlp_swiglu_combine_fwd_mxfp8", "dispatch_mlp_swiglu_combine_fwd_bf16",
             "dispatch_mlp_swiglu_combine_bwd_mxfp8", "dispatch_mlp_swiglu_combine_bwd_bf16",
             "fwd_epilogue", "bwd_epilogue"]
    for n in names:
        assert hasattr(torch.ops.mok, n), n


def test_mutation_schemas():
    import mok  # noqa: F401
    def mutated(op):
        return {a.name for a in op.default._schema.arguments if a.alias_info is not None and a.alias_info.is_write}
    assert mutated(torch.ops.mok.all_gather_top_experts) == {"all_gather_top_experts_buffer"}
    assert mutated(torch.ops.mok.barrier_all) == {"barrier_buffer", "target"}
    assert mutated(torch.ops.mok.schedule) == set()
    assert mutated(torch.ops.mok.dispatch_mlp_swiglu_combine_fwd_bf16) == {"combine_buffer"}
    assert mutated(torch.ops.mok.dispatch_mlp_swiglu_combine_bwd_bf16) == {
        "d_x_routed_buffer", "d_router_weight_buffer", "x_routed", "gate_routed", "up_routed", "hidden_routed"}
    assert mutated(torch.ops.mok.dispatch_mlp_swiglu_combine_bwd_mxfp8) == {
        "d_x_routed_buffer", "d_router_weight_buffer", "x_fp8_t_routed", "x_sc_t_routed", "gate_fp8_routed",
        "gate_sc_routed", "up_fp8_routed", "up_sc_routed", "hidden_fp8_t_routed", "hidden_sc_t_routed"}


def test_argument_errors_are_raised_before_any_launch():
    import mok
    ops = mok.ops
    i32 = torch.int32
    with pytest.raises(ValueError):
        ops.schedule(torch.zeros(3, 512, 2, dtype=i32), 4, 4096, 0)            # ep size 3
    with pytest.raises(ValueError):
        ops.schedule(torch.zeros(4, 500, 2, dtype=i32), 4, 4096, 0)            # tokens not a multiple of 256
    with pytest.raises(ValueError):
        ops.schedule(torch.zeros(4, 512, 2, dtype=i32), 4, 1000, 0)            # capacity not a multiple of 256
    with pytest.raises(ValueError):
        ops.schedule(torch.zeros(4, 512, 2, dtype=i32), 4, 512, 0)             # capacity below one rank's routes
    with pytest.raises(ValueError):
        ops.schedule(torch.zeros(4, 512, 2, dtype=i32), 4, 4096, 4)            # rank out of range
    with pytest.raises(ValueError):
        ops.mxfp8_quantize(torch.zeros(100, 128, dtype=torch.bfloat16), True, False)
    with pytest.raises(TypeError):
        ops.mxfp8_quantize(torch.zeros(128, 128, dtype=torch.bfloat16), 1, False)
    with pytest.raises(ValueError):
        ops.mxfp8_quantize(torch.zeros(128, 128, dtype=torch.bfloat16), False, False)
    with pytest.raises(ValueError):
        ops.fwd_epilogue(torch.zeros(500, 256, dtype=torch.bfloat16), torch.zeros(1000, 256, dtype=torch.bfloat16),
                         torch.zeros(500, 2))
    with pytest.raises(ValueError):
        ops.bwd_epilogue(torch.zeros(512, 256, dtype=torch.bfloat16), torch.zeros(700, 256, dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        ops.barrier_all(torch.zeros(1, dtype=i32), [1, 2, 3, 4], 0, torch.zeros(1, dtype=i32))   # not a CUDA buffer
    with pytest.raises(ValueError):
        ops.all_gather_top_experts(torch.zeros(512, 2, dtype=i32), torch.zeros(4, 512, 2, dtype=i32), 0, 0, 2048)


def test_fake_tensor_shapes():
    import mok
    ops = mok.ops
    T, H, I, El, K, MB, cap, W = 512, 256, 512, 4, 2, 1024, 2048, 4
    with FakeTensorMode():
        dev = "cuda"
        bf = lambda *s: torch.empty(*s, dtype=torch.bfloat16, device=dev)          # noqa: E731
        f8 = lambda *s: torch.empty(*s, dtype=torch.float8_e4m3fn, device=dev)     # noqa: E731
        u8 = lambda *s: torch.empty(*s, dtype=torch.uint8, device=dev)             # noqa: E731
        i32 = lambda *s: torch.empty(*s, dtype=torch.int32, device=dev)            # noqa: E731
        sc = lambda r, c: u8(r // 128, c // 128, 32, 16)                           # noqa: E731
        ptrs = [1, 2, 3, 4]
        sched = (i32(cap), i32(cap), i32(1), i32(El))
        out = ops.schedule(i32(W, T, K), El, cap, 0)
        assert [tuple(t.shape) for t in out] == [(cap,), (cap,), (1,), (El,)]
        q = ops.mxfp8_quantize(bf(El, I, H), True, True)
        assert tuple(q[0].shape) == (El, I, H) and tuple(q[1].shape) == (El * I // 128, H // 128, 32, 16)
        assert tuple(q[2].shape) == (El, H, I) and tuple(q[3].shape) == (El * H // 128, I // 128, 32, 16)
        assert ops.mxfp8_quantize(bf(I, H), True, False)[2] is None
        fwd = ops.dispatch_mlp_swiglu_combine_fwd_bf16(bf(T, H), ptrs, bf(T * K, H), ptrs, bf(I, H), bf(El, I, H), bf(I, H),
                                                       bf(El, I, H), bf(H, I), bf(El, H, I), *sched, K, None, 40, MB, 256)
        assert [tuple(t.shape) for t in fwd] == [(MB, H), (T, I), (MB, I), (T, I), (MB, I), (T, I), (MB, I), (T, H), (MB, H)]
        fwd8 = ops.dispatch_mlp_swiglu_combine_fwd_mxfp8(
            bf(T, H), ptrs, bf(T * K, H), ptrs, bf(I, H), f8(El, I, H), sc(El * I, H), bf(I, H), f8(El, I, H), sc(El * I, H),
            bf(H, I), f8(El, H, I), sc(El * H, I), *sched, K, 4.0, 40, MB, 256)
        assert [tuple(t.shape) for t in fwd8] == [(H, MB), (H // 128, MB // 128, 32, 16), (T, I), (MB, I),
                                                  (MB // 128, I // 128, 32, 16), (T, I), (MB, I), (MB // 128, I // 128, 32, 16),
                                                  (T, I), (I, MB), (I // 128, MB // 128, 32, 16), (T, H), (MB, H)]
        assert fwd8[0].dtype == torch.float8_e4m3fn and fwd8[1].dtype == torch.uint8 and fwd8[12].dtype == torch.bfloat16
        bwd = ops.dispatch_mlp_swiglu_combine_bwd_bf16(
            bf(T, H), ptrs, bf(T * K, H), ptrs, torch.empty(T, K, device=dev), ptrs, torch.empty(T, K, device=dev), ptrs,
            bf(I, H), bf(El, I, H), bf(I, H), bf(El, I, H), bf(H, I), bf(El, H, I),
            bf(MB, H), bf(T, I), bf(MB, I), bf(T, I), bf(MB, I), bf(T, I), bf(MB, I), bf(T, H), ptrs, *sched, K, None, 28, MB, 256)
        assert len(bwd) == 15 and tuple(bwd[10].shape) == (El, I, H) and tuple(bwd[14].shape) == (El, H, I)
        assert tuple(ops.fwd_epilogue(bf(T, H), bf(T * K, H), torch.empty(T, K, device=dev)).shape) == (T, H)
        assert tuple(ops.bwd_epilogue(bf(T, H), bf(T * K, H)).shape) == (T, H)


def test_added_operators_and_wrappers():
    """The operators this build adds on top of the reference's ten, their schemas, fake shapes and argument errors."""
    import mok
    ops = mok.ops
    for n in ("router_topk", "router_topk_gather", "router_topk_bwd", "fwd_epilogue_rows"):
        assert hasattr(torch.ops.mok, n), n
    def mutated(op):
        return {a.name for a in op.default._schema.arguments if a.alias_info is not None and a.alias_info.is_write}
    assert mutated(torch.ops.mok.router_topk) == set()
    assert mutated(torch.ops.mok.router_topk_gather) == {"all_gather_top_experts_buffer"}
    assert mutated(torch.ops.mok.fwd_epilogue_rows) == set()
    # defer_combine is a trailing, defaulted argument of the four layer operators
    for n in ("dispatch_mlp_swiglu_combine_fwd_bf16", "dispatch_mlp_swiglu_combine_bwd_bf16",
              "dispatch_mlp_swiglu_combine_fwd_mxfp8", "dispatch_mlp_swiglu_combine_bwd_mxfp8"):
        last = getattr(torch.ops.mok, n).default._schema.arguments[-1]
        assert last.name == "defer_combine" and last.default_value is False
    with pytest.raises(ValueError):
        ops.router_topk(torch.zeros(512, 64), 6)                                # not a CUDA tensor
    with pytest.raises(ValueError):
        ops.router_topk_bwd(torch.zeros(512, 6, dtype=torch.int64), torch.zeros(512, 6), torch.zeros(512, 6), 64)
    with FakeTensorMode():
        dev = "cuda"
        e, w = ops.router_topk(torch.empty(512, 64, device=dev), 6)
        assert tuple(e.shape) == (512, 6) and e.dtype == torch.int64 and w.dtype == torch.float32
        e, w = ops.router_topk_gather(torch.empty(512, 64, device=dev), 6,
                                      torch.empty(4, 512, 6, dtype=torch.int32, device=dev), 1)
        assert tuple(w.shape) == (512, 6)
        g = ops.router_topk_bwd(e, w, w, 64)
        assert tuple(g.shape) == (512, 64) and g.dtype == torch.float32
        out = ops.fwd_epilogue_rows(torch.empty(512, 256, dtype=torch.bfloat16, device=dev),
                                    torch.empty(4096, 256, dtype=torch.bfloat16, device=dev),
                                    torch.empty(4096, dtype=torch.int32, device=dev),
                                    torch.empty(4096, dtype=torch.int32, device=dev),
                                    torch.empty(1, dtype=torch.int32, device=dev), torch.empty(512, 2, device=dev))
        assert tuple(out.shape) == (512, 256) and out.dtype == torch.bfloat16
    assert mok.ops.SELF_PTRS == [-1]
    assert callable(mok.nn.moe_experts) and issubclass(mok.nn.MoKLayer, torch.nn.Module)
    assert callable(mok.functional.route) and callable(mok.functional.route_and_schedule)


# ------------------------------------------------------------------------------------------
# bench.py helpers that run without a GPU
# ------------------------------------------------------------------------------------------
def test_bench_mx_emulation_matches_the_oracle_quantiser():
    """bench.py checks MXFP8 runs against an fp32 recomputation whose operands go through a block
    quantise-dequantise written with torch ops; it must be the oracle's quantiser bit for bit."""
    import torch
    import bench
    from oracle import mok_oracle as O
    g = torch.Generator().manual_seed(1)
    t = (torch.randn(64, 256, generator=g) * torch.exp(torch.randn(64, 1, generator=g) * 4)).to(torch.bfloat16).float()
    t[3] = 0
    t[5, :32] = 0
    t[7] = 448.0
    t[8] = 2.0 ** -20
    t[9, :32] = torch.tensor([448.0 * 2.0 ** k for k in range(-16, 16)]).to(torch.bfloat16).float()
    for axis in (0, 1):
        assert torch.equal(bench.mx_quant_dequant(t, axis), O._mx(t, axis)), axis


def test_bench_traffic_model_and_roofline_fractions():
    import bench
    full = bench.dominant_traffic("C2", 128, 145664)
    assert full == 6291456 * 128 + 8322 * 145664
    assert bench.dominant_traffic("C4", 32, 1000) is None            # no capture on file: the line prints null
    wl = bench.WORKLOADS["C2"]
    res = {"prof": {"gemm_gate_up_swiglu_routed": (66.18, 100)}, "n_rows": 145664}
    roof = bench.roofline_record("C2", wl, res, 100, 1)
    assert abs(roof["achieved"] - 4 * 16384 * 8 * 2048 * 768 / 0.6618e-3 / 1e12) < 1e-6
    assert roof["frac_vs_burst"] < roof["frac_vs_sustained"]
    short = bench.finish_roofline(dict(roof), 0.07, {"reasons": []})
    assert short["peak"] == roof["burst_peak"] and short["frac"] == roof["frac_vs_burst"]
    capped = bench.finish_roofline(dict(roof), 0.07, {"reasons": ["sw_power_cap"]})
    assert capped["peak"] == roof["sustained_peak"]
    long_run = bench.finish_roofline(dict(roof), 3.0, {"reasons": []})
    assert long_run["frac"] == roof["frac_vs_sustained"]


def test_bench_sampled_check_is_pinned_to_the_oracle():
    """bench.py's after-run parity check recomputes sampled tokens on its own; fed with the oracle's results for
    the same seeded two-rank inputs it must report (almost) no error, in BF16 and in MXFP8 arithmetic."""
    import types
    import torch
    import bench
    from oracle import mok_oracle as O
    cpu = torch.device("cpu")
    for mx in (False, True):
        wl = dict(T=512, H=256, I=256, E=8, K=3, router="linear", backward=True, mxfp8=mx)
        W = 2
        raw = [bench.make_inputs(wl, p, W, cpu, pinned=False) for p in range(W)]
        ranks = [O.RankInputs(x=s["x"], topk_experts=s["topk"], router_weights=s["rw"], w_shared_gate=prm[0],
                              w_shared_up=prm[1], w_shared_down=prm[2], w_routed_gate=prm[3], w_routed_up=prm[4],
                              w_routed_down=prm[5], d_output=s["d_out"]) for s, prm in raw]
        ref = O.layer_forward_backward(ranks, device_rounding=True, mxfp8=mx)
        for rank in range(W):
            r = ref[rank]
            sched = types.SimpleNamespace(tokens_per_expert=torch.from_numpy(r["tokens_per_expert"]),
                                          peer_rank=torch.from_numpy(r["peer_rank"]),
                                          peer_token_idx=torch.from_numpy(r["peer_token_idx"]))
            grads = tuple(r[n] for n in ("d_x", "d_router_weights", "d_w_routed_gate", "d_w_routed_up", "d_w_routed_down"))
            got = bench.sampled_parity(wl, rank, W, cpu, raw[rank][0], r["output"], grads, sched, None, 16)
            want = {"output", "d_x", "d_router_weights"} | (set() if mx else {"d_w_routed_down_rows"})
            assert set(got) == want
            for name, err in got.items():
                assert err < 3e-3, (mx, rank, name, err)


def test_bench_reference_arm_runs_on_rank_zero_only_and_c1_line(tmp_path):
    """Launched as one rank per GPU, the reference arm is a single CPU process: every rank but 0 exits 0 without
    work or output.  The small CPU configuration prints its own line (GFLOP/s, core count, median of >= 10)."""
    import json
    import subprocess
    import sys
    from tests.conftest import ROOT
    bench_py = os.path.join(ROOT, "bench.py")
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    idle = subprocess.run([sys.executable, bench_py, "--impl", "reference", "--gpus", "2", "--steps", "3", "--warmup", "1"],
                          env=env, capture_output=True, text=True, timeout=300)
    assert idle.returncode == 0 and idle.stdout.strip() == ""
    c1 = subprocess.run([sys.executable, bench_py, "--workload", "C1", "--steps", "10"], capture_output=True, text=True,
                        timeout=300)
    assert c1.returncode == 0, c1.stderr[-2000:]
    line = json.loads(c1.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "GFLOP/s" and line["steps"] >= 10
    assert line["cpu_baseline"]["cores"] >= 1 and line["value"] > 0
