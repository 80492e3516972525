"""The library's process-wide environment switches select other kernel shapes for the same arithmetic.  Each switch is
read once per process, so every setting runs in a child process: a small BF16 and a small MXFP8 forward + backward,
checked against the oracle there, and a digest of all results printed for comparison with the default build of the
path."""
import hashlib
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SWITCHES = ("MOK_B200_LEAN_QUANT", "MOK_B200_2CTA", "MOK_B200_MX_2CTA", "MOK_B200_CHUNKS", "MOK_B200_OVERLAP_SHARED")


def child() -> None:
    sys.path[:0] = [ROOT, os.path.join(ROOT, "mixture-of-kittens_b200")]
    import torch
    import torch.distributed as dist
    from oracle import mok_oracle as O
    from tests.helpers import BF16_REL_L2, MXFP8_REL_L2, rel_l2
    from tests.test_gpu_layer import GRAD_NAMES, run_layer

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dist.init_process_group("gloo", rank=0, world_size=1)
    cfg = dict(T=1024, H=512, I=768, E=8, W=1, K=4)
    inp = O.make_rank_inputs(0, seed=23, **cfg)
    digests, worst = {}, {}
    for mxfp8 in (False, True):
        ref = O.layer_forward_backward([inp], swiglu_limit=None, device_rounding=True, mxfp8=mxfp8)[0]
        got = run_layer(dev, dist.group.WORLD, inp, mxfp8=mxfp8, macrobatch=2048, multiplier=4.0)
        h = hashlib.sha256()
        errs = []
        for name in ("output",) + GRAD_NAMES:
            errs.append(rel_l2(ref[name].float(), got[name].float()))
            h.update(got[name].contiguous().cpu().view(torch.uint8).numpy().tobytes())
        key = "mxfp8" if mxfp8 else "bf16"
        digests[key], worst[key] = h.hexdigest(), max(errs)
        assert worst[key] < (MXFP8_REL_L2 if mxfp8 else BF16_REL_L2), (key, errs)
    print("RESULT " + json.dumps({"digests": digests, "worst": worst}), flush=True)
    dist.destroy_process_group()


def run_child(port: int, **env_switches: str) -> dict:
    env = {k: v for k, v in os.environ.items() if k not in SWITCHES}
    env.update(env_switches, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    proc = subprocess.run([sys.executable, os.path.abspath(__file__)], env=env, capture_output=True, text=True, timeout=100)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    line = [ln for ln in proc.stdout.splitlines() if ln.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


@pytest.fixture(scope="module")
def default_results(cuda_device):
    return run_child(29581)


def test_lean_quantising_dispatch_is_bit_identical(cuda_device, default_results):
    """64-thread CTAs on 32 x 128 tiles quantise the same 1x32 and 32x1 blocks as the 256-thread shape."""
    got = run_child(29582, MOK_B200_LEAN_QUANT="1")
    assert got["digests"] == default_results["digests"]


def test_one_cta_gemm_tiles_meet_the_same_bounds(cuda_device, default_results):
    """128 x 256 tiles per CTA instead of 256 x 256 per CTA pair, BF16 and MXFP8 (the child checks against the oracle)."""
    got = run_child(29583, MOK_B200_2CTA="0", MOK_B200_MX_2CTA="0")
    assert got["worst"]["bf16"] < 1e-2 and got["worst"]["mxfp8"] < 3e-2


def test_chunked_pipeline_on_one_rank_is_bit_identical(cuda_device, default_results):
    """Four row chunks per window on two streams, the row gather beside the shared expert: same results."""
    got = run_child(29584, MOK_B200_CHUNKS="4", MOK_B200_OVERLAP_SHARED="1")
    assert got["digests"] == default_results["digests"]


if __name__ == "__main__":
    child()
