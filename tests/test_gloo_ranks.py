"""CPU, world_size 2 over gloo: the host-side logic of the multi-rank path.  Each rank builds its
seeded inputs, the ranks exchange their top-k ids with a gloo all-gather (what the device
all-gather does over NVLink), every rank derives its slot tables with the oracle, and together
they check that the tables partition the routes: every route is served exactly once, by the rank
that owns its expert, in 256-padded expert segments."""
import os

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world, port, out):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    from oracle import mok_oracle as O
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    T, K, E = 512, 3, 8
    El = E // world
    inp = O.make_rank_inputs(rank, T=T, H=256, I=256, E=E, W=world, K=K, seed=3)
    mine = inp.topk_experts.to(torch.int32)
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    topk_all = torch.stack(parts).numpy()
    cap = T * K * max(2, world)
    pr, pt, nt, tpe = O.schedule_tables(topk_all, El, cap, rank)
    valid = pr >= 0
    served = np.zeros((world, T * K), dtype=np.int64)
    np.add.at(served, (pr[valid], pt[valid]), 1)
    total = torch.from_numpy(served)
    dist.all_reduce(total)
    ok = bool((total == 1).all()) and int(nt[0]) == int(tpe.sum()) and bool((tpe % 256 == 0).all())
    owners = topk_all.reshape(world, -1)[pr[valid], pt[valid]] // El
    ok = ok and bool((owners == rank).all())
    flag = torch.tensor([0 if ok else 1])
    dist.all_reduce(flag)
    if rank == 0:
        open(out, "w").write(str(int(flag.item())))
    dist.destroy_process_group()


def test_two_rank_schedule_partitions_routes(tmp_path):
    out = str(tmp_path / "result.txt")
    mp.spawn(_worker, args=(2, 29533, out), nprocs=2)
    assert open(out).read() == "0"
