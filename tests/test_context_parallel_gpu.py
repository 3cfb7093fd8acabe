"""Context parallelism on real GPUs: two ranks (one GPU each, NCCL point-to-point) hold the two halves of the same
sequences; outputs and all seven gradients must be bitwise those of the unsplit run on one GPU.  Skipped on a box with
fewer than two GPUs (the chained-segment test on one GPU, tests/test_segments_gpu.py, covers the kernels themselves)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from cute_triadic_gdn_b200 import _lib, gdn_joint_call
    from cute_triadic_gdn_b200.context_parallel import context_parallel_joint
    from oracle import triadic_oracle as orc
    B, T, H, E = 2, 512, 4, 8
    ins = orc.make_inputs(B, T, H, E, seed=3, dist="mild")
    do = orc.make_grad_output((B, T, H, 128), 4).cuda()
    tl = T // world
    sl = slice(rank * tl, (rank + 1) * tl)
    mine = [t[:, sl].contiguous().cuda().requires_grad_(True) for t in ins]
    o = context_parallel_joint(*mine, head_groups=2)
    o.backward(do[:, sl].contiguous())
    whole = [t.cuda().requires_grad_(True) for t in ins]
    o_ref = gdn_joint_call(*whole)
    o_ref.backward(do)
    ok = torch.equal(o, o_ref[:, sl]) and all(torch.equal(a.grad, b.grad[:, sl]) for a, b in zip(mine, whole))
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as fh:
        fh.write(f"{int(ok)} {_lib.device_status()}")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_match_the_unsplit_run(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        ok, status = open(os.path.join(tmp_path, f"rank{r}.txt")).read().split()
        assert ok == "1" and status == "0", (r, ok, status)
