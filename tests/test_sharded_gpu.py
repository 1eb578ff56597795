"""KV-sharded decode on real GPUs: one process per GPU, both exchange implementations (the merge kernel that carries
the exchange over peer memory, and the NCCL all-gather path) against the unsharded CPU attn(). Needs at least two
visible GPUs; skipped otherwise. Ranks leave only between steps, with nothing in flight."""
import os
import socket
import sys

import numpy as np
import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from conftest import load_package
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    pkg = load_package()
    import oracle
    from llm_infer_b200 import attention
    from llm_infer_b200.sharded import FusedShardedDecode, ShardedDecode, shard_rows
    wl = pkg.workloads
    T = 5000  # not a multiple of the world size or of the tile: ragged shards
    shape = wl.DecodeShape("sharded", 3, 1, 32, 8, 128, T, "f16", "f16")
    q, k, v = wl.decode_inputs(shape)
    r0, r1 = shard_rows(T, world, rank)
    qd = torch.from_numpy(q).to(dev)
    kd, vd = torch.from_numpy(k[:, r0:r1].copy()).to(dev), torch.from_numpy(v[:, r0:r1].copy()).to(dev)
    want = oracle.best().attn_decode(q.astype(np.float32), k, v)[0]

    fused = FusedShardedDecode(1, 32, 8, 128, device=dev)
    out = torch.full((1, 32, 128), float("nan"), device=dev)
    errs = []
    for _ in range(3):  # consecutive steps: record parity alternates, device-side step counter advances
        out.fill_(float("nan"))
        fused(qd, kd, vd, out=out)
        torch.cuda.synchronize()
        errs.append(wl.error_metrics(out[0].cpu().numpy(), want))
    fused.kv_early = True  # the local pass streams ahead of the previous kernel (the cache does not change here)
    for _ in range(2):
        out.fill_(float("nan"))
        fused(qd, kd, vd, out=out)
        torch.cuda.synchronize()
        errs.append(wl.error_metrics(out[0].cpu().numpy(), want))
    status = int(fused.workspace.status.item())

    nccl = ShardedDecode(32, 128, device=dev)
    out2 = nccl(qd, kd, vd)
    torch.cuda.synchronize()
    errs.append(wl.error_metrics(out2.cpu().numpy(), want))
    np.save(os.path.join(result_dir, f"r{rank}.npy"), np.array([max(e[0] for e in errs), max(e[1] for e in errs), status]))
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)  # symmetric-memory handles and the communicator are torn down with the process


def test_two_ranks_fused_and_nccl_exchange(built_lib, pkg, tmp_path):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, str(tmp_path))) for r in range(world)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(timeout=120)
    for pr in procs:
        if pr.is_alive():
            pr.kill()  # the exact processes this test started
            pytest.fail("a rank did not finish within 120 s")
        assert pr.exitcode == 0
    wl = pkg.workloads
    for r in range(world):
        max_abs, max_rel, status = np.load(tmp_path / f"r{r}.npy")
        assert status == 0
        assert max_abs <= wl.ABS_TOL and max_rel <= wl.REL_TOL, (r, max_abs, max_rel)
