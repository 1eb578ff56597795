"""Host logic of the KV-sharded decode (row partition, packed (O, LSE) record, all-gather, merge order) run
as real ranks over gloo on CPU. The per-rank compute is the CPU checker standing in for the CUDA kernels, so
what is tested here is everything around the kernels; the kernels themselves are tested on the GPU."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, load_package


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cpu_decode(port):
    def decode(q, k, v, kv_len=None, *, out, lse, **_):
        # q [1,H,D], k/v [1,T,Hkv,D] torch CPU tensors -> per-head (m, z, o) of the local rows
        H, D = q.shape[1], q.shape[2]
        T, Hkv = k.shape[1], k.shape[2]
        n = T if kv_len is None else int(kv_len)
        kn, vn = k[0].numpy().view(np.uint16), v[0].numpy().view(np.uint16)
        for h in range(H):
            m, z, o = port.state_from_rows(q[0, h].float().numpy(), kn, vn, h // (H // Hkv), 0, n) if T else \
                (-np.inf, 0.0, np.zeros(D, np.float32))
            out[0, h] = torch.from_numpy(o)
            lse[0, h] = float(m + np.log(z)) if z > 0 else float("-inf")
    return decode


def _cpu_merge(port):
    def merge(part_o, part_lse, *, out=None, out_dtype=torch.float32):
        n, H, D = part_o.shape
        res = torch.empty((H, D), dtype=torch.float32) if out is None else out
        for h in range(H):
            o, _ = port.lse_merge(part_o[:, h].contiguous().numpy(), part_lse[:, h].contiguous().numpy())
            res[h] = torch.from_numpy(o)
        return res
    return merge


def _worker(rank, world, port_no, total_rows, fail_rank, result_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port_no)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        pkg = load_package()
        import oracle
        from llm_infer_b200.sharded import ShardedDecode, shard_rows
        port = oracle.Oracle("port")
        wl = pkg.workloads
        shape = wl.DecodeShape("sharded", 3, 1, 8, 2, 64, total_rows, "f16", "f16")
        q, k, v = wl.decode_inputs(shape)  # same seed on every rank: identical full inputs
        r0, r1 = shard_rows(total_rows, world, rank)
        op = ShardedDecode(8, 64, device="cpu", decode_fn=_cpu_decode(port), merge_fn=_cpu_merge(port))
        qt = torch.from_numpy(q)
        kt, vt = torch.from_numpy(k[:, r0:r1].copy()), torch.from_numpy(v[:, r0:r1].copy())
        if rank == fail_rank:
            # host-side fault injection: this rank contributes an empty partial (as if its shard were lost)
            op.local_partial(qt, kt[:, :0], vt[:, :0])
            op.gather()
            got = op.merge()
        else:
            got = op(qt, kt, vt)
        if fail_rank is None:
            want = port.attn_decode(q.astype(np.float32), k, v)[0]
        else:
            f0, f1 = shard_rows(total_rows, world, fail_rank)
            keep = np.r_[0:f0, f1:total_rows]
            want = port.attn_decode(q.astype(np.float32), k[:, keep], v[:, keep])[0]
        np.save(os.path.join(result_dir, f"err{rank}.npy"), np.abs(got.numpy() - want).max())
        np.save(os.path.join(result_dir, f"rec{rank}.npy"), op.gathered.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,total_rows,fail_rank", [(2, 200, None), (3, 1000, None), (2, 1, None), (3, 301, 1)])
def test_sharded_decode_over_gloo(tmp_path, world, total_rows, fail_rank):
    mp.spawn(_worker, args=(world, _free_port(), total_rows, fail_rank, str(tmp_path)), nprocs=world, join=True)
    recs = [np.load(tmp_path / f"rec{r}.npy") for r in range(world)]
    for r in range(world):
        assert float(np.load(tmp_path / f"err{r}.npy")) < 2e-6  # every rank holds the full result
        assert np.array_equal(recs[r], recs[0], equal_nan=True)  # and the same gathered records
    # record r really is rank r's partial: LSE of an empty shard is -inf
    lse = recs[0][:, 8 * 64: 8 * 64 + 8]
    for r in range(world):
        r0, r1 = (0, 0) if r == fail_rank else (r * (total_rows // world),
                                                total_rows if r == world - 1 else (r + 1) * (total_rows // world))
        assert np.isneginf(lse[r]).all() == (r1 == r0)


def _watchdog_worker(rank, world, port_no, result_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port_no)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg = load_package()
    import oracle
    from llm_infer_b200.sharded import GatherTimeout, ShardedDecode
    port = oracle.Oracle("port")
    op = ShardedDecode(8, 64, device="cpu", decode_fn=_cpu_decode(port), merge_fn=_cpu_merge(port), watchdog_s=1.0)
    fired = []
    op.on_timeout = lambda: fired.append(True)
    outcome = "no-collective"
    if rank == 0:
        # rank 1 never joins this step (host-side fault injection: it simply does not call the collective)
        try:
            op.gather()
            outcome = "completed"
        except GatherTimeout:
            outcome = "timeout" if fired else "timeout-without-callback"
    else:
        import time
        time.sleep(3.0)  # alive, connected, but never reaches the step
    with open(os.path.join(result_dir, f"watchdog{rank}.txt"), "w") as f:
        f.write(outcome)
    os._exit(0)  # a collective is still pending on rank 0: leave without tearing the group down


def test_gather_watchdog_fires_when_a_rank_never_joins(tmp_path):
    """The host-side deadline around the all-gather: with one of two ranks skipping the step, the other gets
    GatherTimeout (after its on_timeout hook ran) instead of blocking."""
    ctx = mp.get_context("spawn")
    port_no = _free_port()
    procs = [ctx.Process(target=_watchdog_worker, args=(r, 2, port_no, str(tmp_path))) for r in range(2)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(timeout=120)
        assert not pr.is_alive() and pr.exitcode == 0
    assert (tmp_path / "watchdog0.txt").read_text() == "timeout"
    assert (tmp_path / "watchdog1.txt").read_text() == "no-collective"


def test_shard_rows_partition():
    pkg = load_package()
    from llm_infer_b200.sharded import shard_rows
    for total in (0, 1, 7, 8, 131072, 131073):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_rows(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
