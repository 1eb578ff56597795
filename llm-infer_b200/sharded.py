"""Long-context decode with the KV sequence sharded across the GPUs of one box.

Softmax attention over a set of KV rows is a commutative, associative reduction
under the engine's online-softmax state merge (src/attention.cu:41-65), so the
rows of one sequence can live on different GPUs: rank r of N keeps rows
[r*T/N, (r+1)*T/N) of every kv head in its own HBM, in the engine's unchanged
[row][kv_head][head_dim] layout, and Q is replicated. Per step each rank

  1. runs the same split-KV decode kernel over its rows  -> (O_r [H][D], LSE_r [H]),
  2. all-gathers one packed fp32 record [H*D | H] per rank (NCCL over NVLink),
  3. merges the N records with the same LSE merge kernel   -> O [H][D] on every rank.

One process per GPU; ``torch.distributed`` carries the collective. The compute
functions are injectable so the host logic (partitioning, record packing,
gather, merge order) can be exercised with CPU ranks over gloo.
"""
from __future__ import annotations

import time

import torch
import torch.distributed as dist


class GatherTimeout(RuntimeError):
    """The all-gather of a sharded decode did not complete before its deadline (a rank never joined)."""


def shard_rows(total_rows: int, world: int, rank: int) -> tuple[int, int]:
    """Row range [begin, end) of ``rank``: even split, the last rank takes the remainder."""
    per = total_rows // world
    begin = rank * per
    end = total_rows if rank == world - 1 else begin + per
    return begin, end


class ShardedDecode:
    """Decode attention for one sequence whose KV rows are spread over the ranks of ``group``."""

    def __init__(self, n_heads: int, head_dim: int, *, device, group=None, decode_fn=None, merge_fn=None,
                 watchdog_s: float | None = None):
        """``watchdog_s``: host-side deadline for the all-gather. The collective is then issued asynchronously and
        polled from the host; if it has not completed when the deadline passes (a rank died or never reached the
        step), ``gather()`` raises GatherTimeout instead of blocking for ever, after ``on_timeout`` (if set) has
        run - the place to abort the communicator (ncclCommAbort through the process group) or to mark the rank
        as failed. Nothing is waited for on the device and no GPU wait is left spinning: the decision is made on the
        host. Not for use inside a CUDA-graph capture (the poll needs the host)."""
        self.watchdog_s = watchdog_s
        self.on_timeout = None
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.H, self.D = n_heads, head_dim
        n = n_heads * head_dim + n_heads
        self.rec_len = (n + 3) // 4 * 4  # the merge kernel reads partials with 16-byte loads
        self.record = torch.zeros(self.rec_len, dtype=torch.float32, device=device)
        self.gathered = torch.zeros(self.world, self.rec_len, dtype=torch.float32, device=device)
        if decode_fn is None or merge_fn is None:
            from . import attention  # needs the CUDA library; raises if it is missing
            decode_fn = decode_fn or attention.attn_decode
            merge_fn = merge_fn or attention.attn_merge
        self._decode, self._merge = decode_fn, merge_fn
        self._workspace = None

    # views into the packed record / gather buffer
    def _o(self, buf):
        return buf[..., : self.H * self.D]

    def _lse(self, buf):
        return buf[..., self.H * self.D: self.H * self.D + self.H]

    def local_partial(self, q, k_shard, v_shard, kv_len_local=None):
        """Step 1: this rank's (O, LSE) written straight into the record that will be gathered."""
        o = self._o(self.record).view(1, self.H, self.D)
        lse = self._lse(self.record).view(1, self.H)
        kw = {}
        if self._workspace is not None:
            kw["workspace"] = self._workspace
        self._decode(q, k_shard, v_shard, kv_len_local, out=o, lse=lse, **kw)
        return o, lse

    def gather(self):
        """Step 2: one all-gather of rec_len floats per rank, on the current stream (with a watchdog: polled from the
        host against the deadline)."""
        if self.watchdog_s is None:
            dist.all_gather_into_tensor(self.gathered.view(-1), self.record, group=self.group)
            return self.gathered
        work = dist.all_gather_into_tensor(self.gathered.view(-1), self.record, group=self.group, async_op=True)
        deadline = time.monotonic() + self.watchdog_s
        while True:
            try:
                if work.is_completed():
                    break
                failure = None
            except RuntimeError as e:  # the backend noticed a dead peer before the deadline did
                failure = e
            if failure is not None or time.monotonic() > deadline:
                if self.on_timeout is not None:
                    self.on_timeout()
                why = f"failed: {failure}" if failure is not None else f"did not complete within {self.watchdog_s} s"
                raise GatherTimeout(f"rank {self.rank}: all-gather of the partial (O, LSE) records {why}") from failure
            time.sleep(0.0005)
        work.wait()  # orders the current stream after the collective; returns at once
        return self.gathered

    def merge(self, out=None, out_dtype=torch.float32):
        """Step 3: LSE merge of the N gathered records."""
        part_o = self._o(self.gathered).unflatten(-1, (self.H, self.D))  # [N, H, D], partial stride rec_len
        part_lse = self._lse(self.gathered)  # [N, H]
        return self._merge(part_o, part_lse, out=out, out_dtype=out_dtype)

    def __call__(self, q, k_shard, v_shard, kv_len_local=None, out=None, out_dtype=torch.float32):
        """q [1,H,D] (replicated); k_shard, v_shard [1,T_local,Hkv,D] (this rank's rows) -> out [H,D]."""
        self.local_partial(q, k_shard, v_shard, kv_len_local)
        self.gather()
        return self.merge(out=out, out_dtype=out_dtype)

    def use_workspace(self, workspace) -> None:
        self._workspace = workspace

    def capture(self, q, k_shard, v_shard, out, kv_len_local=None):
        """Record one step (local decode, all-gather, merge) into a CUDA graph and return it.

        A decode step is three small launches and one small collective, so at long-context shard sizes the host's
        launch cost is comparable to the GPU time; replaying a captured graph removes it, which is also how the
        engine drives its decode step (include/model/device.hpp:161-262). The tensors passed here are the ones the
        graph will read and write on every ``replay()``; run at least one eager step first so that NCCL and the
        kernels have done their lazy set-up outside the capture.
        """
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self(q, k_shard, v_shard, kv_len_local, out=out)
        return graph


class FusedShardedDecode:
    """The same sharded decode with the collective carried by the merge kernel itself instead of NCCL.

    Every rank owns an exchange buffer in symmetric (peer-mapped) memory. The merge pass of ``attn_decode_sharded``
    stores each merged cell (a row's 32-float slice and its LSE) straight into all ranks' buffers over NVLink as 64-bit
    words that carry the step number, waits (bounded) until the other ranks' words of that cell show the step and
    finishes the cell: two launches per step, no separate collective and no third kernel. ``torch.distributed`` is
    only used to allocate and exchange the buffer handles. ``kv_early``: the caller vouches that between steps only
    each sequence's newest row is written (by the kernel in front of the step), so the local pass may start streaming
    the older rows before that kernel has finished.
    """

    def __init__(self, batch: int, n_heads: int, n_kv_heads: int, head_dim: int, *, device, group=None,
                 kv_early: bool = False):
        self.kv_early = bool(kv_early)
        import torch.distributed._symmetric_memory as symm_mem

        from . import attention
        self._attention = attention
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        nbytes = attention.exchange_bytes(batch, n_heads, head_dim, self.world)
        self.buffer = symm_mem.empty((nbytes + 3) // 4, dtype=torch.float32, device=device)
        self.buffer.zero_()
        self.handle = symm_mem.rendezvous(self.buffer, self.group)
        self.peer_buffers = [int(p) for p in self.handle.buffer_ptrs]
        self.workspace = attention.DecodeWorkspace(batch, n_heads, n_kv_heads, head_dim, device)
        torch.cuda.synchronize(device)
        dist.barrier(self.group)  # every buffer is zero before anybody's first step

    def __call__(self, q, k_shard, v_shard, kv_len_local=None, out=None, lse=None, out_dtype=torch.float32):
        """q [B,H,D] (replicated); k_shard, v_shard [B,T_local,Hkv,D] (this rank's rows) -> out [B,H,D]."""
        return self._attention.attn_decode_sharded(
            q, k_shard, v_shard, kv_len_local, peer_buffers=self.peer_buffers, world_size=self.world, rank=self.rank,
            step=0, out=out, lse=lse, out_dtype=out_dtype, workspace=self.workspace, kv_early=self.kv_early)

    def capture(self, q, k_shard, v_shard, out, kv_len_local=None):
        """One step as a CUDA graph (the kernel counts steps on the device, so the arguments never change)."""
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self(q, k_shard, v_shard, kv_len_local, out=out)
        return graph
