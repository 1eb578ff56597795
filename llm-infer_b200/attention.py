"""Host-side mirror of the engine's attention interface, over the C ABI.

The engine calls ``attn(out, scores, q, k_cache, v_cache, group, head_dim,
n_kv_heads, kv_len)`` once per query head (include/kernels_cpu.hpp:140-167,
src/model/block.cpp:157-164). The functions here take the same operands — fp32 /
fp16 / bf16 ``q``, 16-bit K/V caches laid out ``[row][kv_head][head_dim]``,
``kv_len`` valid rows — for a whole batch and all heads at once, and run them on
the GPU through ``libllm_infer_attn.so``. PyTorch is used only to hold device
memory and streams; no computation falls back to it.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import binding as _b

_DTYPES = {torch.float32: _b.DTYPE_F32, torch.float16: _b.DTYPE_F16, torch.bfloat16: _b.DTYPE_BF16,
           # int32 tensors stand for prepared activations (ATTN_DTYPE_SPLIT16: one 32-bit word per element)
           torch.int32: 3}


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}") from None


def _stream_ptr(stream) -> int:
    s = torch.cuda.current_stream() if stream is None else stream
    return s.cuda_stream


def _dense(t: torch.Tensor, stream, what: str) -> torch.Tensor:
    """``t`` itself when it is contiguous. Otherwise a contiguous copy, made on the current stream; with an explicit
    ``stream`` that copy would not be ordered with the kernel that reads it (and its memory could be reused before the
    kernel ran), so a non-contiguous operand is refused there."""
    if t.is_contiguous():
        return t
    if stream is not None:
        raise ValueError(f"{what} must be contiguous when an explicit stream is given")
    return t.contiguous()


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("attention operands must be CUDA tensors (there is no CPU path)")


class DecodeWorkspace:
    """Scratch for the split-KV pass (per-CTA partial O and LSE), reusable across calls of one shape."""

    def __init__(self, batch: int, n_heads: int, n_kv_heads: int, head_dim: int, device=None):
        lib = _b.load()
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        with torch.cuda.device(device):
            nbytes = lib.attn_decode_workspace_bytes(batch, n_heads, n_kv_heads, head_dim)
        if nbytes == 0:
            raise _b.AttnError(-2, f"no decode kernel for batch={batch} heads={n_heads}/{n_kv_heads} dim={head_dim}")
        self.key = (batch, n_heads, n_kv_heads, head_dim, device.index)
        self.nbytes = int(nbytes)
        self.buf = torch.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)


def _decode_args(q, k_cache, v_cache, kv_len, out, lse, out_dtype, scale, workspace, max_ctas, stream=None,
                 kv_early=False):
    """Validates the operands of a decode call and fills the C struct. Returns (args, out, workspace)."""
    _require_cuda(q, k_cache, v_cache)
    B, H, D = q.shape
    Bk, T, Hkv, Dk = k_cache.shape
    if (Bk, Dk) != (B, D) or v_cache.shape != k_cache.shape:
        raise ValueError("shape mismatch between q and the caches")
    if k_cache.dtype != v_cache.dtype or k_cache.stride() != v_cache.stride():
        raise ValueError("K and V caches must share dtype and strides")
    if k_cache.stride(3) != 1 or k_cache.stride(2) != D:
        raise ValueError("cache layout must be [row][kv_head][head_dim] with dense heads")
    q = _dense(q, stream, "q")
    if out is None:
        out = torch.empty((B, H, D), dtype=out_dtype, device=q.device)
    elif out.shape != (B, H, D) or not out.is_contiguous():
        raise ValueError("out must be a contiguous [B, H, D] tensor")
    if workspace is None or workspace.key != (B, H, Hkv, D, q.device.index):
        workspace = DecodeWorkspace(B, H, Hkv, D, q.device)

    a = _b.AttnDecodeArgs()
    a.o, a.q, a.k, a.v = out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr()
    a.lse = lse.data_ptr() if lse is not None else None
    a.o_dtype, a.q_dtype, a.kv_dtype = _dtype_code(out), _dtype_code(q), _dtype_code(k_cache)
    a.batch, a.n_heads, a.n_kv_heads, a.head_dim = B, H, Hkv, D
    if kv_len is None:
        a.kv_len, a.kv_len_uniform = None, T
    elif isinstance(kv_len, int):
        if kv_len > T:
            raise ValueError("kv_len exceeds the cache")
        a.kv_len, a.kv_len_uniform = None, kv_len
    else:
        if kv_len.dtype not in (torch.int32, torch.uint32) or kv_len.shape != (B,) or not kv_len.is_cuda:
            raise ValueError("kv_len must be an int32 CUDA tensor of shape [B]")
        a.kv_len, a.kv_len_uniform = kv_len.data_ptr(), 0
    a.kv_row_stride = k_cache.stride(1)
    a.kv_batch_stride = k_cache.stride(0) if B > 1 else max(k_cache.stride(0), 0)
    a.scale = float(scale)
    a.max_ctas = int(max_ctas)
    a.workspace, a.workspace_bytes = workspace.buf.data_ptr(), workspace.nbytes
    a.status = workspace.status.data_ptr()
    a.kv_early = int(bool(kv_early))
    a.kv_capacity = T  # a device-side length beyond the cache is clamped and reported (ATTN_STATUS_BAD_SHAPE)
    return a, out, workspace, q


def attn_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, kv_len=None, *, out=None, lse=None,
                out_dtype=torch.float32, scale: float = 0.0, workspace: DecodeWorkspace | None = None,
                max_ctas: int = 0, kv_early: bool = False, stream=None) -> torch.Tensor:
    """Single-token attention of every query head over its sequence's KV cache.

    q        [B, H, D]        fp32 / fp16 / bf16, already rotated
    k_cache  [B, T, Hkv, D]   fp16 / bf16; only the last dim must be dense, rows and sequences may be strided
    v_cache  same geometry as k_cache
    kv_len   None (all T rows valid), an int, or an int32/uint32 CUDA tensor [B]; the values of a tensor are read
             on the device: one beyond T is clamped to T there and sets ATTN_STATUS_BAD_SHAPE in workspace.status
    kv_early True when the lengths were in place before the previous kernel of the stream was launched and that kernel
             writes no K/V row other than each sequence's last valid one: streaming then starts before it has finished
    returns  out [B, H, D] in out_dtype; fills ``lse`` [B, H] (fp32) when given
    """
    a, out, _, _q = _decode_args(q, k_cache, v_cache, kv_len, out, lse, out_dtype, scale, workspace, max_ctas, stream,
                                 kv_early)
    with torch.cuda.device(out.device):
        _b.check(_b.load().attn_decode(C.byref(a), _stream_ptr(stream)), "attn_decode")
    return out


def attn_decode_sharded(q, k_shard, v_shard, kv_len_local=None, *, peer_buffers, world_size: int, rank: int,
                        step: int = 0, poll_limit: int = 0, out=None, lse=None, out_dtype=torch.float32,
                        scale: float = 0.0, workspace: DecodeWorkspace | None = None, kv_early: bool = False,
                        stream=None) -> torch.Tensor:
    """Decode over this rank's KV rows with the cross-GPU exchange fused into the merge pass (C ABI
    ``attn_decode_sharded``). ``peer_buffers`` holds one device pointer per rank (as int) to that rank's exchange
    buffer, valid on this GPU; ``step = 0`` lets the kernel count steps itself; ``kv_early`` as in attn_decode.
    Returns the final out [B, H, D]."""
    a, out, _, _q = _decode_args(q, k_shard, v_shard, kv_len_local, out, lse, out_dtype, scale, workspace, 0, stream,
                                 kv_early)
    s = _b.AttnDecodeShardedArgs()
    s.decode = a
    s.world_size, s.rank, s.step, s.poll_limit = world_size, rank, step, poll_limit
    for r in range(world_size):
        s.peer_buffers[r] = int(peer_buffers[r])
    with torch.cuda.device(out.device):
        _b.check(_b.load().attn_decode_sharded(C.byref(s), _stream_ptr(stream)), "attn_decode_sharded")
    return out


def exchange_bytes(batch: int, n_heads: int, head_dim: int, world_size: int) -> int:
    return int(_b.load().attn_decode_sharded_exchange_bytes(batch, n_heads, head_dim, world_size))


def exchange_record(buffer: torch.Tensor, batch: int, n_heads: int, head_dim: int, world_size: int, parity: int,
                    source_rank: int):
    """Decodes one record of an exchange buffer (what ``source_rank`` delivered for the step of that parity):
    returns (o [batch*n_heads, head_dim] fp32, lse [batch*n_heads] fp32, steps [cells, c+1] int64 = the step tag of
    every word). For tests and debugging; the layout is described at attn_decode_sharded in the header."""
    c = int(_b.load().attn_decode_sharded_cell_floats(batch, n_heads, head_dim))
    rows, nsl = batch * n_heads, head_dim // c
    rank_words = rows * nsl * (c + 1)
    words = buffer.view(torch.int64)[(parity * world_size + source_rank) * rank_words:][:rank_words].view(rows, nsl, c + 1)
    vals = words.contiguous().view(torch.float32).view(rows, nsl, c + 1, 2)[..., 0]  # low half of each word
    return vals[..., :c].reshape(rows, head_dim), vals[:, 0, c].contiguous(), (words >> 32).view(rows * nsl, c + 1)


def attn_prefill_causal(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, out=None, out_dtype=None,
                        scale: float = 0.0, p_mode: int = _b.PREFILL_P_RESIDUAL, status=None,
                        stream=None) -> torch.Tensor:
    """Causal attention of whole prompts: row t attends rows 0..t (the engine's token-at-a-time prefill,
    tools/infer.cpp:271-274, as one kernel).

    q [B, S, H, D], k / v [B, S, Hkv, D], fp16 or bf16, dense; D = 128 or 64. Returns out [B, S, H, D] in ``out_dtype``
    (fp32 or the input dtype; default the input dtype). ``p_mode`` (binding.PREFILL_P_*) selects how the
    probabilities enter the tensor cores: with a residual term (second MMA; the default and the parity mode) or
    rounded once to the input type.
    """
    _require_cuda(q, k, v)
    lib = _b.load()
    B, S, H, D = q.shape
    Hkv = k.shape[2]
    if k.shape != (B, S, Hkv, D) or v.shape != k.shape or not (q.dtype == k.dtype == v.dtype):
        raise ValueError("q, k, v must share batch, length, head_dim and dtype")
    q, k, v = _dense(q, stream, "q"), _dense(k, stream, "k"), _dense(v, stream, "v")
    if out is None:
        out = torch.empty((B, S, H, D), dtype=out_dtype or q.dtype, device=q.device)
    elif out.shape != (B, S, H, D) or not out.is_contiguous():
        raise ValueError("out must be a contiguous [B, S, H, D] tensor")
    a = _b.AttnPrefillArgs()
    a.o, a.q, a.k, a.v = out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.o_dtype, a.dtype = _dtype_code(out), _dtype_code(q)
    a.batch, a.seq_len, a.n_heads, a.n_kv_heads, a.head_dim = B, S, H, Hkv, D
    a.scale, a.p_mode = float(scale), int(p_mode)
    a.status = status.data_ptr() if status is not None else None
    with torch.cuda.device(q.device):
        _b.check(lib.attn_prefill_causal(C.byref(a), _stream_ptr(stream)), "attn_prefill_causal")
    return out


def rope_kv_insert(q, k, v, k_cache, v_cache, pos, kv_pos, *, theta: float, rotary_dim: int = 0, kv_sink: int = 0,
                   inv_freq=None, q_out=None, q_out_dtype=torch.float32, pos_early: bool = False,
                   stream=None) -> torch.Tensor:
    """Rotate the current token's q and k, insert k and v (fp16) into the caches, re-rotate the sink rows.

    q [B,H,D], k / v [B,Hkv,D] fp32; k_cache / v_cache fp16 [B,T,Hkv,D]; pos, kv_pos int32 CUDA tensors [B].
    Returns the rotated q (``q_out``, fp32 / fp16 / bf16). Mirrors src/model/block.cpp:140-155 for a batch.
    """
    _require_cuda(q, k, v, k_cache, v_cache, pos, kv_pos)
    B, H, D = q.shape
    Hkv = k.shape[1]
    if k.shape != (B, Hkv, D) or v.shape != k.shape or k_cache.shape[0] != B or k_cache.shape[2:] != (Hkv, D):
        raise ValueError("shape mismatch")
    if q.dtype != torch.float32 or k.dtype != torch.float32 or v.dtype != torch.float32 or k_cache.dtype != torch.float16:
        raise TypeError("q, k, v must be fp32 and the caches fp16")
    q, k, v = _dense(q, stream, "q"), _dense(k, stream, "k"), _dense(v, stream, "v")
    if q_out is None:
        q_out = torch.empty((B, H, D), dtype=q_out_dtype, device=q.device)
    a = _b.AttnRopeInsertArgs()
    a.q_out, a.q, a.k, a.v = q_out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.k_cache, a.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
    a.inv_freq = inv_freq.data_ptr() if inv_freq is not None else None
    a.pos, a.kv_pos = pos.data_ptr(), kv_pos.data_ptr()
    a.kv_row_stride = k_cache.stride(1)
    a.kv_batch_stride = k_cache.stride(0) if B > 1 else max(k_cache.stride(0), 0)
    a.batch, a.n_heads, a.n_kv_heads, a.head_dim = B, H, Hkv, D
    a.rotary_dim, a.kv_sink, a.theta = rotary_dim, kv_sink, float(theta)
    a.q_out_dtype = _dtype_code(q_out)
    a.pos_early = int(pos_early)  # pos was written before the previous kernel of the stream was launched
    with torch.cuda.device(q.device):
        _b.check(_b.load().attn_rope_kv_insert(C.byref(a), _stream_ptr(stream)), "attn_rope_kv_insert")
    return q_out


class HostDecodeStep:
    """One decode step of the attention block driven from host buffers, as ONE CUDA-graph launch: the token's fp32
    q, k, v are copied from pinned host memory (one copy), ``attn_rope_kv_insert`` rotates q and k and appends k, v to
    the resident fp16 caches, ``attn_decode`` attends over them, and the output is copied back to pinned host memory.
    The engine drives its CUDA step the same way (a captured graph per step, include/model/device.hpp:161-262).
    Calling the object replays the graph and waits for the result.

    host_in   pinned fp32 [B*H*D + 2*B*Hkv*D]: q, then k, then v of the current token
    k_cache, v_cache  fp16 [B, T, Hkv, D] on the device; pos, kv_pos int32 [B] on the device
    out_host  pinned fp32 [B, H, D]
    kv_early  True when every kv_pos[b] is the sequence's last valid row (the token is appended, no sliding window):
              attention then starts streaming the older rows while the insert kernel still runs
    """

    def __init__(self, host_in, k_cache, v_cache, pos, kv_pos, out_host, *, n_heads: int, theta: float,
                 rotary_dim: int = 0, kv_len=None, workspace: DecodeWorkspace | None = None, kv_early: bool = False):
        if not (host_in.is_pinned() and out_host.is_pinned()):
            raise ValueError("host_in and out_host must be pinned host tensors")
        B, T, Hkv, D = k_cache.shape
        H = n_heads
        n_q, n_kv = B * H * D, B * Hkv * D
        if host_in.numel() != n_q + 2 * n_kv or host_in.dtype != torch.float32 or out_host.shape != (B, H, D):
            raise ValueError("host_in must hold q, k, v of one token per sequence (fp32) and out_host be [B, H, D]")
        dev = k_cache.device
        self.host_in, self.out_host = host_in, out_host
        self._dev_in = torch.empty(n_q + 2 * n_kv, dtype=torch.float32, device=dev)
        q32 = self._dev_in[:n_q].view(B, H, D)
        k32 = self._dev_in[n_q:n_q + n_kv].view(B, Hkv, D)
        v32 = self._dev_in[n_q + n_kv:].view(B, Hkv, D)
        self._q_rot = torch.empty((B, H, D), dtype=torch.float16, device=dev)
        self._out = torch.empty((B, H, D), dtype=torch.float32, device=dev)
        self.workspace = workspace if workspace is not None else DecodeWorkspace(B, H, Hkv, D, dev)

        def launches():
            self._dev_in.copy_(host_in, non_blocking=True)
            rope_kv_insert(q32, k32, v32, k_cache, v_cache, pos, kv_pos, theta=theta, rotary_dim=rotary_dim,
                           q_out=self._q_rot)
            attn_decode(self._q_rot, k_cache, v_cache, kv_len, out=self._out, workspace=self.workspace,
                        kv_early=kv_early)
            out_host.copy_(self._out, non_blocking=True)

        with torch.cuda.device(dev):
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                launches()  # lazy set-up of every kernel happens outside the capture
            torch.cuda.current_stream(dev).wait_stream(side)
            torch.cuda.synchronize(dev)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                launches()
        self._device = dev

    def __call__(self) -> torch.Tensor:
        self.graph.replay()
        torch.cuda.current_stream(self._device).synchronize()  # the caller reads out_host before the next token
        return self.out_host


def _gemv(entry: str, x, w, n: int, out, out2, out3, out_dtype, clip, accumulate, swiglu, k_split, status, stream,
          rows=None):
    """Common part of gemv_f16 / gemv_q8_0: output shapes, the argument structure, the call."""
    B = x.shape[0]
    rows = w.shape[0] if rows is None else rows
    if swiglu and (rows % 2 or out2 is not None or out3 is not None):
        raise ValueError("swiglu needs an even number of rows (gate rows, then up rows) and a single output")
    if out3 is not None and out2 is None:
        raise ValueError("out3 without out2")
    x, w = _dense(x, stream, "x"), _dense(w, stream, "w")
    d = rows // 2 if swiglu else rows
    segs = [t for t in (out2, out3) if t is not None]
    d0 = d - sum(t.shape[1] for t in segs)
    if k_split > 1:
        if out is None:
            out = torch.empty((k_split, B, d0), dtype=torch.float32, device=x.device)
        if out.shape != (k_split, B, d0) or not out.is_contiguous() or segs:
            raise ValueError("with k_split the output is a dense [k_split, B, rows] fp32 tensor")
        first = out[0]
    else:
        if out is None:
            out = torch.empty((B, d0), dtype=out_dtype, device=x.device)
        first = out
    for t in [first] + segs:
        if t.shape[0] != B or t.stride(1) != 1 or t.dtype != out.dtype:
            raise ValueError("outputs must be [B, rows] with dense rows and one dtype")
    if first.shape[1] != d0 or d0 <= 0:
        raise ValueError("output widths do not add up to the rows of w")
    a = _b.AttnGemvArgs()
    a.out, a.x, a.w = out.data_ptr(), x.data_ptr(), w.data_ptr()
    a.out_batch_stride = first.stride(0) if B > 1 else d0
    a.n, a.d, a.batch, a.clip, a.out_dtype = n, d, B, float(clip), _dtype_code(out)
    a.accumulate = int(accumulate)
    a.swiglu = int(swiglu)
    a.k_split = int(k_split)
    a.x_format = _dtype_code(x)  # fp32, or int32 = prepared activations
    a.status = status.data_ptr() if status is not None else None
    if out2 is not None:
        a.out2, a.split1 = out2.data_ptr(), d0
        a.out2_batch_stride = out2.stride(0) if B > 1 else out2.shape[1]
    if out3 is not None:
        a.out3, a.split2 = out3.data_ptr(), d0 + out2.shape[1]
        a.out3_batch_stride = out3.stride(0) if B > 1 else out3.shape[1]
    with torch.cuda.device(x.device):
        _b.check(getattr(_b.load(), entry)(C.byref(a), _stream_ptr(stream)), entry)
    return out


def gemv_f16(x: torch.Tensor, w: torch.Tensor, *, out=None, out2=None, out3=None, out_dtype=torch.float32,
             clip: float = 0.0, accumulate: bool = False, swiglu: bool = False, k_split: int = 1,
             stream=None) -> torch.Tensor:
    """out[b] = clamp(W x[b]): x [B, n] fp32, w [rows, n] fp16 (n fastest) -> out [B, rows] fp32 or fp16 (may be a
    strided view, e.g. a KV-cache row per sequence). Mirrors matmul() of include/kernels_cpu.hpp:69-80 for a batch;
    ``accumulate`` adds into out (residual connection). Fused forms (they and any batch > 1 run on the tensor cores):
    * ``out2`` / ``out3``: the rows are split over out, out2, out3 in that order (stacked Q, K, V projections);
    * ``swiglu``: w holds d gate rows then d up rows, out [B, d] = silu(gate x) * (up x);
    * ``k_split`` > 1: out is [k_split, B, rows], the partial products of k_split equal slices of the inner
      dimension (their sum is the result; ``rmsnorm(..., partials=out)`` adds them into the residual stream)."""
    _require_cuda(x, w)
    B, n = x.shape
    if w.dim() != 2 or w.shape[1] != n or w.dtype != torch.float16 or x.dtype != torch.float32:
        raise ValueError("x must be fp32 [B, n] and w fp16 [rows, n]")
    return _gemv("attn_gemv_f16", x, w, n, out, out2, out3, out_dtype, clip, accumulate, swiglu, k_split, None, stream)


def gemv_q8_0(x: torch.Tensor, w: torch.Tensor, *, out=None, out2=None, out3=None, out_dtype=torch.float32,
              clip: float = 0.0, accumulate: bool = False, swiglu: bool = False, k_split: int = 1, status=None,
              stream=None, rows=None) -> torch.Tensor:
    """The same over Q8_0 weights: w uint8 [rows, n/32*34] (GGML blocks: fp16 scale + 32 signed bytes). Same
    conventions and fused forms as gemv_f16. x and out may also be int32 tensors, which stand for prepared activations
    (one word per element: fp16 value and fp16 residual, written by rmsnorm(out=int32), attn_decode(out=int32) or
    this function itself): the kernel then copies x into shared memory as it is instead of converting it in every CTA.
    w may also be the tiled copy made by repack_q8_0 (uint8 [ceil(rows/16), n/32, 544]): same result, bit for bit,
    from a layout the kernel streams and unpacks faster; ``rows`` then gives the row count when it is not a multiple
    of 16."""
    _require_cuda(x, w)
    B, n = x.shape
    if x.dtype not in (torch.float32, torch.int32) or w.dtype != torch.uint8 or n % 32:
        raise ValueError("x must be fp32 (or int32 = prepared activations) [B, n] and w uint8")
    if w.dim() == 3:
        if w.shape[1] != n // 32 or w.shape[2] != Q8_TILE_BLOCK_BYTES:
            raise ValueError("a tiled Q8_0 matrix is uint8 [ceil(rows/16), n/32, 544]")
        rows = w.shape[0] * 16 if rows is None else rows
        if not 0 < rows <= w.shape[0] * 16:
            raise ValueError("rows does not fit the tiled matrix")
        return _gemv("attn_gemv_q8_0_tiled", x, w, n, out, out2, out3, out_dtype, clip, accumulate, swiglu, k_split,
                     status, stream, rows=rows)
    if w.dim() != 2 or w.shape[1] != n // 32 * 34:
        raise ValueError("w must be uint8 [rows, n/32*34]")
    return _gemv("attn_gemv_q8_0", x, w, n, out, out2, out3, out_dtype, clip, accumulate, swiglu, k_split, status, stream)


Q8_TILE_BLOCK_BYTES = 16 * 34  # one 32-element block of 16 rows in the tiled layout


def repack_q8_0(w: torch.Tensor, *, stream=None) -> torch.Tensor:
    """GGML Q8_0 blocks uint8 [rows, n/32*34] -> the tiled copy uint8 [ceil(rows/16), n/32, 544] that gemv_q8_0 also
    accepts (attn_repack_q8_0_tiled; one launch, meant to run once per matrix when a model is loaded)."""
    _require_cuda(w)
    if w.dim() != 2 or w.dtype != torch.uint8 or w.shape[1] % 34:
        raise ValueError("w must be uint8 [rows, n/32*34]")
    w = _dense(w, stream, "w")
    rows, n = w.shape[0], w.shape[1] // 34 * 32
    out = torch.empty(((rows + 15) // 16, n // 32, Q8_TILE_BLOCK_BYTES), dtype=torch.uint8, device=w.device)
    lib = _b.load()
    if lib.attn_q8_0_tiled_bytes(rows, n) != out.numel():
        raise RuntimeError("tiled size mismatch")
    with torch.cuda.device(w.device):
        _b.check(lib.attn_repack_q8_0_tiled(out.data_ptr(), w.data_ptr(), rows, n, _stream_ptr(stream)),
                 "attn_repack_q8_0_tiled")
    return out


def embed_f16(table: torch.Tensor, tokens: torch.Tensor, *, out=None, status=None, stream=None) -> torch.Tensor:
    """x[b] = fp32(table[tokens[b]]): fp16 table [vocab, dim], uint32/int32 tokens [B] (src/model/model.cpp:101-118)."""
    _require_cuda(table, tokens)
    vocab, dim = table.shape
    if table.dtype != torch.float16 or tokens.dtype not in (torch.int32, torch.uint32) or not table.is_contiguous():
        raise ValueError("table must be dense fp16 [vocab, dim] and tokens 32-bit integers")
    B = tokens.numel()
    if out is None:
        out = torch.empty((B, dim), dtype=torch.float32, device=table.device)
    with torch.cuda.device(table.device):
        _b.check(_b.load().attn_embed_f16(out.data_ptr(), table.data_ptr(), tokens.data_ptr(), B, dim, vocab,
                                          status.data_ptr() if status is not None else None, _stream_ptr(stream)),
                 "attn_embed_f16")
    return out


def embed_q8_0(table: torch.Tensor, tokens: torch.Tensor, *, out=None, status=None, stream=None) -> torch.Tensor:
    """x[b] = dequantised row tokens[b] of a Q8_0 table: uint8 [vocab, dim/32*34] -> fp32 [B, dim]."""
    _require_cuda(table, tokens)
    vocab = table.shape[0]
    dim = table.shape[1] // 34 * 32
    if table.dtype != torch.uint8 or table.shape[1] % 34 or not table.is_contiguous() or \
            tokens.dtype not in (torch.int32, torch.uint32):
        raise ValueError("table must be dense uint8 [vocab, dim/32*34] and tokens 32-bit integers")
    B = tokens.numel()
    if out is None:
        out = torch.empty((B, dim), dtype=torch.float32, device=table.device)
    with torch.cuda.device(table.device):
        _b.check(_b.load().attn_embed_q8_0(out.data_ptr(), table.data_ptr(), tokens.data_ptr(), B, dim, vocab,
                                           status.data_ptr() if status is not None else None, _stream_ptr(stream)),
                 "attn_embed_q8_0")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, *, out=None, partials=None, stream=None) -> torch.Tensor:
    """out[b] = x[b] / sqrt(mean(x[b]^2) + eps) * weight, fp32 (include/kernels_cpu.hpp:43-67); out may be x, or an
    int32 tensor [B, dim] to receive the result as prepared activations for gemv_q8_0.
    With ``partials`` [k, B, dim] (fp32, dense) the row is first completed, x += partials[0] + partials[1] + ...
    (written back to x), then normalised into ``out`` (which must then be another tensor)."""
    _require_cuda(x, weight)
    B, dim = x.shape
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or weight.numel() != dim or not x.is_contiguous():
        raise ValueError("x must be dense fp32 [B, dim] and weight fp32 [dim]")
    if out is None:
        out = torch.empty_like(x)
    n_part, stride, pptr = 0, 0, None
    if partials is not None:
        if partials.dtype != torch.float32 or partials.shape[1:] != (B, dim) or not partials.is_contiguous():
            raise ValueError("partials must be dense fp32 [k, B, dim]")
        n_part, stride, pptr = partials.shape[0], B * dim, partials.data_ptr()
    fn = _b.load().attn_rmsnorm_residual_split if out.dtype == torch.int32 else _b.load().attn_rmsnorm_residual
    with torch.cuda.device(x.device):
        _b.check(fn(out.data_ptr(), x.data_ptr(), pptr, n_part, stride, weight.data_ptr(), B, dim, float(eps),
                    _stream_ptr(stream)), "attn_rmsnorm")
    return out


def swiglu_(hb: torch.Tensor, hb2: torch.Tensor, *, stream=None) -> torch.Tensor:
    """hb = silu(hb) * hb2 in place (src/model/block.cpp:206-210)."""
    _require_cuda(hb, hb2)
    if hb.dtype != torch.float32 or hb2.dtype != torch.float32 or hb.shape != hb2.shape or \
            not (hb.is_contiguous() and hb2.is_contiguous()):
        raise ValueError("hb and hb2 must be dense fp32 tensors of one shape")
    with torch.cuda.device(hb.device):
        _b.check(_b.load().attn_swiglu(hb.data_ptr(), hb2.data_ptr(), hb.numel(), _stream_ptr(stream)), "attn_swiglu")
    return hb


def argmax(logits: torch.Tensor, *, out=None, stream=None) -> torch.Tensor:
    """First index of the maximum of each row of fp32 logits [B, vocab] (tools/infer.cpp:64-74) -> int32 [B]."""
    _require_cuda(logits)
    B, vocab = logits.shape
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise ValueError("logits must be dense fp32 [B, vocab]")
    if out is None:
        out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    with torch.cuda.device(logits.device):
        _b.check(_b.load().attn_argmax(out.data_ptr(), logits.data_ptr(), B, vocab, _stream_ptr(stream)), "attn_argmax")
    return out


def attn_merge(part_o: torch.Tensor, part_lse: torch.Tensor, *, out=None, lse=None, out_dtype=torch.float32,
               stream=None) -> torch.Tensor:
    """Online-softmax merge of partial results (src/attention.cu:41-65 in log-sum-exp form).

    part_o   [n, rows, D] fp32 (partials may be strided in dim 0), part_lse [n, rows] fp32
    returns  out [rows, D]
    """
    _require_cuda(part_o, part_lse)
    lib = _b.load()
    n, rows, D = part_o.shape
    if part_lse.shape != (n, rows) or part_o.dtype != torch.float32 or part_lse.dtype != torch.float32:
        raise ValueError("part_o must be fp32 [n, rows, D] and part_lse fp32 [n, rows]")
    if part_o.stride(2) != 1 or part_o.stride(1) != D or part_lse.stride(1) != 1:
        raise ValueError("rows of a partial must be dense")
    if out is None:
        out = torch.empty((rows, D), dtype=out_dtype, device=part_o.device)
    a = _b.AttnMergeArgs()
    a.o = out.data_ptr()
    a.lse = lse.data_ptr() if lse is not None else None
    a.part_o, a.part_lse = part_o.data_ptr(), part_lse.data_ptr()
    a.o_part_stride = part_o.stride(0) if n > 1 else rows * D
    a.lse_part_stride = part_lse.stride(0) if n > 1 else rows
    a.n_parts, a.rows, a.head_dim, a.o_dtype = n, rows, D, _dtype_code(out)
    with torch.cuda.device(part_o.device):
        _b.check(lib.attn_merge(C.byref(a), _stream_ptr(stream)), "attn_merge")
    return out


# ---- whole prompts at once: the projection GEMM and the row-wise steps around it (rows = tokens of all prompts) ----
def _pair_like(x: torch.Tensor, shape=None):
    shape = tuple(x.shape) if shape is None else tuple(shape)
    return (torch.empty(shape, dtype=torch.float16, device=x.device), torch.empty(shape, dtype=torch.float16, device=x.device))


def gemm_f16(a_hi: torch.Tensor, a_lo, w: torch.Tensor, *, out: torch.Tensor, accumulate: bool = False, status=None,
             stream=None) -> torch.Tensor:
    """out[t] (+)= W (a_hi[t] + a_lo[t]) for all t at once on the tensor cores: a_hi, a_lo fp16 [m, k] (a_lo may be
    None), w fp16 [n_out, k], out fp32 [m, n_out] (rows may be strided). The batched form of matmul()
    (include/kernels_cpu.hpp:69-80) for the tokens of whole prompts."""
    _require_cuda(a_hi, w, out)
    m, k = a_hi.shape
    n_out = w.shape[0]
    if w.shape != (n_out, k) or a_hi.dtype != torch.float16 or w.dtype != torch.float16 or out.dtype != torch.float32 or \
            out.shape != (m, n_out) or out.stride(1) != 1 or not (a_hi.is_contiguous() and w.is_contiguous()):
        raise ValueError("a_hi fp16 [m, k] and w fp16 [n_out, k] dense, out fp32 [m, n_out] with dense rows")
    if a_lo is not None and (a_lo.shape != a_hi.shape or a_lo.dtype != torch.float16 or not a_lo.is_contiguous()):
        raise ValueError("a_lo must match a_hi")
    a = _b.AttnGemmArgs()
    a.c, a.a_hi, a.w = out.data_ptr(), a_hi.data_ptr(), w.data_ptr()
    a.a_lo = a_lo.data_ptr() if a_lo is not None else None
    a.ldc, a.m, a.n_out, a.k = out.stride(0), m, n_out, k
    a.accumulate = int(bool(accumulate))
    a.status = status.data_ptr() if status is not None else None
    with torch.cuda.device(out.device):
        _b.check(_b.load().attn_gemm_f16(C.byref(a), _stream_ptr(stream)), "attn_gemm_f16")
    return out


def rmsnorm_pair(x: torch.Tensor, weight: torch.Tensor, eps: float, *, out=None, stream=None):
    """RMSNorm of every row of x [rows, dim] fp32, written as the fp16 (value, residual) pair that gemm_f16 reads."""
    _require_cuda(x, weight)
    rows, dim = x.shape
    hi, lo = out if out is not None else _pair_like(x)
    with torch.cuda.device(x.device):
        _b.check(_b.load().attn_rmsnorm_f16pair(hi.data_ptr(), lo.data_ptr(), x.data_ptr(), weight.data_ptr(), rows, dim,
                                                float(eps), _stream_ptr(stream)), "attn_rmsnorm_f16pair")
    return hi, lo


def split_pair(x: torch.Tensor, *, out=None, stream=None):
    """Dense fp32 tensor -> fp16 (value, residual) pair of the same shape."""
    _require_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise ValueError("x must be dense fp32")
    hi, lo = out if out is not None else _pair_like(x)
    with torch.cuda.device(x.device):
        _b.check(_b.load().attn_split_f16pair(hi.data_ptr(), lo.data_ptr(), x.data_ptr(), x.numel(), _stream_ptr(stream)),
                 "attn_split_f16pair")
    return hi, lo


def swiglu_pair(gate_up: torch.Tensor, *, out=None, stream=None):
    """gate_up fp32 [rows, 2 hidden] (gate columns, then up columns) -> silu(gate) * up as the fp16 pair [rows, hidden]."""
    _require_cuda(gate_up)
    rows, two_h = gate_up.shape
    if gate_up.dtype != torch.float32 or gate_up.stride(1) != 1 or two_h % 2:
        raise ValueError("gate_up must be fp32 [rows, 2 hidden] with dense rows")
    hidden = two_h // 2
    hi, lo = out if out is not None else _pair_like(gate_up, (rows, hidden))
    with torch.cuda.device(gate_up.device):
        _b.check(_b.load().attn_swiglu_f16pair(hi.data_ptr(), lo.data_ptr(), gate_up.data_ptr(), rows, hidden,
                                               gate_up.stride(0), _stream_ptr(stream)), "attn_swiglu_f16pair")
    return hi, lo


def dequant_q8_0_pair(w: torch.Tensor, *, out=None, stream=None):
    """Q8_0 rows uint8 [rows, n/32*34] -> fp32(scale) * q as the fp16 (value, residual) pair [rows, n]."""
    _require_cuda(w)
    rows = w.shape[0]
    n = w.shape[1] // 34 * 32
    if w.dtype != torch.uint8 or w.shape[1] % 34 or not w.is_contiguous():
        raise ValueError("w must be dense uint8 [rows, n/32*34]")
    if out is None:
        out = (torch.empty((rows, n), dtype=torch.float16, device=w.device), torch.empty((rows, n), dtype=torch.float16, device=w.device))
    hi, lo = out
    with torch.cuda.device(w.device):
        _b.check(_b.load().attn_dequant_q8_0_f16pair(hi.data_ptr(), lo.data_ptr(), w.data_ptr(), rows, n,
                                                     _stream_ptr(stream)), "attn_dequant_q8_0_f16pair")
    return hi, lo


def rope_prompt(qkv: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                token_seq: torch.Tensor, token_pos: torch.Tensor, *, n_heads: int, theta: float, rotary_dim: int = 0,
                qkv_clip: float = 0.0, inv_freq=None, stream=None) -> torch.Tensor:
    """Rotate q and k of every prompt token and insert k, v (fp16) into the token's cache row: qkv fp32 [tokens,
    (H + 2 Hkv) D] as the stacked projection leaves it, q_out fp16 [tokens, H, D], caches fp16 [B, T, Hkv, D],
    token_seq / token_pos int32 [tokens] on the device. Per token what src/model/block.cpp:140-148 does."""
    _require_cuda(qkv, q_out, k_cache, v_cache, token_seq, token_pos)
    tokens = qkv.shape[0]
    _, _, Hkv, D = k_cache.shape
    if qkv.dtype != torch.float32 or qkv.stride(1) != 1 or qkv.shape[1] != (n_heads + 2 * Hkv) * D or \
            q_out.dtype != torch.float16 or q_out.shape != (tokens, n_heads, D) or not q_out.is_contiguous():
        raise ValueError("qkv fp32 [tokens, (H + 2 Hkv) D], q_out dense fp16 [tokens, H, D]")
    a = _b.AttnRopePromptArgs()
    a.q_out, a.qkv, a.k_cache, a.v_cache = q_out.data_ptr(), qkv.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr()
    a.inv_freq = inv_freq.data_ptr() if inv_freq is not None else None
    a.token_seq, a.token_pos = token_seq.data_ptr(), token_pos.data_ptr()
    a.ld, a.kv_row_stride, a.kv_batch_stride = qkv.stride(0), k_cache.stride(1), k_cache.stride(0)
    a.tokens, a.n_heads, a.n_kv_heads, a.head_dim = tokens, n_heads, Hkv, D
    a.rotary_dim, a.theta, a.qkv_clip = rotary_dim, float(theta), float(qkv_clip)
    with torch.cuda.device(qkv.device):
        _b.check(_b.load().attn_rope_prompt(C.byref(a), _stream_ptr(stream)), "attn_rope_prompt")
    return q_out


def gather_rows(x: torch.Tensor, rows: torch.Tensor, *, out: torch.Tensor, stream=None) -> torch.Tensor:
    """out[r] = x[rows[r]] (fp32 rows; rows int32 on the device)."""
    _require_cuda(x, rows, out)
    with torch.cuda.device(x.device):
        _b.check(_b.load().attn_gather_rows(out.data_ptr(), x.data_ptr(), rows.data_ptr(), rows.numel(), x.shape[1],
                                            _stream_ptr(stream)), "attn_gather_rows")
    return out


def kernel_launch_count() -> int:
    return int(_b.load().attn_kernel_launch_count())
