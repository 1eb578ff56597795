"""Host-side mirror of the engine's Model / Block forward for a batch of sequences, every step on the device.

The engine's forward is one token of one sequence at a time (``Model::forward``, src/model/model.cpp:60-98;
``Block::block_cpu_``, src/model/block.cpp:105-223); its CUDA block stops after attention
(src/model/block.cu:235-239). This class runs the same sequence of steps for ``batch`` independent sequences per
call, each with its own position and KV cache, through the C ABI kernels only (GEMV, RMSNorm, RoPE + cache insert,
split-KV attention, SwiGLU, argmax): 9 launches per layer (stacked Q/K/V projection, SwiGLU as the epilogue of the
stacked gate/up projection, residual added by the next norm), none of them on the host, no CPU fallback.

Weights are the engine's: fp16 ``[d][n]`` matrices (n fastest, GGUF dims ``[n_in, n_out]``), fp32 norm vectors,
stacked over the layers here. The KV caches keep the engine's ``[row][kv_head][head_dim]`` fp16 layout, one cache
per layer and sequence.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import attention as A

KV_SINK = 4  # attention-sink rows of the sliding window (include/model/model.hpp)


@dataclass
class ModelConfig:
    """The fields of the engine's ModelConfig (include/model/config.hpp) that the forward pass reads."""
    dim: int
    hidden_dim: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    vocab_size: int
    max_seq_len: int
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rotary_dim: int = 0      # 0 = head_dim
    qkv_clip: float = 0.0    # 0 = no clamp

    def as_dict(self) -> dict:
        return dict(self.__dict__)


WEIGHT_SHAPES = {
    # name -> shape as a function of the config; all fp16 except the norms
    "embed": lambda c: (c.vocab_size, c.dim),
    "wcls": lambda c: (c.vocab_size, c.dim),
    "rms_final": lambda c: (c.dim,),
    "rms_att": lambda c: (c.n_layers, c.dim),
    "rms_ffn": lambda c: (c.n_layers, c.dim),
    "wq": lambda c: (c.n_layers, c.n_heads * c.head_dim, c.dim),
    "wk": lambda c: (c.n_layers, c.n_kv_heads * c.head_dim, c.dim),
    "wv": lambda c: (c.n_layers, c.n_kv_heads * c.head_dim, c.dim),
    "wo": lambda c: (c.n_layers, c.dim, c.n_heads * c.head_dim),
    "w1": lambda c: (c.n_layers, c.hidden_dim, c.dim),
    "w3": lambda c: (c.n_layers, c.hidden_dim, c.dim),
    "w2": lambda c: (c.n_layers, c.dim, c.hidden_dim),
}
NORM_NAMES = ("rms_final", "rms_att", "rms_ffn")


def random_weights(cfg: ModelConfig, seed: int, device="cpu", weight_type: str = "f16") -> dict:
    """Seeded random-init weights of the architecture (there are no checkpoints here): matrices ~ N(0, 1/n_in),
    embedding ~ N(0, 1), stored as fp16 or as Q8_0 blocks (uint8 [..., n/32*34]); norm weights ~ 1 + 0.1 N(0, 1) in
    fp32. Generated on ``device`` one layer at a time, so an 8B-parameter model never exists in fp32."""
    from . import quant
    g = torch.Generator(device=device).manual_seed(seed)
    out = {}
    for name, shape_of in WEIGHT_SHAPES.items():
        shape = shape_of(cfg)
        if name in NORM_NAMES:
            out[name] = 1.0 + 0.1 * torch.randn(shape, generator=g, dtype=torch.float32, device=device)
            continue
        std = 1.0 if name == "embed" else shape[-1] ** -0.5
        parts = []
        lead = shape[0] if len(shape) == 3 else 1
        for _ in range(lead):  # one layer's matrix at a time
            w = torch.randn(shape[-2:], generator=g, dtype=torch.float32, device=device) * std
            parts.append(quant.quantize_q8_0_torch(w) if weight_type == "q8_0" else w.half())
        out[name] = torch.stack(parts) if len(shape) == 3 else parts[0]
    return out


class Llama:
    """Batched token-at-a-time forward, whole-prompt prefill and greedy generation on one GPU."""

    def __init__(self, cfg: ModelConfig, weights: dict, batch: int, device=None, weight_type: str = "f16"):
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        if dev.type != "cuda":
            raise ValueError("the model runs on a CUDA device only (there is no CPU path)")
        self.cfg, self.batch, self.device = cfg, batch, dev
        c = cfg
        self.w = {}
        if weight_type not in ("f16", "q8_0"):
            raise ValueError("weight_type must be 'f16' (the engine's) or 'q8_0'")
        self.weight_type = weight_type
        q8 = weight_type == "q8_0"
        self._gemv = A.gemv_q8_0 if q8 else A.gemv_f16
        self._embed = A.embed_q8_0 if q8 else A.embed_f16
        for name, shape_of in WEIGHT_SHAPES.items():
            t = weights[name]
            shape = shape_of(c)
            if name in NORM_NAMES:
                want = torch.float32
            elif q8:
                want, shape = torch.uint8, shape[:-1] + (shape[-1] // 32 * 34,)
            else:
                want = torch.float16
            if tuple(t.shape) != shape or t.dtype != want:
                raise ValueError(f"weight {name}: expected {shape} {want}, got {tuple(t.shape)} {t.dtype}")
            self.w[name] = t.to(dev).contiguous()
        # The GEMVs take stacked matrices: Q, K and V rows in one launch with three outputs, and gate (w1) rows
        # followed by up (w3) rows with the SwiGLU product as its epilogue. Only the stacks are kept.
        self.w["wqkv"] = torch.cat([self.w.pop("wq"), self.w.pop("wk"), self.w.pop("wv")], dim=1).contiguous()
        self.w["w13"] = torch.cat([self.w.pop("w1"), self.w.pop("w3")], dim=1).contiguous()
        # Weights as the decode step's GEMVs read them. Q8_0: a tiled copy of every matrix, made once here (same bytes,
        # same products bit for bit, streamed and unpacked faster: attn_repack_q8_0_tiled); the GGML blocks stay for the
        # embedding rows and for the whole-prompt path, which expands them to fp16.
        self.wg, self._rows = self.w, {}
        if q8 and c.hidden_dim % 16 == 0:
            self.wg = dict(self.w)
            self._rows = {name: self.w[name].shape[-2] for name in ("wqkv", "wo", "w13", "w2", "wcls")}
            for name in ("wqkv", "wo", "w13", "w2"):
                self.wg[name] = torch.stack([A.repack_q8_0(self.w[name][l]) for l in range(c.n_layers)])
            self.wg["wcls"] = A.repack_q8_0(self.w["wcls"])
        B, f32 = batch, torch.float32
        q_dim, kv_dim = c.n_heads * c.head_dim, c.n_kv_heads * c.head_dim
        z = lambda *s, dtype=f32: torch.zeros(*s, dtype=dtype, device=dev)  # noqa: E731
        self.x = z(B, c.dim)
        # Activations that feed a GEMV: fp32, or with Q8_0 weights the prepared form (int32 words: fp16 value + fp16
        # residual), written by the producing kernel so that no GEMV CTA has to convert them again
        act = torch.int32 if q8 else f32
        self.xb = z(B, c.dim, dtype=act)
        self.q, self.k, self.v = z(B, c.n_heads, c.head_dim), z(B, c.n_kv_heads, c.head_dim), z(B, c.n_kv_heads, c.head_dim)
        self.att = z(B, c.n_heads, c.head_dim, dtype=act)
        self.hb = z(B, c.hidden_dim, dtype=act)
        self.logits = z(B, c.vocab_size)
        self.next_token = z(B, dtype=torch.int32)
        self.tokens = z(B, dtype=torch.int32)   # the step's input tokens; a decode step writes its picks back here
        self._graphs = None
        # The lengths are copied in before a step's first kernel and the kernel in front of the attention (rotary +
        # insert) writes only each sequence's newest row: the attention may start streaming the older rows early
        # (measured: 3.03 -> 3.00 ms per step of the 8B-shaped Q8_0 model at batch 8).
        self.kv_early = True
        self.pos, self.kv_pos, self.kv_len = (z(B, dtype=torch.int32) for _ in range(3))
        self.status = z(1, dtype=torch.int32)
        # one cache per layer and sequence, the engine's layout
        self.k_cache = z(c.n_layers, B, c.max_seq_len, c.n_kv_heads, c.head_dim, dtype=torch.float16)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.workspace = A.DecodeWorkspace(B, c.n_heads, c.n_kv_heads, c.head_dim, dev)
        self._q_dim, self._kv_dim = q_dim, kv_dim
        # The down projection of a batch: when the hidden activations of all sequences do not fit in shared memory next
        # to the weight ring, the inner dimension is split over sets of CTAs and the next RMSNorm adds the partial
        # products into x (same sum, fixed order).
        chunks = c.hidden_dim // 256
        need = B * (c.hidden_dim * 4 + 64)
        k = max(1, -(-need // (140 * 1024)))
        while k <= chunks and chunks % k:
            k += 1
        self._k_split = k if k <= chunks else 1
        self.partials = z(self._k_split, B, c.dim) if self._k_split > 1 else None

    @classmethod
    def from_gguf(cls, path: str, batch: int, device=None) -> "Llama":
        """Load a GGUF file (llama architecture, matrices all F16 or all Q8_0, F32 norms) as written by gguf.write_gguf
        or by any writer of the engine's format (tensor names of src/model/model.cpp:25-38, block.cpp:18-69)."""
        import numpy as np

        from . import gguf
        cfg, w, weight_type = gguf.read_gguf(path)
        weights = {k: torch.from_numpy(np.array(v)) for k, v in w.items()}  # copies out of the read-only map
        return cls(cfg, weights, batch, device, weight_type=weight_type)

    # -- positions: sliding-window arithmetic of src/model/model.cpp:66-68, per sequence --
    def _set_positions(self, pos) -> int:
        c = self.cfg
        pos = [int(p) for p in pos]
        over = [p >= c.max_seq_len for p in pos]
        if any(over) and not all(over):
            raise ValueError("sequences inside and outside the sliding window cannot share a step")
        kv_sink = KV_SINK if all(over) and over else 0
        kv_pos = [kv_sink + ((p - kv_sink) % (c.max_seq_len - kv_sink)) for p in pos]
        kv_len = [c.max_seq_len if p >= c.max_seq_len else p + 1 for p in pos]
        host = torch.tensor([pos, kv_pos, kv_len], dtype=torch.int32).pin_memory()
        self.pos.copy_(host[0], non_blocking=True)
        self.kv_pos.copy_(host[1], non_blocking=True)
        self.kv_len.copy_(host[2], non_blocking=True)
        return kv_sink

    def _launch_step(self, kv_sink: int, want_logits: bool) -> None:
        """Every launch of one step, reading self.tokens / pos / kv_pos / kv_len. With logits the step ends with the
        greedy pick (self.next_token) and feeds it back into self.tokens for the next step."""
        c, w, B = self.cfg, self.wg, self.batch

        def gemv(x, name, l=None, **kw):
            if name in self._rows:  # a tiled copy: its last row group may be padded
                kw["rows"] = self._rows[name]
            return self._gemv(x, w[name] if l is None else w[name][l], **kw)

        self._embed(w["embed"], self.tokens, out=self.x, status=self.status)
        att_flat = self.att.view(B, self._q_dim)
        pending = None  # partial products of the previous layer's down projection, still to be added into x
        for l in range(c.n_layers):
            A.rmsnorm(self.x, w["rms_att"][l], c.norm_eps, out=self.xb, partials=pending)
            pending = None
            gemv(self.xb, "wqkv", l, out=self.q.view(B, self._q_dim), out2=self.k.view(B, self._kv_dim),
                 out3=self.v.view(B, self._kv_dim), clip=c.qkv_clip)
            A.rope_kv_insert(self.q, self.k, self.v, self.k_cache[l], self.v_cache[l], self.pos, self.kv_pos,
                             theta=c.rope_theta, rotary_dim=c.rotary_dim, kv_sink=kv_sink, q_out=self.q,
                             pos_early=True)   # positions are copied in before the step's first kernel
            A.attn_decode(self.q, self.k_cache[l], self.v_cache[l], self.kv_len, out=self.att,
                          workspace=self.workspace, kv_early=self.kv_early)
            gemv(att_flat, "wo", l, out=self.x, accumulate=True)           # x += Wo att
            A.rmsnorm(self.x, w["rms_ffn"][l], c.norm_eps, out=self.xb)
            gemv(self.xb, "w13", l, out=self.hb, swiglu=True)              # hb = silu(W1 xb) * (W3 xb)
            if self._k_split > 1:
                gemv(self.hb, "w2", l, out=self.partials, k_split=self._k_split)
                pending = self.partials                                    # x += W2 hb, added by the next norm
            else:
                gemv(self.hb, "w2", l, out=self.x, accumulate=True)        # x += W2 (silu(W1 xb) * W3 xb)
        if not want_logits:
            return  # prefill mode: no final norm, no classifier (src/model/model.cpp:74-76); x is not read again
        A.rmsnorm(self.x, w["rms_final"], c.norm_eps, out=self.xb, partials=pending)
        gemv(self.xb, "wcls", out=self.logits)
        A.argmax(self.logits, out=self.next_token)
        self.tokens.copy_(self.next_token)

    def can_prefill(self, prompts, n_new: int = 0) -> bool:
        """Whether prefill() can take these prompts: head_dim 128 or 64 (the tensor-core attention kernel), inner
        dimensions in multiples of 64, and every sequence inside its cache (no sliding window during the prompt or after
        it)."""
        c = self.cfg
        dims_ok = c.head_dim in (64, 128) and c.dim % 64 == 0 and c.hidden_dim % 64 == 0 and (c.n_heads * c.head_dim) % 64 == 0
        return dims_ok and max(len(p) for p in prompts) + n_new <= c.max_seq_len

    def prefill(self, prompts, exact: bool = True) -> None:
        """The prompt phase for all sequences at once instead of one token per step: the tokens of every prompt are
        packed into one matrix of rows; per layer one tensor-core GEMM per projection (attn_gemm_f16; Q8_0 weights are
        expanded per matrix into an fp16 value / residual pair first), the rotary kernel that also fills the KV caches,
        causal attention per sequence (attn_prefill_causal straight over that sequence's cache rows), and the
        row-wise norm / SwiGLU steps. Per token this is the engine's forward pass (src/model/block.cpp:105-223) with
        InferenceMode::Prefill for all but the last token of a prompt (src/model/model.cpp:74-76); the last tokens go
        through the final norm, classifier and greedy pick. Afterwards the caches hold rows 0 .. len-1 of every
        sequence and self.next_token / self.tokens / self.logits are what the token-at-a-time loop would have left.
        ``exact`` = False drops the residual terms (activations and Q8_0 weights enter the tensor cores rounded once to
        fp16, one MMA instead of two or three): a third of the tensor work, results within about 1e-3 relative, no
        longer guaranteed to give the token-at-a-time path's greedy tokens."""
        import numpy as np
        c, w, B, dev = self.cfg, self.w, self.batch, self.device
        if len(prompts) != B or not self.can_prefill(prompts):
            raise ValueError("prefill() needs one prompt per sequence, head_dim 64 or 128 and prompts that fit the cache")
        q8 = self.weight_type == "q8_0"
        lens = [len(p) for p in prompts]
        starts = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        T = int(starts[-1])
        host = torch.tensor([t for p in prompts for t in p], dtype=torch.int32).pin_memory()
        seq = torch.from_numpy(np.repeat(np.arange(B, dtype=np.int32), lens)).pin_memory()
        pos = torch.from_numpy(np.concatenate([np.arange(n, dtype=np.int32) for n in lens])).pin_memory()
        last = torch.from_numpy((starts[1:] - 1).astype(np.int32)).pin_memory()
        tokens, token_seq, token_pos, last_rows = (t.to(dev, non_blocking=True) for t in (host, seq, pos, last))
        f32, f16 = torch.float32, torch.float16
        e = lambda *s, dtype=f32: torch.empty(*s, dtype=dtype, device=dev)  # noqa: E731
        q_dim, kv_dim, H, D = self._q_dim, self._kv_dim, c.n_heads, c.head_dim
        x = e(T, c.dim)
        pair_d = (e(T, c.dim, dtype=f16), e(T, c.dim, dtype=f16))
        pair_q = pair_d if q_dim == c.dim else (e(T, q_dim, dtype=f16), e(T, q_dim, dtype=f16))
        pair_h = (e(T, c.hidden_dim, dtype=f16), e(T, c.hidden_dim, dtype=f16))
        qkv = e(T, q_dim + 2 * kv_dim)
        q16 = e(T, H, D, dtype=f16)
        att = e(T, H, D)
        gate_up = e(T, 2 * c.hidden_dim)
        if q8:  # room for the largest matrix of a layer as an fp16 pair
            biggest = max(w[k].shape[1] * (w[k].shape[2] // 34 * 32) for k in ("wqkv", "wo", "w13", "w2"))
            w_hi, w_lo = e(biggest, dtype=f16), e(biggest, dtype=f16)

        def project(a_pair, wmat, out, accumulate):
            if q8:
                rows, n = wmat.shape[0], wmat.shape[1] // 34 * 32
                pair = (w_hi[:rows * n].view(rows, n), w_lo[:rows * n].view(rows, n))
                A.dequant_q8_0_pair(wmat, out=pair)
                A.gemm_f16(a_pair[0], a_pair[1] if exact else None, pair[0], out=out, accumulate=accumulate,
                           status=self.status)
                if exact:
                    A.gemm_f16(a_pair[0], None, pair[1], out=out, accumulate=True, status=self.status)
            else:
                A.gemm_f16(a_pair[0], a_pair[1] if exact else None, wmat, out=out, accumulate=accumulate,
                           status=self.status)

        self._embed(w["embed"], tokens, out=x, status=self.status)
        for l in range(c.n_layers):
            A.rmsnorm_pair(x, w["rms_att"][l], c.norm_eps, out=pair_d)
            project(pair_d, w["wqkv"][l], qkv, False)
            A.rope_prompt(qkv, q16, self.k_cache[l], self.v_cache[l], token_seq, token_pos, n_heads=H,
                          theta=c.rope_theta, rotary_dim=c.rotary_dim, qkv_clip=c.qkv_clip)
            for b in range(B):
                s0, s1, n = int(starts[b]), int(starts[b + 1]), lens[b]
                A.attn_prefill_causal(q16[s0:s1].unsqueeze(0), self.k_cache[l, b, :n].unsqueeze(0),
                                      self.v_cache[l, b, :n].unsqueeze(0), out=att[s0:s1].unsqueeze(0), status=self.status)
            A.split_pair(att.view(T, q_dim), out=pair_q)
            project(pair_q, w["wo"][l], x, True)                          # x += Wo att
            A.rmsnorm_pair(x, w["rms_ffn"][l], c.norm_eps, out=pair_d)
            project(pair_d, w["w13"][l], gate_up, False)                  # gate | up
            A.swiglu_pair(gate_up, out=pair_h)
            project(pair_h, w["w2"][l], x, True)                          # x += W2 (silu(gate) * up)
        # the last token of every prompt: final norm, classifier, greedy pick (the decode step's own kernels)
        A.gather_rows(x, last_rows, out=self.x)
        A.rmsnorm(self.x, w["rms_final"], c.norm_eps, out=self.xb)
        self._gemv(self.xb, self.wg["wcls"], out=self.logits, **({"rows": self._rows["wcls"]} if self._rows else {}))
        A.argmax(self.logits, out=self.next_token)
        self.tokens.copy_(self.next_token)

    def capture(self) -> None:
        """Record the step once per mode (prefill: no classifier; decode: classifier + greedy pick + feedback) as CUDA
        graphs, the way the engine drives its CUDA step (include/model/device.hpp:161-262): a step then costs one
        graph launch instead of 9 launches per layer. Positions inside the sliding window only (kv_sink = 0)."""
        if self._graphs is not None:
            return
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):   # one eager step first: every kernel does its lazy set-up outside the capture
            self._set_positions([0] * self.batch)
            self._launch_step(0, True)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graphs = {}
        for want_logits in (False, True):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._launch_step(0, want_logits)
            graphs[want_logits] = g
        self._graphs = graphs

    def forward(self, tokens, pos, want_logits: bool = True):
        """One token per sequence: tokens int32 [B] on the device (None = keep self.tokens, i.e. the previous picks),
        pos a list of B positions (or one int for all). Returns the logits [B, vocab] (a view of the model's buffer)
        or None in prefill mode. Replays the captured graph when capture() was called and no position has left the
        sliding window."""
        if isinstance(pos, int):
            pos = [pos] * self.batch
        if tokens is not None and tokens is not self.tokens:
            self.tokens.copy_(tokens, non_blocking=True)
        kv_sink = self._set_positions(pos)
        if self._graphs is not None and kv_sink == 0:
            self._graphs[bool(want_logits)].replay()
        else:
            self._launch_step(kv_sink, want_logits)
        return self.logits if want_logits else None

    def generate(self, prompts, n_new: int, want_logits: bool = False, timing: dict | None = None,
                 prompt_mode: str = "auto"):
        """Greedy generation for a ragged batch: prompts is a list of B token-id lists. Every sequence is fed one
        token per step from position 0 (its prompt, then its own picks), exactly the engine's loop
        (tools/infer.cpp:271-300, without the end-of-sequence stop); sequences start late so that all prompts end
        at the same step and the generation steps run as one dense batch. Returns int32 [B, n_new] on the host
        (and the logits each pick was made from, [B, n_new, vocab], when asked). ``timing`` (a dict) receives the
        device time of the prompt phase and of the generation phase in ms (CUDA events). ``prompt_mode``: "token" feeds
        the prompts one token per step as described; "batched" runs prefill() (all prompt tokens at once on the tensor
        cores); "auto" picks "batched" whenever can_prefill() allows it; "batched-single-rounding" is prefill() with
        exact = False."""
        B = self.batch
        if len(prompts) != B or any(len(p) == 0 for p in prompts):
            raise ValueError("one non-empty prompt per sequence of the batch")
        longest = max(len(p) for p in prompts)
        if longest + n_new > self.cfg.max_seq_len and any(len(p) != longest for p in prompts):
            raise ValueError("only prompts of one length may run past max_seq_len (one sink setting per step)")
        delay = [longest - len(p) for p in prompts]
        out = torch.zeros((B, n_new), dtype=torch.int32, device=self.device)
        out_logits = torch.zeros((B, n_new, self.cfg.vocab_size), device=self.device) if want_logits else None
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        if prompt_mode not in ("auto", "token", "batched", "batched-single-rounding"):
            raise ValueError("prompt_mode must be 'auto', 'token', 'batched' or 'batched-single-rounding'")
        batched = prompt_mode.startswith("batched") or (prompt_mode == "auto" and self.can_prefill(prompts, n_new))
        ev[0].record()
        if batched:
            self.prefill(prompts, exact=prompt_mode != "batched-single-rounding")
        for step in range(0 if batched else longest):
            # a sequence that has not started yet is fed its first token at position 0 again (row 0 is rewritten)
            pos = [max(step - d, 0) for d in delay]
            host = torch.tensor([p[q] for p, q in zip(prompts, pos)], dtype=torch.int32).pin_memory()
            self.forward(host, pos, want_logits=(step + 1 == longest))
        ev[1].record()
        for i in range(n_new):
            out[:, i] = self.next_token
            if want_logits:
                out_logits[:, i] = self.logits
            if i + 1 < n_new:
                self.forward(None, [len(p) + i for p in prompts])
        ev[2].record()
        torch.cuda.synchronize(self.device)
        if timing is not None:
            timing.update(prompt_ms=ev[0].elapsed_time(ev[1]), generate_ms=ev[1].elapsed_time(ev[2]),
                          prompt_steps=longest, generate_steps=n_new - 1,
                          prompt_mode="batched (tensor-core GEMMs + causal prefill attention)" if batched
                          else "token-at-a-time")
        if int(self.status.item()) != 0 or int(self.workspace.status.item()) != 0:
            raise RuntimeError("a kernel reported a status bit (token id out of range or a wait that ran out)")
        return (out.cpu(), out_logits.cpu()) if want_logits else out.cpu()
