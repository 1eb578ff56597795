#!/usr/bin/env python
"""Benchmark of the B200 attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1   one step = one batched decode-attention call (split-KV pass + merge pass) on the
        Llama-3-8B-shaped workload: batch 16, 32 query / 8 kv heads, head_dim 128, KV length 4096,
        fp16, inputs resident in HBM. Metric: algorithmic HBM GB/s of that call.
N > 1   one step = one long-context decode with the KV sequence (131072 rows) sharded evenly over
        the N GPUs: local split-KV pass, then one kernel that merges the local partials, exchanges the
        per-GPU (O, LSE) rows through peer memory over NVLink and finishes the LSE merge (replayed from a
        CUDA graph). The NCCL all-gather variant of the same step is timed next to it.
        Launched by torch.distributed.run, one process per GPU. Total work is fixed ("strong").

Prints ONE JSON line (rank 0). `--impl reference` times the engine's own CPU attention
(include/kernels_cpu.hpp, compiled under oracle/_ref, else the C restatement) on the host cores.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def ncu_traffic_bytes():
    """dram__bytes_read.sum + dram__bytes_write.sum of one split-pass launch on the N=1 workload, recorded from a
    profiler capture together with a hash of the kernel's sources; None when the sources have changed since."""
    import hashlib
    path = os.path.join(ROOT, "profiles", "decode_split_traffic.json")
    try:
        with open(path) as f:
            rec = json.load(f)
        h = hashlib.sha256()
        for rel in rec["kernel_sources"]:
            with open(os.path.join(ROOT, rel), "rb") as f:
                h.update(f.read())
        return int(rec["traffic_bytes_per_launch"]) if h.hexdigest() == rec["sha256"] else None
    except Exception:
        return None


def load_package():
    name = "llm_infer_b200"
    if name in sys.modules:
        return sys.modules[name]
    d = os.path.join(ROOT, "llm-infer_b200")
    spec = importlib.util.spec_from_file_location(name, os.path.join(d, "__init__.py"),
                                                  submodule_search_locations=[d])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 0.0)), "measured"
    return 6650.0, 1590.0, "fallback"


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML from a thread while the timed region runs."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting"}

    def __init__(self, device_index: int):
        self.samples = []
        self.reason_bits = 0
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            self._nv = pynvml
            try:
                uuid = "GPU-" + str(torch.cuda.get_device_properties(device_index).uuid)
                self._h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self._h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._h = None

    def _poll(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                self.reason_bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
            except Exception:
                break
            time.sleep(0.001)

    def __enter__(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._poll, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz,
                "reasons": [name for bit, name in self.REASONS.items() if self.reason_bits & bit],
                "samples": len(s)}


# --------------------------------------------------------------------------- CPU baseline
def cpu_reference_arm(wl, shape, steps: int, warmup: int, seconds_budget: float = 25.0):
    """Times the engine's CPU attention on a bounded sample of `shape` (whole sequences, or the first rows of one
    long sequence) on every core this process may use. Returns (GB/s, description dict, steps timed)."""
    import numpy as np
    import oracle

    chk = oracle.best()
    kind = "reference" if chk.kind == "reference" else "port"
    # torch.distributed.run exports OMP_NUM_THREADS=1 to its workers: ask for the host's cores explicitly
    cores = chk.set_num_threads(None)
    # sample: one sequence of the batch; long sequences are cut to 8192 rows so that one step stays well under 0.2 s
    rows = min(shape.kv_len, 8192)
    sample = wl.DecodeShape(shape.name + "-cpu-sample", shape.seed, 1, shape.n_heads, shape.n_kv_heads,
                            shape.head_dim, rows, shape.q_dtype, shape.kv_dtype)
    q, k, v = wl.decode_inputs(sample)
    q32 = wl.widen(q, sample.q_dtype)
    k16, v16 = wl.as_f16_for_oracle(k, sample.kv_dtype), wl.as_f16_for_oracle(v, sample.kv_dtype)
    # warm-up: at least `warmup` calls and half a second (thread pool spin-up, page faults, clock ramp)
    t0 = time.perf_counter()
    n = 0
    while n < max(3, warmup) or time.perf_counter() - t0 < 0.5:
        chk.attn_decode(q32, k16, v16)
        n += 1
    # timed: at least `steps` calls and one second, at most the budget
    t0 = time.perf_counter()
    done = 0
    while True:
        chk.attn_decode(q32, k16, v16)
        done += 1
        el = time.perf_counter() - t0
        if el > seconds_budget or (done >= steps and el >= 1.0):
            break
    dt = (time.perf_counter() - t0) / done
    gbs = sample.algorithmic_bytes() / dt / 1e9
    desc = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": kind,
            "sample": f"1 sequence x {rows} KV rows of the workload per step, {done} steps, "
                      f"{dt * 1e3:.2f} ms/step; OpenMP over the {shape.n_heads} query heads as the engine does",
            "ms_per_step": dt * 1e3}
    return gbs, desc, done


def run_reference(args, world: int, rank: int):
    pkg = load_package()
    wl = pkg.workloads
    if rank != 0:
        return
    shape = wl.C2 if world == 1 else wl.C4
    gbs, desc, done = cpu_reference_arm(wl, shape, args.steps, args.warmup, seconds_budget=120.0)
    line = {
        "impl": "reference", "metric": "decode_attn_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": world,
        "steps": done, "warmup": args.warmup, "ms_per_step": desc["ms_per_step"], "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f16 storage, f32 accumulate",
        "data": "synthetic", "config": workload_config(shape, world),
        "cpu_baseline": {k: desc[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(shape, world: int):
    cfg = {"workload": shape.name, "batch": shape.batch, "kv_len": shape.kv_len, "n_heads": shape.n_heads,
           "n_kv_heads": shape.n_kv_heads, "head_dim": shape.head_dim, "q_dtype": shape.q_dtype,
           "kv_dtype": shape.kv_dtype, "kv_layout": "[seq][kv_head][head_dim] per sequence"}
    if world > 1:
        cfg["parallelism"] = f"kv-sequence sharded over {world} GPUs, exchange of per-GPU (O, LSE), LSE merge"
    return cfg


# --------------------------------------------------------------------------- prefill (tensor-bound part of the metric)
def prefill_measure(torch, attention, wl, steps: int, warmup: int, tflops_peak: float, peak_kind: str):
    """Causal prefill on the Llama-3-8B-shaped workload (batch 4 x 2048, 32/8 heads, head_dim 128, bf16).
    FLOPs are the causal count 4*D*B*H*S*(S+1)/2 (unmasked multiply-adds of QK^T and PV only)."""
    shape = wl.C3
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev)
    gen.manual_seed(shape.seed)
    B, S, H, Hkv, D = shape.batch, shape.seq, shape.n_heads, shape.n_kv_heads, shape.head_dim
    # two input copies rotated: q+k+v+o of one copy are 168 MB, more than the 126 MB L2
    sets = []
    for _ in range(2):
        q = torch.randn((B, S, H, D), generator=gen, device=dev, dtype=torch.float32).bfloat16()
        k = torch.randn((B, S, Hkv, D), generator=gen, device=dev, dtype=torch.float32).bfloat16()
        v = torch.randn((B, S, Hkv, D), generator=gen, device=dev, dtype=torch.float32).bfloat16()
        sets.append((q, k, v, torch.empty_like(q)))
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    res = {}
    for name, mode in (("precise", 0), ("fast", 1)):
        def step(i, mode=mode):
            q, k, v, o = sets[i % 2]
            attention.attn_prefill_causal(q, k, v, out=o, p_mode=mode, status=status)
        for i in range(max(3, warmup)):
            step(i)
        ms = time_steps(torch, step, steps) / steps
        tf = shape.causal_flops / (ms * 1e-3) / 1e12
        res[name] = {"us": round(ms * 1e3, 2), "tflops": round(tf, 1), "frac_of_peak": round(tf / tflops_peak, 3),
                     "tok_per_s": round(B * S / (ms * 1e-3), 1)}
    assert int(status.item()) == 0, "prefill status word reports a timed-out wait"
    return {"workload": shape.name, "dtype": "bf16 in, f32 accumulate, bf16 out", "causal_flops": shape.causal_flops,
            "peak_tflops": tflops_peak, "peak_kind": f"of {peak_kind} (cuBLAS bf16 burst)",
            "modes": res,
            "note": "precise (the default) = probabilities as 16-bit value + residual (two PV MMAs), the mode that meets "
                    "the parity tolerance on every row; fast = one probability rounded to bf16 (one PV MMA, outside "
                    "the tolerance)"}


# --------------------------------------------------------------------------- our arm, 1 GPU
def generate_measure(torch, batch: int = 8, n_new: int = 128, seed: int = 5, prompt_range=(128, 2048), graph=True):
    """End-to-end greedy generation with a random-init Llama-3-8B-shaped model stored as a seed-generated Q8_0 GGUF
    file (32 layers, 4096, 32/8 heads of 128, FFN 14336, vocab 128256, theta 5e5): the weights are generated on the
    device from a seed, quantised, written as a GGUF v3 file the engine's parser accepts, and the model that runs is
    loaded back from that file. A ragged batch of 8 prompts with lengths uniform in [128, 2048] (seeded random token
    ids), 128 new tokens each, token-at-a-time as the engine does, every step one CUDA-graph launch."""
    import shutil
    import tempfile

    import numpy as np
    from llm_infer_b200 import gguf
    from llm_infer_b200 import model as M
    rng = np.random.default_rng(seed)
    lengths = rng.integers(prompt_range[0], prompt_range[1] + 1, size=batch).tolist()
    cfg = M.ModelConfig(dim=4096, hidden_dim=14336, n_layers=32, n_heads=32, n_kv_heads=8, head_dim=128,
                        vocab_size=128256, max_seq_len=max(lengths) + n_new, norm_eps=1e-5, rope_theta=500000.0)
    w = M.random_weights(cfg, seed, device="cuda", weight_type="q8_0")
    # the file goes to memory-backed storage when there is room for it (9 GB), else to the temporary directory
    roots = [d for d in ("/dev/shm", tempfile.gettempdir()) if os.path.isdir(d) and shutil.disk_usage(d).free > 12e9]
    if not roots:
        raise RuntimeError("no room for the 9 GB model file")
    workdir = tempfile.mkdtemp(prefix="llm_infer_b200_", dir=roots[0])
    path = os.path.join(workdir, "llama3-8b-shaped-seed%d.q8_0.gguf" % seed)
    try:
        t0 = time.perf_counter()
        gguf.write_gguf(path, cfg, w, "q8_0")
        write_s = time.perf_counter() - t0
        file_bytes = os.path.getsize(path)
        del w
        torch.cuda.empty_cache()
        t0 = time.perf_counter()
        llama = M.Llama.from_gguf(path, batch)
        torch.cuda.synchronize()
        load_s = time.perf_counter() - t0
    finally:
        shutil.rmtree(workdir, ignore_errors=True)
    weight_bytes = sum(t.numel() * t.element_size() for k, t in llama.w.items() if k != "embed")
    if graph:
        llama.capture()
    prompts = [rng.integers(0, cfg.vocab_size, size=n).tolist() for n in lengths]
    llama.generate([p[:4] for p in prompts], 4)  # warm-up
    timing = {}
    tokens = llama.generate(prompts, n_new, timing=timing)
    gen_ms = timing["generate_ms"] / max(1, timing["generate_steps"])
    # the prompt phase the other two ways, for comparison: one token per step (the engine's loop), and the batched
    # path without the residual terms (not the parity mode)
    t_tok, t_single = {}, {}
    tokens_tok = llama.generate(prompts, 2, timing=t_tok, prompt_mode="token")
    llama.generate(prompts, 2, timing=t_single, prompt_mode="batched-single-rounding")
    res = {
        "workload": "Llama-3-8B-shaped random-init model loaded from a seed-generated Q8_0 GGUF file, batch 8, prompts "
                    f"{lengths}, {n_new} new tokens each, greedy, one CUDA graph launch per step",
        "gguf_file_bytes": file_bytes, "gguf_write_s": round(write_s, 2), "gguf_load_s": round(load_s, 2),
        "generate_tok_per_s": batch * 1e3 / gen_ms, "generate_ms_per_step": gen_ms,
        "prompt_tok_per_s": sum(lengths) * 1e3 / timing["prompt_ms"],
        "prompt_ms": timing["prompt_ms"], "prompt_mode": timing.get("prompt_mode", "token-at-a-time"),
        "prompt_tok_per_s_token_at_a_time": sum(lengths) * 1e3 / t_tok["prompt_ms"],
        "prompt_tok_per_s_single_rounding": sum(lengths) * 1e3 / t_single["prompt_ms"],
        "first_two_tokens_equal_token_at_a_time_path": bool((tokens[:, :2] == tokens_tok).all()),
        "weight_bytes_per_decode_step": weight_bytes,
        "weight_stream_gbs": weight_bytes / (gen_ms * 1e-3) / 1e9,
        "distinct_tokens_generated": int(len(set(tokens.flatten().tolist()))),
    }
    del llama
    torch.cuda.empty_cache()
    return res


def gemv_measure(torch, steps: int, warmup: int, hbm_peak: float, peak_kind: str, kinds=None):
    """The weight GEMVs of one Llama-3-8B-shaped layer alone (rotated weight copies > L2, CUDA events; replayed from a
    CUDA graph and launched one by one): fp16 and Q8_0, batch 1 and 8. Used for profiler captures and the GEMV roofline figures. ``kinds`` restricts the
    run to some of "q8_0", "q8_0_tiled", "f16" (profiler captures of one kernel)."""
    import numpy as np
    from llm_infer_b200 import attention as A, quant
    rng = np.random.default_rng(0)
    d, n = 14336, 4096
    res = {}
    base = rng.standard_normal((2048, n), dtype=np.float32)
    wq8 = torch.from_numpy(quant.quantize_q8_0(base)).cuda().repeat(d // 2048, 1).contiguous()
    wf16 = torch.from_numpy(base.astype(np.float16)).cuda().repeat(d // 2048, 1).contiguous()
    for kind, w, fn in (("q8_0", wq8, A.gemv_q8_0), ("q8_0_tiled", wq8, A.gemv_q8_0), ("f16", wf16, A.gemv_f16)):
        if kinds and kind not in kinds:
            continue
        copies = [w.clone() for _ in range(int(400e6 // (w.numel() * w.element_size())) + 2)]
        if kind == "q8_0_tiled":  # the tiled copy of the same blocks, and activations in the prepared form
            copies = [A.repack_q8_0(c) for c in copies]
        for batch in (1, 8):
            x = torch.randn(batch, n, device="cuda")
            if kind == "q8_0_tiled":
                x = A.rmsnorm(x, torch.ones(n, device="cuda"), 1e-5,
                              out=torch.empty(batch, n, dtype=torch.int32, device="cuda"))
            out = torch.empty(batch, d, device="cuda")
            for i in range(max(3, warmup)):
                fn(x, copies[i % len(copies)], out=out)
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for i in range(steps):
                fn(x, copies[i % len(copies)], out=out)
            t1.record()
            torch.cuda.synchronize()
            eager_us = t0.elapsed_time(t1) * 1e3 / steps
            alg = w.numel() * w.element_size() + batch * (n * 4 + d * 4)
            # The figure of the row: the same calls replayed from one CUDA graph. The host's launch cost (which exceeds
            # the kernel's time when launches come from Python one by one) is out of it, and consecutive launches
            # overlap through programmatic dependent launch, as they do in a model step.
            g = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side), torch.cuda.graph(g):
                for c in copies:
                    fn(x, c, out=out)
            torch.cuda.current_stream().wait_stream(side)
            g.replay()
            torch.cuda.synchronize()
            t0.record()
            for _ in range(10):
                g.replay()
            t1.record()
            torch.cuda.synchronize()
            us = t0.elapsed_time(t1) * 1e3 / (10 * len(copies))
            res[f"{kind}_b{batch}"] = {"us": round(us, 2), "gbs": round(alg / us / 1e3, 1),
                                       "frac": round(alg / us / 1e3 / hbm_peak, 3), "algorithmic_bytes": alg,
                                       "eager_us": round(eager_us, 2)}
        del copies
    res["note"] = (f"{d}x{n} matrix, rotated weight copies > L2; us / gbs / frac = CUDA-graph replay of the calls "
                   f"(device time), eager_us = launched one by one from Python (host launch cost included); frac of "
                   f"{peak_kind} HBM peak {hbm_peak:.1f} GB/s; q8_0 = GGML blocks with fp32 activations, q8_0_tiled = "
                   "the tiled copy of the same blocks with prepared activations (what a model step runs)")
    return res


def decode_trace(torch):
    """Where the time of one attn_decode call goes. Needs the profiling build of the library (python
    llm-infer_b200/build.py --trace, loaded through LLM_INFER_ATTN_LIB): its kernels store the GPU's nanosecond timer
    at a few points per CTA. For each shape one flushed call is traced five times; printed are, in microseconds after
    the first CTA of the split pass started, the median and the maximum over CTAs of every point, for the run with the
    median total."""
    import ctypes as C
    from llm_infer_b200 import attention, binding
    lib = binding.load()
    if not hasattr(lib, "attn_trace_set_buffers"):
        raise SystemExit("--decode-trace needs the profiling build: python llm-infer_b200/build.py --trace && "
                         "LLM_INFER_ATTN_LIB=llm-infer_b200/libllm_infer_attn_trace.so python bench.py --decode-trace")
    lib.attn_trace_set_buffers.argtypes = [C.c_void_p, C.c_void_p]
    lib.attn_trace_set_buffers.restype = None
    dev = torch.device("cuda", 0)
    H, Hkv, D = 32, 8, 128
    split_names = ["entry", "previous kernel done", "set-up done", "q in registers", "first K tile landed",
                   "last tile computed", "partials written", "producer issued last copy"]
    merge_names = ["entry", "split pass done, addresses ready", "partials folded", "row stored"]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    tr_split = torch.zeros(1024 * 8, dtype=torch.int64, device=dev)
    tr_merge = torch.zeros(4096 * 8, dtype=torch.int64, device=dev)
    out = {}
    # what the bracketing events cost by themselves: nothing between them, and one trivial kernel between them
    floors = {"nothing": [], "one_trivial_kernel": []}
    one = torch.zeros(32, device=dev)
    for name in floors:
        for _ in range(7):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if name != "nothing":
                one.add_(1.0)
            e1.record()
            torch.cuda.synchronize()
            floors[name].append(e0.elapsed_time(e1) * 1e3)
        floors[name] = round(sorted(floors[name])[3], 2)
    out["event_floor_us"] = floors
    for b, t in ((1, 64), (1, 4096), (16, 4096), (1, 16384), (1, 32768), (1, 131072)):
        q = torch.randn((b, H, D), device=dev).half()
        k = torch.randn((b, t, Hkv, D), device=dev, dtype=torch.float16)
        v = torch.randn((b, t, Hkv, D), device=dev, dtype=torch.float16)
        o = torch.empty((b, H, D), device=dev)
        ws = attention.DecodeWorkspace(b, H, Hkv, D, dev)
        lib.attn_trace_set_buffers(None, None)
        for _ in range(3):
            attention.attn_decode(q, k, v, out=o, workspace=ws)
        runs = []
        for _ in range(5):
            flush.zero_()
            tr_split.zero_()
            tr_merge.zero_()
            torch.cuda.synchronize()
            lib.attn_trace_set_buffers(tr_split.data_ptr(), tr_merge.data_ptr())
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            flush.zero_()
            e0.record()
            attention.attn_decode(q, k, v, out=o, workspace=ws)
            e1.record()
            torch.cuda.synchronize()
            lib.attn_trace_set_buffers(None, None)
            sp = tr_split.view(-1, 8).cpu().numpy().astype("int64")
            mg = tr_merge.view(-1, 8).cpu().numpy().astype("int64")
            sp = sp[sp[:, 0] > 0]
            mg = mg[mg[:, 0] > 0]
            t0 = int(sp[:, 0].min())
            rec = {"event_us": round(e0.elapsed_time(e1) * 1e3, 2), "split_ctas": int(len(sp)),
                   "split_ctas_with_tiles": int((sp[:, 5] > 0).sum()), "merge_ctas": int(len(mg)), "split": {}, "merge": {}}
            for i, name in enumerate(split_names):
                col = sp[:, i][sp[:, i] > 0]
                if len(col):
                    rel = (col - t0) / 1e3
                    rec["split"][name] = [round(float(sorted(rel)[len(rel) // 2]), 2), round(float(rel.max()), 2)]
            for i, name in enumerate(merge_names):
                col = mg[:, i][mg[:, i] > 0]
                if len(col):
                    rel = (col - t0) / 1e3
                    rec["merge"][name] = [round(float(rel.min()), 2), round(float(sorted(rel)[len(rel) // 2]), 2),
                                          round(float(rel.max()), 2)]
            rec["total_us_first_entry_to_last_store"] = round((int(mg[:, 3].max()) - t0) / 1e3, 2)
            runs.append(rec)
        runs.sort(key=lambda r: r["event_us"])
        out[f"b{b}_kv{t}"] = runs[len(runs) // 2]
        del q, k, v, o, ws
    # The same stamps for the LAST of four back-to-back steps on rotated inputs (no flush, no events in between): how
    # consecutive calls overlap through the programmatic-launch chain, with and without early K/V streaming.
    b, t = 16, 4096
    sets = [(torch.randn((b, H, D), device=dev).half(), torch.randn((b, t, Hkv, D), device=dev, dtype=torch.float16),
             torch.randn((b, t, Hkv, D), device=dev, dtype=torch.float16)) for _ in range(3)]
    o = torch.empty((b, H, D), device=dev)
    ws = attention.DecodeWorkspace(b, H, Hkv, D, dev)
    for early in (False, True):
        runs = []
        for _ in range(5):
            tr_split.zero_()
            tr_merge.zero_()
            torch.cuda.synchronize()
            lib.attn_trace_set_buffers(tr_split.data_ptr(), tr_merge.data_ptr())
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(4):
                q, k, v = sets[i % 3]
                attention.attn_decode(q, k, v, out=o, workspace=ws, kv_early=early)
            e1.record()
            torch.cuda.synchronize()
            lib.attn_trace_set_buffers(None, None)
            sp = tr_split.view(-1, 8).cpu().numpy().astype("int64")
            mg = tr_merge.view(-1, 8).cpu().numpy().astype("int64")
            sp, mg = sp[sp[:, 0] > 0], mg[mg[:, 0] > 0]
            t0 = int(sp[:, 0].min())
            rec = {"four_steps_event_us": round(e0.elapsed_time(e1) * 1e3, 2), "split": {}, "merge": {}}
            for i, name in enumerate(split_names):
                col = sp[:, i][sp[:, i] > 0]
                rel = (col - t0) / 1e3
                rec["split"][name] = [round(float(rel.min()), 2), round(float(sorted(rel)[len(rel) // 2]), 2), round(float(rel.max()), 2)]
            for i, name in enumerate(merge_names):
                col = mg[:, i][mg[:, i] > 0]
                rel = (col - t0) / 1e3
                rec["merge"][name] = [round(float(rel.min()), 2), round(float(sorted(rel)[len(rel) // 2]), 2), round(float(rel.max()), 2)]
            runs.append(rec)
        runs.sort(key=lambda r: r["four_steps_event_us"])
        out[f"loop_b16_kv4096_last_of_4_steps_kv_early={early}"] = runs[len(runs) // 2]
    print(json.dumps({"decode_trace": out, "legend": {"split": "[median, max] over CTAs, us after the first CTA's entry",
                                                        "merge": "[min, median, max] over CTAs, same origin"}}), flush=True)


def attention_symbol_measure(torch, hbm_peak: float):
    """The engine's own kernel symbol (include/kernels.cuh:26: fp32 q/o, fp16 K/V, one sequence, one launch that
    splits and merges) driven the way the engine drives it: a CUDA-graph kernel node whose arguments are refreshed for
    every token (include/model/device.hpp:219-237), then the graph launch. KV 4096 and 131072, 32/8 heads of 128; the
    caches rotate through more copies than fit in L2."""
    import ctypes as C
    from llm_infer_b200 import binding
    lib = binding.load()
    rt = C.CDLL("libcudart.so.12")
    dev = torch.device("cuda", torch.cuda.current_device())
    H, Hkv, D = 32, 8, 128
    nbytes = lib.attention_workspace_bytes(H, Hkv, D)
    ws = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    if lib.attention_configure(H, Hkv, D, 0.0, ws.data_ptr(), nbytes, stream) != 0:
        raise RuntimeError("attention_configure failed")
    q = torch.randn((H, D), device=dev)
    o = torch.empty((H, D), device=dev)
    res = {}
    for T in (4096, 131072):
        per_copy = 2 * T * Hkv * D * 2
        n_copies = max(2, min(64, int(300e6 // per_copy) + 1))
        ks = [torch.randn((T, Hkv, D), device=dev, dtype=torch.float16) for _ in range(n_copies)]
        vs = [torch.randn((T, Hkv, D), device=dev, dtype=torch.float16) for _ in range(n_copies)]
        graph, node, gexec = C.c_void_p(), C.c_void_p(), C.c_void_p()
        assert rt.cudaGraphCreate(C.byref(graph), 0) == 0
        assert lib.attention_graph_add_node(graph, C.byref(node), None, 0, o.data_ptr(), q.data_ptr(), ks[0].data_ptr(),
                                            vs[0].data_ptr(), T) == 0
        rt.cudaGraphInstantiate.argtypes = [C.c_void_p, C.c_void_p, C.c_ulonglong]
        assert rt.cudaGraphInstantiate(C.byref(gexec), graph, 0) == 0
        rt.cudaGraphLaunch.argtypes = [C.c_void_p, C.c_void_p]

        def token(i):
            j = i % n_copies
            lib.attention_graph_exec_update(gexec, node, o.data_ptr(), q.data_ptr(), ks[j].data_ptr(), vs[j].data_ptr(), T)
            rt.cudaGraphLaunch(gexec, stream)

        for i in range(5):
            token(i)
        n = 100 if T <= 4096 else 30
        us = time_steps(torch, token, n) / n * 1e3
        # the kernel alone: plain launches back to back (no node update between them)
        def plain(i):
            j = i % n_copies
            lib.attention_launch(o.data_ptr(), q.data_ptr(), ks[j].data_ptr(), vs[j].data_ptr(), T, stream)

        for i in range(5):
            plain(i)
        kernel_us = time_steps(torch, plain, n) / n * 1e3
        bits = C.c_uint32(0)
        lib.attention_status(C.byref(bits), 0, stream)
        alg = per_copy + 2 * H * D * 4
        res[f"kv{T}"] = {"us_per_token": round(us, 2), "kernel_us": round(kernel_us, 2), "gbs": round(alg / us / 1e3, 1),
                         "frac_of_peak": round(alg / us / 1e3 / hbm_peak, 3), "status_bits": int(bits.value)}
        rt.cudaGraphExecDestroy.argtypes = [C.c_void_p]
        rt.cudaGraphDestroy.argtypes = [C.c_void_p]
        rt.cudaGraphExecDestroy(gexec)
        rt.cudaGraphDestroy(graph)
        del ks, vs
    res["note"] = ("one graph launch per token with the node's arguments refreshed first, back to back; single-launch "
                   "mode (the CTAs that deliver the last partials merge them, in two levels for long sequences)")
    return res


def gemm_measure(torch, steps: int, warmup: int, tflops_peak: float, peak_kind: str, small: bool = False):
    """The projection GEMM of the whole-prompt path alone (attn_gemm_f16: tokens x weights on the tensor cores,
    activations as an fp16 value + residual pair = two MMAs per k-step), on the four projections of a
    Llama-3-8B-shaped layer at the C5 prompt load (9101 tokens). Useful FLOPs = 2 m n k; the tensor cores do twice
    that. ``small`` = one 4096^3 case only (profiler captures)."""
    from llm_infer_b200 import attention as A
    dev = torch.device("cuda", torch.cuda.current_device())
    shapes = [(4096, 4096, 4096)] if small else [(9101, 6144, 4096), (9101, 4096, 4096), (9101, 28672, 4096),
                                                  (9101, 4096, 14336)]
    res = {}
    for m, n, k in shapes:
        hi = torch.randn((m, k), device=dev).half()
        lo = (torch.randn((m, k), device=dev) * 1e-4).half()
        ws = [(torch.randn((n, k), device=dev) * k ** -0.5).half() for _ in range(2)]
        out = torch.empty((m, n), device=dev)
        for i in range(max(3, warmup)):
            A.gemm_f16(hi, lo, ws[i % 2], out=out)
        ms = time_steps(torch, lambda i: A.gemm_f16(hi, lo, ws[i % 2], out=out), steps) / steps
        useful = 2.0 * m * n * k
        res[f"m{m}_n{n}_k{k}"] = {"us": round(ms * 1e3, 1), "useful_tflops": round(useful / ms / 1e9, 1),
                                  "tensor_tflops": round(2 * useful / ms / 1e9, 1),
                                  "tensor_frac_of_peak": round(2 * useful / ms / 1e9 / tflops_peak, 3)}
        del hi, lo, ws, out
    res["note"] = (f"tensor_tflops = 2 x useful (value + residual MMAs); frac of {peak_kind} cuBLAS bf16 burst peak "
                   f"{tflops_peak:.0f} TFLOP/s")
    return res


def time_steps(torch, fn, steps: int):
    """CUDA-event time of `steps` calls of fn(i) on the current stream, in ms."""
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for i in range(steps):
        fn(i)
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end)


def run_single(args):
    import torch

    pkg = load_package()
    from llm_infer_b200 import attention
    wl = pkg.workloads
    shape = wl.C2
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    hbm_peak, tflops_peak, peak_kind = measured_peaks()
    B, H, Hkv, D, T = shape.batch, shape.n_heads, shape.n_kv_heads, shape.head_dim, shape.kv_len
    if args.prefill_only:
        # small-footprint mode for profiler captures of the prefill kernel
        with ClockSampler(0) as clocks:
            res = prefill_measure(torch, attention, wl, args.steps, args.warmup, tflops_peak, peak_kind)
        print(json.dumps({"prefill": res, "clocks": clocks.summary()}), flush=True)
        return

    # Inputs: N(0,1) from a seeded generator, cast once to fp16. Three independent copies are rotated so that
    # consecutive steps never re-read a cache line that could still sit in the 126 MB L2.
    gen = torch.Generator(device=dev)
    gen.manual_seed(shape.seed)
    n_sets = 1 if args.kernel_only else 3
    qs = [torch.randn((B, H, D), generator=gen, device=dev, dtype=torch.float32).half() for _ in range(n_sets)]
    ks = [torch.randn((B, T, Hkv, D), generator=gen, device=dev, dtype=torch.float32).half() for _ in range(n_sets)]
    vs = [torch.randn((B, T, Hkv, D), generator=gen, device=dev, dtype=torch.float32).half() for _ in range(n_sets)]
    out = torch.empty((B, H, D), dtype=torch.float32, device=dev)
    ws = attention.DecodeWorkspace(B, H, Hkv, D, dev)

    def step(i):
        j = i % n_sets
        attention.attn_decode(qs[j], ks[j], vs[j], out=out, workspace=ws)

    for i in range(max(3, args.warmup)):
        step(i)
    torch.cuda.synchronize()

    launches0 = attention.kernel_launch_count()
    with ClockSampler(0) as clocks:
        ms = time_steps(torch, step, args.steps)
    launches = attention.kernel_launch_count() - launches0
    ms_per_step = ms / args.steps
    alg_bytes = shape.algorithmic_bytes(o_bytes=4)
    gbs = alg_bytes / (ms_per_step * 1e-3) / 1e9
    assert int(ws.status.item()) == 0, "device status word reports a timed-out wait"
    if args.kernel_only:
        # small-footprint mode for profiler captures: one input copy (256 MiB > L2), no host copies, no sweep
        print(json.dumps({"metric": "decode_attn_hbm_gbs", "value": gbs, "unit": "GB/s", "ms_per_step": ms_per_step,
                          "steps": args.steps, "config": workload_config(shape, 1), "kernel_only": True,
                          "gpu_launches": int(launches)}), flush=True)
        return

    # ---- end to end through the public API with host buffers. One decode step of the engine's attention block:
    # the token's fp32 q, k, v arrive from pinned host memory in one copy, attn_rope_kv_insert rotates q and k and
    # appends k, v (fp16) to the resident cache, attn_decode attends over it, and the output is copied back and the
    # stream synchronised before the next token. The KV cache itself stays in HBM, as the engine's per-layer cache does.
    n_q, n_kv = B * H * D, B * Hkv * D
    host_in = torch.randn(n_q + 2 * n_kv, dtype=torch.float32).pin_memory()
    pos_dev = torch.full((B,), T - 1, dtype=torch.int32, device=dev)
    out_host = torch.empty((B, H, D), dtype=torch.float32).pin_memory()
    # the public call: one captured graph per cache (copy in, rope + insert, decode, copy out), replayed and waited for
    host_steps = [attention.HostDecodeStep(host_in, ks[j], vs[j], pos_dev, pos_dev, out_host, n_heads=H, theta=500000.0,
                                           workspace=ws) for j in range(n_sets)]

    def e2e_step(i):
        host_steps[i % n_sets]()

    for i in range(3):
        e2e_step(i)
    e2e_steps = args.steps
    e2e_ms = time_steps(torch, e2e_step, e2e_steps) / e2e_steps
    h2d = host_in.numel() * 4
    d2h = out_host.numel() * 4
    e2e = {"value": alg_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
           "what": "attention.HostDecodeStep: fp32 q, k, v of the token copied from pinned host memory (one copy), "
                   "attn_rope_kv_insert + attn_decode through the C ABI, output copied back to pinned host memory - "
                   "one CUDA-graph launch per step, the stream synchronised every step; the KV cache itself stays "
                   "resident in HBM, as the engine's per-layer cache does"}
    q_host = qs[0].cpu().pin_memory()
    q_dev = torch.empty_like(qs[0])

    extra = {}
    # ---- the same call with NOTHING resident: whole KV cache copied from pinned host memory every step
    try:
        k_host = ks[0].cpu().pin_memory()
        v_host = vs[0].cpu().pin_memory()

        def cold_step(i):
            q_dev.copy_(q_host, non_blocking=True)
            ks[1].copy_(k_host, non_blocking=True)
            vs[1].copy_(v_host, non_blocking=True)
            attention.attn_decode(q_dev, ks[1], vs[1], out=out, workspace=ws)
            out_host.copy_(out, non_blocking=True)
            torch.cuda.current_stream().synchronize()

        cold_step(0)
        n_cold = min(args.steps, 5)
        cold_ms = time_steps(torch, cold_step, n_cold) / n_cold
        extra["e2e_cold_cache"] = {"value": alg_bytes / (cold_ms * 1e-3) / 1e9, "unit": "GB/s",
                                   "ms_per_step": cold_ms,
                                   "h2d_bytes_per_step": q_host.numel() * 2 + 2 * k_host.numel() * 2,
                                   "what": "whole KV cache copied host->device every step (PCIe-bound)"}
        del k_host, v_host
    except Exception as e:  # host memory for pinning may be short on some boxes; the headline does not depend on it
        extra["e2e_cold_cache"] = {"error": str(e)[:200]}

    # ---- KV-length sweep of the metric (B = 1 and 16), 4K .. 128K
    del ks, vs
    torch.cuda.empty_cache()
    sweep = []
    Tmax = 131072
    kbig = torch.randn((16, Tmax, Hkv, D), generator=gen, device=dev, dtype=torch.float16)
    vbig = torch.randn((16, Tmax, Hkv, D), generator=gen, device=dev, dtype=torch.float16)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    for b in (1, 16):
        ws_b = attention.DecodeWorkspace(b, H, Hkv, D, dev)
        out_b = torch.empty((b, H, D), dtype=torch.float32, device=dev)
        for t in (4096, 8192, 16384, 32768, 65536, 131072):
            s = wl.DecodeShape("sweep", 1, b, H, Hkv, D, t, "f16", "f16")
            kv_bytes = s.kv_bytes
            reps = 5
            best = None
            starts = [torch.cuda.Event(enable_timing=True) for _ in range(reps)]
            ends = [torch.cuda.Event(enable_timing=True) for _ in range(reps)]
            for r in range(reps + 2):
                if kv_bytes < 400e6:
                    flush.zero_()  # working set smaller than ~3x L2: flush L2 between iterations
                if r >= 2:
                    starts[r - 2].record()
                attention.attn_decode(qs[0][:b], kbig[:b], vbig[:b], t, out=out_b, workspace=ws_b)
                if r >= 2:
                    ends[r - 2].record()
            torch.cuda.synchronize()
            times = sorted(starts[i].elapsed_time(ends[i]) for i in range(reps))
            med = times[reps // 2]
            best = times[0]
            point = {"batch": b, "kv_len": t, "us": round(med * 1e3, 2), "us_best": round(best * 1e3, 2),
                     "gbs": round(s.algorithmic_bytes() / (med * 1e-3) / 1e9, 1),
                     "frac_of_peak": round(s.algorithmic_bytes() / (med * 1e-3) / 1e9 / hbm_peak, 3),
                     "tok_per_s": round(b / (med * 1e-3), 1)}
            if b == 1:
                # The same call in a chain, as the headline step is timed: the 16 sequences of the buffer in turn
                # (16 x kv_bytes >= 256 MB, nothing is found in L2), captured in one CUDA graph so that no host launch
                # cost and no event pair per call is in the figure; consecutive calls overlap through their launch chain.
                g = torch.cuda.CUDAGraph()
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side), torch.cuda.graph(g):
                    for i in range(16):
                        attention.attn_decode(qs[0][:1], kbig[i:i + 1], vbig[i:i + 1], t, out=out_b, workspace=ws_b)
                torch.cuda.current_stream().wait_stream(side)
                g.replay()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(5):
                    g.replay()
                e1.record()
                torch.cuda.synchronize()
                loop_ms = e0.elapsed_time(e1) / 80
                point["chain_us"] = round(loop_ms * 1e3, 2)
                point["chain_frac_of_peak"] = round(s.algorithmic_bytes() / (loop_ms * 1e-3) / 1e9 / hbm_peak, 3)
            sweep.append(point)
    try:
        extra["prefill_c3"] = prefill_measure(torch, attention, wl, 20, 3, tflops_peak, peak_kind)
    except Exception as e:
        extra["prefill_c3"] = {"error": str(e)[:200]}
    extra["kv_sweep"] = {"timing": "us = median of 5 single calls, each between its own pair of CUDA events (the pair "
                                   "alone reads 5 - 6 us), L2 flushed when KV < 400 MB; chain_us (batch 1) = the call "
                                   "in a chain of 80 over 16 different sequences, one CUDA graph",
                         "points": sweep}
    del kbig, vbig, flush
    torch.cuda.empty_cache()
    try:
        extra["gemv_layer"] = gemv_measure(torch, 60, 6, hbm_peak, peak_kind)
    except Exception as e:
        extra["gemv_layer"] = {"error": str(e)[:300]}
    try:
        extra["attention_symbol"] = attention_symbol_measure(torch, hbm_peak)
    except Exception as e:
        extra["attention_symbol"] = {"error": str(e)[:300]}
    try:
        extra["prompt_gemm"] = gemm_measure(torch, 10, 3, tflops_peak, peak_kind)
    except Exception as e:
        extra["prompt_gemm"] = {"error": str(e)[:300]}
    try:
        extra["generate_c5"] = generate_measure(torch)
    except Exception as e:
        extra["generate_c5"] = {"error": str(e)[:300]}

    # ---- CPU baseline on the host cores of this box (bounded sample)
    try:
        _, cpu_desc, _ = cpu_reference_arm(wl, shape, steps=200, warmup=2, seconds_budget=15.0)
        cpu_baseline = {k: cpu_desc[k] for k in ("value", "unit", "cores", "kind", "sample")}
    except Exception as e:
        cpu_baseline = {"value": None, "unit": "GB/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"[:200]}

    line = {
        "metric": "decode_attn_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 storage, f32 accumulate", "data": "synthetic",
        "config": workload_config(shape, 1),
        "l2": f"inputs {shape.kv_bytes >> 20} MiB per step > 126 MB L2, {n_sets} input copies rotated",
        "tok_per_s": B / (ms_per_step * 1e-3),
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gbs / hbm_peak,
                     "traffic": ncu_traffic_bytes(), "peak_kind": f"of {peak_kind}",
                     "frac_of_nominal_8tbs": gbs / 8000.0, "algorithmic_bytes_per_launch": alg_bytes,
                     "note": "duration = CUDA-event time of one step (split pass + merge pass) / steps"},
        "cpu_baseline": cpu_baseline,
        "e2e": e2e,
        "gpu_launches": int(launches),
        "clocks": clocks.summary(),
        "extra": extra,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- our arm, N GPUs
def run_multi(args, world: int, rank: int, local_rank: int):
    import numpy as np
    import torch
    import torch.distributed as dist

    pkg = load_package()
    from llm_infer_b200 import attention
    from llm_infer_b200.sharded import FusedShardedDecode, ShardedDecode, shard_rows
    wl = pkg.workloads
    shape = wl.C4
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    hbm_peak, _, peak_kind = measured_peaks()
    H, Hkv, D, T = shape.n_heads, shape.n_kv_heads, shape.head_dim, shape.kv_len
    r0, r1 = shard_rows(T, world, rank)
    rows = r1 - r0

    # The workload's own seeded inputs, generated on the host by every rank (so the CPU checker on rank 0 sees exactly
    # the rows the GPUs hold); each rank keeps rows [r0, r1). Further copies of the shard (device-generated noise of
    # the same shape) are rotated through so that a timed step never finds its rows in L2; copy 0 is the real one.
    q_np, k_np, v_np = wl.decode_inputs(shape)
    q = torch.from_numpy(q_np).to(dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(shape.seed * 1000 + rank + 1)
    n_sets = max(2, min(8, int(400e6 // (2 * rows * Hkv * D * 2)) + 1))
    ks = [torch.from_numpy(np.ascontiguousarray(k_np[:, r0:r1])).to(dev)]
    vs = [torch.from_numpy(np.ascontiguousarray(v_np[:, r0:r1])).to(dev)]
    for _ in range(n_sets - 1):
        ks.append(torch.randn((1, rows, Hkv, D), generator=gen, device=dev, dtype=torch.float16))
        vs.append(torch.randn((1, rows, Hkv, D), generator=gen, device=dev, dtype=torch.float16))
    if rank != 0:
        del k_np, v_np
    out = torch.empty((1, H, D), dtype=torch.float32, device=dev)

    def agree(ok: bool) -> bool:
        flag = torch.tensor([1.0 if ok else 0.0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        return flag.item() >= 1

    def timed(fn, n):
        """CUDA-event time per call in ms, max over ranks."""
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        dist.barrier()
        x = torch.tensor([time_steps(torch, fn, n) / n], device=dev)
        dist.all_reduce(x, op=dist.ReduceOp.MAX)
        return float(x.item())

    # ---- path A: NCCL all-gather between the local decode and the merge (three launches + one collective)
    nccl = ShardedDecode(H, D, device=dev)
    ws_local = attention.DecodeWorkspace(1, H, Hkv, D, dev)
    nccl.use_workspace(ws_local)
    out_a = out.view(H, D)
    for i in range(max(3, args.warmup)):
        nccl(q, ks[i % n_sets], vs[i % n_sets], out=out_a)
    torch.cuda.synchronize()
    paths = {"nccl_allgather_eager_ms": timed(lambda i: nccl(q, ks[i % n_sets], vs[i % n_sets], out=out_a), args.steps)}
    parts = {"local_decode_us": 1e3 * timed(lambda i: nccl.local_partial(q, ks[i % n_sets], vs[i % n_sets]), 50),
             "all_gather_us": 1e3 * timed(lambda i: nccl.gather(), 50),
             "merge_us": 1e3 * timed(lambda i: nccl.merge(out=out_a), 50)}

    # ---- path B (the product path): exchange fused into the merge kernel over peer memory, two launches per step,
    #      replayed from CUDA graphs (one per input copy) the way the engine replays its decode graph
    step, launch_mode, graphs = None, "nccl-allgather, eager", None
    try:
        fused = FusedShardedDecode(1, H, Hkv, D, device=dev, kv_early=not args.no_sharded_kv_early)
        ok = True
    except Exception as e:  # no peer-mapped memory on this box: stay on path A
        fused, ok = None, False
        paths["fused_error"] = str(e)[:200]
    if agree(ok):
        def fused_step(i):
            fused(q, ks[i % n_sets], vs[i % n_sets], out=out)
        for i in range(max(3, args.warmup)):
            fused_step(i)
        torch.cuda.synchronize()
        paths["fused_peer_store_eager_ms"] = timed(fused_step, args.steps)
        step, launch_mode = fused_step, "fused peer-store exchange, eager"
        try:
            graphs = [fused.capture(q, ks[j], vs[j], out) for j in range(n_sets)]
            ok = True
        except Exception:
            graphs, ok = None, False
        if agree(ok):
            def graph_step(i):
                graphs[i % n_sets].replay()
            paths["fused_peer_store_graph_ms"] = timed(graph_step, args.steps)
            # Both are the product path; consecutive eager steps overlap through the dependent-launch chain, separate
            # graph launches do not, so the faster one (the same on every rank: the times are maxima over ranks) is timed.
            if paths["fused_peer_store_graph_ms"] <= paths["fused_peer_store_eager_ms"]:
                step, launch_mode = graph_step, "fused peer-store exchange, CUDA-graph replay"
        else:
            graphs = None
    else:
        fused = None
    if step is None:
        def step(i):
            nccl(q, ks[i % n_sets], vs[i % n_sets], out=out_a)

    for i in range(max(3, args.warmup)):
        step(i)
    torch.cuda.synchronize()
    dist.barrier()
    launches0 = attention.kernel_launch_count()
    with ClockSampler(local_rank) as clocks:
        dist.barrier()
        ms = time_steps(torch, step, args.steps)
    launches = attention.kernel_launch_count() - launches0
    if graphs is not None and "graph" in launch_mode:
        launches = 2 * args.steps  # split pass + merge/exchange pass per replay (replays bypass the host-side counter)
    t = torch.tensor([ms], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    status_ok = fused is None or int(fused.workspace.status.item()) == 0

    # ---- the fused step itemised: the local part alone (split pass + local merge, no exchange) against the whole
    #      step; what the exchange and the cross-rank merge add is the difference
    local_only_us = 1e3 * timed(lambda i: attention.attn_decode(q, ks[i % n_sets], vs[i % n_sets], out=out,
                                                                workspace=ws_local), 50)
    fused_items = {"local_split_and_merge_us": local_only_us, "whole_step_us": ms_per_step * 1e3,
                   "exchange_and_cross_merge_us": ms_per_step * 1e3 - local_only_us,
                   "streaming_floor_us": 2 * rows * Hkv * D * 2 / (hbm_peak * 1e3)}

    # ---- parity, outside the timed region: the product path on the real rows (copy 0) against the engine's CPU
    #      attn() over the UNSHARDED sequence; every rank's output is checked on rank 0
    out.fill_(float("nan"))
    if fused is not None:
        fused(q, ks[0], vs[0], out=out)
    else:
        nccl(q, ks[0], vs[0], out=out_a)
    torch.cuda.synchronize()
    gathered = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered, out)
    parity = None
    if rank == 0:
        import oracle
        chk = oracle.best()
        chk.set_num_threads(None)
        want = chk.attn_decode(wl.widen(q_np, shape.q_dtype), k_np, v_np)
        errs = [wl.error_metrics(g.cpu().numpy(), want) for g in gathered]
        max_abs, max_rel = max(e[0] for e in errs), max(e[1] for e in errs)
        finite = all(bool(torch.isfinite(g).all()) for g in gathered)
        parity = {"max_abs": max_abs, "max_rel": max_rel, "abs_tol": wl.ABS_TOL, "rel_tol": wl.REL_TOL,
                  "ok": bool(finite and max_abs <= wl.ABS_TOL and max_rel <= wl.REL_TOL), "ranks_checked": world,
                  "checker": f"{chk.kind} attn() over all {T} rows on {chk.num_threads()} host threads",
                  "rel_definition": "|a-b| / max(|b|, 1e-2*rms(b))"}

    # ---- the same workload on ONE GPU, timed by rank 0 in this process while the other ranks wait: the like-for-like
    #      point for strong scaling (two copies of the whole sequence rotated, 512 MiB each > L2)
    strong = None
    if rank == 0:
        del ks, vs
        torch.cuda.empty_cache()
        kf = [torch.from_numpy(k_np).to(dev)]
        vf = [torch.from_numpy(v_np).to(dev)]
        kf.append(torch.randn((1, T, Hkv, D), generator=gen, device=dev, dtype=torch.float16))
        vf.append(torch.randn((1, T, Hkv, D), generator=gen, device=dev, dtype=torch.float16))
        out1 = torch.empty((1, H, D), dtype=torch.float32, device=dev)
        for i in range(4):
            attention.attn_decode(q, kf[i % 2], vf[i % 2], out=out1, workspace=ws_local)
        n1 = max(20, min(args.steps, 100))
        t1_ms = time_steps(torch, lambda i: attention.attn_decode(q, kf[i % 2], vf[i % 2], out=out1,
                                                                  workspace=ws_local), n1) / n1
        attention.attn_decode(q, kf[0], vf[0], out=out1, workspace=ws_local)
        torch.cuda.synchronize()
        e1 = wl.error_metrics(out1.cpu().numpy(), want)
        strong = {"workload": shape.name, "t1_us": t1_ms * 1e3, "tN_us": ms_per_step * 1e3, "n_gpus": world,
                  "speedup": t1_ms / ms_per_step, "efficiency": t1_ms / ms_per_step / world,
                  "t1_parity": {"max_abs": e1[0], "max_rel": e1[1]},
                  "note": "t1 = the whole sequence on one GPU (attn_decode, same process, same clocks), "
                          "tN = this line's ms_per_step"}
        del kf, vf
    dist.barrier()

    # end to end with host buffers: q from pinned host memory, result read back, every step
    if rank == 0:
        ks = [torch.from_numpy(np.ascontiguousarray(k_np[:, r0:r1])).to(dev)]
        vs = [torch.from_numpy(np.ascontiguousarray(v_np[:, r0:r1])).to(dev)]
        n_sets_e2e = 1
    else:
        n_sets_e2e = n_sets
    n_sets_e2e = int(torch.tensor([n_sets_e2e], device=dev).item())
    q_host = q.cpu().pin_memory()
    out_host = torch.empty((1, H, D), dtype=torch.float32).pin_memory()

    def e2e_step(i):
        q.copy_(q_host, non_blocking=True)
        j = i % n_sets_e2e
        if fused is not None:
            fused(q, ks[j], vs[j], out=out)
        else:
            nccl(q, ks[j], vs[j], out=out_a)
        out_host.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_ms = timed(e2e_step, args.steps)

    alg_bytes = shape.algorithmic_bytes(o_bytes=4)
    gbs = alg_bytes / (ms_per_step * 1e-3) / 1e9
    if rank == 0:
        line = {
            "metric": "decode_attn_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16 storage, f32 accumulate", "data": "synthetic",
            "config": workload_config(shape, world),
            "exchange": launch_mode,
            "kv_early": not args.no_sharded_kv_early,
            "l2": f"{rows * Hkv * D * 4 >> 20} MiB of KV per GPU per step, {n_sets} copies rotated",
            "tok_per_s": 1.0 / (ms_per_step * 1e-3),
            "parity": parity,
            "roofline": {"bound": "hbm", "achieved": gbs / world, "peak": hbm_peak, "unit": "GB/s",
                         "frac": gbs / world / hbm_peak, "traffic": None, "peak_kind": f"of {peak_kind}",
                         "note": "per GPU: algorithmic bytes / N / step time (local decode + exchange + merge)"},
            "e2e": {"value": alg_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": q.numel() * 2,
                    "d2h_bytes_per_step": H * D * 4, "ms_per_step": e2e_ms,
                    "what": "q copied from pinned host memory, the sharded decode step, the result copied back and "
                            "the stream synchronised, every step (eager launches)"},
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "extra": {"strong_scaling": strong, "fused_path_breakdown": fused_items, "paths_ms_per_step": paths,
                      "nccl_path_breakdown": parts, "status_ok": status_ok},
        }
        print(json.dumps(line), flush=True)
    ok = agree(rank != 0 or (parity is not None and parity["ok"] and status_ok))
    dist.barrier()
    torch.cuda.synchronize()
    # Tearing the process group down while captured graphs or symmetric-memory handles are alive can block;
    # the line is printed, so leave directly (non-zero when the result was outside the tolerance).
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0 if ok else 1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--prefill-only", action="store_true",
                    help="time only the causal-prefill workload (used for profiler captures)")
    ap.add_argument("--gemv-only", action="store_true",
                    help="time only the weight GEMVs of one layer (fp16 and Q8_0; used for profiler captures)")
    ap.add_argument("--no-sharded-kv-early", action="store_true",
                    help="with --gpus N > 1: do not let the local pass stream K/V rows ahead of the previous kernel "
                         "(by default it does: between the steps of this workload no cache row changes, and in the "
                         "engine only each sequence's newest row would)")
    ap.add_argument("--symbol-only", action="store_true",
                    help="time only the engine's attention kernel symbol (used for profiler captures)")
    ap.add_argument("--gemv-kinds", default="",
                    help="with --gemv-only: comma-separated subset of q8_0,q8_0_tiled,f16")
    ap.add_argument("--generate-only", action="store_true",
                    help="run only the end-to-end greedy generation workload (Q8_0 8B-shaped model) and print it")
    ap.add_argument("--generate-eager", action="store_true",
                    help="with --generate-only: launch every kernel from the host instead of replaying CUDA graphs")
    ap.add_argument("--generate-short", action="store_true",
                    help="with --generate-only: prompts of 8-16 tokens and 8 new tokens (for profiler launch lists)")
    ap.add_argument("--gemm-only", action="store_true",
                    help="time only the whole-prompt projection GEMM (with --steps <= 5: one 4096^3 case, for profiler captures)")
    ap.add_argument("--decode-trace", action="store_true",
                    help="per-CTA time stamps of one attn_decode call (needs the profiling build, see decode_trace)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="time only the resident-input steps of the 1-GPU workload (used for profiler captures)")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, max(world, args.gpus), rank)
        return
    if args.decode_trace:
        import torch
        load_package()
        decode_trace(torch)
        return
    if args.gemm_only:
        import torch
        load_package()
        _, tflops_peak, peak_kind = measured_peaks()
        print(json.dumps({"prompt_gemm": gemm_measure(torch, args.steps, args.warmup, tflops_peak, peak_kind,
                                                      small=args.steps <= 5)}), flush=True)
        return
    if args.symbol_only:
        import torch
        load_package()
        hbm_peak, _, _ = measured_peaks()
        print(json.dumps({"attention_symbol": attention_symbol_measure(torch, hbm_peak)}), flush=True)
        return
    if args.gemv_only:
        import torch
        load_package()
        hbm_peak, _, peak_kind = measured_peaks()
        print(json.dumps({"gemv_layer": gemv_measure(torch, args.steps, args.warmup, hbm_peak, peak_kind,
                                                     args.gemv_kinds.split(",") if args.gemv_kinds else None)}),
              flush=True)
        return
    if args.generate_only:
        import torch
        load_package()
        kw = {"n_new": 8, "prompt_range": (8, 16)} if args.generate_short else {}
        kw["graph"] = not args.generate_eager
        print(json.dumps({"generate_c5": generate_measure(torch, **kw)}), flush=True)
        return
    if world == 1 and args.gpus == 1:
        run_single(args)
    elif world > 1:
        run_multi(args, world, rank, local_rank)
    else:
        raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one process per GPU)")


if __name__ == "__main__":
    main()
