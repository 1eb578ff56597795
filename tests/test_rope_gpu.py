"""GPU parity of the fused rotary-embedding + KV-cache-insert kernel against the engine's CPU code
(include/kernels_cpu.hpp:82-120 driven as in src/model/block.cpp:140-155). Floating point: rotated q within
2e-6 relative of the fp32 CPU result; fp16 cache contents within one fp16 step, and bit-equal for more than 99 %
of the elements (the CPU and GPU cos/sin differ in the last bit for some angles)."""
import ctypes as C
import os

import numpy as np
import pytest

from conftest import GOLDEN

pytestmark = pytest.mark.gpu


def _host_inv_freq(theta, rot):
    libm = C.CDLL("libm.so.6")
    libm.powf.restype = C.c_float
    libm.powf.argtypes = [C.c_float, C.c_float]
    return np.array([np.float32(1.0) / np.float32(libm.powf(theta, np.float32(i) / np.float32(rot)))
                     for i in range(0, rot, 2)], dtype=np.float32)


def _fp16_steps(a, b):
    return np.abs(a.view(np.int16).astype(np.int32) - b.view(np.int16).astype(np.int32))


@pytest.fixture(scope="module")
def attention(built_lib, pkg):
    from llm_infer_b200 import attention as a
    return a


def test_golden_vectors(attention):
    import torch
    g = np.load(os.path.join(GOLDEN, "rope_golden.npz"))
    for name in ("early", "window", "late"):
        pos, kv_pos, sink, theta = g[f"{name}.args"]
        dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
        kc, vc = dev(g[f"{name}.k_cache_in"][None]), dev(g[f"{name}.v_cache_in"][None])
        inv = dev(_host_inv_freq(float(theta), 64))
        q_out = attention.rope_kv_insert(dev(g[f"{name}.q"][None]), dev(g[f"{name}.k"][None]), dev(g[f"{name}.v"][None]),
                                         kc, vc, dev(np.array([pos], np.int32)), dev(np.array([kv_pos], np.int32)),
                                         theta=float(theta), kv_sink=int(sink), inv_freq=inv)
        torch.cuda.synchronize()
        want = g[f"{name}.q_out"]
        assert np.abs(q_out[0].cpu().numpy() - want).max() <= 2e-6 * max(1.0, np.abs(want).max())
        for got, ref in ((kc, g[f"{name}.k_cache_out"]), (vc, g[f"{name}.v_cache_out"])):
            d = _fp16_steps(got[0].cpu().numpy(), ref)
            assert d.max() <= 1 and (d != 0).mean() < 0.01, name


@pytest.mark.parametrize("use_host_freq", [True, False])
def test_batch_against_cpu_per_sequence(attention, checker, use_host_freq):
    import torch
    rng = np.random.default_rng(17)
    B, H, Hkv, D, T, theta = 5, 32, 8, 128, 40, 500000.0
    pos = np.array([0, 1, 777, 4096, 100000], np.int32)
    kv_pos = np.array([0, 1, 17, 39, 21], np.int32)
    sink = 4
    q = rng.standard_normal((B, H, D), dtype=np.float32)
    k = rng.standard_normal((B, Hkv, D), dtype=np.float32)
    v = rng.standard_normal((B, Hkv, D), dtype=np.float32)
    kc = rng.standard_normal((B, T, Hkv, D), dtype=np.float32).astype(np.float16)
    vc = rng.standard_normal((B, T, Hkv, D), dtype=np.float32).astype(np.float16)
    kc[:, :, :, :] = kc  # dense
    kc_d, vc_d = torch.from_numpy(kc.copy()).cuda(), torch.from_numpy(vc.copy()).cuda()
    # sequences whose new row is a sink row cannot occur in the engine (kv_pos >= kv_sink once sinks are active):
    # keep kv_pos >= sink for the sequences that use sinks by calling the kernel with sink = 0 for the early ones
    for use_sink, rows in ((0, [0, 1]), (sink, [2, 3, 4])):
        idx = np.array(rows)
        inv = torch.from_numpy(_host_inv_freq(theta, D)).cuda() if use_host_freq else None
        q_out = attention.rope_kv_insert(torch.from_numpy(q[idx]).cuda(), torch.from_numpy(k[idx]).cuda(),
                                         torch.from_numpy(v[idx]).cuda(), kc_d[idx[0]:idx[-1] + 1], vc_d[idx[0]:idx[-1] + 1],
                                         torch.from_numpy(pos[idx]).cuda(), torch.from_numpy(kv_pos[idx]).cuda(),
                                         theta=theta, kv_sink=use_sink, inv_freq=inv, q_out_dtype=torch.float32)
        torch.cuda.synchronize()
        for n, b in enumerate(rows):
            kc_ref, vc_ref = kc[b].copy(), vc[b].copy()
            q_ref, _ = checker.rope_kv_insert(q[b], k[b], v[b], kc_ref, vc_ref, int(pos[b]), int(kv_pos[b]), use_sink, theta)
            got_q = q_out[n].cpu().numpy()
            # device-evaluated frequencies may differ from the host's powf in the last bit: at position 1e5 that moves
            # the angle by up to ~1e-2 rad for the fastest pairs, as it would between any two libm versions
            tol = 2e-6 if use_host_freq or pos[b] < 1000 else 5e-2
            assert np.abs(got_q - q_ref).max() <= tol * max(1.0, np.abs(q_ref).max()), (b, use_host_freq)
            if use_host_freq:
                for got, ref in ((kc_d[b], kc_ref), (vc_d[b], vc_ref)):
                    d = _fp16_steps(got.cpu().numpy(), ref)
                    assert d.max() <= 1 and (d != 0).mean() < 0.01, b
            else:
                assert np.array_equal(vc_d[b].cpu().numpy().view(np.uint16), vc_ref.view(np.uint16))


def test_rotated_q_feeds_decode_attention(attention, checker, pkg):
    """End of the chain: rope + insert, then decode attention over the updated cache, against the same chain on the CPU."""
    import torch
    wl = pkg.workloads
    rng = np.random.default_rng(23)
    H, Hkv, D, T, theta = 32, 8, 128, 300, 500000.0
    q = rng.standard_normal((1, H, D), dtype=np.float32)
    k = rng.standard_normal((1, Hkv, D), dtype=np.float32)
    v = rng.standard_normal((1, Hkv, D), dtype=np.float32)
    kc = rng.standard_normal((1, T, Hkv, D), dtype=np.float32).astype(np.float16)
    vc = rng.standard_normal((1, T, Hkv, D), dtype=np.float32).astype(np.float16)
    pos = kv_pos = 199
    kc_d, vc_d = torch.from_numpy(kc.copy()).cuda(), torch.from_numpy(vc.copy()).cuda()
    q_rot = attention.rope_kv_insert(torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(),
                                     kc_d, vc_d, torch.tensor([pos], dtype=torch.int32, device="cuda"),
                                     torch.tensor([kv_pos], dtype=torch.int32, device="cuda"), theta=theta,
                                     inv_freq=torch.from_numpy(_host_inv_freq(theta, D)).cuda())
    out = attention.attn_decode(q_rot, kc_d, vc_d, pos + 1)
    torch.cuda.synchronize()
    kc_ref, vc_ref = kc[0].copy(), vc[0].copy()
    q_ref, _ = checker.rope_kv_insert(q[0], k[0], v[0], kc_ref, vc_ref, pos, kv_pos, 0, theta)
    want = checker.attn_decode(q_ref[None], kc_ref[None], vc_ref[None], np.array([pos + 1], np.uint32))
    max_abs, max_rel = wl.error_metrics(out.cpu().numpy(), want)
    assert max_abs <= wl.ABS_TOL and max_rel <= wl.REL_TOL, (max_abs, max_rel)


def test_host_decode_step_graph_matches_the_eager_calls(built_lib, pkg):
    """attention.HostDecodeStep (copy in, rope + insert, decode, copy out as one graph launch) against the same calls
    made one by one; the pinned input is rewritten between replays, so the graph must re-read it every time."""
    import torch
    from llm_infer_b200 import attention as A
    B, H, Hkv, D, T = 3, 8, 2, 128, 96
    g = torch.Generator().manual_seed(5)
    k_cache = torch.randn(B, T, Hkv, D, generator=g).half().cuda()
    v_cache = torch.randn(B, T, Hkv, D, generator=g).half().cuda()
    k_ref, v_ref = k_cache.clone(), v_cache.clone()
    pos = torch.tensor([40, 95, 7], dtype=torch.int32).cuda()
    kv_len = (pos + 1).to(torch.int32)
    host_in = torch.zeros(B * H * D + 2 * B * Hkv * D).pin_memory()
    out_host = torch.zeros(B, H, D).pin_memory()
    step = A.HostDecodeStep(host_in, k_cache, v_cache, pos, pos, out_host, n_heads=H, theta=10000.0, kv_len=kv_len)
    for trial in range(2):
        fresh = torch.randn(host_in.numel(), generator=g)
        host_in.copy_(fresh)
        got = step().clone()
        dev = fresh.cuda()
        n_q, n_kv = B * H * D, B * Hkv * D
        q = A.rope_kv_insert(dev[:n_q].view(B, H, D), dev[n_q:n_q + n_kv].view(B, Hkv, D),
                             dev[n_q + n_kv:].view(B, Hkv, D), k_ref, v_ref, pos, pos, theta=10000.0,
                             q_out_dtype=torch.float16)
        want = A.attn_decode(q, k_ref, v_ref, kv_len).cpu()
        assert torch.equal(got, want), trial
        assert torch.equal(k_cache, k_ref) and torch.equal(v_cache, v_ref)
