"""GPU parity of the split-KV decode path, called through the C ABI, against the
CPU checker (the engine's attn(), include/kernels_cpu.hpp:140-167) on identical
seeded inputs. Tolerance: max abs 2e-3, max rel 1e-2 (relative error measured
against max(|ref|, 1% of the RMS of ref))."""
import os

import numpy as np
import pytest

from conftest import GOLDEN

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def attention(built_lib, pkg):
    import torch
    assert torch.cuda.is_available()
    from llm_infer_b200 import attention as a
    return a


@pytest.fixture(scope="module")
def wl(pkg):
    return pkg.workloads


def _rand(wl, seed, B, H, Hkv, D, T, q_dtype="f32", kv_dtype="f16"):
    shape = wl.DecodeShape("t", seed, B, H, Hkv, D, T, q_dtype, kv_dtype)
    return wl.decode_inputs(shape)


def _oracle(wl, checker, q, k, v, q_dtype, kv_dtype, kv_len=None):
    return checker.attn_decode(wl.widen(q, q_dtype), wl.as_f16_for_oracle(k, kv_dtype),
                               wl.as_f16_for_oracle(v, kv_dtype),
                               None if kv_len is None else np.asarray(kv_len, np.uint32))


def test_golden_vectors(attention, wl):
    from gpu_util import check_close, run_decode
    g = np.load(os.path.join(GOLDEN, "decode_golden.npz"))
    for name in sorted({k.split(".")[0] for k in g.files}):
        lens = g[f"{name}.kv_len"]
        got = run_decode(attention, g[f"{name}.q"], g[f"{name}.k"], g[f"{name}.v"], kv_len=lens)
        check_close(wl, got, g[f"{name}.o"], name)


def test_c1_tinyllama_shape(attention, wl, checker):
    from gpu_util import check_close, run_decode
    q, k, v = wl.decode_inputs(wl.C1)
    got = run_decode(attention, q, k, v)
    check_close(wl, got, checker.attn_decode(q, k, v), "C1")


def test_c2_llama3_batched_full_size(attention, wl, checker):
    from gpu_util import check_close, run_decode
    q, k, v = wl.decode_inputs(wl.C2)
    got = run_decode(attention, q, k, v, q_dtype="f16")
    want = checker.attn_decode(q.astype(np.float32), k, v)
    max_abs, max_rel = check_close(wl, got, want, "C2")
    print(f"C2 max_abs={max_abs:.3e} max_rel={max_rel:.3e}")


def test_c4_long_context_single_gpu(attention, wl, checker):
    from gpu_util import check_close, run_decode
    q, k, v = wl.decode_inputs(wl.C4)
    got, lse = run_decode(attention, q, k, v, q_dtype="f16", lse=True)
    want = checker.attn_decode(q.astype(np.float32), k, v)
    max_abs, max_rel = check_close(wl, got, want, "C4")
    print(f"C4 max_abs={max_abs:.3e} max_rel={max_rel:.3e}")
    assert np.isfinite(lse).all()


@pytest.mark.parametrize("kv_len", [1, 2, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 257, 1000, 4095, 4097])
def test_edge_lengths(attention, wl, checker, kv_len):
    from gpu_util import check_close, run_decode
    q, k, v = _rand(wl, 100 + kv_len, 2, 32, 8, 128, kv_len)
    got = run_decode(attention, q, k, v)
    check_close(wl, got, _oracle(wl, checker, q, k, v, "f32", "f16"), f"kv_len={kv_len}")


@pytest.mark.parametrize("H,Hkv,D", [(4, 4, 64), (8, 1, 128), (8, 2, 64), (16, 4, 128), (32, 4, 64), (64, 8, 128),
                                     (32, 2, 128), (16, 16, 64), (48, 24, 128), (12, 6, 64), (5, 5, 128)])
def test_head_configurations(attention, wl, checker, H, Hkv, D):
    from gpu_util import check_close, run_decode
    q, k, v = _rand(wl, H * 1000 + Hkv * 10 + D, 3, H, Hkv, D, 333)
    got = run_decode(attention, q, k, v)
    check_close(wl, got, _oracle(wl, checker, q, k, v, "f32", "f16"), f"H={H} Hkv={Hkv} D={D}")


def test_ragged_batch_including_empty_sequence(attention, wl, checker):
    from gpu_util import check_close, run_decode
    lens = [1, 700, 0, 64, 699, 5, 333, 128]
    q, k, v = _rand(wl, 7, len(lens), 32, 8, 128, 700)
    got, lse = run_decode(attention, q, k, v, kv_len=lens, lse=True)
    want = _oracle(wl, checker, q, k, v, "f32", "f16", lens)
    check_close(wl, got, want, "ragged")
    assert np.array_equal(got[2], np.zeros_like(got[2]))  # empty sequence -> zeros, as the CPU loop gives
    assert np.isneginf(lse[2]).all() and np.isfinite(np.delete(lse, 2, axis=0)).all()


@pytest.mark.parametrize("q_dtype,kv_dtype,out_dtype", [("f16", "f16", "f32"), ("bf16", "f16", "f32"),
                                                         ("f32", "bf16", "f32"), ("bf16", "bf16", "bf16"),
                                                         ("f16", "f16", "f16")])
def test_dtypes(attention, wl, checker, q_dtype, kv_dtype, out_dtype):
    from gpu_util import run_decode
    q, k, v = _rand(wl, 11, 2, 32, 8, 128, 777, q_dtype, kv_dtype)
    got = run_decode(attention, q, k, v, q_dtype=q_dtype, kv_dtype=kv_dtype, out_dtype=out_dtype)
    want = _oracle(wl, checker, q, k, v, q_dtype, kv_dtype)
    max_abs, max_rel = wl.error_metrics(got, want)
    # 16-bit outputs carry their own rounding (bf16: 2^-9 relative)
    rel_tol = {"f32": wl.REL_TOL, "f16": wl.REL_TOL, "bf16": 1.5e-2}[out_dtype]
    assert max_abs <= wl.ABS_TOL and max_rel <= rel_tol, (max_abs, max_rel)


def test_lse_output(attention, wl, port):
    from gpu_util import run_decode
    q, k, v = _rand(wl, 12, 1, 8, 2, 64, 200)
    _, lse = run_decode(attention, q, k, v, lse=True)
    for h in (0, 3, 7):
        m, z, _ = port.state_from_rows(q[0, h], k[0], v[0], h // 4, 0, 200)
        assert abs(lse[0, h] - (m + np.log(z))) < 1e-4


def test_strided_cache_with_spare_capacity(attention, wl, checker):
    """Cache rows wider than n_kv_heads*head_dim and longer than kv_len, as a preallocated cache has."""
    import torch
    from gpu_util import check_close, to_device
    B, H, Hkv, D, T, cap = 2, 32, 8, 128, 300, 512
    q, k, v = _rand(wl, 13, B, H, Hkv, D, T)
    kbig = torch.zeros((B, cap, Hkv + 1, D), dtype=torch.float16, device="cuda")
    vbig = torch.full((B, cap, Hkv + 1, D), float("nan"), dtype=torch.float16, device="cuda")
    kbig[:, :T, :Hkv] = to_device(k, "f16")
    vbig[:, :T, :Hkv] = to_device(v, "f16")
    out = attention.attn_decode(to_device(q, "f32"), kbig[:, :, :Hkv], vbig[:, :, :Hkv], T)
    torch.cuda.synchronize()
    check_close(wl, out.cpu().numpy(), checker.attn_decode(q, k, v), "strided")


def test_bitwise_deterministic_and_canaries(attention, wl):
    import torch
    from gpu_util import to_device
    q, k, v = _rand(wl, 14, 4, 32, 8, 128, 1500)
    qd, kd, vd = to_device(q, "f32"), to_device(k, "f16"), to_device(v, "f16")
    ws = attention.DecodeWorkspace(4, 32, 8, 128)
    padded = torch.full((4 * 32 * 128 + 512,), float("nan"), dtype=torch.float32, device="cuda")
    out = padded[256:256 + 4 * 32 * 128].view(4, 32, 128)
    attention.attn_decode(qd, kd, vd, out=out, workspace=ws)
    first = out.clone()
    for _ in range(3):
        attention.attn_decode(qd, kd, vd, out=out, workspace=ws)
        assert torch.equal(out, first)
    torch.cuda.synchronize()
    assert torch.isnan(padded[:256]).all() and torch.isnan(padded[-256:]).all()  # nothing written outside o
    assert int(ws.status.item()) == 0


def test_early_streaming_after_an_appending_kernel(attention, wl, checker):
    """kv_early: the split pass may start its K/V copies before the kernel in front of it (here the rotary kernel that
    appends the token's row) has finished, for every tile that cannot hold that row. Back-to-back steps through the
    programmatic-launch chain, ragged and uniform lengths, must give the result of the plain call and of the CPU."""
    import torch
    from gpu_util import check_close, to_device
    B, H, Hkv, D, T = 3, 32, 8, 128, 700
    q, k, v = _rand(wl, 77, B, H, Hkv, D, T, "f32", "f16")
    rng = np.random.default_rng(78)
    lens = np.array([700, 33, 257], dtype=np.int32)
    kd, vd = to_device(k, "f16"), to_device(v, "f16")
    knew = rng.standard_normal((B, Hkv, D), dtype=np.float32)
    vnew = rng.standard_normal((B, Hkv, D), dtype=np.float32)
    pos = torch.from_numpy(lens - 1).cuda()
    lens_d = torch.from_numpy(lens).cuda()
    ws = attention.DecodeWorkspace(B, H, Hkv, D)
    outs = []
    for early in (False, True, True):
        kc, vc = kd.clone(), vd.clone()
        q_rot = attention.rope_kv_insert(torch.from_numpy(q).cuda(), torch.from_numpy(knew).cuda(),
                                         torch.from_numpy(vnew).cuda(), kc, vc, pos, pos, theta=10000.0)
        outs.append(attention.attn_decode(q_rot, kc, vc, lens_d, workspace=ws, kv_early=early))
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])
    want = checker.attn_decode(q_rot.cpu().numpy(), kc.cpu().numpy(), vc.cpu().numpy(), lens.astype(np.uint32))
    check_close(wl, outs[1].cpu().numpy(), want, "kv_early after rope insert")
    assert int(ws.status.item()) == 0


def test_length_beyond_the_cache_is_clamped_and_reported(attention, wl, checker):
    """A corrupted kv_len[] entry larger than the cache: the kernels clamp it to the stated capacity and raise
    ATTN_STATUS_BAD_SHAPE instead of reading past the cache."""
    import torch
    from gpu_util import check_close, to_device
    q, k, v = _rand(wl, 91, 2, 32, 8, 128, 300)
    lens = torch.tensor([100, 5000], dtype=torch.int32, device="cuda")
    ws = attention.DecodeWorkspace(2, 32, 8, 128)
    out = attention.attn_decode(to_device(q, "f32"), to_device(k, "f16"), to_device(v, "f16"), lens, workspace=ws)
    torch.cuda.synchronize()
    assert int(ws.status.item()) == 2  # ATTN_STATUS_BAD_SHAPE
    want = checker.attn_decode(q, k, v, np.array([100, 300], np.uint32))
    check_close(wl, out.cpu().numpy(), want, "clamped length")


def test_checking_build_runs_clean(pkg, wl, checker, tmp_path):
    """The -DATTN_BOUNDS_CHECK build (the decode passes verify their workspace indices and report ATTN_STATUS_BAD_INDEX
    instead of accessing) gives the same results with no status bit on uniform, ragged and single-long-sequence
    shapes, through attn_decode and through the engine's single-launch kernel symbol. Runs in a child process because the library is chosen when the binding is first loaded."""
    import subprocess
    import sys
    from conftest import ROOT
    lib = pkg.build.build_library(check=True)
    code = f"""
import sys, numpy as np, torch
sys.path.insert(0, {ROOT!r}); sys.path.insert(0, {ROOT!r} + '/tests')
from conftest import load_package
pkg = load_package()
from llm_infer_b200 import attention, binding
assert binding.LIB_PATH.endswith('_check.so')
import oracle
wl = pkg.workloads
for (B, T, lens) in ((3, 700, [700, 1, 333]), (1, 20000, None), (16, 512, None)):
    q, k, v = wl.decode_inputs(wl.DecodeShape('c', 5, B, 32, 8, 128, T, 'f32', 'f16'))
    ws = attention.DecodeWorkspace(B, 32, 8, 128)
    l = None if lens is None else torch.tensor(lens, dtype=torch.int32, device='cuda')
    out = attention.attn_decode(torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), l, workspace=ws)
    torch.cuda.synchronize()
    assert int(ws.status.item()) == 0, ws.status.item()
    want = oracle.best().attn_decode(q, k, v, None if lens is None else np.array(lens, np.uint32))
    a, r = wl.error_metrics(out.cpu().numpy(), want)
    assert a <= wl.ABS_TOL and r <= wl.REL_TOL, (a, r)
# the engine's kernel symbol (single launch; two-level merge on the long sequence)
import ctypes as C
lib = binding.load()
n = lib.attention_workspace_bytes(32, 8, 128)
wsb = torch.zeros(n, dtype=torch.uint8, device='cuda')
stream = torch.cuda.current_stream().cuda_stream
assert lib.attention_configure(32, 8, 128, 0.0, wsb.data_ptr(), n, stream) == 0
for T in (300, 20000):
    q, k, v = wl.decode_inputs(wl.DecodeShape('s', 6, 1, 32, 8, 128, T, 'f32', 'f16'))
    qd, kd, vd = (torch.from_numpy(x[0]).cuda() for x in (q, k, v))
    o = torch.empty(32, 128, device='cuda')
    assert lib.attention_launch(o.data_ptr(), qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), T, stream) == 0
    bits = C.c_uint32(7)
    assert lib.attention_status(C.byref(bits), 0, stream) == 0 and bits.value == 0, bits.value
    a, r = wl.error_metrics(o.cpu().numpy(), oracle.best().attn_decode(q, k, v)[0])
    assert a <= wl.ABS_TOL and r <= wl.REL_TOL, (a, r)
print('ok')
"""
    import os
    env = dict(os.environ, LLM_INFER_ATTN_LIB=lib)
    res = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and res.stdout.strip().endswith("ok"), res.stdout + res.stderr


def test_max_ctas_limits_split_without_changing_result(attention, wl, checker):
    from gpu_util import check_close, run_decode
    q, k, v = _rand(wl, 15, 1, 32, 8, 128, 5000)
    want = checker.attn_decode(q, k, v)
    for cap in (1, 2, 7, 148, 0):
        check_close(wl, run_decode(attention, q, k, v, max_ctas=cap), want, f"max_ctas={cap}")


def test_merge_entry_point(attention, wl, port):
    import torch
    q, k, v = wl.decode_inputs(wl.C4, kv_len=999)
    want, part_o, part_lse = port.attn_decode_sharded(q.astype(np.float32)[0], k[0], v[0], 5)
    part_lse[3] = -np.inf  # an empty shard
    want = np.stack([port.lse_merge(part_o[:, h], part_lse[:, h])[0] for h in range(32)])
    lse = torch.empty(32, dtype=torch.float32, device="cuda")
    got = attention.attn_merge(torch.from_numpy(part_o).cuda(), torch.from_numpy(part_lse).cuda(), lse=lse)
    torch.cuda.synchronize()
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=0, atol=1e-5)
    all_empty = torch.full((3, 8), float("-inf"), device="cuda")
    z = attention.attn_merge(torch.randn(3, 8, 128, device="cuda"), all_empty)
    assert torch.equal(z, torch.zeros_like(z))


@pytest.mark.parametrize("n_parts", [1, 7, 24, 25, 49, 97, 148, 301])
@pytest.mark.parametrize("D", [64, 128])
def test_merge_of_many_partials(attention, port, n_parts, D):
    """From one to a few hundred partials per row (a single long sequence leaves one per split-pass CTA): same result
    as the restated LSE merge, empty partials (lse = -inf) included."""
    import torch
    rng = np.random.default_rng(n_parts * 7 + D)
    rows = 5
    part_o = rng.standard_normal((n_parts, rows, D), dtype=np.float32)
    part_lse = (rng.standard_normal((n_parts, rows), dtype=np.float32) * 3).astype(np.float32)
    part_lse[rng.random((n_parts, rows)) < 0.2] = -np.inf
    part_lse[:, 4] = -np.inf  # a row with nothing at all
    lse = torch.empty(rows, dtype=torch.float32, device="cuda")
    got = attention.attn_merge(torch.from_numpy(part_o).cuda(), torch.from_numpy(part_lse).cuda(), lse=lse)
    torch.cuda.synchronize()
    got, lse = got.cpu().numpy(), lse.cpu().numpy()
    for r in range(rows):
        want, want_lse = port.lse_merge(part_o[:, r], part_lse[:, r])
        if np.isinf(part_lse[:, r]).all():
            assert (got[r] == 0).all() and lse[r] == -np.inf
        else:
            np.testing.assert_allclose(got[r], want, rtol=0, atol=2e-5)
            assert abs(lse[r] - want_lse) <= 1e-5 * max(1.0, abs(want_lse))


@pytest.mark.parametrize("n_parts", [1, 5, 6, 7, 16])
@pytest.mark.parametrize("D", [32, 64, 128, 256])
def test_merge_of_many_rows_with_few_partials(attention, port, n_parts, D):
    """Hundreds of rows with a handful of partials each (batched decode) take the warp-per-row form of the merge pass:
    same result as the restated LSE merge, empty partials and empty rows included."""
    import torch
    rng = np.random.default_rng(n_parts * 11 + D)
    rows = 300
    part_o = rng.standard_normal((n_parts, rows, D), dtype=np.float32)
    part_lse = (rng.standard_normal((n_parts, rows), dtype=np.float32) * 3).astype(np.float32)
    part_lse[rng.random((n_parts, rows)) < 0.2] = -np.inf
    part_lse[:, 7] = -np.inf
    lse = torch.empty(rows, dtype=torch.float32, device="cuda")
    got = attention.attn_merge(torch.from_numpy(part_o).cuda(), torch.from_numpy(part_lse).cuda(), lse=lse)
    torch.cuda.synchronize()
    got, lse = got.cpu().numpy(), lse.cpu().numpy()
    for r in range(0, rows, 13):
        want, want_lse = port.lse_merge(part_o[:, r], part_lse[:, r])
        if np.isinf(part_lse[:, r]).all():
            assert (got[r] == 0).all() and lse[r] == -np.inf
        else:
            np.testing.assert_allclose(got[r], want, rtol=0, atol=2e-5)
            assert abs(lse[r] - want_lse) <= 1e-5 * max(1.0, abs(want_lse))
    assert (got[7] == 0).all() and lse[7] == -np.inf


def _sharded_single_gpu(attention, q, k, v, world, rank, bufs, out, status_ws, step=0, poll_limit=0):
    import torch
    return attention.attn_decode_sharded(q, k, v, peer_buffers=[b.data_ptr() for b in bufs], world_size=world,
                                         rank=rank, step=step, poll_limit=poll_limit, out=out, workspace=status_ws)


def test_fused_exchange_with_one_rank_equals_plain_decode(attention, wl, checker):
    """World size 1: the exchange path (peer stores, flags, wait, cross merge) runs against the rank's own buffer."""
    import torch
    from gpu_util import check_close, to_device
    q, k, v = _rand(wl, 41, 2, 32, 8, 128, 3000, "f16", "f16")
    qd, kd, vd = to_device(q, "f16"), to_device(k, "f16"), to_device(v, "f16")
    ws = attention.DecodeWorkspace(2, 32, 8, 128)
    buf = torch.zeros(attention.exchange_bytes(2, 32, 128, 1) // 4, device="cuda")
    want = checker.attn_decode(q.astype(np.float32), k, v)
    for call in range(3):  # consecutive steps alternate the record parity and advance the device-side step counter
        out = torch.full((2, 32, 128), float("nan"), device="cuda")
        _sharded_single_gpu(attention, qd, kd, vd, 1, 0, [buf], out, ws)
        torch.cuda.synchronize()
        check_close(wl, out.cpu().numpy(), want, f"fused exchange, call {call}")
    assert int(ws.status.item()) == 0
    ctl = buf.view(torch.int64)[-2:].tolist()
    assert ctl == [3, 0]  # three steps completed, no cell pending


def test_fused_exchange_times_out_cleanly_when_a_peer_never_arrives(attention, wl, checker):
    """World size 2 with nobody playing rank 1: the wait on rank 1's flags must run out, set the status bit and leave
    the output untouched; the context stays usable (a normal decode works right after)."""
    import torch
    from gpu_util import check_close, to_device
    q, k, v = _rand(wl, 42, 1, 32, 8, 128, 500, "f16", "f16")
    qd, kd, vd = to_device(q, "f16"), to_device(k, "f16"), to_device(v, "f16")
    ws = attention.DecodeWorkspace(1, 32, 8, 128)
    n = attention.exchange_bytes(1, 32, 128, 2) // 4
    mine, absent_peer = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    out = torch.full((1, 32, 128), float("nan"), device="cuda")
    _sharded_single_gpu(attention, qd, kd, vd, 2, 0, [mine, absent_peer], out, ws, step=1, poll_limit=200)
    torch.cuda.synchronize()
    assert int(ws.status.item()) & 1  # ATTN_STATUS_WAIT_TIMEOUT
    assert torch.isnan(out).all()
    # this rank's record did reach the "peer": what a live rank 1 would have merged (step 1 -> parity 1, source rank 0)
    rec_o, rec_lse, steps = attention.exchange_record(absent_peer, 1, 32, 128, 2, parity=1, source_rank=0)
    assert (steps == 1).all()
    want = checker.attn_decode(q.astype(np.float32), k, v)
    check_close(wl, rec_o.view(1, 32, 128).cpu().numpy(), want, "record delivered to the peer buffer")
    assert torch.isfinite(rec_lse).all()
    ws.status.zero_()
    got = attention.attn_decode(qd, kd, vd, workspace=ws)
    torch.cuda.synchronize()
    check_close(wl, got.cpu().numpy(), want, "decode after a timed-out exchange")
    assert int(ws.status.item()) == 0
