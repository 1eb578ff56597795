"""GPU parity of the tcgen05 causal-prefill kernel, called through the C ABI, against the CPU checker: row t of
the result must equal the engine's decode attention with kv_len = t + 1 (src/model/model.cpp:68,
include/kernels_cpu.hpp:140-167). Tolerance: max abs 2e-3, max rel 1e-2 (relative error measured against
max(|ref|, 1% of the RMS of ref)), for the default mode (probabilities as a 16-bit value plus residual)."""
import ctypes as C
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


def _dev(x, dtype):
    import torch
    if dtype == "bf16":
        return torch.from_numpy(x.view(np.int16).copy()).cuda().view(torch.bfloat16)
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


P_RESIDUAL, P_INPUT = 0, 1  # binding.PREFILL_P_*


def _run(attention, q, k, v, dtype, out_fp32=True, p_mode=P_RESIDUAL):
    import torch
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = attention.attn_prefill_causal(_dev(q, dtype), _dev(k, dtype), _dev(v, dtype),
                                        out_dtype=torch.float32 if out_fp32 else None, p_mode=p_mode, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "device status word reports a timed-out wait"
    return out.float().cpu().numpy()


def _want(wl, checker, q, k, v, dtype, **rows):
    return checker.attn_prefill_causal(wl.widen(q, dtype), wl.as_f16_for_oracle(k, dtype),
                                       wl.as_f16_for_oracle(v, dtype), **rows)


def test_golden_vectors(attention, wl):
    from gpu_util import check_close
    g = np.load(os.path.join(GOLDEN, "prefill_golden.npz"))
    name = "s40_mqa_d128"
    got = _run(attention, g[f"{name}.q"], g[f"{name}.k"], g[f"{name}.v"], "f16")
    check_close(wl, got, g[f"{name}.o"], name)


@pytest.mark.parametrize("B,S,H,Hkv,dtype", [
    (1, 1, 4, 1, "bf16"), (1, 2, 4, 2, "f16"), (2, 127, 8, 2, "bf16"), (1, 128, 8, 2, "f16"), (1, 129, 8, 2, "bf16"),
    (2, 255, 4, 4, "bf16"), (1, 256, 4, 4, "f16"), (1, 257, 6, 6, "bf16"), (3, 300, 8, 1, "bf16"),
    (1, 512, 32, 8, "bf16"), (1, 640, 3, 1, "f16"), (1, 1000, 8, 8, "bf16")])
@pytest.mark.parametrize("D", [128, 64])
def test_every_row_against_cpu_attn(attention, wl, checker, B, S, H, Hkv, dtype, D):
    from gpu_util import check_close
    q, k, v = wl.prefill_inputs(wl.PrefillShape("t", S * 7 + H, B, S, H, Hkv, D, dtype))
    got = _run(attention, q, k, v, dtype)
    check_close(wl, got, _want(wl, checker, q, k, v, dtype), f"B{B} S{S} H{H}/{Hkv} D{D} {dtype}")


def test_head_dim_64_16_bit_output(attention, wl, checker):
    """TinyLlama-shaped heads (32 / 4, head_dim 64), bf16 in and out."""
    q, k, v = wl.prefill_inputs(wl.PrefillShape("t", 64, 1, 333, 32, 4, 64, "bf16"))
    got = _run(attention, q, k, v, "bf16", out_fp32=False)
    want = _want(wl, checker, q, k, v, "bf16")
    assert (np.abs(got - want) <= 1e-4 + 2.0 ** -8 * np.abs(want)).all()


def test_c3_llama3_prefill_full_size_sampled_rows(attention, wl, checker):
    """Batch 4 x 2048 rows, 32/8 heads, bf16: every row of the first and last 128-row tile and every 64th row
    in between are compared (the CPU attn() for all 8192 x 32 rows would take about a minute)."""
    from gpu_util import check_close
    q, k, v = wl.prefill_inputs(wl.C3)
    got = _run(attention, q, k, v, "bf16")
    assert np.isfinite(got).all()
    for rows in (dict(row_begin=0, row_end=128), dict(row_begin=1920, row_end=2048),
                 dict(row_begin=128, row_end=1920, row_step=64)):
        want = _want(wl, checker, q, k, v, "bf16", **rows)
        sel = ~np.isnan(want[0, :, 0, 0])
        max_abs, max_rel = check_close(wl, got[:, sel], want[:, sel], f"C3 rows {rows}")
        print(f"C3 {rows}: max_abs={max_abs:.3e} max_rel={max_rel:.3e}")


def test_16_bit_output_and_determinism(attention, wl, checker):
    import torch
    q, k, v = wl.prefill_inputs(wl.PrefillShape("t", 9, 2, 384, 8, 2, 128, "bf16"))
    qd, kd, vd = _dev(q, "bf16"), _dev(k, "bf16"), _dev(v, "bf16")
    padded = torch.zeros(2 * 384 * 8 * 128 + 1024, dtype=torch.bfloat16, device="cuda")
    padded.fill_(float("nan"))
    out = padded[512:512 + 2 * 384 * 8 * 128].view(2, 384, 8, 128)
    attention.attn_prefill_causal(qd, kd, vd, out=out)
    first = out.clone()
    for _ in range(2):
        attention.attn_prefill_causal(qd, kd, vd, out=out)
        assert torch.equal(out, first)
    torch.cuda.synchronize()
    assert torch.isnan(padded[:512]).all() and torch.isnan(padded[-512:]).all()
    got, want = first.float().cpu().numpy(), _want(wl, checker, q, k, v, "bf16")
    # the output itself is stored in bf16 here: half an ulp (2^-9 relative) on top of the kernel's own error
    assert (np.abs(got - want) <= 1e-4 + 2.0 ** -8 * np.abs(want)).all()


def test_single_rounding_mode_is_close_but_not_the_parity_mode(attention, wl, checker):
    """ATTN_PREFILL_P_INPUT_TYPE feeds the tensor cores one probability rounded to the input type: for bf16 an error
    of about 2^-9 of a row's typical output magnitude, which stays within a few 1e-3 absolute but not within the
    strict relative bound."""
    q, k, v = wl.prefill_inputs(wl.PrefillShape("t", 10, 1, 512, 8, 2, 128, "bf16"))
    got = _run(attention, q, k, v, "bf16", p_mode=P_INPUT)
    max_abs, _ = wl.error_metrics(got, _want(wl, checker, q, k, v, "bf16"))
    assert max_abs <= 8e-3


def test_unsupported_head_dim_is_refused(built_lib, pkg):
    import torch
    b = pkg.binding
    t = torch.zeros((1, 16, 4, 96), dtype=torch.float16, device="cuda")
    a = b.AttnPrefillArgs()
    a.o = a.q = a.k = a.v = t.data_ptr()
    a.o_dtype = a.dtype = b.DTYPE_F16
    a.batch, a.seq_len, a.n_heads, a.n_kv_heads, a.head_dim = 1, 16, 4, 4, 96
    assert built_lib.attn_prefill_causal(C.byref(a), None) == -2
