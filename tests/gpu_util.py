"""Helpers for the GPU parity tests: numpy inputs -> device tensors -> C-ABI call -> numpy."""
import numpy as np
import torch

_TORCH = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def to_device(x: np.ndarray, dtype: str) -> torch.Tensor:
    """Storage array (float32 / float16 / uint16 bf16 bits) -> CUDA tensor of that dtype."""
    if dtype == "bf16":
        return torch.from_numpy(x.view(np.int16).copy()).cuda().view(torch.bfloat16)
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


def run_decode(attention, q, k, v, q_dtype="f32", kv_dtype="f16", kv_len=None, out_dtype="f32", lse=False, **kw):
    qd, kd, vd = to_device(q, q_dtype), to_device(k, kv_dtype), to_device(v, kv_dtype)
    lens = None
    if kv_len is not None:
        lens = torch.from_numpy(np.asarray(kv_len, dtype=np.int32)).cuda()
    B, H, D = qd.shape
    lse_t = torch.full((B, H), float("nan"), dtype=torch.float32, device="cuda") if lse else None
    out = attention.attn_decode(qd, kd, vd, lens, out_dtype=_TORCH[out_dtype], lse=lse_t, **kw)
    torch.cuda.synchronize()
    o = out.float().cpu().numpy()
    return (o, lse_t.cpu().numpy()) if lse else o


def check_close(wl, got, want, what=""):
    max_abs, max_rel = wl.error_metrics(got, want)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    assert max_abs <= wl.ABS_TOL, f"{what}: max abs error {max_abs:.3e} > {wl.ABS_TOL}"
    assert max_rel <= wl.REL_TOL, f"{what}: max rel error {max_rel:.3e} > {wl.REL_TOL}"
    return max_abs, max_rel
