"""B200 (sm_100a) attention path for the llm-infer engine: split-KV decode,
causal prefill and KV-sharded multi-GPU decode behind a C ABI
(include/llm_infer_attn.h). The directory name carries a hyphen, so import it
through ``importlib`` under the name ``llm_infer_b200`` (the repository's tests,
benchmark and entry script do exactly that).

Submodules: ``binding`` (ctypes, no torch), ``attention`` (torch tensors in, C ABI
underneath), ``workloads`` (seeded synthetic inputs), ``build`` (nvcc driver).
"""
from . import binding, build, workloads  # noqa: F401

__all__ = ["binding", "build", "workloads"]
