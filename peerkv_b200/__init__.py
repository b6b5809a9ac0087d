"""peerkv_b200 -- peer-parallel split-K decode attention for B200 (sm_100a).

Host side of a C-ABI CUDA library (include/peerkv.h, built by `python -m
peerkv_b200.build`).  It mirrors the call surface of PeerKV's `umallm` package for
this one path:

    peerkv_b200.peer_parallel_attn   <->  umallm.peer_parallel_attn
    peerkv_b200.peerkv               <->  umallm.peerkv  (fused_attn, paged, vllm_backend, register)

There is no CPU or PyTorch fallback: without the built library every call raises.
"""
from ._lib import PeerKVError  # noqa: F401

__version__ = "0.1.0"
