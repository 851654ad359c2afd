"""Kernel entry points. Every op runs the sm_100a kernel on CUDA tensors and an fp32-faithful
PyTorch reference on CPU tensors (the oracle the GPU tests compare against)."""

from ._util import KernelStatusError, check_status, status_tensor
from .attention import (
    decode_num_splits,
    gather_kv,
    paged_decode,
    paged_decode_reference,
    paged_prefill,
    paged_prefill_reference,
)
from .elementwise import (
    embedding,
    rmsnorm,
    rmsnorm_reference,
    rope_kv_append,
    rope_kv_append_reference,
    rope_table,
    swiglu,
    swiglu_backward,
    swiglu_reference,
    transpose,
)
from .gemm import gemm, gemm_reference, linear
from .sampling import sample_with_logprobs, sample_with_logprobs_reference, token_logprobs

__all__ = [
    "KernelStatusError", "check_status", "status_tensor", "decode_num_splits", "gather_kv", "paged_decode",
    "paged_decode_reference", "paged_prefill", "paged_prefill_reference", "embedding", "rmsnorm",
    "rmsnorm_reference", "rope_kv_append", "rope_kv_append_reference", "rope_table", "swiglu", "swiglu_backward",
    "swiglu_reference", "transpose", "gemm", "gemm_reference", "linear", "sample_with_logprobs",
    "sample_with_logprobs_reference", "token_logprobs",
]
