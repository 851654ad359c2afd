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
from .flash import (
    flash_attention,
    flash_attn_varlen,
    flash_attn_varlen_backward,
    flash_attn_varlen_reference,
    flash_paged_prefill,
)
from . import gemm as gemm_mod
from .gemm import gemm, gemm_fp8, lm_head_sample, lm_head_sample_workspace, gemm_reference, gemm_symmetric, quantize_fp8, interleave_gate_up, linear
from .sampling import sample_with_logprobs, sample_with_logprobs_reference, token_logprobs

def set_pdl(on: bool) -> None:
    """Enable programmatic dependent launch for the decode-path kernels (GEMM, norms, RoPE,
    attention, SwiGLU, embedding, sampling): consecutive kernels overlap prologue and tail."""
    from .. import _native

    for lib, fn in (("rb_gemm", "rb_gemm_set_pdl"), ("rb_ops", "rb_ops_set_pdl"), ("rb_attn", "rb_attn_set_pdl")):
        getattr(_native.load(lib), fn)(int(on))


__all__ = [
    "KernelStatusError", "check_status", "status_tensor", "decode_num_splits", "gather_kv", "paged_decode",
    "paged_decode_reference", "paged_prefill", "paged_prefill_reference", "embedding", "rmsnorm",
    "rmsnorm_reference", "rope_kv_append", "rope_kv_append_reference", "rope_table", "swiglu", "swiglu_backward",
    "swiglu_reference", "transpose", "gemm", "gemm_reference", "linear", "sample_with_logprobs",
    "sample_with_logprobs_reference", "token_logprobs", "set_pdl", "interleave_gate_up", "gemm_mod", "gemm_symmetric", "gemm_fp8", "quantize_fp8", "lm_head_sample", "lm_head_sample_workspace", "flash_attention", "flash_attn_varlen",
    "flash_attn_varlen_backward", "flash_attn_varlen_reference", "flash_paged_prefill",
]
