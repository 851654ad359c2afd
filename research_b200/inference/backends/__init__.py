from .generate import GenerationOutput, generate_hf, generate_native, generate_sglang, generate_vllm
from .tokenize import (append_suffix_with_overlap, build_loss_mask, check_token_mismatch, compute_suffix_ids,
                       find_largest_overlap, log_token_mismatch, tokenize_chat, tokenize_message_with_delimiter)

__all__ = ["GenerationOutput", "generate_hf", "generate_native", "generate_sglang", "generate_vllm",
           "append_suffix_with_overlap", "build_loss_mask", "check_token_mismatch", "compute_suffix_ids",
           "find_largest_overlap", "log_token_mismatch", "tokenize_chat", "tokenize_message_with_delimiter"]
