from .data_buffer import (BufferState, DataBuffer, get_samples, get_samples_flat, load_samples_from_jsonl,
                          load_samples_from_list, load_samples_from_parquet, state_from_dict, state_to_dict)

from .sft import (compute_loss_mask, export_samples_to_jsonl, extract_conversation, load_rl_prompts, load_samples_from_export,
                  load_sft_dataset, prepare_sft_sample, tokenize_conversation)

__all__ = ["compute_loss_mask", "export_samples_to_jsonl", "extract_conversation", "load_rl_prompts", "load_samples_from_export",
           "load_sft_dataset", "prepare_sft_sample", "tokenize_conversation", "BufferState", "DataBuffer", "get_samples", "get_samples_flat", "load_samples_from_jsonl",
           "load_samples_from_list", "load_samples_from_parquet", "state_from_dict", "state_to_dict"]
