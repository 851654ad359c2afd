from .data_buffer import (BufferState, DataBuffer, get_samples, get_samples_flat, load_samples_from_jsonl,
                          load_samples_from_list, load_samples_from_parquet, state_from_dict, state_to_dict)

__all__ = ["BufferState", "DataBuffer", "get_samples", "get_samples_flat", "load_samples_from_jsonl",
           "load_samples_from_list", "load_samples_from_parquet", "state_from_dict", "state_to_dict"]
