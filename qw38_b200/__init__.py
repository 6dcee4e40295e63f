"""B200-native Q4_K x Q8 quantized matmul engine: CUDA kernels behind a C ABI, with a thin
host-side mirror of the reference engine's cuda/q4k_q8.hpp interface."""
from .q4k_q8 import (PrefillWeight, Q8Input, Q4KError, pack_q8, q4k_q8_project, q4k_q8_project_ragged, q4k_q8_project_static,
                     q4k_q8_mlp, q8_mlp_workspace_bytes, repack_blocks144, quantize_q4k_blocks, quantize_q4k_weight, validate_weight, dequantize_bf16, unpack_logical, export_q8_1, hidden_rms_q8,
                     swiglu_pack_q8, new_q8_input, set_launch_overlap, launch_overlap)

__all__ = ["PrefillWeight", "Q8Input", "Q4KError", "pack_q8", "q4k_q8_project", "q4k_q8_project_ragged", "q4k_q8_project_static",
           "q4k_q8_mlp", "q8_mlp_workspace_bytes", "repack_blocks144", "quantize_q4k_blocks", "quantize_q4k_weight", "validate_weight", "dequantize_bf16", "unpack_logical", "export_q8_1", "hidden_rms_q8",
           "swiglu_pack_q8", "new_q8_input", "set_launch_overlap", "launch_overlap"]
