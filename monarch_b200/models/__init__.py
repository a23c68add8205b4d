"""Model families: Llama dense decoders (explicit engine + stock-torch twin) and a
Mixtral-style MoE decoder."""
from .llama import (PRESETS, LlamaConfig, LlamaEngine, LocalParamStore, ParamLayout,
                    load_hf_state_dict, to_hf_state_dict)
from .torch_llama import TorchLlama

__all__ = ["PRESETS", "LlamaConfig", "LlamaEngine", "LocalParamStore", "ParamLayout",
           "TorchLlama", "load_hf_state_dict", "to_hf_state_dict"]
