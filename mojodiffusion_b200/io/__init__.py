"""IO: safetensors (reader / writer / sharded), caption-cache tensor bins, configs, PNG / WAV, disk guard."""
from .cap_cache import load_tensor_bin, save_tensor_bin
from .config import (OptimizerConfig, SamplePrompt, SamplePromptFile, TrainConfig, guard_free_space, read_model_config,
                     read_sample_prompts)
from .png import decode_png, encode_png, load_png, save_png, save_wav, tensor_to_uint8
from .safetensors_io import (SafeTensors, ShardedSafeTensors, TensorRef, load_safetensors, save_safetensors,
                             save_sharded)
