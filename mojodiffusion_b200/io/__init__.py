"""IO: safetensors (reader / writer / sharded), caption-cache tensor bins, configs, PNG / WAV, disk guard."""
from .safetensors_io import (SafeTensors, ShardedSafeTensors, TensorRef, load_safetensors, save_safetensors,
                             save_sharded)
