"""mojodiffusion_b200: a Blackwell-native (sm_100a) diffusion and video engine.

PyTorch is the framework layer (modules, autograd glue, sampler loops, data, serving workers); the hot
paths are hand-written CUDA kernels (``csrc/``) built in-tree into ``_C.so`` and reached through
``torch.ops.mdb200``. Sub-packages:

* ``ops``       kernels' Python face: dispatch, autograd functions and the pure-torch fp32 references
* ``models``    MMDiT (FLUX / Qwen-Image), single-stream DiT (Z-Image), video DiT (LTX-2), UNet (SDXL), VAEs
* ``sampling``  flow-matching and DDPM-family schedulers, multistep solvers, guidance, sampler registry
* ``training``  config, LoRA / LyCORIS adapters, optimizers, trainer loop, checkpoints, data cache
* ``parallel``  data / sequence (Ulysses) / tensor / FSDP parallel paths and their fused peer-memory kernels
* ``offload``   block-swap host offload (pinned store, device slots, side stream)
* ``io``        safetensors reader / writer, sharded checkpoints, config loaders, PNG / WAV
* ``serve``     worker process (start / step / cancel / trim) speaking the line-JSON wire protocol
"""
__version__ = "0.1.0"
