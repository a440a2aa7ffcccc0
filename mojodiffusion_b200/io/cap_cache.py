"""Bit-exact tensor bin files for handing text embeddings from an encode process to a DiT process.

Layout (little-endian): int64 magic "KLNCAPV1" (0x4B4C4E4341505631), int64 dtype tag, int64 rank, int64 dims[rank],
then the raw element bytes in the storage dtype (never up-cast), so load(save(t)) is byte identical.
Format and dtype tags: serenitymojo/io/cap_cache.mojo:77-269, serenitymojo/io/dtype.mojo:19-36.
"""
from __future__ import annotations

import struct

import torch

MAGIC = 0x4B4C4E4341505631
_TAGS = {torch.bool: 0, torch.uint8: 1, torch.int8: 2, torch.float8_e5m2: 3, torch.float8_e4m3fn: 4, torch.int16: 5,
         torch.float16: 7, torch.bfloat16: 8, torch.int32: 9, torch.float32: 11, torch.float64: 12, torch.int64: 13}
_DTYPES = {v: k for k, v in _TAGS.items()}


def save_tensor_bin(path, t: torch.Tensor) -> None:
    t = t.detach().to("cpu").contiguous()
    hdr = struct.pack("<qqq", MAGIC, _TAGS[t.dtype], t.dim()) + struct.pack(f"<{t.dim()}q", *t.shape)
    with open(path, "wb") as f:
        f.write(hdr)
        if t.numel():
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())


def load_tensor_bin(path, device="cpu") -> torch.Tensor:
    with open(path, "rb") as f:
        data = f.read()
    if len(data) < 24:
        raise ValueError(f"{path}: truncated header")
    magic, tag, rank = struct.unpack_from("<qqq", data, 0)
    if magic != MAGIC:
        raise ValueError(f"{path}: bad magic {magic:#x}")
    if tag not in _DTYPES or not (0 <= rank <= 8):
        raise ValueError(f"{path}: bad dtype tag {tag} / rank {rank}")
    dims = struct.unpack_from(f"<{rank}q", data, 24)
    dt = _DTYPES[tag]
    n = 1
    for d in dims:
        n *= d
    off = 24 + 8 * rank
    nbytes = n * torch.empty(0, dtype=dt).element_size()
    if len(data) - off != nbytes:
        raise ValueError(f"{path}: payload is {len(data) - off} bytes, expected {nbytes}")
    t = torch.frombuffer(bytearray(data[off:]), dtype=torch.uint8).view(dt).reshape(dims) if n else torch.empty(dims, dtype=dt)
    return t.to(device)
