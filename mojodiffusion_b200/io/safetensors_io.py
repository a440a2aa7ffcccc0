"""safetensors reader (mmap, zero-copy views), byte-exact canonical writer, sharded checkpoints.

File format: 8-byte little-endian header length, JSON header ``{name: {dtype, shape, data_offsets}, "__metadata__"}``,
then the raw tensor bytes. The writer emits a compact header (no whitespace) in insertion order and copies tensor
bytes verbatim in their storage dtype (BF16 / F16 / F8_E4M3 / U8 are never converted), so a file written here is
byte-identical to what the reference's writer produces for the same tensors in the same order.

Reference behaviour: serenitymojo/io/safetensors.mojo:64-239 (reader, 100 MB header cap, madvise prefetch),
serenitymojo/io/sharded.mojo:363-497 (index.json / single file / directory fallback),
serenitymojo/io/safetensors_writer.mojo:129-278, serenitymojo/io/dtype.mojo:39-154.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from collections import OrderedDict
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, List, Mapping, Optional, Tuple

import torch

MAX_HEADER_BYTES = 100 * 1024 * 1024

# safetensors dtype tag <-> torch dtype / element size
_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1), "F8_E4M3": (torch.float8_e4m3fn, 1),
    "F8_E5M2": (torch.float8_e5m2, 1),
}
_TAGS = {v[0]: k for k, v in _DTYPES.items()}


def dtype_from_tag(tag: str) -> torch.dtype:
    return _DTYPES[tag][0]


def tag_from_dtype(dt: torch.dtype) -> str:
    return _TAGS[dt]


def dtype_size(tag: str) -> int:
    return _DTYPES[tag][1]


@dataclass
class TensorRef:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    offset: int  # absolute file offset of the first byte
    size: int

    @property
    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n


class SafeTensors:
    """One mmap'd safetensors file. ``tensor(name)`` returns a CPU tensor viewing the mapping (no copy)."""

    def __init__(self, path: str | os.PathLike):
        self.path = str(path)
        self._f = open(self.path, "rb")
        head = self._f.read(8)
        if len(head) != 8:
            raise ValueError(f"{self.path}: truncated (no header length)")
        (hlen,) = struct.unpack("<Q", head)
        if hlen > MAX_HEADER_BYTES:
            raise ValueError(f"{self.path}: header of {hlen} bytes exceeds the 100 MB cap")
        raw = self._f.read(hlen)
        if len(raw) != hlen:
            raise ValueError(f"{self.path}: truncated header")
        header = json.loads(raw.decode("utf-8"), object_pairs_hook=OrderedDict)
        self.metadata: Dict[str, str] = dict(header.pop("__metadata__", {}) or {})
        self.data_start = 8 + hlen
        fsize = os.fstat(self._f.fileno()).st_size
        self.refs: "OrderedDict[str, TensorRef]" = OrderedDict()
        for name, info in header.items():
            b, e = info["data_offsets"]
            shape = tuple(int(d) for d in info["shape"])
            ref = TensorRef(name, info["dtype"], shape, self.data_start + b, e - b)
            if ref.dtype not in _DTYPES:
                raise ValueError(f"{self.path}: tensor {name} has unknown dtype {ref.dtype}")
            if ref.numel * dtype_size(ref.dtype) != ref.size or ref.offset + ref.size > fsize:
                raise ValueError(f"{self.path}: tensor {name} has inconsistent offsets / is truncated")
            self.refs[name] = ref
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_COPY) if fsize > 0 else None

    @classmethod
    def open(cls, path) -> "SafeTensors":
        return cls(path)

    def keys(self) -> List[str]:
        return list(self.refs.keys())

    def __contains__(self, name: str) -> bool:
        return name in self.refs

    def tensor_info(self, name: str) -> TensorRef:
        return self.refs[name]

    def tensor_bytes(self, name: str) -> memoryview:
        r = self.refs[name]
        return memoryview(self._mm)[r.offset:r.offset + r.size]

    def tensor(self, name: str) -> torch.Tensor:
        r = self.refs[name]
        dt = dtype_from_tag(r.dtype)
        if r.size == 0:
            return torch.empty(r.shape, dtype=dt)
        flat = torch.frombuffer(self._mm, dtype=torch.uint8, count=r.size, offset=r.offset)
        return flat.view(dt).reshape(r.shape)

    def prefetch_tensor(self, name: str) -> None:
        """madvise(WILLNEED) the pages of a tensor (read-ahead for a block that is about to be streamed)."""
        r = self.refs[name]
        if self._mm is None or not hasattr(self._mm, "madvise"):
            return
        page = mmap.PAGESIZE
        start = (r.offset // page) * page
        self._mm.madvise(mmap.MADV_WILLNEED, start, r.offset + r.size - start)

    def close(self):
        # views returned by tensor() keep the mapping alive; closing only drops our handles
        try:
            if self._mm is not None:
                self._mm.close()
        except BufferError:
            pass
        self._f.close()


def _header_bytes(entries: "OrderedDict[str, dict]", metadata: Optional[Mapping[str, str]]) -> bytes:
    hdr: "OrderedDict[str, object]" = OrderedDict()
    if metadata:
        hdr["__metadata__"] = dict(metadata)
    hdr.update(entries)
    return json.dumps(hdr, separators=(",", ":"), ensure_ascii=False).encode("utf-8")


def save_safetensors(path, tensors: Mapping[str, torch.Tensor], metadata: Optional[Mapping[str, str]] = None) -> None:
    """Write tensors in insertion order with a compact header; bytes are copied in the storage dtype."""
    entries: "OrderedDict[str, dict]" = OrderedDict()
    off = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().to("cpu").contiguous()
        tag = tag_from_dtype(t.dtype)
        n = t.numel() * t.element_size()
        entries[name] = {"dtype": tag, "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
        blobs.append(t)
    hb = _header_bytes(entries, metadata)
    tmp = f"{path}.tmp.{os.getpid()}"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for t in blobs:
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
    os.replace(tmp, path)


def load_safetensors(path, device="cpu", dtype: Optional[torch.dtype] = None) -> "OrderedDict[str, torch.Tensor]":
    st = SafeTensors(path)
    out = OrderedDict()
    for k in st.keys():
        t = st.tensor(k)
        t = t.to(device=device, dtype=dtype) if dtype is not None and t.is_floating_point() else t.to(device)
        out[k] = t.clone() if t.device.type == "cpu" else t
    return out


class ShardedSafeTensors:
    """A checkpoint given as ``*.index.json`` (weight_map), a single file, or a directory holding either."""

    def __init__(self, path: str | os.PathLike):
        p = Path(path)
        self.files: Dict[str, SafeTensors] = {}
        self.weight_map: Dict[str, str] = {}
        if p.is_dir():
            idx = sorted(p.glob("*.index.json"))
            if idx:
                p = idx[0]
            else:
                singles = sorted(p.glob("*.safetensors"))
                if not singles:
                    raise FileNotFoundError(f"{path}: no safetensors file or index")
                if len(singles) == 1:
                    p = singles[0]
                else:
                    for s in singles:
                        st = SafeTensors(s)
                        self.files[s.name] = st
                        for k in st.keys():
                            self.weight_map[k] = s.name
                    self.root = Path(path)
                    return
        self.root = p.parent
        if p.name.endswith(".index.json"):
            idx = json.loads(p.read_text())
            self.weight_map = dict(idx["weight_map"])
        else:
            st = SafeTensors(p)
            self.files[p.name] = st
            self.weight_map = {k: p.name for k in st.keys()}

    @classmethod
    def open(cls, path) -> "ShardedSafeTensors":
        return cls(path)

    def _file(self, fname: str) -> SafeTensors:
        if fname not in self.files:
            self.files[fname] = SafeTensors(self.root / fname)
        return self.files[fname]

    def keys(self) -> List[str]:
        return list(self.weight_map.keys())

    def __contains__(self, k):
        return k in self.weight_map

    def tensor_info(self, name: str) -> TensorRef:
        return self._file(self.weight_map[name]).tensor_info(name)

    def tensor_view(self, name: str) -> torch.Tensor:
        return self._file(self.weight_map[name]).tensor(name)

    def prefetch_tensor(self, name: str) -> None:
        self._file(self.weight_map[name]).prefetch_tensor(name)

    def keys_with_prefix(self, prefix: str) -> List[str]:
        return [k for k in self.weight_map if k.startswith(prefix)]


def save_sharded(directory, tensors: Mapping[str, torch.Tensor], max_shard_bytes: int = 5 << 30,
                 stem: str = "model") -> str:
    """Split into shards of at most ``max_shard_bytes`` and write ``<stem>.safetensors.index.json``."""
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    shards: List["OrderedDict[str, torch.Tensor]"] = [OrderedDict()]
    size = 0
    for k, t in tensors.items():
        n = t.numel() * t.element_size()
        if size + n > max_shard_bytes and shards[-1]:
            shards.append(OrderedDict())
            size = 0
        shards[-1][k] = t
        size += n
    wm = {}
    total = 0
    for i, sh in enumerate(shards):
        fname = f"{stem}-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_safetensors(d / fname, sh)
        for k, t in sh.items():
            wm[k] = fname
            total += t.numel() * t.element_size()
    idx = d / f"{stem}.safetensors.index.json"
    idx.write_text(json.dumps({"metadata": {"total_size": total}, "weight_map": wm}, indent=2))
    return str(idx)
