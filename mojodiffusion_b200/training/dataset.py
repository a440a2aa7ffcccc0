"""Pre-computed training cache: one safetensors file per sample with ``latent`` [1,C,h,w], ``text_embedding``
[1,T,J], ``text_mask`` [1,T] (optional ``latent_mask``, ``control_latent``; pixel-space caches carry ``pixel`` [3,H,W]
and ``cap_feats`` [1,seq,F] instead). The reader enumerates a directory (sorted), peeks shapes from the headers only,
groups samples into same-shape buckets, and yields batches staged in pinned host memory so the host->device copy of
step k+1 overlaps step k (serenitymojo/training/klein_dataset.mojo:1-60,136-280; bucket key = (C, H, W, text_seq))."""
from __future__ import annotations

import os
import random
from dataclasses import dataclass
from typing import Dict, Iterator, List, Optional, Tuple

import torch

from ..io.safetensors_io import SafeTensors, load_safetensors, save_safetensors

LATENT_KEY, TEXT_KEY, MASK_KEY = "latent", "text_embedding", "text_mask"
LATENT_MASK_KEY, CONTROL_KEY = "latent_mask", "control_latent"
PIXEL_KEY, CAP_FEATS_KEY = "pixel", "cap_feats"


def write_sample(path, latent: torch.Tensor, text_embedding: torch.Tensor, text_mask: torch.Tensor,
                 latent_mask: Optional[torch.Tensor] = None, control_latent: Optional[torch.Tensor] = None) -> None:
    if latent.dim() != 4 or text_embedding.dim() != 3 or text_mask.dim() != 2:
        raise ValueError("write_sample: latent [1,C,h,w], text_embedding [1,T,J], text_mask [1,T] expected")
    d = {LATENT_KEY: latent.contiguous(), TEXT_KEY: text_embedding.contiguous(), MASK_KEY: text_mask.float().contiguous()}
    if latent_mask is not None:
        d[LATENT_MASK_KEY] = latent_mask.contiguous()
    if control_latent is not None:
        d[CONTROL_KEY] = control_latent.contiguous()
    save_safetensors(path, d)


@dataclass(frozen=True)
class BucketKey:
    channels: int
    height: int
    width: int
    text_seq: int


class LatentCache:
    def __init__(self, directory: str, require_control: bool = False):
        self.dir = directory
        self.files = sorted(f for f in os.listdir(directory) if f.endswith(".safetensors"))
        if not self.files:
            raise FileNotFoundError(f"no cache samples (*.safetensors) in {directory}")
        self.keys: List[BucketKey] = []
        for f in self.files:
            st = SafeTensors(os.path.join(directory, f))
            try:
                names = set(st.keys())
                for need in (LATENT_KEY, TEXT_KEY, MASK_KEY) + ((CONTROL_KEY,) if require_control else ()):
                    if need not in names:
                        raise KeyError(f"{f}: cache sample lacks '{need}'")
                ls, ts = tuple(st.tensor_info(LATENT_KEY).shape), tuple(st.tensor_info(TEXT_KEY).shape)
                if len(ls) != 4:
                    raise ValueError(f"{f}: latent must be rank 4, got {ls}")
                self.keys.append(BucketKey(ls[1], ls[2], ls[3], ts[1]))
            finally:
                st.close()

    def __len__(self):
        return len(self.files)

    def buckets(self) -> Dict[BucketKey, List[int]]:
        out: Dict[BucketKey, List[int]] = {}
        for i, k in enumerate(self.keys):
            out.setdefault(k, []).append(i)
        return out

    def load(self, index: int) -> Dict[str, torch.Tensor]:
        return load_safetensors(os.path.join(self.dir, self.files[index]))


class BatchLoader:
    """Epoch iterator over same-shape batches. Shuffles inside buckets and across batches with a seeded RNG whose
    state advances per epoch; ``rank``/``world`` give each data-parallel rank a disjoint slice of the batch list;
    ``skip`` resumes in the middle of an epoch. Batches are assembled into reusable pinned buffers."""

    def __init__(self, cache: LatentCache, batch_size: int, seed: int = 0, drop_last: bool = True, rank: int = 0,
                 world: int = 1, pin: bool = True, dtype: torch.dtype = torch.bfloat16):
        self.cache, self.bs, self.seed, self.drop_last = cache, batch_size, seed, drop_last
        self.rank, self.world, self.dtype = rank, world, dtype
        self.pin = pin and torch.cuda.is_available()
        self._pinned: Dict[Tuple, torch.Tensor] = {}

    def batches_for_epoch(self, epoch: int) -> List[List[int]]:
        rng = random.Random(self.seed * 1_000_003 + epoch)
        out = []
        for key in sorted(self.cache.buckets(), key=lambda k: (k.channels, k.height, k.width, k.text_seq)):
            idx = list(self.cache.buckets()[key])
            rng.shuffle(idx)
            for i in range(0, len(idx), self.bs):
                b = idx[i:i + self.bs]
                if len(b) == self.bs or not self.drop_last:
                    out.append(b)
        rng.shuffle(out)
        usable = len(out) - len(out) % self.world if self.world > 1 else len(out)
        return out[self.rank:usable:self.world] if self.world > 1 else out

    def steps_per_epoch(self) -> int:
        return len(self.batches_for_epoch(0))

    def _stage(self, name: str, tensors: List[torch.Tensor], dtype) -> torch.Tensor:
        shape = (len(tensors),) + tuple(tensors[0].shape[1:])
        key = (name, shape, dtype)
        buf = self._pinned.get(key)
        if buf is None:
            buf = torch.empty(shape, dtype=dtype, pin_memory=self.pin)
            self._pinned[key] = buf
        for i, t in enumerate(tensors):
            buf[i].copy_(t[0])
        return buf

    def epoch(self, epoch: int, skip: int = 0) -> Iterator[Dict[str, torch.Tensor]]:
        for b in self.batches_for_epoch(epoch)[skip:]:
            samples = [self.cache.load(i) for i in b]
            batch = {
                LATENT_KEY: self._stage(LATENT_KEY, [s[LATENT_KEY] for s in samples], self.dtype),
                TEXT_KEY: self._stage(TEXT_KEY, [s[TEXT_KEY] for s in samples], self.dtype),
                MASK_KEY: self._stage(MASK_KEY, [s[MASK_KEY] for s in samples], torch.float32),
            }
            for opt in (LATENT_MASK_KEY, CONTROL_KEY):
                if all(opt in s for s in samples):
                    batch[opt] = self._stage(opt, [s[opt] for s in samples], self.dtype)
            batch["indices"] = b
            yield batch


class PixelCache:
    """Pixel-space cache (``pixel`` [3,H,W] in [-1,1], ``cap_feats`` [1,seq,F] with per-sample seq, no mask)."""

    def __init__(self, directory: str):
        self.dir = directory
        self.files = sorted(f for f in os.listdir(directory) if f.endswith(".safetensors"))
        if not self.files:
            raise FileNotFoundError(f"no cache samples in {directory}")

    def __len__(self):
        return len(self.files)

    def load(self, index: int):
        d = load_safetensors(os.path.join(self.dir, self.files[index]))
        if PIXEL_KEY not in d or CAP_FEATS_KEY not in d:
            raise KeyError(f"{self.files[index]}: pixel cache needs '{PIXEL_KEY}' and '{CAP_FEATS_KEY}'")
        if d[PIXEL_KEY].dim() != 3:
            raise ValueError("pixel must be [3,H,W]")
        return d
