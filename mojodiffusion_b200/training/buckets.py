"""Aspect-ratio buckets under a pixel-area budget: ladder -> (W, H) canvases, and stage-time assignment of one image
(closest ladder aspect, first wins on ties; resize keeping the original aspect; centre crop). Python's own ``round``
(half-to-even, exact 2-decimal) gives the rounding the bucket keys are defined by
(serenitymojo/training/aspect_buckets.mojo:1-40,150-260)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Sequence


def round_to_multiple(value: float, multiple: int) -> int:
    return max(multiple, round(value / multiple) * multiple)


def default_aspect_ladder() -> List[float]:
    return [1.0, round(4 / 3, 2), round(3 / 4, 2), round(16 / 9, 2), round(9 / 16, 2), round(3 / 2, 2), round(2 / 3, 2)]


def pixel_resolution(megapixels: float, align: int) -> int:
    return round_to_multiple(math.sqrt(megapixels * 1e6), align)


@dataclass
class AspectBucket:
    aspect: float
    width: int
    height: int
    aspect_key_x100: int


@dataclass
class BucketAssignment:
    bucket_index: int
    aspect: float
    target_w: int
    target_h: int
    inter_w: int
    inter_h: int
    crop_x: int
    crop_y: int
    aspect_key_x100: int


def _size_by_area(aspect: float, megapixels: float, w0: int, h0: int, align: int):
    edge = round_to_multiple(float(int(math.sqrt(megapixels * 1e6))), align)
    if aspect == 1.0 and w0 == h0:
        return edge, edge, edge, edge, 1.0
    wt = round_to_multiple(edge * math.sqrt(aspect), align)
    ht = round_to_multiple(edge / math.sqrt(aspect), align)
    adj = round(wt / ht, 2)
    raw = w0 / h0
    if wt < ht:
        wi = wt
        hi = int(wi / raw)
    else:
        hi = ht
        wi = int(hi * raw)
    if wt > wi or ht > hi:                      # intermediary too small: grow once along the original aspect
        if wt > wi:
            wd = wt - wi
            hd = int(wd / raw)
        else:
            hd = ht - hi
            wd = int(hd * raw)
        hi += hd
        wi += wd
    return wt, ht, wi, hi, adj


def _canvas(aspect: float, megapixels: float, align: int):
    px = pixel_resolution(megapixels, align)
    # a synthetic source of exactly that aspect: the canvas depends only on (aspect, area, align)
    wt, ht, _, _, adj = _size_by_area(aspect, megapixels, int(round(aspect * 1000)), 1000, align)
    if adj == 1.0:
        wt = ht = px
    return wt, ht, adj


def generate_aspect_buckets(megapixels: float = 1.0, align: int = 64, ladder: Sequence[float] = None) -> List[AspectBucket]:
    if align % 2:
        raise ValueError("align must be even")
    out, seen = [], set()
    for a in (ladder or default_aspect_ladder()):
        if not a > 0:
            raise ValueError("ladder aspect must be > 0")
        wt, ht, adj = _canvas(a, megapixels, align)
        if (wt, ht) in seen:
            continue
        seen.add((wt, ht))
        out.append(AspectBucket(a, wt, ht, int(round(adj * 100))))
    return out


def assign_aspect_bucket(w0: int, h0: int, megapixels: float = 1.0, align: int = 64, ladder: Sequence[float] = None) -> BucketAssignment:
    ladder = list(ladder or default_aspect_ladder())
    ar = round(w0 / h0, 2)
    idx = min(range(len(ladder)), key=lambda i: abs(ladder[i] - ar))
    a = ladder[idx]
    wt, ht, wi, hi, adj = _size_by_area(a, megapixels, w0, h0, align)
    if adj == 1.0:
        px = pixel_resolution(megapixels, align)
        wt = ht = px
        # square canvas: the intermediary keeps the source aspect with its short side on the canvas edge
        if w0 >= h0:
            hi, wi = px, max(px, int(px * w0 / h0))
        else:
            wi, hi = px, max(px, int(px * h0 / w0))
    return BucketAssignment(idx, a, wt, ht, wi, hi, (wi - wt) // 2, (hi - ht) // 2, int(round(round(wt / ht, 2) * 100)))
