"""Deterministic formatter of Ideogram-4 structured captions.

A structured caption is a JSON object with ``high_level_description``, ``style_description`` and
``compositional_deconstruction`` (background + elements with bounding boxes). ``digest_caption_string`` normalises such
a caption (key order, photo / art-style branch by medium, canonical medium tokens, upper-case de-duplicated hex
palettes, ``aspect_ratio`` dropped) and returns the compact model-ready string; any text that is not such an object is
returned unchanged, byte for byte. Key order is load-bearing: Python dicts keep insertion order, and the output is
``json.dumps(..., separators=(",", ":"), ensure_ascii=False)``.

Behaviour follows the reference's serenitymojo/captioner/ideogram_caption.mojo:739-1350 (itself a port of
ai-toolkit's ``toolkit/ideogram_caption.py``).
"""
from __future__ import annotations

import json
import re
from typing import Any, List, Optional

MAX_IMAGE_PALETTE = 16      # style_description.color_palette
MAX_ELEMENT_PALETTE = 5     # per-element color_palette
MEDIUM_OPTIONS = ("photograph", "illustration", "3d_render", "painting", "graphic_design")

_MEDIUM_ALIASES = {
    "photograph": "photograph", "photo": "photograph",
    "illustration": "illustration",
    "3d render": "3d_render", "3d_render": "3d_render", "3d-render": "3d_render", "3drender": "3d_render",
    "render": "3d_render", "3d": "3d_render",
    "painting": "painting",
    "graphic design": "graphic_design", "graphic_design": "graphic_design", "graphic-design": "graphic_design",
    "graphic": "graphic_design",
}
_HEX6 = re.compile(r"^#[0-9a-fA-F]{6}$")
_HEX3 = re.compile(r"^#[0-9a-fA-F]{3}$")
_NUM = r"(-?\d+(?:\.\d+)?)"
_BBOX_TEXT = re.compile(r'"bbox"\s*:\s*\[\s*' + _NUM + r"\s*,\s*" + _NUM + r"\s*,\s*" + _NUM + r"\s*,\s*" + _NUM + r"\s*\]")


def canon_medium(medium: Any) -> Any:
    """Official medium token when the text is a known alias, otherwise the stripped text (custom mediums are kept)."""
    if not isinstance(medium, str):
        return medium
    key = medium.strip().rstrip(".").strip().lower()
    return _MEDIUM_ALIASES.get(key, medium.strip())


def is_photo_medium(medium: Any) -> bool:
    return canon_medium(medium) == "photograph"


def normalize_hex(color: Any) -> Optional[str]:
    """``#RRGGBB`` in upper case (``#RGB`` expanded) or None when the text is not a hex colour."""
    if not isinstance(color, str):
        return None
    s = color.strip()
    if _HEX6.match(s):
        return "#" + s[1:].upper()
    if _HEX3.match(s):
        return "#" + "".join(ch * 2 for ch in s[1:]).upper()
    return None


def sanitize_palette(values: Any, max_len: int) -> List[str]:
    """Unique valid colours in their first-seen order, at most ``max_len``."""
    out: List[str] = []
    if not isinstance(values, (list, tuple)):
        return out
    for v in values:
        h = normalize_hex(v)
        if h is None or h in out:
            continue
        out.append(h)
        if len(out) >= max_len:
            break
    return out


def normalize_style(style: Any) -> Any:
    """style_description in the strict order aesthetics, lighting, then (photo, medium) for photographs or
    (medium, art_style) otherwise, then color_palette, then unknown keys; the old always-``photo`` shape migrates by medium."""
    if not isinstance(style, dict):
        return style
    raw_medium = style.get("medium")
    medium = canon_medium(raw_medium) if isinstance(raw_medium, str) else ""
    has_medium = raw_medium is not None
    photo, art = style.get("photo"), style.get("art_style")
    if has_medium and medium in MEDIUM_OPTIONS:
        photo_branch = medium == "photograph"
    else:
        photo_branch = not (bool(art) and not bool(photo))
    emit_medium = medium if isinstance(raw_medium, str) else raw_medium
    out = {}
    for k in ("aesthetics", "lighting"):
        if k in style:
            out[k] = style[k]
    if photo_branch:
        if photo:
            out["photo"] = photo
        elif art:
            out["photo"] = art
        if has_medium:
            out["medium"] = emit_medium
    else:
        if has_medium:
            out["medium"] = emit_medium
        if art:
            out["art_style"] = art
        elif photo:
            out["art_style"] = photo
    pal = sanitize_palette(style.get("color_palette"), MAX_IMAGE_PALETTE)
    if pal:
        out["color_palette"] = pal
    for k, v in style.items():
        if k not in ("aesthetics", "lighting", "photo", "art_style", "medium", "color_palette"):
            out[k] = v
    return out


def normalize_element(el: Any) -> Any:
    """Element keys in schema order: type, bbox, (text,) desc, color_palette, then the rest; bbox stays as it is."""
    if not isinstance(el, dict):
        return el
    etype = el.get("type", "obj") if "type" in el else "obj"
    out = {"type": etype}
    if el.get("bbox") is not None:
        out["bbox"] = el["bbox"]
    if etype == "text" and "text" in el:
        out["text"] = el["text"]
    if "desc" in el:
        out["desc"] = el["desc"]
    pal = sanitize_palette(el.get("color_palette"), MAX_ELEMENT_PALETTE)
    if pal:
        out["color_palette"] = pal
    for k, v in el.items():
        if k not in out and k != "color_palette":
            out[k] = v
    return out


def normalize_caption_dict(data: Any) -> Any:
    """Top-level order high_level_description, style_description, compositional_deconstruction, rest; no aspect_ratio."""
    if not isinstance(data, dict):
        return data
    out = {}
    if "high_level_description" in data:
        out["high_level_description"] = data["high_level_description"]
    if "style_description" in data:
        out["style_description"] = normalize_style(data["style_description"])
    decon = data.get("compositional_deconstruction")
    if isinstance(decon, dict):
        nd = {}
        if "background" in decon:
            nd["background"] = decon["background"]
        if isinstance(decon.get("elements"), list):
            nd["elements"] = [normalize_element(e) for e in decon["elements"]]
        for k, v in decon.items():
            if k not in ("background", "elements"):
                nd[k] = v
        out["compositional_deconstruction"] = nd
    elif decon is not None:
        out["compositional_deconstruction"] = decon
    for k, v in data.items():
        if k not in ("high_level_description", "style_description", "compositional_deconstruction", "aspect_ratio"):
            out[k] = v
    return out


def to_model_string(data: Any) -> str:
    return json.dumps(data, separators=(",", ":"), ensure_ascii=False)


def _clamp_1000(token: str) -> int:
    return max(0, min(1000, round(float(token))))      # round(): half to even


def swap_bbox_xy_in_text(text: str) -> str:
    """Rewrite every ``"bbox":[x1,y1,x2,y2]`` of a raw text to the stored ``[y1,x1,y2,x2]`` order, each value clamped to
    0..1000 and each axis ordered, without parsing the surrounding JSON; everything else stays byte for byte."""
    def fix(m: "re.Match") -> str:
        x1, y1, x2, y2 = (_clamp_1000(g) for g in m.groups())
        (x1, x2), (y1, y2) = sorted((x1, x2)), sorted((y1, y2))
        return f'"bbox":[{y1},{x1},{y2},{x2}]'
    return _BBOX_TEXT.sub(fix, text)


def _load_caption(text: str) -> Optional[dict]:
    t = text.strip()
    if not t.startswith("{"):
        return None
    try:
        d = json.loads(t)
    except (ValueError, RecursionError):
        return None
    if isinstance(d, dict) and isinstance(d.get("compositional_deconstruction"), dict):
        return d
    return None


def is_ideogram_caption_str(text: str) -> bool:
    return _load_caption(text) is not None


def digest_caption_string(text: str) -> str:
    """Compact normalised caption, or the input unchanged when it is not a structured caption."""
    d = _load_caption(text)
    return text if d is None else to_model_string(normalize_caption_dict(d))
