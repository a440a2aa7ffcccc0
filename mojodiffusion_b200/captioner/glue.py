"""Prompt building and reply post-processing around a caption generator for the Ideogram-4 structured-caption format.

Two pipelines share the pieces: image -> caption (the generator sees boxes as [x1, y1, x2, y2]; they are stored as
[y1, x1, y2, x2], output pretty-printed) and idea -> caption (boxes already in stored order, output on one line). Both are
``build prompt -> generator -> extract_json -> per-element box repair -> normalize_caption_dict -> json.dumps``. The
generator is the only non-deterministic part and is pluggable (an OpenAI-compatible vision-language server in practice,
``StubGenerator`` in tests). Behaviour follows the reference's serenitymojo/captioner/ideogram_bc_glue.mojo:163-790.

The long system prompts are data, not code: pass their text, or set ``MDB_CAPTION_PROMPTS_DIR`` to a directory holding
``ideogram4_caption_prompt.txt`` / ``ideogram4_upsample_prompt.txt``; otherwise a short built-in template with the same
placeholders is used.
"""
from __future__ import annotations

import json
import math
import os
import re
from typing import Any, List, Optional, Protocol, Tuple

from .ideogram_caption import normalize_caption_dict, swap_bbox_xy_in_text

MAX_AR_DENOMINATOR = 16
_FENCE = re.compile(r"```(?:json)?\s*(.*?)```", re.DOTALL)

_IMAGE_TEMPLATE = (
    "Describe the image as one JSON object with the keys high_level_description, style_description and "
    "compositional_deconstruction (background, elements with type, bbox [x1, y1, x2, y2] on a 0-1000 grid, desc, "
    "color_palette). Aspect ratio: {{aspect_ratio}}. Additional instructions: {{user_instructions}}")
_IDEA_TEMPLATE = (
    "Expand the idea into one JSON object with the keys high_level_description, style_description and "
    "compositional_deconstruction (background, elements with type, bbox [y1, x1, y2, x2] on a 0-1000 grid, desc, "
    "color_palette).\n{{mode_directive}}\nAdditional instructions: {{user_instructions}}\nAspect ratio: "
    "{{aspect_ratio}}\nIdea: {{original_prompt}}")
FAITHFUL_DIRECTIVE = ("- Add only what the structure needs: a concrete background, bounding boxes and the required elements "
                      "or text. Add no subject, prop, story, mood or setting that the idea does not name.")
CREATIVE_DIRECTIVE = ("- Enrich the idea: add fitting detail, supporting elements, lighting and mood while keeping every "
                      "subject and every quoted text of the idea.")


def _template(name: str, builtin: str) -> str:
    d = os.environ.get("MDB_CAPTION_PROMPTS_DIR")
    if d:
        p = os.path.join(d, name)
        if os.path.isfile(p):
            with open(p, "r", encoding="utf-8") as f:
                return f.read()
    return builtin


def image_caption_prompt(caption_prompt: Optional[str], aspect_ratio: str, template: Optional[str] = None) -> str:
    """System prompt of the image -> caption pipeline: ``{{aspect_ratio}}`` then ``{{user_instructions}}`` (the stripped
    user text, or ``None.`` when there is none)."""
    t = template if template is not None else _template("ideogram4_caption_prompt.txt", _IMAGE_TEMPLATE)
    instr = (caption_prompt or "").strip() or "None."
    return t.replace("{{aspect_ratio}}", aspect_ratio).replace("{{user_instructions}}", instr)


def upsample_caption_prompt(aspect_ratio: str, original_prompt: str, creative: bool = False, instructions: str = "",
                            template: Optional[str] = None) -> str:
    """Prompt of the idea -> caption pipeline; substitution order mode_directive, user_instructions, aspect_ratio,
    original_prompt (the idea goes in verbatim)."""
    t = template if template is not None else _template("ideogram4_upsample_prompt.txt", _IDEA_TEMPLATE)
    t = t.replace("{{mode_directive}}", CREATIVE_DIRECTIVE if creative else FAITHFUL_DIRECTIVE)
    t = t.replace("{{user_instructions}}", instructions.strip() or "None.")
    return t.replace("{{aspect_ratio}}", aspect_ratio).replace("{{original_prompt}}", original_prompt)


def extract_json(raw: str) -> Optional[Any]:
    """The JSON value between the first ``{`` and the last ``}`` of a reply (inside its first code fence when it has
    one), or None."""
    text = raw.strip()
    m = _FENCE.search(text)
    if m:
        text = m.group(1).strip()
    start, end = text.find("{"), text.rfind("}")
    if start == -1 or end == -1 or end <= start:
        return None
    try:
        return json.loads(text[start:end + 1])
    except (ValueError, RecursionError):
        return None


def _four(bbox: Any) -> Optional[List[int]]:
    if not isinstance(bbox, (list, tuple)) or len(bbox) != 4:
        return None
    try:
        vals = [float(v) for v in bbox]
        return [max(0, min(1000, round(v))) for v in vals]
    except (TypeError, ValueError, OverflowError):
        return None


def convert_bbox_xyxy(bbox: Any) -> Optional[List[int]]:
    """[x1, y1, x2, y2] -> stored [y1, x1, y2, x2], clamped to 0..1000, each axis ordered; None when degenerate."""
    v = _four(bbox)
    if v is None:
        return None
    (x1, x2), (y1, y2) = sorted((v[0], v[2])), sorted((v[1], v[3]))
    return None if (y2 <= y1 or x2 <= x1) else [y1, x1, y2, x2]


def sanitize_bbox_yxyx(bbox: Any) -> Optional[List[int]]:
    """Stored-order box repaired in place (no swap); None when degenerate."""
    v = _four(bbox)
    if v is None:
        return None
    (y1, y2), (x1, x2) = sorted((v[0], v[2])), sorted((v[1], v[3]))
    return None if (y2 <= y1 or x2 <= x1) else [y1, x1, y2, x2]


def _repair(data: Any, fix) -> Any:
    if isinstance(data, dict) and isinstance(data.get("compositional_deconstruction"), dict):
        els = data["compositional_deconstruction"].get("elements")
        if isinstance(els, list):
            for el in els:
                if isinstance(el, dict) and "bbox" in el:
                    b = fix(el["bbox"])
                    if b is None:
                        del el["bbox"]          # the element stays, without a box
                    else:
                        el["bbox"] = b
    return normalize_caption_dict(data)


def caption_from_image_reply(raw: str) -> str:
    """Reply of the image pipeline -> pretty JSON caption; a reply without parseable JSON only gets its boxes swapped
    in the raw text."""
    d = extract_json(raw)
    if d is None:
        return swap_bbox_xy_in_text(raw)
    return json.dumps(_repair(d, convert_bbox_xyxy), indent=2, ensure_ascii=False)


def caption_from_idea_reply(raw: str) -> Optional[str]:
    """Reply of the idea pipeline -> one-line JSON caption, or None when the reply holds no JSON."""
    d = extract_json(raw)
    if d is None:
        return None
    return json.dumps(_repair(d, sanitize_bbox_yxyx), ensure_ascii=False)


def compute_aspect_ratio(width: int, height: int) -> str:
    """``w:h`` reduced by the gcd; when either side still exceeds 16 the closest p:q with q <= 16."""
    if width <= 0 or height <= 0:
        return "1:1"
    g = math.gcd(width, height)
    rw, rh = width // g, height // g
    if rw <= MAX_AR_DENOMINATOR and rh <= MAX_AR_DENOMINATOR:
        return f"{rw}:{rh}"
    target = width / height
    best = None
    for q in range(1, MAX_AR_DENOMINATOR + 1):
        p = max(1, round(target * q))
        err = abs(p / q - target)
        if best is None or err < best[0]:
            best = (err, p, q)
    return f"{best[1]}:{best[2]}"


def normalize_item(item: Any, default_aspect_ratio: str) -> Optional[Tuple[str, str]]:
    """A work item of the idea pipeline: a bare string, or a dict with ``prompt`` and an optional ``aspect_ratio`` ->
    (idea, aspect ratio); None for anything else or an empty idea."""
    if isinstance(item, str):
        idea, ar = item, default_aspect_ratio
    elif isinstance(item, dict) and isinstance(item.get("prompt"), str):
        idea = item["prompt"]
        a = item.get("aspect_ratio")
        ar = a if (isinstance(a, str) and a) else default_aspect_ratio
    else:
        return None
    return None if not idea.strip() else (idea, ar)


class CaptionGenerator(Protocol):
    def generate(self, prompt: str, image_b64: Optional[str] = None) -> str: ...


class StubGenerator:
    """Returns a fixed reply: drives the whole pipeline in tests without a model."""

    def __init__(self, canned: str):
        self.canned = canned

    def generate(self, prompt: str, image_b64: Optional[str] = None) -> str:
        return self.canned
