"""Host-only caption tooling for the Ideogram-4 structured-caption format (no GPU, no model): the deterministic
normaliser / minifier and the prompt / JSON-extraction glue around a pluggable caption generator."""
from .ideogram_caption import (MAX_ELEMENT_PALETTE, MAX_IMAGE_PALETTE, MEDIUM_OPTIONS, canon_medium, digest_caption_string,
                               is_ideogram_caption_str, is_photo_medium, normalize_caption_dict, normalize_element,
                               normalize_hex, normalize_style, sanitize_palette, swap_bbox_xy_in_text, to_model_string)
from .glue import (CaptionGenerator, StubGenerator, caption_from_image_reply, caption_from_idea_reply, compute_aspect_ratio,
                   convert_bbox_xyxy, extract_json, image_caption_prompt, normalize_item, sanitize_bbox_yxyx,
                   upsample_caption_prompt)
