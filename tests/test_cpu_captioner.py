"""Ideogram-4 structured-caption formatter and the prompt / reply glue (host only)."""
import json
import os

import pytest

from mojodiffusion_b200 import captioner as C


def _caption():
    return {
        "aspect_ratio": "16:9",
        "compositional_deconstruction": {
            "elements": [
                {"desc": "a red kite", "color_palette": ["#f00", "#FF0000", "bad", "#00ff00"], "bbox": [10, 20, 300, 400], "note": 1},
                {"type": "text", "desc": "headline", "text": "SALE", "bbox": [0, 0, 100, 1000]},
            ],
            "background": "a pale sky",
            "extra": True,
        },
        "style_description": {"medium": " Photo. ", "art_style": "film grain", "lighting": "soft", "aesthetics": "calm",
                              "color_palette": ["#abc"] + ["#%06x" % i for i in range(40)]},
        "high_level_description": "A kite over a beach",
        "seed": 7,
    }


def test_digest_orders_keys_migrates_branch_and_cleans_palettes():
    out = C.digest_caption_string(json.dumps(_caption()))
    d = json.loads(out)
    assert " " not in out.split('"A kite')[0]                                       # compact separators
    assert list(d) == ["high_level_description", "style_description", "compositional_deconstruction", "seed"]
    st = d["style_description"]
    assert list(st) == ["aesthetics", "lighting", "photo", "medium", "color_palette"]   # photograph branch, art_style -> photo
    assert st["medium"] == "photograph" and st["photo"] == "film grain"
    assert st["color_palette"][0] == "#AABBCC" and len(st["color_palette"]) == C.MAX_IMAGE_PALETTE
    decon = d["compositional_deconstruction"]
    assert list(decon) == ["background", "elements", "extra"]
    e0, e1 = decon["elements"]
    assert list(e0) == ["type", "bbox", "desc", "color_palette", "note"] and e0["type"] == "obj"
    assert e0["color_palette"] == ["#FF0000", "#00FF00"]
    assert list(e1) == ["type", "bbox", "text", "desc"]
    # art branch: a non-photo medium keeps art_style and puts medium first
    cap = _caption()
    cap["style_description"]["medium"] = "3D-Render"
    st = json.loads(C.digest_caption_string(json.dumps(cap)))["style_description"]
    assert list(st)[:4] == ["aesthetics", "lighting", "medium", "art_style"] and st["medium"] == "3d_render"


def test_prose_and_non_captions_pass_through_unchanged():
    for text in ("a cat on a mat", "  {not json", '{"a": 1}', '[1, 2]', '{"compositional_deconstruction": 3}', ""):
        assert C.digest_caption_string(text) is text or C.digest_caption_string(text) == text
        assert not C.is_ideogram_caption_str(text)
    assert C.is_ideogram_caption_str(' {"compositional_deconstruction": {}} ')


def test_scalar_helpers():
    assert C.canon_medium(" Graphic-Design. ") == "graphic_design" and C.canon_medium(" oil pastel ") == "oil pastel"
    assert C.is_photo_medium("PHOTO") and not C.is_photo_medium("painting")
    assert C.normalize_hex(" #1aF ") == "#11AAFF" and C.normalize_hex("#12345") is None and C.normalize_hex(5) is None
    assert C.sanitize_palette(["#fff", "#FFFFFF", "x", "#000"], 5) == ["#FFFFFF", "#000000"]
    assert C.swap_bbox_xy_in_text('x "bbox" : [ -5, 2000 ,3.5,4 ] y "bbox":[1,2]') == 'x "bbox":[4,0,1000,4] y "bbox":[1,2]'
    assert C.compute_aspect_ratio(1920, 1080) == "16:9" and C.compute_aspect_ratio(0, 5) == "1:1"
    assert C.compute_aspect_ratio(1000, 333) == "3:1"


def test_prompt_building_and_reply_glue():
    p = C.image_caption_prompt("  ", "3:2", template="AR={{aspect_ratio}} I={{user_instructions}} AR2={{aspect_ratio}}")
    assert p == "AR=3:2 I=None. AR2=3:2"
    q = C.upsample_caption_prompt("1:1", " a {{aspect_ratio}} fox ", creative=True, instructions=" bold ",
                                  template="{{mode_directive}}|{{user_instructions}}|{{aspect_ratio}}|{{original_prompt}}")
    assert q.endswith("|bold|1:1| a {{aspect_ratio}} fox ") and q.startswith(C.glue.CREATIVE_DIRECTIVE)
    reply = 'Sure!\n```json\n{"compositional_deconstruction":{"elements":[{"bbox":["100",200,400.4,800],"desc":"d"},{"bbox":[5,5,5,9],"desc":"flat"},{"bbox":[1,2,3],"desc":"short"}],"background":"b"},"high_level_description":"h"}\n```\ntrailing }'
    gen = C.StubGenerator(reply)
    pretty = C.caption_from_image_reply(gen.generate(p))
    d = json.loads(pretty)
    assert pretty.startswith('{\n  "high_level_description": "h",')
    els = d["compositional_deconstruction"]["elements"]
    assert els[0]["bbox"] == [200, 100, 800, 400] and "bbox" not in els[1] and "bbox" not in els[2]
    one_line = C.caption_from_idea_reply(reply)
    assert "\n" not in one_line and json.loads(one_line)["compositional_deconstruction"]["elements"][0]["bbox"] == [100, 200, 400, 800]
    assert C.caption_from_idea_reply("no json here") is None
    assert C.caption_from_image_reply('broken {"bbox":[1,2,3,4]') == 'broken {"bbox":[2,1,4,3]'
    assert C.normalize_item("  fox ", "1:1") == ("  fox ", "1:1")
    assert C.normalize_item({"prompt": "owl", "aspect_ratio": 16}, "4:3") == ("owl", "4:3")
    assert C.normalize_item({"prompt": "owl", "aspect_ratio": "2:1"}, "4:3") == ("owl", "2:1")
    assert C.normalize_item({"prompt": " "}, "1:1") is None and C.normalize_item(3, "1:1") is None


@pytest.mark.skipif(not os.environ.get("MDB_CAPTION_REFS"), reason="set MDB_CAPTION_REFS to a directory holding "
                    "ideogram_caption_adv_fixtures.json / ideogram_bc_glue_adv_fixtures.json")
def test_against_fixture_files():
    root = os.environ["MDB_CAPTION_REFS"]
    a = json.load(open(os.path.join(root, "ideogram_caption_adv_fixtures.json")))
    fa = {"digest_caption_string": C.digest_caption_string, "swap_bbox_xy_in_text": C.swap_bbox_xy_in_text,
          "canon_medium": C.canon_medium, "normalize_hex": C.normalize_hex, "is_ideogram_caption_str": C.is_ideogram_caption_str}
    for name, cases in a.items():
        for c in cases:
            assert fa[name](c["in"]) == c["out"], (name, c["in"])
    b = json.load(open(os.path.join(root, "ideogram_bc_glue_adv_fixtures.json")))
    fb = {"b_extract_json_adv": C.extract_json, "c_extract_json_adv": C.extract_json, "b_full_glue_adv": C.caption_from_image_reply,
          "c_full_glue_adv": C.caption_from_idea_reply, "b_convert_bbox_coerce": C.convert_bbox_xyxy,
          "c_sanitize_bbox_coerce": C.sanitize_bbox_yxyx}
    for name, cases in b.items():
        for c in cases:
            assert fb[name](c["in"]) == c["out"], (name, c["in"])
