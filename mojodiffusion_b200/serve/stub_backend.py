"""CPU stand-in backend: no model, no GPU. ``steps`` simulated denoise steps, then a real PNG (seed-driven gradient with
stripes and a white frame) with the generation parameters embedded. An init image tints the blue plane by ``creativity``
so img2img parameters are visible end to end. Failure injection for tests, by prompt keyword: ``__fail__`` fails at
the middle step, ``__exit__`` makes the process exit non-zero mid-job, ``__hang__`` stops sending events (the control
plane's cancel / kill path must cope) (serenitymojo/serve/stub_backend.mojo:1-140)."""
from __future__ import annotations

import os
import time

import numpy as np

from ..io.png import encode_png
from .backend import GenBackend, JobParams, StepResult, reject_unsupported_common


def render_stub_image(p: JobParams) -> np.ndarray:
    h, w = p.height, p.width
    ys, xs = np.mgrid[0:h, 0:w]
    s = abs(int(p.seed))
    img = np.zeros((h, w, 3), dtype=np.uint8)
    img[..., 0] = (xs * 255) // max(1, w - 1)
    img[..., 1] = (ys * 255) // max(1, h - 1)
    blue = 40 + (((xs + ys) // 16 + s) % 3) * 80 + (s % 16)
    if p.init_image:
        blue = np.full_like(blue, int(p.creativity * 255.0))
    img[..., 2] = np.clip(blue, 0, 255)
    img[:2] = img[-2:] = 255
    return img


class StubBackend(GenBackend):
    name = "stub"

    def __init__(self, step_sleep_s: float = 0.02):
        self.sleep = step_sleep_s
        self.p: JobParams | None = None
        self.cur = 0
        self._cancel = False

    def start(self, params: JobParams) -> None:
        reject_unsupported_common(params, reference=True)
        self.p, self.cur, self._cancel = params, 0, False

    def step(self) -> StepResult:
        p = self.p
        assert p is not None, "step() without start()"
        if self._cancel:
            self.p = None
            return StepResult("cancelled")
        if "__hang__" in p.prompt and self.cur >= 1:
            time.sleep(0.05)                 # alive, but silent: nothing is reported any more
            return _SILENT
        if self.cur < p.steps:
            time.sleep(self.sleep)
            self.cur += 1
            if "__fail__" in p.prompt and self.cur == max(1, p.steps // 2):
                self.p = None
                return StepResult("failed", error="stub: injected failure")
            if "__exit__" in p.prompt and self.cur == max(1, p.steps // 2):
                os._exit(7)
            return StepResult("progress", self.cur, p.steps, "denoise")
        path = p.output_path()
        os.makedirs(p.out_dir or ".", exist_ok=True)
        data = encode_png(render_stub_image(p), {"serenity.genparams.v1": p.genparams_text()})
        tmp = path + ".tmp"
        with open(tmp, "wb") as f:
            f.write(data)
        os.replace(tmp, path)
        self.p = None
        return StepResult("done", output_path=path)


_SILENT = StepResult("silent")
