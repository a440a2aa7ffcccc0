"""Image filter CUDA kernels against the numpy statement of the same formulas: PSNR >= 40 dB on 8-bit output."""
import numpy as np
import pytest
import torch

from mojodiffusion_b200.ops import filters as F
from mojodiffusion_b200.ops import native

pytestmark = pytest.mark.gpu


def _images():
    rng = np.random.default_rng(0)
    ys, xs = np.mgrid[0:200, 0:312].astype(np.float32)
    smooth = np.stack([0.5 + 0.4 * np.sin(xs / 23.0), 0.5 + 0.4 * np.cos(ys / 17.0), (xs + ys) / 512.0, np.ones_like(xs)], -1)
    noisy = np.clip(smooth + rng.normal(0, 0.03, smooth.shape).astype(np.float32) * np.array([1, 1, 1, 0], np.float32), 0, 1)
    return {"synthetic128": F.test_image(), "noisy200x312": noisy.astype(np.float32)}


@pytest.mark.parametrize("name", sorted(F.OPS))
def test_filter_kernel_matches_reference(name):
    native.load(True)
    for label, a in _images().items():
        ref = F.REFERENCE[name](a)
        got = F.image_filter(name, torch.from_numpy(a).cuda()).cpu().numpy()
        p = F.psnr_u8(got, ref)
        frac = float((F.to_u8(got) != F.to_u8(ref)).mean())
        assert p >= 40.0, f"{name} on {label}: PSNR {p:.2f} dB, {frac:.4%} of bytes differ"
    native.check_status()
