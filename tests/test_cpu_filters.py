"""Image filters, CPU statement: structural properties that hold whatever the parameters are."""
import numpy as np
import pytest
import torch

from mojodiffusion_b200.ops import filters as F


@pytest.fixture(scope="module")
def img():
    return torch.from_numpy(F.test_image())


@pytest.mark.parametrize("name", sorted(F.OPS))
def test_filter_runs_and_keeps_shape_and_alpha(img, name):
    out = F.image_filter(name, img)
    assert out.shape == img.shape and out.dtype == torch.float32
    if name not in ("soul",):
        assert torch.equal(out[..., 3], img[..., 3]) or name in ("waterripple", "sway", "jitter")
    finite = torch.isfinite(out)
    assert finite.all() or name == "star"                      # star's core is 0.05 / distance: infinite at a centre
    assert F.psnr_u8(out.numpy(), img.numpy()) > 8.0            # still recognisably the same picture


def test_known_identities(img):
    a = img.numpy()
    assert F.psnr_u8(F.ref_lut3d(a), a) == float("inf")                           # identity LUT
    inv = F.identity_lut()[..., [2, 1, 0, 3]].copy()                              # swap red and blue
    sw = F.ref_lut3d(a, inv)
    assert np.abs(sw[..., 0] - a[..., 2]).max() < 1e-5 and np.abs(sw[..., 2] - a[..., 0]).max() < 1e-5
    assert F.psnr_u8(F.ref_colorbalance(a, (0,) * 9), a) == float("inf")
    assert F.psnr_u8(F.ref_usm(a, amount=0.0), a) == float("inf")
    assert F.psnr_u8(F.ref_soul(a, max_alpha=1.0, progress=0.0), a) == float("inf")
    assert F.psnr_u8(F.ref_sway(a, strength=0.0), a) == float("inf")
    flat = np.full((32, 32, 4), 0.5, np.float32)
    for name in ("smartdenoise", "guided", "deband", "cas", "usm"):
        assert np.abs(F.REFERENCE[name](flat)[..., :3] - 0.5).max() < 1e-4, name  # a flat image stays flat
    lut = F.hqdn3d_lut()
    assert lut.shape == (4, 8192) and lut.dtype == np.int32 and abs(int(lut[0, 4096])) < 16
    k = F.gaussian_taps(3.0)
    assert k.shape == (15,) and abs(float(k.sum()) - 1.0) < 1e-6 and k[7] == k.max()
    with pytest.raises(KeyError):
        F.image_filter("sepia", img)
