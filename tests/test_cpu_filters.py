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


def test_reference_table_against_external_numpy_oracles():
    """Optional: MDB_FILTER_REFS=<directory holding shader_denoise_ref.py, shader_color_adv_ref.py, shader_effects_ref.py>
    imports those numpy oracles and checks every entry of ``filters.REFERENCE`` (the table the CUDA kernels are tested
    against) on the shared test image: at most a handful of 8-bit output values may differ by one step."""
    import importlib.util
    import os

    import numpy as np
    import pytest

    from mojodiffusion_b200.ops import filters as F
    d = os.environ.get("MDB_FILTER_REFS")
    if not d:
        pytest.skip("MDB_FILTER_REFS not set")

    def load(name):
        spec = importlib.util.spec_from_file_location(name, os.path.join(d, name + ".py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod
    den, col, eff = load("shader_denoise_ref"), load("shader_color_adv_ref"), load("shader_effects_ref")
    img = F.test_image()
    for mod in (den, col, eff):
        assert np.array_equal(img, mod.build_test_image())
    cases = {
        "smartdenoise": lambda: den.smartdenoise(img), "hqdn3d": lambda: den.hqdn3d(img), "guided": lambda: den.guided(img),
        "deband": lambda: den.deband(img),
        "colorbalance": lambda: col.colorbalance(img, (0.3, -0.2, 0.1, -0.1, 0.25, -0.15, 0.2, -0.1, 0.3)),
        "cas": lambda: col.cas(img, 0.8), "usm": lambda: col.usm(img, 3.0, 1.5, 0.0), "lut3d": lambda: col.lut3d(img, col.build_identity_lut()),
        "waterripple": lambda: eff.waterripple(img, 24.0, 0.03), "soul": lambda: eff.soul(img, 0.37, 1, 1.8, 0.4, 0),
        "sway": lambda: eff.sway(img, 7.4, 20.0, 20.0, 1), "star": lambda: eff.star(img, 0.37, 10.0, 2.0, 1.0, 0.1, 0.9),
        "lighting": lambda: eff.lighting(img, 0.37, 1, 0.3, 0.3), "jitter": lambda: eff.jitter(img, 0.37, 1, 1.1, 0.02, 0),
    }
    assert set(cases) == set(F.REFERENCE)
    report = {}
    for name, fn in cases.items():
        a, b = F.to_u8(fn()), F.to_u8(F.REFERENCE[name](img))
        diff = np.abs(a.astype(np.int32) - b.astype(np.int32))
        report[name] = (int((diff > 0).sum()), int(diff.max()))
        assert diff.max() <= 1 and (diff > 0).mean() < 1e-3, f"{name}: {report[name]} of {a.size} values differ"
    print(report)
