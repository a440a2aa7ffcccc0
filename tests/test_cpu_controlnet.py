"""Z-Image ControlNet on the tiny architecture: zero-initialised projections reproduce the base, hints land on the named
layers, only the control branch trains, checkpoint round trip, and the train CLI's CONTROLNET method."""
import json
import os
import subprocess
import sys

import torch

from mojodiffusion_b200.models.single_dit import SingleStreamDiT, tiny_single_dit_config
from mojodiffusion_b200.models.zimage_controlnet import (ControlledZImage, ZImageControlNet, control_places, load_controlnet,
                                                        save_controlnet)
from mojodiffusion_b200.training.dataset import write_sample

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _base():
    cfg = tiny_single_dit_config()
    base = SingleStreamDiT(cfg, dtype=torch.float32)
    with torch.no_grad():
        base.init_weights(0)
    return cfg, base


def _inputs(cfg, B=2, hw=(4, 4), T=6):
    g = torch.Generator().manual_seed(2)
    img = torch.randn(B, hw[0] * hw[1], cfg.in_channels, generator=g)
    ctrl = torch.randn(B, hw[0] * hw[1], cfg.in_channels, generator=g)
    cap = torch.randn(B, T, cfg.cap_dim, generator=g)
    return img, ctrl, cap, torch.tensor([0.2, 0.8])[:B], hw


def test_places_and_zero_init_reproduces_the_base():
    assert control_places(30, 6) == [0, 5, 10, 15, 20, 25] and control_places(4, 2) == [0, 2]
    cfg, base = _base()
    net = ZImageControlNet(cfg, 2, dtype=torch.float32).init_from_base(base)
    model = ControlledZImage(base, net)
    img, ctrl, cap, t, hw = _inputs(cfg)
    with torch.no_grad():
        ref = base(img, cap, t, hw)
        out = model(img, cap, t, hw, None, control=ctrl)
        assert torch.equal(ref, out)                                            # zero projections: no contribution
        assert torch.equal(net.control_layers[1].attention.to_q.weight, base.layers[net.places[1]].attention.to_q.weight)
        net.control_layers[0].after_proj.weight.normal_(0, 0.05)
        out2 = model(img, cap, t, hw, None, control=ctrl)
        assert (out2 - ref).abs().max() > 1e-4
        net.control_layers[0].before_proj.weight.normal_(0, 0.05)         # with before_proj at zero the control image is unseen
        out2 = model(img, cap, t, hw, None, control=ctrl)
        out3 = model(img, cap, t, hw, None, control=ctrl * 0.5)
        assert (out3 - out2).abs().max() > 1e-6                                  # the control image matters
        model.scale = 0.0
        assert torch.allclose(model(img, cap, t, hw, None, control=ctrl), ref, atol=1e-6)
    keys = set(net.state_dict())
    assert {"control_layers.0.before_proj.weight", "control_layers.1.after_proj.bias", "control_all_x_embedder.2-1.weight",
            "control_noise_refiner.0.attention.to_q.weight", "control_layers.0.adaLN_modulation.0.weight"} <= keys
    assert "control_layers.1.before_proj.weight" not in keys


def test_only_the_control_branch_receives_gradients_and_learns(tmp_path):
    cfg, base = _base()
    net = ZImageControlNet(cfg, 2, dtype=torch.float32).init_from_base(base)
    model = ControlledZImage(base, net)
    img, ctrl, cap, t, hw = _inputs(cfg)
    target = torch.randn(img.shape, generator=torch.Generator().manual_seed(9)) * 0.1
    opt = torch.optim.AdamW(net.parameters(), lr=3e-3)
    losses = []
    for _ in range(12):
        opt.zero_grad()
        loss = (model(img, cap, t, hw, None, control=ctrl) - target).square().mean()
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert all(p.grad is None for p in base.parameters())
    assert net.control_layers[0].before_proj.weight.grad is not None
    assert losses[-1] < losses[0]
    path = str(tmp_path / "control.safetensors")
    save_controlnet(net, path)
    net2 = ZImageControlNet(cfg, 2, dtype=torch.float32)
    load_controlnet(net2, path)
    with torch.no_grad():
        a = model(img, cap, t, hw, None, control=ctrl)
        b = ControlledZImage(base, net2)(img, cap, t, hw, None, control=ctrl)
    assert torch.equal(a, b)


def test_train_cli_controlnet_method(tmp_path):
    tmp = str(tmp_path)
    cfg = tiny_single_dit_config()
    C = cfg.in_channels // 4
    g = torch.Generator().manual_seed(0)
    cache = os.path.join(tmp, "cache")
    os.makedirs(cache)
    for i in range(4):
        write_sample(os.path.join(cache, f"s{i}.safetensors"), torch.randn(1, C, 8, 8, generator=g), torch.randn(1, 16, cfg.cap_dim, generator=g),
                     torch.ones(1, 16), control_latent=torch.randn(1, C, 8, 8, generator=g))
    ws = os.path.join(tmp, "ws")
    conf = {"model_type": "zimage", "training_method": "CONTROLNET", "controlnet_layers": 2, "learning_rate": 1e-3, "batch_size": 2,
            "max_steps": 3, "save_every": 0, "cache_dir": cache, "workspace_dir": ws, "output_model_destination": "out/control.safetensors",
            "gradient_checkpointing": "OFF", "seed": 1}
    path = os.path.join(tmp, "config.json")
    json.dump(conf, open(path, "w"))
    env = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, "-m", "mojodiffusion_b200.cli.train", path, "--tiny", "--quiet"], capture_output=True, text=True,
                       env=env, cwd=ROOT, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    rep = json.loads(r.stdout.strip().splitlines()[-1])
    assert rep["global_step"] == 3 and os.path.isfile(rep["output"])
    from mojodiffusion_b200.io.safetensors_io import load_safetensors
    sd = load_safetensors(rep["output"])
    assert "control_layers.0.before_proj.weight" in sd and not any(k.startswith("layers.") for k in sd)
    assert float(sd["control_layers.0.after_proj.weight"].float().abs().sum()) > 0         # left its zero start
    # a cache without control latents is refused up front
    write_sample(os.path.join(cache, "s9.safetensors"), torch.randn(1, C, 8, 8), torch.randn(1, 16, cfg.cap_dim), torch.ones(1, 16))
    r = subprocess.run([sys.executable, "-m", "mojodiffusion_b200.cli.train", path, "--tiny", "--quiet"], capture_output=True, text=True,
                       env=env, cwd=ROOT, timeout=600)
    assert r.returncode == 2 and "control_latent" in r.stderr
