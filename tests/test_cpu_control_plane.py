"""Serving control plane, end to end on the CPU: the C++ server drives the Python stub worker over the socket pair.
Covers workflow lowering (own cases + an optional directory of request/lowered pairs), the wire contract, generate ->
progress socket -> PNG with embedded parameters, cancel, injected worker failures (failed job, process exit, silence),
lazy respawn, queue operations, uploads, gallery, presets."""
import base64
import glob
import hashlib
import json
import os
import socket
import struct
import subprocess
import sys
import time
import urllib.error
import urllib.request

import pytest

from mojodiffusion_b200 import _build
from mojodiffusion_b200.io.png import load_png
from mojodiffusion_b200.serve.backend import JobParams, StepResult

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def bins():
    server, lower = _build.build_control_plane()
    return str(server), str(lower)


def lower(bins, req):
    r = subprocess.run([bins[1]], input=json.dumps(req), capture_output=True, text=True)
    return r.returncode, json.loads(r.stdout)


def _t2i_graph(seed=7, steps=12, cfg=5.5, sampler="dpmpp_2m", scheduler="karras", w=768, h=512, batch=1):
    return {
        "10": {"class_type": "CheckpointLoaderSimple", "inputs": {"ckpt_name": "sdxl_base.safetensors"}},
        "11": {"class_type": "CLIPTextEncode", "inputs": {"clip": ["10", 1], "text": "a lighthouse at dusk"}},
        "12": {"class_type": "CLIPTextEncode", "inputs": {"clip": ["10", 1], "text": "lowres"}},
        "13": {"class_type": "EmptyLatentImage", "inputs": {"width": w, "height": h, "batch_size": batch}},
        "14": {"class_type": "KSampler", "inputs": {"model": ["10", 0], "positive": ["11", 0], "negative": ["12", 0],
                                                     "latent_image": ["13", 0], "seed": seed, "steps": steps, "cfg": cfg,
                                                     "sampler_name": sampler, "scheduler": scheduler, "denoise": 0.8}},
        "15": {"class_type": "VAEDecode", "inputs": {"samples": ["14", 0], "vae": ["10", 2]}},
        "16": {"class_type": "SaveImage", "inputs": {"images": ["15", 0], "filename_prefix": "dusk"}},
    }


def test_lowering_api_prompt_and_first_writer_wins(bins):
    rc, out = lower(bins, {"workflow": _t2i_graph(), "cfg": 9.0})
    assert rc == 0
    assert out["model"] == "sdxl_base.safetensors" and out["prompt"] == "a lighthouse at dusk" and out["negative"] == "lowres"
    assert (out["width"], out["height"], out["images"]) == (768, 512, 1)
    assert out["cfg"] == 9.0                                   # the request's own value wins over the graph
    assert (out["seed"], out["steps"], out["sampler"], out["scheduler"], out["creativity"]) == (7, 12, "dpmpp_2m", "karras", 0.8)
    assert out["workflow_save_prefix"] == "dusk" and out["workflow_source"] == "comfy_api_prompt_graph"
    assert out["workflow_schema"] == "serenity.workflow_graph.v1" and out["workflow_node_count"] == 7 and out["workflow_edge_count"] == 9
    assert out["workflow_route_kind"] == "image" and out["workflow_plan"]["terminal_nodes"][0]["type_id"] == "SaveImage"


def test_lowering_custom_sampler_lora_inpaint_and_scalars(bins):
    g = {
        "1": {"class_type": "UNETLoader", "inputs": {"unet_name": "flux2-klein-9b.safetensors"}},
        "2": {"class_type": "CLIPLoader", "inputs": {"clip_name": "qwen.safetensors"}},
        "3": {"class_type": "VAELoader", "inputs": {"vae_name": "flux2-vae.safetensors"}},
        "4": {"class_type": "LoraLoaderModelOnly", "inputs": {"model": ["1", 0], "lora_name": "style.safetensors", "strength_model": 0.7}},
        "5": {"class_type": "CLIPTextEncode", "inputs": {"clip": ["2", 0], "text": ["20", 0]}},
        "20": {"class_type": "PrimitiveString", "inputs": {"value": "make it snow"}},
        "6": {"class_type": "ConditioningZeroOut", "inputs": {"conditioning": ["5", 0]}},
        "7": {"class_type": "LoadImage", "inputs": {"image": "room.png"}},
        "8": {"class_type": "VAEEncode", "inputs": {"pixels": ["7", 0], "vae": ["3", 0]}},
        "9": {"class_type": "ReferenceLatent", "inputs": {"conditioning": ["5", 0], "latent": ["8", 0]}},
        "10": {"class_type": "CFGGuider", "inputs": {"model": ["4", 0], "positive": ["9", 0], "negative": ["6", 0], "cfg": 2.5}},
        "11": {"class_type": "Flux2Scheduler", "inputs": {"steps": ["21", 0]}},
        "21": {"class_type": "PrimitiveInt", "inputs": {"value": 24}},
        "12": {"class_type": "RandomNoise", "inputs": {"noise_seed": 99}},
        "13": {"class_type": "KSamplerSelect", "inputs": {"sampler_name": "euler"}},
        "14": {"class_type": "EmptyFlux2LatentImage", "inputs": {"width": 1024, "height": 1024, "batch_size": 1}},
        "15": {"class_type": "SamplerCustomAdvanced", "inputs": {"noise": ["12", 0], "guider": ["10", 0], "sampler": ["13", 0],
                                                                  "sigmas": ["11", 0], "latent_image": ["14", 0]}},
        "16": {"class_type": "VAEDecode", "inputs": {"samples": ["15", 0], "vae": ["3", 0]}},
        "17": {"class_type": "SaveImage", "inputs": {"images": ["16", 0], "filename_prefix": "snow"}},
    }
    rc, out = lower(bins, {"workflow": g})
    assert rc == 0, out
    assert out["model"] == "flux2-klein-9b.safetensors" and out["prompt"] == "make it snow"
    assert out["lora"] == [{"name": "style.safetensors", "weight": 0.7}]
    assert (out["steps"], out["scheduler"], out["seed"], out["sampler"], out["cfg"]) == (24, "flux2", 99, "euler", 2.5)
    assert out["reference_image"] == "room.png" and out["reference_latent_method"] == "index" and out["reference_latent_count"] == 1
    # inpaint conditioning writes both the image and the mask keys
    g2 = _t2i_graph()
    g2["30"] = {"class_type": "LoadImage", "inputs": {"image": "photo.png"}}
    g2["31"] = {"class_type": "InpaintModelConditioning", "inputs": {"positive": ["11", 0], "negative": ["12", 0], "vae": ["10", 2],
                                                                        "pixels": ["30", 0], "mask": ["30", 1], "noise_mask": True}}
    g2["14"]["inputs"].update(positive=["31", 0], negative=["31", 1], latent_image=["31", 2])
    rc, out = lower(bins, {"workflow": g2})
    assert rc == 0, out
    assert out["init_image"] == out["mask_image"] == out["inpaint_conditioning_image"] == "photo.png"
    assert out["lanpaint_mask_channel"] == "load_image_mask" and out["inpaint_conditioning_noise_mask"] is True


def test_lowering_errors_have_http_classes(bins):
    g = _t2i_graph()
    g["14"]["class_type"] = "KSamplerTurboX"
    rc, out = lower(bins, {"workflow": g})
    assert rc == 3 and out["status"] == 501 and out["type_id"] == "KSamplerTurboX"
    g = _t2i_graph()
    del g["14"]["inputs"]["latent_image"]
    rc, out = lower(bins, {"workflow": g})
    assert rc == 3 and out["status"] == 501 and "missing" in out["error"]
    g = _t2i_graph()
    g["14"]["inputs"]["latent_image"] = ["11", 0]            # a conditioning where a latent is expected
    rc, out = lower(bins, {"workflow": g})
    assert rc == 3 and out["status"] == 422 and "expected LATENT" in out["error"]
    g = _t2i_graph()
    g["11"]["inputs"]["clip"] = ["15", 0]                    # cycle-free but wrong type; and a real cycle:
    g["13"]["inputs"]["width"] = ["40", 0]
    g["40"] = {"class_type": "GetImageSize", "inputs": {"image": ["15", 0]}}
    rc, out = lower(bins, {"workflow": g})
    assert rc == 3 and out["status"] == 422
    rc, out = lower(bins, {"workflow": {"nodes": [{"id": 1, "type_id": "SamplerER_SDE", "fields": {}}], "edges": []}})
    assert rc == 3 and out["status"] == 501 and "er_sde" in out["error"]
    rc, out = lower(bins, {"workflow": {"nodes": [{"id": 1, "type_id": "EmptyLatentImage", "fields": {"width": 512, "height": 512, "batch_size": 1}},
                                                   {"id": 2, "type_id": "RepeatLatentBatch", "fields": {"amount": 65}}],
                                        "edges": [{"from": {"node": 1, "port": "LATENT"}, "to": {"node": 2, "port": "samples"}}]}})
    assert rc == 3 and out["status"] == 422 and "out of range [1..64]" in out["error"]


def test_lowering_canvas_flat_and_passthrough(bins):
    canvas = {"nodes": [
        {"id": 1, "type": "CheckpointLoaderSimple", "widgets_values": ["base.safetensors"],
         "outputs": [{"name": "MODEL", "type": "MODEL"}, {"name": "CLIP", "type": "CLIP"}, {"name": "VAE", "type": "VAE"}]},
        {"id": 2, "type": "CLIPTextEncode", "widgets_values": ["red fox"], "inputs": [{"name": "clip", "type": "CLIP"}],
         "outputs": [{"name": "CONDITIONING", "type": "CONDITIONING"}]},
        {"id": 3, "type": "CLIPTextEncode", "widgets_values": ["blurry"], "inputs": [{"name": "clip", "type": "CLIP"}],
         "outputs": [{"name": "CONDITIONING", "type": "CONDITIONING"}]},
        {"id": 4, "type": "EmptyLatentImage", "widgets_values": [640, 640, 2], "outputs": [{"name": "LATENT", "type": "LATENT"}]},
        {"id": 5, "type": "KSampler", "widgets_values": [123, "fixed", 30, 6.0, "euler", "simple", 1.0],
         "inputs": [{"name": "model"}, {"name": "positive"}, {"name": "negative"}, {"name": "latent_image"}],
         "outputs": [{"name": "LATENT", "type": "LATENT"}]},
        {"id": 6, "type": "VAEDecode", "inputs": [{"name": "samples"}, {"name": "vae"}], "outputs": [{"name": "IMAGE", "type": "IMAGE"}]},
        {"id": 7, "type": "SaveImage", "widgets_values": ["fox"], "inputs": [{"name": "images"}]},
        {"id": 8, "type": "PreviewImage", "mode": 4, "inputs": [{"name": "images"}]},
    ], "links": [[1, 1, 1, 2, 0, "CLIP"], [2, 1, 1, 3, 0, "CLIP"], [3, 1, 0, 5, 0, "MODEL"], [4, 2, 0, 5, 1, "CONDITIONING"],
                 [5, 3, 0, 5, 2, "CONDITIONING"], [6, 4, 0, 5, 3, "LATENT"], [7, 5, 0, 6, 0, "LATENT"], [8, 1, 2, 6, 1, "VAE"],
                 [9, 6, 0, 7, 0, "IMAGE"], [10, 6, 0, 8, 0, "IMAGE"]]}
    rc, out = lower(bins, {"workflow": canvas})
    assert rc == 0, out
    assert out["workflow_source"] == "comfy_ui_canvas_graph" and out["workflow_node_count"] == 7 and out["workflow_edge_count"] == 9
    assert (out["prompt"], out["negative"], out["images"], out["seed"], out["steps"], out["cfg"]) == ("red fox", "blurry", 2, 123, 30, 6.0)
    rc, out = lower(bins, {"workflow": {"params": {"prompt": "x", "steps": 5, "filename_prefix": "p", "loras": [{"name": "a", "weight": 1}]}}})
    assert rc == 0 and out["steps"] == 5 and out["workflow_save_prefix"] == "p" and out["lora"][0]["name"] == "a"
    assert out["workflow_source"] == "flat_params_adapter"
    rc, out = lower(bins, {"model": "m", "prompt": "p"})          # nothing to lower: untouched
    assert rc == 0 and out == {"model": "m", "prompt": "p"}


def test_lowering_reference_pairs_from_directory(bins):
    """Optional: MDB_LOWERING_REFS=<dir with *.request.json / *.lowered.json> checks every pair (extra keys this
    implementation adds, workflow_route_kind and workflow_plan, are allowed)."""
    d = os.environ.get("MDB_LOWERING_REFS")
    if not d:
        pytest.skip("MDB_LOWERING_REFS not set")
    n = 0
    for f in sorted(glob.glob(os.path.join(d, "*.request.json"))):
        lf = f.replace(".request.", ".lowered.")
        if not os.path.exists(lf):
            continue
        r = subprocess.run([bins[1], f], capture_output=True, text=True)
        got, exp = json.loads(r.stdout), json.load(open(lf))
        assert {k: got.get(k) for k in exp} == exp, os.path.basename(f)
        assert set(got) - set(exp) <= {"workflow_route_kind", "workflow_plan"}
        n += 1
    assert n > 0


def test_wire_contract():
    p = JobParams(job_id="j1", model="stub", prompt="hello", out_dir="/tmp")
    v = json.loads(p.start_line())
    assert v["cmd"] == "start" and v["width"] == 512 and v["cfg"] == 4.5 and v["lora"] == [] and v["eta"] == -1.0
    assert v["clip_skip"] == 0 and v["restart_sampling"] is False and v["creativity"] == 0.5 and v["sigma_shift"] == 3.0
    assert not p.start_line().endswith("\n") and len(v) == 71
    q = JobParams.from_wire({"cmd": "start", "width": 1024, "cfg": 7, "lora": [{"name": "x", "weight": 0.5}], "unknown": 1})
    assert q.width == 1024 and q.cfg == 7.0 and q.loras[0].weight == 0.5
    assert StepResult("progress", 3, 20).event() == {"ev": "progress", "step": 3, "total": 20, "phase": "", "preview": ""}
    assert StepResult("done", output_path="/tmp/j1.png").event() == {"ev": "done", "output_path": "/tmp/j1.png"}
    assert StepResult("cancelled").event() == {"ev": "cancelled"} and StepResult("failed", error="boom").terminal


# ---- live server ---------------------------------------------------------------------------------------------------
class Server:
    def __init__(self, bins, out_dir, extra_env=None, extra_args=()):
        env = dict(os.environ, PYTHONPATH=REPO + os.pathsep + os.environ.get("PYTHONPATH", ""), **(extra_env or {}))
        worker = f"{sys.executable} -m mojodiffusion_b200.serve.worker --kind {{kind}}"
        self.proc = subprocess.Popen([bins[0], "--worker", worker, "--out-dir", out_dir, "--port", "0", "--settle-ms", "50", *extra_args],
                                     stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, env=env)
        self.port = json.loads(self.proc.stdout.readline())["listening"]
        self.out_dir = out_dir

    def call(self, method, path, body=None, raw=None):
        data = raw if raw is not None else (json.dumps(body).encode() if body is not None else None)
        rq = urllib.request.Request(f"http://127.0.0.1:{self.port}{path}", data=data, method=method)
        try:
            with urllib.request.urlopen(rq, timeout=30) as r:
                return r.status, json.loads(r.read() or b"{}")
        except urllib.error.HTTPError as e:
            return e.code, json.loads(e.read() or b"{}")

    def ws_events(self, job_id, timeout=60):
        """Minimal WebSocket client: handshake, then text frames until the server closes."""
        s = socket.create_connection(("127.0.0.1", self.port), timeout=timeout)
        key = base64.b64encode(os.urandom(16)).decode()
        s.sendall((f"GET /v1/progress?job={job_id} HTTP/1.1\r\nHost: x\r\nUpgrade: websocket\r\nConnection: Upgrade\r\n"
                   f"Sec-WebSocket-Key: {key}\r\nSec-WebSocket-Version: 13\r\n\r\n").encode())
        buf = b""
        while b"\r\n\r\n" not in buf:
            buf += s.recv(4096)
        head, buf = buf.split(b"\r\n\r\n", 1)
        assert b"101" in head.split(b"\r\n")[0]
        accept = base64.b64encode(hashlib.sha1((key + "258EAFA5-E914-47DA-95CA-C5AB0DC85B11").encode()).digest())
        assert accept in head
        events = []
        while True:
            while len(buf) < 2:
                chunk = s.recv(65536)
                if not chunk:
                    return events
                buf += chunk
            op, ln, off = buf[0] & 0x0F, buf[1] & 0x7F, 2
            if ln == 126:
                while len(buf) < 4:
                    buf += s.recv(65536)
                ln, off = struct.unpack(">H", buf[2:4])[0], 4
            elif ln == 127:
                while len(buf) < 10:
                    buf += s.recv(65536)
                ln, off = struct.unpack(">Q", buf[2:10])[0], 10
            while len(buf) < off + ln:
                buf += s.recv(65536)
            payload, buf = buf[off:off + ln], buf[off + ln:]
            if op == 8:
                s.close()
                return events
            if op == 1:
                events.append(json.loads(payload))

    def wait(self, job_id, timeout=60):
        t0 = time.time()
        while time.time() - t0 < timeout:
            _, j = self.call("GET", f"/v1/job/{job_id}")
            if j["state"] in ("done", "failed", "cancelled"):
                return j
            time.sleep(0.05)
        raise TimeoutError(job_id)

    def close(self):
        self.proc.terminate()
        try:
            self.proc.wait(timeout=10)
        except subprocess.TimeoutExpired:
            self.proc.kill()


@pytest.fixture()
def server(bins, tmp_path):
    s = Server(bins, str(tmp_path / "out"))
    yield s
    s.close()


def test_generate_progress_socket_and_png(server):
    st, h = server.call("GET", "/v1/health")
    assert st == 200 and h["status"] == "ok"
    st, r = server.call("POST", "/v1/generate", {"model": "stub", "prompt": "héllo ✓", "steps": 6, "width": 64, "height": 64, "seed": 3})
    assert st == 200 and r["job_id"] == "job-0001" and r["job_ids"] == ["job-0001"]
    ev = server.ws_events(r["job_id"])
    assert ev[0]["ev"] == "snapshot" and ev[-1]["ev"] == "done" and ev[-1]["state"] == "done"
    steps = [e["step"] for e in ev if e.get("ev") == "progress"]
    assert steps == [1, 2, 3, 4, 5, 6] and all(e["total"] == 6 for e in ev if e.get("ev") == "progress")
    path = ev[-1]["output_path"]
    img, text = load_png(path)
    assert img.shape == (64, 64, 3) and (img[0] == 255).all()
    gp = json.loads(text["serenity.genparams.v1"])
    assert gp["schema"] == "serenity.genparams.v1" and gp["job_id"] == "job-0001" and gp["prompt"] == "héllo ✓" and gp["seed"] == 3
    late = server.ws_events(r["job_id"])                          # a late subscriber still gets the whole history
    assert [e.get("ev") for e in late] == [e.get("ev") for e in ev]
    st, res = server.call("GET", f"/v1/job/{r['job_id']}/result")
    m = res["result"]
    assert m["schema"] == "serenity.server_result.v1" and m["output_width"] == 64 and m["has_genparams_text"] is True
    assert m["output_location"]["inside_root"] is True and m["output_location"]["relative_path"] == "job-0001.png"
    st, g = server.call("GET", "/v1/gallery")
    assert g["items"][0]["id"] == "job-0001" and g["items"][0]["genparams"]["seed"] == 3
    st, it = server.call("POST", "/v1/gallery/job-0001/favorite", {"favorite": True})
    assert it["favorite"] is True
    st, rd = server.call("GET", "/v1/gallery/read?path=" + urllib.request.quote(path))
    assert rd["width"] == 64 and "serenity.genparams.v1" in rd["text"]


def test_workflow_generate_fanout_and_gates(server):
    g = _t2i_graph(w=64, h=64, steps=3, sampler="euler", scheduler="simple", batch=2)
    g["10"]["inputs"]["ckpt_name"] = "stub-model.safetensors"
    st, r = server.call("POST", "/v1/generate", {"workflow": g})
    assert st == 200 and len(r["job_ids"]) == 2
    a, b = (server.wait(i) for i in r["job_ids"])
    assert a["state"] == b["state"] == "done" and (a["image_index"], b["image_index"], b["image_count"]) == (0, 1, 2)
    _, ja = server.call("GET", f"/v1/job/{r['job_ids'][0]}")
    _, jb = server.call("GET", f"/v1/job/{r['job_ids'][1]}")
    assert jb["params"]["seed"] == ja["params"]["seed"] + 1 and ja["params"]["workflow_save_prefix"] == "dusk"
    st, pf = server.call("POST", "/v1/preflight", {"workflow": g})
    assert pf["admitted"] is True and pf["same_gate_as_generate"] is True and pf["kind"] == "stub"
    bad = dict(model="stub", prompt="x", width=100, height=64)
    st, e = server.call("POST", "/v1/generate", bad)
    assert st == 400 and e["schema"] == "serenity.generate.error.v1" and e["same_gate_as_preflight"] is True
    st, pf = server.call("POST", "/v1/preflight", bad)
    assert st == 200 and pf["admitted"] is False and "multiples of 16" in pf["rejection"]["error"]
    st, e = server.call("POST", "/v1/generate", {"model": "ideogram-4", "prompt": "x"})
    assert st == 400 and "blocked" in e["error"]
    g["14"]["class_type"] = "Nope"
    st, e = server.call("POST", "/v1/generate", {"workflow": g})
    assert st == 501 and e["stage"] == "workflow_lowering"
    st, e = server.call("POST", "/v1/generate", raw=b"{not json")
    assert st == 400
    st, caps = server.call("GET", "/v1/capabilities")
    assert any(f["kind"] == "flux" and f["admitted"] for f in caps["families"]) and "euler" in caps["samplers"]


def test_cancel_queue_reorder_remove(server):
    ids = [server.call("POST", "/v1/generate", {"model": "stub", "prompt": f"p{i}", "steps": 40 if i == 0 else 2, "width": 64, "height": 64})[1]["job_id"]
           for i in range(4)]
    time.sleep(0.3)
    st, r = server.call("POST", "/v1/reorder", {"order": [ids[3], ids[2]]})
    assert r["order"][:2] == [ids[3], ids[2]]
    st, r = server.call("POST", "/v1/remove", {"job_id": ids[1]})
    assert r["removed"] == ids[1]
    st, r = server.call("POST", "/v1/remove", {"job_id": ids[0]})
    assert st == 409                                             # running: cancel instead
    st, r = server.call("POST", f"/v1/cancel/{ids[0]}")
    assert r["cancelled"] is True
    assert server.wait(ids[0])["state"] == "cancelled"
    d3, d2 = server.wait(ids[3]), server.wait(ids[2])
    assert d3["state"] == d2["state"] == "done"
    assert os.path.getmtime(d3["output_path"]) <= os.path.getmtime(d2["output_path"])   # reordered: 3 ran before 2
    st, jobs = server.call("GET", "/v1/jobs")
    assert [j["id"] for j in jobs["jobs"]] == [ids[0], ids[2], ids[3]] or {j["id"] for j in jobs["jobs"]} == {ids[0], ids[2], ids[3]}
    assert not os.path.exists(os.path.join(server.out_dir, f"{ids[0]}.png"))


def test_worker_failures_are_contained_and_worker_respawns(server):
    st, r = server.call("POST", "/v1/generate", {"model": "stub", "prompt": "__fail__", "steps": 4, "width": 64, "height": 64})
    j = server.wait(r["job_id"])
    assert j["state"] == "failed" and "injected" in j["error"]
    st, r = server.call("POST", "/v1/generate", {"model": "stub", "prompt": "__exit__ now", "steps": 4, "width": 64, "height": 64})
    j = server.wait(r["job_id"])
    assert j["state"] == "failed" and "peer closed" in j["error"]          # the process died: typed, recoverable
    st, r = server.call("POST", "/v1/generate", {"model": "stub", "prompt": "after the crash", "steps": 2, "width": 64, "height": 64})
    assert server.wait(r["job_id"])["state"] == "done"                    # lazy respawn served the next job
    st, r = server.call("POST", "/v1/generate", {"model": "stub", "prompt": "__hang__", "steps": 50, "width": 64, "height": 64})
    time.sleep(0.5)
    server.call("POST", "/v1/cancel", {"job_id": r["job_id"]})
    assert server.wait(r["job_id"])["state"] == "cancelled"                # a silent worker still honours cancel
    st, h = server.call("GET", "/v1/health")
    assert h["status"] == "ok" and h["in_flight"] == ""


def test_uploads_presets_state(server, tmp_path):
    from mojodiffusion_b200.io.png import encode_png
    import numpy as np
    png = encode_png(np.zeros((8, 8, 3), np.uint8))
    st, r = server.call("POST", "/upload/mask", {"name": "m 1", "data": "data:image/png;base64," + base64.b64encode(png).decode()})
    assert st == 200 and r["path"].endswith("/uploads/m_1.png") and open(r["path"], "rb").read() == png
    st, r = server.call("POST", "/upload/image", raw=b"not a png")
    assert st == 400
    st, r = server.call("POST", "/v1/generate", {"model": "stub", "prompt": "i2i", "steps": 2, "width": 64, "height": 64,
                                                 "init_image": "/nonexistent/x.png"})
    assert st == 400 and "does not exist" in r["error"]
    assert server.call("POST", "/v1/presets/portrait", {"steps": 30})[0] == 200
    assert server.call("GET", "/v1/presets")[1]["presets"] == ["portrait"]
    assert server.call("GET", "/v1/presets/portrait")[1] == {"steps": 30}
    assert server.call("DELETE", "/v1/presets/portrait")[1]["deleted"] == "portrait"
    assert server.call("POST", "/v1/state", {"tab": "generate"})[1] == {"tab": "generate"}
    assert server.call("GET", "/v1/state")[1] == {"tab": "generate"}
    assert server.call("GET", "/v1/nope")[0] == 404


def test_model_swap_restarts_worker_with_flux_kind(bins, tmp_path):
    """A job for another model family replaces the resident worker. The FLUX backend runs its full phase machine on the
    CPU with the tiny architecture and random weights (no checkpoint on disk)."""
    s = Server(bins, str(tmp_path / "out"), {"MDB_FLUX_ARCH": "tiny"})
    try:
        st, r = s.call("POST", "/v1/generate", {"model": "stub", "prompt": "a", "steps": 2, "width": 64, "height": 64})
        assert s.wait(r["job_id"])["state"] == "done" and s.call("GET", "/v1/health")[1]["backend"] == "stub"
        st, r = s.call("POST", "/v1/generate", {"model": "flux1-tiny", "prompt": "a red cube", "steps": 3, "width": 64, "height": 64, "seed": 5})
        ev = s.ws_events(r["job_id"], timeout=300)
        assert ev[-1]["ev"] == "done", ev[-1]
        phases = [e["phase"] for e in ev if e.get("ev") == "progress"]
        assert phases[:2] == ["load", "denoise"] and phases[-1] == "decode"
        img, text = load_png(ev[-1]["output_path"])
        assert img.shape == (64, 64, 3) and json.loads(text["serenity.genparams.v1"])["prompt"] == "a red cube"
        side = json.load(open(ev[-1]["output_path"] + ".worker_result.json"))
        assert side["weights"] == "random-init" and side["text"] == "hash-embedding" and side["steps_run"] == 3
        assert s.call("GET", "/v1/health")[1]["backend"] == "flux"
        assert s.call("GET", f"/v1/job/{r['job_id']}/result")[1]["result"]["worker_sidecar_present"] is True
    finally:
        s.close()


@pytest.mark.parametrize("model,backend,cfg", [("z-image-tiny", "zimage", 4.0), ("qwen-image-tiny", "qwenimage", 1.0),
                                               ("sd_xl_tiny", "sdxl", 5.0), ("ltx-2-tiny", "ltx2", 3.0),
                                               ("sd3.5_tiny", "sd3", 4.5), ("sd15-tiny", "sd15", 6.0),
                                               ("flux2-klein-tiny", "klein", 4.0), ("chroma-tiny", "chroma", 4.0)])
def test_other_families_serve_through_the_worker(bins, tmp_path, model, backend, cfg):
    """Z-Image, Qwen-Image and SDXL jobs run their own phase machines in the worker (tiny architectures, random weights),
    with classifier-free guidance when cfg > 1; the result carries the parameters and a sidecar naming the family."""
    s = Server(bins, str(tmp_path / "out"), {"MDB_ARCH": "tiny"})
    try:
        st, r = s.call("POST", "/v1/generate", {"model": model, "prompt": "a lighthouse", "negative": "blurry", "steps": 2,
                                                 "width": 64, "height": 64, "seed": 9, "cfg": cfg})
        assert st == 200, r
        ev = s.ws_events(r["job_id"], timeout=300)
        assert ev[-1]["ev"] == "done", ev[-1]
        img, text = load_png(ev[-1]["output_path"])
        assert img.shape == (64, 64, 3) and json.loads(text["serenity.genparams.v1"])["prompt"] == "a lighthouse"
        side = json.load(open(ev[-1]["output_path"] + ".worker_result.json"))
        assert side["schema"] == f"serenity.{backend}.daemon_result.v1" and side["weights"] == "random-init"
        assert side["cfg"] == (cfg if cfg > 1 else 1.0) and side["steps_run"] == 2
        assert s.call("GET", "/v1/health")[1]["backend"] == backend
        if backend == "ltx2":                       # video: frames beside the poster image
            assert side["frames"] == 9 and len(os.listdir(side["frames_dir"])) == 9
    finally:
        s.close()


# ---- hires two-pass, video routes, checkpoint scan, node type allowlist ---------------------------------------------
def test_hires_two_pass_runs_under_one_job(server):
    st, r = server.call("POST", "/v1/generate", {"model": "stub", "prompt": "x", "steps": 3, "width": 256, "height": 256, "seed": 1,
                                                 "hires_scale": 2.0, "hires_denoise": 0.4})
    assert st == 200
    ev = server.ws_events(r["job_id"])
    assert [e["ev"] for e in ev].count("done") == 1 and ev[-1]["ev"] == "done"           # one terminal event for both passes
    assert any(e.get("phase") == "hires" for e in ev)
    assert [e["step"] for e in ev if e.get("ev") == "progress" and e.get("phase") != "hires"] == [1, 2, 3, 1, 2, 3]
    img, text = load_png(ev[-1]["output_path"])
    assert img.shape == (512, 512, 3)                                                    # 256 * 2 = 512 < 768 -> refine at 512
    assert int(img[100, 100, 2]) == int(0.4 * 255.0)                                     # the refine pass ran img2img at the hires creativity
    assert not [f for f in os.listdir(server.out_dir) if f.startswith("hires_src_")]      # the upscale source is removed
    st, g = server.call("GET", "/v1/gallery")
    assert [it["id"] for it in g["items"]] == [r["job_id"]]
    st, r2 = server.call("POST", "/v1/generate", {"model": "stub", "prompt": "x", "steps": 2, "width": 512, "height": 384, "hires_scale": 1.5})
    assert load_png(server.wait(r2["job_id"])["output_path"])[0].shape == (1024, 1024, 3)  # 768 -> refine at 1024
    for bad in ({"hires_scale": 9}, {"hires_scale": 0.5}, {"hires_scale": 2, "hires_denoise": 0}):
        st, e = server.call("POST", "/v1/generate", {"model": "stub", "prompt": "x", **bad})
        assert st == 400 and "hires" in e["error"]


def test_video_routes_over_the_ltx_worker(bins, tmp_path):
    s = Server(bins, str(tmp_path / "out"), {"MDB_ARCH": "tiny"})
    try:
        st, v = s.call("GET", "/v1/video")
        assert st == 200 and v["schema"] == "serenity.video_status.v1" and v["container"] == "png-sequence" and v["mp4"] == ""
        st, e = s.call("POST", "/v1/video", {"model": "flux1-tiny", "prompt": "x"})
        assert st == 400 and "video model" in e["error"]
        st, e = s.call("POST", "/v1/video", {"model": "ltx-2-tiny", "prompt": "x", "frames": 10})
        assert st == 400 and "8k + 1" in e["error"]
        st, r = s.call("POST", "/v1/video", {"model": "ltx-2-tiny", "prompt": "a wave", "frames": 9, "fps": 12, "width": 64, "height": 64, "steps": 2, "seed": 4})
        assert st == 200 and r["schema"] == "serenity.video_job.v1" and r["container"] == "png-sequence", r
        st, pending = s.call("GET", "/v1/video/result?job=" + r["job_id"])
        assert st == 200 and pending["schema"] == "serenity.video_result.v1"
        j = s.wait(r["job_id"], timeout=240)
        assert j["state"] == "done", j
        st, res = s.call("GET", "/v1/video/result?job=" + r["job_id"])
        assert res["ready"] is True and res["frame_count"] >= 1 and res["fps"] == 12 and res["mp4"] == "" and res["audio"] is False
        assert res["frames_dir"].endswith(".frames") and abs(res["duration"] - res["frame_count"] / 12) < 1e-9
        assert len([f for f in os.listdir(res["frames_dir"]) if f.endswith(".png")]) == res["frame_count"]
        st, pr = s.call("POST", "/v1/video/probe", {"path": res["frames_dir"]})
        assert st == 200 and pr["frame_count"] == res["frame_count"] and pr["width"] == res["width"] > 0
        st, e = s.call("POST", "/v1/video/probe", {"path": "/etc"})
        assert st == 400
        st, e = s.call("GET", "/v1/video/result?job=job-9999")
        assert st == 404
    finally:
        s.close()


def _fake_safetensors(path, keys):
    header = json.dumps({k: {"dtype": "BF16", "shape": [1], "data_offsets": [0, 2]} for k in keys}).encode()
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(header)) + header + b"\0\0")


def test_models_route_detects_architecture_from_headers(bins, tmp_path):
    md = tmp_path / "models"
    md.mkdir()
    cases = {"a.safetensors": (["double_blocks.0.img_attn.qkv.weight", "single_blocks.0.linear1.weight"], "flux", "header"),
             "b.safetensors": (["noise_refiner.0.attention.to_q.weight", "layers.0.attention.to_q.weight"], "zimage", "header"),
             "c.safetensors": (["double_stream_modulation_img.lin.weight", "double_blocks.0.img_attn.qkv.weight"], "flux-2/klein", "header"),
             "d.safetensors": (["model.diffusion_model.input_blocks.0.0.weight"], "sdxl", "header"),
             "e.safetensors": (["txt_norm.weight", "transformer_blocks.0.attn.add_q_proj.weight"], "qwen-image", "header"),
             "f.safetensors": (["distilled_guidance_layer.in_proj.weight", "double_blocks.0.img_attn.qkv.weight"], "chroma", "header"),
             "my_sdxl_finetune.safetensors": (["whatever.weight"], "sdxl", "name"),
             "g.safetensors": (["layers.0.adaLN_sa_ln.weight", "text_proj.weight"], "ernie-image", "header"),
             "h.safetensors": (["something.else"], "unknown", "none"),
             "style.safetensors": (["lora_unet_down_blocks_0.lora_down.weight", "lora_unet_down_blocks_0.lora_up.weight"], "sdxl", "header")}
    for name, (keys, _, _) in cases.items():
        _fake_safetensors(str(md / name), keys)
    (md / "broken.safetensors").write_bytes(b"\x01")
    s = Server(bins, str(tmp_path / "out"), extra_args=("--models-dir", str(md)))
    try:
        st, r = s.call("GET", "/v1/models")
        got = {m["name"]: m for m in r["models"]}
        for name, (_, arch, source) in cases.items():
            assert got[name]["arch"] == arch and got[name]["arch_source"] == source, (name, got[name])
        assert got["style.safetensors"].get("lora") is True and got["broken.safetensors"]["arch"] == "unknown"
        st, e = s.call("GET", "/v1/gallery/read?path=" + urllib.request.quote(s.out_dir + "X/evil.png"))
        assert st == 400 and "outside" in e["error"]                  # a sibling directory sharing the prefix is outside the root
    finally:
        s.close()


REFERENCE_NODE_TYPES = """BOOLConstant BasicGuider BasicScheduler BetaSamplingScheduler CFGGuider CLIPLoader CLIPTextEncode CLIPTextEncodeFlux
CLIPVisionEncode CLIPVisionLoader CheckpointLoaderSimple ConditioningSetMask ConditioningZeroOut DiffusionModelLoader DualCLIPLoader
EmptyFlux2LatentImage EmptyHunyuanLatentVideo EmptyLatentImage EmptySD3LatentImage ExponentialScheduler FloatConstant GetNode INTConstant
KSampler KSamplerAdvanced KSamplerSelect KarrasScheduler LTXVLoader LaplaceScheduler LoadImage LoraLoader LoraLoaderModelOnly
PolyexponentialScheduler PreviewImage PrimitiveBoolean PrimitiveFloat PrimitiveInt PrimitiveNode PrimitiveString PrimitiveStringMultiline
RandomNoise Reroute SDTurboScheduler SamplerCustom SamplerCustomAdvanced SamplerDPMAdaptative SamplerDPMPP_2M_SDE SamplerDPMPP_2S_Ancestral
SamplerDPMPP_3M_SDE SamplerDPMPP_SDE SamplerER_SDE SamplerEuler SamplerEulerAncestral SamplerEulerAncestralCFGPP SamplerLMS SamplerSASolver
SamplerSEEDS2 SaveImage SeedNode SetNode StringConstant StringConstantMultiline TripleCLIPLoader UNETLoader VAEDecode VAEEncode VAELoader
VPScheduler ZImageLoraModelOnly ImageResizeKJ LTXVSampler LanPaint_MaskBlend WanImageToVideo""".split()


def test_every_listed_node_type_is_registered_and_others_answer_501_with_their_id(bins):
    r = subprocess.run([bins[1], "--node-types"], capture_output=True, text=True)
    assert r.returncode == 0
    types = set(json.loads(r.stdout))
    assert len(types) >= 100, len(types)
    missing = [t for t in REFERENCE_NODE_TYPES if t not in types]
    assert not missing, missing
    # the one-node LTX sampler and the explicit resize lower into flat parameters
    wf = {"nodes": [{"id": 1, "type_id": "LTXVLoader", "fields": {"ckpt_name": "ltx-2.safetensors"}},
                    {"id": 2, "type_id": "LTXVSampler", "fields": {"prompt": "a tide", "width": 768, "height": 512, "num_frames": 41, "frame_rate": 12, "steps": 8}}],
          "edges": [{"from": {"node": 1, "port": "MODEL"}, "to": {"node": 2, "port": "ltxv_model"}}]}
    r = subprocess.run([bins[1]], input=json.dumps({"workflow": wf}), capture_output=True, text=True)
    low = json.loads(r.stdout)
    assert r.returncode == 0, r.stdout
    assert (low["model"], low["prompt"], low["num_frames"], low["fps"], low["steps"], low["width"]) == ("ltx-2.safetensors", "a tide", 41, 12, 8, 768)
    wf = {"nodes": [{"id": 1, "type_id": "LoadImage", "fields": {"image": "in.png"}},
                    {"id": 2, "type_id": "ImageResizeKJ", "fields": {"width": 640, "height": 0}}],
          "edges": [{"from": {"node": 1, "port": "IMAGE"}, "to": {"node": 2, "port": "image"}}]}
    r = subprocess.run([bins[1]], input=json.dumps({"model": "stub", "workflow": wf}), capture_output=True, text=True)
    e = json.loads(r.stdout)
    assert r.returncode == 3 and e["status"] == 501 and "keeps the source dimension" in e["error"]
    req = {"model": "stub", "prompt": "x", "workflow": {"nodes": [{"id": 7, "type_id": "TotallyMadeUpNode", "fields": {}}], "edges": []}}
    r = subprocess.run([bins[1]], input=json.dumps(req), capture_output=True, text=True)
    e = json.loads(r.stdout)
    assert r.returncode == 3 and e["status"] == 501 and e["type_id"] == "TotallyMadeUpNode" and e["node_id"] == 7


def test_encode_phase_runs_text_encoders_in_a_child_process(bins, tmp_path):
    """With MDB_ENCODE_SUBPROCESS=1 the ENCODE phase of the worker spawns a child that tokenises, runs the family's (tiny,
    random-weight) encoders, writes a caption file and exits; the worker's sidecar names the child's pid."""
    s = Server(bins, str(tmp_path / "out"), {"MDB_ARCH": "tiny", "MDB_ENCODE_SUBPROCESS": "1"})
    try:
        st, r = s.call("POST", "/v1/generate", {"model": "z-image-tiny", "prompt": "a red cube", "negative": "blurry", "steps": 2, "cfg": 3.0,
                                                 "width": 64, "height": 64, "seed": 9})
        assert st == 200, r
        j = s.wait(r["job_id"], timeout=240)
        assert j["state"] == "done", j
        side = json.load(open(j["output_path"] + ".worker_result.json"))
        assert side["text"] == "encoder-subprocess" and side["encoder_pid"] > 0
        try:
            os.kill(side["encoder_pid"], 0)
            alive = True
        except OSError:
            alive = False
        assert not alive                                  # the encoder process is gone: its memory went with it
        st, r2 = s.call("POST", "/v1/generate", {"model": "z-image-tiny", "prompt": "a blue sphere", "steps": 2, "width": 64, "height": 64, "seed": 9})
        j2 = s.wait(r2["job_id"], timeout=240)
        a, b = load_png(j["output_path"])[0], load_png(j2["output_path"])[0]
        assert a.shape == b.shape and (a != b).any()      # the prompt reaches the image through the encoders
    finally:
        s.close()


def test_llm_listing_and_magic_prompt_through_a_throw_away_process(bins, tmp_path):
    """/v1/llms lists GGUF files and safetensors model directories (one level deep, sorted); /v1/magic_prompt runs the prompt
    generator as a child process per request and returns its one-line caption; bad requests and a failing generator are
    answered with 400 / 500 and the reason."""
    llm = tmp_path / "llms"
    (llm / "qwen3-4b").mkdir(parents=True)
    (llm / "qwen3-4b" / "config.json").write_text("{}")
    (llm / "qwen3-4b" / "model.safetensors").write_bytes(b"\0" * 32)
    (llm / "sub").mkdir()
    (llm / "sub" / "gemma.gguf").write_bytes(b"\0" * 8)
    (llm / "alpha.gguf").write_bytes(b"\0" * 4)
    (llm / "notes.txt").write_text("x")
    reply = tmp_path / "reply.txt"
    reply.write_text('Here you go:\n```json\n{"compositional_deconstruction":{"elements":[{"desc":"a fox","bbox":[10,20,300,400],"type":"obj"}],'
                     '"background":"snow"},"aspect_ratio":"1:1","high_level_description":"A fox in snow"}\n```\n')
    s = Server(bins, str(tmp_path / "out"), extra_args=("--llm-dir", str(llm), "--magic-cmd", f"{sys.executable} -m mojodiffusion_b200.captioner.magic_prompt"))
    try:
        st, v = s.call("GET", "/v1/llms")
        assert st == 200 and [m["name"] for m in v["llms"]] == ["alpha", "gemma", "qwen3-4b"]
        assert v["llms"][2]["path"].endswith("/qwen3-4b") and v["llms"][2]["size"] == 32 and v["llms"][0]["size"] == 4
        st, v = s.call("POST", "/v1/magic_prompt", {"idea": "  a fox in snow ", "aspect": "1:1", "model": "stub:" + str(reply)})
        assert st == 200, v
        cap = json.loads(v["caption"])
        assert "\n" not in v["caption"] and list(cap) == ["high_level_description", "compositional_deconstruction"]
        assert cap["compositional_deconstruction"]["elements"][0] == {"type": "obj", "bbox": [10, 20, 300, 400], "desc": "a fox"}
        assert s.call("POST", "/v1/magic_prompt", {"idea": " ", "model": "stub:" + str(reply)})[0] == 400
        assert s.call("POST", "/v1/magic_prompt", {"idea": "x", "model": str(tmp_path / "missing")})[0] == 400
        assert s.call("GET", "/v1/magic_prompt")[0] == 405
        reply.write_text("no json in this reply")
        st, v = s.call("POST", "/v1/magic_prompt", {"idea": "x", "model": "stub:" + str(reply)})
        assert st == 500 and "no JSON caption" in v["error"]
    finally:
        s.close()


def test_llm_listing_in_python_matches_the_route_rules(tmp_path):
    from mojodiffusion_b200.captioner.magic_prompt import list_llms
    (tmp_path / "m1").mkdir()
    (tmp_path / "m1" / "config.json").write_text("{}")
    (tmp_path / "m1" / "a.safetensors").write_bytes(b"1234")
    (tmp_path / "z.gguf").write_bytes(b"12")
    got = list_llms(str(tmp_path))
    assert [(e["name"], e["size"]) for e in got] == [("m1", 4), ("z", 2)]
