// mdb-server: HTTP/WebSocket control plane for image generation workers.
//
//   mdb-server --worker "<command with optional {kind}>" --out-dir DIR [--port N] [--models-dir DIR] [--settle-ms N]
//
// One worker process is resident at a time. Each model family ("kind") needs its own worker: a job for another kind
// kills the resident worker (process exit returns its device memory), waits ``settle-ms`` and spawns the next. A worker
// that dies mid-job fails that job only; the next job respawns it. The job book is a FIFO queue with reorder / remove /
// cancel; every job keeps its event log so a WebSocket client that connects late still sees the whole history.
//
// Routes and behaviour follow serenity-server/crates/server/src/main.rs:1326-1532 (driver), :1974-2330 (generate),
// :2335-2460 (progress socket), :3648-3690 (route table), jobs.rs, gallery.rs, result_manifest.rs, capabilities.rs.
#include <dirent.h>
#include <poll.h>
#include <sys/stat.h>
#include <sys/wait.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <csignal>
#include <ctime>
#include <deque>
#include <fstream>
#include <iostream>
#include <mutex>
#include <sstream>
#include <thread>

#include "graph.hpp"
#include "http.hpp"
#include "json.hpp"
#include "wire.hpp"
#include "worker_proc.hpp"

using mdb::Json;
namespace http = mdb::http;
namespace wire = mdb::wire;

// ---- files ---------------------------------------------------------------------------------------------------------
static bool read_file(const std::string& p, std::string* out) {
  std::ifstream f(p, std::ios::binary);
  if (!f) return false;
  std::stringstream ss;
  ss << f.rdbuf();
  *out = ss.str();
  return true;
}
static bool write_file_atomic(const std::string& p, const std::string& data) {
  std::string tmp = p + ".tmp";
  { std::ofstream f(tmp, std::ios::binary | std::ios::trunc); if (!f) return false; f << data; if (!f) return false; }
  return rename(tmp.c_str(), p.c_str()) == 0;
}
static void mkdirs(const std::string& p) {
  std::string cur;
  for (size_t i = 0; i <= p.size(); ++i) {
    if (i == p.size() || p[i] == '/') { if (!cur.empty()) mkdir(cur.c_str(), 0755); }
    if (i < p.size()) cur += p[i];
  }
}
static bool file_exists(const std::string& p) { struct stat st; return stat(p.c_str(), &st) == 0; }
static long long file_size(const std::string& p) { struct stat st; return stat(p.c_str(), &st) == 0 ? static_cast<long long>(st.st_size) : -1; }
static std::string now_http_date() {
  char buf[64];
  time_t t = time(nullptr);
  struct tm g;
  gmtime_r(&t, &g);
  strftime(buf, sizeof buf, "%a, %d %b %Y %H:%M:%S GMT", &g);
  return buf;
}
// true when ``path`` is ``root`` itself or lies under it (the prefix must end at a path separator)
static bool inside_root(const std::string& path, const std::string& root) {
  if (root.empty() || path.compare(0, root.size(), root) != 0 || path.find("..") != std::string::npos) return false;
  return path.size() == root.size() || path[root.size()] == '/' || root.back() == '/';
}
static bool safe_relative(const std::string& p) {
  if (p.empty() || p[0] == '/') return false;
  return p.find("..") == std::string::npos && p.find('\0') == std::string::npos;
}

// PNG header + tEXt chunks (generation parameters travel inside the image)
struct PngInfo { bool ok = false; long long width = 0, height = 0; std::map<std::string, std::string> text; };
static PngInfo read_png_info(const std::string& path) {
  PngInfo info;
  std::string d;
  if (!read_file(path, &d) || d.size() < 33 || d.compare(0, 8, "\x89PNG\r\n\x1a\n") != 0) return info;
  auto be32 = [&](size_t o) { return (static_cast<uint32_t>(static_cast<unsigned char>(d[o])) << 24) | (static_cast<unsigned char>(d[o + 1]) << 16) | (static_cast<unsigned char>(d[o + 2]) << 8) | static_cast<unsigned char>(d[o + 3]); };
  size_t pos = 8;
  while (pos + 12 <= d.size()) {
    uint32_t len = be32(pos);
    std::string tag = d.substr(pos + 4, 4);
    if (pos + 12 + len > d.size()) break;
    if (tag == "IHDR" && len >= 8) { info.width = be32(pos + 8); info.height = be32(pos + 12); info.ok = true; }
    else if (tag == "tEXt") {
      std::string body = d.substr(pos + 8, len);
      size_t z = body.find('\0');
      if (z != std::string::npos) info.text[body.substr(0, z)] = body.substr(z + 1);
    } else if (tag == "IDAT" || tag == "IEND") break;
    pos += 12 + len;
  }
  return info;
}

// ---- model families ---------------------------------------------------------------------------------------------------
struct Family { const char* kind; std::vector<const char*> needles; bool admitted; const char* note; };
static const std::vector<Family>& families() {
  static const std::vector<Family> f = {
      {"stub", {"stub"}, true, "CPU test worker"},
      {"flux", {"flux1", "flux.1", "flux-1", "flux_1", "flux-dev", "flux-schnell"}, true, "FLUX.1 MMDiT"},
      {"klein", {"klein", "flux2", "flux.2", "flux-2"}, true, "FLUX.2 / Klein"},
      {"chroma", {"chroma"}, true, "Chroma"},
      {"zimage", {"zimage", "z-image", "z_image"}, true, "Z-Image single-stream DiT"},
      {"qwenimage", {"qwen"}, true, "Qwen-Image"},
      {"sd3", {"sd3", "sd35", "stable-diffusion-3"}, true, "SD3 / SD3.5"},
      {"sdxl", {"sdxl", "sd_xl", "xl-base"}, true, "SDXL UNet"},
      {"sd15", {"sd15", "v1-5", "sd-v1"}, true, "SD 1.5 UNet"},
      {"ltx2", {"ltx"}, true, "LTX-2 video"},
      {"ideogram4", {"ideogram"}, false, "no local weights format; blocked"},
      {"anima", {"anima"}, false, "not built"},
      {"sensenova", {"sensenova"}, false, "not built"},
      {"lens", {"lens"}, false, "not built"}};
  return f;
}
static const Family* family_of(const std::string& model) {
  std::string m = mdb::graph::lower(model);
  for (auto& f : families()) for (auto* n : f.needles) if (m.find(n) != std::string::npos) return &f;
  return nullptr;
}
static const std::vector<std::string> kSamplers = {"euler", "flowmatch_euler", "dpmpp_2m", "uni_pc", "uni_pc_bh2", "res_2s", "res_multistep", "ddim"};
static const std::vector<std::string> kSchedulers = {"simple", "flowmatch", "sgm_uniform", "normal", "karras", "flux2", "beta", "linear_quadratic"};

// ---- job book -----------------------------------------------------------------------------------------------------------
struct Job {
  std::string id, state = "queued", model, created, output_path, error, phase;
  long long step = 0, total = 0, image_index = 0, image_count = 1;
  Json params;                 // full wire parameters
  Json request;                // lowered request as submitted (for manifests)
  std::vector<std::string> events;   // JSON frames, in order; never shrinks
  bool cancel_requested = false;
  double hires_scale = 0.0, hires_denoise = 0.35;   // control-plane only: a second img2img pass under the same job id
  int pass = 1;
  std::string hires_src, kind_override;
  bool terminal() const { return state == "done" || state == "failed" || state == "cancelled"; }
  Json summary() const {
    Json j = Json::object();
    j.set("id", Json(id)); j.set("job_id", Json(id)); j.set("state", Json(state)); j.set("model", Json(model)); j.set("created", Json(created));
    j.set("step", Json(step)); j.set("total", Json(total));
    j.set("progress", Json(total > 0 ? static_cast<int64_t>(100 * step / total) : static_cast<int64_t>(0)));
    j.set("phase", Json(phase)); j.set("image_index", Json(image_index)); j.set("image_count", Json(image_count));
    j.set("output_path", Json(output_path)); j.set("error", Json(error));
    j.set("prompt", Json(params.str("prompt")));
    return j;
  }
};

struct App {
  std::string out_dir, models_dir, worker_cmd;
  std::string llm_dir;                                   // language models for /v1/llms and /v1/magic_prompt
  std::string magic_cmd = "python -m mojodiffusion_b200.captioner.magic_prompt";
  int settle_ms = 800;
  std::mutex mu;
  std::condition_variable cv;
  std::deque<std::shared_ptr<Job>> jobs;      // submission order; queue order = order of "queued" entries
  std::string in_flight;
  std::atomic<long long> next_id{0};
  std::atomic<bool> shutting_down{false};
  std::string resident_kind;
  http::Server server;

  std::shared_ptr<Job> find(const std::string& id) {
    for (auto& j : jobs) if (j->id == id) return j;
    return nullptr;
  }
  void persist_locked() {
    Json arr = Json::array();
    for (auto& j : jobs) { Json s = j->summary(); s.set("params", j->params); arr.push(s); }
    write_file_atomic(out_dir + "/jobs.json", arr.dump());
  }
  void publish_locked(Job& j, const Json& frame) { j.events.push_back(frame.dump()); server.wake(); }
};

static Json ws_frame_for(const Job& j, const wire::Event& ev) {
  Json f = Json::object();
  f.set("job_id", Json(j.id));
  switch (ev.kind) {
    case wire::Event::Progress: f.set("state", Json("running")); break;
    case wire::Event::Done: f.set("state", Json("done")); break;
    case wire::Event::Failed: f.set("state", Json("failed")); break;
    case wire::Event::Cancelled: f.set("state", Json("cancelled")); break;
    default: f.set("state", Json(j.state));
  }
  f.set("ev", ev.to_json().get("ev"));
  f.set("step", Json(ev.kind == wire::Event::Progress ? ev.step : j.step));
  f.set("total", Json(ev.kind == wire::Event::Progress ? ev.total : j.total));
  long long tot = ev.kind == wire::Event::Progress ? ev.total : j.total, st = ev.kind == wire::Event::Progress ? ev.step : j.step;
  f.set("progress", Json(tot > 0 ? static_cast<int64_t>(100 * st / tot) : static_cast<int64_t>(0)));
  f.set("phase", Json(ev.phase));
  f.set("preview", Json(ev.preview));
  if (ev.kind == wire::Event::Done) f.set("output_path", Json(ev.output_path));
  if (ev.kind == wire::Event::Failed) f.set("error", Json(ev.error));
  return f;
}

// result manifest written beside every finished image
static void write_result_manifest(const App& app, const Job& j) {
  if (j.output_path.empty()) return;
  PngInfo png = read_png_info(j.output_path);
  Json m = Json::object();
  m.set("schema", Json("serenity.server_result.v1"));
  m.set("job_id", Json(j.id));
  m.set("state", Json(j.state));
  m.set("model", Json(j.model));
  m.set("output_path", Json(j.output_path));
  m.set("output_bytes", Json(static_cast<int64_t>(file_size(j.output_path))));
  m.set("output_width", Json(static_cast<int64_t>(png.width)));
  m.set("output_height", Json(static_cast<int64_t>(png.height)));
  m.set("has_genparams_text", Json(png.text.count("serenity.genparams.v1") > 0));
  Json sub = Json::object();
  for (const char* k : {"sampler", "scheduler", "seed", "steps", "cfg", "width", "height"}) sub.set(k, j.params.get(k));
  m.set("submitted", sub);
  Json wf = Json::object();
  for (const char* k : {"workflow_schema", "workflow_executor", "workflow_source", "workflow_route_kind", "workflow_node_count", "workflow_edge_count"})
    if (j.request.present(k)) wf.set(k, j.request.get(k));
  m.set("workflow", wf);
  std::string rel = j.output_path.compare(0, app.out_dir.size(), app.out_dir) == 0 ? j.output_path.substr(app.out_dir.size()) : "";
  Json loc = Json::object();
  loc.set("root_kind", Json("ui_workflow_gallery"));
  loc.set("root", Json(app.out_dir));
  loc.set("inside_root", Json(!rel.empty()));
  loc.set("relative_path", Json(rel.empty() ? rel : rel.substr(rel[0] == '/' ? 1 : 0)));
  m.set("output_location", loc);
  std::string sidecar = j.output_path + ".worker_result.json";
  m.set("worker_sidecar_present", Json(file_exists(sidecar)));
  write_file_atomic(j.output_path + ".serenity_server_result.json", m.dump());
}

// ---- the worker driver thread ----------------------------------------------------------------------------------------------
static std::vector<std::string> split_cmd(const std::string& cmd, const std::string& kind) {
  std::vector<std::string> out;
  std::string cur;
  bool in_q = false;
  for (char c : cmd) {
    if (c == '"') { in_q = !in_q; continue; }
    if (c == ' ' && !in_q) { if (!cur.empty()) out.push_back(cur); cur.clear(); continue; }
    cur += c;
  }
  if (!cur.empty()) out.push_back(cur);
  for (auto& a : out) { size_t p; while ((p = a.find("{kind}")) != std::string::npos) a.replace(p, 6, kind); }
  return out;
}

static bool spawn_and_handshake(App& app, mdb::WorkerProc& w, const std::string& kind, std::string* err) {
  if (!w.spawn(split_cmd(app.worker_cmd, kind), err)) return false;
  auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(600);     // model load happens before "ready"
  std::string line;
  while (std::chrono::steady_clock::now() < deadline && !app.shutting_down) {
    auto r = w.next_line(&line, 200);
    if (r == mdb::WorkerProc::Line) {
      wire::Event ev;
      if (wire::parse_event(line, &ev) && ev.kind == wire::Event::Ready) return true;
      continue;                                     // tolerate log noise before the handshake
    }
    if (r == mdb::WorkerProc::PeerClosed || r == mdb::WorkerProc::IoError) { *err = "worker exited before ready"; w.kill_and_reap(); return false; }
  }
  *err = "worker did not become ready in time";
  w.kill_and_reap();
  return false;
}

static void finish_job(App& app, Job& j, const wire::Event& ev) {      // app.mu held
  if (ev.kind == wire::Event::Done) { j.state = "done"; j.output_path = ev.output_path; j.step = j.total; }
  else if (ev.kind == wire::Event::Failed) { j.state = "failed"; j.error = ev.error; }
  else { j.state = "cancelled"; }
  app.publish_locked(j, ws_frame_for(j, ev));
  if (j.state == "done") write_result_manifest(app, j);
  app.persist_locked();
}

static void driver_thread(App* ap) {
  App& app = *ap;
  mdb::WorkerProc worker;
  while (!app.shutting_down) {
    std::shared_ptr<Job> job;
    {
      std::unique_lock<std::mutex> lk(app.mu);
      app.cv.wait_for(lk, std::chrono::milliseconds(500), [&] {
        if (app.shutting_down) return true;
        for (auto& j : app.jobs) if (j->state == "queued") return true;
        return false;
      });
      if (app.shutting_down) break;
      for (auto& j : app.jobs) if (j->state == "queued") { job = j; break; }
      if (!job) continue;
      if (job->cancel_requested) { wire::Event ev; ev.kind = wire::Event::Cancelled; finish_job(app, *job, ev); continue; }
      job->state = "running";
      app.in_flight = job->id;
    }
    auto fail = [&](const std::string& msg) {
      std::lock_guard<std::mutex> lk(app.mu);
      wire::Event ev; ev.kind = wire::Event::Failed; ev.error = msg;
      finish_job(app, *job, ev);
      app.in_flight.clear();
    };
    const Family* fam = family_of(job->model);
    if (!fam) { fail("no worker kind for model '" + job->model + "'"); continue; }
    job->pass = 1;
    std::string kind = fam->kind;
    if (worker.alive() && kind != app.resident_kind) {
      worker.kill_and_reap();                                            // model swap: exit is what frees device memory
      std::this_thread::sleep_for(std::chrono::milliseconds(app.settle_ms));
    }
    if (!worker.alive()) {
      std::string err;
      if (!spawn_and_handshake(app, worker, kind, &err)) { fail("worker unavailable (spawn failed): " + err); continue; }
      app.resident_kind = kind;
    }
    std::string err;
    if (!worker.send_line(wire::start_line(job->params), &err)) { worker.kill_and_reap(); fail("send_start failed: " + err); continue; }
    bool cancel_sent = false;
    while (true) {
      {
        std::lock_guard<std::mutex> lk(app.mu);
        if (job->cancel_requested && !cancel_sent) { std::string e2; worker.send_line(wire::kCancelLine, &e2); cancel_sent = true; }
      }
      std::string line;
      auto r = worker.next_line(&line, 100);
      if (app.shutting_down) break;
      if (r == mdb::WorkerProc::Idle) continue;
      if (r == mdb::WorkerProc::PeerClosed || r == mdb::WorkerProc::IoError) {
        worker.kill_and_reap();                                          // respawn lazily with the next job
        fail(r == mdb::WorkerProc::PeerClosed ? "worker process exited (peer closed)" : "worker IPC error");
        break;
      }
      wire::Event ev;
      std::string perr;
      if (!wire::parse_event(line, &ev, &perr)) continue;               // a malformed line is dropped, the job goes on
      std::lock_guard<std::mutex> lk(app.mu);
      if (ev.kind == wire::Event::Progress) {
        job->step = ev.step; job->total = ev.total; job->phase = ev.phase;
        app.publish_locked(*job, ws_frame_for(*job, ev));
      } else if (ev.terminal()) {
        if (ev.kind == wire::Event::Done && job->hires_scale > 1.0 && job->pass == 1 && !job->cancel_requested) {
          // Hires two-pass: the base image becomes the init image of an img2img pass at the scaled size (the worker
          // resamples it; snapped to 512 or 1024 like the encoder grids it supports), under the same job id. Only the
          // second pass publishes the terminal event. The base file is moved under a name the gallery does not list.
          std::string base = ev.output_path;
          size_t slash = base.find_last_of('/');
          std::string src = (slash == std::string::npos ? std::string("") : base.substr(0, slash + 1)) + "hires_src_" + (slash == std::string::npos ? base : base.substr(slash + 1));
          if (rename(base.c_str(), src.c_str()) != 0) src = base;
          long long side = std::max(job->params.get("width").as_int(), job->params.get("height").as_int());
          long long target = static_cast<long long>(side * job->hires_scale + 0.5) >= 768 ? 1024 : 512;
          Json p2 = job->params;
          p2.set("init_image", Json(src)); p2.set("creativity", Json(job->hires_denoise));
          p2.set("width", Json(static_cast<int64_t>(target))); p2.set("height", Json(static_cast<int64_t>(target)));
          job->pass = 2; job->hires_src = src; job->phase = "hires";
          wire::Event pe; pe.kind = wire::Event::Progress; pe.step = 0; pe.total = job->total; pe.phase = "hires";
          app.publish_locked(*job, ws_frame_for(*job, pe));
          std::string e2;
          if (!worker.send_line(wire::start_line(p2), &e2)) {
            wire::Event fe; fe.kind = wire::Event::Failed; fe.error = "hires pass-2 send_start failed: " + e2;
            finish_job(app, *job, fe);
            app.in_flight.clear();
            worker.kill_and_reap();
            break;
          }
          continue;
        }
        finish_job(app, *job, ev);
        if (!job->hires_src.empty() && job->hires_src != job->output_path) remove(job->hires_src.c_str());
        app.in_flight.clear();
        break;
      }
    }
  }
  worker.kill_and_reap();
}

// ---- admission ---------------------------------------------------------------------------------------------------------------
static Json limits_json() {
  Json l = Json::object();
  l.set("min_side", Json(64)); l.set("max_side", Json(4096)); l.set("side_multiple", Json(16));
  l.set("max_steps", Json(4096)); l.set("max_images", Json(64));
  l.set("runtime_shapes", Json(true));
  return l;
}
static std::string admission_error(const Json& p) {
  const std::string model = p.str("model");
  if (model.empty()) return "model is required";
  const Family* fam = family_of(model);
  if (!fam) return "unknown model family for '" + model + "'";
  if (!fam->admitted) return std::string("model family '") + fam->kind + "' is blocked: " + fam->note;
  long long w = p.get("width").as_int(), h = p.get("height").as_int(), steps = p.get("steps").as_int(), images = p.get("images").as_int();
  if (w < 64 || w > 4096 || h < 64 || h > 4096 || w % 16 || h % 16) return "width/height must be multiples of 16 within [64, 4096]";
  if (steps < 1 || steps > 4096) return "steps out of range [1, 4096]";
  if (images < 1 || images > 64) return "images out of range [1, 64]";
  auto known = [](const std::vector<std::string>& v, const std::string& s) { return s.empty() || std::find(v.begin(), v.end(), mdb::graph::lower(s)) != v.end(); };
  if (!known(kSamplers, p.str("sampler"))) return "unsupported sampler '" + p.str("sampler") + "'";
  if (!known(kSchedulers, p.str("scheduler"))) return "unsupported scheduler '" + p.str("scheduler") + "'";
  if (p.str("prompt").empty() && std::string(fam->kind) != "stub") return "prompt is required";
  for (const char* k : {"init_image", "mask_image", "reference_image"})
    if (!p.str(k).empty() && p.str(k)[0] == '/' && !file_exists(p.str(k))) return std::string(k) + " does not exist: " + p.str(k);
  return "";
}
static Json capabilities_json() {
  Json c = Json::object();
  c.set("schema", Json("serenity.capabilities.v1"));
  Json fams = Json::array();
  for (auto& f : families()) {
    Json o = Json::object();
    o.set("kind", Json(f.kind)); o.set("admitted", Json(f.admitted)); o.set("note", Json(f.note));
    Json feats = Json::object();
    bool img = std::string(f.kind) != "ltx2";
    feats.set("txt2img", Json(img)); feats.set("img2img", Json(img)); feats.set("inpaint", Json(img)); feats.set("lora", Json(true));
    feats.set("video", Json(!img));
    o.set("features", feats);
    fams.push(o);
  }
  c.set("families", fams);
  Json s = Json::array(); for (auto& x : kSamplers) s.push(Json(x));
  Json sc = Json::array(); for (auto& x : kSchedulers) sc.push(Json(x));
  c.set("samplers", s); c.set("schedulers", sc); c.set("limits", limits_json());
  return c;
}

// ---- request handling ------------------------------------------------------------------------------------------------------------
static void reply(http::Response& rs, int status, const Json& body) { rs.status = status; rs.body = body.dump(); }
static void reply_error(http::Response& rs, int status, const std::string& msg, const char* schema = nullptr) {
  Json e = Json::object();
  if (schema) e.set("schema", Json(schema));
  e.set("error", Json(msg));
  reply(rs, status, e);
}

// lower + validate; on success fills params (wire) and lowered request
static bool prepare(const std::string& body, Json* lowered, Json* params, int* status, Json* report) {
  Json req;
  std::string perr;
  if (!Json::try_parse(body, &req, &perr) || !req.is_object()) {
    *status = 400; *report = Json::object(); report->set("error", Json("invalid request body: " + perr)); return false;
  }
  bool has_wf = req.present("workflow");
  try {
    mdb::graph::lower_request(req);
  } catch (const mdb::graph::GraphError& ge) {
    *status = ge.status;
    Json r = Json::object();
    r.set("schema", Json("serenity.generate.error.v1"));
    r.set("error", Json(ge.text()));
    r.set("stage", Json("workflow_lowering"));
    r.set("same_gate_as_preflight", Json(true));
    if (ge.node_id >= 0) r.set("node_id", Json(static_cast<int64_t>(ge.node_id)));
    if (!ge.type_id.empty()) r.set("type_id", Json(ge.type_id));
    *report = r;
    return false;
  }
  if (has_wf && req.str("workflow_route_kind") == "audio") {
    *status = 501; *report = Json::object();
    report->set("schema", Json("serenity.generate.error.v1"));
    report->set("error", Json("workflow route 'audio' has no worker")); report->set("same_gate_as_preflight", Json(true));
    return false;
  }
  std::string err;
  if (!wire::params_from_request(req, params, &err)) { *status = 400; *report = Json::object(); report->set("error", Json(err)); return false; }
  std::string adm = admission_error(*params);
  if (adm.empty() && req.present("hires_scale")) {
    double hs = req.get("hires_scale").is_number() ? req.get("hires_scale").as_double() : -1.0;
    double hd = req.present("hires_denoise") ? (req.get("hires_denoise").is_number() ? req.get("hires_denoise").as_double() : -1.0) : 0.35;
    if (hs < 1.0 || hs > 4.0) adm = "hires_scale out of range [1, 4]";
    else if (hd <= 0.0 || hd > 1.0) adm = "hires_denoise out of range (0, 1]";
    else if (hs > 1.0 && std::string(family_of(params->str("model"))->kind) == "ltx2") adm = "hires two-pass applies to image models";
  }
  if (!adm.empty()) {
    *status = 400;
    Json r = Json::object();
    r.set("schema", Json("serenity.generate.error.v1"));
    r.set("error", Json(adm));
    r.set("stage", Json("prequeue_gate"));
    r.set("same_gate_as_preflight", Json(true));
    r.set("limits", limits_json());
    *report = r;
    return false;
  }
  *lowered = req;
  return true;
}

static std::vector<std::string> enqueue(App& app, const Json& lowered, Json params) {
  std::vector<std::string> ids;
  long long images = std::max<long long>(1, params.get("images").as_int());
  std::lock_guard<std::mutex> lk(app.mu);
  for (long long i = 0; i < images; ++i) {
    auto j = std::make_shared<Job>();
    char buf[32];
    snprintf(buf, sizeof buf, "job-%04lld", ++app.next_id);
    j->id = buf;
    Json p = params;
    p.set("job_id", Json(j->id));
    p.set("out_dir", Json(app.out_dir));
    p.set("image_index", Json(i));
    p.set("image_count", Json(images));
    p.set("images", Json(1));
    if (i > 0) p.set("seed", Json(params.get("seed").as_int() + i));        // serial fan-out: one seed per image
    Json gp = lowered;
    gp.erase("workflow");
    gp.set_if_missing("schema", Json("serenity.genparams.v1"));
    gp.set("job_id", Json(j->id));
    gp.set("seed", p.get("seed"));
    p.set("params_json", Json(gp.dump()));
    j->params = p;
    j->request = lowered;
    j->model = p.str("model");
    j->created = now_http_date();
    j->total = p.get("steps").as_int();
    j->image_index = i;
    j->image_count = images;
    if (lowered.get("hires_scale").is_number()) j->hires_scale = lowered.get("hires_scale").as_double();
    if (lowered.get("hires_denoise").is_number()) j->hires_denoise = lowered.get("hires_denoise").as_double();
    app.jobs.push_back(j);
    ids.push_back(j->id);
  }
  app.persist_locked();
  app.cv.notify_all();
  return ids;
}

// ---- checkpoint scan: architecture from the safetensors header (first MiB of key names) or from the file name ----------
static std::string header_text(const std::string& path, size_t cap = 1 << 20) {
  std::ifstream f(path, std::ios::binary);
  unsigned char len8[8];
  if (!f || !f.read(reinterpret_cast<char*>(len8), 8)) return "";
  unsigned long long n = 0;
  for (int i = 0; i < 8; ++i) n |= static_cast<unsigned long long>(len8[i]) << (8 * i);
  if (n == 0 || n > (1ull << 33)) return "";
  std::string s(static_cast<size_t>(std::min<unsigned long long>(n, cap)), '\0');
  f.read(&s[0], static_cast<std::streamsize>(s.size()));
  s.resize(static_cast<size_t>(f.gcount()));
  return s;
}
static bool has(const std::string& h, const char* needle) { return h.find(needle) != std::string::npos; }
// substring probes over tensor names, most specific first
static std::string detect_arch(const std::string& h) {
  if (h.empty()) return "unknown";
  if (has(h, "\"noise_refiner.")) return "zimage";
  if (has(h, "\"double_stream_modulation_img")) return "flux-2/klein";
  if (has(h, "\"distilled_guidance_layer")) return "chroma";
  if (has(h, "\"double_blocks.")) return "flux";
  if (has(h, "\"audio_vae.") || has(h, "audio_to_video_attn")) return "ltx2";
  if (has(h, "\"embed_image_indicator.weight\"") || has(h, "\"llm_cond_proj.weight\"")) return "ideogram4";
  if (has(h, "\"model.diffusion_model.joint_blocks") || has(h, "\"joint_blocks.")) return "sd3";
  if (has(h, "\"model.diffusion_model.input_blocks") || has(h, "\"input_blocks.0.")) return "sdxl";
  if (has(h, "\"txt_norm.")) return "qwen-image";
  if (has(h, "\"time_projection.")) return "wan";
  if (has(h, "\"adaLN_sa_ln") || has(h, ".adaLN_sa_ln.")) return "ernie-image";
  if (has(h, "\"net.blocks.0.adaln_modulation_self_attn")) return "anima";
  if (has(h, "scale_shift_table") && has(h, "transformer_blocks.0.attn1.")) return "ltx2";
  if (has(h, "\"decoder.up.") || has(h, "\"decoder.up_blocks.") || has(h, "\"decoder.upsamples.")) return "vae";
  return "unknown";
}
static std::string detect_arch_from_name(const std::string& name) {
  std::string lo = mdb::graph::lower(name);
  auto any = [&](std::initializer_list<const char*> ns) { for (auto* n : ns) if (lo.find(n) != std::string::npos) return true; return false; };
  if (any({"wan2.2", "wan 2.2", "wan-2.2", "wan_2_2", "wan22"})) return "wan2.2";
  if (any({"zimage_l2p", "z-image-l2p", "z_image_l2p", "l2p"})) return "zimage-l2p";
  if (any({"hidream", "hi-dream", "hi_dream"})) return "hidream";
  if (any({"sensenova", "sense_nova", "sense-nova"})) return "sensenova";
  if (any({"qwen"})) return "qwen-image";
  if (any({"sd3", "sd35"})) return "sd3";
  if (any({"sdxl", "stable-diffusion-xl", "animagine"})) return "sdxl";
  if (any({"flux2", "flux-2", "flux_2"})) return "flux-2";
  if (any({"flux1", "flux-1", "flux_1", "flux-dev"})) return "flux";
  if (any({"ltx"})) return "ltx2";
  return "unknown";
}
static std::string detect_lora_target_arch(const std::string& h) {
  if (has(h, "\"noise_refiner.") || has(h, "\"context_refiner.")) return "zimage";
  if (has(h, "\"layers.") && has(h, ".lora_")) return "zimage";
  if (has(h, "zimage") || has(h, "z_image")) return "zimage";
  if (has(h, "\"lora_unet_") || has(h, "\"lora_te1") || has(h, "\"lora_te2")) return "sdxl";
  if (has(h, "\"lora_transformer_distilled_guidance_layer")) return "chroma";
  if (has(h, "\"lora_transformer_single_transformer_blocks") || has(h, "\"lora_transformer_transformer_blocks") || has(h, "\"lora_transformer")) return "flux";
  if (has(h, "qwen")) return "qwen-image";
  if (has(h, "ideogram")) return "ideogram4";
  if (has(h, "ltx") || has(h, "diffusion_model.transformer_blocks")) return "ltx2";
  return "unknown";
}
static bool looks_like_lora(const std::string& h) { return has(h, ".lora_down.") || has(h, ".lora_A.") || has(h, ".lora_up.") || has(h, ".lora_B."); }

static void list_models(const App& app, Json& out) {
  Json arr = Json::array();
  if (!app.models_dir.empty()) {
    if (DIR* d = opendir(app.models_dir.c_str())) {
      while (dirent* e = readdir(d)) {
        std::string n = e->d_name;
        if (n == "." || n == "..") continue;
        std::string full = app.models_dir + "/" + n;
        struct stat st;
        if (stat(full.c_str(), &st) != 0) continue;
        bool dir = S_ISDIR(st.st_mode);
        if (!dir && (n.size() < 12 || n.compare(n.size() - 12, 12, ".safetensors") != 0)) continue;
        Json m = Json::object();
        m.set("name", Json(n)); m.set("path", Json(full)); m.set("bytes", Json(static_cast<int64_t>(dir ? 0 : st.st_size)));
        const Family* f = family_of(n);
        m.set("kind", Json(f ? f->kind : "unknown")); m.set("admitted", Json(f ? f->admitted : false));
        // architecture: the file name decides when it is recognisable, else the tensor names of the header
        std::string arch = detect_arch_from_name(n), source = "name", header;
        if (!dir) header = header_text(full);
        bool lora = !dir && looks_like_lora(header);
        if (lora) { m.set("lora", Json(true)); std::string t = detect_lora_target_arch(header); if (arch == "unknown") { arch = t; source = "header"; } }
        else if (arch == "unknown") { arch = detect_arch(header); source = arch == "unknown" ? "none" : "header"; }
        m.set("arch", Json(arch)); m.set("arch_source", Json(source));
        arr.push(m);
      }
      closedir(d);
    }
  }
  out.set("models", arr);
}

// ---- prompt generator: language models on disk, one throw-away process per request --------------------------------------
static bool ends_with(const std::string& s, const char* suf) { size_t n = strlen(suf); return s.size() >= n && s.compare(s.size() - n, n, suf) == 0; }
static void scan_llms(const std::string& dir, bool deep, std::vector<Json>* out) {
  std::vector<std::string> names;
  if (DIR* d = opendir(dir.c_str())) {
    while (dirent* e = readdir(d)) { std::string n = e->d_name; if (n != "." && n != "..") names.push_back(n); }
    closedir(d);
  } else return;
  std::sort(names.begin(), names.end());
  auto add = [&](const std::string& path, int64_t size) {
    std::string base = path.substr(path.find_last_of('/') + 1);
    size_t dot = base.find_last_of('.');
    Json m = Json::object();
    m.set("id", Json(path)); m.set("name", Json(dot == std::string::npos || !ends_with(base, ".gguf") ? base : base.substr(0, dot)));
    m.set("path", Json(path)); m.set("size", Json(size));
    out->push_back(m);
  };
  bool has_cfg = false; int64_t st_bytes = 0; bool has_st = false;
  for (auto& n : names) { if (n == "config.json") has_cfg = true; if (ends_with(n, ".safetensors")) { has_st = true; st_bytes += file_size(dir + "/" + n); } }
  if (has_cfg && has_st) { add(dir, st_bytes); return; }
  for (auto& n : names) {
    std::string full = dir + "/" + n;
    struct stat st;
    if (stat(full.c_str(), &st) != 0) continue;
    if (S_ISDIR(st.st_mode)) { if (deep) scan_llms(full, false, out); }
    else if (ends_with(n, ".gguf")) add(full, st.st_size);
  }
}
// run argv, collect stdout and stderr (each at most 1 MiB), kill it after timeout_s; returns the exit status or -1
static int run_capture(const std::vector<std::string>& argv, int timeout_s, std::string* out, std::string* err) {
  int po[2], pe[2];
  if (pipe(po) != 0) return -1;
  if (pipe(pe) != 0) { close(po[0]); close(po[1]); return -1; }
  pid_t pid = fork();
  if (pid < 0) { close(po[0]); close(po[1]); close(pe[0]); close(pe[1]); return -1; }
  if (pid == 0) {
    dup2(po[1], 1); dup2(pe[1], 2);
    close(po[0]); close(po[1]); close(pe[0]); close(pe[1]);
    std::vector<char*> av;
    for (auto& a : argv) av.push_back(const_cast<char*>(a.c_str()));
    av.push_back(nullptr);
    execvp(av[0], av.data());
    _exit(127);
  }
  close(po[1]); close(pe[1]);
  auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(timeout_s);
  pollfd fds[2] = {{po[0], POLLIN, 0}, {pe[0], POLLIN, 0}};
  int open_fds = 2;
  bool timed_out = false;
  char buf[4096];
  while (open_fds > 0) {
    auto left = std::chrono::duration_cast<std::chrono::milliseconds>(deadline - std::chrono::steady_clock::now()).count();
    if (left <= 0) { timed_out = true; break; }
    int r = poll(fds, 2, static_cast<int>(std::min<long long>(left, 1000)));
    if (r < 0) break;
    for (int i = 0; i < 2; ++i) {
      if (fds[i].fd < 0 || !(fds[i].revents & (POLLIN | POLLHUP | POLLERR))) continue;
      ssize_t n = read(fds[i].fd, buf, sizeof(buf));
      if (n > 0) { std::string* dst = i == 0 ? out : err; if (dst->size() < (1u << 20)) dst->append(buf, static_cast<size_t>(n)); }
      else { close(fds[i].fd); fds[i].fd = -1; --open_fds; }
    }
  }
  for (auto& f : fds) if (f.fd >= 0) close(f.fd);
  if (timed_out) kill(pid, SIGKILL);
  int status = 0;
  waitpid(pid, &status, 0);
  if (timed_out) { *err += "timed out"; return -1; }
  return WIFEXITED(status) ? WEXITSTATUS(status) : -1;
}
static std::string trim(const std::string& s) {
  size_t a = s.find_first_not_of(" \t\r\n"), b = s.find_last_not_of(" \t\r\n");
  return a == std::string::npos ? "" : s.substr(a, b - a + 1);
}

static Json gallery_items(App& app) {
  Json meta;
  std::string raw;
  if (!read_file(app.out_dir + "/gallery.json", &raw) || !Json::try_parse(raw, &meta) || !meta.is_object()) meta = Json::object();
  Json items = Json::array();
  std::vector<std::string> names;
  if (DIR* d = opendir(app.out_dir.c_str())) {
    while (dirent* e = readdir(d)) { std::string n = e->d_name; if (n.size() > 4 && n.compare(n.size() - 4, 4, ".png") == 0) names.push_back(n); }
    closedir(d);
  }
  std::sort(names.begin(), names.end());
  for (auto& n : names) {
    std::string id = n.substr(0, n.size() - 4), path = app.out_dir + "/" + n;
    PngInfo png = read_png_info(path);
    Json it = Json::object();
    it.set("id", Json(id)); it.set("path", Json(path)); it.set("url", Json("/out/" + n));
    it.set("width", Json(static_cast<int64_t>(png.width))); it.set("height", Json(static_cast<int64_t>(png.height)));
    it.set("bytes", Json(static_cast<int64_t>(file_size(path))));
    Json gp;
    auto t = png.text.find("serenity.genparams.v1");
    if (t != png.text.end() && Json::try_parse(t->second, &gp)) it.set("genparams", gp);
    const Json& m = meta.get(id);
    it.set("favorite", Json(m.get("favorite").as_bool(false)));
    it.set("title", Json(m.str("title", id)));
    Json mf = Json::object();
    mf.set("server", Json(file_exists(path + ".serenity_server_result.json") ? "/out/" + n + ".serenity_server_result.json" : ""));
    it.set("result_manifests", mf);
    items.push(it);
  }
  return items;
}
static void gallery_meta_update(App& app, const std::string& id, const std::string& key, const Json& v) {
  Json meta;
  std::string raw;
  if (!read_file(app.out_dir + "/gallery.json", &raw) || !Json::try_parse(raw, &meta) || !meta.is_object()) meta = Json::object();
  Json e = meta.get(id).is_object() ? meta.get(id) : Json::object();
  e.set(key, v);
  meta.set(id, e);
  write_file_atomic(app.out_dir + "/gallery.json", meta.dump());
}

static bool starts_with(const std::string& s, const char* p) { return s.rfind(p, 0) == 0; }

static void handle(App& app, const http::Request& rq, http::Response& rs) {
  const std::string& p = rq.path;
  const std::string& m = rq.method;
  if (m == "OPTIONS") { rs.status = 204; return; }
  if (p == "/v1/health") {
    Json h = Json::object();
    std::lock_guard<std::mutex> lk(app.mu);
    long long queued = 0;
    for (auto& j : app.jobs) queued += j->state == "queued";
    h.set("status", Json("ok")); h.set("backend", Json(app.resident_kind)); h.set("in_flight", Json(app.in_flight));
    h.set("queued", Json(queued)); h.set("jobs", Json(app.jobs.size())); h.set("out_dir", Json(app.out_dir));
    return reply(rs, 200, h);
  }
  if (p == "/v1/samplers") {
    Json o = Json::object(), s = Json::array(), sc = Json::array();
    for (auto& x : kSamplers) s.push(Json(x));
    for (auto& x : kSchedulers) sc.push(Json(x));
    o.set("schema", Json("serenity.samplers.v1")); o.set("samplers", s); o.set("schedulers", sc);
    return reply(rs, 200, o);
  }
  if (p == "/v1/capabilities") return reply(rs, 200, capabilities_json());
  if (p == "/v1/models") { Json o = Json::object(); list_models(app, o); return reply(rs, 200, o); }
  if ((p == "/v1/preflight" || p == "/v1/generate") && m == "POST") {
    Json lowered, params, report;
    int status = 200;
    bool ok = prepare(rq.body, &lowered, &params, &status, &report);
    if (p == "/v1/preflight") {
      Json o = Json::object();
      o.set("schema", Json("serenity.generate.preflight.v1"));
      o.set("admitted", Json(ok));
      o.set("same_gate_as_generate", Json(true));
      if (!ok) o.set("rejection", report);
      else {
        const Family* f = family_of(params.str("model"));
        o.set("kind", Json(f ? f->kind : ""));
        o.set("lowered", lowered);
      }
      Json root = Json::object();
      root.set("root_kind", Json("ui_workflow_gallery")); root.set("root", Json(app.out_dir)); root.set("artifact_pattern", Json("job-XXXX.png"));
      o.set("output_root", root);
      o.set("limits", limits_json());
      return reply(rs, 200, o);
    }
    if (!ok) return reply(rs, status, report);
    auto ids = enqueue(app, lowered, params);
    Json o = Json::object(), arr = Json::array();
    for (auto& id : ids) arr.push(Json(id));
    o.set("job_id", Json(ids.front())); o.set("job_ids", arr); o.set("state", Json("queued"));
    return reply(rs, 200, o);
  }
  if (p == "/v1/grid" && m == "POST") {
    // XYZ grid: {"base": {...request...}, "axes": [{"key": "cfg", "values": [..]}, ...]} -> one job per combination
    Json body;
    if (!Json::try_parse(rq.body, &body) || !body.get("base").is_object() || !body.get("axes").is_array() || body.get("axes").size() == 0 || body.get("axes").size() > 3)
      return reply_error(rs, 400, "grid needs base (object) and 1..3 axes");
    std::vector<Json> combos = {body.get("base")};
    for (const Json& ax : body.get("axes").items()) {
      if (!ax.get("key").is_string() || !ax.get("values").is_array() || ax.get("values").size() == 0) return reply_error(rs, 400, "grid axis needs key and values");
      std::vector<Json> next;
      for (auto& c : combos) for (const Json& v : ax.get("values").items()) { Json n = c; n.set(ax.str("key"), v); next.push_back(n); }
      combos.swap(next);
      if (combos.size() > 256) return reply_error(rs, 400, "grid has more than 256 cells");
    }
    std::vector<std::pair<Json, Json>> ready;
    for (auto& c : combos) {
      Json lowered, params, report;
      int status = 200;
      if (!prepare(c.dump(), &lowered, &params, &status, &report)) return reply(rs, status, report);   // all or nothing
      ready.emplace_back(lowered, params);
    }
    Json cells = Json::array();
    for (auto& r : ready) for (auto& id : enqueue(app, r.first, r.second)) cells.push(Json(id));
    Json o = Json::object();
    o.set("schema", Json("serenity.grid.v1")); o.set("job_ids", cells); o.set("cells", Json(cells.size()));
    return reply(rs, 200, o);
  }
  if ((p == "/v1/cancel" || starts_with(p, "/v1/cancel/")) && m == "POST") {
    std::string id = p.size() > 11 ? p.substr(11) : "";
    if (id.empty()) { Json b; if (Json::try_parse(rq.body, &b)) id = !b.str("job_id").empty() ? b.str("job_id") : b.str("id"); }
    std::lock_guard<std::mutex> lk(app.mu);
    if (id.empty()) id = app.in_flight;
    auto j = app.find(id);
    if (!j) return reply_error(rs, 404, "no such job: " + id);
    if (j->terminal()) { Json o = j->summary(); o.set("cancelled", Json(false)); return reply(rs, 200, o); }
    j->cancel_requested = true;
    app.cv.notify_all();
    Json o = j->summary();
    o.set("cancelled", Json(true));
    return reply(rs, 200, o);
  }
  if (p == "/v1/progress") {
    std::string id = !rq.param("job").empty() ? rq.param("job") : rq.param("job_id");
    if (mdb::graph::lower(rq.header("upgrade")) != "websocket") {
      std::lock_guard<std::mutex> lk(app.mu);
      auto j = app.find(id);
      if (!j) return reply_error(rs, 404, "no such job: " + id);
      return reply(rs, 200, j->summary());
    }
    rs.upgrade_ws = true;
    rs.ws_topic = id;
    return;
  }
  if (p == "/v1/jobs" && m == "GET") {
    std::lock_guard<std::mutex> lk(app.mu);
    Json arr = Json::array();
    for (auto& j : app.jobs) arr.push(j->summary());
    Json o = Json::object();
    o.set("jobs", arr); o.set("in_flight", Json(app.in_flight));
    return reply(rs, 200, o);
  }
  if (starts_with(p, "/v1/job/")) {
    std::string rest = p.substr(8);
    bool want_result = rest.size() > 7 && rest.compare(rest.size() - 7, 7, "/result") == 0;
    std::string id = want_result ? rest.substr(0, rest.size() - 7) : rest;
    std::lock_guard<std::mutex> lk(app.mu);
    auto j = app.find(id);
    if (!j) return reply_error(rs, 404, "no such job: " + id);
    Json o = j->summary();
    if (want_result) {
      std::string raw;
      Json mf;
      if (!j->output_path.empty() && read_file(j->output_path + ".serenity_server_result.json", &raw) && Json::try_parse(raw, &mf)) o.set("result", mf);
      else o.set("result", Json());
    } else o.set("params", j->params);
    return reply(rs, 200, o);
  }
  if ((p == "/v1/reorder" || p == "/v1/remove") && m == "POST") {
    Json b;
    if (!Json::try_parse(rq.body, &b)) return reply_error(rs, 400, "invalid JSON body");
    std::lock_guard<std::mutex> lk(app.mu);
    if (p == "/v1/remove") {
      std::string id = !b.str("job_id").empty() ? b.str("job_id") : b.str("id");
      for (auto it = app.jobs.begin(); it != app.jobs.end(); ++it)
        if ((*it)->id == id) {
          if ((*it)->state == "running") return reply_error(rs, 409, "job is running; cancel it instead");
          app.jobs.erase(it);
          app.persist_locked();
          Json o = Json::object(); o.set("removed", Json(id));
          return reply(rs, 200, o);
        }
      return reply_error(rs, 404, "no such job: " + id);
    }
    // reorder: {"order": [ids of queued jobs in the wanted order]}: unnamed queued jobs keep their relative order after them
    if (!b.get("order").is_array()) return reply_error(rs, 400, "reorder needs order: [job ids]");
    std::vector<std::shared_ptr<Job>> queued, named;
    for (auto& j : app.jobs) if (j->state == "queued") queued.push_back(j);
    for (const Json& idj : b.get("order").items())
      for (auto& j : queued) if (j->id == idj.as_string() && std::find(named.begin(), named.end(), j) == named.end()) named.push_back(j);
    for (auto& j : queued) if (std::find(named.begin(), named.end(), j) == named.end()) named.push_back(j);
    size_t k = 0;
    for (auto& slot : app.jobs) if (slot->state == "queued") slot = named[k++];
    app.persist_locked();
    Json arr = Json::array();
    for (auto& j : named) arr.push(Json(j->id));
    Json o = Json::object(); o.set("order", arr);
    return reply(rs, 200, o);
  }
  if ((p == "/upload/image" || p == "/upload/mask") && m == "POST") {
    std::string bytes, name;
    Json b;
    if (!rq.body.empty() && rq.body[0] == '{' && Json::try_parse(rq.body, &b)) {
      std::string data = !b.str("data").empty() ? b.str("data") : b.str("image");
      size_t k = data.find("base64,");
      bytes = http::base64_decode(k == std::string::npos ? data : data.substr(k + 7));
      name = b.str("name");
    } else bytes = rq.body;
    if (bytes.size() < 8 || bytes.compare(0, 8, "\x89PNG\r\n\x1a\n") != 0) return reply_error(rs, 400, "upload is not a PNG");
    for (auto& ch : name) if (!isalnum(static_cast<unsigned char>(ch)) && ch != '-' && ch != '_') ch = '_';
    if (name.empty()) name = std::string(p == "/upload/mask" ? "mask-" : "image-") + std::to_string(time(nullptr)) + "-" + std::to_string(++app.next_id);
    mkdirs(app.out_dir + "/uploads");
    std::string path = app.out_dir + "/uploads/" + name + ".png";
    if (!write_file_atomic(path, bytes)) return reply_error(rs, 500, "cannot write upload");
    Json o = Json::object();
    o.set("path", Json(path)); o.set("url", Json("/out/uploads/" + name + ".png")); o.set("bytes", Json(bytes.size()));
    return reply(rs, 200, o);
  }
  if (p == "/v1/gallery" && m == "GET") { Json o = Json::object(); o.set("items", gallery_items(app)); return reply(rs, 200, o); }
  if (p == "/v1/gallery/read" && m == "GET") {
    std::string path = rq.param("path");
    if (!inside_root(path, app.out_dir)) return reply_error(rs, 400, "path outside the gallery root");
    PngInfo png = read_png_info(path);
    if (!png.ok) return reply_error(rs, 404, "not a PNG: " + path);
    Json o = Json::object(), text = Json::object();
    for (auto& kv : png.text) text.set(kv.first, Json(kv.second));
    o.set("width", Json(static_cast<int64_t>(png.width))); o.set("height", Json(static_cast<int64_t>(png.height))); o.set("text", text);
    return reply(rs, 200, o);
  }
  if (starts_with(p, "/v1/gallery/")) {
    std::string rest = p.substr(12), id = rest, action;
    size_t slash = rest.find('/');
    if (slash != std::string::npos) { id = rest.substr(0, slash); action = rest.substr(slash + 1); }
    if (!safe_relative(id)) return reply_error(rs, 400, "bad gallery id");
    std::string path = app.out_dir + "/" + id + ".png";
    if (!file_exists(path)) return reply_error(rs, 404, "no such gallery item: " + id);
    if (m == "DELETE") {
      unlink(path.c_str());
      unlink((path + ".serenity_server_result.json").c_str());
      Json o = Json::object(); o.set("deleted", Json(id));
      return reply(rs, 200, o);
    }
    if (m == "POST" && (action == "favorite" || action == "rename")) {
      Json b;
      Json::try_parse(rq.body, &b);
      if (action == "favorite") gallery_meta_update(app, id, "favorite", Json(b.get("favorite").as_bool(true)));
      else gallery_meta_update(app, id, "title", Json(b.str("title", b.str("name", id))));
    }
    Json all = gallery_items(app);
    for (const Json& it : all.items()) if (it.str("id") == id) return reply(rs, 200, it);
    return reply_error(rs, 404, "no such gallery item: " + id);
  }
  if (p == "/v1/state") {
    std::string path = app.out_dir + "/state/ui_state.json";
    if (m == "POST") {
      Json b;
      if (!Json::try_parse(rq.body, &b)) return reply_error(rs, 400, "invalid JSON body");
      mkdirs(app.out_dir + "/state");
      write_file_atomic(path, b.dump());
      return reply(rs, 200, b);
    }
    std::string raw;
    Json b = Json::object();
    if (read_file(path, &raw)) Json::try_parse(raw, &b);
    return reply(rs, 200, b);
  }
  if (p == "/v1/presets" || starts_with(p, "/v1/presets/")) {
    std::string dir = app.out_dir + "/state/presets";
    mkdirs(dir);
    std::string name = p.size() > 12 ? p.substr(12) : "";
    if (name.empty() && m == "POST") { Json b; if (Json::try_parse(rq.body, &b)) name = b.str("name"); }
    if (name.empty()) {
      Json arr = Json::array();
      if (DIR* d = opendir(dir.c_str())) {
        while (dirent* e = readdir(d)) { std::string n = e->d_name; if (n.size() > 5 && n.compare(n.size() - 5, 5, ".json") == 0) arr.push(Json(n.substr(0, n.size() - 5))); }
        closedir(d);
      }
      Json o = Json::object(); o.set("presets", arr);
      return reply(rs, 200, o);
    }
    if (!safe_relative(name) || name.find('/') != std::string::npos) return reply_error(rs, 400, "bad preset name");
    std::string path = dir + "/" + name + ".json";
    if (m == "POST") {
      Json b;
      if (!Json::try_parse(rq.body, &b)) return reply_error(rs, 400, "invalid JSON body");
      write_file_atomic(path, b.dump());
      return reply(rs, 200, b);
    }
    if (m == "DELETE") { unlink(path.c_str()); Json o = Json::object(); o.set("deleted", Json(name)); return reply(rs, 200, o); }
    std::string raw;
    Json b;
    if (!read_file(path, &raw) || !Json::try_parse(raw, &b)) return reply_error(rs, 404, "no such preset: " + name);
    return reply(rs, 200, b);
  }
  if (starts_with(p, "/out/")) {
    std::string rel = p.substr(5);
    if (!safe_relative(rel)) return reply_error(rs, 400, "bad path");
    std::string data;
    if (!read_file(app.out_dir + "/" + rel, &data)) return reply_error(rs, 404, "not found");
    rs.body = data;
    rs.content_type = rel.size() > 4 && rel.compare(rel.size() - 4, 4, ".png") == 0 ? "image/png"
                      : rel.size() > 5 && rel.compare(rel.size() - 5, 5, ".json") == 0 ? "application/json" : "application/octet-stream";
    return;
  }
  // ---- video: the LTX-2 worker writes a PNG sequence (<job>.frames/NNNN.png) and a sidecar; no container encoder exists
  //      in this build, so "mp4" stays empty and the result names the frame directory instead
  //      (serenitymojo/serve/video_api.mojo:146-477)
  if (p == "/v1/video" && m == "GET") {
    Json o = Json::object();
    o.set("schema", Json("serenity.video_status.v1")); o.set("endpoint", Json("/v1/video"));
    o.set("accepted", Json(true)); o.set("backend", Json("ltx2")); o.set("container", Json("png-sequence"));
    o.set("mp4", Json("")); o.set("audio", Json(false));
    o.set("ffprobe", Json(system("command -v ffprobe >/dev/null 2>&1") == 0));
    Json t = Json::object();
    t.set("target_width", Json(768)); t.set("target_height", Json(512)); t.set("target_frame_count", Json(121)); t.set("target_fps", Json(24));
    o.set("ltx2", t);
    { std::lock_guard<std::mutex> lk(app.mu); o.set("resident", Json(app.resident_kind)); }
    return reply(rs, 200, o);
  }
  if (p == "/v1/video" && m == "POST") {
    Json body;
    if (!Json::try_parse(rq.body, &body) || !body.is_object()) return reply_error(rs, 400, "invalid request body", "serenity.video_error.v1");
    if (body.str("model").empty()) body.set("model", Json("ltx2"));
    const Family* vf = family_of(body.str("model"));
    if (!vf || std::string(vf->kind) != "ltx2") return reply_error(rs, 400, "/v1/video needs a video model (family ltx2), got '" + body.str("model") + "'", "serenity.video_error.v1");
    body.set_if_missing("width", Json(768)); body.set_if_missing("height", Json(512));
    body.set_if_missing("frames", Json(121)); body.set_if_missing("fps", Json(24));
    long long frames = body.get("frames").as_int(), fps = body.get("fps").as_int();
    if (frames < 1 || frames > 1025 || (frames - 1) % 8 != 0) return reply_error(rs, 400, "frames must be 8k + 1 within [1, 1025]", "serenity.video_error.v1");
    if (fps < 1 || fps > 120) return reply_error(rs, 400, "fps out of range [1, 120]", "serenity.video_error.v1");
    body.set("images", Json(1));
    Json lowered, params, report;
    int status = 200;
    if (!prepare(body.dump(), &lowered, &params, &status, &report)) return reply(rs, status, report);
    auto ids = enqueue(app, lowered, params);
    Json o = Json::object();
    o.set("schema", Json("serenity.video_job.v1")); o.set("job_id", Json(ids.front())); o.set("state", Json("queued"));
    o.set("frames", Json(frames)); o.set("fps", Json(fps)); o.set("container", Json("png-sequence"));
    o.set("result", Json("/v1/video/result?job=" + ids.front()));
    return reply(rs, 200, o);
  }
  if (p == "/v1/video/result" && m == "GET") {
    std::string id = rq.param("job");
    std::shared_ptr<Job> j;
    { std::lock_guard<std::mutex> lk(app.mu); j = app.find(id); }
    if (!j) return reply_error(rs, 404, "no such job: " + id, "serenity.video_error.v1");
    Json o = Json::object();
    std::lock_guard<std::mutex> lk(app.mu);
    o.set("schema", Json("serenity.video_result.v1")); o.set("job_id", Json(j->id)); o.set("state", Json(j->state));
    o.set("ready", Json(j->state == "done")); o.set("error", Json(j->error)); o.set("mp4", Json("")); o.set("audio", Json(false));
    o.set("container", Json("png-sequence"));
    long long count = 0, w = 0, h = 0;
    std::string fdir;
    if (j->state == "done" && j->output_path.size() > 4) {
      fdir = j->output_path.substr(0, j->output_path.size() - 4) + ".frames";
      if (DIR* d = opendir(fdir.c_str())) {
        while (dirent* e = readdir(d)) { std::string n = e->d_name; if (n.size() > 4 && n.compare(n.size() - 4, 4, ".png") == 0) ++count; }
        closedir(d);
      }
      PngInfo png = read_png_info(j->output_path);
      w = png.width; h = png.height;
    }
    Json gp;
    double fps = 24.0;
    if (Json::try_parse(j->params.str("params_json"), &gp) && gp.get("fps").is_number()) fps = gp.get("fps").as_double();
    o.set("first_frame", Json(j->output_path)); o.set("frames_dir", Json(count > 0 ? fdir : std::string("")));
    o.set("frame_count", Json(static_cast<int64_t>(count))); o.set("width", Json(static_cast<int64_t>(w))); o.set("height", Json(static_cast<int64_t>(h)));
    o.set("fps", Json(fps)); o.set("duration", Json(fps > 0 ? count / fps : 0.0));
    return reply(rs, 200, o);
  }
  if (p == "/v1/video/probe" && m == "POST") {
    Json body;
    if (!Json::try_parse(rq.body, &body) || body.str("path").empty()) return reply_error(rs, 400, "probe needs a path", "serenity.video_error.v1");
    std::string path = body.str("path");
    if (!inside_root(path, app.out_dir)) return reply_error(rs, 400, "path outside the gallery root", "serenity.video_error.v1");
    struct stat st;
    if (stat(path.c_str(), &st) != 0) return reply_error(rs, 404, "no such file: " + path, "serenity.video_error.v1");
    if (S_ISDIR(st.st_mode)) {                      // a frame directory: count and measure the frames
      long long count = 0;
      std::string first;
      if (DIR* d = opendir(path.c_str())) {
        while (dirent* e = readdir(d)) { std::string n = e->d_name; if (n.size() > 4 && n.compare(n.size() - 4, 4, ".png") == 0) { ++count; if (first.empty() || n < first) first = n; } }
        closedir(d);
      }
      PngInfo png = first.empty() ? PngInfo() : read_png_info(path + "/" + first);
      Json o = Json::object();
      o.set("schema", Json("serenity.video_probe.v1")); o.set("container", Json("png-sequence")); o.set("frame_count", Json(static_cast<int64_t>(count)));
      o.set("width", Json(static_cast<int64_t>(png.width))); o.set("height", Json(static_cast<int64_t>(png.height))); o.set("audio", Json(false));
      return reply(rs, 200, o);
    }
    if (system("command -v ffprobe >/dev/null 2>&1") != 0) return reply_error(rs, 501, "ffprobe is not available on PATH", "serenity.video_error.v1");
    return reply_error(rs, 501, "container probing is not built: only PNG frame directories are produced here", "serenity.video_error.v1");
  }
  if (p == "/v1/llms") {
    std::vector<Json> found;
    if (!app.llm_dir.empty()) scan_llms(app.llm_dir, true, &found);
    std::sort(found.begin(), found.end(), [](const Json& a, const Json& b) { return a.str("name") < b.str("name"); });
    Json arr = Json::array();
    for (auto& f : found) arr.push(f);
    Json o = Json::object();
    o.set("llms", arr);
    return reply(rs, 200, o);
  }
  if (p == "/v1/magic_prompt") {
    if (m != "POST") return reply_error(rs, 405, "POST {idea, aspect, model}");
    Json b;
    if (!Json::try_parse(rq.body, &b)) return reply_error(rs, 400, "bad json");
    std::string idea = trim(b.str("idea")), aspect = b.str("aspect", "1:1"), model = b.str("model");
    if (idea.empty()) return reply_error(rs, 400, "idea required");
    bool stub = model.compare(0, 5, "stub:") == 0;
    if (model.empty() || !file_exists(stub ? model.substr(5) : model))
      return reply_error(rs, 400, "valid model path required");
    // one throw-away process per request: the language model holds device memory only while it generates
    std::vector<std::string> argv = split_cmd(app.magic_cmd, "");
    argv.push_back(model); argv.push_back(aspect); argv.push_back(idea);
    std::string out, err;
    int rc = run_capture(argv, 600, &out, &err);
    std::string caption = trim(out);
    size_t nl = caption.find_last_of('\n');
    if (nl != std::string::npos) caption = caption.substr(nl + 1);          // the last line is the caption
    if (rc != 0) return reply_error(rs, 500, "magic_prompt failed: " + trim(err).substr(0, 2000));
    if (caption.empty()) return reply_error(rs, 500, "empty caption");
    Json o = Json::object();
    o.set("caption", Json(caption));
    return reply(rs, 200, o);
  }
  if (p == "/" || p == "/index.html") {
    rs.content_type = "text/html";
    rs.body = "<!doctype html><title>mdb-server</title><h1>mdb-server</h1><p>POST /v1/generate, GET /v1/jobs, WS /v1/progress?job=ID</p>";
    return;
  }
  reply_error(rs, 404, "no route: " + m + " " + p);
}

static App* g_app = nullptr;
static void on_signal(int) { if (g_app) { g_app->shutting_down = true; g_app->server.stop(); } }

int main(int argc, char** argv) {
  App app;
  int port = 0;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    auto next = [&]() -> std::string { return i + 1 < argc ? argv[++i] : ""; };
    if (a == "--worker") app.worker_cmd = next();
    else if (a == "--out-dir") app.out_dir = next();
    else if (a == "--port") port = atoi(next().c_str());
    else if (a == "--models-dir") app.models_dir = next();
    else if (a == "--llm-dir") app.llm_dir = next();
    else if (a == "--magic-cmd") app.magic_cmd = next();
    else if (a == "--settle-ms") app.settle_ms = atoi(next().c_str());
    else { std::cerr << "unknown argument " << a << "\n"; return 2; }
  }
  if (app.worker_cmd.empty() || app.out_dir.empty()) {
    std::cerr << "usage: mdb-server --worker \"<cmd> [{kind}]\" --out-dir DIR [--port N] [--models-dir DIR] [--llm-dir DIR] [--magic-cmd CMD] [--settle-ms N]\n";
    return 2;
  }
  while (app.out_dir.size() > 1 && app.out_dir.back() == '/') app.out_dir.pop_back();
  mkdirs(app.out_dir);
  signal(SIGPIPE, SIG_IGN);
  g_app = &app;
  signal(SIGINT, on_signal);
  signal(SIGTERM, on_signal);
  std::string err;
  if (!app.server.listen_on(port, &err)) { std::cerr << "listen: " << err << "\n"; return 1; }
  std::cout << "{\"listening\":" << app.server.port() << "}" << std::endl;      // one line: tests read the port from it
  std::thread driver(driver_thread, &app);
  app.server.run(
      [&](const http::Request& rq, http::Response& rs) {
        try { handle(app, rq, rs); }
        catch (const std::exception& e) { reply_error(rs, 500, std::string("internal error: ") + e.what()); }
      },
      [&](const std::string& topic, size_t* cursor, bool* done) {
        std::vector<std::string> frames;
        std::lock_guard<std::mutex> lk(app.mu);
        auto j = app.find(topic);
        if (!j) { if (*cursor == 0) { frames.push_back("{\"error\":\"no such job\"}"); *cursor = 1; } *done = true; return frames; }
        if (*cursor == 0) { Json s = j->summary(); s.set("ev", Json("snapshot")); frames.push_back(s.dump()); }
        size_t sent = *cursor == 0 ? 0 : *cursor - 1;
        while (sent < j->events.size()) frames.push_back(j->events[sent++]);
        *cursor = sent + 1;
        *done = j->terminal() && sent >= j->events.size();
        return frames;
      });
  app.shutting_down = true;
  app.cv.notify_all();
  driver.join();
  return 0;
}
