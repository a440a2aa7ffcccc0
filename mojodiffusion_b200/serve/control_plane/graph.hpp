// Workflow-graph lowering: turns a node graph (ComfyUI API prompt, ComfyUI canvas export, an Ideogram-4 canvas export,
// a typed {nodes, edges} graph, or a flat {params}/{genparams} wrapper) into the flat generation parameters a worker
// understands. Keys already present in the request win ("first writer wins"): the graph only fills what is missing.
//
// Design: a registry of node kinds. Each kind lists its output slots (for the API-prompt "[node, slot]" links) and a
// handler that reads typed inputs through a small context object; the engine repeatedly scans nodes in document order
// and fires every node whose linked inputs exist, until all have fired or no progress is possible (cycle / dangling).
// Errors carry an HTTP class: 501 = this server cannot do what the graph asks, 422 = the graph itself is malformed.
//
// Behaviour follows serenity-server/crates/graph/src/{lib.rs:470-640, execute.rs:486-1160, execute_handlers.rs,
// import.rs:118-566,675-910,1266-1477, util.rs}.
#pragma once
#include <algorithm>
#include <functional>
#include <map>
#include <optional>
#include <set>
#include <string>
#include <vector>

#include "json.hpp"

namespace mdb {
namespace graph {

constexpr const char* kSchema = "serenity.workflow_graph.v1";
constexpr const char* kExecutor = "serenity.workflow_graph.executor.v1";

struct GraphError {
  int status;                 // 501 unsupported, 422 bad request
  std::string message;
  long long node_id = -1;
  std::string type_id;
  std::string text() const {
    std::string s = "[" + std::to_string(status) + "] " + message;
    if (node_id >= 0) s += " (node " + std::to_string(node_id) + ")";
    if (!type_id.empty()) s += " (type " + type_id + ")";
    return s;
  }
};
inline GraphError unsupported(std::string m, long long node = -1, std::string type = "") {
  return GraphError{501, std::move(m), node, std::move(type)};
}
inline GraphError bad_request(std::string m, long long node = -1) { return GraphError{422, std::move(m), node, ""}; }

// ---- values that flow along edges ----------------------------------------------------------------------------
struct Value {
  std::string type;           // MODEL CLIP VAE CONDITIONING IMAGE MASK LATENT NOISE SAMPLER SIGMAS GUIDER INT FLOAT ...
  std::string text;           // model name | conditioning text | image path | sampler name | scheduler | string scalar
  std::string source;         // mask channel / mask source of an image
  long long i = 0;            // int scalar | seed | steps
  double f = 0;               // float scalar | denoise
  bool b = false;
  // latent geometry (also attached to a conditioning that carries a reference latent)
  bool has_geom = false;
  long long width = 0, height = 0, batch = 1;
  std::string init_image, mask_image;
};

struct Node {
  long long id;
  std::string type;
  Json fields;
};
struct Edge {
  long long from_node; std::string from_port;
  long long to_node; std::string to_port;
};
struct TypedGraph {
  std::vector<Node> nodes;
  std::vector<Edge> edges;
};

// ---- field access with the numeric leniency the formats need ------------------------------------------------------
inline std::string fstr(const Json& o, const std::string& k) { return o.str(k); }
inline long long opt_int(const Json& o, const std::string& k, long long d, long long lo, long long hi) {
  if (!o.present(k)) return d;
  const Json& v = o.get(k);
  if (!v.is_int()) throw bad_request("'" + k + "' must be an integer");
  if (v.as_int() < lo || v.as_int() > hi)
    throw bad_request("'" + k + "' out of range [" + std::to_string(lo) + ".." + std::to_string(hi) + "]");
  return v.as_int();
}
inline long long lenient_int(const Json& o, const std::string& k, long long d) {
  if (!o.present(k)) return d;
  const Json& v = o.get(k);
  if (v.is_number()) return v.as_int();
  if (v.is_string()) {
    char* end = nullptr;
    long long r = strtoll(v.as_string().c_str(), &end, 10);
    if (end && *end == 0 && !v.as_string().empty()) return r;
  }
  throw unsupported("workflow graph field " + k + " must be an integer");
}
inline double opt_float(const Json& o, const std::string& k, double d, double lo, double hi) {
  if (!o.present(k)) return d;
  const Json& v = o.get(k);
  double n;
  if (v.is_number()) n = v.as_double();
  else if (v.is_string()) {
    char* end = nullptr;
    n = strtod(v.as_string().c_str(), &end);
    if (!end || *end || v.as_string().empty()) throw unsupported("workflow graph field " + k + " must be numeric");
  } else throw unsupported("workflow graph field " + k + " must be numeric");
  if (n < lo || n > hi) throw unsupported("workflow graph field " + k + " out of range");
  return n;
}
inline bool opt_bool(const Json& o, const std::string& k, bool d) {
  if (!o.present(k)) return d;
  const Json& v = o.get(k);
  if (v.is_bool()) return v.as_bool();
  if (v.is_int()) return v.as_int() != 0;
  if (v.is_string()) {
    std::string l = v.as_string();
    std::transform(l.begin(), l.end(), l.begin(), ::tolower);
    if (l == "true" || l == "yes" || l == "1") return true;
    if (l == "false" || l == "no" || l == "0") return false;
  }
  throw unsupported("workflow graph field " + k + " must be a boolean");
}
inline std::string lower(std::string s) { std::transform(s.begin(), s.end(), s.begin(), ::tolower); return s; }
inline std::string canonical_type(const std::string& t) { return t.rfind("comfy/", 0) == 0 ? t.substr(6) : t; }
inline void copy_field_if_missing(Json& out, const Json& fields, const std::string& src, const std::string& dst) {
  if (fields.present(src)) out.set_if_missing(dst, fields.get(src));
}

// ---- scalar / named node tables ----------------------------------------------------------------------------------
inline std::string scalar_kind(const std::string& t) {
  static const std::map<std::string, std::string> m = {
      {"PrimitiveInt", "INT"}, {"INTConstant", "INT"}, {"easy int", "INT"}, {"SeedNode", "INT"},
      {"PrimitiveFloat", "FLOAT"}, {"FloatConstant", "FLOAT"}, {"easy float", "FLOAT"},
      {"PrimitiveString", "STRING"}, {"PrimitiveStringMultiline", "STRING"}, {"StringConstant", "STRING"},
      {"StringConstantMultiline", "STRING"}, {"easy string", "STRING"},
      {"PrimitiveBoolean", "BOOLEAN"}, {"BOOLConstant", "BOOLEAN"}};
  auto it = m.find(t);
  return it == m.end() ? "" : it->second;
}
inline bool is_scalar_node(const std::string& t) { return !scalar_kind(t).empty() || t == "PrimitiveNode"; }
inline std::string json_scalar_type(const Json& v) {
  return v.is_bool() ? "BOOLEAN" : v.is_int() ? "INT" : v.is_number() ? "FLOAT" : v.is_string() ? "STRING" : "";
}
inline std::string scalar_output_type(const std::string& t, const Json& fields) {
  std::string k = scalar_kind(t);
  if (!k.empty()) return k;
  if (t == "PrimitiveNode") {
    std::string d = fstr(fields, "output_type");
    if (d.empty())
      for (const char* key : {"value", "text", "string"})
        if (fields.has(key)) { d = json_scalar_type(fields.get(key)); break; }
    if (d == "INT" || d == "FLOAT" || d == "STRING" || d == "BOOLEAN") return d;
  }
  return "";
}
inline std::string named_sampler(const std::string& t) {
  static const std::map<std::string, std::string> m = {
      {"SamplerEuler", "euler"}, {"SamplerEulerAncestral", "euler_ancestral"},
      {"SamplerEulerAncestralCFGPP", "euler_ancestral_cfg_pp"}, {"SamplerDPMPP_2M_SDE", "dpmpp_2m_sde"},
      {"SamplerDPMPP_3M_SDE", "dpmpp_3m_sde"}, {"SamplerDPMPP_SDE", "dpmpp_sde"},
      {"SamplerDPMPP_2S_Ancestral", "dpmpp_2s_ancestral"}, {"SamplerDPMAdaptative", "dpm_adaptive"},
      {"SamplerLMS", "lms"}, {"SamplerER_SDE", "er_sde"}, {"SamplerSASolver", "sa_solver"}, {"SamplerSEEDS2", "seeds_2"}};
  auto it = m.find(t);
  return it == m.end() ? "" : it->second;
}
inline std::string named_scheduler(const std::string& t) {
  static const std::map<std::string, std::string> m = {
      {"KarrasScheduler", "karras"}, {"ExponentialScheduler", "exponential"},
      {"PolyexponentialScheduler", "polyexponential"}, {"SDTurboScheduler", "turbo"}, {"VPScheduler", "vp"},
      {"BetaSamplingScheduler", "beta"}, {"LaplaceScheduler", "laplace"}};
  auto it = m.find(t);
  return it == m.end() ? "" : it->second;
}
inline bool worker_supports_sampler(const std::string& n) {
  static const std::set<std::string> s = {"euler", "flowmatch_euler", "flow_match_euler", "dpmpp_2m", "dpm++ 2m", "uni_pc", "uni_pc_bh2"};
  return s.count(lower(n)) > 0;
}
inline bool worker_supports_scheduler(const std::string& n) {
  static const std::set<std::string> s = {"simple", "flowmatch", "flow_match", "sgm_uniform"};
  return s.count(lower(n)) > 0;
}

// ---- execution context ---------------------------------------------------------------------------------------------
class Engine;
struct Ctx {
  Engine& eng;
  const Node& node;
  Json& out;
  bool pending = false;       // a linked input exists but its producer has not fired yet

  bool linked(const std::string& port) const;
  // typed input; required: missing link -> 501; wrong type -> 422
  const Value* in(const std::string& port, const std::string& type, bool required = true);
  const Value* in_any(const std::string& port, bool required);
  // scalar override: if ``port`` is linked use the scalar, else the widget/field default
  long long int_in(const std::string& port, long long field_default);
  double float_in(const std::string& port, double field_default);
  std::string string_in(const std::string& port, std::string field_default);
  bool bool_in(const std::string& port, bool field_default);
  void emit(const std::string& port, Value v);
  void emit_as(const std::string& port, const std::string& type, Value v);
  [[noreturn]] void missing(const std::string& what = "required typed input") const {
    throw unsupported("workflow graph " + node.type + " missing " + what, node.id);
  }
};

using Handler = std::function<void(Ctx&)>;
struct Kind {
  std::vector<std::string> slots;   // output port per API-prompt slot index
  Handler run;
};

class Engine {
 public:
  explicit Engine(const TypedGraph& g) : g_(g) {
    for (const Edge& e : g.edges) {
      auto key = std::make_pair(e.to_node, e.to_port);
      if (links_.count(key)) throw bad_request("workflow graph input has multiple sources: " + e.to_port, e.to_node);
      links_[key] = {e.from_node, e.from_port};
    }
  }
  static const std::map<std::string, Kind>& registry();

  void run(Json& out) {
    std::vector<bool> done(g_.nodes.size(), false);
    size_t remaining = g_.nodes.size();
    while (remaining > 0) {
      bool progressed = false;
      for (size_t i = 0; i < g_.nodes.size(); ++i) {
        if (done[i]) continue;
        if (fire(g_.nodes[i], out)) { done[i] = true; --remaining; progressed = true; }
      }
      if (!progressed) throw bad_request("workflow graph has unresolved or cyclic typed links");
    }
    if (reference_latents > 0) out.set_if_missing("reference_latent_count", Json(reference_latents));
  }

  const std::pair<long long, std::string>* link(long long node, const std::string& port) const {
    auto it = links_.find({node, port});
    return it == links_.end() ? nullptr : &it->second;
  }
  // the only inbound edge of a pass-through node, whatever its port is called
  const std::pair<long long, std::string>* sole_link(long long node) const {
    const std::pair<long long, std::string>* found = nullptr;
    for (auto& kv : links_)
      if (kv.first.first == node) {
        if (found) throw bad_request("workflow graph pass-through node has multiple inputs", node);
        found = &kv.second;
      }
    return found;
  }
  const Value* value(long long node, const std::string& port) const {
    auto it = values_.find({node, port});
    return it == values_.end() ? nullptr : &it->second;
  }
  void put(long long node, const std::string& port, Value v) {
    auto key = std::make_pair(node, port);
    if (values_.count(key)) throw bad_request("workflow graph node produced a duplicate output: " + port, node);
    values_[key] = std::move(v);
  }
  std::map<std::string, std::pair<long long, std::string>> named;   // SetNode / GetNode bus
  long long reference_latents = 0;

 private:
  bool fire(const Node& n, Json& out);
  const TypedGraph& g_;
  std::map<std::pair<long long, std::string>, std::pair<long long, std::string>> links_;
  std::map<std::pair<long long, std::string>, Value> values_;
};

inline bool Ctx::linked(const std::string& port) const { return eng.link(node.id, port) != nullptr; }
inline const Value* Ctx::in_any(const std::string& port, bool required) {
  auto* l = eng.link(node.id, port);
  if (!l) {
    if (required) missing(port + " input");
    return nullptr;
  }
  const Value* v = eng.value(l->first, l->second);
  if (!v) pending = true;
  return v;
}
inline const Value* Ctx::in(const std::string& port, const std::string& type, bool required) {
  const Value* v = in_any(port, required);
  // a conditioning that carries a reference latent may also stand in for that latent
  if (v && type == "LATENT" && v->type == "CONDITIONING" && v->has_geom) return v;
  if (v && v->type != type)
    throw bad_request("workflow graph input " + port + " expected " + type + " but got " + v->type, node.id);
  return v;
}
inline long long Ctx::int_in(const std::string& port, long long d) {
  if (!linked(port)) return d;
  const Value* v = in(port, "INT", false);
  return v ? v->i : d;
}
inline double Ctx::float_in(const std::string& port, double d) {
  if (!linked(port)) return d;
  const Value* v = in_any(port, false);
  if (!v) return d;
  if (v->type == "FLOAT") return v->f;
  if (v->type == "INT") return static_cast<double>(v->i);
  throw bad_request("workflow graph input " + port + " expected FLOAT but got " + v->type, node.id);
}
inline std::string Ctx::string_in(const std::string& port, std::string d) {
  if (!linked(port)) return d;
  const Value* v = in(port, "STRING", false);
  return v ? v->text : d;
}
inline bool Ctx::bool_in(const std::string& port, bool d) {
  if (!linked(port)) return d;
  const Value* v = in(port, "BOOLEAN", false);
  return v ? v->b : d;
}
inline void Ctx::emit(const std::string& port, Value v) { if (!pending) eng.put(node.id, port, std::move(v)); }
inline void Ctx::emit_as(const std::string& port, const std::string& type, Value v) { v.type = type; emit(port, std::move(v)); }

// ---- small value builders -----------------------------------------------------------------------------------------------
inline Value tagged(const char* type) { Value v; v.type = type; return v; }
inline Value text_value(const char* type, std::string text) { Value v; v.type = type; v.text = std::move(text); return v; }
inline Value latent(long long w, long long h, long long batch, std::string init = "", std::string mask = "") {
  Value v; v.type = "LATENT"; v.has_geom = true; v.width = w; v.height = h; v.batch = batch;
  v.init_image = std::move(init); v.mask_image = std::move(mask);
  return v;
}
inline void write_geometry(Json& out, const Value& g) {
  if (!g.has_geom) return;
  if (g.width > 0) out.set_if_missing("width", Json(g.width));
  if (g.height > 0) out.set_if_missing("height", Json(g.height));
  out.set_if_missing("images", Json(g.batch));
  if (!g.init_image.empty()) out.set_if_missing("init_image", Json(g.init_image));
  if (!g.mask_image.empty()) out.set_if_missing("mask_image", Json(g.mask_image));
}
inline Value latent_like(const Value* g, long long dw, long long dh) {
  return g && g->has_geom ? latent(g->width, g->height, g->batch, g->init_image, g->mask_image) : latent(dw, dh, 1);
}
inline void append_lora(Json& out, const std::string& name, double weight) {
  if (name.empty()) throw unsupported("workflow graph LoRA node missing lora_name");
  Json arr = out.present("lora") && out.get("lora").is_array() ? out.get("lora") : Json::array();
  Json e = Json::object();
  e.set("name", Json(name));
  e.set("weight", Json(weight));
  arr.push(e);
  out.set("lora", arr);
}
inline void mark_terminal(Json& out, const std::string& route, const Node& n, const std::string& in_type, const std::string& prefix) {
  std::string cur = out.str("workflow_route_kind");
  std::string merged = cur.empty() || cur == route ? route : (cur == "video" || route == "video") ? "video" : cur;
  out.set("workflow_route_kind", Json(merged));
  Json plan = out.present("workflow_plan") ? out.get("workflow_plan") : Json::object();
  Json terms = plan.present("terminal_nodes") ? plan.get("terminal_nodes") : Json::array();
  Json t = Json::object();
  t.set("node_id", Json(n.id));
  t.set("type_id", Json(n.type));
  t.set("route_kind", Json(route));
  t.set("input_type", Json(in_type));
  t.set("filename_prefix", Json(prefix));
  terms.push(t);
  plan.set("schema", Json("serenity.workflow_plan.v1"));
  plan.set("route_kind", Json(merged));
  plan.set("terminal_nodes", terms);
  out.set("workflow_plan", plan);
}
inline void lanpaint_fields(Json& out, const Json& f) {
  static const std::pair<const char*, const char*> map[] = {
      {"LanPaint_NumSteps", "lanpaint_num_steps"}, {"LanPaint_Lambda", "lanpaint_lambda"},
      {"LanPaint_StepSize", "lanpaint_step_size"}, {"LanPaint_Beta", "lanpaint_beta"},
      {"LanPaint_Friction", "lanpaint_friction"}, {"LanPaint_PromptMode", "lanpaint_prompt_mode"},
      {"Inpainting_mode", "lanpaint_inpainting_mode"}, {"LanPaint_EarlyStop", "lanpaint_early_stop"},
      {"LanPaint_InnerThreshold", "lanpaint_inner_threshold"}, {"LanPaint_InnerPatience", "lanpaint_inner_patience"},
      {"add_noise", "lanpaint_add_noise"}, {"noise_seed", "lanpaint_noise_seed"},
      {"start_at_step", "lanpaint_start_at_step"}, {"end_at_step", "lanpaint_end_at_step"},
      {"return_with_leftover_noise", "lanpaint_return_with_leftover_noise"}};
  for (auto& kv : map) copy_field_if_missing(out, f, kv.first, kv.second);
}

// ---- node handlers ----------------------------------------------------------------------------------------------------
namespace handlers {

inline std::string model_name_field(const Json& f) {
  for (const char* k : {"ckpt_name", "unet_name", "model_name", "checkpoint_path"})
    if (!fstr(f, k).empty()) return fstr(f, k);
  return "";
}
inline void loader(Ctx& c, bool checkpoint) {
  std::string name = model_name_field(c.node.fields);
  if (!name.empty()) c.out.set_if_missing("model", Json(name));
  c.emit("MODEL", text_value("MODEL", name));
  if (checkpoint) { c.emit("CLIP", tagged("CLIP")); c.emit("VAE", tagged("VAE")); }
}
inline void lora(Ctx& c) {
  const bool with_clip = c.node.type == "LoraLoader";
  const Value* m = c.in("model", "MODEL");
  const Value* clip = with_clip ? c.in("clip", "CLIP") : nullptr;
  if (c.pending) return;
  (void)clip;
  if (!m->text.empty()) c.out.set_if_missing("model", Json(m->text));
  double strength = opt_float(c.node.fields, "strength_model", 1.0, -10.0, 10.0);
  double sclip = with_clip ? opt_float(c.node.fields, "strength_clip", 1.0, -10.0, 10.0) : 0.0;
  append_lora(c.out, fstr(c.node.fields, "lora_name"), strength);
  c.emit("MODEL", text_value("MODEL", m->text));
  // a text-encoder LoRA cannot be executed: the CLIP output is poisoned so that any consumer fails on its type
  if (with_clip) c.emit_as("CLIP", sclip == 0.0 ? "CLIP" : "CLIP_LORA_UNSUPPORTED", tagged("CLIP"));
}
inline std::string prompt_text(const Json& f, const std::string& type) {
  std::string t = fstr(f, "text");
  if (!t.empty() || type != "CLIPTextEncodeFlux") return t;
  return !fstr(f, "t5xxl").empty() ? fstr(f, "t5xxl") : fstr(f, "clip_l");
}
inline void text_encode(Ctx& c) {
  c.in("clip", "CLIP");
  std::string text = c.string_in("text", prompt_text(c.node.fields, c.node.type));
  if (c.pending) return;
  c.emit("CONDITIONING", text_value("CONDITIONING", text));
}
inline void qwen_edit_encode(Ctx& c) {
  c.in("clip", "CLIP");
  const Value* img = c.in("image", "IMAGE");
  std::string text = c.string_in("text", prompt_text(c.node.fields, c.node.type));
  if (c.pending) return;
  c.out.set_if_missing("qwen_edit_conditioning_image", Json(img->text));
  c.emit("CONDITIONING", text_value("CONDITIONING", text));
}
inline void empty_latent(Ctx& c) {
  const Json& f = c.node.fields;
  long long w = c.int_in("width", opt_int(f, "width", 512, 16, 2048));
  long long h = c.int_in("height", opt_int(f, "height", 512, 16, 2048));
  long long n = c.int_in("batch_size", opt_int(f, "batch_size", 1, 1, 64));
  long long frames = c.node.type == "EmptyHunyuanLatentVideo" ? c.int_in("length", opt_int(f, "length", 1, 1, 4096)) : 0;
  if (c.pending) return;
  if (c.node.type == "EmptyHunyuanLatentVideo") {
    if (frames < 1 || frames > 4096) throw unsupported("workflow graph EmptyHunyuanLatentVideo length out of range", c.node.id);
    c.out.set_if_missing("num_frames", Json(frames));
    c.out.set_if_missing("frame_count", Json(frames));
  }
  if (w < 16 || w > 2048 || h < 16 || h > 2048)
    throw unsupported("workflow graph EmptyLatentImage scalar dimensions out of range", c.node.id);
  if (n < 1 || n > 64) throw unsupported("workflow graph EmptyLatentImage scalar batch_size out of range", c.node.id);
  c.out.set_if_missing("width", Json(w));
  c.out.set_if_missing("height", Json(h));
  c.out.set_if_missing("images", Json(n));
  c.emit("LATENT", latent(w, h, n));
}
inline void set_seed_field(Json& out, const Json& f, const std::string& key) {
  if (!f.present(key)) return;
  long long s = lenient_int(f, key, -1);
  if (s >= 0) out.set_if_missing("seed", Json(s));
}
inline void ksampler(Ctx& c) {
  const Json& f = c.node.fields;
  const std::string& t = c.node.type;
  const bool adv = t == "KSamplerAdvanced";
  const Value* model = c.in("model", "MODEL");
  const Value* pos = c.in("positive", "CONDITIONING");
  const Value* neg = c.in("negative", "CONDITIONING");
  const Value* lat = c.in("latent_image", "LATENT");
  const std::string seed_port = adv && c.linked("noise_seed") ? "noise_seed" : "seed";
  long long seed_link = c.int_in(seed_port, -1);
  long long steps_link = c.int_in("steps", -1);
  double cfg_link = c.float_in("cfg", 0);
  std::string sampler_link = c.string_in("sampler_name", "");
  std::string sched_link = c.string_in("scheduler", "");
  double denoise_link = c.float_in("denoise", 1.0);
  if (c.pending) return;
  Json& out = c.out;
  if (!model->text.empty()) out.set_if_missing("model", Json(model->text));
  out.set_if_missing("prompt", Json(pos->text));
  out.set_if_missing("negative", Json(neg->text));
  write_geometry(out, *lat);
  long long steps = 0;
  if (c.linked("steps")) {
    if (steps_link < 1 || steps_link > 4096) throw unsupported("workflow graph KSampler scalar steps out of range", c.node.id);
    out.set_if_missing("steps", Json(steps_link));
    steps = steps_link;
  } else {
    copy_field_if_missing(out, f, "steps", "steps");
    if (f.get("steps").is_int()) steps = f.get("steps").as_int();
  }
  if (c.linked(seed_port)) { if (seed_link >= 0) out.set_if_missing("seed", Json(seed_link)); }
  else set_seed_field(out, f, adv && f.present("noise_seed") ? "noise_seed" : "seed");
  if (c.linked("cfg")) out.set_if_missing("cfg", Json(cfg_link)); else copy_field_if_missing(out, f, "cfg", "cfg");
  if (c.linked("sampler_name")) out.set_if_missing("sampler", Json(sampler_link));
  else copy_field_if_missing(out, f, "sampler_name", "sampler");
  if (c.linked("scheduler")) out.set_if_missing("scheduler", Json(sched_link));
  else copy_field_if_missing(out, f, "scheduler", "scheduler");
  if (adv) {
    if (lower(fstr(f, "add_noise")) == "disable")
      throw unsupported("workflow graph KSamplerAdvanced add_noise=disable (continue without re-noising) is not "
                        "representable in the flat denoise model", c.node.id);
    long long end_at = opt_int(f, "end_at_step", 1000000, 0, 10000000);
    if (steps > 0 && end_at < steps)
      throw unsupported("workflow graph KSamplerAdvanced early end_at_step (return_with_leftover_noise) is not "
                        "representable in the flat denoise model", c.node.id);
    long long start_at = opt_int(f, "start_at_step", 0, 0, 4096);
    double cr = steps > 0 ? std::min(1.0, std::max(0.0, 1.0 - static_cast<double>(start_at) / steps)) : 1.0;
    out.set_if_missing("creativity", Json(cr));
  } else if (c.linked("denoise")) {
    if (denoise_link < 0 || denoise_link > 1) throw unsupported("workflow graph KSampler scalar denoise out of range", c.node.id);
    out.set_if_missing("creativity", Json(denoise_link));
  } else {
    copy_field_if_missing(out, f, "denoise", "creativity");
  }
  if (t.rfind("LanPaint_", 0) == 0) lanpaint_fields(out, f);
  c.emit("LATENT", latent_like(lat, 512, 512));
}
inline void guider(Ctx& c, bool cfg) {
  const Value* model = c.in("model", "MODEL");
  const Value* pos = c.in(cfg ? "positive" : "conditioning", "CONDITIONING");
  const Value* neg = cfg ? c.in("negative", "CONDITIONING") : nullptr;
  double cfg_link = cfg ? c.float_in("cfg", 0) : 0;
  if (c.pending) return;
  if (!model->text.empty()) c.out.set_if_missing("model", Json(model->text));
  c.out.set_if_missing("prompt", Json(pos->text));
  if (cfg) {
    c.out.set_if_missing("negative", Json(neg->text));
    if (c.linked("cfg")) c.out.set_if_missing("cfg", Json(cfg_link));
    else copy_field_if_missing(c.out, c.node.fields, "cfg", "cfg");
  }
  // a conditioning that carries a reference latent hands its geometry on through the guider
  Value g = tagged("GUIDER");
  if (pos->has_geom) { g.has_geom = true; g.width = pos->width; g.height = pos->height; g.batch = pos->batch;
                       g.init_image = pos->init_image; g.mask_image = pos->mask_image; }
  c.emit("GUIDER", g);
}
inline void sigmas_node(Ctx& c, const std::string& fixed_scheduler, bool needs_model) {
  const Json& f = c.node.fields;
  if (needs_model) c.in("model", "MODEL");
  std::string sched = fixed_scheduler.empty() ? c.string_in("scheduler", fstr(f, "scheduler").empty() ? "simple" : fstr(f, "scheduler"))
                                              : fixed_scheduler;
  long long steps = c.int_in("steps", opt_int(f, "steps", 20, 1, 4096));
  double den = fixed_scheduler == "flux2" ? 1.0 : c.float_in("denoise", opt_float(f, "denoise", 1.0, 0.0, 1.0));
  if (c.pending) return;
  if (steps < 1 || steps > 4096) throw unsupported("workflow graph " + c.node.type + " scalar steps out of range", c.node.id);
  if (den < 0 || den > 1) throw unsupported("workflow graph " + c.node.type + " scalar denoise out of range", c.node.id);
  Value v = tagged("SIGMAS");
  v.i = steps; v.text = sched; v.f = den;
  c.emit("SIGMAS", v);
}
inline void sampler_custom_advanced(Ctx& c) {
  const Value* noise = c.in("noise", "NOISE");
  const Value* g = c.in("guider", "GUIDER");
  const Value* smp = c.in("sampler", "SAMPLER");
  const Value* sig = c.in("sigmas", "SIGMAS");
  const Value* lat = c.in("latent_image", "LATENT");
  if (c.pending) return;
  (void)g;
  Json& out = c.out;
  out.set_if_missing("seed", Json(noise->i));
  out.set_if_missing("sampler", Json(smp->text));
  out.set_if_missing("steps", Json(sig->i));
  out.set_if_missing("scheduler", Json(sig->text));
  out.set_if_missing("creativity", Json(sig->f));
  if (c.node.type == "LanPaint_SamplerCustomAdvanced") lanpaint_fields(out, c.node.fields);
  write_geometry(out, *lat);
  Value o = latent_like(lat, 0, 0);
  c.emit("LATENT", o);
  Value d = o;
  c.emit("LATENT_DENOISED", d);
}
inline void sampler_custom(Ctx& c) {
  const Json& f = c.node.fields;
  const Value* model = c.in("model", "MODEL");
  const Value* pos = c.in("positive", "CONDITIONING");
  const Value* neg = c.in("negative", "CONDITIONING");
  const Value* smp = c.in("sampler", "SAMPLER");
  const Value* sig = c.in("sigmas", "SIGMAS");
  const Value* lat = c.in("latent_image", "LATENT");
  long long seed = c.int_in("noise_seed", lenient_int(f, "noise_seed", -1));
  double cfg = c.float_in("cfg", opt_float(f, "cfg", 4.5, 0.0, 100.0));
  if (c.pending) return;
  if (!opt_bool(f, "add_noise", true))
    throw unsupported("workflow graph SamplerCustom add_noise=false is not representable in the flat denoise model", c.node.id);
  Json& out = c.out;
  if (!model->text.empty()) out.set_if_missing("model", Json(model->text));
  out.set_if_missing("prompt", Json(pos->text));
  out.set_if_missing("negative", Json(neg->text));
  if (seed >= 0) out.set_if_missing("seed", Json(seed));
  out.set_if_missing("cfg", Json(cfg));
  out.set_if_missing("sampler", Json(smp->text));
  out.set_if_missing("steps", Json(sig->i));
  out.set_if_missing("scheduler", Json(sig->text));
  out.set_if_missing("creativity", Json(sig->f));
  write_geometry(out, *lat);
  Value o = latent_like(lat, 0, 0);
  c.emit("LATENT", o);
  Value d = o;
  c.emit("LATENT_DENOISED", d);
}
inline void load_image(Ctx& c) {
  std::string p = fstr(c.node.fields, "image");
  if (p.empty()) p = fstr(c.node.fields, "path");
  if (p.empty()) throw unsupported("workflow graph " + c.node.type + " missing image path", c.node.id);
  c.emit("IMAGE", text_value("IMAGE", p));
  Value m = text_value("MASK", p);
  m.source = "load_image_mask";
  c.emit("MASK", m);
}
inline void image_passthrough(Ctx& c) {     // scale / resize: the path is what matters downstream
  const Value* img = c.in("image", "IMAGE");
  long long w = c.int_in("width", 1), h = c.int_in("height", 1);
  if (c.pending) return;
  if (w < 1 || w > 8192 || h < 1 || h > 8192) throw unsupported("workflow graph " + c.node.type + " scalar size out of range", c.node.id);
  Value v = text_value("IMAGE", img->text);
  v.source = img->source;
  c.emit("IMAGE", v);
}
inline void vae_encode(Ctx& c) {
  const Value* px = c.in("pixels", "IMAGE");
  c.in("vae", "VAE");
  if (c.pending) return;
  c.emit("LATENT", latent(0, 0, 1, px->text));
}
inline void vae_encode_inpaint(Ctx& c) {
  const Value* px = c.in("pixels", "IMAGE");
  c.in("vae", "VAE");
  const Value* m = c.in("mask", "MASK");
  if (c.pending) return;
  opt_int(c.node.fields, "grow_mask_by", 6, 0, 64);
  c.out.set_if_missing("init_image", Json(px->text));
  c.out.set_if_missing("mask_image", Json(m->text));
  c.out.set_if_missing("lanpaint_mask_channel", Json(m->source));
  c.emit("LATENT", latent(0, 0, 1, px->text, m->text));
}
inline void set_noise_mask(Ctx& c) {
  const Value* s = c.in("samples", "LATENT");
  const Value* m = c.in("mask", "MASK");
  if (c.pending) return;
  c.out.set_if_missing("mask_image", Json(m->text));
  c.out.set_if_missing("lanpaint_mask_channel", Json(m->source));
  Value o = latent_like(s, 0, 0);
  o.mask_image = m->text;
  c.emit("LATENT", o);
}
inline void inpaint_model_conditioning(Ctx& c) {
  const Value* pos = c.in("positive", "CONDITIONING");
  const Value* neg = c.in("negative", "CONDITIONING");
  c.in("vae", "VAE");
  const Value* px = c.in("pixels", "IMAGE");
  const Value* m = c.in("mask", "MASK");
  if (c.pending) return;
  bool noise_mask = opt_bool(c.node.fields, "noise_mask", true);
  Json& out = c.out;
  out.set_if_missing("init_image", Json(px->text));
  out.set_if_missing("inpaint_conditioning_image", Json(px->text));
  out.set_if_missing("inpaint_conditioning_mask", Json(m->text));
  out.set_if_missing("inpaint_conditioning_noise_mask", Json(noise_mask));
  if (noise_mask) {
    out.set_if_missing("mask_image", Json(m->text));
    out.set_if_missing("lanpaint_mask_channel", Json(m->source));
  }
  c.emit("positive", text_value("CONDITIONING", pos->text));
  c.emit("negative", text_value("CONDITIONING", neg->text));
  c.emit("LATENT", latent(0, 0, 1, px->text, noise_mask ? m->text : ""));
}
inline void reference_latent(Ctx& c) {
  const Value* cond = c.in("conditioning", "CONDITIONING");
  const Value* lat = c.linked("latent") ? c.in("latent", "LATENT") : nullptr;
  if (c.pending) return;
  Value o = text_value("CONDITIONING", cond->text);
  if (c.linked("latent")) {
    c.eng.reference_latents += 1;
    if (lat->has_geom) {
      if (!lat->init_image.empty()) {
        c.out.set_if_missing("reference_image", Json(lat->init_image));
        c.out.set_if_missing("reference_latent_method", Json("index"));
      }
      o.has_geom = true; o.width = lat->width; o.height = lat->height; o.batch = lat->batch;
      o.init_image = lat->init_image; o.mask_image = lat->mask_image;
    }
  }
  c.emit("CONDITIONING", o);
}
inline void cond_set_mask(Ctx& c) {
  const Value* cond = c.in("conditioning", "CONDITIONING");
  const Value* m = c.in("mask", "MASK");
  if (c.pending) return;
  double strength = opt_float(c.node.fields, "strength", 1.0, 0.0, 10.0);
  std::string area = lower(fstr(c.node.fields, "set_cond_area"));
  c.out.set_if_missing("conditioning_mask_image", Json(m->text));
  c.out.set_if_missing("conditioning_mask_channel", Json(m->source));
  c.out.set_if_missing("conditioning_mask_strength", Json(strength));
  c.out.set_if_missing("conditioning_mask_set_area_to_bounds", Json(!area.empty() && area != "default"));
  c.emit("CONDITIONING", text_value("CONDITIONING", cond->text));
}
inline void image_to_mask(Ctx& c) {
  const Value* img = c.in("image", "IMAGE");
  if (c.pending) return;
  std::string ch = fstr(c.node.fields, "channel");
  if (ch.empty()) ch = "red";
  std::string l = lower(ch);
  if (l == "alpha") throw unsupported("workflow graph ImageToMask alpha is unsupported on an RGB IMAGE; use LoadImage MASK", c.node.id);
  if (l != "red" && l != "green" && l != "blue") throw unsupported("workflow graph ImageToMask unsupported channel: " + ch, c.node.id);
  Value m = text_value("MASK", img->text);
  m.source = img->source.empty() ? l : img->source;
  c.out.set_if_missing("lanpaint_mask_channel", Json(m.source));
  c.emit("MASK", m);
}
inline void passthrough(Ctx& c, const std::string& out_port) {
  auto* l = out_port == "SET" || out_port == "REROUTE" ? c.eng.sole_link(c.node.id) : nullptr;
  if (!l) throw unsupported("workflow graph " + c.node.type + " missing input", c.node.id);
  const Value* src = c.eng.value(l->first, l->second);
  if (!src) { c.pending = true; return; }
  if (out_port == "SET") {
    static const std::set<std::string> ok = {"MODEL", "CLIP", "VAE", "CONDITIONING", "IMAGE", "MASK", "LATENT", "GUIDER",
                                             "SIGMAS", "NOISE", "SAMPLER", "INT", "FLOAT", "STRING", "BOOLEAN"};
    if (!ok.count(src->type)) throw unsupported("workflow graph SetNode unsupported bus type: " + src->type, c.node.id);
    std::string name;
    for (const char* k : {"name", "variable", "key", "set_name"}) if (name.empty()) name = fstr(c.node.fields, k);
    c.eng.named[name] = {c.node.id, "SET"};
  }
  c.emit(out_port, *src);
}
inline void get_node(Ctx& c) {
  std::string name;
  for (const char* k : {"name", "variable", "key", "set_name"}) if (name.empty()) name = fstr(c.node.fields, k);
  auto it = c.eng.named.find(name);
  const Value* src = it == c.eng.named.end() ? nullptr : c.eng.value(it->second.first, it->second.second);
  if (!src) { c.pending = true; return; }
  std::string declared = fstr(c.node.fields, "output_type");
  if (!declared.empty() && declared != "*" && ("," + declared + ",").find("," + src->type + ",") == std::string::npos)
    throw unsupported("workflow graph GetNode output type mismatch: " + declared + " vs " + src->type, c.node.id);
  c.emit("GET", *src);
}
inline void switch_node(Ctx& c) {
  bool sw = c.bool_in("switch", opt_bool(c.node.fields, "switch", false));
  if (c.pending) return;
  const std::string port = sw ? "on_true" : "on_false";
  if (!c.linked(port)) c.missing();
  const Value* src = c.in_any(port, true);
  if (c.pending) return;
  c.emit("output", *src);
}
inline void scalar(Ctx& c) {
  const Json& f = c.node.fields;
  std::string kind = scalar_output_type(c.node.type, f);
  if (kind.empty()) throw unsupported("workflow graph primitive scalar missing supported output type", c.node.id);
  Value v = tagged(kind.c_str());
  if (kind == "INT") v.i = f.has("value") ? lenient_int(f, "value", 0) : f.has("seed") ? lenient_int(f, "seed", 0) : 0;
  else if (kind == "FLOAT") {
    v.f = f.has("value") ? opt_float(f, "value", 0.0, -1e308, 1e308) : 0.0;
    if (c.node.type == "FloatConstant") v.f = std::round(v.f * 1e6) / 1e6;
  } else if (kind == "STRING") {
    for (const char* k : {"value", "text", "string"}) if (v.text.empty()) v.text = fstr(f, k);
    if (c.node.type == "StringConstantMultiline" && opt_bool(f, "strip_newlines", true)) {
      const std::string& s = v.text;
      if (s.find_first_of("\n\r") != std::string::npos || (!s.empty() && (isblank(s.front()) || isblank(s.back()))))
        throw unsupported("workflow graph StringConstantMultiline strip_newlines transform is unsupported", c.node.id);
    }
  } else v.b = opt_bool(f, "value", false);
  c.emit(kind, v);
}
inline void save(Ctx& c, const std::string& route) {
  const Json& f = c.node.fields;
  std::string in_type;
  if (route == "image") { c.in("images", "IMAGE"); in_type = "IMAGE"; }
  else if (route == "audio") { c.in("audio", "AUDIO"); in_type = "AUDIO"; }
  else {
    const std::string port = c.linked("video") ? "video" : "images";
    const Value* v = c.in_any(port, true);
    if (v) {
      if (v->type != "VIDEO" && v->type != "IMAGE")
        throw bad_request("workflow graph SaveVideo input " + port + " expected VIDEO or IMAGE but got " + v->type, c.node.id);
      in_type = v->type;
    }
  }
  std::string prefix = c.string_in("filename_prefix", fstr(f, "filename_prefix"));
  if (c.pending) return;
  if (!prefix.empty() && route != "audio") c.out.set_if_missing("workflow_save_prefix", Json(prefix));
  if (route == "video") {
    long long fps = opt_int(f, "fps", 24, 1, 240);
    c.out.set_if_missing("fps", Json(fps));
    c.out.set_if_missing("frame_rate", Json(fps));
  }
  mark_terminal(c.out, route, c.node, in_type, prefix);
}

}  // namespace handlers

inline const std::map<std::string, Kind>& Engine::registry() {
  using namespace handlers;
  static const std::map<std::string, Kind> reg = [] {
    std::map<std::string, Kind> r;
    auto add = [&r](std::initializer_list<const char*> names, std::vector<std::string> slots, Handler h) {
      for (const char* n : names) r[n] = Kind{slots, h};
    };
    add({"CheckpointLoaderSimple"}, {"MODEL", "CLIP", "VAE"}, [](Ctx& c) { loader(c, true); });
    add({"UNETLoader", "DiffusionModelLoader", "LTXVLoader"}, {"MODEL"}, [](Ctx& c) { loader(c, false); });
    add({"LoraLoader"}, {"MODEL", "CLIP"}, lora);
    add({"LoraLoaderModelOnly", "ZImageLoraModelOnly"}, {"MODEL"}, lora);
    add({"CLIPLoader", "DualCLIPLoader", "TripleCLIPLoader"}, {"CLIP"}, [](Ctx& c) { c.emit("CLIP", tagged("CLIP")); });
    add({"CLIPVisionLoader"}, {"CLIP_VISION"}, [](Ctx& c) { c.emit("CLIP_VISION", tagged("CLIP_VISION")); });
    add({"CLIPVisionEncode"}, {"CLIP_VISION_OUTPUT"}, [](Ctx& c) {
      c.in("clip_vision", "CLIP_VISION"); c.in("image", "IMAGE");
      c.emit("CLIP_VISION_OUTPUT", tagged("CLIP_VISION_OUTPUT"));
    });
    add({"VAELoader"}, {"VAE"}, [](Ctx& c) { c.emit("VAE", tagged("VAE")); });
    add({"EmptyLatentImage", "EmptySD3LatentImage", "EmptyFlux2LatentImage", "EmptyHunyuanLatentVideo"}, {"LATENT"}, empty_latent);
    add({"CLIPTextEncode", "CLIPTextEncodeFlux"}, {"CONDITIONING"}, text_encode);
    add({"TextEncodeQwenImageEdit", "TextEncodeQwenImageEditPlus"}, {"CONDITIONING"}, qwen_edit_encode);
    add({"ConditioningZeroOut"}, {"CONDITIONING"}, [](Ctx& c) {
      c.in("conditioning", "CONDITIONING");
      c.emit("CONDITIONING", text_value("CONDITIONING", ""));
    });
    add({"ConditioningSetMask"}, {"CONDITIONING"}, cond_set_mask);
    add({"ConditioningConcat"}, {"CONDITIONING"}, [](Ctx& c) {
      const Value* to = c.in("conditioning_to", "CONDITIONING");
      const Value* from = c.in("conditioning_from", "CONDITIONING");
      if (c.pending) return;
      std::string t = to->text.empty() ? from->text : from->text.empty() ? to->text : to->text + ", " + from->text;
      c.emit("CONDITIONING", text_value("CONDITIONING", t));
    });
    add({"ConditioningCombine", "ConditioningAverage"}, {"CONDITIONING"}, [](Ctx& c) {
      throw unsupported("workflow graph " + c.node.type + " cannot be lowered to a single text prompt (the second "
                        "conditioning / blend weight would be dropped); use ConditioningConcat to join prompts", c.node.id);
    });
    add({"FluxGuidance"}, {"CONDITIONING"}, [](Ctx& c) {
      const Value* cond = c.in("conditioning", "CONDITIONING");
      if (c.pending) return;
      copy_field_if_missing(c.out, c.node.fields, "cfg", "cfg");
      Value o = *cond;
      c.emit("CONDITIONING", o);
    });
    add({"ModelSamplingAuraFlow", "ModelSamplingSD3", "DifferentialDiffusion"}, {"MODEL"}, [](Ctx& c) {
      const Value* m = c.in("model", "MODEL");
      if (c.pending) return;
      copy_field_if_missing(c.out, c.node.fields, "shift", "sigma_shift");
      c.emit("MODEL", text_value("MODEL", m->text));
    });
    add({"KSampler", "KSamplerAdvanced", "LanPaint_KSampler", "LanPaint_KSamplerAdvanced"}, {"LATENT"}, ksampler);
    add({"KSamplerSelect"}, {"SAMPLER"}, [](Ctx& c) {
      std::string n = fstr(c.node.fields, "sampler_name");
      if (n.empty()) n = fstr(c.node.fields, "sampler");
      if (n.empty()) n = "euler";
      c.out.set_if_missing("sampler", Json(n));
      c.emit("SAMPLER", text_value("SAMPLER", n));
    });
    for (const char* n : {"SamplerEuler", "SamplerEulerAncestral", "SamplerEulerAncestralCFGPP", "SamplerDPMPP_2M_SDE",
                          "SamplerDPMPP_3M_SDE", "SamplerDPMPP_SDE", "SamplerDPMPP_2S_Ancestral", "SamplerDPMAdaptative",
                          "SamplerLMS", "SamplerER_SDE", "SamplerSASolver", "SamplerSEEDS2"})
      add({n}, {"SAMPLER"}, [](Ctx& c) {
        std::string name = named_sampler(c.node.type);
        if (!worker_supports_sampler(name))
          throw unsupported("workflow graph " + c.node.type + " lowers to unsupported sampler '" + name +
                            "'; the worker supports only euler/flowmatch_euler/dpmpp_2m/uni_pc/uni_pc_bh2", c.node.id);
        c.out.set_if_missing("sampler", Json(name));
        c.emit("SAMPLER", text_value("SAMPLER", name));
      });
    for (const char* n : {"KarrasScheduler", "ExponentialScheduler", "PolyexponentialScheduler", "SDTurboScheduler",
                          "VPScheduler", "BetaSamplingScheduler", "LaplaceScheduler"})
      add({n}, {"SIGMAS"}, [](Ctx& c) {
        std::string name = named_scheduler(c.node.type);
        if (!worker_supports_scheduler(name))
          throw unsupported("workflow graph " + c.node.type + " lowers to unsupported scheduler '" + name +
                            "'; the worker supports only simple/flowmatch/sgm_uniform", c.node.id);
        sigmas_node(c, name, false);
      });
    add({"RandomNoise"}, {"NOISE"}, [](Ctx& c) {
      long long seed = c.int_in("noise_seed", opt_int(c.node.fields, "noise_seed", 0, 0, 4294967295LL));
      if (c.pending) return;
      if (seed < 0 || seed > 4294967295LL) throw unsupported("workflow graph RandomNoise scalar noise_seed out of range", c.node.id);
      c.out.set_if_missing("seed", Json(seed));
      Value v = tagged("NOISE");
      v.i = seed;
      c.emit("NOISE", v);
    });
    add({"CFGGuider"}, {"GUIDER"}, [](Ctx& c) { guider(c, true); });
    add({"BasicGuider"}, {"GUIDER"}, [](Ctx& c) { guider(c, false); });
    add({"Flux2Scheduler"}, {"SIGMAS"}, [](Ctx& c) { sigmas_node(c, "flux2", false); });
    add({"BasicScheduler"}, {"SIGMAS"}, [](Ctx& c) { sigmas_node(c, "", true); });
    add({"SamplerCustomAdvanced", "LanPaint_SamplerCustomAdvanced"}, {"LATENT", "LATENT"}, sampler_custom_advanced);
    add({"SamplerCustom"}, {"LATENT", "LATENT"}, sampler_custom);
    add({"LoadImage", "LoadImageOutput", "LoadImageMask"}, {"IMAGE", "MASK"}, load_image);
    add({"LoadAudio"}, {"AUDIO"}, [](Ctx& c) {
      std::string p = fstr(c.node.fields, "audio");
      if (p.empty()) p = fstr(c.node.fields, "path");
      if (p.empty()) throw unsupported("workflow graph LoadAudio missing audio path", c.node.id);
      c.emit("AUDIO", text_value("AUDIO", p));
    });
    add({"ImageToMask"}, {"MASK"}, image_to_mask);
    add({"MaskToImage"}, {"IMAGE"}, [](Ctx& c) {
      const Value* m = c.in("mask", "MASK");
      if (c.pending) return;
      Value v = text_value("IMAGE", m->text);
      v.source = m->source;
      c.emit("IMAGE", v);
    });
    add({"ThresholdMask"}, {"MASK"}, [](Ctx& c) {
      const Value* m = c.in("mask", "MASK");
      if (c.pending) return;
      c.out.set_if_missing("threshold_mask_value", Json(opt_float(c.node.fields, "value", 0.5, 0.0, 1.0)));
      c.out.set_if_missing("threshold_mask_operator", Json("gt"));
      Value v = *m;
      c.emit("MASK", v);
    });
    add({"GetImageSize"}, {"width", "height", "batch_size"}, [](Ctx& c) {
      c.in("image", "IMAGE");
      if (c.pending) return;
      for (const char* p : {"width", "height", "batch_size"}) c.emit(p, tagged("INT"));
    });
    add({"GetImageSizeAndCount"}, {"IMAGE", "width", "height", "batch_size"}, [](Ctx& c) {
      const Value* img = c.in("image", "IMAGE");
      if (c.pending) return;
      c.emit("IMAGE", *img);
      c.emit("width", tagged("INT"));
      c.emit("height", tagged("INT"));
      Value one = tagged("INT");
      one.i = 1;
      c.emit("batch_size", one);
    });
    add({"ImageScale", "ImageScaleToTotalPixels", "ImageScaleBy"}, {"IMAGE"}, image_passthrough);
    // Explicit resize: representable only when both target sides are given (no keep_proportion, no zero side, no size
    // copied from another image); the sides become the request's width / height and are also INT outputs.
    add({"ImageResizeKJ"}, {"IMAGE", "width", "height"}, [](Ctx& c) {
      const Value* img = c.in("image", "IMAGE");
      const Json& f = c.node.fields;
      long long w = c.int_in("width", opt_int(f, "width", 512, 0, 8192)), h = c.int_in("height", opt_int(f, "height", 512, 0, 8192));
      if (c.linked("get_image_size")) c.in_any("get_image_size", false);
      if (c.pending) return;
      if (c.linked("get_image_size"))
        throw unsupported("workflow graph ImageResizeKJ get_image_size input copies the source image dims, which are not "
                          "resolvable in the flat single-image model", c.node.id);
      if (opt_bool(f, "keep_proportion", false))
        throw unsupported("workflow graph ImageResizeKJ keep_proportion=true derives a dimension from the source image aspect, "
                          "which is not resolvable in the flat single-image model; set explicit width and height instead", c.node.id);
      if (w == 0 || h == 0)
        throw unsupported("workflow graph ImageResizeKJ width/height of 0 keeps the source dimension, which is not resolvable "
                          "in the flat single-image model; set explicit nonzero width and height", c.node.id);
      if (w < 1 || w > 8192 || h < 1 || h > 8192) throw unsupported("workflow graph ImageResizeKJ width/height out of range", c.node.id);
      c.out.set_if_missing("width", Json(w));
      c.out.set_if_missing("height", Json(h));
      Value v = text_value("IMAGE", img->text);
      v.source = img->source;
      c.emit("IMAGE", v);
      Value wi = tagged("INT"), hi = tagged("INT");
      wi.i = w; hi.i = h;
      c.emit("width", wi);
      c.emit("height", hi);
    });
    // Inpaint compositing after decode: the mask and its channel go to the request, the pasted image is what flows on.
    add({"LanPaint_MaskBlend"}, {"IMAGE"}, [](Ctx& c) {
      const Value* a = c.in("image1", "IMAGE");
      const Value* b = c.in("image2", "IMAGE");
      const Value* m = c.in("mask", "MASK");
      if (c.pending) return;
      c.out.set_if_missing("mask_image", Json(m->text));
      c.out.set_if_missing("lanpaint_mask_channel", Json(m->source));
      copy_field_if_missing(c.out, c.node.fields, "blend_overlap", "lanpaint_mask_blend_overlap");
      c.emit("IMAGE", text_value("IMAGE", !b->text.empty() ? b->text : a->text));
    });
    // Image-to-video conditioning (Wan): size and length of the clip, the start image, conditioning passed through.
    add({"WanImageToVideo"}, {"positive", "negative", "LATENT"}, [](Ctx& c) {
      const Value* pos = c.in("positive", "CONDITIONING");
      const Value* neg = c.linked("negative") ? c.in("negative", "CONDITIONING", false) : nullptr;
      c.in("vae", "VAE");
      const Value* img = c.in("image", "IMAGE");
      if (c.linked("clip_vision_output")) c.in("clip_vision_output", "CLIP_VISION_OUTPUT", false);
      if (c.pending) return;
      const Json& f = c.node.fields;
      long long w = opt_int(f, "width", 832, 16, 4096), h = opt_int(f, "height", 480, 16, 4096), n = opt_int(f, "length", 81, 1, 4096);
      c.out.set_if_missing("width", Json(w));
      c.out.set_if_missing("height", Json(h));
      c.out.set_if_missing("num_frames", Json(n));
      c.out.set_if_missing("frame_count", Json(n));
      c.out.set_if_missing("video_conditioning_image", Json(img->text));
      c.emit("positive", text_value("CONDITIONING", pos->text));
      c.emit("negative", text_value("CONDITIONING", neg ? neg->text : ""));
      c.emit("LATENT", latent(w, h, 1, img->text));
    });
    // One-node LTX video sampler: prompt, size, clip length and rate in its widgets; emits latent, video and audio handles.
    add({"LTXVSampler"}, {"LATENT", "VIDEO", "AUDIO"}, [](Ctx& c) {
      const bool by_name = c.linked("ltxv_model");
      if (!by_name && !c.linked("model")) throw unsupported("workflow graph LTXVSampler missing ltxv_model input", c.node.id);
      const Value* m = c.in(by_name ? "ltxv_model" : "model", "MODEL");
      if (c.linked("audio")) c.in("audio", "AUDIO", false);
      if (c.pending) return;
      const Json& f = c.node.fields;
      if (!m->text.empty()) c.out.set_if_missing("model", Json(m->text));
      if (!fstr(f, "prompt").empty()) c.out.set_if_missing("prompt", Json(fstr(f, "prompt")));
      if (!fstr(f, "negative_prompt").empty()) c.out.set_if_missing("negative", Json(fstr(f, "negative_prompt")));
      long long w = opt_int(f, "width", 768, 16, 4096), h = opt_int(f, "height", 512, 16, 4096), n = opt_int(f, "num_frames", 97, 1, 4096);
      long long fps = opt_int(f, "frame_rate", 24, 1, 240);
      c.out.set_if_missing("width", Json(w));
      c.out.set_if_missing("height", Json(h));
      c.out.set_if_missing("num_frames", Json(n));
      c.out.set_if_missing("frame_count", Json(n));
      c.out.set_if_missing("steps", Json(opt_int(f, "steps", 25, 1, 1000)));
      c.out.set_if_missing("seed", Json(opt_int(f, "seed", 0, 0, 4294967295LL)));
      c.out.set_if_missing("cfg", Json(opt_float(f, "cfg", 3.0, 0.0, 100.0)));
      c.out.set_if_missing("fps", Json(fps));
      c.out.set_if_missing("frame_rate", Json(fps));
      copy_field_if_missing(c.out, f, "mode", "video_mode");
      for (const char* k : {"stg_scale", "audio_start_time", "audio_duration"}) copy_field_if_missing(c.out, f, k, k);
      c.emit("LATENT", latent(w, h, 1));
      c.emit("VIDEO", text_value("VIDEO", ""));
      c.emit("AUDIO", text_value("AUDIO", ""));
    });
    add({"ImagePadForOutpaint"}, {"IMAGE", "MASK"}, [](Ctx& c) {
      const Value* img = c.in("image", "IMAGE");
      if (c.pending) return;
      const Json& f = c.node.fields;
      c.out.set_if_missing("outpaint_left", Json(opt_int(f, "left", 0, 0, 4096)));
      c.out.set_if_missing("outpaint_top", Json(opt_int(f, "top", 0, 0, 4096)));
      c.out.set_if_missing("outpaint_right", Json(opt_int(f, "right", 0, 0, 4096)));
      c.out.set_if_missing("outpaint_bottom", Json(opt_int(f, "bottom", 0, 0, 4096)));
      c.out.set_if_missing("outpaint_feathering", Json(opt_int(f, "feathering", 40, 0, 4096)));
      c.emit("IMAGE", text_value("IMAGE", img->text));
      Value m = text_value("MASK", img->text);
      m.source = "image_pad_for_outpaint";
      c.emit("MASK", m);
    });
    add({"VAEEncode"}, {"LATENT"}, vae_encode);
    add({"VAEEncodeForInpaint"}, {"LATENT"}, vae_encode_inpaint);
    add({"RepeatLatentBatch"}, {"LATENT"}, [](Ctx& c) {
      c.in("samples", "LATENT");
      long long amount = c.int_in("amount", opt_int(c.node.fields, "amount", 1, 1, 64));
      if (c.pending) return;
      if (amount < 1 || amount > 64) throw unsupported("workflow graph RepeatLatentBatch scalar amount out of range", c.node.id);
      throw unsupported("workflow graph RepeatLatentBatch requires real latent-batch execution; use flat images=N for "
                        "serial fan-out", c.node.id);
    });
    add({"SetLatentNoiseMask"}, {"LATENT"}, set_noise_mask);
    add({"InpaintModelConditioning"}, {"positive", "negative", "LATENT"}, inpaint_model_conditioning);
    add({"ReferenceLatent"}, {"CONDITIONING"}, reference_latent);
    add({"SetNode"}, {"SET"}, [](Ctx& c) { passthrough(c, "SET"); });
    add({"GetNode"}, {"GET"}, get_node);
    add({"Reroute"}, {"REROUTE"}, [](Ctx& c) { passthrough(c, "REROUTE"); });
    add({"ComfySwitchNode"}, {"output"}, switch_node);
    add({"VAEDecode"}, {"IMAGE"}, [](Ctx& c) {
      c.in("samples", "LATENT"); c.in("vae", "VAE");
      c.emit("IMAGE", text_value("IMAGE", ""));
    });
    add({"SaveImage"}, {}, [](Ctx& c) { save(c, "image"); });
    add({"SaveVideo"}, {}, [](Ctx& c) { save(c, "video"); });
    add({"SaveAudioOpus"}, {}, [](Ctx& c) { save(c, "audio"); });
    add({"PreviewImage"}, {}, [](Ctx& c) {
      if (c.linked("images")) c.in("images", "IMAGE"); else if (c.linked("image")) c.in("image", "IMAGE");
    });
    add({"MarkdownNote", "Note"}, {}, [](Ctx&) {});
    add({"SerenityRefinerUpscaleIntent"}, {}, [](Ctx& c) {
      const Json& f = c.node.fields;
      for (const char* k : {"refiner_method", "refiner_upscale_method", "refiner_model"}) copy_field_if_missing(c.out, f, k, k);
      for (const char* k : {"refiner_upscale", "refiner_control", "refiner_steps", "refiner_cfg"}) copy_field_if_missing(c.out, f, k, k);
      c.out.set_if_missing("refiner_requested", Json(true));
    });
    for (const char* n : {"PrimitiveInt", "INTConstant", "easy int", "SeedNode", "PrimitiveFloat", "FloatConstant", "easy float",
                          "PrimitiveString", "PrimitiveStringMultiline", "StringConstant", "StringConstantMultiline",
                          "easy string", "PrimitiveBoolean", "BOOLConstant", "PrimitiveNode"})
      add({n}, {}, scalar);
    return r;
  }();
  return reg;
}

inline bool Engine::fire(const Node& n, Json& out) {
  auto& reg = registry();
  auto it = reg.find(n.type);
  if (it == reg.end()) throw unsupported("unsupported workflow graph node type: " + n.type, n.id, n.type);
  Ctx c{*this, n, out};
  try {
    it->second.run(c);
  } catch (GraphError& e) {
    if (e.node_id < 0) e.node_id = n.id;
    throw;
  }
  return !c.pending;
}

// ---- body formats -----------------------------------------------------------------------------------------------------
inline long long intish(const Json& v, const char* label) {
  if (v.is_int()) return v.as_int();
  if (v.is_number() && v.as_double() == std::floor(v.as_double())) return static_cast<long long>(v.as_double());
  if (v.is_string()) {
    char* end = nullptr;
    long long r = strtoll(v.as_string().c_str(), &end, 10);
    if (end && !*end && !v.as_string().empty()) return r;
  }
  throw unsupported(std::string("workflow graph ") + label + " must be an integer");
}

inline TypedGraph parse_typed(const Json& body) {
  TypedGraph g;
  if (!body.get("nodes").is_array()) throw unsupported("workflow graph body needs nodes");
  std::set<long long> seen;
  for (const Json& n : body.get("nodes").items()) {
    if (!n.is_object()) throw bad_request("workflow graph node must be an object");
    if (!n.present("id")) throw bad_request("workflow graph node missing id");
    long long id = intish(n.get("id"), "node id");
    if (!seen.insert(id).second) throw bad_request("workflow graph duplicate node id", id);
    std::string type = canonical_type(!n.str("type_id").empty() ? n.str("type_id") : n.str("type"));
    if (type.empty()) throw bad_request("workflow graph node missing type_id", id);
    if (!Engine::registry().count(type)) throw unsupported("unsupported workflow graph node type: " + type, id, type);
    g.nodes.push_back(Node{id, type, n.get("fields").is_object() ? n.get("fields") : Json::object()});
  }
  if (body.get("edges").is_array())
    for (const Json& e : body.get("edges").items()) {
      const Json &f = e.get("from"), &t = e.get("to");
      if (!f.is_object() || !t.is_object()) throw bad_request("workflow graph edge needs from/to endpoints");
      Edge ed{intish(f.get("node"), "edge node"), f.str("port"), intish(t.get("node"), "edge node"), t.str("port")};
      if (ed.from_port.empty() || ed.to_port.empty()) throw bad_request("workflow graph edge endpoint missing port");
      if (!seen.count(ed.from_node) || !seen.count(ed.to_node)) throw bad_request("workflow graph edge references a missing node");
      g.edges.push_back(ed);
    }
  return g;
}

// ComfyUI API prompt: {"<id>": {"class_type": ..., "inputs": {name: literal | [source id, slot]}}}
inline Json api_prompt_body(const Json& wf) {
  if (wf.get("prompt").is_object()) return wf.get("prompt");
  if (wf.get("comfy_prompt").is_object()) return wf.get("comfy_prompt");
  return wf;
}
inline bool looks_like_api_prompt(const Json& wf) {
  Json g = api_prompt_body(wf);
  if (!g.is_object() || g.size() == 0) return false;
  for (auto& m : g.members()) {
    char* end = nullptr;
    strtoll(m.first.c_str(), &end, 10);
    if (m.first.empty() || !end || *end) return false;
    if (!m.second.is_object() || !m.second.get("class_type").is_string() || !m.second.get("inputs").is_object()) return false;
  }
  return true;
}
inline bool is_link(const Json& v) {
  return v.is_array() && v.size() == 2 && (v.at(0).is_string() || v.at(0).is_int()) && v.at(1).is_int();
}
inline std::string api_output_port(const Json& graph, long long src, long long slot) {
  const Json* node = graph.find(std::to_string(src));
  if (!node) throw unsupported("Comfy API prompt link references missing node: " + std::to_string(src));
  std::string type = canonical_type(node->str("class_type"));
  if (is_scalar_node(type) && slot == 0) {
    std::string st = scalar_output_type(type, type == "PrimitiveNode" ? node->get("inputs") : Json::object());
    if (!st.empty()) return st;
  }
  auto it = Engine::registry().find(type);
  if (it == Engine::registry().end()) throw unsupported("unsupported Comfy API prompt output node type: " + type, -1, type);
  if (type.rfind("Save", 0) == 0) throw unsupported("Comfy API prompt terminal save node has no supported output slot");
  if (slot < 0 || static_cast<size_t>(slot) >= it->second.slots.size())
    throw unsupported("unsupported Comfy API prompt output node type: " + type, -1, type);
  // the custom samplers expose (output, denoised_output): both are latents of the same geometry
  if ((type == "SamplerCustom" || type == "SamplerCustomAdvanced" || type == "LanPaint_SamplerCustomAdvanced") && slot == 1)
    return "LATENT_DENOISED";
  return it->second.slots[slot];
}
inline Json api_prompt_to_typed(const Json& graph) {
  Json nodes = Json::array(), edges = Json::array();
  for (auto& m : graph.members()) {
    long long id = strtoll(m.first.c_str(), nullptr, 10);
    std::string type = canonical_type(m.second.str("class_type"));
    if (type.empty()) throw unsupported("Comfy API prompt node missing class_type", id);
    Json fields = Json::object();
    for (auto& in : m.second.get("inputs").members()) {
      if (is_link(in.second)) {
        long long src = intish(in.second.at(0), "link source id");
        Json e = Json::object(), from = Json::object(), to = Json::object();
        from.set("node", Json(src));
        from.set("port", Json(api_output_port(graph, src, in.second.at(1).as_int())));
        to.set("node", Json(id));
        to.set("port", Json(type == "Reroute" && in.first.empty() ? std::string("input") : in.first));
        e.set("from", from);
        e.set("to", to);
        edges.push(e);
      } else {
        fields.set(in.first, in.second);
      }
    }
    Json n = Json::object();
    n.set("id", Json(id));
    n.set("type_id", Json(type));
    n.set("fields", fields);
    nodes.push(n);
  }
  Json body = Json::object();
  body.set("nodes", nodes);
  body.set("edges", edges);
  return body;
}

// ComfyUI canvas export: {"nodes": [{id, type, mode, inputs[], outputs[], widgets_values[]}], "links": [[id, src, slot, dst, slot, type]]}
inline std::string canvas_type(const Json& n) { return canonical_type(!n.str("type").empty() ? n.str("type") : n.str("type_id")); }
inline long long canvas_mode(const Json& n) { return n.get("mode").is_number() ? n.get("mode").as_int() : 0; }
inline bool canvas_inactive(const Json& n) { long long m = canvas_mode(n); return m == 2 || m == 4; }
inline bool looks_like_canvas(const Json& wf) {
  if (!wf.get("nodes").is_array() || !wf.get("links").is_array()) return false;
  for (const Json& n : wf.get("nodes").items()) if (canvas_type(n).empty()) return false;
  return true;
}
inline bool looks_like_ideogram4(const Json& wf) {
  if (!wf.get("nodes").is_array() || !wf.get("links").is_array()) return false;
  const Json& sgs = wf.get("definitions").get("subgraphs");
  if (!sgs.is_array()) return false;
  for (const Json& sg : sgs.items()) if (lower(sg.str("name")).find("ideogram") != std::string::npos) return true;
  return false;
}

struct WidgetField { const char* name; int idx; char kind; Json dflt; };   // kind: s i f b
inline const std::map<std::string, std::vector<WidgetField>>& widget_table() {
  static const std::map<std::string, std::vector<WidgetField>> t = [] {
    std::map<std::string, std::vector<WidgetField>> m;
    m["CheckpointLoaderSimple"] = {{"ckpt_name", 0, 's', ""}};
    m["UNETLoader"] = m["DiffusionModelLoader"] = {{"unet_name", 0, 's', ""}};
    m["LoraLoaderModelOnly"] = m["ZImageLoraModelOnly"] = {{"lora_name", 0, 's', ""}, {"strength_model", 1, 'f', 1.0}};
    m["LoraLoader"] = {{"lora_name", 0, 's', ""}, {"strength_model", 1, 'f', 1.0}, {"strength_clip", 2, 'f', 1.0}};
    m["CLIPTextEncode"] = m["CLIPTextEncodeFlux"] = m["TextEncodeQwenImageEdit"] = m["TextEncodeQwenImageEditPlus"] = {{"text", 0, 's', ""}};
    m["LoadImage"] = m["LoadImageOutput"] = m["LoadImageMask"] = {{"image", 0, 's', ""}};
    m["ImageScaleBy"] = {{"scale_by", 1, 'f', 1.0}};
    m["EmptyLatentImage"] = m["EmptySD3LatentImage"] = m["EmptyFlux2LatentImage"] =
        {{"width", 0, 'i', 512}, {"height", 1, 'i', 512}, {"batch_size", 2, 'i', 1}};
    m["KSampler"] = {{"seed", 0, 'i', -1}, {"steps", 2, 'i', 20}, {"cfg", 3, 'f', 4.5}, {"sampler_name", 4, 's', "euler"},
                     {"scheduler", 5, 's', "simple"}, {"denoise", 6, 'f', 1.0}};
    m["KSamplerAdvanced"] = {{"add_noise", 0, 's', "enable"}, {"noise_seed", 1, 'i', -1}, {"seed", 1, 'i', -1}, {"steps", 3, 'i', 20},
                             {"cfg", 4, 'f', 4.5}, {"sampler_name", 5, 's', "euler"}, {"scheduler", 6, 's', "simple"},
                             {"start_at_step", 7, 'i', 0}, {"end_at_step", 8, 'i', 10000},
                             {"return_with_leftover_noise", 9, 's', "disable"}};
    m["LanPaint_KSampler"] = {{"seed", 0, 'i', -1}, {"steps", 2, 'i', 20}, {"cfg", 3, 'f', 4.5}, {"sampler_name", 4, 's', "euler"},
                              {"scheduler", 5, 's', "simple"}, {"denoise", 6, 'f', 1.0}, {"LanPaint_NumSteps", 7, 'i', -1},
                              {"LanPaint_PromptMode", 8, 's', ""}};
    m["ImagePadForOutpaint"] = {{"left", 0, 'i', 0}, {"top", 1, 'i', 0}, {"right", 2, 'i', 0}, {"bottom", 3, 'i', 0}, {"feathering", 4, 'i', 40}};
    m["ThresholdMask"] = {{"value", 0, 'f', 0.5}};
    m["ConditioningSetMask"] = {{"strength", 0, 'f', 1.0}, {"set_cond_area", 1, 's', "default"}};
    m["SetNode"] = m["GetNode"] = {{"name", 0, 's', ""}};
    m["PrimitiveInt"] = m["INTConstant"] = m["easy int"] = m["SeedNode"] = {{"value", 0, 'i', 0}};
    m["PrimitiveFloat"] = m["FloatConstant"] = m["easy float"] = {{"value", 0, 'f', 0.0}};
    m["StringConstant"] = {{"string", 0, 's', ""}};
    m["StringConstantMultiline"] = {{"string", 0, 's', ""}, {"strip_newlines", 1, 'b', true}};
    m["PrimitiveString"] = m["PrimitiveStringMultiline"] = m["easy string"] = {{"value", 0, 's', ""}};
    m["PrimitiveBoolean"] = m["BOOLConstant"] = {{"value", 0, 'b', false}};
    m["InpaintModelConditioning"] = {{"noise_mask", 0, 'b', true}};
    m["VAEEncodeForInpaint"] = {{"grow_mask_by", 0, 'i', 6}};
    m["RepeatLatentBatch"] = {{"amount", 0, 'i', 1}};
    m["SaveImage"] = {{"filename_prefix", 0, 's', ""}};
    m["ImageToMask"] = {{"channel", 0, 's', ""}};
    m["RandomNoise"] = {{"noise_seed", 0, 'i', -1}};
    m["KSamplerSelect"] = {{"sampler_name", 0, 's', "euler"}};
    m["Flux2Scheduler"] = {{"steps", 0, 'i', 20}};
    m["BasicScheduler"] = {{"scheduler", 0, 's', "simple"}, {"steps", 1, 'i', 20}, {"denoise", 2, 'f', 1.0}};
    for (const char* n : {"KarrasScheduler", "ExponentialScheduler", "PolyexponentialScheduler", "VPScheduler",
                          "BetaSamplingScheduler", "LaplaceScheduler"})
      m[n] = {{"steps", 0, 'i', 20}};
    m["SDTurboScheduler"] = {{"steps", 0, 'i', 20}, {"denoise", 1, 'f', 1.0}};
    m["SamplerCustom"] = {{"add_noise", 0, 'b', true}, {"noise_seed", 1, 'i', -1}, {"cfg", 3, 'f', 4.5}};
    m["CFGGuider"] = m["FluxGuidance"] = {{"cfg", 0, 'f', 4.5}};
    m["ModelSamplingAuraFlow"] = m["ModelSamplingSD3"] = {{"shift", 0, 'f', 3.0}};
    m["ComfySwitchNode"] = {{"switch", 0, 'b', false}};
    return m;
  }();
  return t;
}
inline Json widget_value(const Json& w, const WidgetField& f) {
  const Json& v = w.at(f.idx);
  switch (f.kind) {
    case 's': return v.is_string() ? v : f.dflt;
    case 'i':
      if (v.is_int()) return v;
      if (v.is_number()) return Json(static_cast<int64_t>(v.as_double()));
      if (v.is_string()) { char* e = nullptr; long long r = strtoll(v.as_string().c_str(), &e, 10); if (e && !*e && !v.as_string().empty()) return Json(static_cast<int64_t>(r)); }
      return f.dflt;
    case 'f':
      if (v.is_number()) return Json(v.as_double());
      if (v.is_string()) { char* e = nullptr; double r = strtod(v.as_string().c_str(), &e); if (e && !*e && !v.as_string().empty()) return Json(r); }
      return Json(f.dflt.as_double());
    default:
      if (v.is_bool()) return v;
      if (v.is_int()) return Json(v.as_int() != 0);
      if (v.is_string()) { std::string l = lower(v.as_string()); if (l == "true" || l == "enable" || l == "yes") return Json(true); if (l == "false" || l == "disable" || l == "no") return Json(false); }
      return f.dflt;
  }
}
inline const Json* canvas_node(const Json& nodes, long long id, bool active_only) {
  for (const Json& n : nodes.items())
    if (n.is_object() && n.present("id") && intish(n.get("id"), "node id") == id) return active_only && canvas_inactive(n) ? nullptr : &n;
  return nullptr;
}
inline std::string canvas_output_port(const Json& node, long long slot) {
  const Json& outs = node.get("outputs");
  if (!outs.is_array()) throw unsupported("Comfy UI canvas source node missing outputs");
  if (slot < 0 || static_cast<size_t>(slot) >= outs.size()) throw unsupported("Comfy UI canvas source output slot out of range");
  std::string type = outs.at(slot).str("type"), name = outs.at(slot).str("name"), nt = canvas_type(node);
  if (nt == "SetNode") return "SET";
  if (nt == "GetNode") return "GET";
  if (nt == "Reroute") return "REROUTE";
  if (is_scalar_node(nt) && (type == "INT" || type == "FLOAT" || type == "STRING" || type == "BOOLEAN")) return type;
  if (nt == "InpaintModelConditioning") {
    if (name == "positive" || name == "negative") return name;
    if (type == "LATENT" || name == "latent") return "LATENT";
  }
  if ((nt == "SamplerCustom" || nt == "SamplerCustomAdvanced" || nt == "LanPaint_SamplerCustomAdvanced") && slot == 1) return "LATENT_DENOISED";
  if (type == "INT") return name.empty() ? "INT" : name;
  static const std::set<std::string> typed = {"MODEL", "CLIP", "VAE", "CONDITIONING", "IMAGE", "MASK", "LATENT", "GUIDER", "SIGMAS", "NOISE", "SAMPLER"};
  if (typed.count(type)) return type;
  if (!name.empty()) return name;
  throw unsupported("Comfy UI canvas source output missing type/name");
}
inline std::string canvas_input_port(const Json& node, long long slot) {
  const Json& ins = node.get("inputs");
  if (!ins.is_array()) throw unsupported("Comfy UI canvas target node missing inputs");
  if (slot < 0 || static_cast<size_t>(slot) >= ins.size()) throw unsupported("Comfy UI canvas target input slot out of range");
  std::string port = ins.at(slot).str("name"), nt = canvas_type(node);
  if (nt == "SetNode") return "value";
  if (nt == "Reroute" && port.empty()) return "input";
  if (port.empty()) throw unsupported("Comfy UI canvas target input missing name");
  return port;
}
inline Json canvas_to_typed(const Json& wf) {
  Json nodes = Json::array(), edges = Json::array();
  const Json& src = wf.get("nodes");
  for (const Json& n : src.items()) {
    if (!n.is_object()) throw unsupported("Comfy UI canvas node must be an object");
    if (canvas_inactive(n)) continue;
    std::string type = canvas_type(n);
    Json fields = Json::object();
    const Json& w = n.get("widgets_values");
    auto it = widget_table().find(type);
    if (it != widget_table().end()) for (auto& f : it->second) fields.set(f.name, widget_value(w, f));
    if (type == "PrimitiveNode" && w.is_array() && w.size() > 0) fields.set("value", w.at(0));
    if (type == "GetNode" || type == "SetNode" || is_scalar_node(type)) {
      std::string ot = n.get("outputs").at(0).str("type");
      if (!ot.empty()) fields.set("output_type", Json(ot));
    }
    Json o = Json::object();
    o.set("id", Json(intish(n.get("id"), "node id")));
    o.set("type_id", Json(type));
    o.set("fields", fields);
    nodes.push(o);
  }
  for (const Json& l : wf.get("links").items()) {
    if (!l.is_array() || l.size() < 6) continue;
    long long s = intish(l.at(1), "source node id"), ss = intish(l.at(2), "source output slot");
    long long d = intish(l.at(3), "target node id"), ds = intish(l.at(4), "target input slot");
    const Json *sn = canvas_node(src, s, true), *dn = canvas_node(src, d, true);
    if (!sn || !dn) continue;
    Json e = Json::object(), from = Json::object(), to = Json::object();
    from.set("node", Json(s));
    from.set("port", Json(canvas_output_port(*sn, ss)));
    to.set("node", Json(d));
    to.set("port", Json(canvas_input_port(*dn, ds)));
    e.set("from", from);
    e.set("to", to);
    edges.push(e);
  }
  Json body = Json::object();
  body.set("nodes", nodes);
  body.set("edges", edges);
  return body;
}

// ---- bookkeeping written after a successful lowering -------------------------------------------------------------------
inline std::string route_kind(const Json& req) {
  if (!req.str("workflow_route_kind").empty()) return req.str("workflow_route_kind");
  if (req.has("num_frames") || req.has("frame_count") || req.has("frame_rate") || req.has("video")) return "video";
  if (req.has("model") && (req.has("prompt") || req.has("prompt_raw") || req.has("prompt_json")) && (req.has("width") || req.has("height")))
    return "image";
  return "unknown";
}
inline void record_execution(Json& req, const std::string& source, size_t nodes, size_t edges) {
  std::string route = route_kind(req);
  req.set("workflow_schema", Json(kSchema));
  req.set("workflow_executor", Json(kExecutor));
  req.set("workflow_source", Json(source));
  req.set("workflow_node_count", Json(nodes));
  req.set("workflow_edge_count", Json(edges));
  req.set("workflow_route_kind", Json(route));
  Json plan = req.get("workflow_plan").is_object() ? req.get("workflow_plan") : Json::object();
  plan.set("schema", Json("serenity.workflow_plan.v1"));
  plan.set("route_kind", Json(route));
  plan.set("source", Json(source));
  plan.set("node_count", Json(nodes));
  plan.set("edge_count", Json(edges));
  if (!plan.get("terminal_nodes").is_array()) plan.set("terminal_nodes", Json::array());
  req.set("workflow_plan", plan);
}

inline void run_typed(Json& req, const Json& typed_body, const std::string& source) {
  TypedGraph g = parse_typed(typed_body);
  Engine eng(g);
  eng.run(req);
  record_execution(req, source, g.nodes.size(), g.edges.size());
}

// Ideogram-4 canvas export: the sampler lives in a subgraph whose widgets give the settings; the prompt must come from
// the request (the export builds it with a prompt-builder subgraph that is not executed here).
inline void lower_ideogram4(Json& req, const Json& wf) {
  bool has_prompt = false;
  if (req.present("prompt_json")) {
    const Json& pj = req.get("prompt_json");
    if (!pj.is_string() && !pj.is_object() && !pj.is_array())
      throw unsupported("Ideogram4 Comfy export prompt_json must be a string or JSON object/array");
    std::string raw = pj.is_string() ? pj.as_string() : pj.dump();
    if (raw.empty()) throw unsupported("Ideogram4 Comfy export prompt_json must be non-empty");
    req.set("prompt", Json(raw));
    req.set("prompt_raw", Json(raw));
    has_prompt = true;
  } else if (!req.str("prompt").empty()) {
    has_prompt = true;
  } else if (!req.str("prompt_raw").empty()) {
    req.set_if_missing("prompt", Json(req.str("prompt_raw")));
    has_prompt = true;
  }
  if (!has_prompt)
    throw unsupported("Ideogram4 Comfy export uses a prompt-builder subgraph; provide top-level prompt, prompt_raw, or prompt_json");
  if (!wf.get("nodes").is_array()) throw unsupported("Ideogram4 Comfy export missing nodes array");
  static const std::set<std::string> passive_roots = {"MarkdownNote", "SaveImage", "ResolutionSelector", "PreviewAny", "Ideogram4PromptBuilderKJ",
                                                      "83e6e004-48ea-408e-9024-eb49c3d7dc14", "f5f04613-ee09-4cd9-9ada-a880360891d4"};
  for (const Json& n : wf.get("nodes").items()) {
    if (!n.is_object()) throw unsupported("Ideogram4 Comfy export root node must be an object");
    std::string type = !n.str("type").empty() ? n.str("type") : n.str("type_id");
    long long mode = canvas_mode(n);
    if (type == "LoraLoader" || type == "LoraLoaderModelOnly" || type == "ZImageLoraModelOnly") {
      if (mode != 4) throw unsupported("Ideogram4 Comfy export has active LoRA nodes, but the Ideogram4 backend does not execute LoRA");
    } else if (type == "Seed (rgthree)") {
      if (!req.present("seed")) {
        long long seed = widget_value(n.get("widgets_values"), WidgetField{"seed", 0, 'i', -1}).as_int();
        if (seed < 0) throw unsupported("Ideogram4 Comfy export uses randomized seed; provide top-level seed");
        if (seed > 4294967295LL) throw unsupported("Ideogram4 Comfy export seed exceeds the uint32 seed range; provide top-level seed");
        req.set("seed", Json(seed));
      }
    } else if (!passive_roots.count(type) && mode != 4) {
      throw unsupported("unsupported active Ideogram4 Comfy root node: " + type);
    }
  }
  const Json* sg_nodes = nullptr;
  const Json& sgs = wf.get("definitions").get("subgraphs");
  if (sgs.is_array())
    for (const Json& sg : sgs.items()) {
      std::string name = lower(sg.str("name"));
      if (name.find("text to image") != std::string::npos && name.find("ideogram") != std::string::npos) {
        if (!sg.get("nodes").is_array()) throw unsupported("Ideogram4 Comfy export subgraph missing nodes");
        sg_nodes = &sg.get("nodes");
        break;
      }
    }
  if (!sg_nodes) throw unsupported("Ideogram4 Comfy export missing Text to Image (Ideogram v4) subgraph");
  std::set<std::string> seen;
  std::string mode_name = "Default";
  static const std::set<std::string> inert = {"ConditioningZeroOut", "SamplerCustomAdvanced", "VAEDecode", "RandomNoise", "PrimitiveInt",
                                              "ComfyMathExpression", "JsonExtractString", "StringReplace", "ComfyNumberConvert"};
  auto wi = [](const Json& w, int i, long long d) { return widget_value(w, WidgetField{"", i, 'i', Json(static_cast<int64_t>(d))}).as_int(); };
  auto wfl = [](const Json& w, int i, double d) { return widget_value(w, WidgetField{"", i, 'f', Json(d)}).as_double(); };
  auto ws = [](const Json& w, int i, const std::string& d) { return widget_value(w, WidgetField{"", i, 's', Json(d)}).as_string(); };
  for (const Json& n : sg_nodes->items()) {
    if (!n.is_object()) throw unsupported("Ideogram4 Comfy export subgraph node must be an object");
    if (canvas_mode(n) == 4) continue;
    std::string type = !n.str("type").empty() ? n.str("type") : n.str("type_id");
    const Json& w = n.get("widgets_values");
    if (type == "EmptyFlux2LatentImage") {
      req.set_if_missing("width", Json(wi(w, 0, 1024)));
      req.set_if_missing("height", Json(wi(w, 1, 1024)));
      req.set_if_missing("images", Json(wi(w, 2, 1)));
      seen.insert("latent");
    } else if (type == "UNETLoader") {
      std::string name = lower(ws(w, 0, ""));
      if (name.find("ideogram4_unconditional") != std::string::npos) seen.insert("uncond");
      else if (name.find("ideogram4") != std::string::npos) { seen.insert("cond"); req.set_if_missing("model", Json("ideogram-4-fp8")); }
    } else if (type == "CLIPLoader") { if (lower(ws(w, 0, "")).find("qwen3vl") != std::string::npos) seen.insert("clip"); }
    else if (type == "VAELoader") { if (lower(ws(w, 0, "")).find("flux2") != std::string::npos) seen.insert("vae"); }
    else if (type == "CLIPTextEncode") seen.insert("encode");
    else if (type == "KSamplerSelect") { req.set_if_missing("sampler", Json(ws(w, 0, "euler"))); seen.insert("sampler"); }
    else if (type == "BasicScheduler") { req.set_if_missing("scheduler", Json(ws(w, 0, "simple"))); seen.insert("scheduler"); }
    else if (type == "ModelSamplingAuraFlow") { req.set_if_missing("sigma_shift", Json(wfl(w, 0, 5.0))); seen.insert("aura"); }
    else if (type == "DualModelGuider") { req.set_if_missing("cfg", Json(wfl(w, 0, 7.0))); seen.insert("guider"); }
    else if (type == "CFGOverride") {
      req.set_if_missing("cfg_override", Json(wfl(w, 0, 3.0)));
      req.set_if_missing("cfg_override_start_percent", Json(wfl(w, 1, 0.7)));
      req.set_if_missing("cfg_override_end_percent", Json(wfl(w, 2, 1.0)));
      seen.insert("override");
    } else if (type == "CustomCombo") mode_name = ws(w, 0, mode_name);
    else if (!inert.count(type)) throw unsupported("unsupported Ideogram4 Comfy subgraph node: " + type);
  }
  long long steps = mode_name == "Quality" ? 48 : mode_name == "Default" ? 20 : mode_name == "Turbo" ? 12 : -1;
  if (steps < 0) throw unsupported("unsupported Ideogram4 workflow mode: " + mode_name);
  req.set_if_missing("steps", Json(steps));
  if (seen.size() != 11) throw unsupported("Ideogram4 Comfy export is missing required txt2img sampler nodes");
  record_execution(req, "ideogram4_comfy_ui_export", sg_nodes->size(), wf.get("links").is_array() ? wf.get("links").size() : 0);
}

inline const std::vector<std::string>& flat_param_keys() {
  static const std::vector<std::string> k = {
      "model", "prompt", "negative", "width", "height", "steps", "seed", "cfg", "cfg_override", "cfg_override_start_percent",
      "cfg_override_end_percent", "sampler", "scheduler", "sigma_shift", "variation_seed", "variation_strength", "images",
      "init_image", "mask_image", "creativity", "clip_skip", "eta", "sigma_min", "sigma_max", "restart_sampling", "vae",
      "reference_image", "reference_latent_method", "num_frames", "frame_rate"};
  return k;
}
inline void lower_flat(Json& req, const Json& wf, const std::string& key, const std::string& source) {
  const Json& p = wf.get(key);
  auto copy = [&](const std::string& s, const std::string& d) { if (p.present(s)) req.set_if_missing(d, p.get(s)); };
  for (auto& k : flat_param_keys()) copy(k, k);
  copy("filename_prefix", "workflow_save_prefix");
  copy("loras", "lora");
  record_execution(req, source, 0, 0);
}

// Entry point: lowers ``req`` in place. Requests without a workflow pass through untouched unless the body itself is a graph.
inline void lower_request(Json& req) {
  if (!req.is_object()) throw unsupported("request body must be an object");
  auto api = [&](const Json& wf) {
    Json body = api_prompt_body(wf);
    if (!looks_like_api_prompt(body)) throw unsupported("unsupported Comfy API prompt graph");
    if (req.get("prompt").is_object()) req.set("prompt", Json());     // the graph occupied the "prompt" key
    run_typed(req, api_prompt_to_typed(body), "comfy_api_prompt_graph");
  };
  auto canvas = [&](const Json& wf) { run_typed(req, canvas_to_typed(wf), "comfy_ui_canvas_graph"); };
  if (!req.present("workflow")) {
    Json snap = req;
    if (looks_like_ideogram4(snap)) return lower_ideogram4(req, snap);
    if (looks_like_api_prompt(snap)) return api(snap);
    if (looks_like_canvas(snap)) return canvas(snap);
    return;
  }
  Json wf = req.get("workflow");
  if (!wf.is_object()) throw unsupported("workflow graph body must be an object");
  if (looks_like_ideogram4(wf)) return lower_ideogram4(req, wf);
  if (looks_like_api_prompt(wf)) return api(wf);
  if (looks_like_canvas(wf)) return canvas(wf);
  if (wf.get("params").is_object()) return lower_flat(req, wf, "params", "flat_params_adapter");
  if (wf.get("genparams").is_object()) return lower_flat(req, wf, "genparams", "flat_genparams_adapter");
  bool nodes = wf.get("nodes").is_array(), edges = wf.get("edges").is_array();
  if (nodes && edges) return run_typed(req, wf, "typed_linked_graph");
  if (nodes) throw unsupported("workflow graph body needs edges for typed execution");
  throw unsupported("workflow graph body needs nodes or params/genparams");
}

}  // namespace graph
}  // namespace mdb
