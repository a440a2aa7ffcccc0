// The line protocol between the control plane and a worker process. One JSON object per line, '\n' terminated.
//   control plane -> worker:  {"cmd":"start", <job parameters>}   |  {"cmd":"cancel"}
//   worker -> control plane:  {"ev":"ready"} | {"ev":"progress","step":k,"total":n,"phase":"...","preview":"..."}
//                             | {"ev":"done","output_path":"..."} | {"ev":"failed","error":"..."} | {"ev":"cancelled"}
// Field names, types and defaults of the job parameters are a frozen contract shared with every worker
// (serenity-server/crates/wire/src/lib.rs:10-170, serenitymojo/serve/ipc_codec.mojo, serve/backend.mojo).
#pragma once
#include <string>
#include <vector>

#include "json.hpp"

namespace mdb {
namespace wire {

constexpr const char* kCancelLine = "{\"cmd\":\"cancel\"}";

struct ParamDefault { const char* key; Json value; };

// In wire order. -1 / "" mean "not set: the worker uses its own default".
inline const std::vector<ParamDefault>& param_defaults() {
  static const std::vector<ParamDefault> d = {
      {"job_id", ""}, {"model", ""}, {"prompt", ""}, {"negative", ""}, {"width", 512}, {"height", 512}, {"steps", 20},
      {"seed", 0}, {"cfg", 4.5}, {"cfg_override", -1.0}, {"cfg_override_start_percent", 0.0},
      {"cfg_override_end_percent", 1.0}, {"sampler", ""}, {"scheduler", ""}, {"sigma_shift", 3.0}, {"variation_seed", 0},
      {"variation_strength", 0.0}, {"images", 1}, {"image_index", 0}, {"image_count", 1}, {"workflow_save_prefix", ""},
      {"init_image", ""}, {"mask_image", ""}, {"lanpaint_mask_channel", ""}, {"inpaint_conditioning_image", ""},
      {"inpaint_conditioning_mask", ""}, {"inpaint_conditioning_noise_mask", false}, {"qwen_edit_conditioning_image", ""},
      {"sample_caps_pos", ""}, {"sample_caps_neg", ""}, {"conditioning_mask_image", ""}, {"conditioning_mask_channel", ""},
      {"conditioning_mask_strength", -1.0}, {"conditioning_mask_set_area_to_bounds", false}, {"outpaint_left", -1},
      {"outpaint_top", -1}, {"outpaint_right", -1}, {"outpaint_bottom", -1}, {"outpaint_feathering", -1},
      {"threshold_mask_value", -1.0}, {"threshold_mask_operator", ""}, {"lanpaint_mask_blend_overlap", -1},
      {"lanpaint_num_steps", -1}, {"lanpaint_lambda", -1.0}, {"lanpaint_step_size", -1.0}, {"lanpaint_beta", -1.0},
      {"lanpaint_friction", -1.0}, {"lanpaint_prompt_mode", ""}, {"lanpaint_inpainting_mode", ""}, {"lanpaint_add_noise", ""},
      {"lanpaint_noise_seed", -1}, {"lanpaint_start_at_step", -1}, {"lanpaint_end_at_step", -1},
      {"lanpaint_return_with_leftover_noise", ""}, {"lanpaint_early_stop", -1}, {"lanpaint_inner_threshold", -1.0},
      {"lanpaint_inner_patience", -1}, {"reference_image", ""}, {"reference_latent_method", ""},
      {"reference_latent_count", 0}, {"creativity", 0.5}, {"clip_skip", 0}, {"eta", -1.0}, {"sigma_min", -1.0},
      {"sigma_max", -1.0}, {"restart_sampling", false}, {"vae", ""}, {"out_dir", ""}, {"params_json", ""}};
  return d;
}

// Coerces one request value to the kind of its default (int / float / string / bool). Returns false on a kind clash.
inline bool coerce(const Json& dflt, const Json& v, Json* out) {
  switch (dflt.kind()) {
    case Json::Int:
      if (v.is_int()) { *out = v; return true; }
      if (v.is_number() && v.as_double() == static_cast<double>(static_cast<int64_t>(v.as_double()))) { *out = Json(static_cast<int64_t>(v.as_double())); return true; }
      return false;
    case Json::Float:
      if (v.is_number()) { *out = Json(v.as_double()); return true; }
      return false;
    case Json::String:
      if (v.is_string()) { *out = v; return true; }
      return false;
    case Json::Bool:
      if (v.is_bool()) { *out = v; return true; }
      return false;
    default:
      return false;
  }
}

// Builds the full parameter object (every key present, wire order) from a flat request. ``err`` names the first field of
// the wrong kind.
inline bool params_from_request(const Json& req, Json* params, std::string* err) {
  Json p = Json::object();
  for (auto& d : param_defaults()) {
    Json v = d.value;
    if (req.present(d.key) && !coerce(d.value, req.get(d.key), &v)) {
      if (err) *err = std::string("invalid request body: field '") + d.key + "' has the wrong type";
      return false;
    }
    p.set(d.key, v);
  }
  Json loras = Json::array();
  const Json& l = req.present("lora") ? req.get("lora") : req.get("loras");
  if (l.is_array())
    for (const Json& e : l.items()) {
      if (!e.is_object() || !e.get("name").is_string()) { if (err) *err = "invalid request body: lora entries need a name"; return false; }
      Json o = Json::object();
      o.set("name", e.get("name"));
      o.set("weight", Json(e.present("weight") ? e.get("weight").as_double(1.0) : 1.0));
      loras.push(o);
    }
  p.set("lora", loras);
  *params = p;
  return true;
}

inline std::string start_line(const Json& params) {
  Json line = Json::object();
  line.set("cmd", Json("start"));
  for (auto& m : params.members()) line.set(m.first, m.second);
  return line.dump();
}

struct Event {
  enum Kind { Ready, Progress, Done, Failed, Cancelled, Unknown } kind = Unknown;
  long long step = 0, total = 0;
  std::string phase, preview, output_path, error;
  bool terminal() const { return kind == Done || kind == Failed || kind == Cancelled; }
  Json to_json() const {
    Json j = Json::object();
    switch (kind) {
      case Ready: j.set("ev", Json("ready")); break;
      case Progress:
        j.set("ev", Json("progress")); j.set("step", Json(step)); j.set("total", Json(total));
        j.set("phase", Json(phase)); j.set("preview", Json(preview));
        break;
      case Done: j.set("ev", Json("done")); j.set("output_path", Json(output_path)); break;
      case Failed: j.set("ev", Json("failed")); j.set("error", Json(error)); break;
      case Cancelled: j.set("ev", Json("cancelled")); break;
      default: j.set("ev", Json("unknown"));
    }
    return j;
  }
};

inline bool parse_event(const std::string& line, Event* ev, std::string* err = nullptr) {
  Json j;
  if (!Json::try_parse(line, &j, err) || !j.is_object()) { if (err && err->empty()) *err = "event is not an object"; return false; }
  std::string k = j.str("ev");
  Event e;
  if (k == "ready") e.kind = Event::Ready;
  else if (k == "progress") {
    e.kind = Event::Progress;
    if (!j.get("step").is_int() || !j.get("total").is_int()) { if (err) *err = "progress needs integer step and total"; return false; }
    e.step = j.get("step").as_int(); e.total = j.get("total").as_int();
    e.phase = j.str("phase"); e.preview = j.str("preview");
  } else if (k == "done") {
    e.kind = Event::Done;
    if (!j.get("output_path").is_string()) { if (err) *err = "done needs output_path"; return false; }
    e.output_path = j.str("output_path");
  } else if (k == "failed") {
    e.kind = Event::Failed;
    if (!j.get("error").is_string()) { if (err) *err = "failed needs error"; return false; }
    e.error = j.str("error");
  } else if (k == "cancelled") e.kind = Event::Cancelled;
  else { if (err) *err = "unknown event '" + k + "'"; return false; }
  *ev = e;
  return true;
}

}  // namespace wire
}  // namespace mdb
