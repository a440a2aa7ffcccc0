"""Training dashboard log: one SQLite database (``<dir>/board.db``) plus a blob folder (``<dir>/blobs``) that a
viewer can tail while the run is live. Tables: metadata, sessions, scalars, tensors, artifacts, text_events,
trace_events, eval_results, hparam_metrics, plugin_data, custom_scalar_layouts, pr_curves, audio, graphs, embeddings,
meshes; every write is INSERT OR REPLACE keyed by (tag, step[, index]) so a resumed run overwrites rather than
duplicates (serenitymojo/training/serenityboard.mojo:93-126 schema, :186-300 writer surface; scalar tags loss/train,
grad_norm, lr/default, perf/steps_per_sec, perf/sec_per_step)."""
from __future__ import annotations

import json
import os
import shutil
import sqlite3
import struct
import time
from typing import Optional

SCHEMA = """
PRAGMA journal_mode = WAL;
PRAGMA synchronous = NORMAL;
PRAGMA busy_timeout = 5000;
CREATE TABLE IF NOT EXISTS metadata (key TEXT PRIMARY KEY, value TEXT NOT NULL);
CREATE TABLE IF NOT EXISTS sessions (session_id TEXT NOT NULL, start_time REAL NOT NULL, resume_step INTEGER,
  status TEXT NOT NULL CHECK(status IN ('running','complete','crashed')), PRIMARY KEY (session_id)) WITHOUT ROWID;
CREATE TABLE IF NOT EXISTS scalars (tag TEXT NOT NULL, step INTEGER NOT NULL, wall_time REAL NOT NULL,
  value REAL NOT NULL, PRIMARY KEY (tag, step)) WITHOUT ROWID;
CREATE TABLE IF NOT EXISTS tensors (tag TEXT NOT NULL, step INTEGER NOT NULL, wall_time REAL NOT NULL,
  dtype TEXT NOT NULL, shape TEXT NOT NULL, data BLOB NOT NULL, PRIMARY KEY (tag, step)) WITHOUT ROWID;
CREATE TABLE IF NOT EXISTS artifacts (tag TEXT NOT NULL, step INTEGER NOT NULL, seq_index INTEGER NOT NULL DEFAULT 0,
  wall_time REAL NOT NULL, kind TEXT NOT NULL, mime_type TEXT NOT NULL, blob_key TEXT NOT NULL, width INTEGER,
  height INTEGER, meta TEXT NOT NULL DEFAULT '{}', PRIMARY KEY (tag, step, seq_index)) WITHOUT ROWID;
CREATE TABLE IF NOT EXISTS text_events (tag TEXT NOT NULL, step INTEGER NOT NULL, wall_time REAL NOT NULL,
  value TEXT NOT NULL, PRIMARY KEY (tag, step)) WITHOUT ROWID;
CREATE TABLE IF NOT EXISTS trace_events (step INTEGER NOT NULL, wall_time REAL NOT NULL, phase TEXT NOT NULL,
  duration_ms REAL NOT NULL, details TEXT NOT NULL DEFAULT '{}', PRIMARY KEY (step, phase)) WITHOUT ROWID;
CREATE TABLE IF NOT EXISTS eval_results (suite_name TEXT NOT NULL, case_id TEXT NOT NULL, step INTEGER NOT NULL,
  wall_time REAL NOT NULL, score_name TEXT NOT NULL, score_value REAL NOT NULL, artifact_key TEXT,
  details TEXT NOT NULL DEFAULT '{}', PRIMARY KEY (suite_name, case_id, step, score_name)) WITHOUT ROWID;
CREATE TABLE IF NOT EXISTS hparam_metrics (metric_tag TEXT NOT NULL, value REAL NOT NULL, step INTEGER, wall_time REAL,
  PRIMARY KEY (metric_tag)) WITHOUT ROWID;
CREATE TABLE IF NOT EXISTS plugin_data (plugin_name TEXT NOT NULL, tag TEXT NOT NULL, step INTEGER NOT NULL,
  wall_time REAL NOT NULL, data TEXT NOT NULL, PRIMARY KEY (plugin_name, tag, step)) WITHOUT ROWID;
CREATE TABLE IF NOT EXISTS custom_scalar_layouts (layout_name TEXT NOT NULL, config TEXT NOT NULL,
  PRIMARY KEY (layout_name)) WITHOUT ROWID;
CREATE TABLE IF NOT EXISTS pr_curves (tag TEXT NOT NULL, step INTEGER NOT NULL, class_index INTEGER NOT NULL DEFAULT 0,
  wall_time REAL NOT NULL, num_thresholds INTEGER NOT NULL, data BLOB NOT NULL,
  PRIMARY KEY (tag, step, class_index)) WITHOUT ROWID;
CREATE TABLE IF NOT EXISTS audio (tag TEXT NOT NULL, step INTEGER NOT NULL, seq_index INTEGER NOT NULL DEFAULT 0,
  wall_time REAL NOT NULL, blob_key TEXT NOT NULL, sample_rate INTEGER NOT NULL, num_channels INTEGER NOT NULL DEFAULT 1,
  duration_ms REAL, mime_type TEXT NOT NULL DEFAULT 'audio/wav', label TEXT NOT NULL DEFAULT '',
  PRIMARY KEY (tag, step, seq_index)) WITHOUT ROWID;
CREATE TABLE IF NOT EXISTS graphs (tag TEXT NOT NULL, step INTEGER NOT NULL, wall_time REAL NOT NULL,
  graph_blob_key TEXT NOT NULL, PRIMARY KEY (tag, step)) WITHOUT ROWID;
CREATE TABLE IF NOT EXISTS embeddings (tag TEXT NOT NULL, step INTEGER NOT NULL, wall_time REAL NOT NULL,
  num_points INTEGER NOT NULL, dimensions INTEGER NOT NULL, tensor_blob_key TEXT NOT NULL, metadata_json TEXT,
  metadata_header TEXT, sprite_blob_key TEXT, sprite_single_h INTEGER, sprite_single_w INTEGER,
  PRIMARY KEY (tag, step)) WITHOUT ROWID;
CREATE TABLE IF NOT EXISTS meshes (tag TEXT NOT NULL, step INTEGER NOT NULL, wall_time REAL NOT NULL,
  num_vertices INTEGER NOT NULL, has_faces INTEGER NOT NULL DEFAULT 0, has_colors INTEGER NOT NULL DEFAULT 0,
  num_faces INTEGER NOT NULL DEFAULT 0, vertices_blob_key TEXT NOT NULL, faces_blob_key TEXT, colors_blob_key TEXT,
  config_json TEXT, PRIMARY KEY (tag, step)) WITHOUT ROWID;
CREATE INDEX IF NOT EXISTS idx_scalars_tag ON scalars(tag);
CREATE INDEX IF NOT EXISTS idx_scalars_tag_step ON scalars(tag, step DESC);
CREATE INDEX IF NOT EXISTS idx_tensors_tag_step ON tensors(tag, step DESC);
CREATE INDEX IF NOT EXISTS idx_artifacts_tag_step ON artifacts(tag, step DESC);
CREATE INDEX IF NOT EXISTS idx_text_tag_step ON text_events(tag, step DESC);
CREATE INDEX IF NOT EXISTS idx_eval_suite_step ON eval_results(suite_name, step DESC);
CREATE INDEX IF NOT EXISTS idx_plugin_name_tag ON plugin_data(plugin_name, tag);
CREATE INDEX IF NOT EXISTS idx_pr_curves_tag_step ON pr_curves(tag, step DESC);
CREATE INDEX IF NOT EXISTS idx_audio_tag_step ON audio(tag, step DESC);
CREATE INDEX IF NOT EXISTS idx_graphs_tag_step ON graphs(tag, step DESC);
CREATE INDEX IF NOT EXISTS idx_embeddings_tag_step ON embeddings(tag, step DESC);
CREATE INDEX IF NOT EXISTS idx_meshes_tag_step ON meshes(tag, step DESC);
"""


def _png_dims(path: str):
    try:
        with open(path, "rb") as f:
            head = f.read(24)
        if head[:8] == b"\x89PNG\r\n\x1a\n":
            return struct.unpack(">II", head[16:24])
    except OSError:
        pass
    return None, None


class BoardWriter:
    def __init__(self, output_dir: str, session_id: str, resume_step: int = 0, name: str = "train", commit_every: int = 16):
        self.dir = output_dir
        os.makedirs(os.path.join(output_dir, "blobs"), exist_ok=True)
        self.db = sqlite3.connect(os.path.join(output_dir, "board.db"))
        self.db.executescript(SCHEMA)
        self.session_id = session_id
        self.commit_every, self._pending = commit_every, 0
        self.db.execute("INSERT OR REPLACE INTO sessions (session_id, start_time, resume_step, status) VALUES (?,?,?,?)",
                        (session_id, time.time(), resume_step, "running"))
        self._meta("active_session_id", session_id)
        self._meta("name", name)
        self._meta("status", "running")
        self.db.commit()

    def _meta(self, key: str, value) -> None:
        self.db.execute("INSERT OR REPLACE INTO metadata (key, value) VALUES (?,?)", (key, json.dumps(value)))

    def _tick(self) -> None:
        self._pending += 1
        if self._pending >= self.commit_every:
            self.db.commit()
            self._pending = 0

    def set_status(self, status: str) -> None:
        self.db.execute("UPDATE sessions SET status=? WHERE session_id=?", (status, self.session_id))
        self._meta("status", status)
        self.db.commit()

    def log_scalar(self, tag: str, step: int, value: float) -> None:
        self.db.execute("INSERT OR REPLACE INTO scalars (tag, step, wall_time, value) VALUES (?,?,?,?)",
                        (tag, step, time.time(), float(value)))
        self._tick()

    def log_train_step(self, step: int, loss: float, grad_norm: float, lr: float, step_secs: float) -> None:
        self.log_scalar("loss/train", step, loss)
        self.log_scalar("grad_norm", step, grad_norm)
        self.log_scalar("lr/default", step, lr)
        if step_secs > 0:
            self.log_scalar("perf/steps_per_sec", step, 1.0 / step_secs)
            self.log_scalar("perf/sec_per_step", step, step_secs)

    def log_text(self, tag: str, step: int, value: str) -> None:
        self.db.execute("INSERT OR REPLACE INTO text_events (tag, step, wall_time, value) VALUES (?,?,?,?)",
                        (tag, step, time.time(), value))
        self._tick()

    def log_trace(self, step: int, phase: str, duration_ms: float, details: Optional[dict] = None) -> None:
        self.db.execute("INSERT OR REPLACE INTO trace_events (step, wall_time, phase, duration_ms, details) VALUES (?,?,?,?,?)",
                        (step, time.time(), phase, duration_ms, json.dumps(details or {})))
        self._tick()

    def log_hparams(self, hparams: dict) -> None:
        self._meta("hparams", hparams)
        self.db.commit()

    def log_tensor(self, tag: str, step: int, tensor) -> None:
        t = tensor.detach().float().cpu().contiguous()
        self.db.execute("INSERT OR REPLACE INTO tensors (tag, step, wall_time, dtype, shape, data) VALUES (?,?,?,?,?,?)",
                        (tag, step, time.time(), "float32", json.dumps(list(t.shape)), t.numpy().tobytes()))
        self._tick()

    def log_image_png(self, tag: str, step: int, seq_index: int, png_path: str) -> str:
        blob_key = f"{tag.replace('/', '_')}_{step}_{seq_index}.png"
        shutil.copyfile(png_path, os.path.join(self.dir, "blobs", blob_key))
        w, h = _png_dims(png_path)
        self.db.execute("INSERT OR REPLACE INTO artifacts (tag, step, seq_index, wall_time, kind, mime_type, blob_key, "
                        "width, height, meta) VALUES (?,?,?,?,?,?,?,?,?,?)",
                        (tag, step, seq_index, time.time(), "image", "image/png", blob_key, w, h, "{}"))
        self.db.commit()
        return blob_key

    def log_eval(self, suite: str, case_id: str, step: int, score_name: str, score: float, details: Optional[dict] = None):
        self.db.execute("INSERT OR REPLACE INTO eval_results (suite_name, case_id, step, wall_time, score_name, "
                        "score_value, artifact_key, details) VALUES (?,?,?,?,?,?,?,?)",
                        (suite, case_id, step, time.time(), score_name, float(score), None, json.dumps(details or {})))
        self._tick()

    def close(self, status: str = "complete") -> None:
        self.set_status(status)
        self.db.close()
