"""Worker process: ``python -m mojodiffusion_b200.serve.worker --kind KIND <fd>``.

``<fd>`` is the inherited end of an AF_UNIX stream socket pair. The loop: announce ``{"ev":"ready"}`` once the backend
is constructed, then alternate between reading control lines (non-blocking) and calling ``backend.step()`` while a job
is active. One job at a time; a ``start`` while busy is answered with ``failed``. A closed socket ends the process (the
control plane is gone or is replacing this worker) (serenitymojo/serve/worker.mojo, serve/proc_ipc.mojo,
serve/ipc_codec.mojo)."""
from __future__ import annotations

import argparse
import json
import select
import socket
import sys
import traceback
from typing import Optional

from .backend import GenBackend, JobParams, StepResult


def make_backend(kind: str) -> GenBackend:
    if kind == "stub":
        from .stub_backend import StubBackend
        return StubBackend()
    if kind == "flux":
        from .flux_backend import FluxBackend
        return FluxBackend(kind)
    from .generic_backend import GenericBackend
    return GenericBackend(kind)


class LineSocket:
    def __init__(self, fd: int):
        self.sock = socket.socket(fileno=fd)
        self.sock.setblocking(False)
        self.buf = b""
        self.open = True

    def send(self, obj) -> None:
        data = (json.dumps(obj, separators=(",", ":")) + "\n").encode()
        self.sock.setblocking(True)
        try:
            self.sock.sendall(data)
        except OSError:
            self.open = False
        finally:
            self.sock.setblocking(False)

    def poll_line(self, timeout: float) -> Optional[str]:
        if b"\n" not in self.buf and self.open:
            r, _, _ = select.select([self.sock], [], [], timeout)
            if r:
                try:
                    chunk = self.sock.recv(65536)
                except BlockingIOError:
                    chunk = None
                except OSError:
                    chunk = b""
                if chunk == b"":
                    self.open = False
                elif chunk:
                    self.buf += chunk
        if b"\n" in self.buf:
            line, self.buf = self.buf.split(b"\n", 1)
            return line.decode("utf-8", "replace")
        return None


def run(backend: GenBackend, link: LineSocket) -> int:
    link.send({"ev": "ready"})
    active = False
    while link.open:
        line = link.poll_line(0.0 if active else 0.5)
        if line is not None and line.strip():
            try:
                msg = json.loads(line)
            except json.JSONDecodeError:
                msg = {}                                   # a half-written or garbled line is ignored
            cmd = msg.get("cmd")
            if cmd == "start":
                if active:
                    link.send({"ev": "failed", "error": "worker busy"})
                else:
                    try:
                        backend.start(JobParams.from_wire(msg))
                        active = True
                    except Exception as e:  # noqa: BLE001 - admission errors go back as a failed job
                        link.send({"ev": "failed", "error": f"{type(e).__name__}: {e}"})
            elif cmd == "cancel":
                if active:
                    backend.cancel()
            elif cmd == "trim":
                backend.trim()
            continue
        if active:
            try:
                res = backend.step()
            except Exception as e:  # noqa: BLE001
                traceback.print_exc(file=sys.stderr)
                res = StepResult("failed", error=f"{type(e).__name__}: {e}")
            if res.kind == "silent":
                continue
            link.send(res.event())
            if res.terminal:
                active = False
                backend.trim()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kind", default="stub")
    ap.add_argument("fd", type=int)
    a = ap.parse_args(argv)
    link = LineSocket(a.fd)
    try:
        backend = make_backend(a.kind)
    except Exception as e:  # noqa: BLE001
        link.send({"ev": "failed", "error": f"backend '{a.kind}' unavailable: {e}"})
        return 3
    return run(backend, link)


if __name__ == "__main__":
    sys.exit(main())
