"""Serving: a C++ control plane (``control_plane/``: HTTP/WebSocket, job book, worker lifecycle, workflow-graph lowering)
drives one Python worker process per resident model kind over an AF_UNIX line-JSON socket."""
