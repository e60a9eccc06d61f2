"""JSONL stdio server: ``brain serve --stdio`` (reference: crates/cli/src/run_cli.rs stdio loop and
crates/events/src/lib.rs).  Requests run concurrently on the executor; every reply echoes the
request's ``req_id`` so the client can demultiplex; ``cancel`` with a ``req_id`` aborts that job."""
from __future__ import annotations

import sys
import threading
from typing import Dict, Optional, TextIO

from . import events
from .capability import ActionError, Blob, CancelToken, Invocation, Progress, ValidationError
from .errors import from_exception
from .executor import Busy, Executor


class StdioServer:
    def __init__(self, ex: Executor, inp: Optional[TextIO] = None, out: Optional[TextIO] = None,
                 default_model: Optional[str] = None, defaults: Optional[Dict] = None):
        self.ex = ex
        self.inp = inp or sys.stdin
        self.out = out or sys.stdout
        self.lock = threading.Lock()
        self.jobs: Dict[str, CancelToken] = {}
        self.default_model = default_model
        self.defaults = defaults or {}
        self._threads = []

    def send(self, event: str, req_id=None, **fields):
        line = events.encode(event, req_id, **fields)
        with self.lock:
            self.out.write(line + "\n")
            self.out.flush()

    def _chat_model(self) -> Optional[str]:
        if self.default_model:
            return self.default_model
        for mid, m in self.ex.models().items():
            if m.manifest().is_chat():
                return mid
        return None

    def _run_action(self, req_id, model, action, params, blobs, as_chat=False):
        tok = CancelToken()
        if req_id is not None:
            self.jobs[req_id] = tok
        seq = [0]

        def progress(p: Progress):
            if p.kind == "token":
                if as_chat:
                    self.send("brain_text_chunk", req_id, text=p.text, seq=seq[0], done=False)
                    seq[0] += 1
                else:
                    self.send("action_progress", req_id, step=p.step, total=p.total, message=p.text)
            else:
                self.send("action_progress", req_id, step=p.step, total=p.total,
                          message=dict(p.data, kind=p.kind, text=p.text))
        try:
            out = self.ex.run(model, action, Invocation(params, blobs, tok), progress)
            if as_chat:
                self.send("brain_text_chunk", req_id, text="", seq=seq[0], done=True)
            self.send("action_result", req_id, outputs=out.outputs,
                      blobs=[b.to_json(n) for n, b in out.blobs.items()])
        except ActionError as e:
            if e.kind == "cancelled":
                self.send("cancelled", req_id)
            else:
                self.send("error", req_id, message=str(e))
        except (ValidationError, Busy) as e:
            self.send("error", req_id, message=str(e))
        except KeyError as e:
            self.send("error", req_id, message=f"unknown model {e.args[0]!r}")
        except Exception as e:  # noqa: BLE001 - internal detail stays in the log stream
            self.send("log", req_id, message=f"action failed: {type(e).__name__}")
            self.send("error", req_id, message=from_exception(e).message)
        finally:
            if req_id is not None:
                self.jobs.pop(req_id, None)

    def handle(self, ev: Dict):
        kind, rid = ev["event"], ev.get("req_id")
        if kind == "manifest_request":
            self.send("manifest_result", rid, manifests=[m.manifest().to_json() for m in self.ex.models().values()])
        elif kind == "action_request":
            blobs = {b["name"]: Blob.from_json(b) for b in ev.get("blobs") or []}
            t = threading.Thread(target=self._run_action, daemon=True,
                                 args=(rid, ev.get("model"), ev.get("action"), dict(ev.get("params") or {}), blobs))
            t.start()
            self._threads.append(t)
        elif kind == "user_text":
            model = self._chat_model()
            if model is None:
                self.send("error", rid, message="no chat model is being served")
                return
            params = dict(self.defaults, prompt=ev.get("text", ""))
            t = threading.Thread(target=self._run_action, daemon=True, args=(rid, model, "generate", params, {}, True))
            t.start()
            self._threads.append(t)
        elif kind == "cancel":
            targets = [rid] if rid is not None else list(self.jobs)
            hit = False
            for r in targets:
                tok = self.jobs.get(r)
                if tok is not None:
                    tok.cancel()
                    hit = True
            if not hit:
                self.send("error", rid, message="nothing to cancel")
        else:
            self.send("error", rid, message=f"unknown event '{kind}'")

    def serve(self):
        self.send("ready", models=list(self.ex.models()))
        for line in self.inp:
            line = line.strip()
            if not line:
                continue
            try:
                ev = events.decode(line)
            except ValueError as e:
                self.send("error", message=f"bad request line: {e}")
                continue
            self.handle(ev)
        for t in self._threads:
            t.join(timeout=30)


# ------------------------------------------------------------------------------------ socket transports
class SocketServer:
    """The same JSONL protocol over a Unix domain socket or a loopback TCP port, one session per
    connection (reference: crates/server/src/transport.rs:104-127 ``serve_unix`` / ``serve_tcp``; a
    stale socket file is removed first).  ``start()`` returns once the listener is bound; ``close()``
    stops accepting and closes the listener."""

    def __init__(self, ex: Executor, unix_path: Optional[str] = None, tcp_port: Optional[int] = None,
                 defaults: Optional[Dict] = None, max_connections: int = 64):
        import socket
        if (unix_path is None) == (tcp_port is None):
            raise ValueError("give exactly one of unix_path / tcp_port")
        self.ex, self.defaults = ex, defaults
        self.unix_path = unix_path
        if unix_path is not None:
            import os
            try:
                os.unlink(unix_path)
            except FileNotFoundError:
                pass
            self.sock = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            self.sock.bind(unix_path)
            os.chmod(unix_path, 0o600)          # the socket carries no authentication of its own
        else:
            self.sock = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
            self.sock.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            self.sock.bind(("127.0.0.1", int(tcp_port)))      # loopback only, like the HTTP surfaces
        self.port = self.sock.getsockname()[1] if unix_path is None else None
        self.sock.listen(max_connections)
        self._slots = threading.BoundedSemaphore(max_connections)
        self._closed = False
        self._thread: Optional[threading.Thread] = None

    def _session(self, conn):
        try:
            with conn, conn.makefile("r", encoding="utf-8", newline="\n") as rd, \
                    conn.makefile("w", encoding="utf-8", newline="\n") as wr:
                StdioServer(self.ex, rd, wr, defaults=self.defaults).serve()
        except (OSError, ValueError):
            pass                                 # the peer went away mid-line
        finally:
            self._slots.release()

    def _accept_loop(self):
        while not self._closed:
            try:
                conn, _ = self.sock.accept()
            except OSError:
                return
            if not self._slots.acquire(blocking=False):
                conn.close()                     # at the connection limit: refuse rather than queue
                continue
            threading.Thread(target=self._session, args=(conn,), daemon=True).start()

    def start(self) -> "SocketServer":
        self._thread = threading.Thread(target=self._accept_loop, name="jsonl-accept", daemon=True)
        self._thread.start()
        return self

    def close(self):
        self._closed = True
        try:
            self.sock.close()
        finally:
            if self.unix_path is not None:
                import os
                try:
                    os.unlink(self.unix_path)
                except FileNotFoundError:
                    pass
