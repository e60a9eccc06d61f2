"""HTTP surfaces (reference: crates/apiserve/src/lib.rs:66-108 — one listener per dialect, bound to
localhost only, authentication before routing so every path including unknown ones answers 401
without a key, 8 MiB body cap -> 413, edge load-shed at 256 concurrent -> 503 + Retry-After;
crates/apiserve/src/surface.rs:60-113 key printing)."""
from __future__ import annotations

import asyncio
import json
import threading
from typing import Dict, Optional

from aiohttp import web

from . import auth
from .anthropic import AnthropicSurface
from .errors import ApiError, from_exception
from .executor import Busy, Executor
from .openai import OpenAiSurface

MAX_BODY = 8 << 20
SURFACE_KEY = web.AppKey("surface", object)
DEFAULT_PORTS = {"anthropic": 8787, "openai": 8788, "openrouter": 8789}


def make_app(provider: str, ex: Executor, key: str) -> web.Application:
    dialect = "anthropic" if provider == "anthropic" else "openai"
    scheme = "x-api-key" if provider == "anthropic" else "bearer"

    def error_response(err: ApiError):
        return web.json_response(err.body(dialect), status=err.status, headers=err.headers())

    @web.middleware
    async def guard(request: web.Request, handler):
        if not auth.check(request.headers, scheme, key):
            return error_response(ApiError("invalid_api_key", "Incorrect API key provided."))
        if request.content_length is not None and request.content_length > MAX_BODY:
            return error_response(ApiError("payload_too_large", "Request body exceeds the 8 MiB limit."))
        try:
            ex.edge_enter()
        except Busy as b:
            return error_response(from_exception(b))
        try:
            return await handler(request)
        except ApiError as e:
            return error_response(e)
        except web.HTTPRequestEntityTooLarge:
            return error_response(ApiError("payload_too_large", "Request body exceeds the 8 MiB limit."))
        except web.HTTPNotFound:
            return error_response(ApiError("not_found", f"Unknown route {request.method} {request.path}"))
        except web.HTTPMethodNotAllowed:
            return error_response(ApiError("not_found", f"Unknown route {request.method} {request.path}"))
        except web.HTTPException:
            raise
        except asyncio.CancelledError:
            raise
        except Exception as e:  # noqa: BLE001 - never leak internals
            return error_response(from_exception(e))
        finally:
            ex.edge_leave()

    app = web.Application(middlewares=[guard], client_max_size=MAX_BODY)
    if provider == "anthropic":
        surface = AnthropicSurface(ex)
    else:
        surface = OpenAiSurface(ex, native=(provider == "openrouter"))
    surface.routes(app)
    app[SURFACE_KEY] = surface

    async def stats(_req):
        from ..utils.stats import snapshot
        snap = snapshot(ex, {provider: surface})
        snap.update({"accounting": surface.acct.snapshot(), "in_flight": ex.in_flight()})
        return web.json_response(snap)
    app.router.add_get("/stats", stats)
    return app


class Server:
    """All requested surfaces on one asyncio loop (optionally in a background thread)."""

    def __init__(self, ex: Executor, ports: Dict[str, int], keys: Optional[Dict[str, str]] = None,
                 host: str = "127.0.0.1"):
        self.ex = ex
        self.ports = dict(ports)
        self.keys = dict(keys or {})
        for p in self.ports:
            self.keys.setdefault(p, auth.new_key())
        self.host = host
        self.bound: Dict[str, int] = {}
        self._runners = []
        self._loop: Optional[asyncio.AbstractEventLoop] = None
        self._thread: Optional[threading.Thread] = None
        self._ready = threading.Event()
        self._stop: Optional[asyncio.Event] = None

    async def start(self):
        for provider, port in self.ports.items():
            runner = web.AppRunner(make_app(provider, self.ex, self.keys[provider]), access_log=None)
            await runner.setup()
            site = web.TCPSite(runner, self.host, port)
            await site.start()
            self.bound[provider] = site._server.sockets[0].getsockname()[1]
            self._runners.append(runner)

    async def stop(self):
        for r in self._runners:
            await r.cleanup()
        self._runners.clear()

    async def _main(self):
        self._stop = asyncio.Event()
        await self.start()
        self._ready.set()
        await self._stop.wait()
        await self.stop()

    def start_background(self) -> "Server":
        def run():
            self._loop = asyncio.new_event_loop()
            asyncio.set_event_loop(self._loop)
            self._loop.run_until_complete(self._main())
        self._thread = threading.Thread(target=run, name="http", daemon=True)
        self._thread.start()
        if not self._ready.wait(30):
            raise RuntimeError("HTTP server did not start")
        return self

    def shutdown(self):
        if self._loop is not None and self._stop is not None:
            self._loop.call_soon_threadsafe(self._stop.set)
            self._thread.join(timeout=10)

    def announce(self, out=print):
        for provider, key in self.keys.items():
            out(f"APIKEY {provider} {key}")
        for provider, port in self.bound.items():
            out(f"LISTEN {provider} http://{self.host}:{port}")
