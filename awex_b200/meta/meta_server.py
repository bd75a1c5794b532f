"""Job-global control plane: a small HTTP key/value store used for discovery,
metadata exchange, sets-as-barriers and completion events.

REST surface and wire format are the reference's
(`awex/meta/meta_server.py:61-74`, `awex/util/common.py:93-108`):

==========================  ======  ==============================================
``/v1/get_binary/{key}``    GET     raw bytes; non-bytes values (sets) come back as
                                    length-prefixed pickles; 404 when absent
``/v1/put_binary/{key}``    PUT     store the request body
``/v1/add_object_to_set``   PUT     body is a length-prefixed pickle, added to a set
``/v1/get_json|put_json``   GET/PUT JSON documents
``/v1/delete/{key}``        DELETE  404 when absent
``/v1/has_key/{key}``       GET     ``{"has_key": bool}``
``/v1/keys``, ``/v1/health``GET
``/v1/allocate_auto_grow_id`` POST  monotonically increasing integer
==========================  ======  ==============================================

Keys may contain ``/``.  Objects are pickled, so the server must only be
reachable by the job's own processes.

The server owns an asyncio loop in a daemon thread (``AppRunner``/``TCPSite``),
so port 0 resolves to the socket's real port without a bind/close race.
"""

from __future__ import annotations

import asyncio
import json
import multiprocessing
import os
import pickle
import random
import signal
import threading
import time
import traceback
from typing import Any, Dict, List, Optional, Tuple, Union

import requests
from aiohttp import web

from awex_b200 import logging
from awex_b200.utils.common import from_binary, get_free_port, get_ip_address, to_binary

logger = logging.getLogger(__name__)

MAX_BODY_BYTES = 2 * 1024**3
TOKEN_HEADER = "X-Awex-Token"


def _ok(**fields) -> web.Response:
    return web.json_response({"success": True, **fields})


def _fail(status: int, error: str) -> web.Response:
    return web.json_response({"success": False, "error": error}, status=status)


MAX_SERVER_WAIT_S = 20.0  # longest a single wait_counters request sleeps inside the server; clients re-issue


class MetaServer:
    def __init__(self, host: str = "localhost", port: int = 8080):
        self.host = host
        self.port = port
        self.storage: Dict[str, Any] = {}
        # named counters with server-side waiting (`put_counter` / `wait_counters`): each holds a list of
        # integers whose first element only grows in normal use; a waiter sleeps on the condition instead of polling
        self.counters: Dict[str, List[int]] = {}
        self._counter_cond: Optional[asyncio.Condition] = None
        self.id_counter = 0
        self._loop: Optional[asyncio.AbstractEventLoop] = None
        self._thread: Optional[threading.Thread] = None
        self._runner: Optional[web.AppRunner] = None
        self._ready = threading.Event()
        self._error: Optional[BaseException] = None
        self.app = web.Application(middlewares=[self._guard], client_max_size=MAX_BODY_BYTES)
        r = self.app.router
        r.add_get("/v1/get_binary/{key:.*}", self._h_get_binary)
        r.add_put("/v1/put_binary/{key:.*}", self._h_put_binary)
        r.add_put("/v1/add_object_to_set/{key:.*}", self._h_add_to_set)
        r.add_get("/v1/get_json/{key:.*}", self._h_get_json)
        r.add_put("/v1/put_json/{key:.*}", self._h_put_json)
        r.add_delete("/v1/delete/{key:.*}", self._h_delete)
        r.add_get("/v1/health", self._h_health)
        r.add_get("/v1/keys", self._h_keys)
        r.add_get("/v1/has_key/{key:.*}", self._h_has_key)
        r.add_post("/v1/allocate_auto_grow_id", self._h_alloc_id)
        r.add_put("/v1/put_counter/{key:.*}", self._h_put_counter)
        r.add_get("/v1/wait_counters", self._h_wait_counters)

    # ---- in-process store API --------------------------------------------------------
    def get_binary(self, key: str) -> bytes:
        return self.storage[key]

    def put_binary(self, key: str, binary: bytes) -> None:
        self.storage[key] = binary

    def get_object(self, key: str) -> Any:
        return pickle.loads(self.storage[key])

    def put_object(self, key: str, obj: Any) -> None:
        self.storage[key] = pickle.dumps(obj)

    def get_json(self, key: str):
        return json.loads(self.storage[key].decode("utf-8"))

    def put_json(self, key: str, json_data) -> None:
        self.storage[key] = json.dumps(json_data).encode("utf-8")

    def delete(self, key: str) -> None:
        if key not in self.storage:
            raise ValueError(f"Key '{key}' not found in storage")
        del self.storage[key]

    def get_address(self) -> str:
        return self.host

    def get_port(self) -> int:
        return self.port

    def get_address_and_port(self) -> Tuple[str, int]:
        return self.host, self.port

    # ---- lifecycle ----------------------------------------------------------------------
    def _serve(self) -> None:
        loop = asyncio.new_event_loop()
        asyncio.set_event_loop(loop)
        self._loop = loop
        try:
            self._runner = web.AppRunner(self.app, access_log=None)
            loop.run_until_complete(self._runner.setup())
            site = web.TCPSite(self._runner, self.host, self.port)
            loop.run_until_complete(site.start())
            if self.port == 0:
                self.port = site._server.sockets[0].getsockname()[1]
        except BaseException as exc:  # surfaced by start()
            self._error = exc
            self._ready.set()
            return
        self._ready.set()
        try:
            loop.run_forever()
        finally:
            loop.run_until_complete(self._runner.cleanup())
            loop.close()

    def start(self, timeout: float = 10.0) -> None:
        self._thread = threading.Thread(target=self._serve, daemon=True, name="AwexMetaServer")
        self._thread.start()
        if not self._ready.wait(timeout):
            raise RuntimeError(f"Server failed to respond within timeout on {self.host}:{self.port}")
        if self._error is not None:
            raise RuntimeError(f"Server failed to start on {self.host}:{self.port}: {self._error}") from self._error
        logger.info(f"Meta server is ready on {self.host}:{self.port}")

    def stop(self) -> None:
        if self._loop is not None and self._loop.is_running():
            self._loop.call_soon_threadsafe(self._loop.stop)
        if self._thread is not None:
            self._thread.join(timeout=5)

    # ---- HTTP handlers ------------------------------------------------------------------
    @web.middleware
    async def _guard(self, request, handler):
        # optional shared secret: the store holds pickles and device-memory tokens, and the reference's
        # protocol has no authentication at all; with AWEX_META_SERVER_TOKEN set on both sides every
        # request but the health probe must carry it
        secret = os.environ.get("AWEX_META_SERVER_TOKEN")
        if secret and request.path != "/v1/health" and request.headers.get(TOKEN_HEADER) != secret:
            return _fail(401, "missing or wrong " + TOKEN_HEADER)
        try:
            return await handler(request)
        except web.HTTPException as exc:
            return _fail(exc.status_code, str(exc))
        except Exception as exc:
            return _fail(500, "An error occurred: " + "".join(traceback.format_exception(type(exc), exc, exc.__traceback__)))

    async def _h_get_binary(self, request):
        key = request.match_info["key"]
        if key not in self.storage:
            return _fail(404, f"Key '{key}' not found")
        value = self.storage[key]
        body = value if isinstance(value, bytes) else to_binary(value)
        return web.Response(body=body, content_type="application/octet-stream")

    async def _h_put_binary(self, request):
        key = request.match_info["key"]
        self.storage[key] = await request.read()
        return _ok(message=f"Binary data stored for key '{key}'")

    async def _h_add_to_set(self, request):
        key = request.match_info["key"]
        try:
            member = from_binary(await request.read())
        except Exception as exc:
            return _fail(500, f"Failed to deserialize object: {exc}")
        bucket = self.storage.get(key)
        if not isinstance(bucket, set):
            bucket = self.storage[key] = set()
        bucket.add(member)
        return _ok(message=f"Object stored for key '{key}'", size=len(bucket))

    async def _h_get_json(self, request):
        key = request.match_info["key"]
        if key not in self.storage:
            return _fail(404, f"Key '{key}' not found")
        try:
            return _ok(data=json.loads(self.storage[key].decode("utf-8")))
        except Exception as exc:
            return _fail(500, f"Failed to parse JSON: {exc}")

    async def _h_put_json(self, request):
        key = request.match_info["key"]
        try:
            self.storage[key] = json.dumps(await request.json()).encode("utf-8")
        except Exception as exc:
            return _fail(500, f"Failed to store JSON: {exc}")
        return _ok(message=f"JSON data stored for key '{key}'")

    async def _h_delete(self, request):
        key = request.match_info["key"]
        try:
            self.delete(key)
        except ValueError as exc:
            return _fail(404, str(exc))
        return _ok(message=f"Key '{key}' deleted")

    async def _h_health(self, request):
        return _ok(status="healthy", storage_size=len(self.storage), address=self.host, port=self.port)

    async def _h_has_key(self, request):
        return _ok(has_key=request.match_info["key"] in self.storage)

    async def _h_keys(self, request):
        return _ok(keys=list(self.storage.keys()))

    async def _h_alloc_id(self, request):
        new_id = self.id_counter
        self.id_counter += 1
        return _ok(id=new_id)

    def _cond(self) -> asyncio.Condition:
        if self._counter_cond is None:  # created inside the server's loop
            self._counter_cond = asyncio.Condition()
        return self._counter_cond

    async def _h_put_counter(self, request):
        """Body: a JSON list of integers (or one integer).  Wakes every waiter."""
        key = request.match_info["key"]
        try:
            value = await request.json()
            value = [int(v) for v in value] if isinstance(value, list) else [int(value)]
        except Exception as exc:
            return _fail(400, f"counter value must be an integer or a list of integers: {exc}")
        cond = self._cond()
        async with cond:
            self.counters[key] = value
            cond.notify_all()
        return _ok(value=value)

    async def _h_wait_counters(self, request):
        """``?keys=a,b&min=N&timeout=S``: answers when the first element of every
        listed counter is at least N, or after S seconds; the answer holds the
        counters as they are then (``null`` for one that was never put) and
        ``reached``.  The wait sleeps on a condition inside the server: a waiter
        learns of a put in the time of one reply, without polling."""
        try:
            keys = [k for k in request.query.get("keys", "").split(",") if k]
            least = int(request.query.get("min", "0"))
            timeout = min(max(float(request.query.get("timeout", "0")), 0.0), MAX_SERVER_WAIT_S)
        except ValueError as exc:
            return _fail(400, f"bad wait_counters query: {exc}")

        def reached() -> bool:
            return all(k in self.counters and self.counters[k][0] >= least for k in keys)

        cond = self._cond()
        async with cond:
            ok = reached()
            if not ok and timeout > 0:
                try:
                    await asyncio.wait_for(cond.wait_for(reached), timeout)
                    ok = True
                except asyncio.TimeoutError:
                    ok = reached()
            values = {k: self.counters.get(k) for k in keys}
        return _ok(reached=ok, values=values)


# ---- subprocess hosting -------------------------------------------------------------------
def run_meta_server_process(host: str, port: int, result_queue) -> None:
    """Body of the spawned server process: report (ok, host, port) then idle
    until SIGTERM/SIGINT."""
    try:
        try:
            import uvloop

            asyncio.set_event_loop_policy(uvloop.EventLoopPolicy())
        except Exception:
            pass
        server = MetaServer(host, port)
        server.start()
        result_queue.put((True,) + server.get_address_and_port())
        stop = threading.Event()
        for sig in (signal.SIGINT, signal.SIGTERM):
            signal.signal(sig, lambda *_: stop.set())
        while not stop.wait(1.0):
            pass
        server.stop()
        os._exit(0)
    except Exception as exc:
        logger.exception(f"Failed to start meta server in subprocess: {exc}")
        result_queue.put((False, str(exc), None))
        os._exit(1)


_server_process = None


def _reap(process) -> None:
    if process is not None and process.is_alive():
        process.terminate()
        process.join(timeout=5)
        if process.is_alive():
            process.kill()
            process.join()


def start_meta_server(host: str = "", port: int = 0) -> Tuple[str, int]:
    """Spawn the server in a daemon subprocess; returns (address, port)."""
    global _server_process
    host = host or get_ip_address()
    port = port or get_free_port()
    ctx = multiprocessing.get_context("spawn")
    queue = ctx.Queue()
    process = ctx.Process(target=run_meta_server_process, args=(host, port, queue), name="MetaServerProcess", daemon=True)
    process.start()
    try:
        ok, address, actual_port = queue.get(timeout=120)
    except Exception as exc:
        _reap(process)
        raise RuntimeError(f"Meta server startup failed: {exc!r}") from exc
    if not ok:
        _reap(process)
        raise RuntimeError(f"Meta server startup failed in subprocess: {address}")
    _server_process = process
    start_meta_server._server_process = process
    logger.info(f"[{os.getpid()}] Meta server started in subprocess (PID: {process.pid}) on {address}:{actual_port}")
    return address, actual_port


def stop_meta_server() -> bool:
    global _server_process
    process = _server_process
    if process is None or not process.is_alive():
        return False
    _reap(process)
    _server_process = None
    return True


# ---- client -----------------------------------------------------------------------------------
def retry(fn, client, max_retries: int = 10, initial_delay: float = 1.0, max_delay: float = 10.0):
    """Call ``fn`` up to ``max_retries`` times with a linearly growing delay
    plus jitter; the HTTP session is rebuilt between attempts."""
    for attempt in range(max_retries):
        try:
            return fn()
        except Exception as exc:
            logger.error(f"Retry {attempt + 1}/{max_retries} failed for {getattr(fn, '__name__', fn)}: {exc}")
            if attempt == max_retries - 1:
                raise
            try:
                client._session.close()
            except Exception:
                pass
            client._session = _new_session()
            span = (max_delay - initial_delay) / max(max_retries - 1, 1)
            time.sleep(initial_delay + span * attempt + random.random())


class _Backoff:
    """0.2 s growing by 1.5x to 1 s; 3 s steps once a minute has passed."""

    def __init__(self):
        self.t0 = time.time()
        self.step = 0.2
        self.last_log = 0.0

    def sleep(self, what: str, remaining: float) -> None:
        slow = time.time() - self.t0 > 60
        time.sleep(3.0 if slow else self.step)
        self.step = 3.0 if slow else min(self.step * 1.5, 1.0)
        waited = time.time() - self.t0
        if waited - self.last_log >= 3:
            logger.info(f"Waiting for {what}, waited {waited:.1f}s, remaining wait time: {remaining:.1f}s")
            self.last_log = waited


def _new_session() -> "requests.Session":
    session = requests.Session()
    secret = os.environ.get("AWEX_META_SERVER_TOKEN")
    if secret:
        session.headers[TOKEN_HEADER] = secret
    return session


class MetaServerClient:
    def __init__(self, address: str, port: Union[int, str], max_retries: int = 10):
        self._address = address
        self._port = int(port)
        self._base_url = f"http://{address}:{port}"
        self._session = _new_session()
        self.timeout = 120
        self.max_retries = max_retries

    def _retry(self, fn, max_retries: Optional[int] = None, initial_delay: float = 1.0, max_delay: float = 10.0):
        return retry(fn, self, self.max_retries if max_retries is None else max_retries, initial_delay, max_delay)

    def _url(self, route: str, key: str = "") -> str:
        return f"{self._base_url}/v1/{route}/{key}" if key else f"{self._base_url}/v1/{route}"

    def _get(self, url: str, timeout: float = 120):
        return self._retry(lambda: self._session.get(url, timeout=timeout))

    def _put(self, url: str, data: bytes, timeout: float = 120):
        return self._retry(lambda: self._session.put(url, data=data, timeout=timeout))

    def _delete(self, url: str, timeout: float = 120):
        return self._retry(lambda: self._session.delete(url, timeout=timeout))

    # ---- presence / waiting -----------------------------------------------------------------
    def has_key(self, key: str) -> bool:
        resp = self._get(self._url("has_key", key))
        resp.raise_for_status()
        return bool(resp.json().get("has_key"))

    def _has_key(self, key: str) -> bool:
        try:
            return self.has_key(key)
        except (requests.exceptions.ConnectTimeout, requests.exceptions.ReadTimeout):
            return False

    def wait_key(self, key: str, timeout: float) -> None:
        deadline = time.time() + timeout
        pace = _Backoff()
        while not self._has_key(key):
            remaining = deadline - time.time()
            if remaining <= 0:
                raise TimeoutError(f"Timeout waiting for key '{key}'")
            pace.sleep(f"key '{key}' from meta server", remaining)

    # ---- binary / objects ---------------------------------------------------------------------
    def get_binary(self, key: str, timeout: float = 0) -> bytes:
        if timeout > 0:
            self.wait_key(key, timeout)
        resp = self._get(self._url("get_binary", key))
        if resp.status_code == 404:
            raise ValueError(f"Key '{key}' not found")
        resp.raise_for_status()
        return resp.content

    def put_binary(self, key: str, binary: bytes):
        resp = self._put(self._url("put_binary", key), data=binary)
        resp.raise_for_status()
        return resp.json()

    def get_object(self, key: str, timeout: float = 0, default_value: Any = None) -> Any:
        if timeout > 0:
            try:
                self.wait_key(key, timeout)
            except TimeoutError:
                if default_value is not None:
                    return default_value
                raise
        resp = self._get(self._url("get_binary", key))
        if resp.status_code == 404:
            return default_value
        resp.raise_for_status()
        return from_binary(resp.content)

    def put_object(self, key: str, obj: Any):
        resp = self._put(self._url("put_binary", key), data=to_binary(obj))
        resp.raise_for_status()
        result = resp.json()
        if not result.get("success"):
            raise RuntimeError(f"Failed to put object {key}: {result.get('error')}")
        return result

    def get_object_then_delete(self, key: str, timeout: float = 1024**3) -> Any:
        value = self.get_object(key, timeout)
        self.delete(key)
        return value

    # ---- sets -------------------------------------------------------------------------------------
    def add_object_to_set(self, key: str, obj: Any):
        resp = self._put(self._url("add_object_to_set", key), data=to_binary(obj))
        resp.raise_for_status()
        result = resp.json()
        if not result.get("success"):
            raise RuntimeError(f"Failed to add object to set {key}: {result.get('error')}")
        return result

    def get_set(self, key: str) -> set:
        return self.get_object(key, default_value=set())

    def wait_set_until_size(self, key: str, size: int, timeout: float, delete_after_wait: bool = False) -> None:
        deadline = time.time() + timeout
        pace = _Backoff()
        while len(self.get_object(key, default_value=set())) < size:
            remaining = deadline - time.time()
            if remaining <= 0:
                raise TimeoutError(f"Timeout waiting for set {key} to reach size {size}")
            pace.sleep(f"set {key} to reach size {size}", remaining)
        if delete_after_wait:
            self.delete_if_exists(key)

    def barrier(self, key: str, rank: int, world_size: int, timeout: float) -> None:
        """Everyone adds its rank to ``key`` and waits for ``world_size``
        members.  The key is left in place (deleting it could strand a slower
        waiter); use a fresh key per barrier."""
        self.add_object_to_set(key, rank)
        self.wait_set_until_size(key, world_size, timeout)

    # ---- json ---------------------------------------------------------------------------------------
    def get_json(self, key: str):
        resp = self._get(self._url("get_json", key))
        if resp.status_code == 404:
            raise ValueError(f"Key '{key}' not found")
        resp.raise_for_status()
        return resp.json().get("data")

    def put_json(self, key: str, json_data):
        resp = self._retry(lambda: self._session.put(self._url("put_json", key), json=json_data, timeout=self.timeout))
        resp.raise_for_status()
        return resp.json()

    # ---- misc ----------------------------------------------------------------------------------------
    def delete(self, key: str):
        resp = self._delete(self._url("delete", key))
        resp.raise_for_status()
        return resp.json()

    def delete_if_exists(self, key: str) -> None:
        try:
            resp = self._session.delete(self._url("delete", key), timeout=self.timeout)
            if resp.status_code not in (200, 404):
                resp.raise_for_status()
        except Exception:
            pass

    def health_check(self) -> dict:
        resp = self._get(self._url("health"))
        resp.raise_for_status()
        return resp.json()

    def list_keys(self) -> list:
        resp = self._get(self._url("keys"))
        resp.raise_for_status()
        return resp.json().get("keys", [])

    def allocate_auto_grow_id(self) -> int:
        resp = self._retry(lambda: self._session.post(self._url("allocate_auto_grow_id"), timeout=self.timeout))
        resp.raise_for_status()
        return int(resp.json()["id"])

    # ---- counters with server-side waiting ----------------------------------------------------------
    def put_counter(self, key: str, value) -> None:
        """Set counter ``key`` to an integer or a list of integers and wake its waiters."""
        from urllib.parse import quote

        resp = self._retry(lambda: self._session.put(self._url("put_counter", quote(key, safe="")), json=value, timeout=self.timeout))
        resp.raise_for_status()

    def get_counter(self, key: str):
        """The counter's list of integers, or ``None`` when it was never put."""
        return self.wait_counters([key], 0, 0.0, must_reach=False).get(key)

    def wait_counters(self, keys, at_least: int, timeout: float, must_reach: bool = True) -> Dict[str, Any]:
        """Block until the first element of every counter in ``keys`` is at least
        ``at_least``; returns ``{key: list}``.  The server holds each request for up
        to 20 s and answers the moment the last counter arrives, so a waiter sees a
        put within one round trip.  ``TimeoutError`` after ``timeout`` seconds (with
        ``must_reach``)."""
        from urllib.parse import quote

        keys = list(keys)
        if not keys:
            return {}
        deadline = time.time() + timeout
        query = "keys=" + ",".join(quote(k, safe="") for k in keys) + f"&min={int(at_least)}"
        while True:
            remaining = max(0.0, deadline - time.time())
            hold = min(remaining, MAX_SERVER_WAIT_S)
            url = f"{self._base_url}/v1/wait_counters?{query}&timeout={hold:.3f}"
            resp = self._retry(lambda: self._session.get(url, timeout=hold + self.timeout))
            resp.raise_for_status()
            body = resp.json()
            if body.get("reached") or not must_reach:
                return body.get("values", {})
            if time.time() >= deadline:
                missing = [k for k, v in body.get("values", {}).items() if v is None or v[0] < at_least]
                raise TimeoutError(f"counters {missing} did not reach {at_least} within {timeout:.1f}s")

    def close(self) -> None:
        self._session.close()
