"""Length-prefixed msgpack RPC over TCP: a threaded server dispatching ``{"method", "params"}`` requests to
registered handlers, and a blocking client with timeouts (reference: loongforge/embodied/eval/transport/client.py,
rpc_server.py)."""
from __future__ import annotations

import socket
import socketserver
import struct
import threading
import time
from typing import Any, Callable, Dict, Optional

from . import msgpack_numpy as mp


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    buf = bytearray()
    while len(buf) < n:
        chunk = sock.recv(n - len(buf))
        if not chunk:
            raise ConnectionError("peer closed the connection")
        buf += chunk
    return bytes(buf)


def send_frame(sock: socket.socket, obj: Any) -> None:
    data = mp.packb(obj)
    sock.sendall(struct.pack("<Q", len(data)) + data)


def recv_frame(sock: socket.socket) -> Any:
    (n,) = struct.unpack("<Q", _recv_exact(sock, 8))
    return mp.unpackb(_recv_exact(sock, n))


class RPCServer:
    def __init__(self, host: str = "127.0.0.1", port: int = 0):
        self.handlers: Dict[str, Callable[..., Any]] = {"ping": lambda: "pong"}
        outer = self

        class Handler(socketserver.BaseRequestHandler):
            def handle(self):
                while True:
                    try:
                        req = recv_frame(self.request)
                    except (ConnectionError, OSError, struct.error):
                        return
                    t0 = time.perf_counter()
                    try:
                        fn = outer.handlers[req["method"]]
                        res = {"ok": True, "result": fn(**(req.get("params") or {}))}
                    except Exception as e:  # noqa: BLE001 - errors travel back to the caller
                        res = {"ok": False, "error": f"{type(e).__name__}: {e}"}
                    res["server_ms"] = (time.perf_counter() - t0) * 1e3
                    res["id"] = req.get("id")
                    send_frame(self.request, res)

        class Server(socketserver.ThreadingTCPServer):
            allow_reuse_address = True
            daemon_threads = True

        self.server = Server((host, port), Handler)
        self.host, self.port = self.server.server_address
        self.thread: Optional[threading.Thread] = None

    def register(self, name: str, fn: Callable[..., Any]) -> None:
        self.handlers[name] = fn

    def start(self) -> "RPCServer":
        self.thread = threading.Thread(target=self.server.serve_forever, daemon=True)
        self.thread.start()
        return self

    def stop(self) -> None:
        self.server.shutdown()
        self.server.server_close()


class RPCError(RuntimeError):
    pass


class RPCClient:
    def __init__(self, host: str, port: int, timeout: float = 30.0, retries: int = 20, retry_wait: float = 0.1):
        last = None
        for _ in range(retries):
            try:
                self.sock = socket.create_connection((host, port), timeout=timeout)
                break
            except OSError as e:
                last = e
                time.sleep(retry_wait)
        else:
            raise ConnectionError(f"cannot reach policy server {host}:{port}: {last}")
        self.sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        self._id = 0
        self.last_server_ms = 0.0

    def call(self, method: str, **params) -> Any:
        self._id += 1
        send_frame(self.sock, {"id": self._id, "method": method, "params": params})
        res = recv_frame(self.sock)
        self.last_server_ms = res.get("server_ms", 0.0)
        if not res["ok"]:
            raise RPCError(res["error"])
        return res["result"]

    def close(self) -> None:
        try:
            self.sock.close()
        except OSError:
            pass
