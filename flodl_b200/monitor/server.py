"""Minimal dashboard server on a raw TCP socket: `GET /` serves the dashboard page, `GET /events`
is a server-sent-event stream that first replays everything recorded so far (late joiners see
the whole run) and then pushes each new epoch (flodl/src/monitor/server.rs:62-130)."""
from __future__ import annotations

import json
import socket
import threading
from typing import Callable, List, Optional


class DashboardServer:
    def __init__(self, port: int, page_fn: Callable[[], str], host: str = "127.0.0.1"):
        self._page_fn = page_fn
        self._sock = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self._sock.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self._sock.bind((host, port))
        self._sock.listen(16)
        self._sock.settimeout(0.2)
        self.port = self._sock.getsockname()[1]
        self._lock = threading.Lock()
        self._epochs: List[str] = []
        self._init: dict = {}
        self._clients: List[socket.socket] = []
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._accept_loop, name="monitor-http", daemon=True)
        self._thread.start()

    @classmethod
    def start(cls, port: int, page_fn: Callable[[], str]) -> "DashboardServer":
        return cls(port, page_fn)

    # ---- state pushed by the monitor ------------------------------------------------------------
    def push_epoch(self, payload: str) -> None:
        with self._lock:
            self._epochs.append(payload)
            clients = list(self._clients)
        self._send_all(clients, "epoch", payload)

    def _set(self, key: str, value) -> None:
        with self._lock:
            self._init[key] = value
            clients = list(self._clients)
        self._send_all(clients, "init", json.dumps({key: value}))

    def set_svg(self, svg: str) -> None: self._set("svg", svg)
    def set_label_hash(self, label: Optional[str], hash_: Optional[str]) -> None:
        self._set("label", label)
        self._set("hash", hash_)
    def set_hardware(self, hw: str) -> None: self._set("hardware", hw)
    def set_metadata(self, meta) -> None: self._set("metadata", meta)
    def set_gpu_init(self, info) -> None: self._set("gpu_init", info)

    # ---- plumbing -------------------------------------------------------------------------------
    @staticmethod
    def _sse(event: str, data: str) -> bytes:
        return f"event: {event}\ndata: {data}\n\n".encode()

    def _send_all(self, clients, event: str, data: str) -> None:
        dead = []
        for c in clients:
            try:
                c.sendall(self._sse(event, data))
            except OSError:
                dead.append(c)
        if dead:
            with self._lock:
                self._clients = [c for c in self._clients if c not in dead]

    def _accept_loop(self) -> None:
        while not self._stop.is_set():
            try:
                conn, _ = self._sock.accept()
            except socket.timeout:
                continue
            except OSError:
                return
            threading.Thread(target=self._serve, args=(conn,), daemon=True).start()

    def _serve(self, conn: socket.socket) -> None:
        try:
            conn.settimeout(2.0)
            req = conn.recv(4096).decode("latin-1", "replace")
            path = req.split(" ")[1] if req.startswith("GET ") and len(req.split(" ")) > 1 else "/"
            if path.startswith("/events"):
                conn.sendall(b"HTTP/1.1 200 OK\r\nContent-Type: text/event-stream\r\nCache-Control: no-cache\r\nConnection: keep-alive\r\n\r\n")
                with self._lock:
                    init, epochs = dict(self._init), list(self._epochs)
                    self._clients.append(conn)
                conn.settimeout(None)
                conn.sendall(self._sse("init", json.dumps(init)))
                for e in epochs:                      # late-join backfill
                    conn.sendall(self._sse("epoch", e))
                return                                # the socket stays with the broadcaster
            body = self._page_fn().encode()
            conn.sendall(b"HTTP/1.1 200 OK\r\nContent-Type: text/html; charset=utf-8\r\nContent-Length: " + str(len(body)).encode()
                         + b"\r\nConnection: close\r\n\r\n" + body)
            conn.close()
        except Exception:
            try:
                conn.close()
            except OSError:
                pass

    def shutdown(self) -> None:
        self._stop.set()
        try:
            self._sock.close()
        except OSError:
            pass
        with self._lock:
            clients, self._clients = self._clients, []
        for c in clients:
            try:
                c.close()
            except OSError:
                pass
