"""Node agent: hosts the worker processes of one machine for a controller running elsewhere.

    python -m disagmoe_b200.frontend.node_agent --host 0.0.0.0 --port 7700 [--authkey secret]

The controller connects once per device it places on this node (``Controller(..., worker_addresses={device_id:
(host, port)})``); every connection gets its own worker process that serves the same method-call protocol as a
locally spawned worker. This takes the place of the reference's Ray actors and placement groups
(disagmoe/frontend/controller.py:72-128, ray_helper.py:8-16): no cluster manager is needed, only a reachable port.
"""
from __future__ import annotations

import argparse
import multiprocessing as mp
import threading
from multiprocessing.connection import Client, Listener
from typing import Dict, Optional, Tuple

from .controller import ConnWorker

DEFAULT_AUTHKEY = b"disagmoe_b200"


def _serve_connection(conn) -> None:
    """First message: (device_id, device, env). Then the worker loop of the controller module."""
    from .controller import _worker_main
    hello = conn.recv()
    device_id, device, env = hello
    conn.send(("ok", None))
    _worker_main(conn, device_id, device, env)
    conn.close()


class NodeAgent:
    def __init__(self, host: str = "127.0.0.1", port: int = 7700, authkey: bytes = DEFAULT_AUTHKEY):
        self.listener = Listener((host, port), authkey=authkey)
        self.address = self.listener.address
        self.procs = []
        self._stop = False

    def serve_forever(self) -> None:
        ctx = mp.get_context("spawn")
        while not self._stop:
            try:
                conn = self.listener.accept()
            except OSError:
                break
            # the connection object is handed to a fresh process: one engine per process, as with local workers
            p = ctx.Process(target=_serve_connection, args=(conn,), daemon=True)
            p.start()
            conn.close()                   # the child owns it now
            self.procs.append(p)

    def start_in_thread(self) -> threading.Thread:
        t = threading.Thread(target=self.serve_forever, daemon=True, name="node-agent")
        t.start()
        return t

    def stop(self) -> None:
        self._stop = True
        try:
            self.listener.close()
        except OSError:
            pass
        for p in self.procs:
            p.join(timeout=5)
            if p.is_alive():
                p.terminate()


class RemoteWorkerHandle(ConnWorker):
    """A worker hosted by a :class:`NodeAgent`, reached over TCP (same interface as ``controller.WorkerHandle``)."""

    def __init__(self, device_id: int, device: str, address: Tuple[str, int], env: Optional[Dict[str, str]] = None,
                 authkey: bytes = DEFAULT_AUTHKEY):
        self.device_id = device_id
        self.address = address
        conn = Client(tuple(address), authkey=authkey)
        conn.send((device_id, device, env or {}))
        status, _ = conn.recv()
        assert status == "ok"
        self._init_conn(conn)

    def alive(self) -> bool:
        if self._dead:
            return False
        try:
            # between two calls nothing is expected on the connection: readable + EOF means the peer closed it
            if self.lock.acquire(blocking=False):
                try:
                    if self.conn.poll(0):
                        self.conn.recv()
                finally:
                    self.lock.release()
            return True
        except (EOFError, OSError):
            self._dead = True
            return False

    def stop(self) -> None:
        self._send_stop()
        try:
            self.conn.close()
        except Exception:
            pass


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=7700)
    ap.add_argument("--authkey", default=DEFAULT_AUTHKEY.decode())
    a = ap.parse_args(argv)
    agent = NodeAgent(a.host, a.port, a.authkey.encode())
    print(f"node agent listening on {agent.address}", flush=True)
    try:
        agent.serve_forever()
    finally:
        agent.stop()


if __name__ == "__main__":
    main()
