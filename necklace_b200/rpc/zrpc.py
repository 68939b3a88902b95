"""OneRPC transport: ``Server`` / ``Client`` / ``Node`` on pyzmq.

Same roles as the reference's zerorpc + gevent classes (necklace/rpc/zrpc.py:49-285):
every public method of a ``Server`` subclass is an RPC endpoint, a ``Client`` calls
them as attributes (``cli.fn_worker_reg(msg)``), and a ``Node`` runs the server next
to a set of timers whose default one, ``check_state``, drains a job queue.

Differences.  The server is a ROUTER socket served by a thread (no gevent), the
client a DEALER socket with a per-call deadline and a retry-free, explicit
``RpcTimeout`` / ``RpcRemoteError``; each request carries an id so late replies of
a timed-out call are dropped instead of being mistaken for the next reply;
``Client.ping`` doubles as the heartbeat; and a ``drop_filter`` hook lets tests
lose or delay chosen messages on the host to exercise failure handling.
"""
from __future__ import annotations

import itertools
import queue
import threading
import time
import traceback
import uuid
from collections import OrderedDict

import zmq

from . import msgpck
from .mixinbase import NodeMixin


class NodeBase(object):
    """Root of the node classes (reference: necklace/rpc/zrpc.py:34-35)."""

DEFAULT_URL = "ipc:///tmp/zrpc-1.ipc"


class RpcError(RuntimeError):
    pass


class RpcTimeout(RpcError):
    pass


class RpcRemoteError(RpcError):
    pass


_ctx_lock = threading.Lock()


def _context() -> zmq.Context:
    with _ctx_lock:
        return zmq.Context.instance()


class Server(NodeMixin):
    """Binds ``cfg['url']`` and serves the public methods of the subclass."""

    def __init__(self, ndid=None, cfg=None):
        super().__init__(ndid, cfg)
        self.stopped = False
        self.q = self.cfg.get("q") or queue.Queue()
        self.drop_filter = self.cfg.get("drop_filter")  # fn(name, args, kwargs) -> bool (tests)
        self._thread = None
        self._sock = None
        self.init_sock()

    def init_sock(self):
        self.url = self.cfg.get("url") or DEFAULT_URL
        self._sock = _context().socket(zmq.ROUTER)
        self._sock.setsockopt(zmq.LINGER, 0)
        self._sock.bind(self.url)

    # queue helpers -----------------------------------------------------------
    def q_put(self, q=None, m=None, *args, **kwargs):
        (q or self.q).put(m)

    def q_get(self, q=None, *args, **kwargs):
        try:
            return (q or self.q).get(*args, **kwargs)
        except queue.Empty:
            return None

    # (de)serialisation -------------------------------------------------------
    def msg_pck(self, msg):
        return msgpck.packb(msg)

    def msg_unpck(self, msg):
        return msgpck.unpackb(msg)

    def msg_pkpck(self, msg):
        return msgpck.pkpackb(msg)

    def msg_unpkpck(self, msg):
        return msgpck.unpkpackb(msg)

    def snd_msg(self, cli, func, *args, **kwargs):
        return getattr(cli, func)(*args, **kwargs)

    # built-in endpoints ------------------------------------------------------
    def g_sleep(self, n):
        """Sleep ``n`` seconds (the services' cooperative sleep, also offered on the server:
        the reference's examples/rl/dssvsc.py calls it there)."""
        time.sleep(n)

    def ping(self):
        return "pong"

    def lolita(self):
        return 42

    def add(self, a, b):
        return a + b

    # serving -----------------------------------------------------------------
    def _dispatch(self, name, args, kwargs):
        if name.startswith("_") or not hasattr(self, name):
            raise AttributeError(f"no RPC endpoint {name!r}")
        return getattr(self, name)(*args, **kwargs)

    def run(self):
        poller = zmq.Poller()
        poller.register(self._sock, zmq.POLLIN)
        while not self.stopped:
            try:
                if not dict(poller.poll(100)):
                    continue
                frames = self._sock.recv_multipart()
            except zmq.ZMQError:
                break
            ident, payload = frames[0], frames[-1]
            try:
                req = msgpck.unpackb(payload)
                rid, name = req["id"], req["fn"]
                args, kwargs = req.get("args", []), req.get("kwargs", {})
                if self.drop_filter is not None and self.drop_filter(name, args, kwargs):
                    continue  # simulated loss: no reply, the caller's deadline fires
                rep = {"id": rid, "ok": True, "ret": self._dispatch(name, args, kwargs)}
            except Exception as e:  # noqa: BLE001
                rep = {"id": req.get("id") if isinstance(req, dict) else None, "ok": False,
                       "err": f"{type(e).__name__}: {e}", "tb": traceback.format_exc()}
            try:
                self._sock.send_multipart([ident, msgpck.packb(rep)])
            except zmq.ZMQError:
                break
        try:
            self._sock.close(0)
        except Exception:  # noqa: BLE001
            pass

    def loop(self):
        self.run()

    def start(self):
        if self._thread is None:
            self._thread = threading.Thread(target=self.run, daemon=True,
                                            name=f"rpc-server-{self.ndid}")
            self._thread.start()
        return self._thread

    def stop(self):
        self.stopped = True
        if self._thread is not None and self._thread is not threading.current_thread():
            self._thread.join(timeout=2)


class Client(NodeMixin):
    """Connects to ``cfg['url']``; attribute access yields remote callables."""

    _ids = itertools.count(1)

    def __init__(self, ndid=None, cfg=None):
        super().__init__(ndid, cfg)
        self.timeout = float(self.cfg.get("zc_hb_timeout", 100))
        self.heartbeat = float(self.cfg.get("zc_hb_heartbeat", 10))
        self._lock = threading.Lock()
        self.init_sock()

    def init_sock(self):
        self.url = self.cfg.get("url") or DEFAULT_URL
        self._sock = _context().socket(zmq.DEALER)
        self._sock.setsockopt(zmq.LINGER, 0)
        self._sock.setsockopt(zmq.IDENTITY, uuid.uuid4().bytes)
        self._sock.connect(self.url)

    def msg_pck(self, msg):
        return msgpck.packb(msg)

    def msg_unpck(self, msg):
        return msgpck.unpackb(msg)

    def msg_pkpck(self, msg):
        return msgpck.pkpackb(msg)

    def msg_unpkpck(self, msg):
        return msgpck.unpkpackb(msg)

    def call(self, name, *args, timeout=None, **kwargs):
        rid = next(Client._ids)
        deadline = time.monotonic() + (self.timeout if timeout is None else timeout)
        with self._lock:
            self._sock.send(msgpck.packb({"id": rid, "fn": name, "args": list(args),
                                          "kwargs": kwargs}))
            while True:
                left = deadline - time.monotonic()
                if left <= 0 or not self._sock.poll(int(left * 1000) + 1):
                    raise RpcTimeout(f"{name} on {self.url}: no reply within "
                                     f"{self.timeout if timeout is None else timeout}s")
                rep = msgpck.unpackb(self._sock.recv())
                if rep.get("id") != rid:
                    continue  # stale reply of an earlier call that timed out
                if not rep.get("ok"):
                    raise RpcRemoteError(f"{name} on {self.url}: {rep.get('err')}\n"
                                         f"{rep.get('tb', '')}")
                return rep.get("ret")

    def snd_msg(self, func, *args, **kwargs):
        return self.call(func, *args, **kwargs)

    def alive(self, timeout=None) -> bool:
        try:
            return self.call("ping", timeout=timeout or self.heartbeat) == "pong"
        except RpcError:
            return False

    def __getattr__(self, name):
        if name.startswith("_"):
            raise AttributeError(name)
        return lambda *a, **k: self.call(name, *a, **k)

    def close(self):
        try:
            self._sock.close(0)
        except Exception:  # noqa: BLE001
            pass

    def loop(self):
        pass


class Node:
    """A server plus timers.  Timers are ``[last, interval, fn, args, kwargs]``; the
    default one calls ``check_state`` as often as possible."""

    def __init__(self, cfg, svr=None):
        self.cfg = cfg
        self.svr = svr
        self.clis = {}
        self.timers = OrderedDict()
        self.state = 0
        self.stopped = False
        self.q = queue.Queue()
        self.init_clis()
        self.init_timers()

    def init_clis(self):
        for url in self.cfg.get("clis") or []:
            self.clis[url] = Client(url, {"url": url})

    def init_timers(self):
        self.register_timer(0, self.check_state)

    def func_name(self, func):
        return str(id(func)) + str(uuid.uuid4())

    def register_timer(self, intvl, func, *args, **kwargs):
        self.timers[self.func_name(func)] = [time.time(), intvl, func, args, kwargs]

    def check_state(self, *args, **kwargs):
        pass

    def q_put(self, q=None, m=None, *args, **kwargs):
        (q or self.q).put(m)

    def q_get(self, q=None, *args, **kwargs):
        try:
            return (q or self.q).get(*args, **kwargs)
        except queue.Empty:
            return None

    def g_sleep(self, n):
        if n > 0:
            time.sleep(n)

    def tm_to_sleep(self):
        if not self.timers:
            return 1
        return min(v[1] for v in self.timers.values()) / 2.0

    def run_timers(self):
        now = time.time()
        for v in list(self.timers.values()):
            if now - v[0] >= v[1]:
                v[2](*v[3], **v[4])
                v[0] = now

    def stop(self):
        self.stopped = True

    def start_svr(self):
        if self.svr:
            self.svr.start()

    def loop(self):
        self.start_svr()
        try:
            while not self.stopped:
                self.run_timers()
                self.g_sleep(self.tm_to_sleep())
        finally:
            if self.svr:
                self.svr.stop()
            for c in self.clis.values():
                c.close()
