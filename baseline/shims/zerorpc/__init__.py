"""Minimal zerorpc: ``Server`` exposes the public methods of the object (or of ``self``)
on a bound url, ``Client`` turns attribute access into remote calls.  pyzmq ROUTER / DEALER
sockets, msgpack framing.  A server started through ``gevent.spawn(server.run)`` is served
cooperatively on the caller's thread (see ``_nkhub``); a client that waits for its reply
keeps serving this process's servers meanwhile, as a greenlet blocked on a reply yields to
the server greenlet in the original."""
import itertools
import threading
import time
import uuid

import msgpack
import zmq  # noqa: F401  (the reference does ``from zerorpc import zmq``)

import _nkhub

_ctx = None
_ctx_lock = threading.Lock()


def _context():
    global _ctx
    with _ctx_lock:
        if _ctx is None:
            _ctx = zmq.Context.instance()
        return _ctx


class TimeoutExpired(Exception):
    pass


class LostRemote(Exception):
    pass


class RemoteError(Exception):
    def __init__(self, name, msg, tb=None):
        super().__init__(f"{name}: {msg}\n{tb or ''}")
        self.name, self.msg, self.traceback = name, msg, tb


class Server:
    def __init__(self, methods=None, name=None, context=None, pool_size=None, heartbeat=5):
        self._methods = methods if methods is not None else self
        self._zsock = _context().socket(zmq.ROUTER)
        self._zsock.setsockopt(zmq.LINGER, 0)
        self._zstop = False

    def bind(self, endpoint):
        self._zsock.bind(endpoint)

    def connect(self, endpoint):
        self._zsock.connect(endpoint)

    def _handle_one(self, block=True):
        """Receive and answer one request; returns False when none was waiting."""
        try:
            frames = self._zsock.recv_multipart(0 if block else zmq.NOBLOCK)
        except zmq.Again:
            return False
        except zmq.ZMQError:
            return False
        ident, payload = frames[0], frames[-1]
        rid = None
        try:
            rid, name, args, kwargs = msgpack.unpackb(payload, raw=False)
            if name.startswith("_"):
                raise AttributeError(name)
            ret = getattr(self._methods, name)(*args, **kwargs)
            rep = [rid, True, ret, None]
        except Exception as e:  # noqa: BLE001
            import traceback
            rep = [rid, False, f"{type(e).__name__}: {e}", traceback.format_exc()]
        try:
            self._zsock.send_multipart([ident, msgpack.packb(rep, use_bin_type=True)])
        except zmq.ZMQError:
            pass
        return True

    def run(self):
        """Blocking serve loop (for a server that owns its thread)."""
        poller = zmq.Poller()
        poller.register(self._zsock, zmq.POLLIN)
        while not self._zstop:
            try:
                if dict(poller.poll(50)):
                    self._handle_one(block=False)
            except zmq.ZMQError:
                break

    def stop(self):
        self._zstop = True

    def close(self):
        self._zstop = True
        try:
            self._zsock.close(0)
        except Exception:  # noqa: BLE001
            pass


class Client:
    _ids = itertools.count(1)

    def __init__(self, connect_to=None, context=None, timeout=30, heartbeat=5,
                 passive_heartbeat=False):
        self._ztimeout = timeout
        self._zlock = threading.Lock()
        self._zsock = _context().socket(zmq.DEALER)
        self._zsock.setsockopt(zmq.LINGER, 0)
        self._zsock.setsockopt(zmq.IDENTITY, uuid.uuid4().bytes)
        if connect_to:
            self.connect(connect_to)

    def connect(self, endpoint):
        self._zsock.connect(endpoint)

    def bind(self, endpoint):
        self._zsock.bind(endpoint)

    def _zcall(self, name, *args, **kwargs):
        rid = next(Client._ids)
        timeout = kwargs.pop("timeout", None) or self._ztimeout or 30
        deadline = time.monotonic() + timeout
        with self._zlock:
            self._zsock.send(msgpack.packb([rid, name, list(args), kwargs], use_bin_type=True))
            while True:
                left = deadline - time.monotonic()
                if left <= 0:
                    raise TimeoutExpired(f"timeout after {timeout}s calling {name}")
                if not _nkhub.serve(min(left, 0.05), extra=self._zsock):
                    continue
                rep = msgpack.unpackb(self._zsock.recv(), raw=False)
                if rep[0] != rid:
                    continue
                if not rep[1]:
                    raise RemoteError(name, rep[2], rep[3])
                return rep[2]

    def __call__(self, method, *args, **kwargs):
        return self._zcall(method, *args, **kwargs)

    def __getattr__(self, name):
        if name.startswith("_"):
            raise AttributeError(name)
        return lambda *a, **k: self._zcall(name, *a, **k)

    def close(self):
        try:
            self._zsock.close(0)
        except Exception:  # noqa: BLE001
            pass
