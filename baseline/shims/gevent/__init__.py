"""Stand-in for the few gevent calls the reference makes: ``gevent.spawn(fn, *a)``,
``gevent.sleep(s)``, ``gevent.queue.Queue``.  Cooperative, single-threaded (see ``_nkhub``):
a spawned RPC server is served while the caller sleeps, waits on a queue or waits for an
RPC reply; anything else that is spawned gets a daemon thread."""
import threading
import time

import _nkhub

from . import queue  # noqa: F401


class _Greenlet:
    def __init__(self, thread=None):
        self._thread = thread

    def kill(self):
        pass

    def join(self, timeout=None):
        if self._thread is not None:
            self._thread.join(timeout)

    get = join


def spawn(fn, *args, **kwargs):
    owner = getattr(fn, "__self__", None)
    if owner is not None and hasattr(owner, "_zsock") and getattr(fn, "__name__", "") == "run":
        _nkhub.register(owner)
        return _Greenlet()
    t = threading.Thread(target=fn, args=args, kwargs=kwargs, daemon=True)
    t.start()
    return _Greenlet(t)


def sleep(seconds=0):
    # The reference sprinkles sub-millisecond sleeps ("wait the zrpc call to return") so that
    # the server greenlet can finish sending a reply before the service loop goes on.  Here a
    # reply has always been sent when its handler returns, and serving NEW requests inside
    # such a sleep would let a request that the original stack delivers a millisecond later
    # (zerorpc's per-call latency) overtake the job that the service loop has just taken from
    # its queue.  So sleeps below a millisecond only sleep; longer ones serve requests.
    if seconds and 0 < seconds < 1e-3:
        time.sleep(seconds)
        return
    end = time.monotonic() + max(0.0, seconds or 0.0)
    _nkhub.serve(0.0)
    if not seconds or seconds <= 0:
        return
    while True:
        left = end - time.monotonic()
        if left <= 0:
            return
        _nkhub.serve(min(left, 0.05))


def joinall(greenlets, timeout=None):
    for g in greenlets:
        g.join(timeout)
