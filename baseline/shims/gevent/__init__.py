"""Thread-backed stand-in for the few gevent calls the reference makes:
``gevent.spawn(fn, *a)``, ``gevent.sleep(s)``, ``gevent.queue.Queue``."""
import threading
import time

from . import queue  # noqa: F401


class _Greenlet(threading.Thread):
    def __init__(self, fn, *args, **kwargs):
        super().__init__(target=fn, args=args, kwargs=kwargs, daemon=True)
        self.start()

    def kill(self):
        pass

    def get(self, timeout=None):
        self.join(timeout)


def spawn(fn, *args, **kwargs):
    return _Greenlet(fn, *args, **kwargs)


def sleep(seconds=0):
    # gevent.sleep(0) yields to the other greenlets; a short real sleep lets the server
    # thread take the interpreter lock
    time.sleep(seconds if seconds and seconds > 0 else 0.0002)


def joinall(greenlets, timeout=None):
    for g in greenlets:
        g.join(timeout)
