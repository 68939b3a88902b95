"""One cooperative scheduler per process for the gevent / zerorpc stand-ins.

gevent runs every greenlet of a process on one thread and switches only where a greenlet
blocks (``gevent.sleep``, a queue ``get``, waiting for an RPC reply), and the reference
depends on that: an RPC handler runs to completion before the service loop continues, and
the service loop handles a queued job before the next request is looked at.  The stand-ins
keep those semantics: RPC servers started with ``gevent.spawn(server.run)`` are not threads
but sockets registered here, and they are served exactly while the caller is blocked in one
of those three places."""
import time

import zmq

_servers = []


def register(server):
    if server not in _servers:
        _servers.append(server)


def unregister(server):
    if server in _servers:
        _servers.remove(server)


def serve(timeout=0.0, extra=None):
    """Wait up to ``timeout`` seconds for a request on any registered server socket (or for
    ``extra``, a client socket waiting for its reply, to become readable), then run the
    handler of the oldest request on each ready socket.  Returns True if ``extra`` is
    readable."""
    socks = [s for s in _servers if not s._zstop]
    if not socks and extra is None:
        if timeout > 0:
            time.sleep(timeout)
        return False
    poller = zmq.Poller()
    for s in socks:
        poller.register(s._zsock, zmq.POLLIN)
    if extra is not None:
        poller.register(extra, zmq.POLLIN)
    try:
        ready = dict(poller.poll(max(0, int(timeout * 1000))))
    except zmq.ZMQError:
        return False
    for s in socks:
        if s._zsock in ready:
            # One request per socket per call: the caller (a queue ``get``, a sleep, a reply
            # wait) then looks at its own condition again, so a job that this request queued
            # is taken up before a request that arrives later is handled, which is the
            # order a gevent hub gives (the woken greenlet runs before later I/O events).
            s._handle_one(block=False)
    return extra is not None and extra in ready
