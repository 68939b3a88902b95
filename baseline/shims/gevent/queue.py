"""``gevent.queue.Queue``: a queue whose blocking ``get`` serves the process's RPC servers
while it waits (the cooperative yield of the original)."""
import collections
import time

import _nkhub


class Empty(Exception):
    pass


class Full(Exception):
    pass


class Queue:
    def __init__(self, maxsize=None):
        self._d = collections.deque()

    def qsize(self):
        return len(self._d)

    def empty(self):
        return not self._d

    def put(self, item, block=True, timeout=None):
        self._d.append(item)

    put_nowait = put

    def get_nowait(self):
        if not self._d:
            raise Empty()
        return self._d.popleft()

    def get(self, block=True, timeout=None):
        if self._d:
            return self._d.popleft()
        if not block:
            raise Empty()
        end = None if timeout is None else time.monotonic() + timeout
        while True:
            left = 0.05 if end is None else min(0.05, end - time.monotonic())
            if left <= 0:
                raise Empty()
            _nkhub.serve(left)
            if self._d:
                return self._d.popleft()


JoinableQueue = LifoQueue = PriorityQueue = Queue
