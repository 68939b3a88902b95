"""``gevent.queue`` names on top of the standard library queue."""
from queue import Empty, Full, LifoQueue, PriorityQueue, Queue  # noqa: F401

JoinableQueue = Queue
