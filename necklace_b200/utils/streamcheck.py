"""Stream-ordering assertions for code that spreads work over several CUDA streams.

The reference orders everything by synchronising everything (current-stream + device sync
around every collective, necklace/trainer/tnoppt.py:551-554).  Here collectives of gradient
buckets run on a side stream while backward continues, ordered by events only; this checker
is the debug aid for that: it keeps a logical clock per stream (a vector clock, advanced by
every recorded access, merged by event waits) and raises when a buffer is touched on one
stream while the last conflicting access on another stream is not ordered before it.

    chk = StreamOrderChecker()
    chk.access("bucket0", "main", write=True)        # backward writes the gradients
    ev = chk.record("main"); chk.wait("side", ev)    # event recorded on main, side waits
    chk.access("bucket0", "side", write=True)        # collective on the side stream: fine
    chk.access("bucket0", "main", write=True)        # next step zeroes them: raises, no join

It checks the program's ordering logic, not the hardware: the same calls are made on a CPU
run.  The engines create one when ``NKB_DEBUG_STREAMS=1``."""
from __future__ import annotations

import os


class StreamOrderError(RuntimeError):
    pass


class StreamOrderChecker:
    def __init__(self):
        self.clock: dict = {}          # stream -> {stream: time}: what this stream has seen
        self.last_write: dict = {}     # buffer -> (stream, time, note)
        self.last_reads: dict = {}     # buffer -> {stream: (time, note)}
        self.checked = 0

    def _vc(self, stream):
        return self.clock.setdefault(stream, {stream: 0})

    def _tick(self, stream):
        vc = self._vc(stream)
        vc[stream] += 1
        return vc[stream]

    def record(self, stream):
        """An event recorded on ``stream``: a snapshot of all it has seen so far."""
        self._tick(stream)
        return dict(self._vc(stream))

    def wait(self, stream, event) -> None:
        """``stream`` waits for ``event``: everything before the event is ordered before
        whatever ``stream`` does next."""
        vc = self._vc(stream)
        for s, t in event.items():
            if t > vc.get(s, 0):
                vc[s] = t

    def join(self, stream, other) -> None:
        """``stream.wait_stream(other)``."""
        self.wait(stream, self.record(other))

    def _ordered(self, who, stream, time) -> bool:
        return stream == who or self._vc(who).get(stream, 0) >= time

    def access(self, buf, stream, write: bool, note: str = "") -> None:
        self.checked += 1
        lw = self.last_write.get(buf)
        if lw is not None and not self._ordered(stream, lw[0], lw[1]):
            raise StreamOrderError(
                f"{'write' if write else 'read'} of {buf!r} on stream {stream!r} ({note}) is not "
                f"ordered after the write on stream {lw[0]!r} ({lw[2]})")
        if write:
            for s, (t, n) in self.last_reads.get(buf, {}).items():
                if not self._ordered(stream, s, t):
                    raise StreamOrderError(
                        f"write of {buf!r} on stream {stream!r} ({note}) is not ordered after "
                        f"the read on stream {s!r} ({n})")
        t = self._tick(stream)
        if write:
            self.last_write[buf] = (stream, t, note)
            self.last_reads[buf] = {}
        else:
            self.last_reads.setdefault(buf, {})[stream] = (t, note)


def from_env():
    """A checker when ``NKB_DEBUG_STREAMS`` is set to something other than 0, else None."""
    return StreamOrderChecker() if os.environ.get("NKB_DEBUG_STREAMS", "0") not in ("", "0") \
        else None
