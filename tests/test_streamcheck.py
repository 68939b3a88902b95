"""The logical stream-order checker (utils/streamcheck.py) on the schedule the training engine
uses for overlapped gradient buckets: backward writes gradients on the main stream, a
bucket's collective runs on the side stream after an event, the main stream joins the side
stream before it touches the buffers again."""
import pytest

from necklace_b200.utils.streamcheck import StreamOrderChecker, StreamOrderError, from_env


def _step(chk, join=True, wait=True, buckets=3):
    for b in reversed(range(buckets)):                       # backward fills the last bucket first
        chk.access(f"bucket{b}", "main", True, "gradients")
        if wait:
            chk.wait("side", chk.record("main"))
        chk.access(f"bucket{b}", "side", True, "collective")
    if join:
        chk.join("main", "side")


def test_engine_schedule_is_ordered_over_many_steps():
    chk = StreamOrderChecker()
    for _ in range(4):
        _step(chk)
    assert chk.checked == 4 * 3 * 2


def test_missing_join_is_reported_at_the_next_write():
    chk = StreamOrderChecker()
    _step(chk, join=False)
    with pytest.raises(StreamOrderError, match="not ordered after the write on stream 'side'"):
        _step(chk)


def test_missing_event_wait_is_reported_at_once():
    chk = StreamOrderChecker()
    with pytest.raises(StreamOrderError, match="on stream 'side'"):
        _step(chk, wait=False)


def test_reads_on_two_streams_do_not_conflict_but_a_later_write_must_follow_both():
    chk = StreamOrderChecker()
    chk.access("params", "main", True, "optimizer")
    chk.wait("side", chk.record("main"))
    chk.access("params", "side", False, "all-gather source")
    chk.access("params", "main", False, "forward")
    with pytest.raises(StreamOrderError, match="after the read on stream 'side'"):
        chk.access("params", "main", True, "optimizer, next step")
    chk.join("main", "side")
    chk.access("params", "main", True, "optimizer, next step")


def test_switch(monkeypatch):
    monkeypatch.delenv("NKB_DEBUG_STREAMS", raising=False)
    assert from_env() is None
    monkeypatch.setenv("NKB_DEBUG_STREAMS", "1")
    assert isinstance(from_env(), StreamOrderChecker)
