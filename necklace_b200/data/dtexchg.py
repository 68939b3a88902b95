"""Data exchanger between workers (reference: necklace/data/dtexchg.py:3-9, a stub whose
``exchange`` does nothing).  Here ``exchange`` calls the function it was given."""


class DataExchanger(object):
    def __init__(self, cfg=None, exchange_fn=None):
        self.cfg = cfg or {}
        self.exchange_fn = exchange_fn

    def exchange(self, *args, **kwargs):
        if self.exchange_fn is None:
            return None
        return self.exchange_fn(*args, **kwargs)
