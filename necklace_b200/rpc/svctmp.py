"""Service templates: node identity, the message envelope and the state queue.

Envelope (a msgpack map), identical to the reference's
(necklace/rpc/svctmp.py:63-100):

    request  {fn, role, ndid, rank, url, msg: {...kwargs}}
    reply    {fn, role, ndid, rank, url, ret, msg: {...kwargs}}

Node ids are ``svr-<rank>`` / ``cli-<rank>``.  ``TmplServer.q_put_state`` pushes
``(state, args, kwargs)`` onto the job queue that ``TmplService.check_state``
(the node's only timer) drains; endpoints therefore return at once and the work
happens on the service loop's thread.
"""
from __future__ import annotations

from . import zrpc


class TmplClient(zrpc.Client):
    def __init__(self, cfg=None):
        cfg = cfg or {}
        self.rank = cfg.get("rank") or 0
        super().__init__("cli-" + str(self.rank), cfg)


class TmplServer(zrpc.Server):
    def __init__(self, cfg=None):
        cfg = cfg or {}
        self.rank = cfg.get("rank") or 0
        self.role = cfg.get("role")
        super().__init__("svr-" + str(self.rank), cfg)
        self.state = 0

    def q_put_state(self, state, *args, **kwargs):
        self.state = state
        self.q_put(self.q, (self.state, args, kwargs))

    def mk_rpc_cli(self, cli_url, **extra):
        return TmplClient({"url": cli_url, **extra})

    def _envelope(self, fn):
        return {"fn": fn, "role": self.role, "ndid": self.ndid, "rank": self.rank,
                "url": self.url}

    def mk_rpc_msg(self, fn, *args, **kwargs):
        m = self._envelope(fn)
        m["msg"] = kwargs
        return m

    def mk_rpc_ret(self, fn, ret, *args, **kwargs):
        m = self._envelope(fn)
        m["ret"] = ret
        m["msg"] = kwargs
        return m

    def rep_err_msg(self, fn, msg):
        return self.msg_pck({"fn": fn, "ret": "err", "msg": msg})

    def do_rpc_call(self, cli, fn, *args, **kwargs):
        """Pack the envelope, call ``fn`` on ``cli`` and unpack the reply."""
        ret = self.snd_msg(cli, fn, self.msg_pck(self.mk_rpc_msg(fn, **kwargs)))
        return self.msg_unpck(ret) if isinstance(ret, (bytes, bytearray)) else ret


class TmplService(zrpc.Node):
    def __init__(self, cfg=None):
        super().__init__(cfg or {})

    def q_put_state(self, state, *args, **kwargs):
        self.svr.state = state
        self.q_put(self.svr.q, (self.svr.state, args, kwargs))

    def q_get_state(self, *args, **kwargs):
        s = self.q_get(self.svr.q if self.svr is not None else self.q, *args, **kwargs)
        if not s:
            return None, None, None
        return s

    def init_timers(self):
        self.register_timer(0, self.check_state)

    def check_state(self, *args, **kwargs):
        pass  # subclasses do all their work here
