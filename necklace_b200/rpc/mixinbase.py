"""Empty mixin bases kept for user code that subclasses them
(reference: necklace/rpc/mixinbase.py:4-9)."""


class NodeMixin:
    def __init__(self, ndid=None, cfg=None, *args, **kwargs):
        self.ndid = ndid
        self.cfg = cfg or {}


class ServiceMixin:
    pass


# the reference's names of the two bases (necklace/rpc/mixinbase.py:4-9)
SVRMixinBase = NodeMixin
SVCMixinBase = ServiceMixin
