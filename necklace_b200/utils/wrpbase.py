"""Base class of user function wrappers such as the loss or a metric
(reference: necklace/utils/wrpbase.py:4-19): keeps complex user logic outside the
framework while giving it access to the network and the context."""


class NklcWrapperBase:
    def __init__(self, net=None, ctx=None, *args, **kwargs):
        self.net = net
        self.ctx = ctx
        self.args, self.kwargs = args, kwargs

    def __call__(self, *args, **kwargs):
        raise NotImplementedError
