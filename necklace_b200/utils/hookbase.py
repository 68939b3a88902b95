"""Base class of user hooks (reference: necklace/utils/hookbase.py:4-30).

A hook is called before or after a training event (train, epoch, data batch,
batch, batch gradients, train step) with the trainer as first argument; a
callable object is preferred over a bare function so it can keep state."""


class NklcHookBase:
    def __init__(self, net=None, ctx=None, *args, **kwargs):
        self.net = net
        self.ctx = ctx
        self.args, self.kwargs = args, kwargs

    def __call__(self, trnr=None, *args, **kwargs):
        raise NotImplementedError
