"""``nn.extend``: the layers under their extend-namespace names (``Linear``, ``Embedding``, ``MaxPool2d``,
``LayerNorm``, ...); every name resolves to the class of ``nn``.  Parity: mindspore/python/mindspore/nn/extend/."""


def __getattr__(name):
    if name.startswith("__"):
        raise AttributeError(name)
    from .. import nn
    try:
        return getattr(nn, name)
    except AttributeError:
        raise AttributeError("module 'nn.extend' has no attribute %r" % name)
