"""Packing helpers of the two-component layout.  Parity: python/mindspore/hypercomplex/utils.py:26,33."""
import torch

from ..common.tensor import as_tensor


def get_x_and_y(tensor):
    """The two components of a ``[2, ...]`` tensor."""
    t = tensor.as_subclass(torch.Tensor) if isinstance(tensor, torch.Tensor) else torch.as_tensor(tensor)
    if t.shape[0] != 2:
        raise ValueError("the first dimension must be 2, but got shape %s" % (tuple(t.shape),))
    return as_tensor(t[0]), as_tensor(t[1])


def to_2channel(real, imag, dtype=None):
    """Stacks two equal-shaped tensors into the ``[2, ...]`` layout."""
    r, i = torch.as_tensor(real), torch.as_tensor(imag)
    if r.shape != i.shape:
        raise ValueError("real and imag parts must have the same shape, but got %s and %s"
                         % (tuple(r.shape), tuple(i.shape)))
    out = torch.stack([r.as_subclass(torch.Tensor), i.as_subclass(torch.Tensor)])
    return as_tensor(out.to(dtype) if dtype is not None else out)
