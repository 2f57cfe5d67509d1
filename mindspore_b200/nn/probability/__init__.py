"""Probability: ``distribution`` (parametrised distributions as cells), ``bijector`` (invertible transforms) and
``TransformedDistribution`` (python/mindspore/nn/probability/{distribution,bijector}/*.py).  The densities come from
``torch.distributions``; the method names are MindSpore's (``prob``, ``log_prob``, ``cdf``, ``survival_function``,
``mean``, ``var``, ``sd``, ``entropy``, ``kl_loss``, ``cross_entropy``, ``sample``), each accepting the distribution
parameters again as optional call arguments."""
from . import bijector, bnn_layers, distribution  # noqa: F401
