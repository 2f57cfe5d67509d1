"""Distributions as cells (see the package docstring)."""
from __future__ import annotations

import torch
import torch.distributions as D

from ...ops.primitive import _wrap_out
from ..cell import Cell

__all__ = ["Distribution", "Normal", "Bernoulli", "Categorical", "Uniform", "Exponential", "Gamma", "Beta", "Poisson",
           "Geometric", "Cauchy", "LogNormal", "Gumbel", "Logistic", "HalfNormal", "StudentT", "Laplace",
           "TransformedDistribution"]


def _t(x):
    if x is None:
        return None
    return x.float() if isinstance(x, torch.Tensor) else torch.as_tensor(x, dtype=torch.float32)


class Distribution(Cell):
    """Base: subclasses name their parameters in ``_param_names`` and build the torch distribution in ``_make``."""
    _param_names = ()

    def __init__(self, *values, seed=None, dtype=torch.float32, name=None):
        super().__init__()
        self.dtype, self.seed = dtype, seed
        self.name = name or type(self).__name__
        self._defaults = dict(zip(self._param_names, values))
        self._check(self._defaults)

    def _check(self, params):
        pass

    def _make(self, **p):
        raise NotImplementedError

    def _dist(self, args):
        vals = dict(self._defaults)
        for k, v in zip(self._param_names, args):
            if v is not None:
                vals[k] = v
        missing = [k for k, v in vals.items() if v is None]
        if missing:
            raise ValueError("%s: parameters %s were given neither at construction nor at the call" % (self.name, missing))
        self._check(vals)
        return self._make(**{k: _t(v) for k, v in vals.items()})

    # ------------------------------------------------------------------ public functions
    def prob(self, value, *args):
        return _wrap_out(torch.exp(self._dist(args).log_prob(_t(value))))

    def log_prob(self, value, *args):
        return _wrap_out(self._dist(args).log_prob(_t(value)))

    def cdf(self, value, *args):
        return _wrap_out(self._dist(args).cdf(_t(value)))

    def log_cdf(self, value, *args):
        return _wrap_out(torch.log(self._dist(args).cdf(_t(value))))

    def survival_function(self, value, *args):
        return _wrap_out(1 - self._dist(args).cdf(_t(value)))

    def log_survival(self, value, *args):
        return _wrap_out(torch.log1p(-self._dist(args).cdf(_t(value))))

    def mean(self, *args):
        return _wrap_out(self._dist(args).mean)

    def mode(self, *args):
        return _wrap_out(self._dist(args).mode)

    def var(self, *args):
        return _wrap_out(self._dist(args).variance)

    def sd(self, *args):
        return _wrap_out(self._dist(args).stddev)

    def entropy(self, *args):
        return _wrap_out(self._dist(args).entropy())

    def sample(self, shape=(), *args):
        if self.seed is not None:
            torch.manual_seed(int(self.seed))
            self.seed = None                                  # the seed fixes the first draw; later draws continue
        return _wrap_out(self._dist(args).sample(tuple(shape)))

    def kl_loss(self, dist, *args):
        """KL(self || other) where the other distribution is of type ``dist`` with the leading ``args`` as its
        parameters; the remaining args override this distribution's parameters."""
        other_cls = _BY_NAME.get(dist if isinstance(dist, str) else type(dist).__name__)
        if other_cls is None:
            raise ValueError("unknown distribution %r" % (dist,))
        n = len(other_cls._param_names)
        other = other_cls._make(other_cls, **{k: _t(v) for k, v in zip(other_cls._param_names, args[:n])})
        return _wrap_out(D.kl_divergence(self._dist(args[n:]), other))

    def cross_entropy(self, dist, *args):
        n = len(_BY_NAME[dist if isinstance(dist, str) else type(dist).__name__]._param_names)
        return _wrap_out(self.entropy(*args[n:]) + self.kl_loss(dist, *args))

    def get_dist_args(self, *args):
        vals = dict(self._defaults)
        for k, v in zip(self._param_names, args):
            if v is not None:
                vals[k] = v
        return tuple(_wrap_out(_t(vals[k])) for k in self._param_names)

    def get_dist_type(self):
        return type(self).__name__

    def construct(self, name, *args, **kwargs):
        fn = getattr(self, name, None)
        if fn is None or name.startswith("_"):
            raise ValueError("%s has no function %r" % (self.name, name))
        return fn(*args, **kwargs)


def _positive(params, *names):
    for n in names:
        v = params.get(n)
        if v is not None and bool((torch.as_tensor(v) <= 0).any()):
            raise ValueError("%s must be positive" % n)


class Normal(Distribution):
    _param_names = ("mean", "sd")

    def __init__(self, mean=None, sd=None, seed=None, dtype=torch.float32, name="Normal"):
        super().__init__(mean, sd, seed=seed, dtype=dtype, name=name)

    def _check(self, p):
        _positive(p, "sd")

    def _make(self, mean, sd):
        return D.Normal(mean, sd)


class LogNormal(Normal):
    _param_names = ("mean", "sd")

    def _make(self, mean, sd):
        return D.LogNormal(mean, sd)


class HalfNormal(Distribution):
    _param_names = ("sd",)

    def __init__(self, sd=None, seed=None, dtype=torch.float32, name="HalfNormal"):
        super().__init__(sd, seed=seed, dtype=dtype, name=name)

    def _make(self, sd):
        return D.HalfNormal(sd)


class Bernoulli(Distribution):
    _param_names = ("probs",)

    def __init__(self, probs=None, seed=None, dtype=torch.int32, name="Bernoulli"):
        super().__init__(probs, seed=seed, dtype=dtype, name=name)

    def _check(self, p):
        v = p.get("probs")
        if v is not None and bool(((torch.as_tensor(v) < 0) | (torch.as_tensor(v) > 1)).any()):
            raise ValueError("probs must be in [0, 1]")

    def _make(self, probs):
        return D.Bernoulli(probs=probs)

    def cdf(self, value, *args):
        p = self._dist(args).probs
        v = _t(value)
        return _wrap_out(torch.where(v < 0, torch.zeros_like(v * p), torch.where(v < 1, (1 - p) * torch.ones_like(v), torch.ones_like(v * p))))


class Categorical(Distribution):
    _param_names = ("probs",)

    def __init__(self, probs=None, seed=None, dtype=torch.int32, name="Categorical"):
        super().__init__(probs, seed=seed, dtype=dtype, name=name)

    def _make(self, probs):
        return D.Categorical(probs=probs)

    def prob(self, value, *args):
        return _wrap_out(torch.exp(self._dist(args).log_prob(torch.as_tensor(value).long())))

    def log_prob(self, value, *args):
        return _wrap_out(self._dist(args).log_prob(torch.as_tensor(value).long()))

    def cdf(self, value, *args):
        p = self._dist(args).probs
        return _wrap_out(torch.cumsum(p, -1)[..., torch.as_tensor(value).long()])


class Uniform(Distribution):
    _param_names = ("low", "high")

    def __init__(self, low=None, high=None, seed=None, dtype=torch.float32, name="Uniform"):
        super().__init__(low, high, seed=seed, dtype=dtype, name=name)

    def _make(self, low, high):
        return D.Uniform(low, high, validate_args=False)

    def prob(self, value, *args):
        d = self._dist(args)
        v = _t(value)
        return _wrap_out(torch.where((v >= d.low) & (v <= d.high), 1 / (d.high - d.low), torch.zeros_like(v)))


class Exponential(Distribution):
    _param_names = ("rate",)

    def __init__(self, rate=None, seed=None, dtype=torch.float32, name="Exponential"):
        super().__init__(rate, seed=seed, dtype=dtype, name=name)

    def _check(self, p):
        _positive(p, "rate")

    def _make(self, rate):
        return D.Exponential(rate)


class Gamma(Distribution):
    _param_names = ("concentration", "rate")

    def __init__(self, concentration=None, rate=None, seed=None, dtype=torch.float32, name="Gamma"):
        super().__init__(concentration, rate, seed=seed, dtype=dtype, name=name)

    def _check(self, p):
        _positive(p, "concentration", "rate")

    def _make(self, concentration, rate):
        return D.Gamma(concentration, rate)

    def cdf(self, value, *args):
        d = self._dist(args)
        return _wrap_out(torch.special.gammainc(d.concentration, d.rate * _t(value)))


class Beta(Distribution):
    _param_names = ("concentration1", "concentration0")

    def __init__(self, concentration1=None, concentration0=None, seed=None, dtype=torch.float32, name="Beta"):
        super().__init__(concentration1, concentration0, seed=seed, dtype=dtype, name=name)

    def _make(self, concentration1, concentration0):
        return D.Beta(concentration1, concentration0)


class Poisson(Distribution):
    _param_names = ("rate",)

    def __init__(self, rate=None, seed=None, dtype=torch.float32, name="Poisson"):
        super().__init__(rate, seed=seed, dtype=dtype, name=name)

    def _check(self, p):
        _positive(p, "rate")

    def _make(self, rate):
        return D.Poisson(rate)

    def cdf(self, value, *args):
        d = self._dist(args)
        return _wrap_out(torch.special.gammaincc(torch.floor(_t(value)) + 1, d.rate))


class Geometric(Distribution):
    _param_names = ("probs",)

    def __init__(self, probs=None, seed=None, dtype=torch.int32, name="Geometric"):
        super().__init__(probs, seed=seed, dtype=dtype, name=name)

    def _make(self, probs):
        return D.Geometric(probs=probs)

    def cdf(self, value, *args):
        d = self._dist(args)
        return _wrap_out(1 - (1 - d.probs) ** (torch.floor(_t(value)) + 1))


class Cauchy(Distribution):
    _param_names = ("loc", "scale")

    def __init__(self, loc=None, scale=None, seed=None, dtype=torch.float32, name="Cauchy"):
        super().__init__(loc, scale, seed=seed, dtype=dtype, name=name)

    def _make(self, loc, scale):
        return D.Cauchy(loc, scale)


class Gumbel(Distribution):
    _param_names = ("loc", "scale")

    def __init__(self, loc=None, scale=None, seed=None, dtype=torch.float32, name="Gumbel"):
        super().__init__(loc, scale, seed=seed, dtype=dtype, name=name)

    def _make(self, loc, scale):
        return D.Gumbel(loc, scale)


class Laplace(Distribution):
    _param_names = ("loc", "scale")

    def __init__(self, loc=None, scale=None, seed=None, dtype=torch.float32, name="Laplace"):
        super().__init__(loc, scale, seed=seed, dtype=dtype, name=name)

    def _make(self, loc, scale):
        return D.Laplace(loc, scale)


class Logistic(Distribution):
    _param_names = ("loc", "scale")

    def __init__(self, loc=None, scale=None, seed=None, dtype=torch.float32, name="Logistic"):
        super().__init__(loc, scale, seed=seed, dtype=dtype, name=name)

    def _make(self, loc, scale):
        base = D.Uniform(torch.zeros_like(loc + scale), torch.ones_like(loc + scale))
        return D.TransformedDistribution(base, [D.SigmoidTransform().inv, D.AffineTransform(loc, scale)])

    def mean(self, *args):
        return self.get_dist_args(*args)[0]

    def var(self, *args):
        return _wrap_out((self.get_dist_args(*args)[1] * torch.pi) ** 2 / 3)

    def sd(self, *args):
        return _wrap_out(self.get_dist_args(*args)[1] * torch.pi / 3 ** 0.5)

    def entropy(self, *args):
        return _wrap_out(torch.log(self.get_dist_args(*args)[1]) + 2)


class StudentT(Distribution):
    _param_names = ("df", "mean", "sd")

    def __init__(self, df=None, mean=0.0, sd=1.0, seed=None, dtype=torch.float32, name="StudentT"):
        super().__init__(df, mean, sd, seed=seed, dtype=dtype, name=name)

    def _make(self, df, mean, sd):
        return D.StudentT(df, mean, sd)


class TransformedDistribution(Distribution):
    """Distribution of ``bijector(x)`` with ``x ~ distribution``."""

    def __init__(self, bijector, distribution, seed=None, name="transformed_distribution"):
        Cell.__init__(self)
        self.bijector, self.distribution, self.seed, self.name = bijector, distribution, seed, name
        self._defaults = {}

    def _dist(self, args):
        return D.TransformedDistribution(self.distribution._dist(args), [self.bijector._transform()])

    def mean(self, *args):
        if getattr(self.bijector, "is_linear", False):
            return _wrap_out(self.bijector.forward(self.distribution.mean(*args)))
        raise NotImplementedError("mean of a transformed distribution is only defined for linear bijectors")


_BY_NAME = {c.__name__: c for c in (Normal, LogNormal, HalfNormal, Bernoulli, Categorical, Uniform, Exponential, Gamma,
                                    Beta, Poisson, Geometric, Cauchy, Gumbel, Laplace, Logistic, StudentT)}
