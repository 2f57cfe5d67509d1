"""nn.probability: distributions against scipy.stats, bijectors against closed forms."""
import math

import numpy as np
import pytest
import scipy.stats as st
import torch

from mindspore_b200.nn.probability import bijector as msb
from mindspore_b200.nn.probability import distribution as msd


def test_distributions_match_scipy():
    x = np.array([0.3, 1.2, 2.5])
    cases = [
        (msd.Normal(0.5, 2.0), st.norm(0.5, 2.0)), (msd.Exponential(1.5), st.expon(scale=1 / 1.5)),
        (msd.Gamma(2.0, 3.0), st.gamma(2.0, scale=1 / 3.0)), (msd.Cauchy(0.1, 0.7), st.cauchy(0.1, 0.7)),
        (msd.Laplace(0.2, 1.3), st.laplace(0.2, 1.3)), (msd.Gumbel(0.0, 2.0), st.gumbel_r(0.0, 2.0)),
        (msd.LogNormal(0.1, 0.5), st.lognorm(0.5, scale=math.exp(0.1))), (msd.Logistic(1.0, 2.0), st.logistic(1.0, 2.0)),
        (msd.Uniform(0.0, 3.0), st.uniform(0.0, 3.0)), (msd.HalfNormal(1.5), st.halfnorm(scale=1.5)),
    ]
    for ours, ref in cases:
        np.testing.assert_allclose(ours.prob(x).numpy(), ref.pdf(x), rtol=1e-4, err_msg=ours.name)
        np.testing.assert_allclose(ours.cdf(x).numpy(), ref.cdf(x), rtol=1e-4, atol=1e-6, err_msg=ours.name)
        np.testing.assert_allclose(ours.survival_function(x).numpy(), ref.sf(x), rtol=1e-3, atol=1e-6)
        if not isinstance(ours, msd.Cauchy):
            np.testing.assert_allclose(float(ours.mean()), ref.mean(), rtol=1e-4)
            np.testing.assert_allclose(float(ours.var()), ref.var(), rtol=1e-4)
        np.testing.assert_allclose(float(ours.entropy()), ref.entropy(), rtol=1e-4, atol=1e-5)
    k = np.array([0.0, 1.0, 4.0])
    np.testing.assert_allclose(msd.Poisson(3.0).prob(k).numpy(), st.poisson(3.0).pmf(k), rtol=1e-4)
    np.testing.assert_allclose(msd.Poisson(3.0).cdf(k).numpy(), st.poisson(3.0).cdf(k), rtol=1e-4)
    np.testing.assert_allclose(msd.Geometric(0.3).cdf(k).numpy(), st.geom(0.3, loc=-1).cdf(k), rtol=1e-5)
    np.testing.assert_allclose(msd.Bernoulli(0.3).prob(np.array([0.0, 1.0])).numpy(), [0.7, 0.3], rtol=1e-6)
    c = msd.Categorical([0.2, 0.3, 0.5])
    assert abs(float(c.prob(2)) - 0.5) < 1e-6 and abs(float(c.cdf(1)) - 0.5) < 1e-6


def test_call_time_parameters_kl_and_sampling():
    n = msd.Normal()
    assert abs(float(n.log_prob(1.0, 1.0, 2.0)) - st.norm(1.0, 2.0).logpdf(1.0)) < 1e-5
    with pytest.raises(ValueError):
        n.prob(0.0)
    with pytest.raises(ValueError):
        msd.Normal(0.0, -1.0)
    kl = float(msd.Normal(0.0, 1.0).kl_loss("Normal", 1.0, 2.0))
    assert abs(kl - (math.log(2) + 2 / 8 - 0.5)) < 1e-6
    ce = float(msd.Normal(0.0, 1.0).cross_entropy("Normal", 1.0, 2.0))
    assert abs(ce - (kl + st.norm(0, 1).entropy())) < 1e-5
    a = msd.Normal(0.0, 1.0, seed=7).sample((1000,))
    b = msd.Normal(0.0, 1.0, seed=7).sample((1000,))
    assert torch.equal(a, b) and abs(float(a.mean())) < 0.15
    assert msd.Normal(0.0, 1.0)("prob", 0.0) == msd.Normal(0.0, 1.0).prob(0.0)


def test_bijectors_and_transformed_distribution():
    sa = msb.ScalarAffine(2.0, 1.0)
    assert float(sa.forward(3.0)) == 7.0 and float(sa.inverse(7.0)) == 3.0
    assert abs(float(sa.forward_log_jacobian(3.0)) - math.log(2)) < 1e-6
    assert abs(float(sa.inverse_log_jacobian(7.0)) + math.log(2)) < 1e-6
    assert float(msb.Invert(sa).forward(7.0)) == 3.0
    sp = msb.Softplus(2.0)
    assert abs(float(sp.forward(0.7)) - math.log1p(math.exp(1.4)) / 2) < 1e-6
    assert abs(float(sp.inverse(sp.forward(0.7))) - 0.7) < 1e-5
    assert abs(float(msb.PowerTransform(0.5).forward(2.0)) - 4.0) < 1e-6
    assert abs(float(msb.Exp().forward_log_jacobian(1.5)) - 1.5) < 1e-6
    g = msb.GumbelCDF(0.5, 2.0)
    assert abs(float(g.forward(1.0)) - st.gumbel_r(0.5, 2.0).cdf(1.0)) < 1e-6
    assert abs(float(g.inverse(g.forward(1.0))) - 1.0) < 1e-5
    ln = msd.TransformedDistribution(msb.Exp(), msd.Normal(0.1, 0.5))
    x = np.array([0.5, 1.0, 2.0])
    np.testing.assert_allclose(ln.prob(x).numpy(), st.lognorm(0.5, scale=math.exp(0.1)).pdf(x), rtol=1e-4)
    aff = msd.TransformedDistribution(sa, msd.Normal(0.0, 1.0))
    assert abs(float(aff.mean()) - 1.0) < 1e-6
    np.testing.assert_allclose(aff.cdf(x).numpy(), st.norm(1.0, 2.0).cdf(x), rtol=1e-4)
