"""EB200_K_MAXPOOL2D on the GPU against the oracle's loop nests, bit for bit: window sizes
1-4, planes whose rows are and are not 8-byte aligned (64-bit and scalar accesses), planes
the windows do not cover completely, ties inside a window, the fused ReLU; and the two
pooling layers of config 4 at batch 512."""
import numpy as np
import pytest

from harp_b200 import desc as D
from oracle import c_emit as O
from test_pool import SHAPES, pool_inputs
from util import run_gpu

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("p,h,w,k", SHAPES + [(300, 28, 30, 2), (1000, 7, 7, 2)])
@pytest.mark.parametrize("relu", [False, True])
def test_pool_forward_and_gradient_match_the_oracle(dev, p, h, w, k, relu):
    for ties in (True, False):
        x, g = pool_inputs(p, h, w, k, seed=p + h, ties=ties)
        kf = D.maxpool2d(p, h, w, k, relu)
        y, kern = run_gpu(dev, kf, [x])
        assert kern.impl == f"maxpool2d_k{k}" + ("_relu" if relu else "") and kern.launches == 1
        assert y.tobytes() == O.run(kf, [x]).tobytes()
        kg = D.maxpool2d(p, h, w, k, relu, grad=True)
        gx, kern = run_gpu(dev, kg, [g, x, y])
        assert kern.impl.endswith("_grad")
        assert gx.tobytes() == O.run(kg, [g, x, y]).tobytes()


@pytest.mark.parametrize("p,h,w", [(512 * 32, 26, 26), (512 * 64, 11, 11)])
def test_pool_layers_of_config_4_at_the_8_gpu_shard(dev, p, h, w):
    rng = np.random.default_rng(7)
    x = rng.standard_normal((p, h, w)).astype(np.float32)
    g = rng.standard_normal((p, h // 2, w // 2)).astype(np.float32)
    kf, kg = D.maxpool2d(p, h, w, 2, True), D.maxpool2d(p, h, w, 2, True, grad=True)
    y, _ = run_gpu(dev, kf, [x])
    assert y.tobytes() == O.run(kf, [x], openmp=True).tobytes()
    gx, _ = run_gpu(dev, kg, [g, x, y])
    assert gx.tobytes() == O.run(kg, [g, x, y], openmp=True).tobytes()
    # size-independent properties: pooled maxima dominate their windows; the gradient mass that arrives is the
    # gradient of the windows with a positive maximum times the number of taps that attain it
    r = np.maximum(x, 0)[:, :h // 2 * 2, :w // 2 * 2].reshape(p, h // 2, 2, w // 2, 2)
    assert (y.reshape(p, h // 2, 1, w // 2, 1) >= r).all()
    hits = ((r == y.reshape(p, h // 2, 1, w // 2, 1)) & (r > 0)).sum(axis=(2, 4))
    np.testing.assert_allclose(gx.astype(np.float64).sum(), (g.astype(np.float64) * hits).sum(), rtol=1e-6)
