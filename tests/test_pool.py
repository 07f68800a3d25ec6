"""max_pool2d as one kernel each way (EB200_K_MAXPOOL2D): the oracle's loop nests against
torch on the CPU, the front end's fused op against its strided-view spelling, and the
planner's classification.  The GPU runs are in test_gpu_pool.py."""
import ctypes as C

import numpy as np
import pytest
import torch
import torch.nn.functional as TF

from harp_b200 import capi
from harp_b200 import desc as D
from harp_b200.frontend import Program, Tensor
from oracle import c_emit as O
from oracle.executor import OracleExecutor

SHAPES = [(6, 26, 26, 2), (5, 11, 11, 2), (3, 13, 10, 2), (4, 9, 10, 3), (2, 8, 13, 4), (1, 2, 2, 2), (7, 5, 4, 1)]


def pool_inputs(p, h, w, k, seed=0, ties=True):
    rng = np.random.default_rng(seed)
    # small integers: many equal taps inside a window, zeros and negatives for the ReLU mask
    x = (rng.integers(-3, 4, (p, h, w)) if ties else rng.standard_normal((p, h, w))).astype(np.float32)
    g = rng.standard_normal((p, h // k, w // k)).astype(np.float32)
    return x, g


@pytest.mark.parametrize("p,h,w,k", SHAPES)
@pytest.mark.parametrize("relu", [False, True])
def test_oracle_pool_matches_torch(p, h, w, k, relu):
    x, g = pool_inputs(p, h, w, k, ties=False)       # distinct values: torch sends the gradient to ONE maximum
    y = O.run(D.maxpool2d(p, h, w, k, relu), [x])
    xt = torch.tensor(x[None], requires_grad=True)
    yt = TF.max_pool2d(TF.relu(xt) if relu else xt, k)
    assert (y.reshape(p, h // k, w // k) == yt[0].detach().numpy()).all()
    gx = O.run(D.maxpool2d(p, h, w, k, relu, grad=True), [g, x, y])
    yt.backward(torch.tensor(g[None]))
    ref = xt.grad[0].numpy()
    if relu:
        # at windows whose taps are all <= 0 the maximum 0 is shared by every tap: eclat's mask gives each
        # the gradient before the ReLU's own mask removes the negative ones; torch picks one tap
        keep = np.repeat(np.repeat(y.reshape(p, h // k, w // k) > 0, k, 1), k, 2)
        full = np.zeros((p, h, w), bool)
        full[:, :keep.shape[1], :keep.shape[2]] = keep
        assert (gx.reshape(p, h, w)[full] == ref[full]).all()
        assert (gx.reshape(p, h, w)[x < 0] == 0).all()
    else:
        assert (gx.reshape(p, h, w) == ref).all()


@pytest.mark.parametrize("n,c,h,w,k", [(2, 3, 11, 11, 2), (2, 2, 8, 12, 2), (1, 2, 9, 7, 3)])
def test_fused_pool_equals_the_strided_view_spelling(n, c, h, w, k):
    rng = np.random.default_rng(5)
    xv = rng.integers(-2, 3, (n, c, h, w)).astype(np.float32)     # ties and zeros on purpose
    wv = rng.standard_normal((n, c, h // k, w // k)).astype(np.float32)

    def run(fused):
        x = Tensor.input(xv, requires_grad=True)
        x2 = x * 1.5                                                  # a producer in front, a consumer behind
        y = x2.max_pool2d_fused(k, relu=True) if fused else x2.relu().max_pool2d(k)
        loss = (y * Tensor.input(wv)).sum()
        (gx,) = loss.backward([x])
        p = Program([loss, y, gx], OracleExecutor(), fuse="chains")
        p.run()
        return [p.fetch(t) for t in (loss, y, gx)], p
    a, pa = run(True)
    b, _ = run(False)
    for u, v in zip(a, b):
        assert u.tobytes() == v.tobytes()
    assert sum(d.kclass == D.K_MAXPOOL2D for d in pa.kernel_descs()) == 2


def test_planner_serves_pool_descriptors_and_rejects_bad_ones():
    def query(k):
        info = D.CKernelInfo()
        cd = k.to_c()
        capi.call("eb200_kernel_query", C.byref(cd), 148, C.byref(info))
        return info
    i = query(D.maxpool2d(4096 * 32, 26, 26, 2, relu=True))
    assert i.impl.decode() == "maxpool2d_k2_relu" and i.launches == 1 and i.specialised == 1
    assert i.algo_bytes == 4 * (4096 * 32 * 26 * 26 + 4096 * 32 * 13 * 13)
    i = query(D.maxpool2d(64, 11, 11, 2, relu=False, grad=True))
    assert i.impl.decode() == "maxpool2d_k2_grad"
    assert i.algo_bytes == 4 * (2 * 64 * 25 + 64 * 100 + 64 * 121)
    with pytest.raises(capi.Eb200Error) as e:                     # window larger than the kernels carry
        query(D.maxpool2d(4, 16, 16, 5))
    assert e.value.status == capi.ERR_UNSUPPORTED
    k = D.maxpool2d(4, 16, 16, 2, grad=True)
    k.inputs[1].numel -= 1                                        # x one element short
    with pytest.raises(capi.Eb200Error) as e:
        query(k)
    assert e.value.status == capi.ERR_BOUNDS
