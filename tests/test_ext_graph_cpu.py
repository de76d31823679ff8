"""The runner's graph binding on the reference's own "cpu:float" context (no GPU needed): a
ResNet-18 built with nnabla's CgVariable / CgFunction / connect() and run by CgVariable::forward
gives the logits of the same functions called one by one, with and without clear_buffer."""
import numpy as np
import pytest

from nnabla_b200 import nbla_graph, resnet18
from oracle import ops, ref

pytestmark = pytest.mark.skipif(not (nbla_graph.available() and ref.available()),
                                reason="runner / reference CPU library not built")


def test_graph_engine_on_cpu_context_matches_function_by_function():
    rng = np.random.RandomState(0)
    params = resnet18.init_parameters(rng, num_classes=100)
    x = rng.randn(2, 3, 64, 64).astype(np.float32)
    cz = lambda w, shape=None: np.zeros(shape or w.shape, np.float32)
    g = nbla_graph.Graph("cpu:float")
    xv = g.variable(x)
    y = resnet18.Runner(g, params, cz, None, fixed_point_hint=False)(xv)
    assert y.shape == (2, 100)
    want = resnet18.Runner(ops.reference(), params, cz, None, fixed_point_hint=False)(x)
    for clear in (True, False, True):
        g.forward(y, clear_buffer=clear)
        assert np.array_equal(g.data(y), want)
    prof = g.profile(y)
    names = [n for n, _ in prof]
    assert names.count("BinaryWeightConvolution") == 19 and names.count("FixedPointQuantize") == 17
    assert names[0] == "Convolution" and names[-1] == "Affine" and all(ms >= 0 for _, ms in prof)
    # new input data, same graph
    x2 = rng.randn(2, 3, 64, 64).astype(np.float32)
    g.set_data(xv, x2)
    g.forward(y)
    assert np.array_equal(g.data(y), resnet18.Runner(ops.reference(), params, cz, None, fixed_point_hint=False)(x2))
    g.close()


def test_graph_errors_surface_as_exceptions():
    g = nbla_graph.Graph("cpu:float")
    x = g.variable(np.zeros((1, 4, 8, 8), np.float32))
    with pytest.raises(RuntimeError, match="divisible by group|group"):
        g.convolution(x, np.zeros((6, 4, 3, 3), np.float32), None, 1, (1, 1), (1, 1), (1, 1), 3)
    with pytest.raises(RuntimeError, match="unknown backend"):
        nbla_graph.Graph("cuda:float")
    g.close()
