"""``torch.ops.mlcg.*``: the operator names and schemas mlcg's native package registers (radius.cu:313-314,
exclusion_pairs.cpp:64-65), and ``exclusion_pair_to_ptr`` against the reference's own compiled code."""
import numpy as np
import pytest
import torch

import mlcg_b200
from mlcg_b200 import ops
from oracle import radius_ref, ref_runner

needs_ref = pytest.mark.skipif(not ref_runner.available(), reason="oracle/_ref/radius_kernel.so not built (python oracle/build_ref.py <mlcg checkout>)")


def test_operators_are_registered_with_the_reference_schemas():
    assert ops.REGISTERED
    assert str(torch.ops.mlcg.radius_cuda.default._schema) == "mlcg::" + ops.RADIUS_CUDA_SCHEMA
    assert str(torch.ops.mlcg.exclusion_pair_to_ptr.default._schema) == "mlcg::" + ops.EXCLUSION_PAIR_TO_PTR_SCHEMA


@needs_ref
def test_schemas_equal_those_of_the_reference_extension():
    (radius_schema, excl_schema), = ref_runner.run([{"op": "schemas"}])
    assert str(torch.ops.mlcg.radius_cuda.default._schema) == radius_schema
    assert str(torch.ops.mlcg.exclusion_pair_to_ptr.default._schema) == excl_schema


def _pair_cases():
    rng = np.random.default_rng(2)
    cases = [(np.array([[2, 1, 3, 2, 2], [1, 2, 2, 2, 3]], dtype=np.int64), 4)]          # the input of the comment at exclusion_pairs.cpp:16-18
    for n, p in [(50, 400), (7, 0), (1, 3), (300, 5000), (12, 12)]:
        cases.append((rng.integers(0, n, (2, p)).astype(np.int64), n))
    return cases


@needs_ref
def test_exclusion_pair_to_ptr_vs_reference_binary():
    """The C restatement, the package's function and the registered operator against exclusion_pairs.cpp compiled as it is."""
    cases = _pair_cases()
    results = ref_runner.run([{"op": "exclusion_pair_to_ptr", "pairs": torch.from_numpy(p), "num_nodes": n} for p, n in cases])
    for (pairs, n), (ref_xs, ref_ptr) in zip(cases, results):
        xs, y_ptr = radius_ref.exclusion_pair_to_ptr(pairs, n)
        assert xs.tolist() == ref_xs.tolist() and y_ptr.tolist() == ref_ptr.tolist()
        for fn in (mlcg_b200.exclusion_pair_to_ptr, torch.ops.mlcg.exclusion_pair_to_ptr):
            txs, tptr = fn(torch.from_numpy(pairs), n)
            assert torch.equal(txs, ref_xs) and torch.equal(tptr, ref_ptr)


def test_radius_cuda_refuses_host_tensors():
    with pytest.raises(RuntimeError, match="must be CUDA tensor"):
        torch.ops.mlcg.radius_cuda(torch.zeros(3, 3), None, 1.0, 10, True, None, None)


def test_fake_implementations_give_shapes():
    from torch._subclasses.fake_tensor import FakeTensorMode
    from torch.fx.experimental.symbolic_shapes import ShapeEnv
    with FakeTensorMode(shape_env=ShapeEnv(), allow_non_fake_inputs=True):
        x = torch.empty(5, 3, device="cuda")
        ei, dist = torch.ops.mlcg.radius_cuda(x, None, 1.0, 10, True, None, None)
        assert ei.shape[0] == 2 and ei.dtype == torch.int64 and dist.dtype == x.dtype and ei.shape[1] == dist.shape[0]
        xs, ptr = torch.ops.mlcg.exclusion_pair_to_ptr(torch.empty(2, 7, dtype=torch.long), 4)
        assert tuple(xs.shape) == (7,) and tuple(ptr.shape) == (5,)


@pytest.mark.gpu
def test_registered_radius_cuda_equals_the_package_function():
    gen = torch.Generator().manual_seed(0)
    x = (torch.rand(300, 3, generator=gen) * 8).cuda()
    ptr = torch.tensor([0, 100, 100, 300], device="cuda")
    pairs = torch.randint(0, 300, (2, 500), generator=gen).cuda()
    xs, yptr = torch.ops.mlcg.exclusion_pair_to_ptr(pairs, 300)
    for args in ((x, ptr, 2.5, 16, True, None, None), (x, None, 2.0, 1000, False, None, None), (x, ptr, 2.5, 8, True, xs, yptr)):
        a = torch.ops.mlcg.radius_cuda(*args)
        b = mlcg_b200.radius_cuda(*args)
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
