"""Config-1 workload on the GPU against the NumPy statement of the same generator."""
import numpy as np
import pytest
import torch

from mojo_linuxperiments_b200.oracle import philox as P

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,world", [(1 << 20, 1), (1 << 20, 4), (100003, 3), (7, 1)])
def test_fill_uniform_reduce_matches_oracle_for_any_split(n, world):
    from mojo_linuxperiments_b200.ops.workload import FillReduce
    ref = P.uniform_pm1(n, 0)
    total = 0.0
    pieces = []
    for r in range(world):
        fr = FillReduce(n, world, r)
        fr.run(0)
        torch.cuda.synchronize()
        pieces.append(fr.buf.cpu().numpy())
        total += float(fr.result.item())
        fr.run(0)                                   # the arrival counter resets itself
        torch.cuda.synchronize()
    got = np.concatenate(pieces)
    assert np.array_equal(got, ref)
    assert total == float(ref.astype(np.float64).sum())        # exact: the values are multiples of 2^-23
