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


def test_kernels_can_tell_where_they_run():
    """Every CTA reports its SM and the rank tag it was launched with: the device-side counterpart of the host runtime's
    getcpu / rseq cross-check."""
    import torch
    from mojo_linuxperiments_b200.ops import workload as W
    props = torch.cuda.get_device_properties(0)
    tags = W.where_am_i(ctas=4 * props.multi_processor_count, rank_tag=7).cpu()
    torch.cuda.synchronize()
    assert (tags[:, 2] == 7).all() and tags[:, 3].tolist() == list(range(tags.shape[0]))
    assert (tags[:, 0] >= 0).all() and (tags[:, 0] < tags[:, 1]).all()
    assert int(tags[0, 1]) >= props.multi_processor_count
    assert tags[:, 0].unique().numel() >= props.multi_processor_count // 2      # the grid spread over the device
