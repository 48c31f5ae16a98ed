"""The seeded synthetic workloads: the torch generator of the shells (used on
the GPU for the RES=1024 batches) must give exactly the rows of the numpy one,
which is the generator the oracle shares."""
import numpy as np
import pytest

from flexgemm_b200 import workloads
from oracle import submconv_oracle as orc


@pytest.mark.parametrize("res,batch,scales", [(32, 1, None), (64, 3, [1.0, 0.8, 0.93]), (96, 2, [0.8 + 0.2 * 0.3178, 1.0]), (7, 1, None)])
def test_torch_shell_generator_matches_numpy(res, batch, scales):
    a = workloads.shell_coords(res, batch, scales)
    b = workloads.shell_coords_torch(res, batch, scales, planes_per_chunk=5).numpy()
    assert a.dtype == b.dtype == np.int32
    assert np.array_equal(a, b)
    assert np.array_equal(a, orc.shell_coords(res, batch=batch, scales=tuple(scales) if scales else None))


def test_headline_shell_size():
    assert workloads.shell_coords_torch(256).shape == (163736, 4)
