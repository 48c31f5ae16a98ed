"""The pipeline microbenchmark entry point runs every mode to completion (bounded waits never give up) and reports
its counters.  It measures, it has no result to compare with an oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def buffers():
    dev = torch.device("cuda:0")
    rows = torch.zeros(20000, 256, dtype=torch.float16, device=dev)
    dense = torch.zeros(27 * 256 * 256, dtype=torch.float16, device=dev)
    return rows, dense


@pytest.mark.parametrize("name,mode,sa,sb", [
    ("mma", 4, 3, 3), ("tma", 1, 3, 3), ("gather", 2, 3, 3), ("gather4", 2 | 16, 3, 3), ("independent", 7, 3, 3),
    ("coupled", 15, 3, 3), ("coupled_deep", 15, 5, 2), ("lean", 15 | 64, 3, 3), ("lean_tma", 13 | 64, 3, 3), ("coupled_gather4", 15 | 16, 3, 3), ("pair", 32, 3, 3), ("pair4", 32, 4, 4),
    ("m64", 4 | 128, 3, 3), ("store", 256, 3, 3), ("store_bulk128", 512, 3, 3), ("store_bulk512", 1024, 3, 3), ("mma_and_store", 4 | 256, 3, 3),
])
def test_modes_run(buffers, name, mode, sa, sb):
    from flexgemm_b200.kernels import cuda as K
    rows, dense = buffers
    ms, counters = K.microbench_pipeline(mode, rows, dense, iters=64, stages_a=sa, stages_b=sb)
    assert ms > 0.0
    if mode & (8 | 32):
        assert counters[4] > 0          # the MMA lane ran its loop
    K.check_status(rows.device)         # no bounded wait gave up


def test_issue_delay_shows(buffers):
    """Idle cycles of the MMA lane between two stages are not hidden by the tensor pipe's queue: 512 cycles per stage over
    256 stages must show in the launch's duration."""
    from flexgemm_b200.kernels import cuda as K
    rows, dense = buffers
    base = min(K.microbench_pipeline(4, rows, dense, iters=256)[0] for _ in range(3))
    slow = min(K.microbench_pipeline(4, rows, dense, iters=256, issue_delay=512)[0] for _ in range(3))
    assert slow > base + 0.5 * 256 * 512 / 1.965e6      # at least half of the inserted cycles (ms at 1965 MHz)


def test_rejects_bad_arguments(buffers):
    from flexgemm_b200.kernels import cuda as K
    rows, dense = buffers
    with pytest.raises(Exception):
        K.microbench_pipeline(15, rows, dense, iters=8, stages_a=7, stages_b=3)     # ring deeper than supported
    with pytest.raises(Exception):
        K.microbench_pipeline(15, rows, dense, iters=8, stages_a=6, stages_b=6)     # beyond an SM's shared memory
    with pytest.raises(Exception):
        K.microbench_pipeline(8, rows, dense, iters=8)                              # coupled without MMAs
