"""Row-partitioned training on 2 GPUs with the dense hub region forced on every rank's partition (tensor-core product
of the rank's longest rows x the most referenced rows of the gathered table) against the single-GPU model: same bits.
Kept apart from test_gpu_multi.py, and collected after it, because this combination has not run on GPUs yet."""
import pytest

from test_gpu_multi import check_two_gpu_gcn

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("transport", ["peer", "nccl"])
def test_two_gpu_gcn_with_hub_region_matches_single_gpu(cuda, tmp_path, transport):
    check_two_gpu_gcn(tmp_path, "dealt", "global", transport, 256)
