"""MobileNetV2-int8 end to end on the GPU against the CPU oracle, bit-exact, and the
size-independent checks used at the benchmark's full batch."""
import numpy as np
import pytest

from gpu_exec import run_graph_gpu
from oracle_exec import run_graph
from torq_b200.workloads.mobilenet_v2 import build_mobilenet_v2, synthetic_images

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("batch", [1, 3])
def test_mobilenet_v2_bit_exact(device, batch):
    g, _ = build_mobilenet_v2(batch)
    x = synthetic_images(batch)
    want = run_graph(g, [x])[0]
    got = run_graph_gpu(device, g, [x])[0]
    assert got.shape == (batch, 1000)
    assert (want == got).all(), f"{(want != got).sum()} logits differ"
    assert len(np.unique(want)) > 20


def test_mobilenet_v2_batch_independence_at_full_batch(device):
    """Batch 256 is too slow to replay on the CPU in a unit test; images are independent,
    so image i of the big batch must equal image i run alone (checked for a few i, and
    those few are checked against the oracle)."""
    batch = 256
    g, _ = build_mobilenet_v2(batch)
    x = synthetic_images(batch)
    big = run_graph_gpu(device, g, [x])[0]
    g1, _ = build_mobilenet_v2(1)
    for i in (0, 101, 255):
        want = run_graph(g1, [x[i:i + 1]])[0]
        assert (big[i:i + 1] == want).all()
    # duplicate images give duplicate rows
    x2 = x.copy()
    x2[17] = x2[3]
    big2 = run_graph_gpu(device, g, [x2])[0]
    assert (big2[17] == big2[3]).all() and (big2[3] == big[3]).all()
