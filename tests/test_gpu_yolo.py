"""YOLOv8n-style int8 detector on the GPU against the CPU oracle, bit-exact: exercises 3x3
stride-1/2 convolutions, the SiLU table, 5x5 max pooling, nearest 2x resize, rescaled
concat and the shortcut add in one graph."""
import numpy as np
import pytest

from gpu_exec import run_graph_gpu
from oracle_exec import run_graph
from torq_b200.workloads.yolov8n import build_yolov8n, synthetic_images

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("batch,res", [(1, 64), (2, 160)])
def test_yolov8n_bit_exact(device, batch, res):
    g, _ = build_yolov8n(batch, res)
    x = synthetic_images(batch, res)
    want = run_graph(g, [x])
    got = run_graph_gpu(device, g, [x])
    assert len(got) == 6
    for w, o in zip(want, got):
        assert w.shape == o.shape and (w == o).all(), f"{(w != o).sum()} of {w.size} differ"
        assert len(np.unique(w)) > 16
