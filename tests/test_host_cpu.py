"""Host-side checks of strassen_triton_b200.host that need no GPU: argument validation, the panel
split, and that the streamed product refuses to exist without a CUDA device (no CPU path)."""
import pytest
import torch

from strassen_triton_b200 import host
from strassen_triton_b200.sharded import panel_bounds


def test_panels_are_whole_tiles_and_cover_every_row():
    for rows, panels in [(16384, 16), (16384, 8), (1280, 3), (256, 8), (100, 4), (4096 + 256, 4)]:
        b = panel_bounds(rows, panels, host.HostStreamedMatmul.PANEL_QUANTUM)
        assert b[0][0] == 0 and b[-1][1] == rows
        assert all(x[1] == y[0] for x, y in zip(b, b[1:]))
        assert len(b) <= max(1, panels)
        assert all((p1 - p0) % 256 == 0 for p0, p1 in b[:-1])        # only the last panel may be ragged
        assert len({p1 - p0 for p0, p1 in b[:-1]}) <= 1              # equal panels: B's blocks are reused


def test_shape_errors_come_before_any_device_work():
    with pytest.raises(ValueError):
        host.matmul_from_host(torch.zeros(4, 4), torch.zeros(5, 4))
    with pytest.raises(ValueError):
        host.matmul_from_host(torch.zeros(4), torch.zeros(4, 4))


@pytest.mark.skipif(torch.cuda.is_available(), reason="the refusal is what a machine without a GPU shows")
def test_no_cpu_fallback():
    with pytest.raises(RuntimeError, match="no CPU path"):
        host.HostStreamedMatmul(512, 512, 512)
    with pytest.raises(RuntimeError, match="no CPU path"):
        host.matmul_from_host(torch.zeros(256, 256, dtype=torch.bfloat16), torch.zeros(256, 256, dtype=torch.bfloat16))
