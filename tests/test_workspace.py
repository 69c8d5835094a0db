"""The scratch buffers of a step: one buffer per (name, dtype) that grows and never shrinks, views handed
out again without new work, and a generation count that tells captured CUDA graphs when a buffer moved."""
import torch

from janus_b200.engine.workspace import Workspace


def test_views_are_remembered_and_share_the_buffer():
    ws = Workspace(torch.device("cpu"))
    a = ws.get("x", (4, 8), torch.float32)
    assert a.shape == (4, 8) and ws.generation == 1
    assert ws.get("x", (4, 8), torch.float32) is a                      # the same view, no new tensor
    b = ws.get("x", (2, 8), torch.float32)                              # smaller: same storage, no growth
    assert b.data_ptr() == a.data_ptr() and ws.generation == 1
    c = ws.get("x", (4, 8), torch.bfloat16)                             # another dtype is another buffer
    assert c.data_ptr() != a.data_ptr() and ws.generation == 2
    assert ws.bytes_held() == 4 * 8 * 4 + 4 * 8 * 2


def test_growth_moves_the_buffer_and_forgets_its_views():
    ws = Workspace(torch.device("cpu"))
    a = ws.get("x", (4, 8), torch.float32)
    a.fill_(1.0)
    big = ws.get("x", (16, 8), torch.float32)
    assert ws.generation == 2 and big.shape == (16, 8)
    again = ws.get("x", (4, 8), torch.float32)
    assert again is not a and again.data_ptr() == big.data_ptr()        # a view of the new buffer
    other = ws.get("y", (3,), torch.float32)
    assert ws.get("y", [3], torch.float32) is other                     # a list names the same shape
    for i in range(5000):                                               # the memory of views is bounded
        ws.get("x", (1, 1 + i % 100), torch.float32)
    assert len(ws._views) <= 4097
