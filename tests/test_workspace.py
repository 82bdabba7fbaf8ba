"""The activation scratch by tag (no GPU needed): stable addresses, growth, views handed out again,
(the engine's settings and switches: tests/test_engine_config.py)."""
import os

import torch

from imparo_b200.parts.base import Workspace


def test_a_tag_keeps_its_address_until_it_has_to_grow():
    ws = Workspace(torch.device("cpu"))
    a = ws.get("x", (4, 8), torch.float32)
    g0 = ws.generation
    b = ws.get("x", (2, 8), torch.float32)                 # smaller: the same memory, no new generation
    assert b.data_ptr() == a.data_ptr() and ws.generation == g0
    assert ws.get("x", (4, 8), torch.float32) is a          # the same view object is handed out again
    c = ws.get("x", (16, 8), torch.float32)                # larger: the buffer moves, captured graphs are stale
    assert ws.generation == g0 + 1 and c.shape == (16, 8)
    d = ws.get("x", (4, 8), torch.float32)                 # views of the old buffer are not handed out again
    assert d.data_ptr() == c.data_ptr() and d is not a
    assert ws.get("x", (4, 8), torch.bfloat16).data_ptr() != d.data_ptr()       # a dtype has a buffer of its own


def test_small_buffers_grow_by_doubling():
    ws = Workspace(torch.device("cpu"))
    ws.get("s", (100,), torch.float32)
    ws.get("s", (101,), torch.float32)
    g = ws.generation
    ws.get("s", (190,), torch.float32)                     # within the doubled size: no move
    assert ws.generation == g
    assert ws.bytes() == 200 * 4
