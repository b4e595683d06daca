"""The packed layout is part of a layer's state_dict: the same bytes decode to different codes
under the two layouts, so loading tensors of the other layout must fail loudly."""
import pytest
import torch

from qfactory import QLinear, layout


def test_state_dict_carries_the_packed_layout():
    a = QLinear.empty(1, 256, 128, 4, 128, False, device="cpu", layout="tile")
    sd = a.state_dict()
    assert "_extra_state" in sd and int(sd["_extra_state"][0]) == layout.LAYOUT_TILE
    QLinear.empty(1, 256, 128, 4, 128, False, device="cpu", layout="tile").load_state_dict(sd)
    with pytest.raises(RuntimeError, match="packed-layout mismatch"):
        QLinear.empty(1, 256, 128, 4, 128, False, device="cpu", layout="fragment").load_state_dict(sd)
    # 'auto' resolves to the fragment layout for this shape: a tile checkpoint does not load into it
    with pytest.raises(RuntimeError, match="packed-layout mismatch"):
        QLinear.empty(1, 256, 128, 4, 128, False, device="cpu").load_state_dict(sd)


def test_state_dict_round_trip_keeps_the_bytes():
    g = torch.Generator().manual_seed(0)
    a = QLinear.empty(1, 256, 128, 4, 128, False, device="cpu", layout="fragment")
    a.w.copy_(torch.randint(-128, 128, a.w.shape, generator=g, dtype=torch.int8))
    b = QLinear.empty(1, 256, 128, 4, 128, False, device="cpu", layout="fragment")
    b.load_state_dict(a.state_dict())
    assert torch.equal(a.w, b.w) and b.packed_layout == layout.LAYOUT_FRAGMENT
