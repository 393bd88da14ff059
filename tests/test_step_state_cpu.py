"""The StepState layout against the reference's golden offsets (its tests/contract/test_step_state.py:7-21, re-derived by
running the reference's StepStateLayout: tests/golden/reference_outputs.json). No GPU."""
import pytest

from lithos_metal_b200.step_state import StepStateLayout
from oracle import spec_models


def test_layout_is_the_reference_layout(golden):
    L = StepStateLayout(t_max=8, gamma_max=7)
    assert L.offsets == golden["step_state"]["offsets_8_7"]
    assert L.size == golden["step_state"]["size_8_7"] == 176 and L.size % 16 == 0
    assert L.counts["draft_tokens"] == 7 and L.counts["pending_tokens"] == 8


def test_pack_unpack_roundtrip():
    L = StepStateLayout(t_max=4, gamma_max=3)
    vals = {"step": 7, "t_this_step": 3, "pending_tokens": [11, 12, 13], "confidence": [0.5, 0.25, 0.125], "anchor": -1, "done": 0, "ring_head": 9}
    data = L.pack(vals)
    assert len(data) == L.size
    back = L.unpack(data)
    assert back["step"] == 7 and back["pending_tokens"] == [11, 12, 13, 0] and back["anchor"] == -1
    assert back["confidence"] == [0.5, 0.25, 0.125]
    with pytest.raises(ValueError):
        L.pack({"pending_tokens": [1, 2, 3, 4, 5]})
    with pytest.raises(ValueError):
        StepStateLayout(t_max=2, gamma_max=4)
    assert StepStateLayout(t_max=1, gamma_max=0).counts["draft_tokens"] == 1


def test_python_models_cover_the_golden_accept_cases(golden):
    for case, g in golden["accept_scan"].items():
        got, writes, log = spec_models.accept_scan(g["state"], g["tokens"], g["ring_cap"], g["eos"], g["ctx_cap"])
        assert got == g["expect"], case
        if not got["error"]:
            committed = got["position"] - g["state"]["position"] - (g["state"]["t_this_step"] - 1 - g["state"]["verify_len"])
            assert log == (committed << 16) | (g["state"]["verify_len"] << 8) | got["accepted"], case
