"""The lm_head restatement (oracle/head.py) against what the reference's own definitions gave on the seeded inputs (tests/golden
section ``lm_head``, made by tests/golden/make_golden.py from monolith/nn/oracle.py linear + rms_norm). Floating-point contraction:
the sums are formed in another order, so a logit may sit one BF16 unit from the reference's where the sum falls next to a
rounding boundary; nothing more, and almost all are equal."""
import json
import os

import numpy as np

from oracle import head
from tests.golden.make_golden import lm_head_inputs

HERE = os.path.dirname(os.path.abspath(__file__))


def golden_codes(section, key):
    return np.frombuffer(bytes.fromhex(section[key]), dtype=np.uint16).reshape(section["rows"], section["vocab"])


def close_enough(got, want):
    return head.close(got, want)


def test_oracle_equals_the_reference_outputs():
    with open(os.path.join(HERE, "golden", "reference_outputs.json")) as f:
        g = json.load(f)["lm_head"]
    x, w, gamma = lm_head_inputs(g["seed"], g["rows"], g["hidden"], g["vocab"])
    assert close_enough(head.lm_head(x, w), golden_codes(g, "plain"))
    assert close_enough(head.lm_head(x, w, gamma, g["eps"], True), golden_codes(g, "norm_one_plus"))
    assert close_enough(head.lm_head(x, w, gamma, g["eps"], False), golden_codes(g, "norm_plain_weight"))
    assert not close_enough(head.lm_head(x, w), golden_codes(g, "norm_one_plus"))          # (the check can fail)
