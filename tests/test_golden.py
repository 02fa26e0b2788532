"""The CPU oracle against the fixtures that the reference's own reference.py produced.

This is what pins the oracle on machines where the reference checkout is absent.  The expected
agreement is bit-exact: the oracle issues the same torch operations in the same order, so any
difference means the port drifted from reference.py.
"""

import numpy as np
import pytest
import torch

from golden_cases import CASES
from runners import assert_same_inputs, build_inputs, golden_state_sample, load_golden, run_oracle

# the full-size cases that the CPU suite can afford; the rest run with the GPU tests
CPU_HEAVY = {"moe_35b_bf16_b1_s0", "moe_35b_bf16_b8_s0", "dense_27b_bf16_b1", "attn_35b_bf16_t32768",
             "linear_35b_bf16_b1"}
CPU_CASES = [c for c in CASES if (not c.heavy) or c.name in CPU_HEAVY]


@pytest.mark.parametrize("case", CPU_CASES, ids=lambda c: c.name)
def test_oracle_matches_reference_fixture(case):
    golden = load_golden(case.name)
    spec = build_inputs(case)
    assert_same_inputs(case, spec, golden)
    got = run_oracle(case, spec)
    if case.op == "linear":
        steps = golden["out_steps"].tolist()
        for slot, si in enumerate(steps):
            np.testing.assert_array_equal(got["outs"][si].float().numpy(), golden["outs"][slot])
        np.testing.assert_allclose(np.asarray(got["state_norms"]), golden["state_norms"], rtol=1e-12)
        np.testing.assert_array_equal(golden_state_sample(got["state"]), golden["state_sample"])
        return
    np.testing.assert_array_equal(got["out"].float().numpy(), golden["out"])
    if case.op == "moe":
        np.testing.assert_array_equal(got["indices"].numpy(), golden["indices"])
        np.testing.assert_array_equal(got["weights"].numpy(), golden["weights"])


def test_every_case_has_a_fixture():
    for case in CASES:
        g = load_golden(case.name)
        assert "fingerprint" in g and len(g["fingerprint"]) >= 1
