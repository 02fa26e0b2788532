"""The CPU oracle against the fixtures that the reference's own reference.py produced.

This is what pins the oracle on machines where the reference checkout is absent.  On the machine
that generated the fixtures the agreement is bit-exact (the oracle issues the same torch
operations in the same order); on another CPU torch may choose different BLAS kernels, so the
comparison allows fp32 reassociation noise (tests/parity.py) - routing indices and the
element-wise recurrent state stay exact everywhere.
"""

import numpy as np
import pytest
import torch

from golden_cases import CASES
from parity import assert_oracle_matches_fixture
from runners import assert_same_inputs, build_inputs, golden_state_sample, load_golden, run_oracle

# the full-size cases that the CPU suite can afford; the rest run with the GPU tests
CPU_HEAVY = {"moe_35b_bf16_b1_s0", "moe_35b_bf16_b8_s0", "dense_27b_bf16_b1", "attn_35b_bf16_t32768",
             "linear_35b_bf16_b1"}
CPU_CASES = [c for c in CASES if (not c.heavy) or c.name in CPU_HEAVY]


def check_oracle_against_fixture(case, got, golden):
    if case.op == "linear":
        steps = golden["out_steps"].tolist()
        for slot, si in enumerate(steps):
            out = got["outs"][si]
            assert_oracle_matches_fixture(out, torch.from_numpy(golden["outs"][slot]).to(out.dtype), f"{case.name} step {si}")
        np.testing.assert_allclose(np.asarray(got["state_norms"]), golden["state_norms"], rtol=1e-9)
        np.testing.assert_array_equal(golden_state_sample(got["state"]), golden["state_sample"])
        return
    assert_oracle_matches_fixture(got["out"], torch.from_numpy(golden["out"]).to(got["out"].dtype), case.name)
    if case.op == "moe":
        np.testing.assert_array_equal(got["indices"].numpy(), golden["indices"])
        np.testing.assert_allclose(got["weights"].numpy(), golden["weights"], rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("case", CPU_CASES, ids=lambda c: c.name)
def test_oracle_matches_reference_fixture(case):
    golden = load_golden(case.name)
    spec = build_inputs(case)
    assert_same_inputs(case, spec, golden)
    check_oracle_against_fixture(case, run_oracle(case, spec), golden)


def test_every_case_has_a_fixture():
    for case in CASES:
        g = load_golden(case.name)
        assert "fingerprint" in g and len(g["fingerprint"]) >= 1
