"""End-to-end regression scenarios on CPU (the harness compares every iteration's loss and grad norm with a recorded
baseline; the 2-rank tensor / pipeline / expert parallel scenarios are checked against the 1-rank baselines)."""
import os

import pytest

from tests.e2e import harness

SCEN = os.path.join(os.path.dirname(__file__), "e2e", "scenarios")


@pytest.mark.parametrize("name", ["tiny_llama_pretrain.yaml", "tiny_llama_tp2_dp1.yaml", "embodied_pi05.yaml", "embodied_dreamzero.yaml",
                                  "tiny_llama_cp2.yaml", "tiny_llama_4l_pretrain.yaml", "tiny_llama_4l_pp2_vpp2.yaml",
                                  "tiny_qwen3_moe_pretrain.yaml", "tiny_qwen3_moe_tp2_ep2.yaml",
                                  "tiny_deepseek_pretrain.yaml", "tiny_deepseek_v4_pretrain.yaml", "tiny_qwen3_next_pretrain.yaml",
                                  "tiny_glm_pretrain.yaml", "tiny_minimax_pretrain.yaml", "tiny_mimo_pretrain.yaml",
                                  "tiny_llama_sft_mock.yaml", "tiny_deepseek_tp2.yaml", "tiny_deepseek_v4_pp2.yaml",
                                  "tiny_qwen3_next_tp2.yaml", "tiny_glm_pp2.yaml", "tiny_minimax_ep2.yaml"])
def test_scenario_matches_baseline(name):
    errs = harness.run(os.path.join(SCEN, name))
    assert not errs, "\n".join(errs)


def test_compare_reports_mismatches():
    base = [{"iteration": 1, "lm_loss": 10.0, "grad_norm": 1.0, "elapsed_time_ms": 100.0},
            {"iteration": 2, "lm_loss": 9.0, "grad_norm": 1.0, "elapsed_time_ms": 100.0}]
    ok = [{"iteration": 1, "lm_loss": 10.1, "grad_norm": 1.01, "elapsed_time_ms": 500.0},
          {"iteration": 2, "lm_loss": 9.05, "grad_norm": 0.99, "elapsed_time_ms": 103.0}]
    assert harness.compare(ok, base, ["lm_loss", "grad_norm", "elapsed_time_ms"]) == []
    bad = [dict(ok[0]), dict(ok[1], lm_loss=9.5, elapsed_time_ms=120.0)]
    errs = harness.compare(bad, base, ["lm_loss", "elapsed_time_ms"])
    assert len(errs) == 2 and "lm_loss" in errs[0] and "elapsed_time_ms" in errs[1]
