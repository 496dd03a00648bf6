"""The record of what bf16 activations cost (tests/golden/bf16_study.json, made on the CPU by
tests/golden/make_bf16_study.py with the restated kernels): checked for the facts the engine's choice
of fp16 rests on. The GPU side of the same record is tests/test_model_gpu.py::
test_bf16_engine_matches_its_cpu_emulation."""
import json
from pathlib import Path

from decide_b200 import check

STUDY = json.loads((Path(__file__).parent / "golden" / "bf16_study.json").read_text())


def test_study_covers_the_full_model():
    assert STUDY["made_by"] == "tests/golden/make_bf16_study.py"
    assert STUDY["bars"] == {"max_abs_dlogit": check.MAX_DLOGIT, "max_abs_dp": check.MAX_DP}
    assert len(STUDY["logits_bf16"]) == STUDY["answers"] and len(STUDY["logits_bf16"][0]) == STUDY["candidates"]
    # the restated kernels in fp32 are the gold forward (the Hugging Face model code) to rounding
    assert STUDY["fp32_restated_vs_hf_model"]["max_abs_dlogit"] < 1e-3


def test_fp16_meets_the_bars_and_bf16_does_not():
    v = STUDY["variants"]
    assert v["f16"]["meets_bars"] and v["f16"]["max_abs_dlogit_vs_fp32"] <= check.MAX_DLOGIT
    assert not v["bf16"]["meets_bars"] and v["bf16"]["max_abs_dlogit_vs_fp32"] > check.MAX_DLOGIT


def test_the_cheap_mitigation_fails_and_the_working_one_doubles_the_gemms():
    """hi + lo activations only on the projections that feed the residual (out, down) leave bf16 outside the bar;
    on every projection they restore it, at twice the tensor-core work of all GEMMs (more than the 10% worth paying)."""
    v = STUDY["variants"]
    assert not v["bf16+exact(out,down)"]["meets_bars"]
    assert v["bf16+exact(in,out,gate_up,down)"]["meets_bars"]
    extra = STUDY["extra_gemm_work_of_exact_inputs"]
    assert 0.25 < extra["out,down"] < 0.40 and extra["all"] == 1.0
