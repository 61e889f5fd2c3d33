"""The plain implementation against the reference's own logits.

tests/golden/model_golden.npz holds what the reference's Llama model (models/llama/llama_model.cpp,
driven through its prefill()/decode() calls by tests/golden/model_driver.cpp on a GPU) returned for
a tiny_a model written in 32-bit: three prompts whole, one prompt cut at every length, one prompt
in two portions through prefill_start_pos, and eight decode steps of three requests together.
tests/plain_llama.py, which every engine test is held to, has to give the same rows.

Outside this anchor, because the reference has no code for them: llama3 rope scaling (only
rope_theta is read, llama_model.cpp:183), an eps other than 1e-5 (:507), pages of another size
than 16 (:113), head_dim other than hidden / heads (:105), and one pass over prompt portions and
decode tokens together.  Those rest on the formulas, stated twice (tests/test_plain_restated.py).
"""
import os

import numpy as np
import pytest
import torch

import plain_llama
import tiny_models

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "model_golden.npz")
TOL = 1e-4          # 32-bit sums in the reference (cuBLAS SGEMM, expf) against 64-bit plain ones


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


@pytest.fixture(scope="module")
def plain_rows(tmp_path_factory, golden):
    import sys
    sys.path.insert(0, os.path.dirname(GOLDEN))
    from make_model_golden import weights_probe
    d = tiny_models.make_model_dir(str(tmp_path_factory.mktemp("golden") / "tiny_a"), "tiny_a",
                                   dtype=torch.float32)
    probe = np.array(weights_probe(d))
    assert np.allclose(probe, golden["weights_probe"], rtol=1e-12, atol=1e-12), \
        "the tiny_a weights are no longer those the golden file was made with: run make_model_golden.py again"
    cfg, w = plain_llama.load_model_dir(d)
    seqs = [[int(t) for t in row if t >= 0] for row in golden["tokens"]]
    return [plain_llama.forward_logits(cfg, w, s) for s in seqs]


@pytest.mark.parametrize("kind, rows", [("whole", 3), ("prefix", 17), ("portions", 1), ("decode", 24)])
def test_plain_implementation_gives_the_reference_logits(golden, plain_rows, kind, rows):
    pick = [i for i, k in enumerate(golden["kind"]) if k == kind]
    assert len(pick) == rows
    worst = 0.0
    for i in pick:
        r, pos = int(golden["request"][i]), int(golden["position"][i])
        ref = golden["logits"][i].astype(np.float64)
        assert np.abs(ref).max() > 0.1                       # real logits, not zeros
        d = float(np.abs(plain_rows[r][pos].numpy() - ref).max())
        worst = max(worst, d)
        assert d <= TOL, f"{kind}: request {r} position {pos}: {d:.3e}"
        assert int(plain_rows[r][pos].argmax()) == int(ref.argmax())
    assert worst > 0.0                                       # two computations, not one copied
