"""The plain sampler against the reference's own sampler.

tests/golden/sampler_golden.json holds histograms of tokens drawn by the reference's
core/src/sampling.cpp (built and run by tests/golden/make_sampler_golden.py).  The reference seeds
its generator from the machine, so the comparison is of distributions: what it drew must have
probability in the plain sampler, what the plain sampler finds likely must have been drawn, and
the frequencies must agree within the spread of that many draws."""
import json
import math
import pathlib

import numpy as np
import pytest

from plain_llama import sample_distribution_plain

GOLDEN = json.loads((pathlib.Path(__file__).parent / "golden" / "sampler_golden.json").read_text())


def driver_logits(case, vocab):
    """The generator of tests/golden/sampler_driver.cpp, in 32-bit arithmetic."""
    state = (12345 + 977 * case) & 0xFFFFFFFF
    out = []
    for _ in range(vocab):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        out.append(float(np.float32(np.float32((state >> 16) / 65536.0) * np.float32(8.0))
                         - np.float32(4.0)))
    return out


@pytest.mark.parametrize("case", GOLDEN["cases"], ids=lambda c: f"case{c['case']}")
def test_plain_sampler_matches_reference_histogram(case):
    vocab = GOLDEN["vocab"]
    logits = driver_logits(case["case"], vocab)
    prev = [(7 * i + 3 * case["case"]) % vocab for i in range(case["n_prev"])]
    probs = sample_distribution_plain(
        logits, float(np.float32(case["temperature"])), case["top_k"], float(np.float32(case["top_p"])),
        float(np.float32(case["repetition_penalty"])), prev)
    hist, n = case["hist"], case["draws"]
    assert sum(hist) == n
    if case["temperature"] == 0:
        assert hist.index(1) == probs.index(1.0)
        return
    for tok in range(vocab):
        p, f = probs[tok], hist[tok] / n
        if hist[tok]:
            assert p > 0, f"reference drew token {tok}, which the plain sampler masks"
        if p > 30.0 / n:
            assert hist[tok], f"token {tok} has probability {p:.4f} but was never drawn"
        assert abs(f - p) <= 5.0 * math.sqrt(max(p * (1 - p), 1.0 / n) / n) + 1.0 / n, \
            f"token {tok}: drawn {f:.5f}, plain {p:.5f}"


def test_golden_covers_every_option():
    cases = GOLDEN["cases"]
    assert any(c["top_k"] > 0 and c["top_p"] < 1 and c["repetition_penalty"] != 1 and c["temperature"] > 0
               for c in cases)
    assert any(c["temperature"] == 0 and c["repetition_penalty"] != 1 for c in cases)
    assert any(c["top_k"] >= GOLDEN["vocab"] for c in cases)
