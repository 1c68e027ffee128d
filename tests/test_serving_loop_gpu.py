"""The stand-in serving loop (tests/serving_loop.py) at a small size: two decoder layers, two bursts of two
steps, both launch modes.  Checks that the attention inside the model matches fp32 attention over every sampled
request's token list, that the captured step is replayed across the re-plan between the bursts, and that
nothing was flagged on the device."""
import pytest

import serving_loop

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", ["three_level", "chains_32x4"])
def test_serving_loop_small(shape):
    res = serving_loop.main(["--shape", shape, "--layers", "2", "--steps", "2", "--bursts", "2", "--mode", "both"])
    assert len(res) == 1
    r = res[0]
    assert r["parity_ok"], r
    assert r["device_status"] == 0
    assert r["step_us_eager"] > 0 and r["step_us_graph"] > 0 and r["attention_us_per_step_eager"] > 0
