"""Random Movarax configurations through the engine against the plain model, in float32: unequal prompts over page and
chunk borders in one batch, decoded together to their ends, then the same prompts again from a captured graph."""
import numpy as np
import pytest

import movarax_models as mm
from helpers import assert_logits
from plain import movarax_plain as plain

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", range(14))
def test_a_random_configuration_follows_the_plain_model(tmp_path, case):
    from abacus_b200.engine import Engine, load_model
    rng = np.random.default_rng(4000 + case)
    raw = mm.random_config(rng)
    mm.CONFIGS["fuzz"] = raw
    try:
        folder, _, tensors = mm.write_folder(tmp_path, "fuzz", seed=case)
    finally:
        del mm.CONFIGS["fuzz"]
    engine = Engine(load_model(folder, "float32"), max_tokens=64 * 16)
    lens, cut = [200, 1, 70], [150, 1, 66]
    seqs = [[int(t) for t in rng.integers(0, raw["vocab"], n)] for n in lens]
    oracle = []
    for s in seqs:
        want = plain.forward(raw, tensors, s)
        oracle.append((want, float(np.abs(want - plain.forward(raw, tensors, s, real=np.float64)).max())))
    slots = [engine.open() for _ in seqs]
    first = engine.step([(slot, s[:c], [c - 1]) for slot, s, c in zip(slots, seqs, cut)]).cpu().numpy()
    for i, (want, noise) in enumerate(oracle):
        assert_logits(first[i:i + 1], want[cut[i] - 1:cut[i]], "float32", f"case {case}: prompt {i} of {raw}", noise)
    step = 0
    while True:
        live = [i for i in range(len(seqs)) if cut[i] + step < lens[i]]
        if not live:
            break
        got = engine.step([(slots[i], [seqs[i][cut[i] + step]], [0]) for i in live]).cpu().numpy()
        for j, i in enumerate(live):
            assert_logits(got[j:j + 1], oracle[i][0][cut[i] + step:cut[i] + step + 1], "float32",
                          f"case {case}: request {i} at {cut[i] + step} of {raw}", oracle[i][1])
        step += 1
    for slot in slots:
        engine.close(slot)
    for _ in range(2):  # the second sighting of a shape of prompts is captured as a graph, the third replays it
        slots = [engine.open() for _ in seqs]
        again = engine.step([(slot, s[:c], [c - 1]) for slot, s, c in zip(slots, seqs, cut)]).cpu().numpy()
        for slot in slots:
            engine.close(slot)
        np.testing.assert_array_equal(again, first)
    engine.check_status()
