"""Temetar without a GPU: its configuration, its registry entry, its tensor names, its run order, and the page
book of a window that keeps a sequence's first pages."""
import json

import numpy as np
import pytest

import temetar_models as tm
from plain import temetar_plain as plain


def test_config_is_read_and_written_back():
    from abacus_b200.config import ConfigError, TemetarConfig, architecture_of
    raw, ranks = tm.config("P")
    assert architecture_of(raw).name == "Temetar"  # by the "architecture" key
    cfg = TemetarConfig.from_dict(raw)
    assert cfg.streams == 3 and cfg.loop == (1, 3, 2) and cfg.bigram == (53, 7, 13) and cfg.residual_mult == 0.8
    assert cfg.run_order() == [0, 1, 2, 1, 2, 3] == plain.run_order(4, raw["loop"])
    assert TemetarConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    att = cfg.layers[0].mixer
    assert (att.heads, att.kv_heads, att.dim, att.vdim, att.window, att.keep_first, att.rot_dims) == (4, 2, 16, 24, 12, 3, 8)
    q = TemetarConfig.from_dict(tm.config("Q")[0])
    assert q.streams is None and q.bigram is None and q.loop is None and q.layers[1].mixer.window is None
    for broken in ({"layers": []}, {"vocab": 0}, {"layers": [{"type": "mamba", "mixer": {}}]}, {"streams": 9},
                   {"loop": {"start": 2, "stop": 1, "times": 2}}):
        with pytest.raises(ConfigError):
            TemetarConfig.from_dict({**raw, **broken})


def test_spec_and_tensor_names_follow_the_configuration():
    from abacus_b200.config import TemetarConfig, get_architecture
    arch = get_architecture("Temetar")
    for name in tm.CONFIGS:
        raw, ranks = tm.config(name)
        tensors = tm.weights(name)
        cfg = arch.complete_config(TemetarConfig.from_dict(raw), {n: t.shape for n, t in tensors.items()})
        for i, (ra, rg) in ranks.items():
            assert (cfg.layers[i].mixer.decay_rank, cfg.layers[i].mixer.gate_rank) == (ra, rg)
        spec = cfg.to_spec()
        expected, _ = arch.tensor_names(spec, None)
        assert {n: tuple(s) for n, s in expected.items()} == {n: t.shape for n, t in tensors.items()}
        assert [e.layer for e in spec.schedule] == plain.run_order(len(raw["layers"]), raw.get("loop"))
        assert all(e.source is None for e in spec.schedule)  # every pass has a cache or state of its own
        assert spec.final_norm.one_plus and spec.layers[0].mixer_norm.one_plus
    spec = TemetarConfig.from_dict(tm.config("Q")[0]).with_ranks({n: t.shape for n, t in tm.weights("Q").items()}).to_spec()
    assert spec.layers[0].streams == 1 and not spec.layers[0].learned and spec.frame_spec.buckets == 0
    assert spec.layers[2].mixer.window == 70 and spec.layers[1].mixer.window is None and spec.layers[1].mixer.sink


def test_a_window_group_with_pinned_pages_keeps_the_first_and_rings_the_rest():
    from abacus_b200.cache.pages import PageBook
    book = PageBook(n_pages=16, tokens_per_page=64, ring_pages=2, pinned_pages=1)
    book.open(0)
    assert book.pages_for(10) == 1 and book.pages_for(64 * 3) == 3 and book.pages_for(64 * 40) == 3
    added = book.grow(0, 64 * 40)
    assert [logical for logical, _ in added] == [0, 1, 2] and book.pages.n_free == 13
    assert book.grow(0, 64 * 80) == []
    book.close(0)
    assert book.pages.n_free == 16
    plain_ring = PageBook(n_pages=16, tokens_per_page=64, ring_pages=2)
    assert plain_ring.pages_for(64 * 40) == 2


def test_the_plain_mechanisms_agree_with_their_definitions_on_small_cases():
    """The oracle's own pieces on cases worked by hand."""
    # the window with kept first keys: position 9, window 3, keep 2 sees 0, 1 and 7, 8, 9
    assert list(np.nonzero(plain.visible(10, 3, 2)[9])[0]) == [0, 1, 7, 8, 9]
    assert list(np.nonzero(plain.visible(10, 3, 0)[2])[0]) == [0, 1, 2]
    # the sink takes its share: one key with score 0 and a sink of 0 -> weight 1/2
    w = plain.softmax_with_sink(np.zeros((1, 1, 1)), np.zeros(1), np.ones((1, 1), dtype=bool))
    assert abs(w[0, 0, 0] - 0.5) < 1e-7
    # the convolution: taps (a, b), last column the current token's
    y = plain.short_convolution(np.array([[1.0], [2.0], [3.0]]), np.array([[10.0, 1.0]]))
    assert y[:, 0].tolist() == [1.0, 12.0, 23.0]
    # the delta rule writes what it reads back: one key channel, no decay, b = 1 -> o = v k q
    o = plain.delta_recurrence(np.ones((2, 1, 1)), np.ones((2, 1, 1)), np.array([[[2.0]], [[5.0]]]), np.ones((2, 1, 1)),
                               np.ones((2, 1)))
    assert o[:, 0, 0].tolist() == [2.0, 5.0]
    # the pair table: first token takes the last row
    x = plain.embedding([3, 4], np.eye(6), 2.0, np.arange(8.0)[:, None] * np.ones((8, 6)), {"buckets": 7, "mul_prev": 2, "mul_cur": 3})
    assert x[0, 3] == 2.0 + 7.0 and x[1, 4] == 2.0 + (3 * 2 + 4 * 3) % 7
