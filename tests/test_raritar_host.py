"""Host-side parts of the Raritar design that need no GPU: the configuration reader, the frequency table, the registry, the
pool's layout for layers with several kinds of state, and the oracle's own consistency (a sequence recomputed from its first
token must not depend on what follows a position)."""
import math

import pytest
import torch

from tests import raritar_oracle as O


def test_config_reader_and_registry():
    from promptcache_b200.model import MODEL_REGISTRY
    from promptcache_b200.model.raritar import RaritarConfig
    assert "Raritar" in MODEL_REGISTRY and "Mutolix" in MODEL_REGISTRY
    cfg = RaritarConfig(O.make_config([O.attn_layer(), O.attn_layer(kv_from=0, mlp=False)], width=48, taps=3))
    assert (cfg.width, cfg.taps, cfg.num_hidden_layers, cfg.residual_mult) == (48, 3, 2, 0.6)
    assert cfg.layers[1]["mixer"]["kv_from"] == 0 and cfg.layers[1]["mlp"] is None
    bad = O.make_config([O.attn_layer()])
    bad["layers"][0]["type"] = "conv"
    with pytest.raises(ValueError):
        RaritarConfig(bad)
    bad = O.make_config([O.attn_layer()])
    bad["layers"][0]["mlp"]["kind"] = "dense"
    with pytest.raises(ValueError):
        RaritarConfig(bad)


def test_frequency_table():
    from promptcache_b200.model.raritar import scaled_frequencies
    plain = scaled_frequencies(16, 10000.0, None)
    assert plain == pytest.approx([10000.0 ** (-2 * i / 16) for i in range(8)])
    sc = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    got = scaled_frequencies(16, 10000.0, sc)
    assert got == pytest.approx(O.rotary_frequencies(16, 10000.0, sc), rel=1e-14)
    for f, g in zip(plain, got):
        wl = 2 * math.pi / f
        if wl < 16:
            assert g == f
        elif wl > 64:
            assert g == pytest.approx(f / 8)
        else:
            assert f / 8 <= g <= f
    assert scaled_frequencies(0, 10000.0, sc) == []


def test_pool_layout_for_layers_with_several_states():
    from promptcache_b200.model._state import ConvTailSpec, KVSpec, SeqState, SlotPool
    pool = SlotPool([(KVSpec(2, 8, 4), ConvTailSpec(4, 16)), (ConvTailSpec(4, 16),), None], torch.float32, "cpu", n_slots=1, cap=128)
    assert set(pool.layers[0]) == {"k", "v", "tail"} and set(pool.layers[1]) == {"tail"} and pool.layers[2] == {}
    assert tuple(pool.layers[0]["tail"].shape) == (1, 2, 3, 16)
    a = SeqState(pool)
    pool.layers[0]["tail"][a.slot] = 5.0
    pool.layers[0]["k"][a.slot, :, :3] = 2.0
    b = SeqState(pool)                       # the pool doubles; what live slots hold is carried over
    assert pool.n_slots == 2 and float(pool.layers[0]["tail"][a.slot].min()) == 5.0 and float(pool.layers[0]["k"][a.slot, :, :3].min()) == 2.0
    pool.reserve(b.slot, 300)
    assert pool.cap >= 300 and float(pool.layers[0]["k"][a.slot, :, :3].min()) == 2.0
    assert (a.steps, a.last_token) == (0, -1)
    a.free()
    assert SeqState(pool).slot == 0          # a freed slot is handed out again


def test_oracle_is_causal_and_windowed():
    cfg = O.make_config([O.attn_layer(window=5, keep_first=1), O.attn_layer(kv_from=0, window=3, keep_first=0)], width=24)
    W = O.random_model(cfg, seed=1)
    toks = [3, 9, 27, 20, 1, 2, 3, 4, 5, 6, 7, 8]
    full = O.forward(cfg, W, toks)
    assert torch.allclose(O.forward(cfg, W, toks[:7]), full[:7], atol=1e-12)
    assert O.visible(10, 6, 5, 1) and not O.visible(10, 5, 5, 1) and O.visible(10, 0, 5, 1) and not O.visible(10, 1, 5, 1)
    assert not O.visible(3, 4, 5, 1)
    assert O.bigram_rows([4, 5, 6], 11, 29, 5) == [11, (4 * 29 + 5 * 5) % 11, (5 * 29 + 6 * 5) % 11]
    z = torch.tensor([0.1, 2.0, 0.3, 1.9, -1.0, 0.0], dtype=O.F64)
    chosen, w = O.route(z, torch.zeros(6, dtype=O.F64), 2, 3, 1)
    assert chosen == [1, 0]                  # only the best group (outputs 0, 1) can be chosen, although output 3 scores higher than 0
    assert float(sum(w)) < 1.0               # the weights are plain scores, not renormalised
