"""Host-side parts of the slot-pool models (no GPU): checkpoint reader, config, slot pool, batch description, registry."""
import json
import os

import pytest
import torch

from tests import mutolix_oracle as O
from promptcache_b200 import weights as wio
from promptcache_b200._native_seq import Batch
from promptcache_b200.model._state import KVSpec, MatrixMemorySpec, SeqState, SlotPool
from promptcache_b200.model.mutolix import MutolixConfig


def test_safetensors_roundtrip(tmp_path):
    t = {"a.b": torch.randn(3, 5).to(torch.bfloat16), "s": torch.tensor(0.25, dtype=torch.bfloat16), "i": torch.arange(7, dtype=torch.int32),
         "f": torch.randn(2, 2, 2)}
    path = str(tmp_path / "m.safetensors")
    wio.save_file(t, path)
    meta, base = wio.read_header(path)
    assert set(meta) == set(t) and base % 8 == 0
    back = wio.load_file(path)
    for k, v in t.items():
        assert back[k].dtype == v.dtype and back[k].shape == v.shape and torch.equal(back[k], v)
    as32 = wio.load_file(path, dtype=torch.float32)
    assert as32["a.b"].dtype == torch.float32 and as32["i"].dtype == torch.int32


def test_safetensors_rejects_bad_files(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(ValueError):
        wio.read_header(str(p))


def test_config_reads_every_size_from_the_file():
    cfg, _ = O.random_model([O.mlstm_layer(heads=3, dim=8, vdim=24, gate_cap=7.5), O.attn_layer(heads=6, kv_heads=3, dim=8, vdim=16, every=0, ff=None)],
                            width=48, vocab=77, emb_scale=1.25, eps=3e-6)
    c = MutolixConfig(json.loads(json.dumps(cfg)))
    assert (c.vocab_size, c.width, c.embedding_scale, c.eps, c.num_hidden_layers) == (77, 48, 1.25, 3e-6, 2)
    assert c.layers[0]["mixer"]["gate_cap"] == 7.5 and c.layers[0]["mlp"] is None
    assert "q_temp" not in c.layers[1]["mixer"]
    with pytest.raises(ValueError):
        MutolixConfig({"vocab": 4, "width": 4, "layers": [{"type": "conv", "mixer": {}}]})


def test_slot_pool_reuse_and_growth():
    pool = SlotPool([KVSpec(2, 4, 6), MatrixMemorySpec(2, 4, 6)], torch.float32, "cpu", n_slots=2, cap=128)
    a, b = SeqState(pool), SeqState(pool)
    assert {a.slot, b.slot} == {0, 1} and pool.n_slots == 2
    pool.layers[0]["k"][a.slot, :, :3] = 1.0
    pool.layers[1]["s"][b.slot] = 2.0
    pool.rows[a.slot] = 3
    v0 = pool.version
    c = SeqState(pool)                       # a third sequence: the pool doubles, live content is carried over
    assert pool.n_slots == 4 and pool.version > v0 and c.slot == 2
    assert float(pool.layers[0]["k"][a.slot, :, :3].min()) == 1.0 and float(pool.layers[1]["s"][b.slot].min()) == 2.0
    pool.reserve(a.slot, 300)                # more rows per slot
    assert pool.cap >= 300 and pool.cap % 128 == 0 and float(pool.layers[0]["k"][a.slot, :, :3].min()) == 1.0
    freed = b.slot
    b.free()
    b.free()                                 # idempotent
    d = SeqState(pool)
    assert d.slot == freed and d.rows == 0   # a released slot is handed out again, empty
    del d
    assert freed not in pool.rows            # garbage collection gives the slot back


def test_slot_pool_token_limit():
    pool = SlotPool([KVSpec(1, 4, 4)], torch.float32, "cpu", max_tokens=200)
    s = SeqState(pool)
    pool.reserve(s.slot, 200)
    assert pool.cap == 256
    with pytest.raises(ValueError):
        pool.reserve(s.slot, 1000)


def test_batch_description_layout():
    b = Batch([5, 2], [0, 7], [3, 1], torch.device("cpu"))
    assert b.tok_seq.tolist() == [0, 0, 0, 1] and b.tok_pos.tolist() == [0, 1, 2, 7]
    assert b.seq_slot.tolist() == [5, 2] and b.seq_pos0.tolist() == [0, 7] and b.seq_len.tolist() == [3, 1] and b.seq_off.tolist() == [0, 3]
    assert (b.n_tokens, b.n_seqs, b.max_len) == (4, 2, 3)


def test_registry_names_the_design(tmp_path):
    from promptcache_b200.model import MODEL_REGISTRY, load_model
    assert "Mutolix" in MODEL_REGISTRY and "LlamaForCausalLM" in MODEL_REGISTRY
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Nothing"}))
    with pytest.raises(ValueError):
        load_model(str(tmp_path))


def test_oracle_recurrence_is_consistent_with_its_own_state():
    """The oracle's recurrence run whole equals the same recurrence run in two halves through its state."""
    torch.manual_seed(0)
    T, H, D, V = 9, 2, 4, 6
    q, k, v = torch.randn(T, H, D, dtype=O.F64), torch.randn(T, H, D, dtype=O.F64), torch.randn(T, H, V, dtype=O.F64)
    ig, fg = torch.randn(T, H, dtype=O.F64), -torch.rand(T, H, dtype=O.F64)
    whole, _ = O.mlstm_recurrence(q, k, v, ig, fg)
    a, st = O.mlstm_recurrence(q[:4], k[:4], v[:4], ig[:4], fg[:4])
    b, _ = O.mlstm_recurrence(q[4:], k[4:], v[4:], ig[4:], fg[4:], st)
    assert torch.allclose(torch.cat([a, b]), whole, atol=1e-12)
