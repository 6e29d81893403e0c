"""Host-side parts of the hybrid sequence models that need no GPU: configuration, registry, checkpoint files, the
page / state-slot manager, and self-checks of the float64 oracle that the GPU tests compare against."""
import json
import math
import os

import pytest
import torch

import seq_cases
import seq_oracle as O
from livecc_b200 import build as lbuild
from livecc_b200 import registry
from livecc_b200.checkpoint import iter_safetensors, read_safetensors, seq_param_specs, synthetic_seq_tensors, write_safetensors
from livecc_b200.config import SeqModelConfig
from livecc_b200.kv_cache import PAGE_SIZE, SeqCache, SeqStatePool


# ---- configuration and registry ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", sorted(seq_cases.CASES))
def test_config_round_trip(name):
    d = seq_cases.CASES[name]
    cfg = SeqModelConfig.from_json(d)
    cfg.validate()
    again = SeqModelConfig.from_json(json.loads(json.dumps(cfg.to_json())))
    assert again == cfg
    assert [L.type for L in cfg.layers] == [L["type"] for L in d["layers"]]
    assert cfg.alpha == d["postln_alpha"] and cfg.embed_scale == d["embedding"]["scale"] and cfg.eps == d["norm"]["eps"]


def test_config_rejects_what_is_not_served():
    d = json.loads(json.dumps(seq_cases.CASES["mixed"]))
    d["layers"][0]["type"] = "lstm"
    with pytest.raises(NotImplementedError):
        SeqModelConfig.from_json(d)
    d = json.loads(json.dumps(seq_cases.CASES["mixed"]))
    d["layers"][1]["mlp"]["kind"] = "experts"
    with pytest.raises(NotImplementedError):
        SeqModelConfig.from_json(d)
    d = json.loads(json.dumps(seq_cases.CASES["ssd_only"]))
    d["layers"][0]["mixer"]["groups"] = 3   # 4 heads over 3 groups
    with pytest.raises(ValueError):
        SeqModelConfig.from_json(d).validate()


def test_registry_names_the_engine_class_by_config():
    assert registry.architecture_of({"architecture": "Bimopel"}) == "Bimopel"
    assert registry.architecture_of({"architectures": ["Qwen2VLForConditionalGeneration"]}) == "Qwen2VLForConditionalGeneration"
    assert registry.architecture_of({"model_type": "qwen2_vl"}) == "qwen2_vl"
    with pytest.raises(ValueError):
        registry.architecture_of({})
    with pytest.raises(NotImplementedError):
        registry.model_class("NoSuchModel")
    assert registry.model_class("Bimopel").__name__ == "SeqLMForCausalLM"
    assert registry.model_class("qwen2_vl").__name__ == "LiveCCB200ForConditionalGeneration"


def test_build_profile_names_existing_sources():
    for prof, names in lbuild.PROFILES.items():
        for n in names:
            assert (lbuild.CSRC / f"{n}.cu").exists(), (prof, n)
        assert lbuild.lib_path(prof).name == f"liblivecc_{prof}_sm100a.so"
    assert lbuild.lib_path(None) == lbuild.LIB_PATH


# ---- checkpoint files ----------------------------------------------------------------------------------------------------
def test_safetensors_round_trip_and_synthetic_checkpoint(tmp_path):
    cfg = SeqModelConfig.from_json(seq_cases.CASES["mixed"])
    t = synthetic_seq_tensors(cfg, seed=5)
    assert set(t) == {n for n, _, _ in seq_param_specs(cfg)}
    assert all(v.dtype == torch.bfloat16 for v in t.values())
    t["table"] = torch.arange(12, dtype=torch.int32).reshape(3, 4)
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    back = dict(iter_safetensors(str(tmp_path)))
    assert set(back) == set(t)
    for k in t:
        assert back[k].dtype == t[k].dtype and torch.equal(back[k], t[k]), k
    assert dict(read_safetensors(str(tmp_path / "model.safetensors")))["table"][2, 1] == 9
    t2 = synthetic_seq_tensors(cfg, seed=5)
    assert all(torch.equal(t2[k], t[k]) for k in t2)             # a pure function of (config, seed)
    with pytest.raises(FileNotFoundError):
        list(iter_safetensors(str(tmp_path / "nothing")))


# ---- pages and state slots -----------------------------------------------------------------------------------------------
def _pool(chunks=(40,), pages=4, slots=1):
    attn = {i + 1: (2, 8, 4, c) for i, c in enumerate(chunks)}
    floats = [16] + [8] * len(chunks)
    return SeqStatePool(attn, floats, torch.float32, torch.device("cpu"), initial_pages=pages, initial_slots=slots)


def test_pages_behind_the_chunk_go_back_and_are_used_again():
    pool = _pool(chunks=(40,), pages=4)
    a = SeqCache(pool)
    a.ensure_tokens(130)                       # pages 0, 1, 2
    assert a.live_pages() == 3 and len(pool.free) == 1
    a.advance(130)                             # chunk [120, 160): positions < 120 are dead -> page 0 (0..63) goes back
    assert pool.keep_from(130) == 120 and a.pages[0] is None and a.live_pages() == 2 and len(pool.free) == 2
    b = SeqCache(pool)
    b.ensure_tokens(70)
    assert b.live_pages() == 2 and len(pool.free) == 0
    assert set(p for p in b.pages) & set(p for p in a.pages if p is not None) == set()
    a.ensure_tokens(200)                       # pool grows; old pages keep their ids and contents
    assert pool.num_pages >= 5 and a.live_pages() == 3
    assert a.page_table[:4].tolist()[1:] == a.pages[1:4]
    a.advance(70)                              # 200 tokens: chunk [200, 240) -> pages 0..2 dead
    assert a.live_pages() == 1
    a.release()
    b.release()
    assert sorted(pool.free) == list(range(pool.num_pages))


def test_two_chunk_sizes_keep_the_larger_window_and_plain_causal_keeps_all():
    pool = _pool(chunks=(10, 64))
    assert pool.keep_from(130) == 128
    assert pool.keep_from(127) == 64
    pool = _pool(chunks=(10, 0))
    assert pool.keep_from(500) == 0
    none = SeqStatePool({}, [4], torch.float32, torch.device("cpu"))
    c = SeqCache(none)
    c.ensure_tokens(1000)
    assert c.live_pages() == 0 and none.keep_from(77) == 77


def test_state_slot_is_zeroed_for_its_next_user():
    pool = _pool(slots=1)
    a = SeqCache(pool)
    pool.state[0][a.slot].fill_(3.0)
    pool.state[1][a.slot].fill_(-1.0)
    slot = a.slot
    b = SeqCache(pool)                          # second slot: the pool grows, a's state survives
    assert b.slot != slot and pool.state[0][slot].eq(3.0).all()
    a.release()
    c = SeqCache(pool)
    assert c.slot == slot and pool.state[0][slot].eq(0).all() and pool.state[1][slot].eq(0).all()
    assert pool.state_bytes_per_sequence() == 4 * 24 and pool.bytes_per_token() == 2 * (8 + 4) * 4


def test_page_table_growth_keeps_entries():
    pool = _pool(chunks=(0,), pages=2)
    a = SeqCache(pool)
    a.ensure_tokens(PAGE_SIZE * 70)
    assert a.page_table.numel() >= 70 and a.page_table[:70].tolist() == a.pages


# ---- the oracle itself -----------------------------------------------------------------------------------------------------
def test_oracle_sink_softmax_is_a_softmax_over_an_extra_zero_score():
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(9, 2, 4, generator=g, dtype=torch.float64) for _ in range(3))
    out = O.chunk_sink_attention(q, k[:, :1], v[:, :1], chunk=4, scale=0.7)
    i, h = 6, 1                                  # chunk [4, 8): keys 4, 5, 6
    s = torch.stack([q[i, h] @ k[j, 0] for j in (4, 5, 6)]) * 0.7
    p = torch.softmax(torch.cat([torch.zeros(1, dtype=torch.float64), s]), 0)[1:]
    want = sum(p[n] * v[j, 0] for n, j in enumerate((4, 5, 6)))
    assert torch.allclose(out[i, h], want, atol=1e-12)
    first = O.chunk_sink_attention(q, k[:, :1], v[:, :1], chunk=4, scale=0.7)[4, 0]   # first token of a chunk sees itself only
    e = math.exp(float(q[4, 0] @ k[4, 0]) * 0.7)
    assert torch.allclose(first, e / (1 + e) * v[4, 0], atol=1e-12)


def test_oracle_recurrences_match_their_closed_forms():
    g = torch.Generator().manual_seed(1)
    T, H, d, dv = 6, 2, 3, 4
    q, k, dec = (torch.rand(T, H, d, generator=g, dtype=torch.float64) for _ in range(3))
    v = torch.randn(T, H, dv, generator=g, dtype=torch.float64)
    o = O.gla_scan(q, k, v, dec)
    t, h = 4, 1
    want = torch.zeros(dv, dtype=torch.float64)
    for s in range(t + 1):
        w = k[s, h] * torch.stack([dec[r, h] for r in range(s + 1, t + 1)]).prod(0) if s < t else k[s, h]
        want += (q[t, h] * w).sum() * v[s, h]
    assert torch.allclose(o[t, h], want, atol=1e-12)
    x = torch.randn(T, H, dv, generator=g, dtype=torch.float64)
    B, C = (torch.randn(T, 1, d, generator=g, dtype=torch.float64) for _ in range(2))
    dt = torch.rand(T, H, generator=g, dtype=torch.float64)
    a_log, skip = torch.tensor([0.3, -0.2], dtype=torch.float64), torch.tensor([1.5, 0.5], dtype=torch.float64)
    y = O.ssd_scan(x, B, C, dt, a_log, skip, 1)
    want = skip[h] * x[t, h]
    for s in range(t + 1):
        decay = math.exp(-math.exp(float(a_log[h])) * float(dt[s + 1:t + 1, h].sum()))
        want = want + decay * float(dt[s, h]) * float(B[s, 0] @ C[t, 0]) * x[s, h]
    assert torch.allclose(y[t, h], want, atol=1e-12)


def test_oracle_convolution_pads_with_zeros_and_weights_the_current_token_last():
    x = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None]
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64)
    out = O.causal_conv_silu(x, w, torch.zeros(1, dtype=torch.float64))
    pre = torch.tensor([1.0, 12.0, 123.0, 234.0, 345.0], dtype=torch.float64)
    assert torch.allclose(out[:, 0], pre * torch.sigmoid(pre))
