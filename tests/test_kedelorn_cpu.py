"""Host-side parts of the Kedelorn design (no GPU): config.json parsing and validation, rotary frequency tables, the weight
layout the library reads, the registry, and the page pool of latent caches."""
import copy
import json
import math

import pytest
import torch

import kedelorn_cases as K
import kedelorn_oracle as O
from livecc_b200.checkpoint import iter_safetensors, seq_param_specs, synthetic_seq_tensors, write_safetensors
from livecc_b200.config import RotaryConfig, SeqModelConfig
from livecc_b200.kv_cache import PAGE_SIZE, SeqCache, SeqStatePool
from livecc_b200.registry import architecture_of, model_class
from livecc_b200.seq_engine import SeqWeights


@pytest.mark.parametrize("name", sorted(K.CASES))
def test_config_round_trip_and_validation(name):
    d = K.CASES[name]
    cfg = SeqModelConfig.from_json(d)
    cfg.validate()
    assert cfg.block == "prenorm_hc" and cfg.norm_offset == 1.0 and cfg.positions is None and cfg.streams == d["streams"]
    assert SeqModelConfig.from_json(cfg.to_json()) == cfg
    assert json.loads(json.dumps(cfg.to_json()))["layers"][0]["type"] == d["layers"][0]["type"]


def test_config_rejects_what_the_kernels_do_not_serve():
    d = copy.deepcopy(K.CASES["mixed"])
    d["layers"][2]["mixer"]["kv_from"] = 3                  # not an earlier latent-attention layer with its own cache
    with pytest.raises(ValueError):
        SeqModelConfig.from_json(d).validate()
    d = copy.deepcopy(K.CASES["mixed"])
    d["layers"][2]["mixer"]["kv_rank"] += 1                 # another geometry than the cache it reads
    with pytest.raises(ValueError):
        SeqModelConfig.from_json(d).validate()
    d = copy.deepcopy(K.CASES["mixed"])
    d["layers"][0]["mixer"]["decay"] = [0.5]                # one decay per head
    with pytest.raises(ValueError):
        SeqModelConfig.from_json(d).validate()
    d = copy.deepcopy(K.CASES["mixed"])
    d["layers"][0]["mlp"]["router"]["top"] = 9
    with pytest.raises(ValueError):
        SeqModelConfig.from_json(d).validate()
    d = copy.deepcopy(K.CASES["mixed"])
    d["layers"][0]["mlp"]["kind"] = "other"
    with pytest.raises(NotImplementedError):
        SeqModelConfig.from_json(d)
    d = copy.deepcopy(K.CASES["mixed"])
    d["streams"] = 9
    with pytest.raises(ValueError):
        SeqModelConfig.from_json(d).validate()


@pytest.mark.parametrize("rot", [K.rot(8, 10000.0), K.rot(6, 300.0, (4.0, 32, 8.0, 2.0)), K.rot(16, 5e5, (8.0, 1024, 32.0, 1.0)),
                                 K.rot(4, 50.0, (2.0, 16, 1.0, 1.0))])
def test_rotary_frequency_table(rot):
    freq, mag = RotaryConfig.from_json(rot).frequencies()
    want, want_mag = O.rotary_frequencies(rot)
    assert torch.allclose(torch.tensor(freq, dtype=torch.float64), want, rtol=1e-13, atol=0)
    assert mag == pytest.approx(want_mag, rel=1e-13)
    if "scaling" in rot:
        f = rot["scaling"]["factor"]
        plain = [rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)]
        assert all(p / f * (1 - 1e-12) <= x <= p * (1 + 1e-12) for x, p in zip(freq, plain))   # between interpolated and kept
        assert mag == pytest.approx(0.1 * math.log(f) + 1.0)


def test_weight_layout():
    d = K.CASES["mixed"]
    cfg = SeqModelConfig.from_json(d)
    t = synthetic_seq_tensors(cfg, seed=3)
    assert sorted(t) == sorted(n for n, _, _ in seq_param_specs(cfg))
    w = SeqWeights(cfg, t, torch.float32, torch.device("cpu"))
    assert w.unused == [] and w.inv_freq is None
    W, n = cfg.width, cfg.streams
    assert torch.equal(w.final_norm, t["final.norm"].float() + 1.0) and torch.equal(w.layers[0]["norm1"], t["l0.norm1"].float() + 1.0)
    hc = w.layers[0]["hc2"]
    assert hc.shape == (2 * n + n * n,) and torch.equal(hc[2 * n:].reshape(n, n), t["l0.hc2.mix"].float())
    r, a = cfg.layers[0].retention, cfg.layers[1].latent
    assert w.layers[0]["t_in"].shape == ((2 * r.heads * r.dim + 2 * r.heads * r.vdim + 7) // 8 * 8, W)     # rows padded to 8
    assert torch.allclose(w.layers[0]["t_log_decay"].double().exp(), torch.tensor(r.decay, dtype=torch.float64), rtol=1e-6)
    rows = a.heads * (a.dim + a.rot_dim) + a.kv_rank + a.rot_dim + a.heads
    assert w.layers[1]["a_in"].shape == ((rows + 7) // 8 * 8, W)
    assert torch.equal(w.layers[1]["a_in"][rows - a.heads:rows], t["l1.mix.g"].float())
    assert w.layers[1]["a_uk_t"].shape == (a.heads, a.kv_rank, a.dim)
    assert torch.equal(w.layers[1]["a_uk_t"][1, :, 2], t["l1.mix.uk"].float()[a.dim + 2])
    a2 = cfg.layers[2].latent                                       # reads layer 1's cache: no latent projection
    assert "a_latent_norm" not in w.layers[2] and w.layers[2]["a_in"].shape[0] == (a2.heads * (a2.dim + a2.rot_dim) + a2.heads + 7) // 8 * 8
    e = cfg.layers[0].moe
    assert w.layers[0]["e_up"].shape == (e.experts, e.ff, W) and w.layers[0]["e_down"].shape == (e.experts, W, e.ff)
    assert torch.equal(w.layers[0]["e_router"][e.experts], t["l0.mlp.shared.sg"].float()[0])      # the shared gate's row
    assert "norm2" not in w.layers[3] and "hc2" not in w.layers[3]  # a layer without a feed-forward
    bad = dict(t)
    bad["l1.mix.uk"] = bad["l1.mix.uk"][:-1]
    with pytest.raises(ValueError):
        SeqWeights(cfg, bad, torch.float32, torch.device("cpu"))


def test_checkpoint_file_round_trip_and_registry(tmp_path):
    d = K.CASES["odd"]
    t = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=4)
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    back = dict(iter_safetensors(str(tmp_path)))
    assert sorted(back) == sorted(t) and all(torch.equal(back[k], t[k]) for k in t)
    assert architecture_of(d) == "Kedelorn"
    assert model_class("Kedelorn").__name__ == "SeqLMForCausalLM"


def test_latent_caches_keep_one_pool_and_every_page():
    # layers 0 and 2 own a latent cache (K rows only), layer 1 reads layer 0's and has none, layer 3 is recurrent
    pool = SeqStatePool({0: (1, 20, 0, 0), 2: (1, 12, 0, 0)}, [0, 0, 0, 96], torch.float32, torch.device("cpu"), initial_pages=2)
    assert pool.k[0].shape == (2, 1, PAGE_SIZE, 20) and pool.v[0] is None and 1 not in pool.k
    assert pool.bytes_per_token() == 4 * 32 and pool.state_bytes_per_sequence() == 4 * 96
    c = SeqCache(pool)
    c.ensure_tokens(3 * PAGE_SIZE + 1)                     # grows the pool; old rows are copied
    assert pool.num_pages >= 4 and c.live_pages() == 4
    c.advance(3 * PAGE_SIZE + 1)
    assert c.live_pages() == 4 and pool.keep_from(c.seq_len) == 0      # plain causal attention never gives a page back early
    pool.state[3][c.slot].fill_(1.0)
    slot = c.slot
    c.release()
    c2 = SeqCache(pool)
    assert c2.slot == slot and float(pool.state[3][slot].abs().sum()) == 0.0 and len(pool.free) == pool.num_pages - 0
