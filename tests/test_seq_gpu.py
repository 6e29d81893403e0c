"""The hybrid sequence models on the GPU against the float64 oracle (tests/seq_oracle.py): every mechanism alone, whole
prompts against token-by-token decoding, portions down to two tokens, batches against each request alone, pages and
state slots that are used again, chunk edges and page borders, long decoding, unusual sizes, and greedy generation
through the engine's own entry point. fp32 storage is compared tightly; bf16 storage within bf16 rounding."""
import json
import os
import subprocess
import sys

import pytest
import torch

import seq_cases
import seq_oracle as O
from livecc_b200.checkpoint import synthetic_seq_tensors, write_safetensors
from livecc_b200.config import SeqModelConfig

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_models = {}


def model_of(name, dtype="float32", seed=11):
    from livecc_b200.seq_engine import SeqLMForCausalLM

    key = (name, dtype, seed)
    if key not in _models:
        d = seq_cases.CASES[name]
        cfg = SeqModelConfig.from_json(d)
        tensors = synthetic_seq_tensors(cfg, seed=seed)
        _models[key] = (SeqLMForCausalLM.from_state_dict(cfg, tensors, dtype), d, tensors)
    return _models[key]


_oracle = {}


def oracle(name, toks, seed=11, **kw):
    key = (name, tuple(toks), seed, tuple(sorted(kw.items())))
    if key not in _oracle:
        _, d, tensors = model_of(name, "float32", seed)
        _oracle[key] = O.forward(d, tensors, toks, **kw)
    return _oracle[key]


def rel(got, want):
    """Largest row error: rms(got - want) / rms(want) over the last axis."""
    got, want = got.double().cpu(), want.double()
    return float(((got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-30)).max())


def run(m, toks, cuts, want_all=True):
    """One request through forward_step in portions ending at `cuts`; returns the logits of every position."""
    c = m.new_cache()
    rows, lo = [], 0
    for hi in list(cuts) + [len(toks)]:
        if hi <= lo:
            continue
        rows.append(m.forward_step([(c, toks[lo:hi])], [list(range(hi - lo))]).cpu())
        lo = hi
    c.release()
    return torch.cat(rows)


F32_TOL = 2e-5
BF16_TOL = 4e-2


# ---- every mechanism alone, and together, against the oracle ------------------------------------------------------------
@pytest.mark.parametrize("name", ["ssd_only", "parallel_only", "mixed", "odd"])
def test_whole_prompt_every_layer_matches_the_oracle_fp32(name):
    m, d, _ = model_of(name)
    toks = seq_cases.tokens(75, d["vocab"])
    want_lg, want_layers = oracle(name, toks)
    c = m.new_cache()
    lg, dump = m.forward_step([(c, toks)], [list(range(len(toks)))], layer_dump=True)
    c.release()
    for li in range(len(d["layers"])):
        assert rel(dump[li], want_layers[li]) < F32_TOL, f"residual stream after layer {li} ({d['layers'][li]['type']})"
    assert rel(lg, want_lg) < F32_TOL


@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_bf16_storage_stays_within_rounding_on_both_linear_paths(name, monkeypatch):
    from livecc_b200.seq_engine import SeqLMForCausalLM

    _, d, tensors = model_of(name)
    toks = seq_cases.tokens(90, d["vocab"], seed=3)
    want_lg, _ = oracle(name, toks)
    outs = []
    for tc in ("1", "0"):                       # tensor-core GEMM where the shape allows it / CUDA-core kernels only
        monkeypatch.setenv("LIVECC_B200_SEQ_TC", tc)
        m = SeqLMForCausalLM.from_state_dict(SeqModelConfig.from_json(d), tensors, "bfloat16")
        outs.append(run(m, toks, []))
        assert rel(outs[-1], want_lg) < BF16_TOL
        assert rel(run(m, toks, [60] + list(range(61, 90))), want_lg) < BF16_TOL
    assert rel(outs[0], outs[1].double()) < BF16_TOL


# ---- prefill against decoding, portions, first tokens ---------------------------------------------------------------------
@pytest.mark.parametrize("name", ["ssd_only", "parallel_only", "mixed", "odd"])
def test_token_by_token_decoding_equals_the_whole_prompt(name):
    m, d, _ = model_of(name)
    toks = seq_cases.tokens(70, d["vocab"], seed=1)
    want_lg, _ = oracle(name, toks)
    assert rel(run(m, toks, range(1, 70)), want_lg) < F32_TOL          # every token alone, from the first one
    assert rel(run(m, toks, [41] + list(range(42, 70))), want_lg) < F32_TOL


@pytest.mark.parametrize("cuts", [[2, 4, 6, 9, 11, 40, 42], [1, 3, 64, 66], [23, 24, 25, 47, 49, 65], [63, 65, 67, 69]])
def test_portions_of_any_size_down_to_two_tokens(cuts):
    m, d, _ = model_of("mixed")
    toks = seq_cases.tokens(80, d["vocab"], seed=2)
    want_lg, _ = oracle("mixed", toks)
    assert rel(run(m, toks, cuts), want_lg) < F32_TOL


def test_first_tokens_of_a_sequence():
    m, d, _ = model_of("mixed")
    for n in (1, 2, 3):
        toks = seq_cases.tokens(n, d["vocab"], seed=20 + n)
        assert rel(run(m, toks, []), oracle("mixed", toks)[0]) < F32_TOL


# ---- chunk edges and page borders ------------------------------------------------------------------------------------------
def test_chunk_edges_and_page_borders_in_prompts_and_in_decoding():
    """Chunks of 40 over pages of 64 with a sharp softmax: positions 39/40/41, 63/64/65 (a page border inside the chunk
    [40, 80)), 79/80/81, 119/120/121, 127/128/129, once inside a prompt portion and once decoded alone."""
    m, d, _ = model_of("sharp")
    toks = seq_cases.tokens(170, d["vocab"], seed=4)
    want_lg, _ = oracle("sharp", toks)
    whole = run(m, toks, [])
    assert rel(whole, want_lg) < F32_TOL
    # the test's weights do show the faults it is after: an oracle without the sink, or with chunks one token longer or
    # shorter, is far outside the tolerance
    assert rel(whole, oracle("sharp", toks, sink=False)[0]) > 100 * F32_TOL
    assert rel(whole, oracle("sharp", toks, chunk_shift=1)[0]) > 100 * F32_TOL
    assert rel(whole, oracle("sharp", toks, chunk_shift=-1)[0]) > 100 * F32_TOL
    edges = [39, 40, 41, 63, 64, 65, 79, 80, 81, 119, 120, 121, 127, 128, 129]
    decoded = run(m, toks, [30] + list(range(31, 170)))
    assert rel(decoded[edges], want_lg[edges]) < F32_TOL
    assert rel(decoded, want_lg) < F32_TOL
    assert rel(run(m, toks, [39, 41, 64, 79, 82, 120, 128, 130]), want_lg) < F32_TOL


def test_a_key_far_back_in_the_recurrent_state_is_still_seen():
    """State-space layers only, decay rates set close to zero: the logits at the end depend on the first token through the
    carried state alone, 150 tokens and 110 decode steps later."""
    from livecc_b200.seq_engine import SeqLMForCausalLM

    d = seq_cases.CASES["ssd_only"]
    cfg = SeqModelConfig.from_json(d)
    tensors = synthetic_seq_tensors(cfg, seed=12)
    for i in range(len(d["layers"])):
        tensors[f"l{i}.mix.A_log"].fill_(-7.0)
    m = SeqLMForCausalLM.from_state_dict(cfg, tensors, "float32")
    toks = seq_cases.tokens(150, d["vocab"], seed=5)
    other = [(toks[0] + 1) % d["vocab"]] + toks[1:]
    a, b = O.forward(d, tensors, toks)[0], O.forward(d, tensors, other)[0]
    assert rel(b[-1:], a[-1:]) > 100 * F32_TOL, "the test's weights forget the first token"
    assert rel(run(m, toks, [40] + list(range(41, 150))), a) < F32_TOL
    assert rel(run(m, other, [40] + list(range(41, 150))), b) < F32_TOL


# ---- the sequence-parallel kernels of prompt portions ----------------------------------------------------------------------
def _check_long(d, tensors, n, cuts, seed, tol=F32_TOL):
    from livecc_b200.seq_engine import SeqLMForCausalLM

    m = SeqLMForCausalLM.from_state_dict(SeqModelConfig.from_json(d), tensors, "float32")
    toks = seq_cases.tokens(n, d["vocab"], seed=seed)
    want_lg, want_layers = O.forward(d, tensors, toks)
    c = m.new_cache()
    lg, dump = m.forward_step([(c, toks)], [list(range(n))], layer_dump=True)
    c.release()
    for li in range(len(d["layers"])):
        assert rel(dump[li], want_layers[li]) < tol, f"residual stream after layer {li}"
    assert rel(lg, want_lg) < tol
    assert rel(run(m, toks, cuts), want_lg) < tol


def test_long_prompts_cross_many_blocks_of_the_recurrence_and_key_tiles():
    """333 tokens: five full 64-row blocks of the recurrence and a ragged sixth, attention chunks of 24 and 10 that never
    line up with the 64-key tiles; then portions that start and end inside blocks (the carried state enters mid-way)."""
    _, d, tensors = model_of("mixed")
    _check_long(d, tensors, 333, [100, 131, 133, 260, 292], seed=50)


def test_strong_and_weak_decays_in_the_block_form():
    """Decays near zero (a row forgets everything before it within a few tokens: the block form must not overflow where
    it divides cumulative decays) and near one, mixed over channels and heads."""
    d = seq_cases.CASES["odd"]
    cfg = SeqModelConfig.from_json(d)
    tensors = synthetic_seq_tensors(cfg, seed=13)
    b = tensors["l0.mix.right.a2.b"]
    b.copy_(torch.linspace(-60.0, 12.0, b.numel()).to(b.dtype))          # tau = 1: log decay down to -60 per token
    tensors["l1.mix.A_log"].copy_(torch.tensor([3.0, -6.0]).to(tensors["l1.mix.A_log"].dtype))
    tensors["l1.mix.dt_bias"].copy_(torch.tensor([4.0, 0.0]).to(tensors["l1.mix.dt_bias"].dtype))
    _check_long(d, tensors, 200, [70, 137], seed=51, tol=2 * F32_TOL)


@pytest.mark.parametrize("dim,vdim", [(72, 136), (136, 72)])
def test_heads_wider_than_one_tile(dim, vdim):
    """Key, value and state sizes above 64 and 128 (several tiles per head, ragged last tiles), a chunk that is longer than
    two key tiles, a last key tile that ends on the row itself. Head size 72 runs the attention's two-group form, 136 the
    one-group form."""
    layers = [seq_cases.par(heads=2, kv_heads=1, dim=dim, vdim=vdim, chunk=150, scale=0.2, r_heads=1, r_dim=70, r_vdim=67, tau=8.0, ff=None),
              seq_cases.ssd(heads=2, vdim=66, state=68, groups=1, conv=3, norm_groups=2)]
    d = seq_cases.config(layers, width=32, vocab=64)
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=14)
    _check_long(d, tensors, 215, [64, 128, 129, 193], seed=52)
    # the same sizes in bf16 storage: the tensor-core attention pads 72 channels to 80 (136 to 144) and cuts 136 outputs into 128 + 8
    from livecc_b200.seq_engine import SeqLMForCausalLM

    toks = seq_cases.tokens(215, d["vocab"], seed=52)
    want = O.forward(d, tensors, toks)[0]
    m = SeqLMForCausalLM.from_state_dict(SeqModelConfig.from_json(d), tensors, "bfloat16")
    # (row 0 is left out: there the normalised linear-attention output is sign(q.k) v / rms(v), and q.k of this seed's first
    # token is close enough to zero for bf16 rounding to matter)
    assert rel(run(m, toks, [])[1:], want[1:]) < BF16_TOL
    assert rel(run(m, toks, [64, 129, 193] + list(range(194, 215)))[1:], want[1:]) < BF16_TOL


def test_a_prompt_longer_than_one_pass_of_the_block_form():
    """4300 rows in one step: the block form of the recurrence runs a second pass that starts from the state the first
    left (a pass covers 64 blocks of 64 rows). Compared with the same prompt fed in portions of 31 rows, which all take the
    token-by-token kernel (the one the other tests hold to the oracle)."""
    m, d, _ = model_of("mixed")
    toks = seq_cases.tokens(4300, d["vocab"], seed=60)
    whole = run(m, toks, [])
    parts = run(m, toks, range(31, 4300, 31))
    assert rel(whole[4000:], parts[4000:].double()) < 2 * F32_TOL
    assert rel(whole, parts.double()) < 2 * F32_TOL


def test_tiled_attention_kernels_take_any_row_count(monkeypatch):
    """Windows too long for the one-CTA-per-row kernel's score buffer go to the tiled kernels whatever the row count; the
    switch forces that route, so decode steps and portions of 2 to 15 rows run on them: fp32 tiles, and bf16 tensor-core tiles in
    both forms (aligned head sizes, and sizes that are not multiples of 8)."""
    from livecc_b200.seq_engine import SeqLMForCausalLM

    monkeypatch.setenv("LIVECC_B200_SEQ_ATTN_TILED", "1")
    code = ("import sys, json, torch; sys.path[:0] = [%r, %r]; import seq_cases, seq_oracle as O;"
            "from livecc_b200.checkpoint import synthetic_seq_tensors; from livecc_b200.config import SeqModelConfig;"
            "from livecc_b200.seq_engine import SeqLMForCausalLM\n"
            "def rel(g, w):\n"
            "    g, w = g.double().cpu(), w.double(); return float(((g - w).pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-30)).max())\n"
            "out = {}\n"
            "for name in ('mixed', 'odd'):\n"
            "    d = seq_cases.CASES[name]; cfg = SeqModelConfig.from_json(d); t = synthetic_seq_tensors(cfg, seed=11)\n"
            "    toks = seq_cases.tokens(70, d['vocab'], seed=1); want = O.forward(d, t, toks)[0]\n"
            "    for dt in ('float32', 'bfloat16'):\n"
            "        m = SeqLMForCausalLM.from_state_dict(cfg, t, dt); c = m.new_cache(); rows = []; lo = 0\n"
            "        for hi in [3, 5, 20, 21, 22, 30, 45] + list(range(46, 71)):\n"
            "            rows.append(m.forward_step([(c, toks[lo:hi])], [list(range(hi - lo))]).cpu()); lo = hi\n"
            "        out[name + ':' + dt] = rel(torch.cat(rows), want)\n"
            "print('RESULT ' + json.dumps(out))\n") % (os.path.dirname(os.path.abspath(__file__)), os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    # a process of its own: the library reads the switch once
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, env=dict(os.environ))
    assert r.returncode == 0, r.stderr[-2000:]
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    for key, err in res.items():
        # bf16: the worst of 70 rows of the small "odd" model (no soft cap, tau = 1) sits at the edge of BF16_TOL on either route
        assert err < (F32_TOL if key.endswith("float32") else 1.5 * BF16_TOL), (key, err)


# ---- batches, pages and slots that are used again -----------------------------------------------------------------------------
def test_a_batch_of_unequal_requests_equals_each_alone():
    m, d, _ = model_of("mixed")
    reqs = [seq_cases.tokens(n, d["vocab"], seed=30 + n) for n in (57, 9, 130)]
    alone = [run(m, t, []) for t in reqs]
    caches = [m.new_cache() for _ in reqs]
    # step 1: unequal prompt portions; step 2: one decodes, one continues its prompt, one finishes
    cut = [40, 8, 70]
    lg1 = m.forward_step([(c, t[:k]) for c, t, k in zip(caches, reqs, cut)], [list(range(k)) for k in cut]).cpu()
    lg2 = m.forward_step([(c, t[k:]) for c, t, k in zip(caches, reqs, cut)], [list(range(len(t) - k)) for t, k in zip(reqs, cut)]).cpu()
    o1 = o2 = 0
    for t, k, want in zip(reqs, cut, alone):
        got = torch.cat([lg1[o1:o1 + k], lg2[o2:o2 + len(t) - k]])
        o1, o2 = o1 + k, o2 + len(t) - k
        assert rel(got, want.double()) < F32_TOL
        assert rel(got, oracle("mixed", t)[0]) < F32_TOL
    for c in caches:
        c.release()


def test_slots_and_pages_of_finished_requests_are_used_again():
    from livecc_b200.seq_engine import SeqLMForCausalLM

    _, d, tensors = model_of("mixed")
    m = SeqLMForCausalLM.from_state_dict(SeqModelConfig.from_json(d), tensors, "float32", max_tokens=128)   # a pool of 4 pages
    a, b, c3 = (seq_cases.tokens(n, d["vocab"], seed=40 + n) for n in (140, 90, 33))
    want_b, want_c = oracle("mixed", b)[0], oracle("mixed", c3)[0]
    ca = m.new_cache()
    m.forward_step([(ca, a)])                   # fills pages and leaves a non-zero state behind
    slot_a, pages_a = ca.slot, [p for p in ca.pages if p is not None]
    ca.release()
    cb = m.new_cache()
    assert cb.slot == slot_a
    got_b = m.forward_step([(cb, b[:50])], [list(range(50))]).cpu()
    cc = m.new_cache()                          # a second live request while b is half way
    got_c = m.forward_step([(cc, c3)], [list(range(len(c3)))]).cpu()
    got_b = torch.cat([got_b, m.forward_step([(cb, b[50:])], [list(range(40))]).cpu()])
    assert set(pages_a) & set(p for p in cb.pages + cc.pages if p is not None), "the freed pages were not handed out again"
    assert rel(got_b, want_b) < F32_TOL and rel(got_c, want_c) < F32_TOL
    live_before = cb.live_pages()
    more = seq_cases.tokens(60, d["vocab"], seed=77)
    m.forward_step([(cb, more)])                # 150 tokens: both chunk sizes have left the first pages
    assert cb.live_pages() <= live_before and cb.pages[0] is None
    cb.release(); cc.release()
    assert len(m.pool.free) == m.pool.num_pages and len(m.pool.free_slots) == m.pool.num_slots


# ---- long decoding, generation ---------------------------------------------------------------------------------------------
def test_long_decoding_stays_on_the_oracle():
    m, d, _ = model_of("odd")
    toks = seq_cases.tokens(260, d["vocab"], seed=6)
    want_lg, _ = oracle("odd", toks)
    got = run(m, toks, [4] + list(range(5, 260)))
    assert rel(got, want_lg) < 2 * F32_TOL


def test_greedy_generation_through_the_engine_entry_point():
    m, d, tensors = model_of("mixed")
    prompt = seq_cases.tokens(37, d["vocab"], seed=8)
    want = O.greedy(d, tensors, prompt, 20)
    ids = torch.tensor([prompt])
    out = m.generate(ids, max_new_tokens=20, output_logits=True)
    assert out.sequences[0, :37].tolist() == prompt and out.sequences[0, 37:].tolist() == want
    # the logits of every step are the oracle's for the sequence so far
    full, _ = oracle("mixed", prompt + want)
    assert rel(torch.stack(out.logits), full[36:36 + 20]) < F32_TOL
    assert out.past_key_values.get_seq_length() == 37 + 19       # the last token is selected, not yet run
    out.past_key_values.release()
    # eager launches instead of graph replay, and a prompt cut into portions: the same ids
    m.use_cuda_graph = False
    try:
        assert m.generate(ids, max_new_tokens=20, prefill_chunk=5).sequences[0, 37:].tolist() == want
    finally:
        m.use_cuda_graph = True
    # a stop id ends the call early and later steps leave the state alone; a second turn continues from the cache
    stop = want[6]
    first = want.index(stop)
    out = m.generate(ids, max_new_tokens=20, eos_token_id=stop)
    assert out.sequences[0, 37:].tolist() == want[:first + 1]
    assert out.past_key_values.get_seq_length() == 37 + first
    turn2 = out.sequences[0].tolist() + seq_cases.tokens(5, d["vocab"], seed=9)
    out2 = m.generate(torch.tensor([turn2]), past_key_values=out.past_key_values, max_new_tokens=4)
    assert out2.sequences[0, len(turn2):].tolist() == O.greedy(d, tensors, turn2, 4)
    out2.past_key_values.release()
    bf, _, _ = model_of("mixed", "bfloat16")
    got = bf.generate(ids, max_new_tokens=8).sequences[0, 37:].tolist()
    assert len(got) == 8 and all(0 <= t < d["vocab"] for t in got)


def test_trace_replay_command_line(tmp_path):
    d = seq_cases.CASES["mixed"]
    cfg = SeqModelConfig.from_json(d)
    tensors = synthetic_seq_tensors(cfg, seed=11)
    mdir = tmp_path / "model"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(d))
    write_safetensors(str(mdir / "model.safetensors"), tensors)
    a, b = seq_cases.tokens(50, d["vocab"], seed=50), seq_cases.tokens(7, d["vocab"], seed=51)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": a[:33], "want": [0, 32]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": a[33:35], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": a[35:], "want": [14]}], "end": ["x"]},
             {"step": 3, "entries": [{"id": "y", "tokens": b, "want": [6]}], "end": ["y"]}]
    out = tmp_path / "out"
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", str(mdir), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "64"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    assert not (out / "1.f32").exists()
    import numpy as np

    la, lb = O.forward(d, tensors, a)[0], O.forward(d, tensors, b)[0]
    g0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4")).reshape(2, -1)
    g2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4")).reshape(1, -1)
    g3 = torch.from_numpy(np.fromfile(out / "3.f32", dtype="<f4")).reshape(1, -1)
    assert rel(g0, la[[0, 32]]) < F32_TOL and rel(g2, la[[49]]) < F32_TOL and rel(g3, lb[[6]]) < F32_TOL
