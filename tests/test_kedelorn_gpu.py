"""Kedelorn on the GPU against the float64 oracle (tests/kedelorn_oracle.py): every mechanism alone and together, whole
prompts against token-by-token decoding, portions down to two tokens, batches against each request alone, pages and state
slots that are used again, far keys and page borders with a sharp softmax, the sink and the router's correction, long
decoding, unusual sizes, and greedy generation through the engine's own entry point. fp32 storage is compared tightly;
bf16 storage within bf16 rounding."""
import json
import os
import subprocess

import pytest
import torch

import kedelorn_cases as K
import kedelorn_oracle as O
from livecc_b200.checkpoint import synthetic_seq_tensors, write_safetensors
from livecc_b200.config import SeqModelConfig

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F32_TOL = 2e-5
BF16_TOL = 4e-2

_models = {}


def build(d, tensors, dtype="float32", **kw):
    from livecc_b200.seq_engine import SeqLMForCausalLM

    return SeqLMForCausalLM.from_state_dict(SeqModelConfig.from_json(d), tensors, dtype, **kw)


def model_of(name, dtype="float32", seed=21):
    key = (name, dtype, seed)
    if key not in _models:
        d = K.CASES[name]
        tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=seed)
        _models[key] = (build(d, tensors, dtype), d, tensors)
    return _models[key]


_oracle = {}


def oracle(name, toks, seed=21, **kw):
    key = (name, tuple(toks), seed, tuple(sorted(kw.items())))
    if key not in _oracle:
        _, d, tensors = model_of(name, "float32", seed)
        _oracle[key] = O.forward(d, tensors, toks, **kw)
    return _oracle[key]


def rel(got, want):
    """Largest row error: rms(got - want) / rms(want) over the last axis."""
    got, want = got.double().cpu(), want.double()
    return float(((got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-30)).max())


def bf16_ok(got, want):
    """bf16 storage: a router score close to the next one, or a first-token retention output close to zero, can fall the
    other way under rounding and move that row by far more than rounding; such rows are allowed to be few, the bulk stays
    within bf16 rounding."""
    got, want = got.double().cpu(), want.double()
    e = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-30)
    return float(e.median()) < BF16_TOL / 2 and float((e > BF16_TOL).double().mean()) <= 0.1 and bool(torch.isfinite(e).all())


def run(m, toks, cuts):
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


ALL = ["retention_only", "latent_only", "shared_cache", "moe_only", "mixed", "odd"]


# ---- every mechanism alone, and together, against the oracle ------------------------------------------------------------
@pytest.mark.parametrize("name", ALL)
def test_whole_prompt_every_layer_matches_the_oracle_fp32(name):
    m, d, _ = model_of(name)
    toks = K.tokens(75, d["vocab"])
    want_lg, want_layers = oracle(name, toks)
    c = m.new_cache()
    lg, dump = m.forward_step([(c, toks)], [list(range(len(toks)))], layer_dump=True)
    c.release()
    for li in range(len(d["layers"])):
        assert rel(dump[li], want_layers[li]) < F32_TOL, f"sum of the streams after layer {li} ({d['layers'][li]['type']})"
    assert rel(lg, want_lg) < F32_TOL


@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_bf16_storage_stays_within_rounding_on_both_linear_paths(name, monkeypatch):
    _, d, tensors = model_of(name)
    toks = K.tokens(90, d["vocab"], seed=3)
    want_lg, _ = oracle(name, toks)
    for tc in ("1", "0"):                       # tensor-core kernels where the shape allows them / CUDA-core kernels only
        monkeypatch.setenv("LIVECC_B200_SEQ_TC", tc)
        m = build(d, tensors, "bfloat16")
        assert bf16_ok(run(m, toks, []), want_lg)
        assert bf16_ok(run(m, toks, [60] + list(range(61, 90))), want_lg)


def test_the_sink_and_the_router_correction_show_in_these_weights():
    """An oracle without the sink term, or one that chooses experts without the correction, is far outside the tolerance:
    the other tests would notice either being left out."""
    m, d, _ = model_of("mixed")
    toks = K.tokens(75, d["vocab"])
    got = run(m, toks, [])
    assert rel(got, oracle("mixed", toks)[0]) < F32_TOL
    assert rel(got, oracle("mixed", toks, sink=False)[0]) > 100 * F32_TOL
    assert rel(got, oracle("mixed", toks, correction=False)[0]) > 100 * F32_TOL


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations_in_three_schedules(seed):
    """Random stacks (tests/kedelorn_cases.py::random_config): the whole prompt, most of it then token by token, and portions of
    changing size down to two tokens, all against the oracle in fp32. bf16 storage runs every stack (finite logits) and is
    held to rounding where the stack is shallow: through six narrow layers of unit-norm heads and routers, rounding noise
    grows past any fixed bound."""
    import random

    d = K.random_config(seed)
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=30 + seed)
    rng = random.Random(seed)
    T = rng.choice([70, 150, 260])
    toks = K.tokens(T, d["vocab"], seed=60 + seed)
    want = O.forward(d, tensors, toks)[0]
    portions, p = [], 0
    while p < T - 20:
        p += rng.choice([2, 3, 5, 16, 37, 64])
        portions.append(min(p, T - 20))
    m = build(d, tensors)
    for cuts in ([], [T - 20] + list(range(T - 19, T)), portions + list(range(T - 19, T))):
        assert rel(run(m, toks, cuts), want) < F32_TOL
    got = run(build(d, tensors, "bfloat16"), toks, portions)
    assert bool(torch.isfinite(got).all())
    if len(d["layers"]) <= 3:
        assert bf16_ok(got, want)


# ---- prefill against decoding, portions, first tokens ---------------------------------------------------------------------
@pytest.mark.parametrize("name", ALL)
def test_token_by_token_decoding_equals_the_whole_prompt(name):
    m, d, _ = model_of(name)
    toks = K.tokens(70, d["vocab"], seed=1)
    want_lg, _ = oracle(name, toks)
    assert rel(run(m, toks, range(1, 70)), want_lg) < F32_TOL          # every token alone, from the first one
    assert rel(run(m, toks, [41] + list(range(42, 70))), want_lg) < F32_TOL


@pytest.mark.parametrize("cuts", [[2, 4, 6, 9, 11, 40, 42], [1, 3, 64, 66], [23, 24, 25, 47, 49, 65], [63, 65, 67, 69]])
def test_portions_of_any_size_down_to_two_tokens(cuts):
    m, d, _ = model_of("mixed")
    toks = K.tokens(80, d["vocab"], seed=2)
    want_lg, _ = oracle("mixed", toks)
    assert rel(run(m, toks, cuts), want_lg) < F32_TOL


def test_first_tokens_of_a_sequence():
    m, d, _ = model_of("mixed")
    for n in (1, 2, 3):
        toks = K.tokens(n, d["vocab"], seed=20 + n)
        assert rel(run(m, toks, []), oracle("mixed", toks)[0]) < F32_TOL


# ---- far keys, page borders -----------------------------------------------------------------------------------------------
def _far_key_model():
    """One latent-attention layer whose weights make one far key stand out: token A (the key) and token B (the query) have
    one-hot embeddings; after the norm they reach the rotary key part / every head's rotary query part through one large
    weight on the slowest-turning pair, so B's score against A dwarfs every other score wherever A sits."""
    d = K.CASES["sharp"]
    cfg = SeqModelConfig.from_json(d)
    tensors = synthetic_seq_tensors(cfg, seed=22)
    mx = d["layers"][0]["mixer"]
    A, B, ja, jb = 5, 9, 3, 11
    R, D, DR, H = mx["kv_rank"], mx["dim"], mx["rot_dim"], mx["heads"]
    slow = DR // 2 - 1
    for tok, col in ((A, ja), (B, jb)):
        tensors["embed"][tok].zero_()
        tensors["embed"][tok, col] = 1.0
    tensors["l0.mix.dkv"][R + slow, ja] = 3.0
    for h in range(H):
        tensors["l0.mix.q"][h * (D + DR) + D + slow, jb] = 3.0
    return d, tensors, A, B


@pytest.mark.parametrize("far_at", [0, 1, 62, 63, 64, 65, 127, 128, 200])
def test_a_far_key_among_hundreds_at_page_borders(far_at):
    """A sits once at `far_at` (first tokens, just before / on / after a page border, deep inside), B queries it from the
    end of a 300-token sequence: in one prompt, decoded alone, and at the start of a two-token portion."""
    d, tensors, A, B = _far_key_model()
    toks = [t if t not in (A, B) else 17 for t in K.tokens(300, d["vocab"], seed=7)]
    toks[far_at], toks[-1], toks[-2] = A, B, B
    moved = list(toks)
    moved[far_at] = 17
    want = O.forward(d, tensors, toks)[0]
    assert rel(O.forward(d, tensors, moved)[0][-2:], want[-2:]) > 1e3 * F32_TOL, "the far key does not stand out"
    m = build(d, tensors)
    assert rel(run(m, toks, []), want) < F32_TOL
    assert rel(run(m, toks, [250] + list(range(251, 300))), want) < F32_TOL
    assert rel(run(m, toks, [66, 129, 298]), want) < F32_TOL


@pytest.mark.parametrize("far_at", [0, 255, 256, 511, 512, 690])
def test_key_splits_of_long_windows(far_at):
    """Windows of more than 512 keys in steps of a few rows: the keys are split over several CTAs in tiles of 256 and the
    splits are merged with the sink's term. The far key sits in the first tile, at tile edges, and in the last, ragged
    tile; fp32 and bf16 storage; decoded alone and in portions of two and three rows; then the same through generation,
    where only the device knows the window's length."""
    d, tensors, A, B = _far_key_model()
    toks = [t if t not in (A, B) else 17 for t in K.tokens(700, d["vocab"], seed=8)]
    toks[far_at], toks[-1], toks[-3] = A, B, B
    want = O.forward(d, tensors, toks)[0]
    cuts = [650, 652, 655] + list(range(656, 700))
    assert rel(run(build(d, tensors), toks, cuts), want) < F32_TOL
    assert bf16_ok(run(build(d, tensors, "bfloat16"), toks, cuts), want)
    if far_at == 511:
        m = build(d, tensors)
        new = O.greedy(d, tensors, toks[:600], 6)
        out = m.generate(torch.tensor([toks[:600]]), max_new_tokens=6, output_logits=True)
        assert out.sequences[0, 600:].tolist() == new
        assert rel(torch.stack(out.logits), O.forward(d, tensors, toks[:600] + new)[0][599:605]) < F32_TOL
        out.past_key_values.release()


def test_a_key_far_back_in_the_retention_state_is_still_seen():
    """Retention layers only, decays close to one: the logits at the end depend on the first token through the carried
    state alone, 150 tokens and 110 decode steps later."""
    d = json.loads(json.dumps(K.CASES["retention_only"]))
    for L in d["layers"]:
        L["mixer"]["decay"] = [0.999] * L["mixer"]["heads"]
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=23)
    m = build(d, tensors)
    toks = K.tokens(150, d["vocab"], seed=5)
    other = [(toks[0] + 1) % d["vocab"]] + toks[1:]
    a, b = O.forward(d, tensors, toks)[0], O.forward(d, tensors, other)[0]
    assert rel(b[-1:], a[-1:]) > 100 * F32_TOL, "the test's weights forget the first token"
    assert rel(run(m, toks, [40] + list(range(41, 150))), a) < F32_TOL
    assert rel(run(m, other, [40] + list(range(41, 150))), b) < F32_TOL


# ---- long prompts: the block form of the recurrence, many key tiles ------------------------------------------------------
def test_long_prompts_cross_many_blocks_of_the_recurrence_and_key_tiles():
    """333 tokens: five full 64-row blocks of the recurrence and a ragged sixth, six key tiles; then portions that start and
    end inside blocks and tiles (the carried state and the cached rows enter mid-way)."""
    m, d, _ = model_of("mixed")
    toks = K.tokens(333, d["vocab"], seed=50)
    want_lg, want_layers = oracle("mixed", toks)
    c = m.new_cache()
    lg, dump = m.forward_step([(c, toks)], [list(range(333))], layer_dump=True)
    c.release()
    for li in range(len(d["layers"])):
        assert rel(dump[li], want_layers[li]) < F32_TOL, f"sum of the streams after layer {li}"
    assert rel(lg, want_lg) < F32_TOL
    assert rel(run(m, toks, [100, 131, 133, 260, 292]), want_lg) < F32_TOL


@pytest.mark.parametrize("rank,rot_dim,vdim", [(136, 8, 24), (60, 12, 140), (248, 8, 16), (300, 10, 8)])
def test_latents_wider_than_one_tile(rank, rot_dim, vdim):
    """Cache rows of 144, 72 and 256 channels (several channel steps per key tile, two output tiles for a 136- or
    248-channel latent), in fp32 and in bf16 on the tensor-core attention; rows of 310 channels are beyond its head size
    and run on the CUDA-core tiles in both storage types."""
    layers = [K.lat(heads=2, dim=12, rot_dim=rot_dim, vdim=vdim, kv_rank=rank, scale=0.2, scaling=None, mlp=None),
              K.ret(heads=2, dim=70, vdim=67, decay=(0.9, 0.99), rot_dims=34, mlp=None)]
    d = K.config(layers, width=32, vocab=64)
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=24)
    toks = K.tokens(215, d["vocab"], seed=52)
    want = O.forward(d, tensors, toks)[0]
    m = build(d, tensors)
    assert rel(run(m, toks, []), want) < F32_TOL
    assert rel(run(m, toks, [64, 128, 129, 193]), want) < F32_TOL
    m = build(d, tensors, "bfloat16")
    assert bf16_ok(run(m, toks, []), want)
    assert bf16_ok(run(m, toks, [64, 129, 193] + list(range(194, 215))), want)


def test_many_rows_per_expert_and_experts_without_rows():
    """300 rows over 33 experts (top 5) and over 2 experts (top 1): lists longer than one tile, lists of a few rows, empty
    lists; the same rows decoded one by one take the few-row kernel."""
    m, d, _ = model_of("odd")
    toks = K.tokens(300, d["vocab"], seed=53)
    want = oracle("odd", toks)[0]
    assert rel(run(m, toks, []), want) < F32_TOL
    assert rel(run(m, toks, [280, 290] + list(range(291, 300))), want) < F32_TOL


def test_experts_on_the_tensor_cores(monkeypatch):
    """bf16 storage with enough routed rows and 8-aligned expert shapes: expert lists are padded to whole 128-row tiles and
    both expert products run as one grouped tensor-core GEMM each (relu^2 in the first one's epilogue). 400 tokens over 5
    experts (lists longer than a tile, ragged last tiles) and over 9 experts with top 1 (some lists shorter than a tile);
    against the oracle, against the CUDA-core route, and with the prompt cut so that later portions take the few-row route."""
    layers = [K.lat(heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=16, mlp=K.moe(experts=5, top=2, ff=72, scale=1.0, shared=80)),
              K.ret(heads=2, dim=8, vdim=8, decay=(0.9, 0.95), rot_dims=4, mlp=K.moe(experts=9, top=1, ff=64, scale=2.0, shared=0))]
    d = K.config(layers, width=64, vocab=64)
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=25)
    toks = K.tokens(400, d["vocab"], seed=54)
    want = O.forward(d, tensors, toks)[0]
    m = build(d, tensors, "bfloat16")
    n0 = m.kernel_launches()
    got = run(m, toks, [])
    assert m.kernel_launches() - n0 < 60, "the step took the per-list kernels"
    assert bf16_ok(got, want)
    assert bf16_ok(run(m, toks, [300, 390, 395]), want)
    monkeypatch.setenv("LIVECC_B200_SEQ_TC", "0")
    assert bf16_ok(run(build(d, tensors, "bfloat16"), toks, []), want)
    assert rel(run(build(d, tensors, "float32"), toks, []), want) < F32_TOL


def test_routed_feed_forward_in_post_norm_blocks(monkeypatch):
    """The routed feed-forward is a mechanism of the family, not of one design: state-space and parallel layers in post-norm
    blocks with routed experts, where the weighted sum of the expert rows is a kernel of its own before the post-norm
    residual. The post-norm oracle gets this file's routed feed-forward in place of its dense one."""
    import seq_cases
    import seq_oracle

    mlp = K.moe(experts=6, top=2, ff=16, scale=1.5, shared=24)
    layers = [dict(seq_cases.ssd(), mlp=mlp), dict(seq_cases.par(), mlp=mlp)]
    d = seq_cases.config(layers, width=40)
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=26)
    monkeypatch.setattr(seq_oracle, "feed_forward",
                        lambda h, w, pre: O.routed_ff(h, {k[len(pre):]: v for k, v in w.items() if k.startswith(pre)}, mlp))
    toks = K.tokens(120, d["vocab"], seed=55)
    want = seq_oracle.forward(d, tensors, toks)[0]
    m = build(d, tensors)
    assert rel(run(m, toks, []), want) < F32_TOL
    assert rel(run(m, toks, [50, 52] + list(range(100, 120))), want) < F32_TOL


# ---- batches, pages and slots that are used again -----------------------------------------------------------------------------
def test_a_batch_of_unequal_requests_equals_each_alone():
    m, d, _ = model_of("mixed")
    reqs = [K.tokens(n, d["vocab"], seed=30 + n) for n in (57, 9, 130)]
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
    _, d, tensors = model_of("mixed")
    m = build(d, tensors, max_tokens=128)       # a pool of 4 pages
    a, b, c3 = (K.tokens(n, d["vocab"], seed=40 + n) for n in (140, 90, 33))
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
    assert cb.live_pages() == 2 and cb.pages[0] is not None        # plain causal attention keeps every page
    cb.release(); cc.release()
    assert len(m.pool.free) == m.pool.num_pages and len(m.pool.free_slots) == m.pool.num_slots


# ---- long decoding, generation ---------------------------------------------------------------------------------------------
def test_long_decoding_stays_on_the_oracle():
    m, d, _ = model_of("odd")
    toks = K.tokens(260, d["vocab"], seed=6)
    want_lg, _ = oracle("odd", toks)
    assert rel(run(m, toks, [4] + list(range(5, 260))), want_lg) < 2 * F32_TOL


def test_greedy_generation_through_the_engine_entry_point():
    m, d, tensors = model_of("mixed")
    prompt = K.tokens(37, d["vocab"], seed=8)
    want = O.greedy(d, tensors, prompt, 20)
    ids = torch.tensor([prompt])
    out = m.generate(ids, max_new_tokens=20, output_logits=True)
    assert out.sequences[0, :37].tolist() == prompt and out.sequences[0, 37:].tolist() == want
    full, _ = oracle("mixed", prompt + want)
    assert rel(torch.stack(out.logits), full[36:36 + 20]) < F32_TOL     # the logits of every step are the oracle's
    assert out.past_key_values.get_seq_length() == 37 + 19              # the last token is selected, not yet run
    out.past_key_values.release()
    m.use_cuda_graph = False                    # eager launches instead of graph replay, and a prompt cut into portions
    try:
        assert m.generate(ids, max_new_tokens=20, prefill_chunk=5).sequences[0, 37:].tolist() == want
    finally:
        m.use_cuda_graph = True
    stop = want[6]                              # a stop id ends the call early; a second turn continues from the cache
    first = want.index(stop)
    out = m.generate(ids, max_new_tokens=20, eos_token_id=stop)
    assert out.sequences[0, 37:].tolist() == want[:first + 1]
    turn2 = out.sequences[0].tolist() + K.tokens(5, d["vocab"], seed=9)
    out2 = m.generate(torch.tensor([turn2]), past_key_values=out.past_key_values, max_new_tokens=4)
    assert out2.sequences[0, len(turn2):].tolist() == O.greedy(d, tensors, turn2, 4)
    out2.past_key_values.release()
    bf, _, _ = model_of("mixed", "bfloat16")
    got = bf.generate(ids, max_new_tokens=8).sequences[0, 37:].tolist()
    assert len(got) == 8 and all(0 <= t < d["vocab"] for t in got)


def test_generation_grows_across_key_tiles():
    """A replayed decode step was captured when the window held 100 keys; 200 tokens later it holds 300, which is three key
    tiles for the one split the captured grid has. Every step's logits against the oracle over the generated sequence."""
    m, d, tensors = model_of("latent_only")
    prompt = K.tokens(100, d["vocab"], seed=10)
    out = m.generate(torch.tensor([prompt]), max_new_tokens=200, eos_token_id=-1, output_logits=True)
    seq = out.sequences[0].tolist()
    assert len(seq) == 300 and seq[:100] == prompt
    want = O.forward(d, tensors, seq)[0][99:299]
    assert rel(torch.stack(out.logits), want) < 2 * F32_TOL
    out.past_key_values.release()


def test_trace_replay_command_line(tmp_path):
    d = K.CASES["mixed"]
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=21)
    mdir = tmp_path / "model"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(d))
    write_safetensors(str(mdir / "model.safetensors"), tensors)
    a, b = K.tokens(50, d["vocab"], seed=50), K.tokens(7, d["vocab"], seed=51)
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
