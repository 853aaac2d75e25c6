"""Lugizen on the GPU against the float64 oracle (tests/lugizen_oracle.py): every mechanism alone and together, whole prompts
against token-by-token decoding, portions down to two tokens, batches against each request alone, pages behind the window
and pages and slots that are used again, keys far away, at page borders and just inside / just outside the window with a
sharp softmax, a first token that only the recurrent state carries, the convolution's carried inputs, values mixed across
layers, the router's weights, long decoding, unusual sizes, and greedy generation through the engine's own entry point. fp32
storage is compared tightly; bf16 storage within bf16 rounding."""
import json
import os
import subprocess

import pytest
import torch

import lugizen_cases as K
import lugizen_oracle as O
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
    """(logits, residual stream after every layer)"""
    key = (name, tuple(toks), seed, tuple(sorted(kw.items())))
    if key not in _oracle:
        _, d, tensors = model_of(name, "float32", seed)
        _oracle[key] = O.forward(d, tensors, toks, layer_outputs=True, **kw)
    return _oracle[key]


def rel(got, want):
    """Largest row error: rms(got - want) / rms(want) over the last axis."""
    got, want = got.double().cpu(), want.double()
    return float(((got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-30)).max())


def rows_rel(got, want):
    got, want = got.double().cpu(), want.double()
    return (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-30)


def close32(got, want):
    """fp32 storage against the oracle: every row within the tolerance, but for the few rows (at most 2 in 100) in which a
    sublayer's output nearly cancels: the norm behind the sublayer scales such a row up, rounding included, and plain fp32
    arithmetic moves it by more than the product does. Those stay within ten times the tolerance."""
    e = rows_rel(got, want)
    return float(e.max()) < 10 * F32_TOL and float((e > F32_TOL).double().mean()) <= 0.02


def bf16_ok(got, want, routed=False):
    """bf16 storage: the bulk of the rows stays within bf16 rounding and few rows lie beyond twice that. routed: a stack with
    routers. A router logit close to the next one can fall the other way under rounding; the norm behind the feed-forward then
    hands the residual stream a full-size row in another direction, and the attention and delta-rule layers behind it carry
    that to every later position: such a stack is held to rounding in the median only."""
    got, want = got.double().cpu(), want.double()
    e = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-30)
    if not bool(torch.isfinite(e).all()):
        return False
    if routed:
        return float(e.median()) < BF16_TOL
    return float(e.median()) < BF16_TOL / 2 and float((e > BF16_TOL).double().mean()) <= 0.1


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


ALL = ["delta_only", "attention_only", "latent_only", "dense", "mixed", "moe", "odd"]


# ---- every mechanism alone, and together, against the oracle ------------------------------------------------------------
@pytest.mark.parametrize("name", ALL)
def test_whole_prompt_every_layer_matches_the_oracle_fp32(name):
    m, d, _ = model_of(name)
    toks = K.tokens(150, d["vocab"])
    want_lg, want_layers = oracle(name, toks)
    c = m.new_cache()
    lg, dump = m.forward_step([(c, toks)], [list(range(len(toks)))], layer_dump=True)
    c.release()
    for li in range(len(d["layers"])):
        assert close32(dump[li], want_layers[li]), f"residual stream after layer {li}"
    assert close32(lg, want_lg)


@pytest.mark.parametrize("name", ["delta_only", "attention_only", "latent_only", "dense", "mixed", "odd"])
def test_bf16_storage_stays_within_rounding_on_both_linear_paths(name, monkeypatch):
    _, d, tensors = model_of(name)
    toks = K.tokens(160, d["vocab"], seed=3)
    want_lg, _ = oracle(name, toks)
    routed = any(L["mlp"] and L["mlp"]["kind"] == "moe" for L in d["layers"])
    for tc in ("1", "0"):                       # tensor-core kernels where the shape allows them / CUDA-core kernels only
        monkeypatch.setenv("LIVECC_B200_SEQ_TC", tc)
        m = build(d, tensors, "bfloat16")
        assert bf16_ok(run(m, toks, []), want_lg, routed)
        assert bf16_ok(run(m, toks, [120] + list(range(121, 160))), want_lg, routed)


@pytest.mark.parametrize("name,what", [("mixed", "canon"), ("mixed", "vmix"), ("attention_only", "temp"), ("latent_only", "window"),
                                       ("moe", "router_weights")])
def test_each_mechanism_shows_in_these_weights(name, what):
    """An oracle that drops the convolution in front of the mixers, the mixing of values across layers, the temperatures, the
    window, or weights the chosen experts equally is far outside the tolerance: the other tests would notice a product that
    left any of them out."""
    m, d, _ = model_of(name)
    toks = K.tokens(75, d["vocab"])
    got = run(m, toks, [])
    assert close32(got, oracle(name, toks)[0])
    assert rel(got, oracle(name, toks, leave_out=(what,))[0]) > 100 * F32_TOL


@pytest.mark.parametrize("seed", range(12))
def test_random_configurations_in_three_schedules(seed):
    """Random stacks (tests/lugizen_cases.py::random_config): the whole prompt, most of it then token by token, and portions of
    changing size down to two tokens, all against the oracle in fp32; bf16 storage runs every stack and is held to rounding
    where the stack is shallow."""
    import random

    d = K.random_config(seed)
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=30 + seed)
    rng = random.Random(seed)
    T = rng.choice([70, 150, 260])
    toks = K.tokens(T, d["vocab"], seed=60 + seed)
    want = O.forward(d, tensors, toks)
    portions, p = [], 0
    while p < T - 20:
        p += rng.choice([2, 3, 5, 16, 37, 64])
        portions.append(min(p, T - 20))
    m = build(d, tensors)
    for cuts in ([], [T - 20] + list(range(T - 19, T)), portions + list(range(T - 19, T))):
        assert close32(run(m, toks, cuts), want)
    got = run(build(d, tensors, "bfloat16"), toks, portions)
    assert bool(torch.isfinite(got).all())
    if len(d["layers"]) <= 3:
        assert bf16_ok(got, want, routed=any(L["mlp"] and L["mlp"]["kind"] == "moe" for L in d["layers"]))


# ---- prefill against decoding, portions, first tokens ---------------------------------------------------------------------
@pytest.mark.parametrize("name", ALL)
def test_token_by_token_decoding_equals_the_whole_prompt(name):
    m, d, _ = model_of(name)
    toks = K.tokens(90, d["vocab"], seed=1)
    want_lg, _ = oracle(name, toks)
    assert rel(run(m, toks, range(1, 90)), want_lg) < F32_TOL          # every token alone, from the first one
    assert rel(run(m, toks, [41] + list(range(42, 90))), want_lg) < F32_TOL


@pytest.mark.parametrize("cuts", [[2, 4, 6, 9, 11, 40, 42], [1, 3, 64, 66], [23, 24, 25, 47, 49, 65], [63, 65, 67, 69], [8, 9, 17, 33, 35]])
def test_portions_of_any_size_down_to_two_tokens(cuts):
    """(cuts at 8 / 9 and 16 / 17 rows: the convolution kernels' row blocks and the scan's staging blocks)"""
    m, d, _ = model_of("mixed")
    toks = K.tokens(80, d["vocab"], seed=2)
    want_lg, _ = oracle("mixed", toks)
    assert rel(run(m, toks, cuts), want_lg) < F32_TOL


def test_first_tokens_of_a_sequence():
    for name in ("mixed", "odd"):
        m, d, _ = model_of(name)
        for n in (1, 2, 3, 4):
            toks = K.tokens(n, d["vocab"], seed=20 + n)
            assert rel(run(m, toks, []), oracle(name, toks)[0]) < F32_TOL
            assert rel(run(m, toks, range(1, n)), oracle(name, toks)[0]) < F32_TOL


# ---- the recurrent state and the convolutions' carried inputs ------------------------------------------------------------
def test_a_first_token_that_only_the_recurrent_state_carries():
    """One delta-rule layer whose decays are close to 1 and whose keys have room (40 channels, so that later writes take
    little of an old one away): what the first token wrote is still read 120 tokens later, through every cut of the prompt;
    changing the first token moves the last rows by far more than the tolerance."""
    d = K.config([K.delta(heads=2, kv_heads=2, dim=40, vdim=6, mlp=None)], width=16, vocab=40)
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=23)
    tensors["l0.mix.A_log"].fill_(-9.0)
    toks = K.tokens(120, d["vocab"], seed=70)
    other = [(toks[0] + 1) % d["vocab"]] + toks[1:]
    want = O.forward(d, tensors, toks)
    assert rel(O.forward(d, tensors, other)[-3:], want[-3:]) > 100 * F32_TOL, "the first token does not reach the end"
    m = build(d, tensors)
    for cuts in ([], [1], [2, 50], [110] + list(range(111, 120)), list(range(1, 120))):
        assert rel(run(m, toks, cuts), want) < F32_TOL
    assert bf16_ok(run(build(d, tensors, "bfloat16"), toks, [2, 50, 118]), want)


@pytest.mark.parametrize("decay", ["strong", "weak"])
def test_strong_and_weak_decays(decay):
    d = K.config([K.delta(heads=3, kv_heads=1, dim=12, vdim=5, conv=4, mlp=None)], width=16, vocab=40, taps=0)
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=26)
    tensors["l0.mix.A_log"].fill_(4.0 if decay == "strong" else -12.0)
    toks = K.tokens(200, d["vocab"], seed=71)
    want = O.forward(d, tensors, toks)
    m = build(d, tensors)
    assert rel(run(m, toks, []), want) < F32_TOL
    assert rel(run(m, toks, [100, 102] + list(range(150, 200))), want) < F32_TOL


@pytest.mark.parametrize("taps,conv", [(1, 1), (2, 5), (5, 2), (8, 8)])
def test_convolutions_of_any_length_carry_their_inputs(taps, conv):
    """The convolution in front of the mixer and the mixer's own q / k / v convolutions with 1 to 8 taps: portions shorter than
    the taps, equal to them and longer, and single tokens, read the inputs that earlier portions left."""
    d = K.config([K.delta(conv=conv, mlp=None), K.att(mlp=None), K.delta(heads=2, kv_heads=2, dim=4, vdim=4, conv=conv, mlp="dense")],
                 width=16, vocab=40, taps=taps)
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=31)
    toks = K.tokens(60, d["vocab"], seed=72)
    want = O.forward(d, tensors, toks)
    m = build(d, tensors)
    for cuts in ([], [1, 2, 3, 5, 8, 9, 17, 18, 20, 27, 35, 36], list(range(1, 60)), [7, 15, 16, 48]):
        assert rel(run(m, toks, cuts), want) < F32_TOL, cuts


def test_values_mixed_with_the_first_mixing_layers_values():
    """Four attention layers: the second and fourth mix their values with the first one's, the third does not; the first mixing
    layer may also sit behind other layers. The mix weights are set apart (0.9 and 0.1) so that swapping them would show."""
    layers = [K.delta(mlp=None), K.att(heads=2, kv_heads=2, dim=6, vdim=5, v_mix=True, mlp=None), K.att(heads=4, kv_heads=2, dim=4, vdim=5, v_mix=True, mlp="dense"),
              K.att(heads=3, kv_heads=3, dim=4, vdim=7, mlp=None), K.att(heads=2, kv_heads=2, dim=8, vdim=5, rot_dims=8, v_mix=True, mlp=None)]
    d = K.config(layers, width=20, vocab=40)
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=32)
    tensors["l2.mix.vmix"].fill_(0.9), tensors["l4.mix.vmix"].fill_(0.1)
    toks = K.tokens(100, d["vocab"], seed=73)
    want = O.forward(d, tensors, toks)
    assert rel(O.forward(d, tensors, toks, leave_out=("vmix",)), want) > 100 * F32_TOL
    m = build(d, tensors)
    assert rel(run(m, toks, []), want) < F32_TOL
    assert rel(run(m, toks, [50, 52] + list(range(70, 100))), want) < F32_TOL
    assert bf16_ok(run(build(d, tensors, "bfloat16"), toks, [50]), want)


# ---- far keys, page borders, the window's edges ---------------------------------------------------------------------------
def _one_hot_tokens(tensors, A, B, ja, jb):
    """Tokens A and B get one-hot embeddings in columns ja / jb that no other token uses; the convolution in front of the mixer
    is switched off so that the mixer reads exactly these rows."""
    tensors["l0.canon1"].zero_()
    tensors["embed"][:, ja] = 0.0
    tensors["embed"][:, jb] = 0.0
    for tok, col in ((A, ja), (B, jb)):
        tensors["embed"][tok].zero_()
        tensors["embed"][tok, col] = 2.0


def _key_model(scale=3.0):
    """One attention layer whose weights make one key stand out: token A (the key) and token B (the query) reach one
    un-rotated channel of the key head / of every query head through one large weight, and no other token reaches it. After
    the unit-rms norm B's score against A is about dim * scale * temperature, against every other key about zero, wherever
    A sits; A's value row is large, so whether A is seen moves the output by far more than the tolerance."""
    d = json.loads(json.dumps(K.CASES["sharp"]))
    mx = d["layers"][0]["mixer"]
    mx["scale"] = scale
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=22)
    A, B, ja, jb = 5, 9, 3, 11
    D, H, ch = mx["dim"], mx["heads"], mx["dim"] - 1          # the last channel of a head does not turn
    _one_hot_tokens(tensors, A, B, ja, jb)
    tensors["l0.mix.temp"].fill_(1.0)
    tensors["l0.mix.k"][ch, :] = 0.0
    tensors["l0.mix.k"][ch, ja] = 20.0
    tensors["l0.mix.v"][:, ja] = 6.0
    for h in range(H):
        tensors["l0.mix.q"][h * D + ch, :] = 0.0
        tensors["l0.mix.q"][h * D + ch, jb] = 20.0
    return d, tensors, A, B


def _latent_key_model(window, scale=0.3):
    """The same for a latent-attention layer: A alone reaches latent channel r0 (which the latent norm then makes about
    sqrt(rank)), one un-rotated key channel of every head reads only r0; B alone reaches query-latent channel s0, and the
    same channel of every query head reads only s0. B's score against A is about 16 sqrt(rank * q_rank) * scale."""
    d = json.loads(json.dumps(K.CASES["sharp_latent"]))
    mx = d["layers"][0]["mixer"]
    mx["mask"]["size"], mx["scale"] = window, scale
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=24)
    A, B, ja, jb, r0, s0, d0 = 5, 9, 3, 11, 2, 4, 1
    H, D, DR = mx["heads"], mx["dim"], mx["rot_dim"]
    _one_hot_tokens(tensors, A, B, ja, jb)
    tensors["l0.mix.dkv.norm"].fill_(1.0), tensors["l0.mix.dq.norm"].fill_(1.0)
    tensors["l0.mix.dkv"][r0, :] = 0.0
    tensors["l0.mix.dkv"][r0, ja] = 20.0
    tensors["l0.mix.dq"][s0, :] = 0.0
    tensors["l0.mix.dq"][s0, jb] = 20.0
    for h in range(H):
        tensors["l0.mix.uk"][h * D + d0, :] = 0.0
        tensors["l0.mix.uk"][h * D + d0, r0] = 4.0
        tensors["l0.mix.uq"][h * (D + DR) + d0, :] = 0.0
        tensors["l0.mix.uq"][h * (D + DR) + d0, s0] = 4.0
    tensors["l0.mix.uv"][:, r0] = 3.0
    return d, tensors, A, B


def _with_key(d, n, key_at, A, B, query_at, seed):
    toks = [t if t not in (A, B) else 17 for t in K.tokens(n, d["vocab"], seed=seed)]
    toks[key_at] = A
    for q in query_at:
        toks[q] = B
    return toks


@pytest.mark.parametrize("far_at", [0, 1, 62, 63, 64, 65, 127, 128, 200])
def test_a_far_key_among_hundreds_at_page_borders(far_at):
    """Plain causal attention over a 300-token sequence: A sits once at `far_at` (first tokens, just before / on / after a
    page border, deep inside), B queries it from the end: in one prompt, decoded alone, and at the start of a two-token
    portion; in fp32 and in bf16 on the tensor-core attention."""
    d, tensors, A, B = _key_model()
    toks = _with_key(d, 300, far_at, A, B, [298, 299], seed=7)
    moved = list(toks)
    moved[far_at] = 17
    want = O.forward(d, tensors, toks)
    assert rel(O.forward(d, tensors, moved)[-2:], want[-2:]) > 1e3 * F32_TOL, "the far key does not stand out"
    m = build(d, tensors)
    assert rel(run(m, toks, []), want) < F32_TOL
    assert rel(run(m, toks, [250] + list(range(251, 300))), want) < F32_TOL
    assert rel(run(m, toks, [66, 129, 298]), want) < F32_TOL
    assert bf16_ok(run(build(d, tensors, "bfloat16"), toks, [66, 129, 298]), want)


def test_a_far_key_over_key_splits_and_through_generation():
    """1000 cached keys in steps of one to three rows: the keys are split over several CTAs and merged by the last to arrive.
    The standing-out key at tile edges; decoded alone and in portions of two and three rows; then through generation, where
    only the device knows the position."""
    d, tensors, A, B = _key_model()
    n = 1000
    m = build(d, tensors)
    for key_at in (0, 127, 128, 383, 384, 511, 512, 998):
        toks = _with_key(d, n, key_at, A, B, [n - 1, n - 3], seed=13)
        want = O.forward(d, tensors, toks)
        cuts = [950, 952, 955] + list(range(956, n))
        assert rel(run(m, toks, cuts), want) < F32_TOL, key_at
        if key_at in (0, 512):
            assert bf16_ok(run(build(d, tensors, "bfloat16"), toks, cuts), want)
    toks = _with_key(d, n, 280, A, B, [n - 1], seed=14)
    new = O.greedy(d, tensors, toks[:960], 4)
    out = m.generate(torch.tensor([toks[:960]]), max_new_tokens=4, output_logits=True)
    assert out.sequences[0, 960:].tolist() == new
    assert rel(torch.stack(out.logits), O.forward(d, tensors, toks[:960] + new)[959:963]) < F32_TOL
    out.past_key_values.release()


@pytest.mark.parametrize("window", [1, 2, 7, 63, 64, 65, 100, 128, 129, 300])
@pytest.mark.parametrize("inside", [True, False])
def test_keys_just_inside_and_just_outside_the_window(window, inside):
    """Latent attention: the query at position i, the key at i - window + 1 (the last one the window keeps) or at i - window
    (the first one it drops): windows shorter than, equal to and longer than a page, a key tile and the row kernel's range; in
    one prompt, with the query decoded alone, at the start and at the end of short portions, and through the tiled kernels in
    bf16."""
    d, tensors, A, B = _latent_key_model(window)
    n, i = 420, 401
    key_at = i - window + 1 if inside else i - window
    toks = _with_key(d, n, key_at, A, B, [i], seed=11)
    want = O.forward(d, tensors, toks)
    other = O.forward(d, tensors, toks, leave_out=("window",))
    if window > 1:      # (a window of one position holds the query alone)
        gap = rel(other[i:i + 1], want[i:i + 1])
        assert gap < 1e-4 if inside else gap > 0.05, "the test's key does not show the window's edge"
    m = build(d, tensors)
    for cuts in ([], [i] + list(range(i + 1, n)), [key_at + 1, i, i + 2], [i - 1, i + 1], [200, i - 30]):
        assert rel(run(m, toks, cuts), want) < F32_TOL, cuts
    bf = build(d, tensors, "bfloat16")
    assert bf16_ok(run(bf, toks, []), want)
    assert bf16_ok(run(bf, toks, [i] + list(range(i + 1, n))), want)


def test_the_first_tokens_a_window_keeps_and_the_next_ones():
    """Every position of a prompt longer than the window against the oracle, with the first key made to stand out: rows
    0 .. window-1 see it, row `window` is the first that does not."""
    d, tensors, A, B = _latent_key_model(70)
    toks = _with_key(d, 150, 0, A, B, [68, 69, 70, 71], seed=12)
    want = O.forward(d, tensors, toks)
    m = build(d, tensors)
    for cuts in ([], [60] + list(range(61, 150)), [2, 69, 71], [64, 70]):
        assert rel(run(m, toks, cuts), want) < F32_TOL


def test_long_windows_in_steps_of_a_few_rows_split_the_keys():
    """A latent window of 700 positions in steps of one to three rows, the key at the window's first position, just before
    it, and at tile edges; then through generation."""
    d, tensors, A, B = _latent_key_model(700)
    n = 1000
    m = build(d, tensors)
    for key_at in (n - 1 - 700, n - 700, 383, 384, 511, 512, 998):
        toks = _with_key(d, n, key_at, A, B, [n - 1, n - 3], seed=13)
        want = O.forward(d, tensors, toks)
        cuts = [950, 952, 955] + list(range(956, n))
        assert rel(run(m, toks, cuts), want) < F32_TOL, key_at
        if key_at in (n - 700, 512):
            assert bf16_ok(run(build(d, tensors, "bfloat16"), toks, cuts), want)
    toks = _with_key(d, n, 280, A, B, [n - 1], seed=14)
    new = O.greedy(d, tensors, toks[:960], 4)
    out = m.generate(torch.tensor([toks[:960]]), max_new_tokens=4, output_logits=True)
    assert out.sequences[0, 960:].tolist() == new
    assert rel(torch.stack(out.logits), O.forward(d, tensors, toks[:960] + new)[959:963]) < F32_TOL
    out.past_key_values.release()


# ---- long prompts, wide heads, experts ------------------------------------------------------------------------------------
def test_long_prompts_cross_many_key_tiles_and_staging_blocks():
    m, d, _ = model_of("odd")
    toks = K.tokens(333, d["vocab"], seed=50)
    want_lg, want_layers = oracle("odd", toks)
    c = m.new_cache()
    lg, dump = m.forward_step([(c, toks)], [list(range(333))], layer_dump=True)
    c.release()
    for li in range(len(d["layers"])):
        assert rel(dump[li], want_layers[li]) < F32_TOL, f"residual stream after layer {li}"
    assert rel(lg, want_lg) < F32_TOL
    assert rel(run(m, toks, [100, 131, 133, 260, 292]), want_lg) < F32_TOL


@pytest.mark.parametrize("dim,vdim,rot_dims,heads,kv", [(136, 40, 40, 2, 1), (72, 136, 72, 4, 2), (256, 256, 64, 2, 2), (300, 24, 10, 1, 1)])
def test_attention_heads_wider_than_one_tile(dim, vdim, rot_dims, heads, kv):
    d = K.config([K.att(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, rot_dims=rot_dims, scale=dim ** -0.5, mlp=None)], width=32, vocab=64)
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=24)
    toks = K.tokens(215, d["vocab"], seed=52)
    want = O.forward(d, tensors, toks)
    m = build(d, tensors)
    assert rel(run(m, toks, []), want) < F32_TOL
    assert rel(run(m, toks, [64, 128, 129, 193]), want) < F32_TOL
    m = build(d, tensors, "bfloat16")
    assert bf16_ok(run(m, toks, []), want)
    assert bf16_ok(run(m, toks, [64, 129, 193] + list(range(194, 215))), want)


@pytest.mark.parametrize("heads,kv,dim,vdim", [(2, 1, 128, 64), (4, 2, 64, 128), (1, 1, 200, 24), (3, 3, 17, 130), (2, 2, 512, 8)])
def test_delta_rule_heads_of_many_sizes(heads, kv, dim, vdim):
    """Key sizes below, at and above the 16 state entries a thread keeps times the lanes of a warp; value sizes that do and do
    not fill a CTA's columns; in fp32 and bf16 (where the input projection runs on the tensor cores)."""
    d = K.config([K.delta(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, decay_rank=8, gate_rank=8, mlp=None)], width=64, vocab=64)
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=33)
    toks = K.tokens(70, d["vocab"], seed=55)
    want = O.forward(d, tensors, toks)
    m = build(d, tensors)
    assert rel(run(m, toks, []), want) < F32_TOL
    assert rel(run(m, toks, [33, 35] + list(range(50, 70))), want) < F32_TOL
    assert bf16_ok(run(build(d, tensors, "bfloat16"), toks, [40]), want)


def test_many_rows_per_expert_and_experts_without_rows():
    """300 rows over 33 experts (top 5) and over 2 experts (top 1): lists longer than one tile, lists of a few rows, empty
    lists; the same rows decoded one by one take the few-row kernel."""
    m, d, _ = model_of("odd")
    toks = K.tokens(300, d["vocab"], seed=53)
    want = oracle("odd", toks)[0]
    assert rel(run(m, toks, []), want) < F32_TOL
    assert rel(run(m, toks, [280, 290] + list(range(291, 300))), want) < F32_TOL


def test_experts_and_feed_forward_on_the_tensor_cores(monkeypatch):
    """bf16 storage with enough routed rows and 8-aligned shapes: expert lists are padded to whole 128-row tiles and both
    expert products run as one grouped tensor-core GEMM each (the gated activation in the first one's epilogue when the
    expert width is a multiple of 16, as a row kernel when it is not); the dense feed-forward's gelu rides in its first
    product. Against the oracle, against the CUDA-core route, and with the prompt cut so that later portions take the few-row
    route."""
    layers = [K.att(heads=2, kv_heads=1, dim=8, mlp=K.moe(experts=5, top=2, ff=72)),
              K.delta(heads=2, kv_heads=2, dim=8, vdim=8, mlp=K.dense(136)),
              K.lat(heads=4, dim=16, rot_dim=8, vdim=16, kv_rank=64, q_rank=64, window=64, mlp=K.moe(experts=9, top=1, ff=64)),
              K.att(heads=2, kv_heads=2, dim=8, mlp=K.moe(experts=4, top=4, ff=80))]
    d = K.config(layers, width=64, vocab=64)
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=25)
    toks = K.tokens(400, d["vocab"], seed=54)
    want = O.forward(d, tensors, toks)
    m = build(d, tensors, "bfloat16")
    n0 = m.kernel_launches()
    got = run(m, toks, [])
    assert m.kernel_launches() - n0 < 90, "the step took the per-list kernels"
    assert bf16_ok(got, want, routed=True)
    assert bf16_ok(run(m, toks, [300, 390, 395]), want, routed=True)
    monkeypatch.setenv("LIVECC_B200_SEQ_TC", "0")
    assert bf16_ok(run(build(d, tensors, "bfloat16"), toks, []), want, routed=True)
    assert rel(run(build(d, tensors, "float32"), toks, []), want) < F32_TOL


def test_router_weights_are_the_softmax_over_the_chosen_logits():
    """Router rows scaled up so that the chosen logits lie far apart: equal weights and the softmax over the chosen logits
    then differ by orders of magnitude more than the tolerance; top = 1 gives weight 1."""
    d = K.config([K.att(mlp=K.moe(experts=6, top=3, ff=8)), K.att(mlp=K.moe(experts=4, top=1, ff=8))], width=16, vocab=40)
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=34)
    tensors["l0.mlp.router"] *= 4.0
    toks = K.tokens(60, d["vocab"], seed=56)
    want = O.forward(d, tensors, toks)
    assert rel(O.forward(d, tensors, toks, leave_out=("router_weights",)), want) > 100 * F32_TOL
    m = build(d, tensors)
    assert rel(run(m, toks, []), want) < F32_TOL
    assert rel(run(m, toks, [30, 32] + list(range(40, 60))), want) < F32_TOL


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


def test_pages_behind_the_window_go_back_and_freed_pages_and_slots_are_used_again():
    d = K.config([K.lat(window=70, mlp="dense"), K.delta(mlp=None), K.lat(heads=1, dim=4, rot_dim=2, vdim=4, kv_rank=6, q_rank=5, window=20, mlp="moe")], width=24)
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=29)
    m = build(d, tensors, max_tokens=256)
    a, b, c3 = (K.tokens(n, d["vocab"], seed=40 + n) for n in (300, 230, 33))
    want_a, want_b, want_c = (O.forward(d, tensors, t) for t in (a, b, c3))
    ca = m.new_cache()
    got_a = torch.cat([m.forward_step([(ca, a[:200])], [list(range(200))]).cpu(), m.forward_step([(ca, a[200:])], [list(range(100))]).cpu()])
    assert rel(got_a, want_a) < F32_TOL
    # 300 tokens cached, the widest window is 70: the next token reads from position 231, which lies in the fourth page
    assert ca.pages[:3] == [None] * 3 and ca.pages[3] is not None and ca.live_pages() == 2
    slot_a, pages_a = ca.slot, [p for p in ca.pages if p is not None]
    ca.release()
    cb = m.new_cache()
    assert cb.slot == slot_a                    # the slot's recurrent state and carried inputs start from zero again
    got_b = m.forward_step([(cb, b[:150])], [list(range(150))]).cpu()
    cc = m.new_cache()                          # a second live request while b is half way
    got_c = m.forward_step([(cc, c3)], [list(range(len(c3)))]).cpu()
    got_b = torch.cat([got_b] + [m.forward_step([(cb, b[i:i + 2])], [[0, 1]]).cpu() for i in range(150, 230, 2)])
    assert set(pages_a) & set(p for p in cb.pages + cc.pages if p is not None), "the freed pages were not handed out again"
    assert rel(got_b, want_b) < F32_TOL and rel(got_c, want_c) < F32_TOL
    cb.release(); cc.release()
    assert len(m.pool.free) == m.pool.num_pages and len(m.pool.free_slots) == m.pool.num_slots


def test_a_stack_with_plain_attention_keeps_every_page():
    m, d, _ = model_of("mixed")
    c = m.new_cache()
    m.forward_step([(c, K.tokens(200, d["vocab"], seed=44))])
    assert c.live_pages() == 4 and all(p is not None for p in c.pages)
    c.release()


# ---- long decoding, generation ---------------------------------------------------------------------------------------------
def test_long_decoding_stays_on_the_oracle():
    m, d, _ = model_of("odd")
    toks = K.tokens(300, d["vocab"], seed=6)
    want_lg, _ = oracle("odd", toks)
    assert rel(run(m, toks, [4] + list(range(5, 300))), want_lg) < 2 * F32_TOL


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


def test_generation_moves_the_window_across_pages_under_graph_replay():
    """A replayed decode step was captured at position 100; 200 tokens later the latent window (9 positions) has moved across
    three page borders and the recurrent state has taken 200 more writes. Every step's logits against the oracle over the
    generated sequence."""
    m, d, tensors = model_of("mixed")
    prompt = K.tokens(100, d["vocab"], seed=10)
    out = m.generate(torch.tensor([prompt]), max_new_tokens=200, eos_token_id=-1, output_logits=True)
    seq = out.sequences[0].tolist()
    assert len(seq) == 300 and seq[:100] == prompt
    want = O.forward(d, tensors, seq)[99:299]
    assert rel(torch.stack(out.logits), want) < 2 * F32_TOL
    out.past_key_values.release()


@pytest.mark.parametrize("dtype,name", [("float32", "mixed"), ("bfloat16", "latent_only")])
def test_trace_replay_command_line(tmp_path, dtype, name):
    """(bf16 storage on a stack without routers: with only four rows compared, one router choice that falls the other way
    under rounding would decide the result.)"""
    d = K.CASES[name]
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
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", str(mdir), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", "64"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    assert not (out / "1.f32").exists()
    import numpy as np

    la, lb = O.forward(d, tensors, a), O.forward(d, tensors, b)
    g0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4")).reshape(2, -1)
    g2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4")).reshape(1, -1)
    g3 = torch.from_numpy(np.fromfile(out / "3.f32", dtype="<f4")).reshape(1, -1)
    got, want = torch.cat([g0, g2, g3]), torch.cat([la[[0, 32]], la[[49]], lb[[6]]])
    assert rel(got, want) < (F32_TOL if dtype == "float32" else BF16_TOL)
