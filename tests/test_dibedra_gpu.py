"""Dibedra on the GPU against the float64 oracle (tests/dibedra_oracle.py): every mechanism alone and together, whole prompts
against token-by-token decoding, portions down to two tokens, batches against each request alone, pages that the window has
left and pages and slots that are used again, keys far away, at page borders and just inside / just outside the window with
a sharp softmax, the router's correction, groups and identity experts, layers that run with another layer's weights, long
decoding, unusual sizes, and greedy generation through the engine's own entry point. fp32 storage is compared tightly; bf16
storage within bf16 rounding."""
import json
import os
import subprocess

import pytest
import torch

import dibedra_cases as K
import dibedra_oracle as O
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
        _oracle[key] = O.forward(d, tensors, toks, layer_dump=True, **kw)
    return _oracle[key]


def rel(got, want):
    """Largest row error: rms(got - want) / rms(want) over the last axis."""
    got, want = got.double().cpu(), want.double()
    return float(((got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-30)).max())


def bf16_ok(got, want):
    """bf16 storage: a router score close to the next one can fall the other way under rounding and move that row by far
    more than rounding; such rows are allowed to be few, the bulk stays within bf16 rounding."""
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


ALL = ["attention_only", "dense", "moe", "looped", "odd"]


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
        assert rel(dump[li], want_layers[li]) < F32_TOL, f"residual stream after layer {li}"
    assert rel(lg, want_lg) < F32_TOL


@pytest.mark.parametrize("name", ["looped", "odd"])
def test_bf16_storage_stays_within_rounding_on_both_linear_paths(name, monkeypatch):
    _, d, tensors = model_of(name)
    toks = K.tokens(160, d["vocab"], seed=3)
    want_lg, _ = oracle(name, toks)
    for tc in ("1", "0"):                       # tensor-core kernels where the shape allows them / CUDA-core kernels only
        monkeypatch.setenv("LIVECC_B200_SEQ_TC", tc)
        m = build(d, tensors, "bfloat16")
        assert bf16_ok(run(m, toks, []), want_lg)
        assert bf16_ok(run(m, toks, [120] + list(range(121, 160))), want_lg)


def test_the_window_the_correction_and_the_groups_show_in_these_weights():
    """An oracle that lets rows see every earlier key, chooses experts without the correction, or ignores the groups is far
    outside the tolerance: the other tests would notice any of them being left out."""
    m, d, _ = model_of("moe")
    toks = K.tokens(75, d["vocab"])
    got = run(m, toks, [])
    assert rel(got, oracle("moe", toks)[0]) < F32_TOL
    assert rel(got, oracle("moe", toks, window_off=True)[0]) > 100 * F32_TOL
    assert rel(got, oracle("moe", toks, use_correction=False)[0]) > 100 * F32_TOL
    assert rel(got, oracle("moe", toks, use_groups=False)[0]) > 100 * F32_TOL


def test_identity_experts_return_the_normed_row():
    """Every router output but one is an identity expert and the correction forces the choice onto them: the feed-forward
    is then (sum of the chosen scores) x the normed row, exactly; and with the correction reversed, only the one
    real expert is chosen."""
    d = K.config([K.att(mlp=K.moe(experts=1, top=2, ff=8, limit=1.0, identity=3))], width=16, vocab=40)
    for force_identity in (True, False):
        tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=27)
        tensors["l0.mlp.correction"] = torch.tensor([-5.0, 1.0, 2.0, 3.0] if force_identity else [5.0, -1.0, -2.0, -9.0]).to(torch.bfloat16)
        toks = K.tokens(40, d["vocab"], seed=4)
        want = O.forward(d, tensors, toks)
        for dtype in ("float32", "bfloat16"):
            got = run(build(d, tensors, dtype), toks, [30, 32])
            assert rel(got, want) < F32_TOL if dtype == "float32" else bf16_ok(got, want)


@pytest.mark.parametrize("seed", range(10))
def test_random_configurations_in_three_schedules(seed):
    """Random stacks (tests/dibedra_cases.py::random_config): the whole prompt, most of it then token by token, and portions of
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
        assert rel(run(m, toks, cuts), want) < F32_TOL
    got = run(build(d, tensors, "bfloat16"), toks, portions)
    assert bool(torch.isfinite(got).all())
    if len(d["layers"]) <= 3:
        assert bf16_ok(got, want)


# ---- prefill against decoding, portions, first tokens ---------------------------------------------------------------------
@pytest.mark.parametrize("name", ALL)
def test_token_by_token_decoding_equals_the_whole_prompt(name):
    m, d, _ = model_of(name)
    toks = K.tokens(90, d["vocab"], seed=1)
    want_lg, _ = oracle(name, toks)
    assert rel(run(m, toks, range(1, 90)), want_lg) < F32_TOL          # every token alone, from the first one
    assert rel(run(m, toks, [41] + list(range(42, 90))), want_lg) < F32_TOL


@pytest.mark.parametrize("cuts", [[2, 4, 6, 9, 11, 40, 42], [1, 3, 64, 66], [23, 24, 25, 47, 49, 65], [63, 65, 67, 69]])
def test_portions_of_any_size_down_to_two_tokens(cuts):
    m, d, _ = model_of("looped")
    toks = K.tokens(80, d["vocab"], seed=2)
    want_lg, _ = oracle("looped", toks)
    assert rel(run(m, toks, cuts), want_lg) < F32_TOL


def test_first_tokens_of_a_sequence():
    m, d, _ = model_of("looped")
    for n in (1, 2, 3):
        toks = K.tokens(n, d["vocab"], seed=20 + n)
        assert rel(run(m, toks, []), oracle("looped", toks)[0]) < F32_TOL


def test_layers_that_share_weights_keep_caches_of_their_own():
    """Four runs of one attention layer's weights: if they shared a cache, a run would read keys another run wrote."""
    base = [K.att(heads=2, kv_heads=1, dim=8, window=50, mlp="dense")]
    d = K.config(base + [K.shared(base, 0)] * 3, width=16, vocab=40)
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=28)
    assert not any(n.startswith(("l1.", "l2.", "l3.")) for n in tensors)
    toks = K.tokens(100, d["vocab"], seed=5)
    want = O.forward(d, tensors, toks)
    m = build(d, tensors)
    assert rel(run(m, toks, []), want) < F32_TOL
    assert rel(run(m, toks, [60, 62] + list(range(63, 100))), want) < F32_TOL
    # the owner may come later in the stack
    d2 = K.config([K.shared(base, 0), K.att(heads=2, kv_heads=1, dim=8, window=50, mlp="dense")], width=16, vocab=40)
    d2["layers"][0]["weights_of"] = 1
    t2 = synthetic_seq_tensors(SeqModelConfig.from_json(d2), seed=28)
    assert sorted({n.split(".")[0] for n in t2 if n.startswith("l")}) == ["l1"]
    assert rel(run(build(d2, t2), toks, [50]), O.forward(d2, t2, toks)) < F32_TOL


# ---- far keys, page borders, the window's edges ---------------------------------------------------------------------------
def _key_model(window, scale=3.0):
    """One attention layer whose weights make one key stand out: token A (the key) and token B (the query) have one-hot
    embeddings and the norm passes them (zero bias); they reach one un-rotated channel of the key head / of every query head
    through one large weight, and no other token reaches that channel. After the per-head norm B's score against A is about
    dim * scale, against every other key about zero, wherever A sits; A's value row (its un-normed key) is large, so
    whether A is seen changes the output by far more than the tolerance."""
    d = json.loads(json.dumps(K.CASES["sharp"]))
    mx = d["layers"][0]["mixer"]
    mx["mask"]["size"], mx["scale"] = window, scale
    cfg = SeqModelConfig.from_json(d)
    tensors = synthetic_seq_tensors(cfg, seed=22)
    A, B, ja, jb = 5, 9, 3, 11
    D, H, ch = mx["dim"], mx["heads"], mx["dim"] - 1          # the last channel of a head does not turn
    tensors["l0.norm1.b"].zero_()
    tensors["l0.mix.q.norm"].fill_(1.0), tensors["l0.mix.k.norm"].fill_(1.0)
    tensors["embed"][:, ja] = 0.0
    tensors["embed"][:, jb] = 0.0
    for tok, col in ((A, ja), (B, jb)):
        tensors["embed"][tok].zero_()
        tensors["embed"][tok, col] = 2.0
    tensors["l0.mix.k"][ch, :] = 0.0
    tensors["l0.mix.k"][ch, ja] = 20.0
    for h in range(H):
        tensors["l0.mix.q"][h * D + ch, :] = 0.0
        tensors["l0.mix.q"][h * D + ch, jb] = 20.0
    return d, tensors, A, B


def _with_key(d, n, key_at, A, B, query_at, seed):
    toks = [t if t not in (A, B) else 17 for t in K.tokens(n, d["vocab"], seed=seed)]
    toks[key_at] = A
    for q in query_at:
        toks[q] = B
    return toks


@pytest.mark.parametrize("far_at", [0, 1, 62, 63, 64, 65, 127, 128, 200])
def test_a_far_key_among_hundreds_at_page_borders(far_at):
    """A window of 400 positions over a 300-token sequence: A sits once at `far_at` (first tokens, just before / on / after
    a page border, deep inside), B queries it from the end: in one prompt, decoded alone, and at the start of a two-token
    portion; in fp32 and in bf16 on the tensor-core attention."""
    d, tensors, A, B = _key_model(400)
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


@pytest.mark.parametrize("window", [1, 2, 7, 63, 64, 65, 100, 128, 129, 300])
@pytest.mark.parametrize("inside", [True, False])
def test_keys_just_inside_and_just_outside_the_window(window, inside):
    """The query at position i, the key at i - window + 1 (the last one the window keeps) or at i - window (the first one it
    drops): windows shorter than, equal to and longer than a page, a key tile and the row kernel's range; in one prompt, with
    the query decoded alone, at the start and at the end of short portions, and through the tiled kernels in bf16."""
    d, tensors, A, B = _key_model(window)
    n, i = 420, 401
    key_at = i - window + 1 if inside else i - window
    toks = _with_key(d, n, key_at, A, B, [i], seed=11)
    want = O.forward(d, tensors, toks)
    other = O.forward(d, tensors, toks, window_off=True)
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
    d, tensors, A, B = _key_model(70)
    toks = _with_key(d, 150, 0, A, B, [68, 69, 70, 71], seed=12)
    want = O.forward(d, tensors, toks)
    m = build(d, tensors)
    for cuts in ([], [60] + list(range(61, 150)), [2, 69, 71], [64, 70]):
        assert rel(run(m, toks, cuts), want) < F32_TOL


def test_long_windows_in_steps_of_a_few_rows_split_the_keys():
    """A window of 700 positions in steps of one to three rows: the keys are split over several CTAs and merged by the last to
    arrive; the walk starts at the tile that holds the window's first key. The standing-out key sits at the window's first
    position, just before it, and at tile edges; decoded alone and in portions of two and three rows; then through
    generation, where only the device knows the position."""
    d, tensors, A, B = _key_model(700)
    n = 1000
    for key_at in (n - 1 - 700, n - 700, 383, 384, 511, 512, 998):
        toks = _with_key(d, n, key_at, A, B, [n - 1, n - 3], seed=13)
        want = O.forward(d, tensors, toks)
        cuts = [950, 952, 955] + list(range(956, n))
        m = build(d, tensors)
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
def test_long_prompts_cross_many_key_tiles():
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


@pytest.mark.parametrize("dim,rot_dims,heads,kv", [(136, 40, 2, 1), (72, 72, 4, 2), (256, 64, 2, 2), (300, 10, 1, 1)])
def test_heads_wider_than_one_tile(dim, rot_dims, heads, kv):
    """Heads of 136, 72 and 256 channels (several channel steps per key tile, two output tiles), in fp32 and in bf16 on the
    tensor-core attention; heads of 300 channels are beyond its head size and run on the CUDA-core tiles."""
    d = K.config([K.att(heads=heads, kv_heads=kv, dim=dim, window=90, rot_dims=rot_dims, scale=dim ** -0.5, mlp=None)], width=32, vocab=64)
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=24)
    toks = K.tokens(215, d["vocab"], seed=52)
    want = O.forward(d, tensors, toks)
    m = build(d, tensors)
    assert rel(run(m, toks, []), want) < F32_TOL
    assert rel(run(m, toks, [64, 128, 129, 193]), want) < F32_TOL
    m = build(d, tensors, "bfloat16")
    assert bf16_ok(run(m, toks, []), want)
    assert bf16_ok(run(m, toks, [64, 129, 193] + list(range(194, 215))), want)


def test_many_rows_per_expert_and_experts_without_rows():
    """300 rows over 33 experts + 3 identity experts (top 5, 4 of 6 groups) and over 2 experts (top 1): lists longer than one
    tile, lists of a few rows, empty lists; the same rows decoded one by one take the few-row kernel."""
    m, d, _ = model_of("odd")
    toks = K.tokens(300, d["vocab"], seed=53)
    want = oracle("odd", toks)[0]
    assert rel(run(m, toks, []), want) < F32_TOL
    assert rel(run(m, toks, [280, 290] + list(range(291, 300))), want) < F32_TOL


def test_experts_and_feed_forward_on_the_tensor_cores(monkeypatch):
    """bf16 storage with enough routed rows and 8-aligned shapes: expert lists are padded to whole 128-row tiles and both
    expert products run as one grouped tensor-core GEMM each; the dense feed-forward's gelu rides in its first product.
    400 tokens over 5 experts + 1 identity expert and over 9 experts with top 1; against the oracle, against the CUDA-core
    route, and with the prompt cut so that later portions take the few-row route."""
    layers = [K.att(heads=2, kv_heads=1, dim=8, window=40, mlp=K.moe(experts=5, top=2, ff=72, limit=1.0, identity=1)),
              K.att(heads=2, kv_heads=2, dim=8, window=300, mlp=K.dense(136)),
              K.att(heads=4, kv_heads=1, dim=16, window=64, rot_dims=16, mlp=K.moe(experts=9, top=1, ff=64, limit=2.0, identity=0, groups=(3, 2)))]
    d = K.config(layers, width=64, vocab=64)
    tensors = synthetic_seq_tensors(SeqModelConfig.from_json(d), seed=25)
    toks = K.tokens(400, d["vocab"], seed=54)
    want = O.forward(d, tensors, toks)
    m = build(d, tensors, "bfloat16")
    n0 = m.kernel_launches()
    got = run(m, toks, [])
    assert m.kernel_launches() - n0 < 60, "the step took the per-list kernels"
    assert bf16_ok(got, want)
    assert bf16_ok(run(m, toks, [300, 390, 395]), want)
    monkeypatch.setenv("LIVECC_B200_SEQ_TC", "0")
    assert bf16_ok(run(build(d, tensors, "bfloat16"), toks, []), want)
    assert rel(run(build(d, tensors, "float32"), toks, []), want) < F32_TOL


# ---- batches, pages and slots that are used again -----------------------------------------------------------------------------
def test_a_batch_of_unequal_requests_equals_each_alone():
    m, d, _ = model_of("looped")
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
        assert rel(got, oracle("looped", t)[0]) < F32_TOL
    for c in caches:
        c.release()


def test_pages_behind_the_window_go_back_and_freed_pages_are_used_again():
    d = K.config([K.att(window=70, mlp="dense"), K.att(heads=2, kv_heads=2, dim=6, window=20, rot_dims=2, mlp="moe")], width=24)
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
    assert cb.slot == slot_a
    got_b = m.forward_step([(cb, b[:150])], [list(range(150))]).cpu()
    cc = m.new_cache()                          # a second live request while b is half way
    got_c = m.forward_step([(cc, c3)], [list(range(len(c3)))]).cpu()
    got_b = torch.cat([got_b] + [m.forward_step([(cb, b[i:i + 2])], [[0, 1]]).cpu() for i in range(150, 230, 2)])
    assert set(pages_a) & set(p for p in cb.pages + cc.pages if p is not None), "the freed pages were not handed out again"
    assert rel(got_b, want_b) < F32_TOL and rel(got_c, want_c) < F32_TOL
    cb.release(); cc.release()
    assert len(m.pool.free) == m.pool.num_pages and len(m.pool.free_slots) == m.pool.num_slots


# ---- long decoding, generation ---------------------------------------------------------------------------------------------
def test_long_decoding_stays_on_the_oracle():
    m, d, _ = model_of("odd")
    toks = K.tokens(300, d["vocab"], seed=6)
    want_lg, _ = oracle("odd", toks)
    assert rel(run(m, toks, [4] + list(range(5, 300))), want_lg) < 2 * F32_TOL


def test_greedy_generation_through_the_engine_entry_point():
    m, d, tensors = model_of("looped")
    prompt = K.tokens(37, d["vocab"], seed=8)
    want = O.greedy(d, tensors, prompt, 20)
    ids = torch.tensor([prompt])
    out = m.generate(ids, max_new_tokens=20, output_logits=True)
    assert out.sequences[0, :37].tolist() == prompt and out.sequences[0, 37:].tolist() == want
    full, _ = oracle("looped", prompt + want)
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
    bf, _, _ = model_of("looped", "bfloat16")
    got = bf.generate(ids, max_new_tokens=8).sequences[0, 37:].tolist()
    assert len(got) == 8 and all(0 <= t < d["vocab"] for t in got)


def test_generation_moves_the_window_across_pages_under_graph_replay():
    """A replayed decode step was captured at position 100; 200 tokens later every window (17, 10 and 5 positions) has moved
    across three page borders. Every step's logits against the oracle over the generated sequence."""
    m, d, tensors = model_of("looped")
    prompt = K.tokens(100, d["vocab"], seed=10)
    out = m.generate(torch.tensor([prompt]), max_new_tokens=200, eos_token_id=-1, output_logits=True)
    seq = out.sequences[0].tolist()
    assert len(seq) == 300 and seq[:100] == prompt
    want = O.forward(d, tensors, seq)[99:299]
    assert rel(torch.stack(out.logits), want) < 2 * F32_TOL
    out.past_key_values.release()


@pytest.mark.parametrize("dtype,name", [("float32", "looped"), ("bfloat16", "dense")])
def test_trace_replay_command_line(tmp_path, dtype, name):
    """(bf16 storage on the stack without routers: with only four rows compared, one router choice that falls the other way
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
