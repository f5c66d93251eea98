"""The Bamipel decoder on the GPU against the plain implementation of tests/plain_bamipel.py:
each mixer alone, whole prompts, prefill then token by token, portions down to two tokens,
mixed batches over few pages and slots, edges of windows and pages, far keys and far writes, the first
tokens, long decoding, other sizes, and greedy generation through the engine's entry point."""
import numpy as np
import pytest

import bamipel_util as bu
import plain_bamipel as plain
import replay_util as ru

pytestmark = pytest.mark.gpu

# Largest |difference| relative to the largest |logit| of the plain float64 result on the same stored weights,
# and the root mean square of the differences relative to that of the logits.  float32: rounding of float32
# sums only.  bfloat16: activations between kernels are rounded to 8 bits of mantissa.
TOL = {"float32": 1e-4, "bfloat16": 4e-2}
RMS_TOL = {"float32": 2e-5, "bfloat16": 1.5e-2}
LENGTHS = (5, 17, 33, 100, 1, 71, 40, 9)


def rms_err(got, ref):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    return float(np.sqrt(np.mean((got - ref) ** 2)) / (np.sqrt(np.mean(ref ** 2)) + 1e-30))


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, cfg, seed in (("A", bu.BAM_A, 3), ("B", bu.BAM_B, 4)):
        d = bu.write_model(str(tmp_path_factory.mktemp("bamipel" + name)), cfg, seed)
        c, w = plain.load(d)
        seqs = bu.sequences(cfg["vocab"], LENGTHS, seed=11)
        out[name] = (d, cfg, seqs, [plain.forward(c, w, s) for s in seqs])
    return out


def check(got, ref, dtype, what="", rms_tol=None):
    assert sorted(got) == list(range(len(ref)))
    for i in range(len(ref)):
        assert got[i].shape == ref[i].shape
        err, rms = ru.rel_err(got[i], ref[i]), rms_err(got[i], ref[i])
        assert err < TOL[dtype] and rms < (rms_tol or RMS_TOL[dtype]), f"{what} request {i}: relative error {err:.3g}, rms {rms:.3g}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("scheme", ["whole", "prefill_then_decode", "portions", "mixed"])
def test_replay(models, name, dtype, scheme):
    d, cfg, seqs, ref = models[name]
    if scheme == "mixed":
        steps = ru.mixed(seqs, live=4, seed=2)
        # the four longest at once need 100+71+40+33 -> 17 pages of 16 with rounding; slots and pages are used again
        runner = bu.make_runner(d, dtype, max_tokens=17 * 16, context=112)
    else:
        steps = {"whole": ru.whole, "prefill_then_decode": lambda s: ru.prefill_then_decode(s, tail=20),
                 "portions": ru.portions}[scheme](seqs)
        runner = bu.make_runner(d, dtype, max_tokens=112, max_requests=1)
    check(ru.run_in_process(runner, steps), ref, dtype, scheme)


def test_batch_of_unequal_requests_equals_each_alone(models):
    """float32: a row's sums run in one order whatever else is in the batch."""
    d, cfg, seqs, ref = models["A"]
    alone = ru.run_in_process(bu.make_runner(d, "float32", 112, max_requests=1), ru.whole(seqs))
    runner = bu.make_runner(d, "float32", max_tokens=512, max_requests=8, context=112)
    steps = [{"entries": [(i, s, list(range(len(s)))) for i, s in enumerate(seqs)], "end": list(range(len(seqs)))}]
    together = ru.run_in_process(runner, steps)
    for i in range(len(seqs)):
        assert ru.rel_err(together[i], alone[i]) < 2e-6


ALONE = {
    "delta": bu.delta(2, 2, 16, 24, 4),
    "delta_grouped_odd_sizes": bu.delta(6, 2, 20, 12, 2),
    "delta_wide_keys": bu.delta(1, 1, 144, 40, 3),
    "latent": bu.latent(4, 16, 8, 16, 24, 32, window=9, base=100.0, scale=0.5),
    "latent_one_head_no_window": bu.latent(1, 8, 24, 40, 72, 8, window=None, base=1.0e4, scale=0.3),
    "latent_tensor_core_sizes": bu.latent(5, 24, 16, 40, 56, 32, window=21, base=300.0, scale=0.4),
    "latent_many_heads_wide_values": bu.latent(34, 8, 16, 8, 16, 80, window=None, base=50.0, scale=0.3),
    "attention_gqa_small_values": bu.attention(4, 1, 16, 8, 8, 100.0, 0.5),
    "attention_odd_sizes_window": bu.attention(3, 3, 24, 40, 24, 10.0, 0.3, scaling=(2.0, 1.0, 8.0, 16), window=7),
    "attention_tensor_core_sizes": bu.attention(4, 2, 64, 64, 48, 1.0e4, 0.2),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("layer", list(ALONE.values()), ids=list(ALONE))
def test_each_mixer_alone(tmp_path, layer, dtype):
    """One layer without feed-forward: whole, and in portions through the cache or state."""
    cfg = bu.config(48, 90, [layer])
    d = bu.write_model(str(tmp_path), cfg, seed=7)
    c, w = plain.load(d)
    seqs = bu.sequences(90, (37, 3, 64), seed=5)
    ref = [plain.forward(c, w, s) for s in seqs]
    for steps in (ru.whole(seqs), ru.portions(seqs, sizes=(2, 9, 1, 1, 30, 2))):
        check(ru.run_in_process(bu.make_runner(d, dtype, 64, max_requests=1), steps), ref, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_fit_no_vector_access(tmp_path, dtype):
    """Width, vocabulary, ranks and head sizes that are multiples of neither 8 nor 4: every kernel takes its scalar path."""
    layers = [bu.delta(3, 1, 12, 10, 3, ff=36),
              bu.latent(3, 10, 6, 14, 18, 22, window=5, base=77.0, scale=0.4, ff=30),
              bu.attention(2, 1, 12, 10, 6, 300.0, 0.35, scaling=(3.0, 1.0, 5.0, 20))]
    cfg = bu.config(50, 77, layers + [bu.again(layers, 0)], eps=3e-6)
    d = bu.write_model(str(tmp_path), cfg, seed=13)
    c, w = plain.load(d)
    seqs = bu.sequences(77, (41, 2, 19), seed=6)
    ref = [plain.forward(c, w, s) for s in seqs]
    # bfloat16: sums over ten to fifty terms average less of the rounding than the wider models' sums do (measured 1.8e-2;
    # the float32 run of the same kernels' float32 instances holds the usual bound)
    rms_tol = 2.5e-2 if dtype == "bfloat16" else None
    for steps in (ru.whole(seqs), ru.portions(seqs, sizes=(3, 2, 17, 1, 5)), ru.mixed(seqs, live=2, seed=1)):
        check(ru.run_in_process(bu.make_runner(d, dtype, 96, max_requests=2, context=48), steps), ref, dtype, rms_tol=rms_tol)


@pytest.mark.parametrize("taps", [1, 2, 5])
def test_convolution_taps_and_first_tokens(tmp_path, taps):
    """The first tokens of a sequence see zeros in front of it; a portion of one or two tokens is shorter
    than the convolution's history; with one tap there is no history at all."""
    cfg = bu.config(40, 70, [bu.delta(2, 1, 8, 8, taps, ff=48)])
    d = bu.write_model(str(tmp_path), cfg, seed=9)
    c, w = plain.load(d)
    seqs = bu.sequences(70, (9, 2, 1, 30), seed=1)
    ref = [plain.forward(c, w, s) for s in seqs]
    runner = bu.make_runner(d, "float32", 32, max_requests=1)
    for steps in (ru.whole(seqs), ru.portions(seqs, sizes=(1, 1, 2, 1, 3, 17, 2)), ru.prefill_then_decode(seqs, tail=6)):
        check(ru.run_in_process(runner, steps), ref, "float32", f"taps={taps}")
    if taps > 1:        # and the history matters: without the earlier taps the second token's logits differ
        w2 = dict(w)
        for name in ("l0.mix.q.conv", "l0.mix.k.conv", "l0.mix.v.conv"):
            w2[name] = w[name].copy(); w2[name][:, :-1] = 0.0
        assert ru.rel_err(plain.forward(c, w2, seqs[0])[1:], ref[0][1:]) > 100 * TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["latent", "attention"])
def test_window_and_page_edges(tmp_path, dtype, kind):
    """Keys just inside and just outside a sliding window, windows that end inside a page and pages that end inside a
    window, the first tokens (which see fewer keys than a window), for prompt portions that start at, before and
    after an edge and for single decoded tokens.  A large score scale makes single keys dominate."""
    window, page = 24, 16
    make = (lambda wd: bu.latent(2, 16, 16, 16, 16, 16, window=wd, base=30.0, scale=2.5)) if kind == "latent" else \
           (lambda wd: bu.attention(2, 1, 16, 16, 16, 30.0, 1.2, window=wd))
    cfg = bu.config(32, 60, [make(window)])
    d = bu.write_model(str(tmp_path), cfg, seed=21)
    c, w = plain.load(d)
    seq = bu.sequences(60, (100,), seed=2)[0]
    ref = plain.forward(c, w, seq)
    # the edge shows: with the window one position longer, or one shorter, the logits behind the first window change
    for other in (window + 1, window - 1):
        assert ru.rel_err(plain.forward({**c, "layers": [make(other)]}, w, seq)[window:], ref[window:]) > 5 * TOL[dtype]
    cuts = [(100,), (window, window, 100), (window - 1, 2, window - 1, 2, 100), (window + 1, page - 1, 2, 100),
            (page, page, page, 100), (47,) + (1,) * 53, (23,) + (1,) * 77, (2, 2, 100)]
    for sizes in cuts:
        steps = ru.portions([seq], sizes=sizes)
        got = ru.run_in_process(bu.make_runner(d, dtype, 112, page_size=page, max_requests=1), steps)
        assert ru.rel_err(got[0], ref) < TOL[dtype], f"cut {sizes[:5]}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [1, 2, 16, 32, 33])
def test_smallest_and_page_sized_windows(tmp_path, dtype, window):
    """A window of one position (a token sees only itself), of two, of exactly one and two pages, and of one more:
    pages behind the window go back to the pool while the request runs, in prompts and in decoding."""
    layers = [bu.latent(2, 16, 16, 16, 16, 16, window=window, base=30.0, scale=0.5),
              bu.attention(2, 1, 16, 16, 16, 30.0, 0.3, window=window)]
    cfg = bu.config(32, 60, layers)
    d = bu.write_model(str(tmp_path), cfg, seed=23)
    c, w = plain.load(d)
    seqs = bu.sequences(60, (70, 35), seed=4)
    ref = [plain.forward(c, w, s) for s in seqs]
    # the pool is smaller than what the two requests would hold without windows: 5 pages of 16 for 105 tokens
    pool = 80 if window <= 16 else 112
    for steps in (ru.portions(seqs, sizes=(15, 2, 17, 1, 1, 16, 2)), ru.prefill_then_decode(seqs, tail=30)):
        runner = bu.make_runner(d, dtype, pool, page_size=16, max_requests=1, context=80)
        if window <= 16:        # only the windowed groups exist, so the request never holds more than window / 16 + 2 pages
            assert all(g.need.window == window for g in runner.cache.paged)
        check(ru.run_in_process(runner, steps), ref, dtype, f"window={window}")


def _far_sequences(first):
    """Two sequences of 400 tokens that differ in their first ``first`` tokens only (tokens 0 and 1 stand nowhere else)."""
    later = [2 + t % 48 for t in bu.sequences(50, (400 - first,), seed=8)[0]]
    return [t % 2 for t in range(first)] + later, [(t + 1) % 2 for t in range(first)] + later


def _far_check(d, dtype, first=1):
    c, w = plain.load(d)
    seq, other = _far_sequences(first)
    ref, ref_other = plain.forward(c, w, seq), plain.forward(c, w, other)
    effect = ru.rel_err(ref_other[-8:], ref[-8:])
    assert effect > 5 * TOL[dtype]                                       # the far token matters
    # float32: rounding of sums.  bfloat16: every logit here hangs on a handful of rounded numbers (one layer, weights
    # made so that one key or a few writes decide), so the largest difference is held to a tenth of what the far
    # token changes, and the root mean square to the usual bound.
    limit = TOL[dtype] if dtype == "float32" else max(TOL[dtype], effect / 10)
    runner = bu.make_runner(d, dtype, 416, page_size=32, max_requests=1)
    for s, r in ((other, ref_other), (seq, ref)):                        # the same slot and pages twice
        steps = ru.portions([s], sizes=(130, 2, 67, 1, 1, 100, 64)) if s is seq else ru.prefill_then_decode([s], tail=40)
        got = ru.run_in_process(runner, steps)
        assert ru.rel_err(got[0], r) < limit and rms_err(got[0], r) < RMS_TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds(tmp_path, dtype):
    """Causal attention without a window: the first token's key is made to stand out for every later query (along the
    dimensions that are not rotated), so its value shows hundreds of tokens later, across pages, after portions and
    for decoded tokens."""
    cfg = bu.config(32, 50, [bu.attention(2, 2, 16, 8, 8, 1.0e4, 1.0)])

    def marked(tensors):
        bu.mark_first_tokens(tensors)
        wq, wk = tensors["l0.mix.q"], tensors["l0.mix.k"]
        for head in range(2):
            rows = slice(head * 16 + 8, head * 16 + 16)                    # the unrotated half of the head
            wk[rows, bu.FIRST_A] = wk[rows, bu.FIRST_B] = 1.0               # both first tokens: the same loud key
            wk[rows, bu.LATER] = 0.0
            wq[rows, bu.LATER] = 1.0                                        # every later query points at it
    _far_check(bu.write_model(str(tmp_path), cfg, seed=33, edit=marked), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_write_reaches_through_the_state(tmp_path, dtype):
    """A head that hardly forgets and later tokens that hardly write: what the first tokens wrote into the state still
    shows hundreds of tokens later, after portions, decoded tokens, and a slot that another request used before.
    (Five first tokens: a state of rank one would make the normed read-out a sign function of q.k, which no
    rounding survives.)"""
    cfg = bu.config(32, 50, [bu.delta(2, 1, 16, 16, 3)])

    def slow_decay(tensors):
        bu.mark_first_tokens(tensors)
        tensors["l0.mix.A_log"].copy_(torch_tensor([-9.0, -8.0]))
        wb = tensors["l0.mix.b"]
        wb.zero_()
        wb[:, bu.FIRST_A] = wb[:, bu.FIRST_B] = 2.0                         # the first token writes with beta near 1
        wb[:, bu.LATER] = -2.5                                             # every later one with beta near 0
    _far_check(bu.write_model(str(tmp_path), cfg, seed=35, edit=slow_decay), dtype, first=5)


def torch_tensor(values):
    import torch
    return torch.tensor(values, dtype=torch.float32)


def test_gates_norms_and_rotation_order_show_in_the_logits(tmp_path):
    """Variants of the plain implementation that a wrong reading would compute give other logits, so the
    comparison would see them: the norm before the rotation's partial dimensions, a gate per element, no unit norm."""
    cfg = bu.config(32, 40, [bu.attention(2, 1, 16, 8, 8, 5.0, 0.7)])
    d = bu.write_model(str(tmp_path), cfg, seed=5)
    c, w = plain.load(d)
    seq = bu.sequences(40, (30,), seed=3)[0]
    ref = plain.forward(c, w, seq)
    w2 = dict(w); w2["l0.mix.g"] = np.zeros_like(w["l0.mix.g"])           # every gate 1/2
    assert ru.rel_err(plain.forward(c, w2, seq), ref) > 1e-3
    c2 = {**c, "layers": [bu.attention(2, 1, 16, 8, 16, 5.0, 0.7)]}       # all dimensions rotated instead of the first 8
    assert ru.rel_err(plain.forward(c2, w, seq), ref) > 1e-3
    got = ru.run_in_process(bu.make_runner(d, "float32", 32, max_requests=1), ru.whole([seq]))
    assert ru.rel_err(got[0], ref) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_with_graphs(models, dtype):
    """300 tokens one by one behind a short prompt, replayed from CUDA graphs, two requests side by side."""
    d, cfg, _, _ = models["B"]
    c, w = plain.load(d)
    seqs = bu.sequences(cfg["vocab"], (330, 317), seed=4)
    ref = [plain.forward(c, w, s) for s in seqs]
    runner = bu.make_runner(d, dtype, 704, page_size=16, max_requests=2, graphs=True, context=352)
    assert runner.model.graph_safe
    steps = ru.batched_decode(seqs, tails=[300, 300])
    got = ru.run_in_process(runner, steps)
    assert runner.graph_replays > 250
    check(got, ref, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_binary(models, tmp_path, dtype):
    d, cfg, seqs, ref = models["A"]
    steps = ru.mixed(seqs, live=4, seed=5)
    got = ru.run_trace_binary(d, dtype, steps, str(tmp_path), max_tokens=5 * 64, vocab=cfg["vocab"])
    check(got, ref, dtype)


def test_greedy_generation_through_the_engine(models):
    """Engine.generate (scheduler, sampler, pipelined decode) gives the plain implementation's greedy tokens."""
    from hfee_b200 import Engine, SamplingOptions
    d, cfg, seqs, _ = models["A"]
    c, w = plain.load(d)
    prompts = [seqs[0], seqs[1], seqs[7], seqs[2], seqs[6]]
    want = [plain.greedy(c, w, p, 12) for p in prompts]
    eng = Engine(d, dtype="float32", page_size=16, max_context=128, max_requests=3, max_batch_tokens=48, prefill_chunk=11)
    got = [r.token_ids for r in eng.generate(prompts, SamplingOptions.greedy(num_predict=12))]
    assert got == want


def test_command_line_generates(models):
    """``bin/hfee-b200 run`` on a Bamipel folder: greedy tokens of the plain implementation, and a seeded draw
    through the sampling chain that repeats."""
    import os, subprocess, sys
    d, cfg, seqs, _ = models["B"]
    c, w = plain.load(d)
    toks = plain.greedy(c, w, [5, 6, 7], 6)
    exe = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "hfee-b200")
    base = [sys.executable, exe, "run", d, "--prompt-ids", "5,6,7", "--num-predict", "6", "--dtype", "float32", "--num-ctx", "256"]
    p = subprocess.run(base + ["--temperature", "0", "--repeat-penalty", "1"], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr
    assert p.stdout.split("\n")[0].split() == [str(t) for t in toks]
    draws = [subprocess.run(base + ["--temperature", "0.9", "--top-k", "20", "--seed", "7"], capture_output=True, text=True,
                            timeout=300).stdout.split("\n")[0] for _ in range(2)]
    assert draws[0] == draws[1] and len(draws[0].split()) == 6
