"""Kikunex through the product path (bin/trace_run -> registry -> BatchScheduler -> sequence-batch engine and its
kernels) against the plain float64 restatement in tests/kikunex_oracle.py.  Small random models with bf16-representable
weights; --dtype float32 is compared tightly, bfloat16 loosely."""
import subprocess

import numpy as np
import pytest

import kikunex_oracle as ko
from seq_util import rel_err, run_trace, whole

pytestmark = pytest.mark.gpu
TOL32 = 1e-4   # fp32 kernels against float64: rounding only (a lost key, sink or state costs > 1e-2)
TOL16 = 4e-2   # bf16 products


def toks(n, vocab, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, n)]


def ref_logits(cfg, w, tokens):
    return ko.forward(cfg, w, tokens)[0]


def single(rid, tokens, end=False):
    """One step per token."""
    steps = [{"entries": [{"id": rid, "tokens": [x], "want": [0]}]} for x in tokens]
    if end and steps:
        steps[-1]["end"] = [rid]
    return steps


def row_errors(got, ref):
    return np.array([rel_err(got[i:i + 1], ref[i:i + 1]) for i in range(len(ref))])


def assert_rows(got, ref, tol=TOL32):
    err = row_errors(got, ref)
    assert err.max() < tol, f"first bad position {int(np.argmax(err >= tol))} of {len(ref)}, worst {err.max():.3g}"


@pytest.fixture(scope="module")
def base(tmp_path_factory):
    """Both mixers and both feed-forwards, a loop of three passes over two layers, sizes that differ wherever they can
    (query rank and key/value rank, plain and rotated dimensions, key and value sizes, a window that is no multiple of
    a key tile or a page, a linear-attention value size past one column block, groups kept != experts chosen)."""
    layers = [(ko.lightning_mixer(heads=3, dim=8, vdim=12), ko.dense_mlp(40)),
              (ko.latent_mixer(heads=4, dim=12, rot_dim=8, vdim=10, kv_rank=24, q_rank=20, window=21), ko.moe_mlp(6, 2, 16, (3, 2))),
              (ko.lightning_mixer(heads=2, dim=20, vdim=36, decay=[0.97, 0.999]), ko.moe_mlp(8, 3, 12, (4, 3), scale=2.0)),
              (ko.latent_mixer(heads=2, dim=6, rot_dim=4, vdim=14, kv_rank=12, q_rank=28, window=70, base=500.0), None)]
    cfg = ko.make_config(width=48, vocab=61, layers=layers, loop=(1, 3, 3))
    w = ko.make_weights(cfg, seed=1, sharp=2.0)
    return cfg, w, ko.write_model(tmp_path_factory.mktemp("kiku_base"), cfg, w)


# ---- every mechanism on its own -------------------------------------------------------------------------------------
CASES = {
    "latent": [(ko.latent_mixer(), None)],
    "latent_one_head": [(ko.latent_mixer(heads=1, dim=16, rot_dim=2, vdim=5, kv_rank=9, q_rank=7, window=3), None)],
    "latent_window_one": [(ko.latent_mixer(window=1), None)],                      # a token sees itself and the sink
    "latent_window_past_the_prompt": [(ko.latent_mixer(window=500), None)],
    "latent_partly_rotated": [(ko.latent_mixer(rot_dim=12, rot_dims=8), None)],    # the last 4 rotated dimensions pass unchanged
    "latent_unrotated": [(ko.latent_mixer(rot_dim=6, rot_dims=0), None)],
    "latent_wide": [(ko.latent_mixer(heads=3, dim=40, rot_dim=24, vdim=72, kv_rank=136, q_rank=50, window=40, scale=0.2), None)],
    "lightning": [(ko.lightning_mixer(), None)],
    "lightning_one_head": [(ko.lightning_mixer(heads=1, dim=5, vdim=3, decay=[0.9]), None)],
    "lightning_no_decay": [(ko.lightning_mixer(heads=2, dim=8, vdim=8, decay=[1.0, 0.5]), None)],
    "lightning_wide": [(ko.lightning_mixer(heads=2, dim=72, vdim=80, decay=[0.95, 0.9995]), None)],
    "dense_only": [(ko.lightning_mixer(), ko.dense_mlp(56))],
    "moe_only": [(ko.lightning_mixer(), ko.moe_mlp(6, 2, 16, (3, 2)))],
    "moe_no_groups": [(ko.latent_mixer(), ko.moe_mlp(5, 2, 16, None))],
    "moe_top1": [(ko.latent_mixer(), ko.moe_mlp(6, 1, 16, (2, 1), scale=0.75))],
    "moe_groups_of_one": [(ko.latent_mixer(), ko.moe_mlp(6, 2, 16, (6, 3)))],      # a group's score is its only expert's
    "moe_all_groups_kept": [(ko.latent_mixer(), ko.moe_mlp(8, 3, 16, (4, 4)))],
    "moe_many_experts": [(ko.latent_mixer(), ko.moe_mlp(80, 5, 8, (40, 7)))],      # more experts and groups than a warp has lanes
    "moe_all_chosen": [(ko.lightning_mixer(), ko.moe_mlp(4, 4, 16, (2, 2)))],
}


@pytest.mark.parametrize("case", sorted(CASES))
def test_mechanism_alone(tmp_path, case):
    # a large eps in some cases: it must reach every norm (the scalar ones, the latents', the linear attention's)
    big_eps = case in ("latent_one_head", "lightning_one_head", "dense_only", "latent_wide")
    cfg = ko.make_config(width=40, vocab=50, layers=CASES[case], logit_scale=1.0 if "one_head" in case else 0.6,
                         eps=0.05 if big_eps else 3e-6)
    w = ko.make_weights(cfg, seed=3, sharp=3.0)
    if case in ("dense_only", "moe_only"):  # the mixer's output projection is zero: what is left of the layer is the feed-forward
        w["l0.mix.o"] = np.zeros_like(w["l0.mix.o"])
    if case == "moe_only":                  # choice scores below zero too: a dropped group must count as -inf, not 0
        w["l0.mlp.correction"] = ko.bf16_round(w["l0.mlp.correction"] - 1.0)
    d = ko.write_model(tmp_path, cfg, w)
    t = toks(75, cfg["vocab"], 5)
    ref, trace = ko.forward(cfg, w, t)
    logits, resid = run_trace(d, [whole("a", t)], residual=True)
    got = resid[0].reshape(trace.shape)
    assert np.abs(got - trace).max() < 1e-4 * max(1.0, np.abs(trace).max())
    assert_rows(logits[0], ref)


def test_residual_after_every_layer_run(base):
    cfg, w, d = base
    t = toks(33, cfg["vocab"], 7)
    _, trace = ko.forward(cfg, w, t)
    assert trace.shape[0] == 1 + 2 * 3 + 1
    _, resid = run_trace(d, [whole("a", t)], residual=True)
    got = resid[0].reshape(trace.shape)
    for r in range(trace.shape[0]):
        assert np.abs(got[r] - trace[r]).max() < 1e-4 * max(1.0, np.abs(trace[r]).max()), f"layer run {r}"


@pytest.mark.parametrize("loop,runs", [((0, 2, 3), 7), ((1, 2, 1), 3), ((0, 3, 2), 6), ((2, 3, 4), 6), (None, 3)])
def test_loop_shapes(tmp_path, loop, runs):
    """Three passes, one pass (its vector is still added, the embedding output is not), a loop over every layer, a loop
    at the end, no loop: every pass has a cache and a state of its own."""
    layers = [(ko.latent_mixer(window=9), ko.dense_mlp(24)), (ko.lightning_mixer(), ko.moe_mlp(4, 2, 8, (2, 1))),
              (ko.latent_mixer(heads=2, window=30), None)]
    cfg = ko.make_config(width=40, vocab=60, layers=layers, loop=loop)
    w = ko.make_weights(cfg, seed=101, sharp=2.0)
    d = ko.write_model(tmp_path, cfg, w)
    t = toks(45, cfg["vocab"], 102)
    ref, trace = ko.forward(cfg, w, t)
    assert trace.shape[0] == runs
    logits, resid = run_trace(d, [whole("a", t[:30], end=False)] + single("a", t[30:]), residual=True)
    got = resid[0].reshape(runs, 30, cfg["width"])
    for r in range(runs):
        assert np.abs(got[r] - trace[r][:30]).max() < 1e-4 * max(1.0, np.abs(trace[r]).max()), r
    assert_rows(np.concatenate(logits), ref)


# ---- whole prompts; windows, tiles and pages ------------------------------------------------------------------------
@pytest.mark.parametrize("page", [4, 16, 64])
def test_long_prompt_every_position(base, page):
    cfg, w, d = base
    t = toks(203, cfg["vocab"], 11)  # past three key tiles of 64 and six chunks of the recurrence, no multiple of a page
    logits, _ = run_trace(d, [whole("a", t)], page=page)
    assert_rows(logits[0], ref_logits(cfg, w, t))


@pytest.mark.parametrize("window", [2, 17, 64, 65, 100])
def test_the_key_at_the_window_edge_carries_the_output(tmp_path, window):
    """One token's key is made to win every softmax it takes part in: the queries are sharp and that token's latent is
    large along the direction all queries look at.  While it is inside the window the output is its value; from the
    position where it leaves, the output changes completely.  It is placed so that it leaves inside the prompt, and a
    second one so that it leaves while tokens are decoded one by one (across key tiles and pages)."""
    m = ko.latent_mixer(heads=2, dim=8, rot_dim=4, vdim=6, kv_rank=10, q_rank=8, window=window, scale=1.0)
    cfg = ko.make_config(width=24, vocab=30, layers=[(m, None)])
    w = ko.make_weights(cfg, seed=9, sharp=1.0)
    w["l0.shift"] = np.zeros_like(w["l0.shift"])
    special = 7
    n_prompt, n_all = 150, 150 + window + 20
    t = [x if x != special else special + 1 for x in toks(n_all, cfg["vocab"], 13)]
    t[20] = special            # leaves the window inside the prompt
    t[n_prompt - 5] = special  # leaves it during decoding
    # every query looks along latent coordinate 0 (the rotated part and the other coordinates are switched off); the
    # special token's latent is almost purely coordinate 0, every other token's has none of it
    w["l0.mix.uq"] = np.zeros_like(w["l0.mix.uq"])
    w["l0.mix.dq.norm"] = np.ones_like(w["l0.mix.dq.norm"])
    w["l0.mix.uq"][0::12, :] = 0.5          # the first plain dimension of each head reads the whole query latent
    w["l0.mix.uk"] = np.zeros_like(w["l0.mix.uk"])
    w["l0.mix.uk"][0::8, 0] = 4.0           # ... and is matched by latent coordinate 0
    w["l0.mix.dq"] = np.abs(w["l0.mix.dq"])
    w["embed"] = np.abs(w["embed"])         # positive embeddings x positive W_dq: the query latent is positive
    w["l0.mix.dkv"][0] = 0.0
    w["l0.mix.dkv"][0, 0] = 8.0
    w["embed"][:, 0] = 0.0
    w["embed"][special, 0] = 4.0
    ref = ref_logits(cfg, w, t)
    # the construction works: logits right after the special key leaves differ from those right before
    for p in (20, n_prompt - 5):
        assert rel_err(ref[p + window:p + window + 1], ref[p + window - 1:p + window]) > 0.1
    d = ko.write_model(tmp_path, cfg, w)
    logits, _ = run_trace(d, [whole("a", t[:n_prompt], end=False)] + single("a", t[n_prompt:]), page=16)
    assert_rows(np.concatenate(logits), ref)


def test_the_sink_takes_its_share(tmp_path):
    """Large sinks: most of the softmax mass goes to them, so leaving one out (or scaling it) multiplies the output."""
    cfg = ko.make_config(width=32, vocab=40, layers=[(ko.latent_mixer(heads=3, window=12), None)])
    w = ko.make_weights(cfg, seed=21)
    w["l0.mix.sink"] = np.array([4.0, -3.0, 1.5])
    d = ko.write_model(tmp_path, cfg, w)
    t = toks(40, cfg["vocab"], 22)
    logits, _ = run_trace(d, [whole("a", t[:25], end=False)] + single("a", t[25:]))
    assert_rows(np.concatenate(logits), ref_logits(cfg, w, t))


def test_far_tokens_stay_in_the_recurrent_state(tmp_path):
    """Only the first token has a key at all (the key projection reads one input coordinate, which only that token's
    embedding has; no token shift), so the state is its key times its value for ever -- undecayed in one head, slowly
    decaying in the other -- and every later output comes from it alone: hundreds of tokens, several chunks, two
    portions and many single steps later."""
    cfg = ko.make_config(width=32, vocab=40, layers=[(ko.lightning_mixer(heads=2, dim=8, vdim=8, decay=[1.0, 0.999]), None)])
    w = ko.make_weights(cfg, seed=31)
    special = 5
    t = [x if x != special else special + 1 for x in toks(330, cfg["vocab"], 32)]
    t[0] = special
    w["l0.shift"] = np.zeros_like(w["l0.shift"])
    w["embed"][:, 0] = 0.0
    w["embed"][special, 0] = 4.0
    w["l0.mix.k"][:, 1:] = 0.0
    w["l0.mix.k"][:, 0] = ko.bf16_round(np.abs(w["l0.mix.k"][:, 0]) + 1.0)
    ref = ref_logits(cfg, w, t)
    t2 = list(t)
    t2[0] = special + 1
    assert rel_err(ref_logits(cfg, w, t2)[-1:], ref[-1:]) > 1e-2  # the construction works
    d = ko.write_model(tmp_path, cfg, w)
    steps = [whole("a", t[:200], end=False), whole("a", t[200:300], end=False)] + single("a", t[300:])
    logits, _ = run_trace(d, steps)
    assert_rows(np.concatenate(logits), ref)


# ---- prompt against token-by-token decoding, long decoding ----------------------------------------------------------
def test_prefill_equals_stepwise_decoding(base):
    cfg, w, d = base
    t = toks(90, cfg["vocab"], 17)
    ref = ref_logits(cfg, w, t)
    split = [whole("p", t[:2], end=False)] + single("p", t[2:])
    logits, _ = run_trace(d, single("s", t) + split, page=8)   # "s": from the very first token
    a, b = np.concatenate(logits[:len(t)]), np.concatenate(logits[len(t):])
    assert_rows(a, ref)
    assert_rows(b, ref)
    assert_rows(a, b)


def test_long_decoding(base):
    """Decoding far past every window, key tile, page and chunk size."""
    cfg, w, d = base
    t = toks(40 + 260, cfg["vocab"], 19)
    logits, _ = run_trace(d, [whole("a", t[:40], end=False)] + single("a", t[40:]), page=16)
    assert_rows(np.concatenate(logits), ref_logits(cfg, w, t))


@pytest.mark.parametrize("sizes", [(2, 2, 2, 2), (5, 64, 3, 17), (33, 2, 70), (1, 99, 2)])
def test_prompt_in_portions(base, sizes):
    """A prompt fed in several steps: every portion starts from the cache, the shift state and the recurrent state the
    portions before it left.  A second request of another length rides along."""
    cfg, w, d = base
    t = toks(sum(sizes), cfg["vocab"], 81)
    other = toks(2 * len(sizes) + 1, cfg["vocab"], 82)
    steps, at = [], 0
    for i, n in enumerate(sizes):
        o = other[2 * i:2 * i + 2] if i + 1 < len(sizes) else other[2 * i:]
        steps.append({"entries": [{"id": "o", "tokens": o, "want": list(range(len(o)))},
                                  {"id": "p", "tokens": t[at:at + n], "want": list(range(n))}]})
        at += n
    logits, _ = run_trace(d, steps, page=8, max_tokens=512)
    got_o = np.concatenate([lg[:len(st["entries"][0]["tokens"])] for lg, st in zip(logits, steps)])
    got_p = np.concatenate([lg[len(st["entries"][0]["tokens"]):] for lg, st in zip(logits, steps)])
    assert_rows(got_p, ref_logits(cfg, w, t))
    assert_rows(got_o, ref_logits(cfg, w, other))


# ---- batches ----------------------------------------------------------------------------------------------------------
def test_unequal_batch_equals_each_alone(base):
    cfg, w, d = base
    prompts = {"x": toks(1, cfg["vocab"], 21), "y": toks(67, cfg["vocab"], 22), "z": toks(130, cfg["vocab"], 23)}
    tails = {k: toks(n, cfg["vocab"], 30 + i) for i, (k, n) in enumerate({"x": 3, "y": 30, "z": 7}.items())}
    steps = [{"entries": [{"id": k, "tokens": p, "want": list(range(len(p)))} for k, p in prompts.items()]}]
    for j in range(30):
        live = [k for k in prompts if j < len(tails[k])]
        steps.append({"entries": [{"id": k, "tokens": [tails[k][j]], "want": [0]} for k in live],
                      "end": [k for k in live if j == len(tails[k]) - 1]})
    logits, _ = run_trace(d, steps, page=8, max_tokens=320)
    for k in prompts:
        rows, at = [], 0
        for kk, p in prompts.items():
            if kk == k:
                rows.append(logits[0][at:at + len(p)])
            at += len(p)
        for j in range(len(tails[k])):
            live = [kk for kk in prompts if j < len(tails[kk])]
            rows.append(logits[1 + j][live.index(k)][None])
        assert_rows(np.concatenate(rows), ref_logits(cfg, w, prompts[k] + tails[k]))


def test_pages_slots_and_states_are_reused(base):
    """The pool holds one request at a time: each runs in the pages, the slot and the state memory that the one before
    it gave back, and must see nothing of it."""
    cfg, w, d = base
    reqs = [toks(n, cfg["vocab"], 40 + i) for i, n in enumerate([50, 33, 64, 7, 50])]
    steps = []
    for i, t in enumerate(reqs):
        steps.append(whole(f"r{i}", t[:-3], end=False))
        steps += single(f"r{i}", t[-3:], end=True)
    logits, _ = run_trace(d, steps, page=4, max_tokens=64, extra=["--max-seqs", "1"])
    at = 0
    for t in reqs:
        assert_rows(np.concatenate(logits[at:at + 4]), ref_logits(cfg, w, t))
        at += 4


def test_a_freed_slot_restarts_from_an_empty_state(base):
    """Two slots; requests come and go in an order that hands a slot with a long history to a request that starts by
    decoding from its first token."""
    cfg, w, d = base
    a, b, c = toks(80, cfg["vocab"], 61), toks(12, cfg["vocab"], 62), toks(9, cfg["vocab"], 63)
    steps = [{"entries": [{"id": "a", "tokens": a, "want": [79]}, {"id": "b", "tokens": b[:6], "want": [5]}], "end": ["a"]}]
    for j in range(6):  # c takes a's slot and decodes from its first token beside b
        steps.append({"entries": [{"id": "b", "tokens": [b[6 + j]], "want": [0]}, {"id": "c", "tokens": [c[j]], "want": [0]}]})
    logits, _ = run_trace(d, steps, max_tokens=128, extra=["--max-seqs", "2"])
    got_b = np.concatenate([logits[0][1:2]] + [lg[0:1] for lg in logits[1:]])
    got_c = np.concatenate([lg[1:2] for lg in logits[1:]])
    assert_rows(got_b, ref_logits(cfg, w, b)[5:])
    assert_rows(got_c, ref_logits(cfg, w, c)[:6])
    assert_rows(logits[0][0:1], ref_logits(cfg, w, a)[79:])


def test_first_tokens_and_single_token_requests(base):
    cfg, w, d = base
    ts = [toks(n, cfg["vocab"], 50 + n) for n in (1, 2, 3)]
    logits, _ = run_trace(d, [whole(f"q{i}", t) for i, t in enumerate(ts)])
    for t, lg in zip(ts, logits):
        assert_rows(lg, ref_logits(cfg, w, t))


def test_many_requests_in_one_batch(base):
    """80 prompts of 1..5 tokens in one step, then decoded together."""
    cfg, w, d = base
    reqs = [toks(1 + i % 5, cfg["vocab"], 200 + i) + toks(2, cfg["vocab"], 400 + i) for i in range(80)]
    steps = [{"entries": [{"id": f"r{i}", "tokens": r[:-2], "want": [len(r) - 3]} for i, r in enumerate(reqs)]}]
    for j in (2, 1):
        steps.append({"entries": [{"id": f"r{i}", "tokens": [r[-j]], "want": [0]} for i, r in enumerate(reqs)]})
    logits, _ = run_trace(d, steps, max_tokens=1024)
    for i, r in enumerate(reqs):
        got = np.stack([logits[0][i], logits[1][i], logits[2][i]])
        assert_rows(got, ref_logits(cfg, w, r)[-3:])


# ---- bf16, other sizes, generation ------------------------------------------------------------------------------------
def test_bfloat16_products(tmp_path):
    """bf16 products round the router's input too: every expert is chosen, so that no routing flip drowns the comparison."""
    layers = [(ko.lightning_mixer(heads=3, dim=8, vdim=12), ko.dense_mlp(40)),
              (ko.latent_mixer(window=21), ko.moe_mlp(4, 4, 16, (2, 2))),
              (ko.lightning_mixer(heads=2, dim=20, vdim=36), None)]
    cfg = ko.make_config(width=72, vocab=101, layers=layers, loop=(0, 2, 2))
    w = ko.make_weights(cfg, seed=5)
    d = ko.write_model(tmp_path, cfg, w)
    t = toks(140, cfg["vocab"], 61)
    logits, _ = run_trace(d, [whole("a", t[:120], end=False)] + single("a", t[120:]), dtype="bfloat16")
    assert rel_err(np.concatenate(logits), ref_logits(cfg, w, t)) < TOL16


@pytest.mark.parametrize("dims,window", [((24, 8, 40), 17), ((104, 24, 72), 64), ((136, 56, 128), 150)])
def test_bfloat16_prompts_on_the_tensor_cores(tmp_path, dims, window):
    """Prompt steps that start their sequences expand the latents into per-head keys and values and take the tensor-core
    attention (head sizes that are multiples of 8); single-token steps score against the cached latents.  Both see the
    same bf16 inputs, so they agree far more tightly than either agrees with float64 -- a key lost at a window's or a
    tile's edge, or a forgotten sink, would not.  A ragged batch: requests of 1, 70 and 200 tokens."""
    dim, rot, vdim = dims
    layers = [(ko.latent_mixer(heads=3, dim=dim, rot_dim=rot, vdim=vdim, kv_rank=48, q_rank=40, window=window), None),
              (ko.latent_mixer(heads=2, dim=dim, rot_dim=rot, vdim=vdim, kv_rank=32, q_rank=24, window=2 * window + 3),
               ko.dense_mlp(64))]
    cfg = ko.make_config(width=64, vocab=90, layers=layers, loop=(0, 1, 2))
    w = ko.make_weights(cfg, seed=91, sharp=2.0)
    d = ko.write_model(tmp_path, cfg, w)
    reqs = {"a": toks(1, 90, 92), "b": toks(70, 90, 93), "c": toks(200, 90, 94)}
    block = [{"entries": [{"id": k, "tokens": reqs[k], "want": list(range(len(reqs[k])))} for k in "abc"], "end": ["a", "b", "c"]}]
    steps = block + [st for k in "abc" for st in single(k + "1", reqs[k], end=True)]
    logits, _ = run_trace(d, steps, dtype="bfloat16", page=16, max_tokens=512)
    got_block, got_single = logits[0], np.concatenate(logits[1:])
    ref = np.concatenate([ref_logits(cfg, w, reqs[k]) for k in "abc"])
    assert rel_err(got_block, ref) < TOL16 and rel_err(got_single, ref) < TOL16
    err = row_errors(got_block, got_single)
    assert err.max() < 1.5e-2, f"first bad row {int(np.argmax(err >= 1.5e-2))}"


@pytest.mark.parametrize("dtype,tol", [("float32", TOL32), ("bfloat16", TOL16)])
def test_sizes_that_fit_no_vector(tmp_path, dtype, tol):
    """Width, ranks, inner sizes and head sizes that are not multiples of 8 (nor of 4): no 16-byte row anywhere."""
    layers = [(ko.latent_mixer(heads=3, dim=7, rot_dim=6, vdim=5, kv_rank=11, q_rank=13, window=19), ko.moe_mlp(3, 3, 10, None)),
              (ko.lightning_mixer(heads=3, dim=5, vdim=7), ko.dense_mlp(22))]
    cfg = ko.make_config(width=44, vocab=77, layers=layers, loop=(0, 1, 2))
    w = ko.make_weights(cfg, seed=111)
    d = ko.write_model(tmp_path, cfg, w)
    t = toks(110, cfg["vocab"], 112)
    logits, _ = run_trace(d, [whole("a", t[:100], end=False)] + single("a", t[100:]), dtype=dtype)
    assert rel_err(np.concatenate(logits), ref_logits(cfg, w, t)) < tol


def test_larger_shapes_take_the_block_paths(tmp_path):
    """Enough tokens and wide enough layers for the tiled and grouped products (and, in bf16, the tensor-core ones)."""
    layers = [(ko.latent_mixer(heads=8, dim=32, rot_dim=16, vdim=32, kv_rank=64, q_rank=96, window=100), ko.moe_mlp(8, 2, 128, (4, 2))),
              (ko.lightning_mixer(heads=4, dim=32, vdim=64), ko.dense_mlp(512))]
    cfg = ko.make_config(width=256, vocab=300, layers=layers, loop=(0, 2, 2))
    w = ko.make_weights(cfg, seed=77, sharp=2.0)
    d = ko.write_model(tmp_path, cfg, w)
    t = toks(300, cfg["vocab"], 78)
    ref = ref_logits(cfg, w, t)
    want = list(range(0, 300, 7)) + [299]
    for dtype, tol in (("float32", TOL32), ("bfloat16", TOL16)):
        logits, _ = run_trace(d, [whole("a", t, want=want)], dtype=dtype)
        err = row_errors(logits[0], ref[want])
        if dtype == "float32":
            assert err.max() < tol
        else:  # two of eight experts: bf16 rounding of the router's input flips a close choice now and then
            assert np.median(err) < tol / 2 and (err > tol).mean() <= 0.1 and err.max() < 4 * tol, np.sort(err)[-5:]


def random_design(seed):
    """A model of the size a checkpoint of this family might have: every size and constant drawn, layer order too."""
    rng = np.random.default_rng(seed)
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]  # noqa: E731
    layers = []
    for _ in range(int(rng.integers(4, 8))):
        if rng.random() < 0.5:
            m = ko.latent_mixer(heads=pick(2, 4, 6, 8), dim=pick(16, 24, 32, 48), rot_dim=pick(8, 16, 32), vdim=pick(16, 40, 48, 64),
                                kv_rank=pick(32, 48, 80, 128), q_rank=pick(24, 64, 112), window=int(rng.integers(5, 130)),
                                base=float(pick(1e4, 1e5, 1e6)))
        else:
            H = pick(2, 3, 4, 6)
            m = ko.lightning_mixer(heads=H, dim=pick(16, 32, 48), vdim=pick(16, 32, 64),
                                   decay=[float(x) for x in np.exp(-1.0 / rng.uniform(1.5, 900.0, H))])
        r = rng.random()
        if r < 0.25:
            f = None
        elif r < 0.5:
            f = ko.dense_mlp(pick(96, 160, 320))
        else:
            count = pick(2, 3, 4)
            f = ko.moe_mlp(count * pick(2, 3, 4), pick(1, 2, 3, 4), pick(32, 48, 96), (count, int(rng.integers(1, count + 1))),
                           scale=float(rng.uniform(0.5, 3.0)))
            f["router"]["top"] = min(f["router"]["top"], f["router"]["groups"]["keep"] * f["router"]["experts"] // count)
        layers.append((m, f))
    n = len(layers)
    start = int(rng.integers(0, n))
    loop = (start, int(rng.integers(start + 1, n + 1)), int(rng.integers(1, 4))) if rng.random() < 0.8 else None
    cfg = ko.make_config(width=pick(96, 160, 224), vocab=int(rng.integers(200, 500)), layers=layers, loop=loop,
                         eps=float(pick(1e-6, 1e-5, 1e-4)), logit_scale=float(rng.uniform(0.3, 1.5)))
    return cfg, ko.make_weights(cfg, seed=1000 + seed, sharp=1.5)


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5])
def test_random_designs(tmp_path, seed):
    """Whole prompts of unequal requests in one batch, then decoded together until the shorter ones end, in both
    compute types."""
    cfg, w = random_design(seed)
    d = ko.write_model(tmp_path, cfg, w)
    V = cfg["vocab"]
    reqs = {"a": toks(150, V, seed), "b": toks(37, V, seed + 10), "c": toks(1, V, seed + 20)}
    tails = {"a": toks(40, V, seed + 30), "b": toks(25, V, seed + 40), "c": toks(9, V, seed + 50)}
    steps = [{"entries": [{"id": k, "tokens": reqs[k], "want": list(range(len(reqs[k])))} for k in "abc"]}]
    for j in range(40):
        live = [k for k in "abc" if j < len(tails[k])]
        steps.append({"entries": [{"id": k, "tokens": [tails[k][j]], "want": [0]} for k in live],
                      "end": [k for k in live if j == len(tails[k]) - 1]})
    refs = {k: ref_logits(cfg, w, reqs[k] + tails[k]) for k in "abc"}
    for dtype in ("float32", "bfloat16"):
        logits, _ = run_trace(d, steps, dtype=dtype, max_tokens=400)
        loose = []
        for k in "abc":
            rows, at = [], 0
            for kk in "abc":
                if kk == k:
                    rows.append(logits[0][at:at + len(reqs[kk])])
                at += len(reqs[kk])
            for j in range(len(tails[k])):
                live = [kk for kk in "abc" if j < len(tails[kk])]
                rows.append(logits[1 + j][live.index(k)][None])
            got = np.concatenate(rows)
            if dtype == "float32":
                assert_rows(got, refs[k])
            else:
                loose.append(row_errors(got, refs[k]))
        if loose:  # a close routing choice flips under bf16 rounding now and then: it touches that row and, fading, the next
            err = np.concatenate(loose)
            assert np.median(err) < TOL16 / 2 and (err > TOL16).mean() <= 0.05, np.sort(err)[-5:]


def test_greedy_generation_through_the_scheduler(base):
    from kuiperllama_b200 import build
    cfg, w, d = base
    tools = build.build_seq_tools()
    prompts = [toks(9, cfg["vocab"], 71), toks(30, cfg["vocab"], 72), toks(2, cfg["vocab"], 73)]
    cmd = [str(tools / "kuiper_generate"), "--model", str(d), "--dtype", "float32", "--new", "12", "--page", "8"]
    for p in prompts:
        cmd += ["--prompt", " ".join(map(str, p))]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    got = [[int(x) for x in ln.split()] for ln in r.stdout.strip().splitlines()]
    for p, g in zip(prompts, got):
        assert g == ko.greedy(cfg, w, p, 12)
