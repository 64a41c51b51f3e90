"""Fobolorn through the product path (bin/trace_run -> registry -> BatchScheduler -> sequence-batch engine and its
kernels) against the plain float64 restatement in tests/fobolorn_oracle.py.  Small random models, bf16-representable
weights; --dtype float32 is compared tightly, bfloat16 loosely."""
import numpy as np
import pytest
import torch

from fobolorn_oracle import forward, greedy, make_config, make_weights, write_model
from seq_util import ROOT, rel_err, run_trace, whole

pytestmark = pytest.mark.gpu
TOL32 = 1e-4   # fp32 kernels against float64: rounding only (peaky softmax amplifies it; a lost key costs > 1e-2)
TOL16 = 4e-2   # bf16 products


def toks(n, vocab, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, n)]


def ref_logits(cfg, w, tokens):
    return forward(cfg, w, tokens).numpy()


@pytest.fixture(scope="module")
def base(tmp_path_factory):
    """Two different layers, a loop over one of them, odd sizes (dim not a multiple of 4, a value size between one
    and two key tiles of columns), a temperature step every 5 positions."""
    cfg = make_config(width=72, vocab=101, layers=3, heads=6, kv_heads=2, dim=18, vdim=40, experts=5, top=2, ff=24,
                      shared_ff=40, loop=(1, 3, 2), q_temp=(0.4, 5))
    cfg["layers"][2]["mixer"].update(heads=3, kv_heads=3, dim=32, vdim=72)          # no grouping, wide values
    cfg["layers"][1]["mlp"]["router"].update(experts=3, top=3)                       # every expert chosen
    w = make_weights(cfg, seed=1, sharp=2.5)
    d = write_model(tmp_path_factory.mktemp("fobo_base"), cfg, w)
    return cfg, w, d


# ---- every mechanism on its own -------------------------------------------------------------------------------------
def one_layer(tmp_path, **kw):
    cfg = make_config(layers=1, **kw)
    w = make_weights(cfg, seed=3, sharp=3.0)
    return cfg, w, write_model(tmp_path, cfg, w)


@pytest.mark.parametrize("case", ["attention_only", "no_temperature", "no_shared", "experts_only", "top1", "mha",
                                  "one_kv_head", "scale_const", "many_experts", "big_heads"])
def test_mechanism_alone(tmp_path, case):
    kw = dict(width=48, vocab=50, heads=4, kv_heads=2, dim=12, vdim=20, experts=4, top=2, ff=16, shared_ff=24)
    if case == "attention_only":
        kw.update(mlp=False)
    elif case == "no_temperature":
        kw.update(q_temp=None)
    elif case == "no_shared":
        kw.update(shared_ff=0)
    elif case == "top1":
        kw.update(top=1, router_scale=0.75)
    elif case == "mha":
        kw.update(kv_heads=4)
    elif case == "one_kv_head":
        kw.update(kv_heads=1)
    elif case == "scale_const":
        kw.update(scale=0.31)
    elif case == "many_experts":  # more experts than a warp has lanes
        kw.update(experts=40, top=5)
    elif case == "big_heads":     # past the sizes the tensor-core attention is compiled for
        kw.update(dim=136, vdim=200, heads=2, kv_heads=1)
    cfg, w, d = one_layer(tmp_path, **kw)
    if case == "experts_only":  # the mixer's output projection is zero: what is left of the layer is the feed-forward
        w["l0.mix.o"] = torch.zeros_like(w["l0.mix.o"])
        write_model(d, cfg, w)
    t = toks(37, cfg["vocab"], 5)
    resid_ref = []
    ref = forward(cfg, w, t, resid_ref).numpy()
    logits, resid = run_trace(d, [whole("a", t)], residual=True)
    got_resid = resid[0].reshape(1, len(t), cfg["width"])
    assert np.abs(got_resid[0] - resid_ref[0].numpy()).max() < 2e-4
    assert rel_err(logits[0], ref) < TOL32


def test_residual_after_every_layer_run(base):
    cfg, w, d = base
    t = toks(29, cfg["vocab"], 7)
    resid_ref = []
    forward(cfg, w, t, resid_ref)
    _, resid = run_trace(d, [whole("a", t)], residual=True)
    got = resid[0].reshape(len(resid_ref), len(t), cfg["width"])
    assert len(resid_ref) == 1 + 2 * 2  # layer 0, then layers 1..2 twice
    for r, ref in enumerate(resid_ref):
        assert np.abs(got[r] - ref.numpy()).max() < 1e-4 * max(1.0, float(ref.abs().max())), f"layer run {r}"


@pytest.mark.parametrize("loop,runs", [((0, 2, 3), 7), ((1, 2, 1), 3), ((0, 3, 2), 6), ((2, 3, 4), 6), (None, 3)])
def test_loop_shapes(tmp_path, loop, runs):
    """Three passes, a single pass (its vector is still added once), a loop over every layer, a loop at the end, no loop:
    every pass has a cache of its own, and the pass vector is added once, right before the pass's first layer."""
    cfg = make_config(width=40, vocab=60, layers=3, heads=4, kv_heads=2, dim=16, vdim=8, experts=4, top=2, ff=16,
                      shared_ff=16, loop=loop, q_temp=(0.3, 7))
    w = make_weights(cfg, seed=101, sharp=2.0)
    d = write_model(tmp_path, cfg, w)
    t = toks(45, cfg["vocab"], 102)
    resid_ref = []
    ref = forward(cfg, w, t, resid_ref).numpy()
    assert len(resid_ref) == runs
    steps = [whole("a", t[:30], end=False)] + [{"entries": [{"id": "a", "tokens": [x], "want": [0]}]} for x in t[30:]]
    logits, resid = run_trace(d, steps, residual=True)
    got = resid[0].reshape(runs, 30, cfg["width"])
    for r in range(runs):
        assert np.abs(got[r] - resid_ref[r].numpy()[:30]).max() < 2e-4 * max(1.0, float(resid_ref[r].abs().max())), r
    assert rel_err(np.concatenate(logits), ref) < TOL32


# ---- whole prompts, far keys, page and tile borders -----------------------------------------------------------------
@pytest.mark.parametrize("page", [4, 16, 64])
def test_long_prompt_every_position(base, page):
    cfg, w, d = base
    t = toks(203, cfg["vocab"], 11)  # past three key tiles of 64, not a multiple of any page size
    ref = ref_logits(cfg, w, t)
    logits, _ = run_trace(d, [whole("a", t)], page=page)
    err = [rel_err(logits[0][i:i + 1], ref[i:i + 1]) for i in range(len(t))]
    assert max(err) < TOL32, f"first bad position {int(np.argmax(np.array(err) >= TOL32))}"


def test_one_far_key_carries_the_output(tmp_path):
    """Every query is made to look at position 3 only (one key scaled up, peaky softmax): a cache that loses or
    misplaces that key changes every later logit."""
    cfg = make_config(width=32, vocab=40, layers=1, heads=2, kv_heads=1, dim=8, vdim=16, mlp=False, q_temp=None, scale=4.0)
    w = make_weights(cfg, seed=9)
    special = 7
    t = toks(150, cfg["vocab"], 13)
    t = [x if x != special else special + 1 for x in t]
    t[3] = special
    # keys are unit-normed, so make the special token's key point along the mean query direction by weights alone:
    # the key projection reads only the special token's embedding direction strongly
    w["embed"][special] = 6.0 * torch.sign(w["embed"][special])
    ref = ref_logits(cfg, w, t)
    d = write_model(tmp_path, cfg, w)
    steps = [whole("a", t[:100], end=False)] + [{"entries": [{"id": "a", "tokens": [x], "want": [0]}]} for x in t[100:]]
    logits, _ = run_trace(d, steps, page=16)
    got = np.concatenate([logits[0]] + logits[1:])
    assert rel_err(got, ref) < TOL32


# ---- prompt against token-by-token decoding, long decoding ----------------------------------------------------------
def test_prefill_equals_stepwise_decoding(base):
    cfg, w, d = base
    t = toks(90, cfg["vocab"], 17)
    ref = ref_logits(cfg, w, t)
    one_by_one = [{"entries": [{"id": "s", "tokens": [x], "want": [0]}]} for x in t]     # from the very first token
    split = [whole("p", t[:2], end=False)] + [{"entries": [{"id": "p", "tokens": [x], "want": [0]}]} for x in t[2:]]
    logits, _ = run_trace(d, one_by_one + split, page=8)
    a = np.concatenate(logits[:len(t)])
    b = np.concatenate(logits[len(t):])
    assert rel_err(a, ref) < TOL32 and rel_err(b, ref) < TOL32
    assert rel_err(a, b) < TOL32


def test_long_decoding_crosses_tiles_and_temperature_steps(base):
    cfg, w, d = base
    t = toks(60 + 150, cfg["vocab"], 19)
    ref = ref_logits(cfg, w, t)
    steps = [whole("a", t[:60], end=False)] + [{"entries": [{"id": "a", "tokens": [x], "want": [0]}]} for x in t[60:]]
    logits, _ = run_trace(d, steps, page=16)
    got = np.concatenate(logits)
    err = [rel_err(got[i:i + 1], ref[i:i + 1]) for i in range(len(t))]
    assert max(err) < TOL32, f"first bad position {int(np.argmax(np.array(err) >= TOL32))}"


@pytest.mark.parametrize("sizes", [(2, 2, 2, 2), (5, 64, 3, 17), (33, 2, 70), (1, 99, 2)])
def test_prompt_in_portions(base, sizes):
    """A prompt fed in several steps of more than one token: every portion starts where the cache stands, so its rows
    see the earlier portions' keys (and its own, causally).  A second request of another length rides along."""
    cfg, w, d = base
    t = toks(sum(sizes), cfg["vocab"], 81)
    other = toks(2 * len(sizes) + 1, cfg["vocab"], 82)
    ref, ref_o = ref_logits(cfg, w, t), ref_logits(cfg, w, other)
    steps, at = [], 0
    for i, n in enumerate(sizes):
        o = other[2 * i:2 * i + 2] if i + 1 < len(sizes) else other[2 * i:]
        steps.append({"entries": [{"id": "o", "tokens": o, "want": list(range(len(o)))},
                                  {"id": "p", "tokens": t[at:at + n], "want": list(range(n))}]})
        at += n
    logits, _ = run_trace(d, steps, page=8, max_tokens=512)
    got_o = np.concatenate([lg[:len(st["entries"][0]["tokens"])] for lg, st in zip(logits, steps)])
    got_p = np.concatenate([lg[len(st["entries"][0]["tokens"]):] for lg, st in zip(logits, steps)])
    assert rel_err(got_p, ref) < TOL32 and rel_err(got_o, ref_o) < TOL32


# ---- batches --------------------------------------------------------------------------------------------------------
def test_unequal_batch_equals_each_alone(base):
    cfg, w, d = base
    prompts = {"x": toks(1, cfg["vocab"], 21), "y": toks(67, cfg["vocab"], 22), "z": toks(130, cfg["vocab"], 23)}
    tails = {k: toks(n, cfg["vocab"], 30 + i) for i, (k, n) in enumerate({"x": 3, "y": 12, "z": 7}.items())}
    steps = [{"entries": [{"id": k, "tokens": p, "want": list(range(len(p)))} for k, p in prompts.items()]}]
    for j in range(12):
        live = [k for k in prompts if j < len(tails[k])]
        steps.append({"entries": [{"id": k, "tokens": [tails[k][j]], "want": [0]} for k in live],
                      "end": [k for k in live if j == len(tails[k]) - 1]})
    logits, _ = run_trace(d, steps, page=8, max_tokens=256)
    for k in prompts:
        full = prompts[k] + tails[k]
        ref = ref_logits(cfg, w, full)
        rows = []
        at = 0
        for kk, p in prompts.items():
            if kk == k:
                rows.append(logits[0][at:at + len(p)])
            at += len(p)
        for j in range(len(tails[k])):
            live = [kk for kk in prompts if j < len(tails[kk])]
            rows.append(logits[1 + j][live.index(k)][None])
        assert rel_err(np.concatenate(rows), ref) < TOL32, k


def test_pages_and_slots_are_reused(base):
    """The pool holds one request at a time: each request runs in pages and in the slot the one before it gave back,
    and must see nothing of it."""
    cfg, w, d = base
    reqs = [toks(n, cfg["vocab"], 40 + i) for i, n in enumerate([50, 33, 64, 7, 50])]
    steps = []
    for i, t in enumerate(reqs):
        steps.append(whole(f"r{i}", t[:-3], end=False))
        steps += [{"entries": [{"id": f"r{i}", "tokens": [x], "want": [0]}]} for x in t[-3:-1]]
        steps.append({"entries": [{"id": f"r{i}", "tokens": [t[-1]], "want": [0]}], "end": [f"r{i}"]})
    logits, _ = run_trace(d, steps, page=4, max_tokens=64, extra=["--max-seqs", "1"])
    at = 0
    for t in reqs:
        got = np.concatenate(logits[at:at + 4])
        at += 4
        assert rel_err(got, ref_logits(cfg, w, t)) < TOL32


def test_first_tokens_and_single_token_requests(base):
    cfg, w, d = base
    ts = [toks(n, cfg["vocab"], 50 + n) for n in (1, 2, 3)]
    logits, _ = run_trace(d, [whole(f"q{i}", t) for i, t in enumerate(ts)])
    for t, lg in zip(ts, logits):
        assert rel_err(lg, ref_logits(cfg, w, t)) < TOL32


# ---- bf16, generation -------------------------------------------------------------------------------------------------
def test_bfloat16_products(tmp_path):
    """bf16 products round scores too: a tame softmax (no sharpening) keeps the comparison about the kernels."""
    cfg = make_config(width=72, vocab=101, layers=2, heads=6, kv_heads=2, dim=18, vdim=40, experts=5, top=2, ff=24,
                      shared_ff=40, loop=(0, 1, 2), q_temp=(0.2, 50))
    w = make_weights(cfg, seed=5)
    d = write_model(tmp_path, cfg, w)
    t = toks(140, cfg["vocab"], 61)
    ref = ref_logits(cfg, w, t)
    steps = [whole("a", t[:120], end=False)] + [{"entries": [{"id": "a", "tokens": [x], "want": [0]}]} for x in t[120:]]
    logits, _ = run_trace(d, steps, dtype="bfloat16")
    assert rel_err(np.concatenate(logits), ref) < TOL16


@pytest.mark.parametrize("sizes", [((64, 128), (128, 64)), ((40, 24), (72, 104))])
def test_bfloat16_prompt_attention_on_the_tensor_cores(tmp_path, sizes):
    """Head sizes up to 128 in bf16 (multiples of 8; sizes below 64 or 128 run zero-padded): prompt steps take the tensor-core attention, single-token steps the split-key
    kernel.  Both see the same bf16 inputs, so they agree far more tightly than either agrees with float64 -- a key
    lost at a tile, page or portion edge would not.  Three query heads per key/value head (a 64-row tile cuts through a
    token's heads), every expert chosen (no routing flips between the two runs), a ragged batch and a prompt in portions."""
    cfg = make_config(width=128, vocab=90, layers=2, heads=6, kv_heads=2, dim=sizes[0][0], vdim=sizes[0][1], experts=3,
                      top=3, ff=32, shared_ff=64, loop=(0, 1, 2), q_temp=(0.3, 40))
    cfg["layers"][1]["mixer"].update(heads=2, kv_heads=2, dim=sizes[1][0], vdim=sizes[1][1])
    w = make_weights(cfg, seed=91, sharp=2.0)
    d = write_model(tmp_path, cfg, w)
    reqs = {"a": toks(1, 90, 92), "b": toks(70, 90, 93), "c": toks(200, 90, 94), "p": toks(204, 90, 95)}
    cuts = (50, 90, 64)
    block = [{"entries": [{"id": k, "tokens": reqs[k], "want": list(range(len(reqs[k])))} for k in "abc"], "end": ["a", "b", "c"]}]
    at = 0
    for n in cuts:
        block.append({"entries": [{"id": "p", "tokens": reqs["p"][at:at + n], "want": list(range(n))}]})
        at += n
    single = [{"entries": [{"id": k + "1", "tokens": [x], "want": [0]}]} for k in "abcp" for x in reqs[k]]
    logits, _ = run_trace(d, block + single, dtype="bfloat16", page=16, max_tokens=1024)
    got_block = np.concatenate(logits[:1 + len(cuts)])
    got_single = np.concatenate(logits[1 + len(cuts):])
    ref = np.concatenate([ref_logits(cfg, w, reqs[k]) for k in "abcp"])
    assert rel_err(got_block, ref) < TOL16 and rel_err(got_single, ref) < TOL16
    err = [rel_err(got_block[i:i + 1], got_single[i:i + 1]) for i in range(len(ref))]
    assert max(err) < 1.5e-2, f"first bad row {int(np.argmax(np.array(err) >= 1.5e-2))}"


@pytest.mark.parametrize("dtype,tol,experts,top", [("float32", TOL32, 6, 2), ("bfloat16", TOL16, 3, 3)])
def test_sizes_that_fit_no_vector(tmp_path, dtype, tol, experts, top):
    """Width, inner sizes and head sizes that are not multiples of 8 (nor of 4): no 16-byte row, no tensor-core tile.
    In bf16 every expert is chosen: at these widths a routing flip under bf16 rounding would drown the comparison."""
    cfg = make_config(width=44, vocab=77, layers=2, heads=3, kv_heads=1, dim=10, vdim=12, experts=experts, top=top, ff=20,
                      shared_ff=28, loop=(0, 1, 2), q_temp=(0.2, 9))
    cfg["layers"][1]["mixer"].update(heads=2, kv_heads=2, dim=7, vdim=5)
    w = make_weights(cfg, seed=111)
    d = write_model(tmp_path, cfg, w)
    t = toks(110, cfg["vocab"], 112)
    ref = ref_logits(cfg, w, t)
    steps = [whole("a", t[:100], end=False)] + [{"entries": [{"id": "a", "tokens": [x], "want": [0]}]} for x in t[100:]]
    logits, _ = run_trace(d, steps, dtype=dtype)
    got = np.concatenate(logits)
    err = [rel_err(got[i:i + 1], ref[i:i + 1]) for i in range(len(t))]
    assert rel_err(got, ref) < tol, f"worst rows {np.argsort(err)[-5:]} {np.sort(err)[-5:]}"


def test_many_requests_in_one_batch(base):
    """More requests than any size constant of the engine: 80 prompts of 1..5 tokens in one step, then decoded together."""
    cfg, w, d = base
    reqs = [toks(1 + i % 5, cfg["vocab"], 200 + i) + toks(2, cfg["vocab"], 400 + i) for i in range(80)]
    steps = [{"entries": [{"id": f"r{i}", "tokens": r[:-2], "want": [len(r) - 3]} for i, r in enumerate(reqs)]}]
    for j in (2, 1):
        steps.append({"entries": [{"id": f"r{i}", "tokens": [r[-j]], "want": [0]} for i, r in enumerate(reqs)]})
    logits, _ = run_trace(d, steps, max_tokens=1024)
    for i, r in enumerate(reqs):
        ref = ref_logits(cfg, w, r)[-3:]
        got = np.stack([logits[0][i], logits[1][i], logits[2][i]])
        assert rel_err(got, ref) < TOL32, i


def test_greedy_generation_through_the_scheduler(base):
    import subprocess
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
        assert g == greedy(cfg, w, p, 12)


def test_larger_shapes_take_the_block_paths(tmp_path):
    """Enough tokens and wide enough layers for the tiled and grouped products (and, in bf16, the tensor-core one)."""
    cfg = make_config(width=256, vocab=300, layers=2, heads=8, kv_heads=2, dim=64, vdim=64, experts=8, top=2, ff=128,
                      shared_ff=256, loop=(0, 2, 2), q_temp=(0.5, 64))
    w = make_weights(cfg, seed=77, sharp=2.0)
    d = write_model(tmp_path, cfg, w)
    t = toks(300, cfg["vocab"], 78)
    ref = ref_logits(cfg, w, t)
    want = list(range(0, 300, 7)) + [299]
    for dtype, tol in (("float32", TOL32), ("bfloat16", TOL16)):
        logits, _ = run_trace(d, [whole("a", t, want=want)], dtype=dtype)
        assert rel_err(logits[0], ref[want]) < tol, dtype
