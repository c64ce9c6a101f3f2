"""-m gpu: the layered executor (Retezen) against the plain float64 statement in stack_oracle.py.

Small configurations with random weights (sizes chosen so that heads != kv heads, key size != value size, top > 1,
layers differ from each other, rows that are and are not 16-byte multiples); fp32 compute for sharp comparisons, bf16 for
the serving precision.  Covered: the attention kernel alone with crafted peaks at every edge of the window and of the
pooled blocks, in portions of any size over rings that wrap; every other mechanism through one- and two-layer models;
whole prompts against token-by-token decoding and against portions down to two tokens; a cache that is given back and
used again; long decoding over wrapped rings; greedy / sampled generation and per-position probabilities through the
library's own entry points; the trace runner as a subprocess.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import stack_oracle as O
from yalm_b200 import api

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def open_model(folder, dtype=api.F32, chunk=None, context=0):
    """chunk: rows per pass, which also sizes the rings (window + chunk slots)."""
    old = os.environ.get("YALM_STACK_CHUNK")
    if chunk is not None:
        os.environ["YALM_STACK_CHUNK"] = str(chunk)
    try:
        m = api.Model(folder, context, dtype).cuda(0)
    finally:
        if chunk is not None:
            if old is None:
                del os.environ["YALM_STACK_CHUNK"]
            else:
                os.environ["YALM_STACK_CHUNK"] = old
    return m, api.InferenceState(m)


def close(m, s):
    s.close()
    m.close()


def four_layers():
    return O.make_config(layers=[
        O.attn_layer(mlp=O.dense()),
        O.attn_layer(mlp=O.moe(top=2)),
        O.attn_layer(heads=4, kv_heads=4, dim=20, vdim=32, window=7, pool=2, scale=0.5, v_mix=False, mlp=None),
        O.attn_layer(window=9, pool=4, mlp=O.moe(ff=24, experts=3, top=3)),
    ])


def checkpoint(tmp_path, cfg, seed=0, sharp=1.0, store="BF16"):
    W = O.random_weights(cfg, seed, sharp)
    return O.write_checkpoint(str(tmp_path / ("m%d" % seed)), cfg, W, store), O.as_f64(W)


def tokens_for(cfg, n, seed=1):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


def close_enough(got, want, tol):
    scale = max(1.0, float(np.abs(want).max()))
    err = float(np.abs(got - want).max())
    assert err <= tol * scale, f"max |delta| {err:.3e} > {tol * scale:.3e}"


F32_TOL = 3e-4


# ---- the attention kernel alone ------------------------------------------------------------------------------------------
def crafted_qkv(T, H, G, dk, dv, window, pool, seed):
    """Random keys and values; every query points (5x the unit vector) at one key chosen among the places where a rule could
    be one off: the oldest token inside the window, the newest outside it, the first and last member of the newest block that
    is seen and of the block that is not yet, the query's own position, position 0."""
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((T, H, dk))
    k = rng.standard_normal((T, G, dk))
    v = rng.standard_normal((T, G, dv))
    for i in range(T):
        nb = max(0, (i - window + 1) // pool) if (window > 0 and pool > 0 and i - window + 1 >= 0) else 0
        cand = [i, 0, i - window + 1, i - window, nb * pool - 1, (nb - 1) * pool, nb * pool, nb * pool + pool - 1] if window > 0 else [i, 0, i // 2]
        cand = [j for j in cand if 0 <= j <= i]
        for h in range(H):
            j = cand[(i + h) % len(cand)]
            kk = k[j, h // (H // G)]
            q[i, h] = 5.0 * kk / np.linalg.norm(kk) + 0.1 * q[i, h]
    return q, k, v


@pytest.mark.parametrize("window,pool", [(10, 4), (1, 1), (5, 8), (8, 8), (12, 1), (0, 0), (9, 0), (6, 3)])
@pytest.mark.parametrize("chunk", [1, 2, 7, 64])
def test_attention_edges_in_any_portion(window, pool, chunk):
    T, H, G, dk, dv = 64, 4, 2, 16, 24
    q, k, v = crafted_qkv(T, H, G, dk, dv, window, pool, seed=window * 31 + pool)
    want = O.window_pool_attention(q, k, v, window, pool, 0.4)
    span = max(window, pool) if window > 0 else T
    for ring in ({span + chunk - 1, span + chunk + 5, 2 * T} if window > 0 else {T}):   # the tightest ring wraps every few rows
        got = api.attn_window_pool(q, k, v, H, G, window, pool, 0.4, max(ring, 1), chunk)
        close_enough(got, want, 2e-5)


def test_attention_far_key_among_hundreds_and_odd_sizes():
    # key size not a multiple of 4 (scalar loads), value size over 32 x 2 lanes, one dominant key far back inside a long window
    T, H, G, dk, dv, window, pool = 700, 3, 3, 10, 70, 600, 16
    rng = np.random.default_rng(5)
    q, k, v = rng.standard_normal((T, H, dk)) * 0.3, rng.standard_normal((T, G, dk)), rng.standard_normal((T, G, dv))
    q[T - 1, 0] = 6.0 * k[T - window, 0] / np.linalg.norm(k[T - window, 0])         # the oldest token the last query still sees
    q[T - 1, 1] = 6.0 * k[T - window - 1, 1] / np.linalg.norm(k[T - window - 1, 1])  # one older: not seen, and its block not yet
    want = O.window_pool_attention(q, k, v, window, pool, 1.0, rows=[T - 3, T - 2, T - 1])[-3:]
    got = api.attn_window_pool(q, k, v, H, G, window, pool, 1.0, 1024, 256)[-3:]
    close_enough(got, want, 2e-5)


def test_attention_bf16_cache_means_are_taken_over_the_cached_values():
    T, H, G, dk, dv, window, pool = 48, 4, 2, 16, 32, 6, 4
    q, k, v = crafted_qkv(T, H, G, dk, dv, window, pool, seed=3)
    want = O.window_pool_attention(q, k, v, window, pool, 0.4, cache_round=O.round_bf16)
    got = api.attn_window_pool(q, k, v, H, G, window, pool, 0.4, 16, 5, cache_f32=False)
    close_enough(got, want, 2e-5)


@pytest.mark.parametrize("dk,dv,H,G", [(8, 8, 1, 1), (32, 64, 6, 2), (256, 16, 2, 2), (16, 256, 10, 2), (128, 128, 4, 1)])
@pytest.mark.parametrize("window,pool,chunk", [(10, 4, 1), (33, 8, 3), (64, 1, 1), (0, 0, 2), (40, 32, 15)])
def test_attention_rows_split_over_lane_groups(dk, dv, H, G, window, pool, chunk):
    # bf16 rings with power-of-two sizes: dk / 8 lanes share a key row (1 .. 32 lanes), query heads of a kv head go four at a
    # time (6 / 2 and 10 / 2 leave a partly filled group), short portions split the keys over CTAs and merge them
    T = 150
    q, k, v = crafted_qkv(T, H, G, dk, dv, window, pool, seed=dk + 3 * dv + window)
    want = O.window_pool_attention(q, k, v, window, pool, 0.3, cache_round=O.round_bf16)
    span = max(window, pool) if window > 0 else T
    for ring in ({span + chunk - 1, span + chunk + 11} if window > 0 else {T}):
        got = api.attn_window_pool(q, k, v, H, G, window, pool, 0.3, ring, chunk, cache_f32=False)
        close_enough(got, want, 3e-5)


@pytest.mark.parametrize("dk,dv,H,G,window,pool,chunk", [
    (64, 32, 4, 2, 44, 4, 64), (128, 128, 2, 1, 36, 6, 23), (64, 128, 3, 3, 100, 16, 200), (128, 64, 4, 1, 7, 3, 64),
    (64, 64, 2, 2, 0, 0, 70), (128, 32, 2, 1, 150, 1, 64), (64, 32, 4, 4, 33, 64, 16), (128, 128, 4, 2, 64, 64, 128)])
def test_attention_on_the_tensor_cores(dk, dv, H, G, window, pool, chunk):
    # portions of 16 rows and more over bf16 rings take the mma route; same crafted peaks at every edge
    T = 200
    q, k, v = crafted_qkv(T, H, G, dk, dv, window, pool, seed=dk + dv + window)
    want = O.window_pool_attention(O.round_bf16(q), k, v, window, pool, 0.2, cache_round=O.round_bf16)
    span = max(window, pool) if window > 0 else T
    got = api.attn_window_pool(q, k, v, H, G, window, pool, 0.2, span + chunk - 1 if window > 0 else T, chunk, cache_f32=False)
    close_enough(got, want, 1.5e-2)       # the weights are rounded to bf16 as the operand of P V


# ---- mechanisms through small models ---------------------------------------------------------------------------------
@pytest.mark.parametrize("name,layers", [
    ("attention only", [O.attn_layer(mlp=None, v_mix=False)]),
    ("attention + dense", [O.attn_layer(mlp=O.dense(ff=50, limit=0.5), v_mix=False)]),
    ("attention + experts, top 1", [O.attn_layer(mlp=O.moe(ff=33, experts=4, top=1))]),
    ("attention + experts, top = all", [O.attn_layer(mlp=O.moe(ff=16, experts=3, top=3))]),
    ("value blending", [O.attn_layer(mlp=None), O.attn_layer(mlp=None, v_mix=False, window=4, pool=1), O.attn_layer(mlp=None)]),
    ("value blending that starts at the second layer", [O.attn_layer(mlp=None, v_mix=False), O.attn_layer(mlp=O.dense(ff=24)), O.attn_layer(mlp=None)]),
    ("one head, pool 1", [O.attn_layer(heads=1, kv_heads=1, dim=8, vdim=8, window=3, pool=1, mlp=O.dense(ff=8, limit=0.0))]),
])
def test_each_mechanism(tmp_path, name, layers):
    cfg = O.make_config(layers=layers)
    folder, W = checkpoint(tmp_path, cfg, seed=len(name), sharp=3.0)
    toks = tokens_for(cfg, 40)
    m, s = open_model(folder)
    got = s.forward_rows(toks, 0, range(len(toks)))
    close(m, s)
    close_enough(got, O.forward(cfg, W, toks), F32_TOL)


def test_router_logits_that_saturate_the_sigmoid(tmp_path):
    # large router logits: in fp32 sigmoid(z) is exactly 1 from z ~ 17 on, so ranking the rounded scores would tie experts whose
    # scores still differ; the oracle ranks in float64, the library by the logits
    cfg = O.make_config(width=320, vocab=90, layers=[O.attn_layer(heads=6, kv_heads=1, dim=32, vdim=32, window=20, pool=5,
                                                                   mlp=O.moe(ff=48, experts=6, top=1))])
    W = O.random_weights(cfg, 21)       # width 320: logits of std ~14; in 33 of the 200 rows the two largest fp32 scores are equal
    folder = O.write_checkpoint(str(tmp_path / "sat"), cfg, W, "BF16")
    toks = tokens_for(cfg, 200)
    m, s = open_model(folder)
    got = s.forward_rows(toks, 0, range(len(toks)))
    close(m, s)
    close_enough(got, O.forward(cfg, O.as_f64(W), toks), F32_TOL)


def test_sizes_that_are_not_vector_multiples(tmp_path):
    # width 100 / ff 30 / key size 10: no 16-byte rows anywhere, so every product takes the scalar route, also in bf16
    cfg = O.make_config(width=100, vocab=77, layers=[O.attn_layer(heads=2, kv_heads=1, dim=10, vdim=6, mlp=O.dense(ff=30)),
                                                     O.attn_layer(heads=2, kv_heads=1, dim=10, vdim=6, mlp=O.moe(ff=14, experts=3, top=2))])
    folder, W = checkpoint(tmp_path, cfg, seed=4)
    toks = tokens_for(cfg, 50)
    want = O.forward(cfg, W, toks)
    m, s = open_model(folder)
    close_enough(s.forward_rows(toks, 0, range(50)), want, F32_TOL)
    close(m, s)
    m, s = open_model(folder, api.BF16)
    close_enough(s.forward_rows(toks, 0, range(50)), O.forward(cfg, W, toks, cache_round=O.round_bf16), 2e-2)
    close(m, s)


@pytest.mark.parametrize("store", ["BF16", "F32"])
def test_whole_prompt_decoding_and_portions_agree_with_the_oracle(tmp_path, store):
    cfg = four_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=7, sharp=2.0, store=store)
    T = 90
    toks = tokens_for(cfg, T)
    want = O.forward(cfg, W, toks)
    m, s = open_model(folder)
    whole = s.forward_rows(toks, 0, range(T))
    close_enough(whole, want, F32_TOL)
    s.end_sequence()
    # token by token
    one = np.concatenate([s.forward_rows(toks[i:i + 1], i, [0]) for i in range(T)])
    close_enough(one, want, F32_TOL)
    s.end_sequence()
    # portions of changing size, down to two tokens, cut in the middle of windows and blocks; rows without logits in between
    cuts, at, got = [2, 3, 17, 1, 2, 29, 2, 5, 1, 1, 2, 25], 0, []
    assert sum(cuts) == T
    for n in cuts:
        want_rows = [r for r in range(n) if (at + r) % 3 != 1]
        got.append((np.array(want_rows) + at, s.forward_rows(toks[at:at + n], at, want_rows)))
        at += n
    for rows, lg in got:
        if len(rows):
            close_enough(lg, want[rows], F32_TOL)
    close(m, s)


def test_cache_given_back_and_used_again(tmp_path):
    cfg = four_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=8)
    a, b = tokens_for(cfg, 70, 2), tokens_for(cfg, 33, 3)
    m, s = open_model(folder, chunk=8)      # small rings: both sequences wrap them
    s.forward_rows(a, 0, [])
    s.end_sequence()
    second = s.forward_rows(b, 0, range(len(b)))
    close_enough(second, O.forward(cfg, W, b), F32_TOL)
    # a sequence may also be abandoned by starting over at position 0; anything else than the next position is refused
    s.forward_rows(a[:10], 0, [])
    with pytest.raises(api.YalmError):
        s.forward_rows(a[10:12], 15, [])
    third = s.forward_rows(b, 0, range(len(b)))
    close(m, s)
    np.testing.assert_array_equal(second, third)


@pytest.mark.parametrize("chunk", [1, 4, 16])
def test_rings_wrap_in_prompts_and_in_long_decoding(tmp_path, chunk):
    cfg = four_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=9, sharp=2.0)
    T = 230
    toks = tokens_for(cfg, T)
    want = O.forward(cfg, W, toks)
    m, s = open_model(folder, chunk=chunk)
    assert m.ring_slots(0) == 64 and m.ring_slots(0) < T     # window 12 + chunk, rounded up to 64 slots: the prompt wraps it three times
    rows = list(range(0, T, 7)) + [T - 1]
    close_enough(s.forward_rows(toks, 0, sorted(set(rows))), want[sorted(set(rows))], F32_TOL)
    s.end_sequence()
    # a short prompt, then 200 tokens one by one
    s.forward_rows(toks[:30], 0, [])
    dec = np.concatenate([s.forward_rows(toks[i:i + 1], i, [0]) for i in range(30, T)])
    close(m, s)
    close_enough(dec, want[30:], F32_TOL)


def test_pooled_blocks_in_the_cache(tmp_path):
    cfg = O.make_config(layers=[O.attn_layer(window=5, pool=3, mlp=None, v_mix=False)])
    folder, W = checkpoint(tmp_path, cfg, seed=10)
    toks = tokens_for(cfg, 20)
    m, s = open_model(folder)
    s.forward_rows(toks[:7], 0, [])
    s.forward_rows(toks[7:8], 7, [])
    s.forward_rows(toks[8:20], 8, [])
    mix = cfg["layers"][0]["mixer"]
    G, dk, nblk = mix["kv_heads"], mix["dim"], cfg["max_positions"] // 3 + 1
    pooled = m.stack_read(0, 2, G * nblk * dk).reshape(G, nblk, dk)
    ring = m.ring_slots(0)
    keys = m.stack_read(0, 0, G * ring * dk).reshape(G, ring, dk)
    close(m, s)
    x = W["embed"][toks] + W["pos"][:20]
    k = O.qk_norm_whole(x @ W["l0.mix.k"].T, W["l0.mix.k.norm"], cfg["norm"]["eps"]).reshape(20, G, dk)
    np.testing.assert_allclose(keys[:, :20].transpose(1, 0, 2), k, atol=1e-5)
    for b in range(6):          # blocks 0 .. 5 are complete after 20 tokens (18 of them), block 6 is not
        np.testing.assert_allclose(pooled[:, b], k[3 * b:3 * b + 3].mean(0), atol=1e-5)
    assert not pooled[:, 6].any()


# ---- the library's own entry points ------------------------------------------------------------------------------------
def test_generation_through_the_entry_points(tmp_path):
    cfg = four_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=11, sharp=2.0)
    prompt, n = tokens_for(cfg, 21), 14
    want = O.greedy(cfg, W, prompt, n)
    m, s = open_model(folder)
    # Model::forward per token + host arg-max (the CLI's loop)
    assert s.generate(prompt, n) == want
    s.end_sequence()
    # Model::forward_batch for the prompt, then the device loop (graph replay after the first step)
    s.forward_batch(prompt[:-1], 0)
    assert s.generate_greedy(prompt[-1], len(prompt) - 1, n) == want
    s.end_sequence()
    s.forward_batch(prompt[:-1], 0)
    toks, lg = s.generate_greedy(prompt[-1], len(prompt) - 1, n, keep_logits=True)
    assert toks == want
    close_enough(lg, O.forward(cfg, W, prompt + want)[len(prompt) - 1:-1], F32_TOL)
    s.end_sequence()
    # sampling on the device: reproducible for a seed, in range, and temperature 0 is greedy
    s.forward_batch(prompt[:-1], 0)
    a = s.generate_sampled(prompt[-1], len(prompt) - 1, n, 0.8, seed=5)
    s.end_sequence()
    s.forward_batch(prompt[:-1], 0)
    b = s.generate_sampled(prompt[-1], len(prompt) - 1, n, 0.8, seed=5)
    s.end_sequence()
    s.forward_batch(prompt[:-1], 0)
    c = s.generate_sampled(prompt[-1], len(prompt) - 1, n, 0.0)
    close(m, s)
    assert a == b and all(0 <= t < cfg["vocab"] for t in a) and c == want


def test_per_position_probabilities(tmp_path):
    cfg = four_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=12)
    toks = tokens_for(cfg, 60)
    lg = O.forward(cfg, W, toks[:-1])
    p = np.exp(lg - lg.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    want = p[np.arange(59), toks[1:]]
    m, s = open_model(folder, chunk=16)
    got = s.forward_batch(toks[:-1], 0, targets=toks[1:])
    close(m, s)
    np.testing.assert_allclose(got, want, rtol=2e-3, atol=1e-6)


def test_serving_precision(tmp_path):
    # bf16 operands: whole prompt (tensor-core products) and token-by-token decoding (fp32 activations) both stay within the
    # rounding of the operands of the float64 model with a bf16 cache, and agree with each other
    cfg = four_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=13)
    T = 80
    toks = tokens_for(cfg, T)
    want = O.forward(cfg, W, toks, cache_round=O.round_bf16)
    m, s = open_model(folder, api.BF16)
    whole = s.forward_rows(toks, 0, range(T))
    s.end_sequence()
    s.forward_rows(toks[:40], 0, [])
    dec = np.concatenate([s.forward_rows(toks[i:i + 1], i, [0]) for i in range(40, T)])
    close(m, s)

    def rows_close(got, ref):
        # per-row error relative to the row's spread.  With random weights a few rows sit on a router tie that operand
        # rounding flips (another expert: a different, equally valid row), so a tenth of the rows may be off; the rest must be
        # within the rounding of bf16 operands
        e = np.sqrt(((got - ref) ** 2).mean(1)) / np.sqrt((ref ** 2).mean(1))
        assert np.median(e) < 1e-2 and (e > 4e-2).mean() <= 0.1, (float(np.median(e)), float(e.max()))

    rows_close(whole, want)
    rows_close(dec, want[40:])


def test_command_line_on_a_checkpoint_directory(tmp_path):
    import re
    exe = os.path.join(ROOT, "build", "main")
    if not os.path.exists(exe):
        subprocess.check_call(["make", "-s", "-C", ROOT, "cli"])
    cfg = four_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=15, sharp=2.0)
    prompt = tokens_for(cfg, 17)
    text = " ".join(map(str, prompt))
    r = subprocess.run([exe, folder, "-m", "completion", "-i", text, "-n", "6", "-t", "0", "-p", "fp32"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    ids = [l for l in r.stdout.splitlines() if re.fullmatch(r"(\d+ )+", l)]
    assert ids and [int(x) for x in ids[-1].split()] == O.greedy(cfg, W, prompt, 6)
    r = subprocess.run([exe, folder, "-m", "perplexity", "-i", text, "-p", "fp32"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lg = O.forward(cfg, W, prompt[:-1])
    lp = lg - lg.max(1, keepdims=True)
    lp = lp - np.log(np.exp(lp).sum(1, keepdims=True))
    want = float(np.exp(-lp[np.arange(16), prompt[1:]].mean()))
    got = float(re.search(r"perplexity: ([0-9.eE+-]+)", r.stdout).group(1))
    assert abs(got - want) <= 2e-3 * want, (got, want)


def test_trace_runner(tmp_path):
    cfg = four_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=14)
    a, b = tokens_for(cfg, 25, 4), tokens_for(cfg, 9, 5)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:20], "want": [3, 19]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[20:22], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[22:], "want": [2]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": b, "want": [8]}], "end": ["b"]}]
    out = tmp_path / "out"
    out.mkdir()
    env = dict(os.environ, YALM_B200_LIB=api.LIB_PATH)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == ["done 0", "done 1", "done 2", "done 3"]
    wa, wb = O.forward(cfg, W, a), O.forward(cfg, W, b)
    V = cfg["vocab"]
    close_enough(np.fromfile(out / "0.f32", "<f4").reshape(-1, V), wa[[3, 19]], F32_TOL)
    assert not (out / "1.f32").exists()
    close_enough(np.fromfile(out / "2.f32", "<f4").reshape(-1, V), wa[[24]], F32_TOL)
    close_enough(np.fromfile(out / "3.f32", "<f4").reshape(-1, V), wb[[8]], F32_TOL)
