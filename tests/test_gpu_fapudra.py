"""-m gpu: the Fapudra design on the layered executor against the plain float64 statement in fapudra_oracle.py.

The kernels alone (device arrays through the C ABI): the matrix-state recurrence in both of its forms, the short
convolution and the sigmoid attention, each run in portions of several sizes against one whole pass of the oracle, the
attention with crafted queries that single out one key at every edge of its visible set.  Then small models with random
weights (two kinds of layers, sizes that differ between layers and avoid powers of two, head groups, more than one norm
part, a router whose group rule bites): every mechanism through the residual after its layer; whole prompts against
token-by-token decoding and portions down to two tokens; state given back and used again; long decoding over a wrapping
key ring; serving precision; greedy generation through the library's entry points, the command line and the trace runner.
"""
import ctypes as C
import json
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

import fapudra_oracle as O
from yalm_b200 import api

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F32_TOL = 3e-4
vp, i32, f32 = C.c_void_p, C.c_int, C.c_float


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.ascontiguousarray(a), dtype=dtype).cuda().contiguous()


def ptr(t):
    return vp(t.data_ptr()) if t is not None else None


def ok(rc, what):
    torch.cuda.synchronize()
    assert rc == 0, "%s returned %d" % (what, rc)


def close_enough(got, want, tol=F32_TOL):
    scale = max(1.0, float(np.abs(want).max()))
    err = float(np.abs(np.asarray(got, np.float64) - want).max())
    assert err <= tol * scale, f"max |delta| {err:.3e} > {tol * scale:.3e}"


def portions(T, sizes):
    at, k = 0, 0
    while at < T:
        n = min(sizes[k % len(sizes)], T - at)
        yield at, n
        at, k = at + n, k + 1


# ---- the recurrence kernel alone -----------------------------------------------------------------------------------------
def run_scan(k, q, v, decay, beta, vscale, skip, rep, sizes):
    """k, q (T, G, D); v (T, H, P); the state is carried between calls of the sizes given."""
    L = api.lib()
    L.yalm_state_scan_rows.argtypes = [vp, i32, vp, i32, vp, i32, vp, i32, vp, i32, i32, vp, i32, vp, i32, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp]
    T, G, D = k.shape
    H, P = v.shape[1], v.shape[2]
    state = torch.full((H, P, D), 7.0, device="cuda")       # garbage: a call at position 0 must not read it
    out = torch.zeros(T, H * P, device="cuda")
    per_channel = int(decay.ndim == 3)
    kd, qd, vd, dd = dev(k.reshape(T, -1)), dev(q.reshape(T, -1)), dev(v.reshape(T, -1)), dev(decay.reshape(T, -1))
    bd = dev(beta) if beta is not None else None
    sd = dev(vscale) if vscale is not None else None
    kk = dev(skip) if skip is not None else None
    for at, n in portions(T, sizes):
        ok(L.yalm_state_scan_rows(ptr(out[at:]), H * P, ptr(kd[at:]), G * D, ptr(qd[at:]), G * D, ptr(vd[at:]), H * P, ptr(dd[at:]), dd.shape[1], per_channel,
                                  ptr(sd[at:]) if sd is not None else None, H, ptr(bd[at:]) if bd is not None else None, H, ptr(kk), ptr(state), n, H, rep, D, P,
                                  at, None, None), "state_scan_rows")
    return out.cpu().numpy().reshape(T, H, P), state.cpu().numpy()


@pytest.mark.parametrize("D,P,H,rep", [(8, 5, 2, 1), (20, 16, 4, 2), (64, 40, 3, 3), (100, 17, 2, 1), (256, 8, 1, 1)])
@pytest.mark.parametrize("sizes", [[1000], [1], [2, 1, 7, 30]])
def test_delta_rule_recurrence(D, P, H, rep, sizes):
    rng = np.random.default_rng(D + P)
    T, G = 45, H // rep
    k = rng.standard_normal((T, G, D))
    k /= np.linalg.norm(k, axis=-1, keepdims=True)
    q = rng.standard_normal((T, G, D)) / np.sqrt(D)
    v = rng.standard_normal((T, H, P))
    g = rng.uniform(0.5, 1.0, (T, H, D))
    beta = rng.uniform(0.1, 1.0, (T, H))
    grp = np.arange(H) // rep
    want, S = O.matrix_state_scan(k[:, grp], q[:, grp], v, g, beta=beta)
    got, state = run_scan(k, q, v, g, beta, None, None, rep, sizes)
    close_enough(got, want, 1e-5)
    close_enough(state, S.transpose(0, 2, 1), 1e-5)       # the library keeps (head, column, row)


@pytest.mark.parametrize("sizes", [[1000], [1], [3, 2, 9]])
def test_state_space_recurrence(sizes):
    rng = np.random.default_rng(3)
    T, H, G, N, P = 40, 6, 2, 24, 10
    B, Cm = rng.standard_normal((T, G, N)), rng.standard_normal((T, G, N))
    x = rng.standard_normal((T, H, P))
    dt = rng.uniform(0.01, 1.0, (T, H))
    a = np.exp(-rng.uniform(0.1, 2.0, H) * dt)
    skip = rng.standard_normal(H)
    grp = np.arange(H) // (H // G)
    want, _ = O.matrix_state_scan(B[:, grp], Cm[:, grp], x, a, vscale=dt, skip=skip)
    got, _ = run_scan(B, Cm, x, a, None, dt, skip, H // G, sizes)
    close_enough(got, want, 1e-5)


@pytest.mark.parametrize("taps", [1, 2, 4, 5])
@pytest.mark.parametrize("sizes", [[1000], [1], [2], [1, 2, 40, 3]])
def test_short_convolution_in_portions(taps, sizes):
    L = api.lib()
    L.yalm_conv_act_rows.argtypes = [vp, i32, vp, i32, vp, vp, vp, i32, i32, i32, i32, vp, vp]
    rng = np.random.default_rng(taps)
    T, Cn, ld = 77, 150, 163
    x, w, b = rng.standard_normal((T, ld)), rng.standard_normal((Cn, taps)), rng.standard_normal(Cn)
    want = O.silu(O.causal_conv(x[:, 5:5 + Cn], w, b))
    xd, wd, bd = dev(x), dev(w), dev(b)
    out = torch.zeros(T, Cn, device="cuda")
    state = torch.full((Cn, max(1, taps - 1)), 9.0, device="cuda")
    for at, n in portions(T, sizes):
        ok(L.yalm_conv_act_rows(ptr(out[at:]), Cn, vp(xd[at:].data_ptr() + 20), ld, ptr(wd), ptr(bd), ptr(state), n, Cn, taps, at, None, None), "conv_act_rows")
    close_enough(out.cpu().numpy(), want, 1e-5)


# ---- the sigmoid attention alone -------------------------------------------------------------------------------------------
def run_sigmoid_attention(q, k, rel, hb, gate, window, keep, scale, far, ring, sizes, cache_f32=1, mma=False):
    L = api.lib()
    L.yalm_attn_sigmoid_mma.argtypes = [vp, i32, vp, i32, vp, vp, vp, i32, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, f32, i32, i32, vp, vp]
    L.yalm_qk_bias_append_rows.argtypes = [vp, vp, i32, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp]
    L.yalm_attn_sigmoid_rows.argtypes = [vp, i32, vp, i32, vp, vp, vp, i32, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, f32, i32, i32, i32, vp, vp]
    L.yalm_attn_sigmoid_workspace.restype = C.c_size_t
    T, H, d = q.shape
    G = k.shape[1]
    ld = (H + G) * d
    rows = dev(np.concatenate([q.reshape(T, -1), k.reshape(T, -1)], 1))
    ct = torch.float32 if cache_f32 else torch.bfloat16
    ringb = torch.full((G, ring, d), 5.0, device="cuda", dtype=ct)
    firstb = torch.full((G, max(1, keep), d), 5.0, device="cuda", dtype=ct)
    bucket = dev([O.distance_bucket(n, rel.shape[0], far) for n in range(T)], torch.int32)
    reld, hbd, gd = dev(rel), dev(hb), dev(gate.reshape(T, -1)) if gate is not None else None
    ws = torch.zeros(L.yalm_attn_sigmoid_workspace(d), device="cuda")
    out = torch.zeros(T, H * d, device="cuda")
    kp = window > 0 and keep or 0
    # the per-head table form of the same bias; every other call goes without it
    table = dev((rel[[O.distance_bucket(n, rel.shape[0], far) for n in range(T)]] + hb).T) if mma and window % 2 else None
    for at, n in portions(T, sizes):
        ok(L.yalm_qk_bias_append_rows(ptr(rows[at:]), vp(rows[at:].data_ptr() + 4 * H * d), ld, None, None, ptr(ringb), ptr(firstb), n, H, G, d, ring, kp,
                                      cache_f32, at, None, None), "qk_bias_append_rows")
        if mma:
            ok(L.yalm_attn_sigmoid_mma(ptr(out[at:]), H * d, ptr(rows[at:]), ld, ptr(ringb), ptr(firstb), ptr(gd[at:]) if gd is not None else None, H * d,
                                       ptr(reld), ptr(bucket), ptr(hbd), ptr(table), T, n, H, G, d, ring, window, kp, scale, T, at, None, None), "attn_sigmoid_mma")
            continue
        ok(L.yalm_attn_sigmoid_rows(ptr(out[at:]), H * d, ptr(rows[at:]), ld, ptr(ringb), ptr(firstb), ptr(gd[at:]) if gd is not None else None, H * d, ptr(reld),
                                    ptr(bucket), ptr(hbd), ptr(ws), n, H, G, d, ring, window, kp, scale, cache_f32, T, at, None, None), "attn_sigmoid_rows")
    return out.cpu().numpy().reshape(T, H, d)


def crafted(T, H, G, d, window, keep, seed):
    """Keys are random; with the head bias far below zero every weight vanishes, except that query i of head a points at
    ONE key (its score lifted far above the bias), cycling through the edges of what it may see: the oldest key inside the
    window, the newest outside, the last kept first token, the first one not kept, position 0, itself.  A key wrongly
    seen or missed changes the output by a whole key vector."""
    rng = np.random.default_rng(seed)
    k = rng.standard_normal((T, G, d))
    q = np.zeros((T, H, d))
    for i in range(T):
        cands = [i - window + 1, i - window, keep - 1, keep, 0, i, i - 1, i - window - 1] if window else [0, i, i // 2, 1]
        for a in range(H):
            j = min(max(cands[(i + a) % len(cands)], 0), i)
            kj = k[j, a // (H // G)]
            q[i, a] = kj / (kj @ kj) * 40.0
    return q, k


@pytest.mark.parametrize("window,keep,sizes,ring", [(9, 3, [1000], 120), (9, 3, [1], 10), (9, 3, [2, 5, 1, 13], 22), (16, 0, [7], 23), (0, 0, [6, 1], 120),
                                                    (5, 8, [3], 8), (33, 2, [64], 97)])
def test_sigmoid_attention_edges_in_any_portion(window, keep, sizes, ring):
    T, H, G, d = 110, 6, 2, 12
    q, k = crafted(T, H, G, d, window, keep, seed=window)
    rng = np.random.default_rng(1)
    rel, hb, gate = rng.standard_normal((10, H)), np.full(H, -20.0), rng.standard_normal((T, H, d))
    want = O.sigmoid_attention_core(q, k, rel, hb, window, keep, 1.0, far=30) * O.sigmoid(gate)
    got = run_sigmoid_attention(q, k, rel, hb, gate, window, keep, 1.0, 30, ring, sizes)
    close_enough(got, want, 1e-5)
    if window:      # the crafted rows tell a window that is one key too long, and a kept token more, from the right ones
        assert np.abs(O.sigmoid_attention_core(q, k, rel, hb, window + 1, keep, 1.0, far=30) * O.sigmoid(gate) - want).max() > 0.3
        assert np.abs(O.sigmoid_attention_core(q, k, rel, hb, window, keep + 1, 1.0, far=30) * O.sigmoid(gate) - want).max() > 0.3


def test_sigmoid_attention_far_keys_among_hundreds():
    T, H, G, d, window, keep = 700, 2, 1, 20, 64, 5
    rng = np.random.default_rng(2)
    k = rng.standard_normal((T, G, d))
    q = rng.standard_normal((T, H, d)) * 0.1
    k3 = k[3, 0]
    q[650:, 0] = k3 / (k3 @ k3) * 40.0      # decoded-late queries point at kept token 3, hundreds of positions back
    q[650:, 1] = k[6, 0] / (k[6, 0] @ k[6, 0]) * 40.0   # ... and at token 6, which is not kept and long gone
    rel, hb = rng.standard_normal((16, H)) * 0.3, np.full(H, -12.0)
    want = O.sigmoid_attention_core(q, k, rel, hb, window, keep, 1.0, far=100)
    got = run_sigmoid_attention(q, k, rel, hb, None, window, keep, 1.0, 100, 664, [600, 50] + [1] * 50)
    close_enough(got, want, 1e-5)
    without = O.sigmoid_attention_core(q[:661], k[:661], rel, hb, window, 0, 1.0, far=100)
    assert np.abs(want[660, 0] - without[660, 0] - k3).max() < 1e-3       # the kept token's share is one whole key vector
    # the whole context without a window: the far key is one among 700
    want = O.sigmoid_attention_core(q, k, rel, hb, 0, 0, 1.0, far=100)
    got = run_sigmoid_attention(q, k, rel, hb, None, 0, 0, 1.0, 100, T, [630, 1, 1, 68])
    close_enough(got, want, 1e-5)


@pytest.mark.parametrize("d,H,G,sizes", [(16, 4, 2, [5, 1, 9]), (8, 4, 2, [1]), (64, 8, 2, [1, 3]), (256, 2, 2, [13, 1]), (16, 8, 1, [12]), (32, 16, 2, [13]), (24, 4, 2, [4])])
def test_sigmoid_attention_over_a_bf16_ring(d, H, G, sizes):
    """Decode-sized calls over the serving cache: rows read as 16-byte pieces by lane groups (head sizes 8 * 2^k; 24: lane per key)."""
    T = 60
    q, k = crafted(T, H, G, d, 11, 2, seed=4)
    rng = np.random.default_rng(d)
    rel, hb, gate = rng.standard_normal((8, H)), np.full(H, -20.0), rng.standard_normal((T, H, d))
    kr = O.from_bf16_bits(O.to_bf16_bits(k.astype(np.float32))).reshape(k.shape).astype(np.float64)
    want = O.sigmoid_attention_core(q, kr, rel, hb, 11, 2, 1.0, far=20) * O.sigmoid(gate)
    got = run_sigmoid_attention(q, k, rel, hb, gate, 11, 2, 1.0, 20, 24, sizes, cache_f32=0)
    close_enough(got, want, 1e-5)
    assert np.abs(O.sigmoid_attention_core(q, kr, rel, hb, 12, 2, 1.0, far=20) * O.sigmoid(gate) - want).max() > 0.3


@pytest.mark.parametrize("d,window,keep,sizes,ring", [(32, 9, 3, [1000], 240), (64, 70, 5, [64, 17, 100], 170), (128, 33, 40, [16, 130], 163), (64, 0, 0, [90, 16], 230),
                                                      (64, 130, 0, [200], 330)])
def test_sigmoid_attention_on_the_tensor_cores(d, window, keep, sizes, ring):
    T, H, G = 230, 4, 2
    q, k = crafted(T, H, G, d, window, keep, seed=d)
    rng = np.random.default_rng(6)
    rel, hb, gate = rng.standard_normal((12, H)), np.full(H, -20.0), rng.standard_normal((T, H, d))
    kr = O.from_bf16_bits(O.to_bf16_bits(k.astype(np.float32))).reshape(k.shape).astype(np.float64)
    qr = O.from_bf16_bits(O.to_bf16_bits(q.astype(np.float32))).reshape(q.shape).astype(np.float64)
    want = O.sigmoid_attention_core(qr, kr, rel, hb, window, keep, 1.0, far=50) * O.sigmoid(gate)
    got = run_sigmoid_attention(q, k, rel, hb, gate, window, keep, 1.0, 50, ring, sizes, cache_f32=0, mma=True)
    close_enough(got, want, 1e-2)       # the weights are rounded to bf16 for the second product
    if window:
        assert np.abs(O.sigmoid_attention_core(qr, kr, rel, hb, window + 1, keep, 1.0, far=50) * O.sigmoid(gate) - want).max() > 0.3


# ---- models --------------------------------------------------------------------------------------------------------------
def open_model(folder, dtype=api.F32, chunk=None, context=0):
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
        O.parallel_layer(mlp=O.moe()),
        O.mamba2_layer(mlp=O.moe(ff=16, experts=4, top=3, groups=2, keep=2)),
        O.mamba2_layer(heads=3, vdim=8, state=20, groups=1, norm_groups=3, conv=4, mlp=None),
        O.parallel_layer(heads=3, kv_heads=3, dim=20, window=6, keep_first=0, rheads=2, rkv=2, rdim=24, rvdim=8, conv=2, mlp=O.moe(experts=8, top=2, groups=4, keep=1)),
    ])


def checkpoint(tmp_path, cfg, seed=0, store="BF16", edit=None):
    W = O.random_weights(cfg, seed)
    if edit:
        edit(W)
    return O.write_checkpoint(str(tmp_path / ("m%d" % seed)), cfg, W, store), O.as_f64(W)


def tokens_for(cfg, n, seed=1):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


ONE_LAYER = {
    "state space": [O.mamba2_layer()],
    "state space, one group, one norm part, no experts": [O.mamba2_layer(groups=1, norm_groups=1, conv=2)],
    "parallel": [O.parallel_layer()],
    "parallel, every head its own keys, longer convolution": [O.parallel_layer(kv_heads=4, rkv=4, conv=5, window=4, keep_first=6)],
    "experts, groups that bite": [O.mamba2_layer(mlp=O.moe(experts=8, top=2, groups=4, keep=1))],
    "experts, all groups kept, all experts used": [O.mamba2_layer(mlp=O.moe(experts=4, top=4, groups=2, keep=2))],
}


@pytest.mark.parametrize("name", list(ONE_LAYER))
def test_each_mechanism_through_the_residual_after_its_layer(tmp_path, name):
    cfg = O.make_config(layers=ONE_LAYER[name])

    def sharpen(W):            # router logits far apart: the group rule and the choice are not close calls
        if "l0.mlp.router" in W:
            W["l0.mlp.router"] = O.from_bf16_bits(O.to_bf16_bits(W["l0.mlp.router"] * 6)).reshape(W["l0.mlp.router"].shape)
    folder, W = checkpoint(tmp_path, cfg, seed=5, edit=sharpen)
    T = 40
    toks = tokens_for(cfg, T)
    layers = []
    want = O.forward(cfg, W, toks, layers)
    m, s = open_model(folder)
    buf = np.zeros((1, T, cfg["width"]), np.float32)
    m.stack_tap(buf)
    got = s.forward_rows(toks, 0, range(T))
    m.stack_tap(None)
    close(m, s)
    close_enough(buf[0], layers[0])
    close_enough(got, want)


@pytest.mark.parametrize("store", ["BF16", "F32"])
def test_whole_prompt_decoding_and_portions_agree_with_the_oracle(tmp_path, store):
    cfg = four_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=7, store=store)
    T = 90
    toks = tokens_for(cfg, T)
    want = O.forward(cfg, W, toks)
    m, s = open_model(folder)
    close_enough(s.forward_rows(toks, 0, range(T)), want)
    s.end_sequence()
    one = np.concatenate([s.forward_rows(toks[i:i + 1], i, [0]) for i in range(T)])
    close_enough(one, want)
    s.end_sequence()
    cuts, at, got = [2, 3, 17, 1, 2, 29, 2, 5, 1, 1, 2, 25], 0, []
    assert sum(cuts) == T
    for n in cuts:
        rows = [r for r in range(n) if (at + r) % 3 != 1]
        got.append((np.array(rows) + at, s.forward_rows(toks[at:at + n], at, rows)))
        at += n
    for rows, lg in got:
        if len(rows):
            close_enough(lg, want[rows])
    close(m, s)


def test_decode_rows_with_the_block_fusions(tmp_path, monkeypatch):
    """Norm + token shift inside the projection's launch, the residual add as the tail of the block's last product."""
    monkeypatch.setenv("YALM_STACK_FUSE_BLOCK", "1")
    cfg = O.make_config(width=64, layers=[O.parallel_layer(dim=16, rdim=16, rvdim=16, mlp=O.moe()), O.mamba2_layer(vdim=16, mlp=None),
                                          O.mamba2_layer(vdim=16, mlp=O.moe(ff=16, experts=4, top=3, groups=2, keep=2))])
    folder, W = checkpoint(tmp_path, cfg, seed=12)
    T = 70
    toks = tokens_for(cfg, T)
    want = O.forward(cfg, W, toks)
    for dtype, tol in ((api.F32, F32_TOL), (api.BF16, 3e-2)):
        m, s = open_model(folder, dtype)
        s.forward_rows(toks[:9], 0, [])
        one = np.concatenate([s.forward_rows(toks[i:i + 1], i, [0]) for i in range(9, T)])
        s.end_sequence()
        first = np.concatenate([s.forward_rows(toks[i:i + 1], i, [0]) for i in range(5)])      # a sequence that starts with single rows
        close(m, s)
        close_enough(one, want[9:], tol)
        close_enough(first, want[:5], tol)


def test_decode_rows_on_side_streams_equal_the_serial_order(tmp_path, monkeypatch):
    """A decode row's experts and second mixer run on side streams (parallel branches of the captured step); the arithmetic is
    the same, so logits and greedy tokens are identical to the one-stream order."""
    cfg = four_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=13)
    toks = tokens_for(cfg, 60)
    runs = []
    for flag in ("1", "0"):
        monkeypatch.setenv("YALM_STACK_BRANCHES", flag)
        m, s = open_model(folder)
        s.forward_rows(toks[:7], 0, [])
        one = np.concatenate([s.forward_rows(toks[i:i + 1], i, [0]) for i in range(7, 60)])
        gen = s.generate_greedy(toks[0], 60, 12)
        close(m, s)
        runs.append((one, gen))
    np.testing.assert_array_equal(runs[0][0], runs[1][0])
    assert runs[0][1] == runs[1][1]
    close_enough(runs[0][0], O.forward(cfg, W, toks)[7:])


def test_state_given_back_and_used_again(tmp_path):
    cfg = four_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=8)
    a, b = tokens_for(cfg, 70, 2), tokens_for(cfg, 33, 3)
    m, s = open_model(folder, chunk=8)
    s.forward_rows(a, 0, [])
    s.end_sequence()
    second = s.forward_rows(b, 0, range(len(b)))
    close_enough(second, O.forward(cfg, W, b))
    s.forward_rows(a[:10], 0, [])                     # abandoned: the next sequence starts over at position 0
    with pytest.raises(api.YalmError):
        s.forward_rows(a[10:12], 15, [])
    third = s.forward_rows(b, 0, range(len(b)))
    close(m, s)
    np.testing.assert_array_equal(second, third)


@pytest.mark.parametrize("chunk", [1, 4, 16])
def test_long_decoding_over_a_wrapping_ring(tmp_path, chunk):
    cfg = four_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=9)
    T = 230
    toks = tokens_for(cfg, T)
    want = O.forward(cfg, W, toks)
    m, s = open_model(folder, chunk=chunk)
    assert m.ring_slots(0) == 64 and m.ring_slots(0) < T
    rows = sorted(set(list(range(0, T, 7)) + [T - 1]))
    close_enough(s.forward_rows(toks, 0, rows), want[rows])
    s.end_sequence()
    s.forward_rows(toks[:30], 0, [])
    dec = np.concatenate([s.forward_rows(toks[i:i + 1], i, [0]) for i in range(30, T)])
    close(m, s)
    close_enough(dec, want[30:])


def test_serving_precision(tmp_path):
    cfg = four_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=10)
    T = 120
    toks = tokens_for(cfg, T)
    want = O.forward(cfg, W, toks)
    m, s = open_model(folder, api.BF16)
    whole = s.forward_rows(toks, 0, range(T))
    s.end_sequence()
    s.forward_rows(toks[:40], 0, [])
    dec = np.concatenate([s.forward_rows(toks[i:i + 1], i, [0]) for i in range(40, T)])
    close(m, s)

    def rows_close(got, ref):
        e = np.abs(got - ref).max(1) / max(1.0, np.abs(ref).max())
        assert np.median(e) < 2e-2 and (e > 6e-2).mean() <= 0.1, (float(np.median(e)), float(e.max()))
    rows_close(whole, want)
    rows_close(dec, want[40:])


def test_generation_through_the_entry_points(tmp_path):
    cfg = four_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=11)
    prompt, n = tokens_for(cfg, 21), 14
    want = O.greedy(cfg, W, prompt, n)
    m, s = open_model(folder)
    assert s.generate(prompt, n) == want
    s.end_sequence()
    s.forward_batch(prompt[:-1], 0)
    assert s.generate_greedy(prompt[-1], len(prompt) - 1, n) == want      # the captured decode step, replayed
    s.end_sequence()
    s.forward_batch(prompt[:-1], 0)
    toks, lg = s.generate_greedy(prompt[-1], len(prompt) - 1, n, keep_logits=True)
    assert toks == want
    close_enough(lg, O.forward(cfg, W, prompt + want)[len(prompt) - 1:-1])
    s.end_sequence()
    s.forward_batch(prompt[:-1], 0)
    a = s.generate_sampled(prompt[-1], len(prompt) - 1, n, 0.8, seed=5)
    s.end_sequence()
    s.forward_batch(prompt[:-1], 0)
    b = s.generate_sampled(prompt[-1], len(prompt) - 1, n, 0.8, seed=5)
    close(m, s)
    assert a == b and all(0 <= t < cfg["vocab"] for t in a)


def test_command_line_on_a_checkpoint_directory(tmp_path):
    exe = os.path.join(ROOT, "build", "main")
    if not os.path.exists(exe):
        subprocess.check_call(["make", "-s", "-C", ROOT, "cli"])
    cfg = four_layers()
    folder, W = checkpoint(tmp_path, cfg, seed=15)
    prompt = tokens_for(cfg, 17)
    text = " ".join(map(str, prompt))
    r = subprocess.run([exe, folder, "-m", "completion", "-i", text, "-n", "6", "-t", "0", "-p", "fp32"], capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    ids = [l for l in r.stdout.splitlines() if re.fullmatch(r"(\d+ )+", l)]
    assert ids and [int(x) for x in ids[-1].split()] == O.greedy(cfg, W, prompt, 6)


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
    close_enough(np.fromfile(out / "0.f32", "<f4").reshape(-1, V), wa[[3, 19]])
    assert not (out / "1.f32").exists()
    close_enough(np.fromfile(out / "2.f32", "<f4").reshape(-1, V), wa[[24]])
    close_enough(np.fromfile(out / "3.f32", "<f4").reshape(-1, V), wb[[8]])
