"""Plain, slow float64 statement of the Fapudra design's mechanisms, one function per mechanism, and a maker of small
random checkpoints.  Nothing here is shared with the library: the tests compare the library's kernels, state manager and
step function against these functions.

Notation: T tokens, row t = position t; matrices are (out, in) and applied as x @ W.T; W[name] is a tensor of the
checkpoint.  A layer: h = g * rms(x);  hs = h + (h[t-1] - h) * shift (the mixer's input; h[-1] = 0);
x <- x + mixer(hs) + experts(h).
"""
import math

import numpy as np

from stack_oracle import from_bf16_bits, to_bf16_bits, write_checkpoint  # noqa: F401  (the container writer)


# ---- small pieces ------------------------------------------------------------------------------------------------------
def rms(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def token_shift(h, mu):
    """h (T, W) -> h + (previous row - h) * mu, the previous row of row 0 being zero."""
    prev = np.concatenate([np.zeros_like(h[:1]), h[:-1]], 0)
    return h + (prev - h) * mu


def causal_conv(x, w, b=None):
    """x (T, C), w (C, taps): out[t, c] = sum_j w[c, j] x[t - (taps - 1) + j, c] (+ b[c]); rows before 0 are zero."""
    T, C = x.shape
    taps = w.shape[1]
    pad = np.concatenate([np.zeros((taps - 1, C)), x], 0)
    out = np.zeros((T, C))
    for j in range(taps):
        out += pad[j:j + T] * w[:, j]
    return out if b is None else out + b


# ---- the state-space mixer ----------------------------------------------------------------------------------------------
def mamba2_mixer(h, W, p, m, eps):
    """m: heads, vdim, state, groups, norm_groups, conv.  Per head a (state, vdim) matrix S:
    a = exp(-exp(A_log) dt);  M <- a M + dt B x^T;  y = M^T C + D x."""
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner, T = H * P, h.shape[0]
    u = h @ W[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + W[p + "dt_bias"])
    decay = np.exp(-np.exp(W[p + "A_log"]) * dt)  # (T, H)
    grp = np.arange(H) // (H // G)
    S = np.zeros((H, N, P))
    y = np.zeros((T, H, P))
    for t in range(T):
        S = decay[t][:, None, None] * S + dt[t][:, None, None] * B[t, grp][:, :, None] * x[t][:, None, :]
        y[t] = np.einsum("hnp,hn->hp", S, C[t, grp]) + W[p + "D"][:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)
    ng = m["norm_groups"]
    y = rms(y.reshape(T, ng, inner // ng), eps).reshape(T, inner) * W[p + "norm"]
    return y @ W[p + "o"].T


# ---- the two halves of the parallel mixer ----------------------------------------------------------------------------------
def distance_bucket(n, rows, far):
    """Row of the distance-bias table for distance n >= 0: exact below rows // 2, logarithmic up to `far`, then the last."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def sees(i, j, window, keep):
    return j <= i and (i - j < window or j < keep)


def sigmoid_attention_core(q, k, rel, head_bias, window, keep, scale, far):
    """q (T, H, d), k (T, G, d) -> (T, H, d): position i sees j <= i with i - j < window (window 0: all) or j < keep;
    weight sigmoid(q.k scale + rel[bucket(i - j), head] + head_bias[head]), not normalised; the values are the keys."""
    T, H, d = q.shape
    G = k.shape[1]
    bucket = np.array([distance_bucket(n, rel.shape[0], far) for n in range(T)])
    out = np.zeros((T, H, d))
    for i in range(T):
        js = [j for j in range(i + 1) if window == 0 or sees(i, j, window, keep)]
        for a in range(H):
            kk = k[js, a // (H // G)]
            s = kk @ q[i, a] * scale + rel[bucket[i - np.array(js)], a] + head_bias[a]
            out[i, a] = sigmoid(s) @ kk
    return out


def sigmoid_attention(h, W, p, m):
    """Grouped-query attention with biased projections, values = keys, sliding window plus the sequence's first
    `keep_first` tokens, and a sigmoid output gate."""
    H, G, d, T = m["heads"], m["kv_heads"], m["dim"], h.shape[0]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(T, H, d)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).reshape(T, G, d)
    out = sigmoid_attention_core(q, k, W[p + "rel"], W[p + "pb"], m["mask"]["size"], m["mask"]["keep_first"], m["scale"], m["bias_max"])
    out = out.reshape(T, H * d) * sigmoid(h @ W[p + "g"].T)
    return out @ W[p + "o"].T


def matrix_state_scan(k, q, v, decay, beta=None, vscale=None, skip=None):
    """k, q (T, H, D), v (T, H, P), decay a (T, H) or (T, H, D): M <- a M; e = beta (v - M^T k) or vscale v;
    M <- M + k e^T; y = M^T q + skip v.  Returns (y, final M)."""
    T, H, D = k.shape
    P = v.shape[2]
    S = np.zeros((H, D, P))
    o = np.zeros((T, H, P))
    for t in range(T):
        g = decay[t][:, :, None] if decay.ndim == 3 else decay[t][:, None, None]
        S = g * S
        if beta is not None:
            u = beta[t][:, None] * (v[t] - np.einsum("hdp,hd->hp", S, k[t]))
        else:
            u = (vscale[t][:, None] if vscale is not None else 1.0) * v[t]
        S = S + k[t][:, :, None] * u[:, None, :]
        o[t] = np.einsum("hdp,hd->hp", S, q[t])
        if skip is not None:
            o[t] += skip[:, None] * v[t]
    return o, S


def gated_delta_mixer(h, W, p, m, eps):
    """Per head a (dim, vdim) matrix S with one decay per key channel:
    M <- diag(a) M;  e = beta (v - M^T k);  M <- M + k e^T;  y = M^T q."""
    H, G, d, P, T = m["heads"], m["kv_heads"], m["dim"], m["vdim"], h.shape[0]
    q = silu(causal_conv(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, G, d)
    k = silu(causal_conv(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, G, d)
    v = silu(causal_conv(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, P)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ W[p + "b"].T)                                             # (T, H)
    step = softplus((h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]).reshape(T, H, d)
    g = np.exp(-np.exp(W[p + "A_log"])[None, :, None] * step)                     # (T, H, d)
    grp = np.arange(H) // (H // G)
    S = np.zeros((H, d, P))
    o = np.zeros((T, H, P))
    for t in range(T):
        kt, qt = k[t, grp], q[t, grp]
        S = g[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - np.einsum("hdp,hd->hp", S, kt))
        S = S + kt[:, :, None] * u[:, None, :]
        o[t] = np.einsum("hdp,hd->hp", S, qt)
    gate = sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T).reshape(T, H, P)
    o = rms(o, eps) * W[p + "norm"] * gate
    return o.reshape(T, H * P) @ W[p + "o"].T


def parallel_mixer(h, W, p, m, eps):
    return m["left_scale"] * sigmoid_attention(h, W, p + "left.", m["left"]) + m["right_scale"] * gated_delta_mixer(h, W, p + "right.", m["right"], eps)


# ---- experts ---------------------------------------------------------------------------------------------------------------
def route(z, top, groups, keep):
    """z (E,) router logits -> (chosen experts, weights): softmax scores; the experts form `groups` equal groups of
    neighbours, a group scores its best expert, only the `keep` best groups stay eligible; the `top` best eligible
    experts, weighted by their scores over the sum of the chosen scores."""
    s = np.exp(z - z.max())
    s = s / s.sum()
    E = len(s)
    per = E // groups
    gs = s.reshape(groups, per).max(1)
    kept = np.argsort(-gs, kind="stable")[:keep]
    ok = np.zeros(E, bool)
    for g in kept:
        ok[g * per:(g + 1) * per] = True
    ids = np.argsort(-np.where(ok, s, -1.0), kind="stable")[:top]
    return ids, s[ids] / (s[ids].sum() + 1e-20)


def expert(h, wg, wu, wd, limit):
    g = np.minimum(h @ wg.T, limit)
    u = np.clip(h @ wu.T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ wd.T


def experts_ffn(h, W, p, f, router_input=None):
    r = f["router"]
    z = (h if router_input is None else router_input) @ W[p + "router"].T
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        ids, w = route(z[t], r["top"], r["groups"]["count"], r["groups"]["keep"])
        for e, we in zip(ids, w):
            out[t] += we * expert(h[t], W[p + "e%d.gate" % e], W[p + "e%d.up" % e], W[p + "e%d.down" % e], f["expert"]["limit"])
    return out


# ---- the model -----------------------------------------------------------------------------------------------------------
def forward(cfg, W, tokens, layers_out=None):
    """Logits (T, vocab) of a whole sequence."""
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    x = W["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"] + W["pos"][:T]
    x = rms(x, eps) * W["embed.norm"]
    for i, L in enumerate(cfg["layers"]):
        p = "l%d." % i
        h = rms(x, eps) * W[p + "norm1"]
        hs = token_shift(h, W[p + "shift"])
        if L["type"] == "mamba2":
            y = mamba2_mixer(hs, W, p + "mix.", L["mixer"], eps)
        elif L["type"] == "parallel":
            y = parallel_mixer(hs, W, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        if L.get("mlp"):
            y = y + experts_ffn(h, W, p + "mlp.", L["mlp"])
        x = x + y
        if layers_out is not None:
            layers_out.append(x.copy())
    x = rms(x, eps) * W["final.norm"]
    z = x @ W["head"].T
    c = cfg["logit_softcap"]
    return c * np.tanh(z / c)


def greedy(cfg, W, prompt, n_gen):
    toks = list(prompt)
    for _ in range(n_gen):
        toks.append(int(np.argmax(forward(cfg, W, toks)[-1])))
    return toks[len(prompt):]


# ---- small random models -----------------------------------------------------------------------------------------------
def moe(ff=24, experts=6, top=2, groups=3, keep=2, limit=1.5):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}}


def mamba2_layer(heads=4, vdim=12, state=8, groups=2, norm_groups=2, conv=3, mlp=None):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}, "mlp": mlp}


def parallel_layer(heads=4, kv_heads=2, dim=16, window=9, keep_first=3, bias_max=40, scale=0.4, rheads=4, rkv=2, rdim=12, rvdim=20, conv=3,
                   left_scale=0.7, right_scale=1.2, mlp=None):
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "bias_max": bias_max, "scale": scale,
                               "mask": {"size": window, "keep_first": keep_first}},
                      "right": {"heads": rheads, "kv_heads": rkv, "dim": rdim, "vdim": rvdim, "conv": conv},
                      "left_scale": left_scale, "right_scale": right_scale}, "mlp": mlp}


def make_config(width=48, vocab=96, max_positions=256, layers=None, eps=1e-4, embed_scale=3.0, softcap=9.0):
    return {"architecture": "Fapudra", "width": width, "vocab": vocab, "max_positions": max_positions, "norm": {"eps": eps},
            "embedding": {"scale": embed_scale}, "logit_softcap": softcap, "layers": layers}


def random_weights(cfg, seed=0, rel_rows=10, low_rank=5):
    """name -> float32 array whose values are exactly representable in bfloat16."""
    rng = np.random.default_rng(seed)
    Wd, V = cfg["width"], cfg["vocab"]
    t = {}

    def mat(o, i, s=None):
        return (rng.standard_normal((o, i)) * (s if s else 1.0 / np.sqrt(i))).astype(np.float32)

    def vec(n, s=1.0, mean=0.0):
        return (mean + s * rng.standard_normal(n)).astype(np.float32)

    def scalar(lo, hi):
        return np.float32(rng.uniform(lo, hi)).reshape(())

    t["embed"], t["pos"], t["embed.norm"] = mat(V, Wd, 1.0), mat(cfg["max_positions"], Wd, 0.5), scalar(0.8, 1.3)
    t["final.norm"], t["head"] = scalar(0.8, 1.3), mat(V, Wd)
    for i, L in enumerate(cfg["layers"]):
        p, m = "l%d." % i, L["mixer"]
        t[p + "norm1"], t[p + "shift"] = scalar(0.8, 1.3), rng.uniform(0.0, 1.0, Wd).astype(np.float32)
        if L["type"] == "mamba2":
            H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, ch = H * P, H * P + 2 * G * N
            t[p + "mix.in"] = mat(2 * inner + 2 * G * N + H, Wd)
            t[p + "mix.conv"], t[p + "mix.conv.b"] = mat(ch, m["conv"], 0.5), vec(ch, 0.2)
            t[p + "mix.dt_bias"], t[p + "mix.A_log"], t[p + "mix.D"] = vec(H, 0.5, -1.0), vec(H, 0.4, -0.5), vec(H, 0.5, 1.0)
            t[p + "mix.norm"], t[p + "mix.o"] = vec(inner, 0.2, 1.0), mat(Wd, inner)
        else:
            a, b = m["left"], m["right"]
            nq, nk = a["heads"] * a["dim"], a["kv_heads"] * a["dim"]
            q = p + "mix.left."
            t[q + "q"], t[q + "q.b"], t[q + "k"], t[q + "k.b"] = mat(nq, Wd), vec(nq, 0.3), mat(nk, Wd), vec(nk, 0.3)
            t[q + "rel"], t[q + "pb"] = mat(rel_rows, a["heads"], 1.0), vec(a["heads"], 0.5, -1.0)
            t[q + "g"], t[q + "o"] = mat(nq, Wd), mat(Wd, nq, 0.5 / np.sqrt(nq))
            r = p + "mix.right."
            nk, nv = b["kv_heads"] * b["dim"], b["heads"] * b["vdim"]
            nd = b["heads"] * b["dim"]
            t[r + "q"], t[r + "k"], t[r + "v"] = mat(nk, Wd), mat(nk, Wd), mat(nv, Wd)
            t[r + "q.conv"], t[r + "k.conv"], t[r + "v.conv"] = mat(nk, b["conv"], 0.6), mat(nk, b["conv"], 0.6), mat(nv, b["conv"], 0.6)
            t[r + "b"], t[r + "A_log"], t[r + "norm"] = mat(b["heads"], Wd), vec(b["heads"], 0.4, -1.0), vec(b["vdim"], 0.2, 1.0)
            t[r + "a1"], t[r + "a2"], t[r + "dt_bias"] = mat(low_rank, Wd), mat(nd, low_rank), vec(nd, 0.5, -1.0)
            t[r + "g1"], t[r + "g2"], t[r + "o"] = mat(low_rank, Wd), mat(nv, low_rank), mat(Wd, nv)
        f = L.get("mlp")
        if f:
            ff = f["expert"]["ff"]
            for e in range(f["router"]["experts"]):
                t[p + "mlp.e%d.gate" % e], t[p + "mlp.e%d.up" % e], t[p + "mlp.e%d.down" % e] = mat(ff, Wd, 0.3), mat(ff, Wd, 0.3), mat(Wd, ff)
            t[p + "mlp.router"] = mat(f["router"]["experts"], Wd, 0.5)
    return {k: from_bf16_bits(to_bf16_bits(v)).reshape(v.shape) for k, v in t.items()}


def as_f64(weights):
    return {k: np.asarray(v, np.float64) for k, v in weights.items()}
