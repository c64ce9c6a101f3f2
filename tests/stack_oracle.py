"""Plain, slow float64 statement of the layered architectures' mechanisms, one function per mechanism, and a writer of
small random checkpoints (config.json + model.safetensors).  Nothing here is shared with the library: the tests compare
the library's kernels and step function against these functions.

Notation: x (T, width) residual stream, position t = row t; W matrices are (out, in) and applied as x @ W.T.
"""
import json
import os
import struct

import numpy as np


# ---- mechanisms --------------------------------------------------------------------------------------------------------
def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def norm_one_plus(x, w, eps):
    """RMS norm whose weight is stored around zero."""
    return rms(x, eps) * (1.0 + w)


def qk_norm_whole(p, w, eps):
    """RMS norm over a whole projection row (all heads' channels at once), plain weight."""
    return rms(p, eps) * w


def value_mix(v, v_first, lam):
    return (1.0 - lam) * v + lam * v_first


def visible(i, window, pool):
    """(tokens, blocks) position i attends to: tokens j with 0 <= i - j < window, and block b once its last token
    b * pool + pool - 1 is at or before i - window."""
    toks = [j for j in range(i + 1) if window == 0 or i - j < window]
    blocks = []
    if window > 0 and pool > 0:
        b = 0
        while b * pool + pool - 1 <= i - window:
            blocks.append(b)
            b += 1
    return toks, blocks


def window_pool_attention(q, k, v, window, pool, scale, cache_round=None, rows=None):
    """q (T, H, dk), k (T, G, dk), v (T, G, dv) -> (T, H, dv).  Keys / values are used as the cache holds them
    (cache_round: the cache's rounding, identity if None); a block's key / value is the mean of its members' cached ones.
    rows: only these query positions are computed (the others stay zero)."""
    T, H, dk = q.shape
    G, dv = k.shape[1], v.shape[2]
    if cache_round is not None:
        k, v = cache_round(k), cache_round(v)
    out = np.zeros((T, H, dv))
    for i in (range(T) if rows is None else rows):
        toks, blocks = visible(i, window, pool)
        for h in range(H):
            g = h // (H // G)
            keys = [k[b * pool:(b + 1) * pool, g].mean(0) for b in blocks] + [k[j, g] for j in toks]
            vals = [v[b * pool:(b + 1) * pool, g].mean(0) for b in blocks] + [v[j, g] for j in toks]
            s = np.array([kk @ q[i, h] for kk in keys]) * scale
            w = np.exp(s - s.max())
            w /= w.sum()
            out[i, h] = sum(wi * vi for wi, vi in zip(w, vals))
    return out


def dense_ffn(x, wg, wu, wd, limit):
    g = np.minimum(x @ wg.T, limit) if limit > 0 else x @ wg.T
    u = np.clip(x @ wu.T, -limit, limit) if limit > 0 else x @ wu.T
    return (g / (1.0 + np.exp(-1.702 * g)) * (u + 1.0)) @ wd.T


def route(x, wr, top):
    """Sigmoid scores of the router logits; the `top` largest (ties: lower index) and their scores."""
    s = 1.0 / (1.0 + np.exp(-(x @ wr.T)))
    ids = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return ids, np.take_along_axis(s, ids, -1)


def moe_ffn(x, wr, experts, top):
    """experts: list of (gate, up, down).  The selected score scales the expert's INPUT; outputs are summed."""
    ids, wts = route(x, wr, top)
    y = np.zeros_like(x)
    for t in range(x.shape[0]):
        for e, w in zip(ids[t], wts[t]):
            wg, wu, wd = experts[e]
            h = w * x[t]
            a = wg @ h
            y[t] += wd @ (a / (1.0 + np.exp(-a)) * (wu @ h))
    return y


# ---- the whole model ---------------------------------------------------------------------------------------------------
def forward(cfg, W, tokens, cache_round=None, layers_out=None):
    """Logits (T, vocab) of a Retezen model for one sequence.  W: name -> float64 array."""
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    x = W["embed"][tokens] + W["pos"][:T]
    v_first = None
    for i, L in enumerate(cfg["layers"]):
        p, m = "l%d." % i, L["mixer"]
        H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        q = qk_norm_whole(x @ W[p + "mix.q"].T, W[p + "mix.q.norm"], eps)
        k = qk_norm_whole(x @ W[p + "mix.k"].T, W[p + "mix.k.norm"], eps)
        v = x @ W[p + "mix.v"].T
        if m.get("v_mix"):
            if v_first is None:
                v_first = v
            else:
                v = value_mix(v, v_first, W[p + "mix.vmix"])
        a = window_pool_attention(q.reshape(T, H, dk), k.reshape(T, G, dk), v.reshape(T, G, dv), m["mask"]["size"], m["mask"]["pool"], m["scale"],
                                  cache_round)
        x = x + norm_one_plus(a.reshape(T, H * dv) @ W[p + "mix.o"].T, W[p + "norm1"], eps)
        f = L.get("mlp")
        if f:
            if f["kind"] == "dense":
                y = dense_ffn(x, W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"], f["limit"])
            else:
                E = f["router"]["experts"]
                ex = [(W[p + "mlp.e%d.gate" % e], W[p + "mlp.e%d.up" % e], W[p + "mlp.e%d.down" % e]) for e in range(E)]
                y = moe_ffn(x, W[p + "mlp.router"], ex, f["router"]["top"])
            x = x + norm_one_plus(y, W[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return norm_one_plus(x, W["final.norm"], eps) @ W["head"].T * cfg["logit_scale"]


def greedy(cfg, W, prompt, n_gen, cache_round=None):
    toks = list(prompt)
    out = []
    for _ in range(n_gen):
        lg = forward(cfg, W, toks, cache_round)[-1]
        out.append(int(np.argmax(lg)))
        toks.append(out[-1])
    return out


# ---- checkpoints -------------------------------------------------------------------------------------------------------
def to_bf16_bits(a):
    """float32 -> bfloat16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def from_bf16_bits(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def round_bf16(a):
    return from_bf16_bits(to_bf16_bits(np.asarray(a, np.float32))).astype(np.float64).reshape(np.shape(a))


def make_config(width=96, vocab=160, max_positions=256, layers=None, eps=1e-4, logit_scale=0.7):
    return {"architecture": "Retezen", "width": width, "vocab": vocab, "max_positions": max_positions, "norm": {"eps": eps},
            "logit_scale": logit_scale, "layers": layers}


def attn_layer(heads=6, kv_heads=2, dim=24, vdim=40, window=12, pool=3, scale=0.3, v_mix=True, mlp=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window, "pool": pool},
                                           "scale": scale, "v_mix": v_mix}, "mlp": mlp}


def dense(ff=72, limit=1.5):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff=40, experts=5, top=2):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def random_weights(cfg, seed=0, sharp=1.0):
    """name -> float32 array whose values are exactly representable in bfloat16.  `sharp` scales the q norm weights, which
    makes the softmax peaky so that one key more or less in the visible set moves the output."""
    rng = np.random.default_rng(seed)
    Wd, V = cfg["width"], cfg["vocab"]
    t = {}

    def mat(o, i, s=None):
        return (rng.standard_normal((o, i)) * (s if s else 1.0 / np.sqrt(i))).astype(np.float32)

    t["embed"], t["pos"] = mat(V, Wd, 1.0), mat(cfg["max_positions"], Wd, 0.5)
    t["final.norm"], t["head"] = (rng.standard_normal(Wd) * 0.2).astype(np.float32), mat(V, Wd)
    for i, L in enumerate(cfg["layers"]):
        p, m = "l%d." % i, L["mixer"]
        nq, nk, nv, no = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"], m["heads"] * m["vdim"]
        t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"], t[p + "mix.o"] = mat(nq, Wd), mat(nk, Wd), mat(nv, Wd), mat(Wd, no)
        t[p + "mix.q.norm"] = ((1.0 + 0.3 * rng.standard_normal(nq)) * sharp).astype(np.float32)
        t[p + "mix.k.norm"] = (1.0 + 0.3 * rng.standard_normal(nk)).astype(np.float32)
        t[p + "mix.vmix"] = np.float32(rng.uniform(0.2, 0.8)).reshape(())
        t[p + "norm1"], t[p + "norm2"] = (rng.standard_normal(Wd) * 0.2).astype(np.float32), (rng.standard_normal(Wd) * 0.2).astype(np.float32)
        f = L.get("mlp")
        if f and f["kind"] == "dense":
            t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"] = mat(f["ff"], Wd, 0.4), mat(f["ff"], Wd, 0.4), mat(Wd, f["ff"])
        elif f:
            for e in range(f["router"]["experts"]):
                ff = f["expert"]["ff"]
                t[p + "mlp.e%d.gate" % e], t[p + "mlp.e%d.up" % e], t[p + "mlp.e%d.down" % e] = mat(ff, Wd, 0.3), mat(ff, Wd, 0.3), mat(Wd, ff)
            t[p + "mlp.router"] = mat(f["router"]["experts"], Wd, 0.5)
    return {k: from_bf16_bits(to_bf16_bits(v)).reshape(v.shape) for k, v in t.items()}


def write_checkpoint(folder, cfg, weights, store="BF16"):
    """config.json + model.safetensors (u64 header length | JSON header | data), tensors stored as BF16 or F32."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, off = {}, [], 0
    for name, a in weights.items():
        raw = (to_bf16_bits(a) if store == "BF16" else np.ascontiguousarray(a, np.float32)).tobytes()
        header[name] = {"dtype": store, "shape": list(a.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    h = json.dumps(header).encode()
    h += b" " * (-len(h) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))
    return folder


def as_f64(weights):
    return {k: np.asarray(v, np.float64) for k, v in weights.items()}
