"""Plain, slow restatement of the Kodupel layer equations in numpy float64, one function per mechanism.

Nothing here is shared with the product path: attention is a loop over heads on a full score matrix, the recurrence
a loop over tokens with outer products, the experts a loop over tokens and chosen experts.  A whole prompt is computed
at once; by causality the value at a position is also the truth for any way of cutting the prompt into portions or
decoding it token by token.
"""
import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def unit_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def out_norm(y, w, eps):
    """RMS norm times (1 + w): the checkpoint keeps w, not the multiplier."""
    return unit_rms(y, eps) * (1.0 + w)


def rotation_tables(n, dims, base, scaling):
    """cos, sin (n, dims / 2) for positions 0..n-1; scaling = dict(factor, original, fast, slow) or None."""
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    mag = 1.0
    if scaling:
        def where(turns):
            return dims * math.log(scaling["original"] / (2 * math.pi * turns)) / (2 * math.log(base))
        lo = max(math.floor(where(scaling["fast"])), 0)
        hi = min(math.ceil(where(scaling["slow"])), dims - 1)
        ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / scaling["factor"] * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(scaling["factor"]) + 1.0
    ang = np.arange(n, dtype=np.float64)[:, None] * f[None, :]
    return np.cos(ang) * mag, np.sin(ang) * mag


def rotate_pairs(x, cos, sin, dims):
    """x (n, heads, d): dimensions (2i, 2i+1), i < dims / 2, turn by the position's angle; the rest pass."""
    y = x.copy()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    y[..., 0:dims:2] = a * cos[:, None, :] - b * sin[:, None, :]
    y[..., 1:dims:2] = b * cos[:, None, :] + a * sin[:, None, :]
    return y


def unit_sink_attention(q, k, v, scale):
    """q (n, H, d), k (n, G, d), v (n, G, dv): causal, query head h on key/value head h // (H / G); the denominator of
    the softmax holds one extra 1."""
    n, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((n, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        for i in range(n):
            s = (k[: i + 1, g] @ q[i, h]) * scale
            e = np.exp(s)
            out[i, h] = (e / (1.0 + e.sum())) @ v[: i + 1, g]
    return out


def attention_mixer(W, p, l, x, eps, shared):
    """l: the layer's parsed dict (KodupelConfig.layers[i]); shared: {layer index: (k, v)} of the layers before."""
    n = x.shape[0]
    H, G, d, dv = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
    sc = None
    if l["yarn_factor"] > 0:
        sc = dict(factor=l["yarn_factor"], original=l["yarn_original"], fast=l["yarn_fast"], slow=l["yarn_slow"])
    cos, sin = rotation_tables(n, l["rot_dims"], l["rot_base"], sc) if l["rot_dims"] else (None, None)

    def turn(t):
        return rotate_pairs(t, cos, sin, l["rot_dims"]) if l["rot_dims"] else t

    q = (x @ W[p + "q"].T + W[p + "q.b"]).reshape(n, H, d)
    q = turn(unit_rms(q, eps) * W[p + "q.norm"])
    if l["kv_from"] >= 0:
        k, v = shared[l["kv_from"]]
    else:
        k = (x @ W[p + "k"].T + W[p + "k.b"]).reshape(n, G, d)
        k = turn(unit_rms(k, eps) * W[p + "k.norm"])
        v = unit_rms((x @ W[p + "v"].T + W[p + "v.b"]).reshape(n, G, dv), eps)
    o = unit_sink_attention(q, k, v, l["scale"]) * sigmoid(x @ W[p + "g"].T)[:, :, None]
    return o.reshape(n, H * dv) @ W[p + "o"].T + W[p + "o.b"], (k, v)


def delta_rule_scan(r, k, v, w, a, S0=None):
    """r, k, w, a (n, H, dk), v (n, H, dv): S <- diag(w) S - (a u)(u^T S) + k v^T with u the unit key, both subtracted
    terms from the old S; o = S^T r.  Returns (o (n, H, dv), final S (H, dk, dv))."""
    n, H, dk = k.shape
    dv = v.shape[2]
    S = np.zeros((H, dk, dv)) if S0 is None else S0.copy()
    o = np.zeros((n, H, dv))
    for t in range(n):
        for h in range(H):
            u = k[t, h] / math.sqrt(float(k[t, h] @ k[t, h]) + 1e-6)
            old = S[h]
            S[h] = w[t, h][:, None] * old - np.outer(a[t, h] * u, u @ old) + np.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ r[t, h]
    return o, S


def delta_mixer(W, p, l, x, eps):
    n = x.shape[0]
    H, d = l["heads"], l["dim"]
    r, k, v = ((x @ W[p + nm].T).reshape(n, H, d) for nm in "rkv")
    w = np.exp(-math.exp(-0.5) * sigmoid(np.tanh(x @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"])).reshape(n, H, d)
    a = sigmoid(x @ W[p + "a"].T + W[p + "a.b"]).reshape(n, H, d)
    o, S = delta_rule_scan(r, k, v, w, a)
    o = unit_rms(o, eps).reshape(n, H * d) * W[p + "norm"] * sigmoid(x @ W[p + "g"].T)
    return o @ W[p + "o"].T, S


def route(x, w_router, correction, top):
    """-> (chosen experts (n, top), their weights (n, top)): the largest sigmoid score + correction, weights without it."""
    s = sigmoid(x @ w_router.T)
    order = np.argsort(-(s + correction), axis=-1, kind="stable")[:, :top]
    return order, np.take_along_axis(s, order, axis=-1)


def expert(W, p, x, limit):
    g = np.minimum(W[p + "gate"] @ x, limit)
    u = np.clip(W[p + "up"] @ x, -limit, limit)
    return W[p + "down"] @ (g * sigmoid(1.702 * g) * (u + 1.0))


def experts_ff(W, p, l, x):
    chosen, weight = route(x, W[p + "router"], W[p + "correction"], l["top"])
    out = np.zeros_like(x)
    for t in range(x.shape[0]):
        for e, s in zip(chosen[t], weight[t]):
            out[t] += s * expert(W, p + "e%d." % e, x[t], l["limit"])
    return out


def forward(cfg, W, tokens):
    """cfg: KodupelConfig; W: name -> float64 array.  -> (logits (n, vocab), residual stream after every layer
    (layers, n, width), final recurrent states {layer: (H, d, d)})."""
    eps = cfg.norm_eps
    x = W["embed"][np.asarray(tokens)] * cfg.embed_scale
    shared, states, per_layer = {}, {}, []
    for i, l in enumerate(cfg.layers):
        p = "l%d." % i
        if l["type"] == "attention":
            y, shared[i] = attention_mixer(W, p + "mix.", l, x, eps, shared)
        else:
            y, states[i] = delta_mixer(W, p + "mix.", l, x, eps)
        x = x + out_norm(y, W[p + "norm1"], eps)
        if l["experts"]:
            x = x + out_norm(experts_ff(W, p + "mlp.", l, x), W[p + "norm2"], eps)
        per_layer.append(x.copy())
    return out_norm(x, W["final.norm"], eps) @ W["head"].T, np.stack(per_layer), states


def random_weights(cfg, seed=0, router_gain=4.0):
    """name -> float32 array whose values are exact in bfloat16.  Router rows are scaled up so that the choice of
    experts does not hang on a rounding."""
    rng = np.random.default_rng(seed)
    shapes = cfg.tensor_shapes()
    W = {}
    for name, shp in sorted(shapes.items()):
        last = name.rsplit(".", 1)[-1]
        if name.endswith((".q.norm", ".k.norm", "mix.norm")):
            a = 1.0 + 0.2 * rng.standard_normal(shp)
        elif last in ("norm1", "norm2") or name == "final.norm":
            a = 0.1 * rng.standard_normal(shp)
        elif last in ("b", "w0", "correction"):
            a = 0.3 * rng.standard_normal(shp)
        elif name == "embed":
            a = rng.standard_normal(shp)
        elif last == "router":
            a = router_gain * rng.standard_normal(shp) / math.sqrt(shp[-1])
        else:
            a = rng.standard_normal(shp) / math.sqrt(shp[-1])
        W[name] = bf16_round(a.astype(np.float32))
    return W


def bf16_round(a):
    """float32 array rounded to the nearest bfloat16 (ties to even), still float32."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).reshape(np.shape(a))
