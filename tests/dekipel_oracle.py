"""Plain, slow restatement of the Dekipel layer equations in numpy float64, one function per mechanism.

Nothing here is shared with the product path: keys and values are expanded from the latents (the product never does
that), the convolution is a loop over taps on a zero-padded array, the softmax is written out with its sink term.
A whole prompt is computed at once; the value at a position is, by causality, also the truth for any way of cutting
the prompt into portions or decoding it token by token.
"""
import numpy as np


def rms_norm(x, w, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def group_rms_norm(x, w, groups, eps):
    t, d = x.shape
    parts = x.reshape(t, groups, d // groups)
    parts = parts / np.sqrt(np.mean(parts * parts, axis=-1, keepdims=True) + eps)
    return parts.reshape(t, d) * w


def conv_mix(h, w):
    """h (n, D), w (D, taps): h_t + sum_j w[:, j] h_(t - taps + 1 + j), zeros before the start."""
    n, d = h.shape
    taps = w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, d)), h], axis=0)
    out = h.copy()
    for t in range(n):
        for j in range(taps):
            out[t] += w[:, j] * padded[t + j]
    return out


def sink_softmax_attention(q, k, v, sink, scale):
    """q (n, H, d), k (n, H, d), v (n, H, dv), sink (H): causal; the denominator also holds exp(sink_h)."""
    n, H, _ = q.shape
    out = np.zeros((n, H, v.shape[2]))
    for h in range(H):
        for i in range(n):
            s = (k[: i + 1, h] @ q[i, h]) * scale
            m = max(s.max(), sink[h])
            e = np.exp(s - m)
            out[i, h] = (e[:, None] * v[: i + 1, h]).sum(0) / (e.sum() + np.exp(sink[h] - m))
    return out


def latent_mixer(u, W, p, lc, latent, eps):
    """u (n, D) mixer input.  latent: the cached c of the source layer (kv_from) or None.  Returns (out, c)."""
    n = u.shape[0]
    H, d, dv = lc["heads"], lc["dim"], lc["vdim"]
    cq = rms_norm(u @ W[p + "mix.dq"].T, W[p + "mix.dq.norm"], eps)
    q = (cq @ W[p + "mix.uq"].T).reshape(n, H, d)
    c = latent if latent is not None else rms_norm(u @ W[p + "mix.dkv"].T, W[p + "mix.dkv.norm"], eps)
    k = (c @ W[p + "mix.uk"].T).reshape(n, H, d)
    v = (c @ W[p + "mix.uv"].T).reshape(n, H, dv)
    o = sink_softmax_attention(q, k, v, W[p + "mix.sink"], lc["scale"]).reshape(n, H * dv)
    gate = 1.0 / (1.0 + np.exp(-(u @ W[p + "mix.g"].T)))
    return (o * gate) @ W[p + "mix.o"].T, c


def relu2_ff(u, W, p):
    a = np.maximum(u @ W[p + "mlp.up"].T, 0.0)
    return (a * a) @ W[p + "mlp.down"].T


def forward(cfg, W, tokens):
    """cfg: DekipelConfig-like (layers, norm_eps, norm_groups, canon_taps); W: name -> float64 arrays.
    Returns (logits (n, V), residual stream after every layer (L, n, D))."""
    eps, G = cfg.norm_eps, cfg.norm_groups
    x = W["embed"][np.asarray(tokens)]
    latents, streams = {}, []
    for i, lc in enumerate(cfg.layers):
        p = "l%d." % i
        u = conv_mix(group_rms_norm(x, W[p + "norm1"], G, eps), W[p + "canon1"])
        src = latents[lc["kv_from"]] if lc["kv_from"] >= 0 else None
        y, c = latent_mixer(u, W, p, lc, src, eps)
        if lc["kv_from"] < 0:
            latents[i] = c
        x = x + group_rms_norm(y, W[p + "norm1b"], G, eps)
        if lc["ff"]:
            u = conv_mix(group_rms_norm(x, W[p + "norm2"], G, eps), W[p + "canon2"])
            x = x + group_rms_norm(relu2_ff(u, W, p), W[p + "norm2b"], G, eps)
        streams.append(x.copy())
    return group_rms_norm(x, W["final.norm"], G, eps) @ W["head"].T, np.stack(streams)


def random_weights(cfg, seed, sink_range=1.0):
    """Random bfloat16-representable weights: name -> float32 arrays (exact in bfloat16)."""
    rng = np.random.default_rng(seed)

    def bf(a):
        u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
        return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)

    out = {}
    for name, shape in cfg.tensor_shapes().items():
        base = name.split(".")[-1]
        if base in ("norm1", "norm1b", "norm2", "norm2b") or name.endswith(".norm"):
            a = rng.uniform(0.7, 1.3, shape)
        elif base == "sink":
            a = rng.uniform(-sink_range, sink_range, shape)
        elif base in ("canon1", "canon2"):
            a = rng.uniform(-0.5, 0.5, shape)
        elif name == "embed":
            a = rng.standard_normal(shape)
        else:
            a = rng.standard_normal(shape) / np.sqrt(shape[-1])
        out[name] = bf(a)
    return out
