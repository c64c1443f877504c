"""Kodupel front end (zl_kodupel_* C-ABI): configuration from config.json, weight loading, and the step call.

Kodupel is a decoder-only family whose config.json lists the layers one by one.  A layer is x += norm1(mixer(x)),
x += norm2(experts(x)) with RMS norms (weight 1 + w) on the sublayers' outputs only and an fp32 residual stream
x = embedding.scale * embed[token].  Mixers:

  * "attention": grouped key/value heads, biased q / k / v / o projections, RMS norm per head on queries and keys,
    rotation of the first rot.dims dimensions in adjacent pairs with YaRN-scaled frequencies, value heads of unit RMS,
    a causal softmax whose denominator holds an extra 1, one sigmoid gate per head; "kv_from": j reads layer j's cache;
  * "general_delta": per head a (dim, dim) fp32 state S <- diag(w) S - (a u)(u^T S) + k v^T, o = S^T r, then per-head
    RMS norm, a weight, a sigmoid gate and the output projection.

The feed-forward is a mixture of clamped gated experts, chosen by sigmoid scores plus a correction, weighted by the
scores.  config.json:

    {"architecture": "Kodupel", "vocab": V, "width": D, "embedding": {"scale": s}, "norm": {"eps": e},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", optional "kv_from",
                           "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"} or absent}},
                 "mlp": {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"}} or null},
                {"type": "general_delta", "mixer": {"heads", "dim"}, "mlp": ...}, ...]}

Checkpoint tensors: embed, head, final.norm, per layer l<i>.norm1 / norm2, attention l<i>.mix.{q, q.b, k, k.b, v, v.b,
q.norm, k.norm, g, o, o.b}, delta rule l<i>.mix.{r, k, v, a, a.b, g, w1, w2, w0, norm, o} (the inner size of the decay
path is w1's row count), experts l<i>.mlp.{router, correction, e<j>.gate, e<j>.up, e<j>.down}; Linears are (out, in).
"""
import ctypes

import numpy as np

from . import _lib
from .safetensors_io import is_bf16

MIXERS = {"attention": 0, "general_delta": 1}


class KodupelLayer(ctypes.Structure):
    """zl_kodupel_layer_t"""
    _fields_ = [("type", ctypes.c_int), ("heads", ctypes.c_int), ("kv_heads", ctypes.c_int), ("dim", ctypes.c_int),
                ("vdim", ctypes.c_int), ("kv_from", ctypes.c_int), ("rot_dims", ctypes.c_int), ("rot_base", ctypes.c_float),
                ("yarn_factor", ctypes.c_float), ("yarn_original", ctypes.c_float), ("yarn_fast", ctypes.c_float),
                ("yarn_slow", ctypes.c_float), ("scale", ctypes.c_float), ("decay_rank", ctypes.c_int),
                ("experts", ctypes.c_int), ("top", ctypes.c_int), ("ff", ctypes.c_int), ("limit", ctypes.c_float)]


class KodupelCConfig(ctypes.Structure):
    """zl_kodupel_config_t"""
    _fields_ = [("num_layers", ctypes.c_int), ("width", ctypes.c_int), ("vocab", ctypes.c_int), ("eps", ctypes.c_float),
                ("embed_scale", ctypes.c_float), ("dtype", ctypes.c_int), ("max_batch", ctypes.c_int),
                ("max_seq", ctypes.c_int), ("max_step_tokens", ctypes.c_int), ("use_pdl", ctypes.c_int),
                ("use_graph", ctypes.c_int)]


class KodupelConfig:
    """Parsed config.json of a Kodupel model.  `layers` is a list of dicts with every key of zl_kodupel_layer_t;
    decay_rank 0 means "take it from the checkpoint" (the row count of l<i>.mix.w1)."""

    def __init__(self, vocab, width, layers, norm_eps=1e-5, embed_scale=1.0):
        self.vocab, self.width = int(vocab), int(width)
        self.norm_eps, self.embed_scale = float(norm_eps), float(embed_scale)
        self.layers = layers
        for i, l in enumerate(layers):
            if l["type"] == "attention":
                if l["heads"] % l["kv_heads"]:
                    raise ValueError("layer %d: heads is not a multiple of kv_heads" % i)
                if l["rot_dims"] % 2 or l["rot_dims"] > l["dim"]:
                    raise ValueError("layer %d: rot.dims must be even and at most dim" % i)
                j = l["kv_from"]
                if j >= 0:
                    s = layers[j] if j < i else None
                    if not (s and s["type"] == "attention" and s["kv_from"] < 0 and
                            all(s[k] == l[k] for k in ("kv_heads", "dim", "vdim"))):
                        raise ValueError("layer %d: kv_from must name an earlier attention layer with keys and values of "
                                         "its own and the same shape" % i)
            if l["experts"] and not 0 < l["top"] <= l["experts"]:
                raise ValueError("layer %d: router.top must be between 1 and router.experts" % i)

    @classmethod
    def from_dict(cls, d):
        layers = []
        for i, l in enumerate(d["layers"]):
            kind = l.get("type")
            if kind not in MIXERS:
                raise ValueError("layer %d: unknown mixer type %r" % (i, kind))
            mx, mlp = l["mixer"], l.get("mlp")
            out = dict(type=kind, heads=int(mx["heads"]), dim=int(mx["dim"]), kv_heads=0, vdim=0, kv_from=-1, rot_dims=0,
                       rot_base=10000.0, yarn_factor=0.0, yarn_original=0.0, yarn_fast=0.0, yarn_slow=0.0, scale=0.0,
                       decay_rank=0, experts=0, top=0, ff=0, limit=0.0)
            if kind == "attention":
                rot = mx.get("rot") or {}
                sc = rot.get("scaling") or {}
                kv_from = mx.get("kv_from")
                out.update(kv_heads=int(mx.get("kv_heads", mx["heads"])), vdim=int(mx.get("vdim", mx["dim"])),
                           kv_from=-1 if kv_from is None else int(kv_from), rot_dims=int(rot.get("dims", 0)),
                           rot_base=float(rot.get("base", 10000.0)), scale=float(mx.get("scale", int(mx["dim"]) ** -0.5)))
                if sc:
                    out.update(yarn_factor=float(sc["factor"]), yarn_original=float(sc["original"]),
                               yarn_fast=float(sc["fast"]), yarn_slow=float(sc["slow"]))
            else:
                out.update(decay_rank=int(mx.get("decay_rank", 0)))
            if mlp is not None:
                if mlp.get("kind", "moe") != "moe":
                    raise ValueError("layer %d: unknown feed-forward kind %r" % (i, mlp.get("kind")))
                out.update(experts=int(mlp["router"]["experts"]), top=int(mlp["router"]["top"]), ff=int(mlp["expert"]["ff"]),
                           limit=float(mlp["expert"]["limit"]))
            layers.append(out)
        return cls(d["vocab"], d["width"], layers, (d.get("norm") or {}).get("eps", 1e-5),
                   (d.get("embedding") or {}).get("scale", 1.0))

    def to_dict(self):
        out = []
        for l in self.layers:
            if l["type"] == "attention":
                mx = {k: l[k] for k in ("heads", "kv_heads", "dim", "vdim", "scale")}
                mx["rot"] = {"base": l["rot_base"], "dims": l["rot_dims"]}
                if l["yarn_factor"] > 0:
                    mx["rot"]["scaling"] = {"factor": l["yarn_factor"], "original": l["yarn_original"], "fast": l["yarn_fast"],
                                            "slow": l["yarn_slow"]}
                if l["kv_from"] >= 0:
                    mx["kv_from"] = l["kv_from"]
            else:
                mx = {"heads": l["heads"], "dim": l["dim"]}
            mlp = None
            if l["experts"]:
                mlp = {"kind": "moe", "expert": {"ff": l["ff"], "limit": l["limit"]},
                       "router": {"experts": l["experts"], "top": l["top"]}}
            out.append({"type": l["type"], "mixer": mx, "mlp": mlp})
        return {"architecture": "Kodupel", "vocab": self.vocab, "width": self.width, "layers": out,
                "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embed_scale}}

    def tensor_shapes(self):
        """name -> shape of every checkpoint tensor (decay_rank must be known)."""
        D, s = self.width, {}
        s["embed"] = s["head"] = (self.vocab, D)
        s["final.norm"] = (D,)
        for i, l in enumerate(self.layers):
            p, H, d = "l%d." % i, l["heads"], l["dim"]
            s[p + "norm1"] = (D,)
            if l["type"] == "attention":
                G, vd = l["kv_heads"], l["vdim"]
                s[p + "mix.q"], s[p + "mix.q.b"], s[p + "mix.q.norm"] = (H * d, D), (H * d,), (d,)
                if l["kv_from"] < 0:
                    s[p + "mix.k"], s[p + "mix.k.b"], s[p + "mix.k.norm"] = (G * d, D), (G * d,), (d,)
                    s[p + "mix.v"], s[p + "mix.v.b"] = (G * vd, D), (G * vd,)
                s[p + "mix.g"], s[p + "mix.o"], s[p + "mix.o.b"] = (H, D), (D, H * vd), (D,)
            else:
                for n in "rkvag":
                    s[p + "mix." + n] = (H * d, D)
                s[p + "mix.a.b"] = s[p + "mix.w0"] = s[p + "mix.norm"] = (H * d,)
                s[p + "mix.w1"], s[p + "mix.w2"] = (l["decay_rank"], D), (H * d, l["decay_rank"])
                s[p + "mix.o"] = (D, H * d)
            if l["experts"]:
                s[p + "norm2"] = (D,)
                s[p + "mlp.router"], s[p + "mlp.correction"] = (l["experts"], D), (l["experts"],)
                for e in range(l["experts"]):
                    s[p + "mlp.e%d.gate" % e] = s[p + "mlp.e%d.up" % e] = (l["ff"], D)
                    s[p + "mlp.e%d.down" % e] = (D, l["ff"])
        return s


DTYPES = {"bf16": 1, "bfloat16": 1, "f32": 2, "float32": 2}


class KodupelDecoder:
    """One model instance on the current CUDA device.  Slots (0..max_batch-1) each own `max_seq` key / value rows per
    attention layer and the recurrent states of the delta-rule layers; the engine's scheduler decides which sequence
    lives in which slot.  The native model is created when the sizes are complete: at once if every delta-rule layer's
    decay_rank is given, otherwise when load_state_dict sees the checkpoint."""

    architecture = "Kodupel"
    supports_dtypes = ("bfloat16", "float32")
    supports_ragged_steps = True

    def __init__(self, config, dtype="bf16", max_batch=1, max_seq=512, max_step_tokens=512, use_pdl=True, use_graph=True):
        self.lib = _lib.load()
        self.config = config
        self.vocab_size = config.vocab
        self.dtype = dtype
        self.max_batch, self.max_seq = int(max_batch), int(max_seq)
        self.max_step_tokens = max(int(max_step_tokens), self.max_batch)
        self.use_pdl, self.use_graph = use_pdl, use_graph
        self.h = None
        if all(l["type"] != "general_delta" or l["decay_rank"] > 0 for l in config.layers):
            self._create()

    def _create(self):
        c = self.config
        self.cfg = KodupelCConfig(len(c.layers), c.width, c.vocab, c.norm_eps, c.embed_scale, DTYPES[self.dtype],
                                  self.max_batch, self.max_seq, self.max_step_tokens, int(self.use_pdl), int(self.use_graph))
        arr = (KodupelLayer * len(c.layers))()
        for i, l in enumerate(c.layers):
            arr[i] = KodupelLayer(MIXERS[l["type"]], l["heads"], l["kv_heads"], l["dim"], l["vdim"], l["kv_from"], l["rot_dims"],
                                  l["rot_base"], l["yarn_factor"], l["yarn_original"], l["yarn_fast"], l["yarn_slow"],
                                  l["scale"], l["decay_rank"], l["experts"], l["top"], l["ff"], l["limit"])
        h = ctypes.c_void_p()
        _lib.check(self.lib.zl_kodupel_create(ctypes.byref(self.cfg), arr, ctypes.byref(h)))
        self.h = h

    @classmethod
    def from_config_dict(cls, d, **kw):
        return cls(KodupelConfig.from_dict(d), **kw)

    def close(self):
        if getattr(self, "h", None):
            self.lib.zl_kodupel_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def load_state_dict(self, state_dict):
        """name -> numpy array: bfloat16 bit patterns (safetensors_io.Bf16Array) or float32."""
        for i, l in enumerate(self.config.layers):
            if l["type"] == "general_delta" and l["decay_rank"] <= 0:
                name = "l%d.mix.w1" % i
                if name not in state_dict:
                    raise ValueError("tensor %s is missing" % name)
                l["decay_rank"] = int(np.asarray(state_dict[name]).shape[0])
        if self.h is None:
            self._create()
        needed = self.config.tensor_shapes()
        for name, arr in state_dict.items():
            a = np.ascontiguousarray(arr)
            if name not in needed:
                continue                      # a checkpoint may carry tensors this family does not use
            if not (is_bf16(arr) or a.dtype == np.float32):
                raise ValueError("tensor %s: expected bfloat16 or float32, got %s" % (name, a.dtype))
            if tuple(a.shape) != tuple(needed[name]):
                raise ValueError("tensor %s: shape %s, expected %s" % (name, tuple(a.shape), tuple(needed[name])))
            rows, cols = (1, a.size) if a.ndim <= 1 else (a.shape[0], a.size // a.shape[0])
            _lib.check(self.lib.zl_kodupel_load_tensor(self.h, name.encode(), a.ctypes.data_as(ctypes.c_void_p), rows, cols,
                                                       a.itemsize))
        _lib.check(self.lib.zl_kodupel_finalize(self.h))

    def init_synthetic(self, seed=0):
        for l in self.config.layers:
            if l["type"] == "general_delta" and l["decay_rank"] <= 0:
                l["decay_rank"] = 64
        if self.h is None:
            self._create()
        _lib.check(self.lib.zl_kodupel_init_synthetic(self.h, seed))

    def step(self, tokens, slots, positions, want_rows=(), want_logits=True):
        """One step over T rows.  Returns (next tokens (n_want), logits (n_want, vocab) or None) for the wanted rows."""
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        s = np.ascontiguousarray(slots, dtype=np.int32)
        p = np.ascontiguousarray(positions, dtype=np.int32)
        w = np.ascontiguousarray(want_rows, dtype=np.int32)
        nxt = np.empty(w.size, dtype=np.int32)
        logits = np.empty((w.size, self.vocab_size), dtype=np.float32) if want_logits else None
        _lib.check(self.lib.zl_kodupel_step(
            self.h, t.ctypes.data_as(ctypes.c_void_p), s.ctypes.data_as(ctypes.c_void_p), p.ctypes.data_as(ctypes.c_void_p),
            t.size, w.ctypes.data_as(ctypes.c_void_p) if w.size else None, w.size,
            logits.ctypes.data_as(ctypes.c_void_p) if (want_logits and w.size) else None,
            nxt.ctypes.data_as(ctypes.c_void_p) if w.size else None))
        return nxt, logits

    # the two calls LlamaDecoder offers, on top of step()
    def prefill(self, task, tokens, pos0=0, want_logits=False):
        n = len(tokens)
        nxt, logits = None, None
        for c0 in range(0, n, self.max_step_tokens):
            chunk = tokens[c0:c0 + self.max_step_tokens]
            last = c0 + len(chunk) == n
            nxt, logits = self.step(chunk, [task] * len(chunk), range(pos0 + c0, pos0 + c0 + len(chunk)),
                                    [len(chunk) - 1] if last else [], want_logits)
        return (int(nxt[0]), logits) if want_logits else int(nxt[0])

    def decode(self, tokens, positions, want_logits=False):
        b = len(tokens)
        nxt, logits = self.step(tokens, range(b), positions, range(b), want_logits)
        return (nxt, logits) if want_logits else nxt

    def set_state(self, tokens, positions):
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        p = np.ascontiguousarray(positions, dtype=np.int32)
        _lib.check(self.lib.zl_kodupel_set_state(self.h, t.ctypes.data_as(ctypes.c_void_p), p.ctypes.data_as(ctypes.c_void_p),
                                                 t.size))

    def step_device(self, b):
        _lib.check(self.lib.zl_kodupel_step_device(self.h, b))

    def sync(self):
        _lib.check(self.lib.zl_kodupel_sync(self.h))

    def stream(self):
        return self.lib.zl_kodupel_stream(self.h)

    def capture_layers(self, on=True):
        _lib.check(self.lib.zl_kodupel_capture_layers(self.h, int(on)))

    def read_layers(self, n_tokens):
        out = np.empty((len(self.config.layers), n_tokens, self.config.width), dtype=np.float32)
        _lib.check(self.lib.zl_kodupel_read_layers(self.h, out.ctypes.data_as(ctypes.c_void_p), n_tokens))
        return out

    def read_state(self, layer, slot):
        l = self.config.layers[layer]
        out = np.empty((l["heads"], l["dim"], l["dim"]), dtype=np.float32)
        _lib.check(self.lib.zl_kodupel_read_state(self.h, layer, slot, out.ctypes.data_as(ctypes.c_void_p)))
        return out

    def stats(self):
        wb, kn = ctypes.c_double(), ctypes.c_int()
        _lib.check(self.lib.zl_kodupel_stats(self.h, ctypes.byref(wb), ctypes.byref(kn)))
        return wb.value, kn.value
