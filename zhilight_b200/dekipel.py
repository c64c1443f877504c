"""Dekipel front end (zl_dekipel_* C-ABI): configuration from config.json, weight loading, and the step call.

Dekipel is a decoder-only family of latent-attention layers: low-rank query and key-value latents, no positional
rotation, a causal softmax with a per-head sink, a sigmoid output gate, optionally another layer's latent cache; every
sublayer sits between a pre- and a post-norm (RMS norm in groups) and reads its input through a short causal
convolution; the feed-forward is relu^2.  All sizes and constants are read from config.json:

    {"architecture": "Dekipel", "vocab": V, "width": D, "norm": {"eps": e, "groups": G}, "canon": {"taps": K},
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads", "dim", "vdim", "q_rank", "kv_rank", "scale", optional "kv_from"},
                 "mlp": {"kind": "dense", "ff": F} or null}, ...]}

Checkpoint tensors: embed, head, final.norm, and per layer l<i>.norm1/norm1b/norm2/norm2b, l<i>.canon1/canon2,
l<i>.mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, sink, g, o}, l<i>.mlp.{up, down}; Linears are (out, in).
"""
import ctypes

import numpy as np

from . import _lib
from .safetensors_io import is_bf16

MIXERS = ("latent_attention",)


class DekipelLayer(ctypes.Structure):
    """zl_dekipel_layer_t"""
    _fields_ = [("heads", ctypes.c_int), ("dim", ctypes.c_int), ("vdim", ctypes.c_int), ("q_rank", ctypes.c_int),
                ("kv_rank", ctypes.c_int), ("kv_from", ctypes.c_int), ("ff", ctypes.c_int), ("scale", ctypes.c_float)]


class DekipelCConfig(ctypes.Structure):
    """zl_dekipel_config_t"""
    _fields_ = [("num_layers", ctypes.c_int), ("width", ctypes.c_int), ("vocab", ctypes.c_int),
                ("norm_groups", ctypes.c_int), ("canon_taps", ctypes.c_int), ("eps", ctypes.c_float),
                ("dtype", ctypes.c_int), ("max_batch", ctypes.c_int), ("max_seq", ctypes.c_int),
                ("max_step_tokens", ctypes.c_int), ("use_pdl", ctypes.c_int), ("use_graph", ctypes.c_int)]


class DekipelConfig:
    """Parsed config.json of a Dekipel model."""

    def __init__(self, vocab, width, layers, norm_eps=1e-5, norm_groups=1, canon_taps=1):
        self.vocab, self.width = int(vocab), int(width)
        self.norm_eps, self.norm_groups, self.canon_taps = float(norm_eps), int(norm_groups), int(canon_taps)
        self.layers = layers          # list of dicts: heads, dim, vdim, q_rank, kv_rank, scale, kv_from (-1), ff (0)
        if self.width % self.norm_groups:
            raise ValueError("width is not a multiple of norm.groups")
        for i, l in enumerate(layers):
            j = l["kv_from"]
            if j >= 0 and not (j < i and layers[j]["kv_from"] < 0 and layers[j]["kv_rank"] == l["kv_rank"]):
                raise ValueError("layer %d: kv_from must name an earlier layer with its own latents of the same size" % i)

    @classmethod
    def from_dict(cls, d):
        layers = []
        for i, l in enumerate(d["layers"]):
            if l.get("type") not in MIXERS:
                raise ValueError("layer %d: unknown mixer type %r" % (i, l.get("type")))
            mx, mlp = l["mixer"], l.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise ValueError("layer %d: unknown feed-forward kind %r" % (i, mlp.get("kind")))
            kv_from = mx.get("kv_from")
            layers.append(dict(heads=int(mx["heads"]), dim=int(mx["dim"]), vdim=int(mx["vdim"]), q_rank=int(mx["q_rank"]),
                               kv_rank=int(mx["kv_rank"]), scale=float(mx.get("scale", int(mx["dim"]) ** -0.5)),
                               kv_from=-1 if kv_from is None else int(kv_from), ff=0 if mlp is None else int(mlp["ff"])))
        norm, canon = d.get("norm", {}), d.get("canon", {})
        return cls(d["vocab"], d["width"], layers, norm.get("eps", 1e-5), norm.get("groups", 1), canon.get("taps", 1))

    def to_dict(self):
        out = []
        for l in self.layers:
            mx = {k: l[k] for k in ("heads", "dim", "vdim", "q_rank", "kv_rank", "scale")}
            if l["kv_from"] >= 0:
                mx["kv_from"] = l["kv_from"]
            out.append({"type": "latent_attention", "mixer": mx, "mlp": {"kind": "dense", "ff": l["ff"]} if l["ff"] else None})
        return {"architecture": "Dekipel", "vocab": self.vocab, "width": self.width, "layers": out,
                "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "canon": {"taps": self.canon_taps}}

    def tensor_shapes(self):
        """name -> shape of every checkpoint tensor."""
        D, s = self.width, {}
        s["embed"] = s["head"] = (self.vocab, D)
        s["final.norm"] = (D,)
        for i, l in enumerate(self.layers):
            p, H = "l%d." % i, l["heads"]
            s[p + "norm1"] = s[p + "norm1b"] = (D,)
            s[p + "canon1"] = (D, self.canon_taps)
            s[p + "mix.dq"], s[p + "mix.dq.norm"] = (l["q_rank"], D), (l["q_rank"],)
            s[p + "mix.uq"] = (H * l["dim"], l["q_rank"])
            if l["kv_from"] < 0:
                s[p + "mix.dkv"], s[p + "mix.dkv.norm"] = (l["kv_rank"], D), (l["kv_rank"],)
            s[p + "mix.uk"], s[p + "mix.uv"] = (H * l["dim"], l["kv_rank"]), (H * l["vdim"], l["kv_rank"])
            s[p + "mix.sink"], s[p + "mix.g"], s[p + "mix.o"] = (H,), (H * l["vdim"], D), (D, H * l["vdim"])
            if l["ff"]:
                s[p + "norm2"] = s[p + "norm2b"] = (D,)
                s[p + "canon2"] = (D, self.canon_taps)
                s[p + "mlp.up"], s[p + "mlp.down"] = (l["ff"], D), (D, l["ff"])
        return s


DTYPES = {"bf16": 1, "bfloat16": 1, "f32": 2, "float32": 2}


class DekipelDecoder:
    """One model instance on the current CUDA device.  Slots (0..max_batch-1) each own `max_seq` cache rows per layer and
    the layers' convolution states; the caller (the engine's scheduler) decides which sequence lives in which slot."""

    architecture = "Dekipel"
    supports_dtypes = ("bfloat16", "float32")
    supports_ragged_steps = True

    def __init__(self, config, dtype="bf16", max_batch=1, max_seq=512, max_step_tokens=512, use_pdl=True, use_graph=True):
        self.lib = _lib.load()
        self.config = config
        self.vocab_size = config.vocab
        self.max_batch, self.max_seq = int(max_batch), int(max_seq)
        self.max_step_tokens = max(int(max_step_tokens), self.max_batch)
        self.cfg = DekipelCConfig(len(config.layers), config.width, config.vocab, config.norm_groups, config.canon_taps,
                                  config.norm_eps, DTYPES[dtype], self.max_batch, self.max_seq, self.max_step_tokens,
                                  int(use_pdl), int(use_graph))
        arr = (DekipelLayer * len(config.layers))()
        for i, l in enumerate(config.layers):
            arr[i] = DekipelLayer(l["heads"], l["dim"], l["vdim"], l["q_rank"], l["kv_rank"], l["kv_from"], l["ff"], l["scale"])
        h = ctypes.c_void_p()
        _lib.check(self.lib.zl_dekipel_create(ctypes.byref(self.cfg), arr, ctypes.byref(h)))
        self.h = h

    @classmethod
    def from_config_dict(cls, d, **kw):
        return cls(DekipelConfig.from_dict(d), **kw)

    def close(self):
        if getattr(self, "h", None):
            self.lib.zl_dekipel_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def load_state_dict(self, state_dict):
        """name -> numpy array: bfloat16 bit patterns (safetensors_io.Bf16Array) or float32."""
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
            _lib.check(self.lib.zl_dekipel_load_tensor(self.h, name.encode(), a.ctypes.data_as(ctypes.c_void_p), rows, cols,
                                                       a.itemsize))
        _lib.check(self.lib.zl_dekipel_finalize(self.h))

    def init_synthetic(self, seed=0):
        _lib.check(self.lib.zl_dekipel_init_synthetic(self.h, seed))

    def step(self, tokens, slots, positions, want_rows=(), want_logits=True):
        """One step over T rows.  Returns (next tokens (n_want), logits (n_want, vocab) or None) for the wanted rows."""
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        s = np.ascontiguousarray(slots, dtype=np.int32)
        p = np.ascontiguousarray(positions, dtype=np.int32)
        w = np.ascontiguousarray(want_rows, dtype=np.int32)
        nxt = np.empty(w.size, dtype=np.int32)
        logits = np.empty((w.size, self.vocab_size), dtype=np.float32) if want_logits else None
        _lib.check(self.lib.zl_dekipel_step(
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
        _lib.check(self.lib.zl_dekipel_set_state(self.h, t.ctypes.data_as(ctypes.c_void_p), p.ctypes.data_as(ctypes.c_void_p),
                                                 t.size))

    def step_device(self, b):
        _lib.check(self.lib.zl_dekipel_step_device(self.h, b))

    def sync(self):
        _lib.check(self.lib.zl_dekipel_sync(self.h))

    def stream(self):
        return self.lib.zl_dekipel_stream(self.h)

    def capture_layers(self, on=True):
        _lib.check(self.lib.zl_dekipel_capture_layers(self.h, int(on)))

    def read_layers(self, n_tokens):
        out = np.empty((len(self.config.layers), n_tokens, self.config.width), dtype=np.float32)
        _lib.check(self.lib.zl_dekipel_read_layers(self.h, out.ctypes.data_as(ctypes.c_void_p), n_tokens))
        return out

    def stats(self):
        wb, kn = ctypes.c_double(), ctypes.c_int()
        _lib.check(self.lib.zl_dekipel_stats(self.h, ctypes.byref(wb), ctypes.byref(kn)))
        return wb.value, kn.value
