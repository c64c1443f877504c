"""Serving engine: slot allocation, the step function and a continuous-batching scheduler with sampling.

The reference keeps these in src/generator (batch_generator.cpp: task queue, dynamic batch, chunked prompts,
beam / random sampling); here the engine is model-agnostic host code over a registered decoder's `step` call:

  * `SlotPool`      which sequence owns which cache slot; a finished sequence gives its slot (cache rows, states) back;
  * `Engine.forward_step(entries)`  THE step function: runs the rows the caller brings -- prompt portions and single
    decode tokens in one batch -- against the caches and states earlier steps left, cutting portions that exceed the
    decoder's step size; everything that generates or replays goes through it;
  * `Engine.generate(...)`  the scheduler: admits waiting requests while slots are free, feeds prompts in portions of at
    most `max_step_tokens` rows next to the running requests' decode tokens, samples, retires.
"""
import collections

import numpy as np


class SlotPool:
    def __init__(self, n):
        self.free = list(range(n))
        self.owner = {}

    def alloc(self, owner):
        if not self.free:
            return None
        s = min(self.free)
        self.free.remove(s)
        self.owner[s] = owner
        return s

    def release(self, slot):
        if slot in self.owner:
            del self.owner[slot]
            self.free.append(slot)


class SamplingParams:
    """temperature 0 = greedy (the device-side argmax); otherwise softmax(logits / temperature) restricted to the
    top_k largest and the smallest set whose mass reaches top_p, drawn with a per-request generator."""

    def __init__(self, temperature=0.0, top_k=0, top_p=1.0, seed=0):
        self.temperature, self.top_k, self.top_p, self.seed = float(temperature), int(top_k), float(top_p), int(seed)

    @property
    def greedy(self):
        return self.temperature <= 0.0


def sample_token(logits, params, rng):
    z = np.asarray(logits, dtype=np.float64) / params.temperature
    order = np.argsort(-z, kind="stable")
    if params.top_k > 0:
        order = order[:params.top_k]
    p = np.exp(z[order] - z[order[0]])
    p /= p.sum()
    if params.top_p < 1.0:
        keep = int(np.searchsorted(np.cumsum(p), params.top_p, side="left")) + 1
        order, p = order[:keep], p[:keep] / p[:keep].sum()
    return int(order[rng.choice(len(order), p=p)])


class Sequence:
    def __init__(self, rid, slot, prompt=(), max_new_tokens=0, sampling=None, eos=None):
        self.id, self.slot = rid, slot
        self.tokens = list(prompt)     # prompt + generated
        self.n_prompt = len(self.tokens)
        self.pos = 0                   # rows already in the cache
        self.max_new_tokens, self.eos = max_new_tokens, eos
        self.sampling = sampling or SamplingParams()
        self.rng = np.random.default_rng(self.sampling.seed)
        self.output = []
        self.done = False


class Engine:
    def __init__(self, model):
        self.model = model
        self.slots = SlotPool(model.max_batch)
        self.seqs = {}

    # ---- sequences ---------------------------------------------------------------------------------------------------
    def open(self, rid, **kw):
        """Give request `rid` a slot; None when all slots are taken."""
        if rid in self.seqs:
            return self.seqs[rid]
        slot = self.slots.alloc(rid)
        if slot is None:
            return None
        self.seqs[rid] = Sequence(rid, slot, **kw)
        return self.seqs[rid]

    def close(self, rid):
        seq = self.seqs.pop(rid, None)
        if seq is not None:
            self.slots.release(seq.slot)

    # ---- the step function -------------------------------------------------------------------------------------------
    def forward_step(self, entries, want_logits=True):
        """entries: [(rid, tokens, want)] -- request rid's next tokens and the offsets among them whose output is wanted.
        Returns {rid: (next_tokens (len(want)), logits (len(want), vocab) or None)}.  Rows are packed into model steps
        of at most max_step_tokens rows, a request's rows consecutive and in order."""
        cap = self.model.max_step_tokens
        out = {rid: ([], []) for rid, _, _ in entries}
        work = collections.deque()
        for rid, tokens, want in entries:
            seq = self.seqs[rid]
            if seq.pos + len(tokens) > self.model.max_seq:
                raise ValueError("request %r exceeds max_seq" % (rid,))
            work.append((seq, list(tokens), sorted(set(int(w) for w in want)), 0))
        while work:
            toks, slots, poss, rows, owners, used = [], [], [], [], [], set()
            later = collections.deque()
            while work:
                seq, tokens, want, done = work.popleft()
                room = cap - len(toks)
                if room <= 0 or seq.slot in used:
                    later.append((seq, tokens, want, done))
                    continue
                used.add(seq.slot)
                n = min(room, len(tokens) - done)
                base = len(toks)
                toks += tokens[done:done + n]
                slots += [seq.slot] * n
                poss += list(range(seq.pos, seq.pos + n))
                for w in want:
                    if done <= w < done + n:
                        rows.append(base + w - done)
                        owners.append(seq.id)
                seq.pos += n
                if done + n < len(tokens):
                    later.append((seq, tokens, want, done + n))
            work = later
            nxt, logits = self.model.step(toks, slots, poss, rows, want_logits)
            for i, rid in enumerate(owners):
                out[rid][0].append(int(nxt[i]))
                if want_logits:
                    out[rid][1].append(logits[i])
        return {rid: (np.array(n, dtype=np.int32), (np.stack(l) if l else np.zeros((0, self.model.vocab_size), np.float32))
                      if want_logits else None) for rid, (n, l) in out.items()}

    # ---- the scheduler -----------------------------------------------------------------------------------------------
    def generate(self, prompts, max_new_tokens=16, sampling=None, eos=None, on_step=None):
        """prompts: list of token-id lists.  Returns the generated ids per prompt.  Continuous batching: every step takes
        one decode token of every running request plus prompt portions of the admitted ones, up to max_step_tokens rows."""
        cap = self.model.max_step_tokens
        waiting = collections.deque(enumerate(prompts))
        results = [None] * len(prompts)
        running = []
        for i, p in enumerate(prompts):
            if len(p) == 0 or len(p) + max_new_tokens > self.model.max_seq:
                raise ValueError("prompt %d is empty or does not fit max_seq" % i)
        while waiting or running:
            while waiting:
                i, p = waiting[0]
                sp = sampling[i] if isinstance(sampling, (list, tuple)) else sampling
                seq = self.open(("gen", i), prompt=p, max_new_tokens=max_new_tokens, sampling=sp, eos=eos)
                if seq is None:
                    break
                waiting.popleft()
                running.append(seq)
            entries, budget = [], cap
            for seq in running:                       # decode rows first: a running request is never starved by prompts
                if seq.pos >= seq.n_prompt and budget > 0:
                    entries.append((seq.id, [seq.tokens[-1]], [0]))
                    budget -= 1
            for seq in running:
                if seq.pos < seq.n_prompt and budget > 0:
                    n = min(budget, seq.n_prompt - seq.pos)
                    last = seq.pos + n == seq.n_prompt
                    entries.append((seq.id, seq.tokens[seq.pos:seq.pos + n], [n - 1] if last else []))
                    budget -= n
            need_logits = any(not self.seqs[rid].sampling.greedy for rid, _, w in entries if w)
            res = self.forward_step(entries, want_logits=need_logits)
            if on_step:
                on_step(entries)
            for rid, _, want in entries:
                if not want:
                    continue
                seq = self.seqs[rid]
                nxt, logits = res[rid]
                tok = int(nxt[0]) if seq.sampling.greedy else sample_token(logits[0], seq.sampling, seq.rng)
                seq.tokens.append(tok)
                seq.output.append(tok)
                if len(seq.output) >= seq.max_new_tokens or (seq.eos is not None and tok == seq.eos):
                    seq.done = True
            for seq in [s for s in running if s.done]:
                results[seq.id[1]] = seq.output
                running.remove(seq)
                self.close(seq.id)
        return results
