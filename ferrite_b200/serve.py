"""The sampling head of a batch of logits on the device: what the reference's server reads back instead of whole rows
(models/serve.py:31-47, pinned by test/test_sim.py:2141-2156), and the slot engine that drives the decode path for
several requests at once (models/serve.py:247-330: admit, fill, advance, take): requests take free slots of one shared
KV cache, a slot that still holds a prefix of the new prompt keeps it, prompts go in chunk by chunk, and one recorded
step decodes a token of every slot.  The HTTP server, the tokenizer, kept sessions, speculative decoding and the text
shapes of the reference's serving product are host code outside the decode path and are not here."""
import math

import numpy as np

from .tensor import Tensor


def parts_of(cols, most=4096):
    """The fewest equal parts of a row of `cols` logits that are at most `most` wide (1 when nothing divides it)."""
    for p in range(1, cols // 64 + 1):
        if cols % p == 0 and cols // p <= most:
            return p
    return 1


def heads(logits, t=None, k=64):
    """Each row's head of fp32 logits [rows, vocabulary]: its k largest, largest first, the lower column first among
    equals, and their columns (values, ids); and, given t (a column of each row's 1/temperature, fp32), the log of the
    sum of exp(x t) over the whole row in fp32 (lse).  Two rounds of top-k - the best of each part of the row, then the
    best of those by their labels - so no round looks at more than a few thousand values per row and pick; the sum
    is taken part by part as well (short fp32 sums, then a sum of the parts') about the row's maximum, which the head
    already holds."""
    assert logits.dtype == "fp32" and logits.batch == 1 and k <= 64, "fp32 logits, one matrix, k of at most 64"
    parts = parts_of(logits.cols) if logits.cols >= 2 * 4096 else 1
    if parts > 1:
        best, cols = logits.topk(min(k, logits.cols // parts), parts)
        values, ids = best.topk(k, labels=cols)
    else:
        values, ids = logits.topk(k)
    values, ids = values.realize(), ids.realize()
    if t is None:
        return values, ids
    top = values[:, :, :1]  # the row's maximum
    sums = ((logits.split(parts) - top) * t).exp().sum(2)  # [parts, rows, 1]
    lse = (sums.sum(0).log() + top * t).realize()
    return values, ids, lse


class Request:
    """A prompt's tokens and how to go on from them: max_tokens new tokens or until one in eos; temperature 0 is greedy,
    else a draw at that temperature among the top_k (at most 64, 0: the whole head) most likely, from the row's head alone
    (models/serve.py:49-67, 100-126, the part of Request.sample the head decides).  made: the tokens so far; cached: how
    many of the prompt's tokens its slot already held."""

    def __init__(self, ids, max_tokens=16, temperature=0.0, top_k=0, eos=(), seed=None):
        assert len(ids) >= 1 and 0 <= top_k <= 64, "a prompt of at least one token; top_k within the head of 64"
        self.ids, self.max_tokens, self.temperature, self.top_k, self.eos = list(ids), max_tokens, temperature, top_k, set(eos)
        self.rng, self.made, self.cached, self.finish = np.random.default_rng(seed), [], 0, None

    def sample(self, values, ids, lse):
        """The next token from a row's head: its largest logits, their tokens, and the row's log-sum-exp at 1/temperature."""
        if self.temperature == 0:
            return int(ids[0])
        t = 1 / self.temperature
        p = np.exp((np.float64(values) - np.float64(values[0])) * t)  # in the largest's scale
        if self.top_k:
            run = np.cumsum(p[:self.top_k])
            return int(ids[min(int(np.searchsorted(run, self.rng.random() * run[-1], side="right")), self.top_k - 1)])
        total = math.exp(float(lse) - float(values[0]) * t)  # the whole row's mass; a draw past the head's takes the head's last
        run = np.cumsum(p)
        return int(ids[min(int(np.searchsorted(run, self.rng.random() * total, side="right")), len(ids) - 1)])

    def take(self, token, room):
        """token is its next one; True once it is finished (an end of sequence, max_tokens, or no room left in its slot)."""
        if token in self.eos:
            self.finish = "stop"
        else:
            self.made.append(token)
            if len(self.made) >= self.max_tokens or not room:
                self.finish = "length"
        return self.finish is not None


def reach(held, ids):
    """How much of the prompt ids a slot that holds the keys of the tokens `held` already has: their common run, less one
    so that the prompt's last token always runs (its logits give the first new token) (models/serve.py:238-240)."""
    n = 0
    while n < min(len(held), len(ids)) and held[n] == ids[n]:
        n += 1
    return min(n, len(ids) - 1)


class Engine:
    """Several requests decoding together in the slots of one KV cache (models/serve.py:247-330).  The device work sits
    behind `backend`: prefill(u, ids, first, t) runs a chunk of slot u's prompt at places first.. and gives the head of
    its last token's logits; decode(ids, places, ts) runs one token of every slot and gives every slot's head.  A free
    slot's token is 0 at its part's last place, which marks it not live (models/llama.py:448-449).

        admit(r)   into the free slot that already holds the most of r's prompt (a slot keeps its last request's keys:
                   a shared system prompt is prefilled once), ties to the one used longest ago;
        fill(u)    the next chunk of slot u's prompt; the last chunk's head gives the request's first token;
        advance()  one decode step of every slot whose request is past its prompt;
        run(rs)    the three in turn until every request is finished."""

    def __init__(self, backend, slots, places, chunk=64):
        self.backend, self.slots, self.places, self.chunk = backend, slots, places, chunk
        self.busy, self.held, self.used = [None] * slots, [[] for _ in range(slots)], [0] * slots
        self.prefilled = self.decoded = 0

    def admit(self, r):
        free = [u for u, b in enumerate(self.busy) if b is None]
        assert free and len(r.ids) < self.places, "a free slot, and a prompt shorter than a slot's places"
        u = max(free, key=lambda u: (reach(self.held[u], r.ids), -self.used[u]))
        self.used[u], self.busy[u] = max(self.used) + 1, r
        n = reach(self.held[u], r.ids)
        self.held[u], r.cached = r.ids[:n], n
        return u

    def fill(self, u):
        r, at = self.busy[u], len(self.held[u])
        ids = r.ids[at:at + self.chunk]
        head = self.backend.prefill(u, ids, at, 1 / r.temperature if r.temperature else 1.0)
        self.held[u] = self.held[u] + ids
        self.prefilled += len(ids)
        if len(self.held[u]) == len(r.ids):
            self.take(u, head)

    def take(self, u, head):
        r = self.busy[u]
        if r.take(r.sample(*head), len(self.held[u]) + 1 < self.places - 1):
            self.busy[u] = None  # (its keys stay in the slot for a request that shares its prompt)

    def advance(self):
        live = [r if r is not None and r.made and len(self.held[u]) >= len(r.ids) else None for u, r in enumerate(self.busy)]
        if not any(r is not None for r in live):
            return False
        ids = [r.made[-1] if r else 0 for r in live]
        places = [len(h) if r else self.places - 1 for h, r in zip(self.held, live)]
        heads_ = self.backend.decode(ids, places, [1 / r.temperature if r and r.temperature else 1.0 for r in live])
        self.decoded += sum(r is not None for r in live)
        for u, r in enumerate(live):
            if r is not None:
                self.held[u].append(r.made[-1])
                self.take(u, heads_[u])
        return True

    def run(self, requests):
        waiting = list(requests)
        while waiting or any(b is not None for b in self.busy):
            while waiting and None in self.busy:
                self.admit(waiting.pop(0))
            for u, r in enumerate(self.busy):
                if r is not None and len(self.held[u]) < len(r.ids):
                    self.fill(u)
            self.advance()
        return requests


class DeviceBackend:
    """The engine's device side: the slots' shared KV cache, a prompt's chunk through forward over the slot's own rows
    (the prefill-shaped attention), and one recorded step for a token of every slot, each followed by `heads` so that
    only 64 values, 64 tokens and a log-sum-exp per row are read back."""

    def __init__(self, rt, weights, c, slots, places):
        from . import llama
        from .tensor import jit
        self.rt, self.w, self.c, self.slots, self.llama = rt, weights, c, slots, llama
        self.part = places
        self.kv = llama.kv_cache(c, slots * places, llama.zeros(rt))
        self.parts = [llama.slot(c, self.kv, u, slots) for u in range(slots)]

        def step(ids, at, t):
            logits = llama.forward(ids, at, weights, c, self.kv, slots).realize()
            return self._pack(heads(logits[0], t))
        self.step = jit(step)

    def _pack(self, h):
        """values | ids | lse side by side in one fp32 matrix (token ids below 2^24 are exact in fp32): one readback."""
        values, ids, lse = h
        return values.cat(ids.float(), lse, axis=2).realize()

    def _unpack(self, packed):
        a = packed.numpy()[0]
        return [(row[:64], row[64:128].astype(np.int64), row[128]) for row in a]

    def on(self, row, dtype="int32"):
        return Tensor.of(self.rt, [row], dtype)

    def prefill(self, u, ids, first, t):
        out = self.llama.forward(self.on(ids), self.on(list(range(first, first + len(ids)))), self.w, self.c, self.parts[u])
        return self._unpack(self._pack(heads(out, Tensor.of(self.rt, [[t]], "fp32"))))[0]

    def decode(self, ids, places, ts):
        return self._unpack(self.step(self.on(ids), self.on(places), Tensor.of(self.rt, [[t] for t in ts], "fp32")))
