"""Drafting by copying from the request's own context (prompt lookup): the drafter of the reference's batched
speculative step that needs no second model (spec/lookup.py; used in scheduler.py:448-456 before the DFlash2 drafter).

The request's tokens (prompt, then everything emitted, the newest last) are indexed by bigram. A proposal is what
followed the longest earlier occurrence of the current suffix: among the most recent occurrences of the last two tokens
(at most CANDIDATES of them) the one whose match extends furthest backwards (up to MAX_MATCH tokens) wins, and up to
MAX_DRAFT of the tokens that followed it are proposed. Whether a proposal is worth a verify pass is decided from
running means of how many drafted tokens were accepted, kept per match-length bucket (the reference's priors), against
what a step costs without it: here there is no neural drafter to compete with (DFlash2 needs its checkpoint), so the
bar is a fixed expected gain.
"""
from __future__ import annotations

MAX_DRAFT, CANDIDATES, MAX_MATCH = 7, 24, 64
BUCKETS = (2, 3, 4, 6, 10, 16)            # match lengths that open a new bucket
PRIORS = (0.6, 1.0, 1.8, 2.6, 3.6, 4.6)   # accepted drafts expected per bucket before anything was observed
PRIOR_WEIGHT, MIN_RATE = 4.0, 0.03


class RunningMean:
    """A mean that starts from a prior worth `weight` observations and never averages over more than 1 / MIN_RATE."""

    def __init__(self, value, weight):
        self.value, self.n = float(value), float(weight)

    def add(self, x):
        self.n += 1.0
        self.value += max(1.0 / self.n, MIN_RATE) * (x - self.value)


def bucket_of(match_len: int) -> int:
    b = 0
    for i, lo in enumerate(BUCKETS):
        if match_len >= lo:
            b = i
    return b


class Lookup:
    def __init__(self, min_gain: float = 0.5):
        """min_gain: propose only when the bucket's running mean of accepted drafts is at least this."""
        self.min_gain = min_gain
        self.means = [RunningMean(p, PRIOR_WEIGHT) for p in PRIORS]
        self.proposed = self.steps = self.accepted = 0
        self.reset([])

    def reset(self, ids):
        self.hist = [int(t) for t in ids]
        self.index = {}          # (token, next token) -> positions of the second token, ascending
        self.indexed = 0
        self.pending = None

    def _index_upto(self, end):
        h = self.hist
        while self.indexed < end:
            p = self.indexed
            if p >= 1:
                self.index.setdefault((h[p - 1], h[p]), []).append(p)
            self.indexed += 1

    def find(self, max_draft=MAX_DRAFT):
        """(continuation, match length) of the best earlier occurrence of the current suffix, or None."""
        h, n = self.hist, len(self.hist)
        if n < 3:
            return None
        self._index_upto(n - 1)                      # (never the current position itself)
        where = self.index.get((h[n - 2], h[n - 1]))
        if not where:
            return None
        best_len, best_pos = 0, -1
        for p in reversed(where[-CANDIDATES:]):      # the most recent occurrences first
            if p + 1 >= n:
                continue
            m = 2
            while m < MAX_MATCH and m <= p and h[p - m] == h[n - 1 - m]:
                m += 1
            if m > best_len:
                best_len, best_pos = m, p
        if best_pos < 0:
            return None
        cont = h[best_pos + 1: min(best_pos + 1 + max_draft, n)]
        return (cont, best_len) if cont else None

    def propose(self, max_draft=MAX_DRAFT):
        """Up to max_draft drafted tokens for this step, or [] when copying is not expected to pay."""
        self.steps += 1
        self.pending = None
        f = self.find(max_draft)
        if f is None:
            return []
        cont, m = f
        b = bucket_of(m)
        if min(self.means[b].value, len(cont)) < self.min_gain:
            return []
        self.pending = b
        self.proposed += 1
        return list(cont)

    def record(self, emitted):
        """The step's outcome: the tokens it emitted (accepted drafts, then the model's own next token)."""
        acc = max(0, len(emitted) - 1)
        if self.pending is not None:
            self.means[self.pending].add(acc)
            self.accepted += acc
        self.pending = None
        self.hist.extend(int(t) for t in emitted)
