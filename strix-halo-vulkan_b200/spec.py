"""Speculative decoding with the MTP draft head: the host loop of the reference's
`Speculator.round` (llm/spec.go:703-852) over the C ABI.

A round drafts up to `depth` tokens with the one-layer draft head (seeded from the trunk's
residual and the next token's embedding, llm/mtp.go:352-384), verifies them in ONE trunk pass
that returns every row's logits, keeps the longest prefix the trunk agrees with
(`Graph.keep`, llm/graph.go:1189-1233) and owes the draft the trunk's true residual rows so its
KV cache catches up next round (llm/spec.go:837-844). Every emitted token is picked from the
trunk's own logits over a prefix that is the sequence, so the output equals plain decoding
whatever the draft proposes (llm/spec.go:54-60).
"""
import numpy as np

SPEC_DEPTH_DEFAULT = 2       # llm/spec.go:880
DRAFT_VOCAB_DEFAULT = 65536  # llm/spec.go:886


def argmax(logits):
    return int(np.argmax(logits))   # ties to the lowest id (llm/sample.go:359-367)


class Speculator:
    """One sequence's speculative loop. Several of them share a slotted graph, one per slot
    (NewSlotSpeculator, llm/spec.go; llm/spec_slots_test.go:199): each call first makes its slot the
    graph's and the draft cache's current one (Graph.UseSlot + MTPHead.UseSlot, llm/mtp.go:500-529), so
    rounds of different slots may be interleaved in any order."""

    def __init__(self, graph, depth=SPEC_DEPTH_DEFAULT, draft_vocab=0, slot=None):
        if depth < 1 or depth > 4:
            raise ValueError("depth is 1..4")
        self.g, self.depth, self.draft_vocab, self.slot = graph, depth, draft_vocab, slot
        self.h = None          # trunk residual of the last fed position
        self.pend = None       # the token emitted but not yet fed to the trunk
        self.owe_h, self.owe_x = [], []
        self.stats = dict(rounds=0, drafted=0, accepted=0, tokens=0)

    def _select(self):
        if self.slot is not None:
            self.g.use_slot(self.slot)        # moves the draft cache's slot along
            self.g.draft_use_slot(self.slot)

    def prime(self, ids, pick=argmax):
        """Prefill the trunk, prime the draft's cache with every (residual, next token) pair of
        the prompt (llm/spec.go:285-328) and return the first emitted token."""
        ids = np.asarray(ids, dtype=np.int32)
        g = self.g
        self._select()
        g.reset()
        res_rows, logits = [], None
        mt = g.max_tokens
        for o in range(0, len(ids), mt):
            logits, res = g.extend_residual(ids[o:o + mt])
            res_rows.append(res)
        res = np.concatenate(res_rows)
        g.draft_rewind(0)
        mt = min(mt, g.draft_max_rows())
        for o in range(0, len(ids) - 1, mt):
            n = min(mt, len(ids) - 1 - o)
            g.draft_rows(res[o:o + n], ids[o + 1:o + 1 + n], 16)   # cache only; logits are not needed
        self.h, self.pend = res[-1].copy(), pick(logits)
        self.owe_h, self.owe_x = [], []
        return self.pend

    def round(self, propose=None, pick=argmax, room=None):
        """One speculative round. Returns the tokens emitted (at least one). `propose(logits, k)`
        names draft k's token (default: the draft head's argmax); `pick(logits)` names the
        trunk's token of a row."""
        g = self.g
        self._select()
        at = g.past()
        depth = self.depth if room is None else max(1, min(self.depth, room - 1))
        if g.draft_past() != at - 1 - len(self.owe_x):
            raise RuntimeError(f"draft cache is at {g.draft_past()}, expected {at - 1 - len(self.owe_x)}")
        # 1. drafts: the owed rows and the first draft in one call, then each further draft from the
        #    draft's own residual
        rows = [self.pend]
        hs = np.stack(self.owe_h + [self.h])
        xs = self.owe_x + [self.pend]
        res, lg = g.draft_rows(hs, xs, self.draft_vocab)
        self.owe_h, self.owe_x = [], []
        res_last, lg_last = res[-1], lg[-1]
        for k in range(depth):
            d = int(propose(lg_last, k)) if propose is not None else argmax(lg_last)
            rows.append(d)
            if k + 1 < depth:
                res, lg = g.draft_rows(res_last[None, :], [d], self.draft_vocab)
                res_last, lg_last = res[0], lg[0]
        # 2. one verification pass over all rows
        g.speculate(True)
        logits, vres = g.extend_rows(rows)
        # 3. row i's pick is the trunk's token after rows[0..i]; stop at the first disagreement
        out = []
        for i in range(len(rows)):
            t = pick(logits[i])
            out.append(t)
            if i + 1 == len(rows) or rows[i + 1] != t:
                break
        keep = len(out)
        g.keep(keep)
        g.speculate(False)
        # 4. the draft's cache keeps the cell of the real pending token and is owed the rest
        g.draft_rewind(at)
        for i in range(1, keep):
            self.owe_h.append(vres[i - 1].copy())
            self.owe_x.append(rows[i])
        self.h, self.pend = vres[keep - 1].copy(), out[-1]
        self.stats["rounds"] += 1
        self.stats["drafted"] += len(rows) - 1
        self.stats["accepted"] += keep - 1
        self.stats["tokens"] += keep
        return out
