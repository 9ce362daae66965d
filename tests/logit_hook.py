"""Records the logits of every sampled row that an engine computes, so that a test can
compare them (not the tokens drawn from them, which a near-tie may flip in bfloat16) with
the plain implementation once the sequences are known."""

import numpy as np


class LogitRecorder:
    """Wraps ``runner.run``.  Every wanted row is kept with its request and the position of
    the token it belongs to; rows of a step that replays a graph are copied out of the
    graph's fixed output buffer at once, on the launching stream."""

    def __init__(self, runner):
        self.rows = []          # (request id, position, kept logits tensor, row in it)
        self.steps = []         # (rows of the step, whether all its entries were single tokens)
        inner = runner.run

        def run(entries):
            logits = inner(entries)
            kept = logits.clone()
            i = 0
            for e in entries:
                for w in e.want:
                    self.rows.append((e.request_id, e.start + int(w), kept, i))
                    i += 1
            self.steps.append((len(entries), all(len(e.tokens) == 1 for e in entries)))
            return logits

        runner.run = run

    def compare(self, sequences, plain_logits, limit, what=""):
        """``sequences``: request id -> its whole token sequence (prompt and output);
        ``plain_logits(request id)`` -> [len, vocab] of the plain implementation on that
        sequence.  Every recorded row whose position lies inside the sequence must agree
        within ``limit`` of the sequence's largest logit.  Returns (rows compared, worst)."""
        refs, worst, n = {}, 0.0, 0
        for rid, pos, kept, i in self.rows:
            seq = sequences.get(rid)
            if seq is None or pos >= len(seq):
                continue        # a row computed for a request that had already ended
            if rid not in refs:
                refs[rid] = plain_logits(rid)
            ref = refs[rid]
            got = kept[i].float().cpu().numpy().astype(np.float64)
            err = np.abs(got - ref[pos]).max() / np.abs(ref).max()
            assert err < limit, f"{what}: request {rid}, position {pos}: relative error {err:.3e} (limit {limit:.0e})"
            worst = max(worst, err)
            n += 1
        return n, worst
