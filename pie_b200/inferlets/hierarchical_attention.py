"""hierarchical-attention: a long document is read in segments; after each segment the inferlet
appends a few summary tokens that attend to that segment, and from then on tokens see only the
summaries of older segments plus the current segment (per-token attention masks). The runtime's
page trim drops the pages no mask row can see. Counterpart of inferlets/hierarchical-attention-rust
(-python, -js)."""
import json

from ._common import load_model, make_sampler

NAME = "hierarchical-attention"


def rows_for(start, n, visible):
    """BRLE mask rows for n tokens at positions start..: each sees the `visible` ranges and itself
    causally within its own segment. `visible` is a sorted list of (lo, hi) position ranges."""
    rows = []
    for i in range(n):
        pos, cur, runs = start + i, 0, []
        spans = visible + [(start, pos + 1)]
        for lo, hi in spans:
            runs += [lo - cur, hi - lo]
            cur = hi
        rows.append(runs)
    return rows


async def main(args):
    args = args or {}
    model = load_model(args)
    tok = model.tokenizer()
    doc = args.get("document_tokens") or tok.encode(args.get("document", "lorem ipsum dolor sit amet " * 24))
    seg, nsum, max_tokens = int(args.get("segment", 32)), int(args.get("summary_tokens", 2)), int(args.get("max_tokens", 8))
    from pie_b200.sdk import Context
    ctx = Context(model)
    sampler = make_sampler(args)
    visible, pos, summaries = [], 0, 0
    for s0 in range(0, len(doc), seg):
        chunk = doc[s0:s0 + seg]
        fwd = ctx.forward().input_at(chunk, list(range(pos, pos + len(chunk))))
        fwd.attention_mask(rows_for(pos, len(chunk), visible))
        await fwd.execute()
        seg_span = (pos, pos + len(chunk))
        pos += len(chunk)
        # summary slots: sampled continuation tokens that see the segment; later tokens see only them
        feed = chunk[-1:]
        sum_lo = pos
        for _ in range(nsum):
            fwd = ctx.forward().input_at(feed, [pos])
            fwd.attention_mask(rows_for(pos, 1, visible + [seg_span] + ([(sum_lo, pos)] if pos > sum_lo else [])))
            h = fwd.sample([0], sampler)
            feed = [(await fwd.execute()).token(h)]
            pos += 1
        visible.append((sum_lo, pos))
        summaries += nsum
    tokens, feed = [], doc[-1:]
    q_lo = pos
    while len(tokens) < max_tokens:
        fwd = ctx.forward().input_at(feed, [pos])
        fwd.attention_mask(rows_for(pos, 1, visible + ([(q_lo, pos)] if pos > q_lo else [])))
        h = fwd.sample([0], sampler)
        t = (await fwd.execute()).token(h)
        tokens.append(t)
        feed, pos = [t], pos + 1
    ctx.release()
    return json.dumps({"tokens": tokens, "segments": -(-len(doc) // seg), "summary_tokens": summaries,
                       "visible_positions": sum(hi - lo for lo, hi in visible)})
