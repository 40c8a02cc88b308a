"""mcts: Monte-Carlo tree search over continuations. Nodes are contexts forked from their parent
(they share its pages); selection is UCT, expansion samples `branching` short continuations, the
value of a leaf is the model's mean log-probability of its own tokens, and values are backed up to
the root. Counterpart of inferlets/mcts-rust (and mcts-python / mcts-js)."""
import json
import math

from pie_b200.sdk import Logprobs

from ._common import load_model, make_sampler, prefill_shared, prompt_context

NAME = "mcts"


class Node:
    def __init__(self, ctx, last, parent=None, tokens=()):
        self.ctx, self.last, self.parent, self.tokens = ctx, last, parent, list(tokens)
        self.children, self.visits, self.value = [], 0, 0.0

    def uct(self, c):
        if self.visits == 0:
            return float("inf")
        return self.value / self.visits + c * math.sqrt(math.log(self.parent.visits + 1) / self.visits)


async def rollout_value(node, step_tokens, args, seed):
    """Sample a continuation from the node and score it by its teacher-forced mean log-probability."""
    ctx = node.ctx.fork().append(node.last)
    toks = await ctx.generate(make_sampler(dict(args, temperature=args.get("temperature", 1.0), seed=seed)),
                              max_tokens=step_tokens).stop([]).collect_tokens()
    ctx.release()
    sc = node.ctx.fork()
    seq = list(node.last) + toks
    fwd = sc.forward().input(seq)
    hs = [fwd.probe(j, Logprobs([seq[j + 1]])) for j in range(len(seq) - 1)]
    out = await fwd.execute()
    sc.release()
    return toks, sum(out.logprobs(h)[0] for h in hs) / max(1, len(hs))


async def main(args):
    args = args or {}
    model = load_model(args)
    iters, branching = int(args.get("iterations", 6)), int(args.get("branching", 2))
    step_tokens, c = int(args.get("step_tokens", 4)), float(args.get("exploration", 1.0))
    root_ctx = prompt_context(model, args, "Think.")
    root = Node(root_ctx, await prefill_shared(root_ctx))
    seed, nodes = int(args.get("seed", 1)), 1
    for _ in range(iters):
        node = root
        while node.children:                               # selection
            node = max(node.children, key=lambda n: n.uct(c))
        for _b in range(branching):                        # expansion + evaluation
            seed += 1
            toks, value = await rollout_value(node, step_tokens, args, seed)
            child_ctx = node.ctx.fork().append(node.last + toks[:-1])
            await child_ctx.flush()
            child = Node(child_ctx, toks[-1:], node, node.tokens + toks)
            node.children.append(child)
            nodes += 1
            n = child
            while n is not None:                           # back-propagation
                n.visits += 1
                n.value += value
                n = n.parent
    best = root
    while best.children:
        best = max(best.children, key=lambda n: n.visits)
    out = {"tokens": best.tokens, "nodes": nodes, "root_visits": root.visits,
           "best_mean_value": best.value / max(1, best.visits)}

    def free(n):
        for ch in n.children:
            free(ch)
        n.ctx.release()
    free(root)
    return json.dumps(out)
