"""knowledge-graph: the model extracts (subject, relation, object) triples from a passage under a
JSON-schema constraint; the triples become a directed graph; a breadth-first walk from the entity
of the question collects the facts within `depth` hops; those facts are the context of the final
answer. The query context's prompt is prefilled while the graph is built on the CPU.
Counterpart of inferlets/knowledge-graph/src/lib.rs."""
import asyncio
import json
from collections import defaultdict, deque

from pie_b200.sdk import Context, JsonSchema

from ._common import load_model, make_sampler

NAME = "knowledge-graph"

TRIPLES = {"type": "object", "required": ["triples"], "properties": {"triples": {
    "type": "array", "minItems": 1, "maxItems": 4,
    "items": {"type": "array", "minItems": 3, "maxItems": 3, "items": {"type": "string", "maxLength": 12}}}}}


def bfs_facts(edges, start, depth):
    graph = defaultdict(list)
    for s, r, o in edges:
        graph[s].append((r, o))
        graph[o].append(("inverse " + r, s))
    seen, facts, q = {start}, [], deque([(start, 0)])
    while q:
        node, d = q.popleft()
        if d >= depth:
            continue
        for r, o in graph.get(node, []):
            facts.append(f"{node} {r} {o}")
            if o not in seen:
                seen.add(o)
                q.append((o, d + 1))
    return facts


async def main(args):
    args = args or {}
    model = load_model(args)
    passage = args.get("passage", "Ada wrote notes. Notes describe engines.")
    ex = Context(model)
    ex.user("Extract triples as JSON from: " + passage).cue()
    extract = ex.generate(make_sampler(args), max_tokens=int(args.get("extract_tokens", 96)), constrain=JsonSchema(TRIPLES))
    # overlap: the answer context's system prompt is prefilled while extraction decodes
    qa = Context(model)
    qa.system("Answer from the facts only.")
    raw, _ = await asyncio.gather(extract.collect_text(), qa.flush())
    ex.release()
    try:
        triples = [tuple(t) for t in json.loads(raw)["triples"] if len(t) == 3]
    except (ValueError, KeyError, TypeError):
        triples = []
    start = args.get("entity") or (triples[0][0] if triples else "")
    facts = bfs_facts(triples, start, int(args.get("depth", 2)))
    qa.user("Facts: " + "; ".join(facts) + ". Question: " + args.get("question", "What is known?")).cue()
    answer = await qa.generate(make_sampler(args), max_tokens=int(args.get("max_tokens", 12))).collect_text()
    qa.release()
    return json.dumps({"triples": [list(t) for t in triples], "facts": facts, "answer": answer})
