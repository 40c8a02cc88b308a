"""json-schema-validation: generate JSON constrained to a schema, parse it, check required keys.
Counterpart of inferlets/json-schema-validation/src/lib.rs."""
import json

from pie_b200.sdk import JsonSchema

from ._common import load_model, make_sampler, prompt_context

NAME = "json-schema-validation"

DEFAULT_SCHEMA = {"type": "object",
                  "properties": {"name": {"type": "string", "maxLength": 24}, "age": {"type": "integer"},
                                 "member": {"type": "boolean"}},
                  "required": ["name", "age", "member"]}


async def main(args):
    args = args or {}
    model = load_model(args)
    schema = args.get("schema", DEFAULT_SCHEMA)
    ctx = prompt_context(model, args, "Describe a person as JSON.")
    gen = ctx.generate(make_sampler(args), max_tokens=int(args.get("max_tokens", 512)))
    doc = await gen.collect_json(schema=schema)
    ctx.release()
    missing = [k for k in (schema.get("required") or []) if k not in doc]
    return json.dumps({"value": doc, "valid": not missing, "missing": missing})
