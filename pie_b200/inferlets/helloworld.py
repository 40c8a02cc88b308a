"""helloworld: the smallest inferlet - no model call. Counterpart of inferlets/helloworld."""
from pie_b200.sdk import runtime

NAME = "helloworld"


async def main(args):
    runtime.print_out("Hello, world!")
    return f"Hello from instance {runtime.instance_id()} (runtime {runtime.version()})"
