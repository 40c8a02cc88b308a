"""launch-callee: child side of the launch demo - echoes its input in upper case.
Counterpart of inferlets/launch-callee/src/lib.rs."""
NAME = "launch-callee"


async def main(args):
    return str((args or {}).get("text", "")).upper()
