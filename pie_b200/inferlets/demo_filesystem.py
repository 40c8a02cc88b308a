"""demo-filesystem: write, list and read back files in the process's private scratch directory;
a path that escapes it is refused. Counterpart of inferlets/demo-filesystem/src/lib.rs."""
import json

from pie_b200.sdk import io

NAME = "demo-filesystem"


async def main(args):
    args = args or {}
    io.write_text("notes/hello.txt", args.get("text", "hello from an inferlet"))
    io.write_bytes("blob.bin", bytes(range(16)))
    escaped = False
    try:
        io.scratch_path("../outside.txt")
        escaped = True
    except PermissionError:
        pass
    return json.dumps({"files": io.listdir(), "text": io.read_text("notes/hello.txt"),
                       "blob_len": len(io.read_bytes("blob.bin")), "escape_refused": not escaped})
