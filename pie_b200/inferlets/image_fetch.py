"""image-fetch: fetch a URL over HTTP (subject to the engine's network allowlist) and report what
came back. Counterpart of inferlets/image-fetch/src/lib.rs (wasi:http outgoing request)."""
import hashlib
import json

from pie_b200.sdk import io

NAME = "image-fetch"


async def main(args):
    url = (args or {}).get("url", "http://127.0.0.1:8080/")
    try:
        r = await io.http_fetch(url, timeout=float((args or {}).get("timeout", 10)))
    except PermissionError as e:
        return json.dumps({"ok": False, "denied": str(e)})
    return json.dumps({"ok": True, "status": r.status, "bytes": len(r.body),
                       "sha256": hashlib.sha256(r.body).hexdigest(),
                       "content_type": r.headers.get("Content-Type", "")})
