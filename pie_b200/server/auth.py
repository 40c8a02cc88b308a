"""Client authentication: public-key challenge-response against a per-user key list, or the
engine's internal token (printed at start-up; wrong tokens are answered after a delay).

Handshake: `auth_identify(username)` -> base64 challenge -> `auth_prove(signature)` verified
against the user's registered OpenSSH public keys (ed25519, rsa, ecdsa). Counterpart of
runtime/src/auth.rs, auth/keys.rs, auth/users.rs and the handshake in runtime/src/server.rs:481-595.
"""
from __future__ import annotations

import base64
import json
import os
import secrets
from pathlib import Path
from typing import Dict, List, Optional

from cryptography.exceptions import InvalidSignature
from cryptography.hazmat.primitives import hashes, serialization
from cryptography.hazmat.primitives.asymmetric import ec, ed25519, padding, rsa


class AuthError(Exception):
    pass


class UserStore:
    """username -> list of OpenSSH public key lines, kept in one JSON file."""

    def __init__(self, path: str):
        self.path = Path(path).expanduser()
        self.users: Dict[str, List[str]] = {}
        if self.path.exists():
            self.users = json.loads(self.path.read_text() or "{}")

    def save(self) -> None:
        self.path.parent.mkdir(parents=True, exist_ok=True)
        self.path.write_text(json.dumps(self.users, indent=1))

    def add(self, username: str, pubkey_line: str) -> None:
        load_public_key(pubkey_line)    # validates
        self.users.setdefault(username, [])
        if pubkey_line not in self.users[username]:
            self.users[username].append(pubkey_line.strip())
        self.save()

    def remove(self, username: str) -> bool:
        ok = self.users.pop(username, None) is not None
        self.save()
        return ok

    def keys(self, username: str) -> List[str]:
        return list(self.users.get(username, []))


def load_public_key(line: str):
    return serialization.load_ssh_public_key(line.strip().encode())


def verify(pubkey_line: str, message: bytes, signature: bytes) -> bool:
    key = load_public_key(pubkey_line)
    try:
        if isinstance(key, ed25519.Ed25519PublicKey):
            key.verify(signature, message)
        elif isinstance(key, rsa.RSAPublicKey):
            key.verify(signature, message, padding.PKCS1v15(), hashes.SHA256())
        elif isinstance(key, ec.EllipticCurvePublicKey):
            key.verify(signature, message, ec.ECDSA(hashes.SHA256()))
        else:
            return False
        return True
    except InvalidSignature:
        return False


def sign(private_key, message: bytes) -> bytes:
    """Client side: sign a challenge with a loaded private key."""
    if isinstance(private_key, ed25519.Ed25519PrivateKey):
        return private_key.sign(message)
    if isinstance(private_key, rsa.RSAPrivateKey):
        return private_key.sign(message, padding.PKCS1v15(), hashes.SHA256())
    if isinstance(private_key, ec.EllipticCurvePrivateKey):
        return private_key.sign(message, ec.ECDSA(hashes.SHA256()))
    raise AuthError("unsupported key type")


def load_private_key(path: str, password: Optional[bytes] = None):
    data = Path(path).expanduser().read_bytes()
    try:
        return serialization.load_ssh_private_key(data, password)
    except ValueError:
        return serialization.load_pem_private_key(data, password)


def generate_ed25519():
    """(private key object, OpenSSH public key line) - used by tests and `pie auth keygen`."""
    k = ed25519.Ed25519PrivateKey.generate()
    pub = k.public_key().public_bytes(serialization.Encoding.OpenSSH, serialization.PublicFormat.OpenSSH).decode()
    return k, pub


class Authenticator:
    def __init__(self, enabled: bool, users: Optional[UserStore] = None):
        self.enabled = enabled
        self.users = users
        self.internal_token = secrets.token_urlsafe(24)

    def new_challenge(self) -> bytes:
        return os.urandom(32)

    def check_token(self, token: str) -> bool:
        return secrets.compare_digest(token, self.internal_token)

    def check_signature(self, username: str, challenge: bytes, signature_b64: str) -> bool:
        if self.users is None:
            return False
        try:
            sig = base64.b64decode(signature_b64)
        except Exception:  # noqa: BLE001
            return False
        return any(verify(k, challenge, sig) for k in self.users.keys(username))
