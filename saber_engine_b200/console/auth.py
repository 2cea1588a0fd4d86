"""Credentials of the console and its proxy: named keys stored as salted hashes and checked in
constant time, revocation, and a per-address lockout after repeated failures.

Parity: `crates/saber-console/src/auth.rs` (salted hashes, constant-time check, `Limiter`),
`src/proxy.rs:17-22` (a key's label rides the usage row; a revoked key is refused; wrong keys count
toward the address's lockout).
"""
from __future__ import annotations

import hashlib
import hmac
import secrets
import time
from dataclasses import dataclass, field
from typing import Optional


def hash_key(secret: str, salt: str) -> str:
    return hashlib.sha256((salt + ":" + secret).encode()).hexdigest()


@dataclass
class KeyRecord:
    label: str
    salt: str
    digest: str
    revoked: bool = False


@dataclass
class KeyRing:
    keys: list = field(default_factory=list)

    def issue(self, label: str) -> str:
        """New key for `label`; the secret is returned ONCE and only its salted hash is kept."""
        if any(k.label == label and not k.revoked for k in self.keys):
            raise ValueError(f"a live key named {label!r} exists")
        secret, salt = "sk-" + secrets.token_urlsafe(24), secrets.token_hex(8)
        self.keys.append(KeyRecord(label, salt, hash_key(secret, salt)))
        return secret

    def revoke(self, label: str) -> bool:
        hit = False
        for k in self.keys:
            if k.label == label and not k.revoked:
                k.revoked, hit = True, True
        return hit

    def check(self, secret: str) -> Optional[str]:
        """Label of the live key `secret` is, else None.  Every record is hashed and compared (no
        early exit), so the time does not tell which key came close."""
        found = None
        for k in self.keys:
            ok = hmac.compare_digest(hash_key(secret, k.salt), k.digest)
            if ok and not k.revoked:
                found = k.label
        return found

    def to_json(self) -> list:
        return [vars(k) for k in self.keys]

    @staticmethod
    def from_json(items: list) -> "KeyRing":
        return KeyRing([KeyRecord(**i) for i in items])


class Limiter:
    """Failed-auth lockout per client address: `max_fails` failures inside `window_s` lock the
    address out for `lock_s`."""

    def __init__(self, max_fails: int = 8, window_s: float = 60.0, lock_s: float = 300.0, clock=time.monotonic):
        self.max_fails, self.window_s, self.lock_s, self.clock = max_fails, window_s, lock_s, clock
        self._fails: dict = {}
        self._locked: dict = {}

    def locked(self, addr: str) -> bool:
        until = self._locked.get(addr)
        if until is None:
            return False
        if self.clock() >= until:
            del self._locked[addr]
            return False
        return True

    def fail(self, addr: str) -> None:
        now = self.clock()
        f = [t for t in self._fails.get(addr, []) if now - t < self.window_s] + [now]
        self._fails[addr] = f
        if len(f) >= self.max_fails:
            self._locked[addr] = now + self.lock_s
            self._fails[addr] = []

    def ok(self, addr: str) -> None:
        self._fails.pop(addr, None)
