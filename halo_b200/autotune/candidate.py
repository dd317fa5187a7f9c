"""Kernel candidates as canonical text: `name=value` pairs joined by `;`, names [a-z0-9_]{1,32} in sorted order, values
signed 64-bit decimals, at most 4096 bytes, no duplicates (src/autotune/types.cpp:13-66).  The backend interface stores
the kernel as `variant=<id>` (docs/adr/ADR-001-backend-interface.md:457-459)."""
from __future__ import annotations

import re
from dataclasses import dataclass

_NAME = re.compile(r"^[a-z0-9_]{1,32}$")
_I64 = (-(1 << 63), (1 << 63) - 1)


@dataclass(frozen=True)
class Candidate:
    params: tuple[tuple[str, int], ...]

    @staticmethod
    def of(**kv: int) -> "Candidate":
        for k, v in kv.items():
            if not _NAME.match(k):
                raise ValueError(f"candidate: bad parameter name {k!r}")
            if not isinstance(v, int) or isinstance(v, bool) or not _I64[0] <= v <= _I64[1]:
                raise ValueError(f"candidate: {k} = {v!r} is not a signed 64-bit integer")
        c = Candidate(tuple(sorted(kv.items())))
        if len(c.to_string().encode()) > 4096:
            raise ValueError("candidate: text longer than 4096 bytes")
        return c

    @staticmethod
    def parse(text: str) -> "Candidate":
        if text == "":
            return Candidate(())
        if len(text.encode()) > 4096 or text.endswith(";"):
            raise ValueError(f"candidate: malformed text {text!r}")
        kv: dict[str, int] = {}
        for part in text.split(";"):
            name, sep, val = part.partition("=")
            if not sep or not _NAME.match(name) or name in kv or not re.match(r"^-?[0-9]+$", val):
                raise ValueError(f"candidate: malformed pair {part!r}")
            kv[name] = int(val)
        c = Candidate.of(**kv)
        if c.to_string() != text:
            raise ValueError(f"candidate: {text!r} is not in canonical (sorted) form")
        return c

    def to_string(self) -> str:
        return ";".join(f"{k}={v}" for k, v in self.params)

    def get(self, name: str, default: int | None = None) -> int | None:
        return dict(self.params).get(name, default)
