"""A small FileCheck: enough of the directive language to run the CHECK lines of LLVM-lit style
test files (CHECK, CHECK-SAME, CHECK-LABEL, CHECK-NEXT, CHECK-NOT, CHECK-COUNT-<n>, {{regex}} blocks) against text."""
from __future__ import annotations

import re
from typing import List, Tuple

_DIRECTIVE = re.compile(r"//\s*(CHECK(?:-[A-Z]+)*(?:-\d+)?):\s?(.*)$")


def directives(source: str, prefix: str = "CHECK") -> List[Tuple[str, str]]:
    out = []
    for line in source.splitlines():
        m = _DIRECTIVE.search(line)
        if not m:
            continue
        kind, pat = m.group(1), m.group(2).strip()
        rest = kind[len(prefix) + 1:] if kind.startswith(prefix + "-") else None
        if kind == prefix or rest in ("SAME", "LABEL", "NEXT", "NOT"):
            out.append((kind[len(prefix):].lstrip("-") or "PLAIN", pat))
        elif rest is not None and re.fullmatch(r"COUNT-\d+", rest):
            out.extend([("PLAIN", pat)] * int(rest.split("-")[1]))     # n matches one after the other
    return out


def _to_regex(pat: str) -> "re.Pattern[str]":
    parts, pos = [], 0
    for m in re.finditer(r"\{\{(.*?)\}\}", pat):
        parts.append(re.escape(pat[pos:m.start()]))
        parts.append("(?:" + m.group(1) + ")")
        pos = m.end()
    parts.append(re.escape(pat[pos:]))
    # runs of blanks match any run of blanks, as in FileCheck
    return re.compile(re.sub(r"(\\ )+", r"\\s+", "".join(parts)))


def check(text: str, checks: List[Tuple[str, str]]) -> Tuple[bool, str]:
    """Returns (ok, message).  Matching is sequential: every directive searches after the previous match."""
    lines = text.splitlines()
    li, col = 0, 0                      # current position: line index, column
    pending_not: List[str] = []
    for kind, pat in checks:
        rx = _to_regex(pat)
        if kind == "NOT":
            pending_not.append(pat)
            continue
        found = None
        if kind == "SAME":
            if li < len(lines):
                m = rx.search(lines[li], col)
                if m:
                    found = (li, m.end())
        elif kind == "NEXT":
            if li + 1 < len(lines):
                m = rx.search(lines[li + 1])
                if m:
                    found = (li + 1, m.end())
        else:
            for k in range(li, len(lines)):
                m = rx.search(lines[k], col if k == li else 0)
                if m:
                    found = (k, m.end())
                    break
        if not found:
            return False, f"CHECK-{kind}: '{pat}' not found after line {li + 1}"
        for npat in pending_not:
            nrx = _to_regex(npat)
            for k in range(li, found[0] + 1):
                if nrx.search(lines[k]):
                    return False, f"CHECK-NOT: '{npat}' found on line {k + 1}"
        pending_not = []
        li, col = found
    for npat in pending_not:
        nrx = _to_regex(npat)
        for k in range(li, len(lines)):
            if nrx.search(lines[k]):
                return False, f"CHECK-NOT: '{npat}' found on line {k + 1}"
    return True, "ok"
