"""Keyword blocklist for prompts: exact, whitespace-normalised and light-stemmed matching against word lists
(``<dir>/exact_match/*``, ``<dir>/custom/*``, whitelist in ``<dir>/whitelist/*``; one term per line). Parity target:
the ``Blocklist`` guardrail of the reference (cosmos_predict2/_src/imaginaire/auxiliary/guardrail/blocklist). A small
built-in list is used when no directory is configured. No NLTK dependency: tokens are lower-cased,
punctuation-stripped and plural / -ing / -ed suffixes removed."""

from __future__ import annotations

import os
import re
import string
from typing import Iterable, List, Optional, Set, Tuple

from .core import ContentSafetyGuardrail

_BUILTIN = ["child pornography", "csam", "bestiality", "how to make a bomb", "nerve agent synthesis", "snuff film"]
CENSOR = "*"


def _stem(w: str) -> str:
    for suf in ("ingly", "edly", "ing", "ies", "ed", "es", "s"):
        if len(w) > len(suf) + 2 and w.endswith(suf):
            return w[: -len(suf)] + ("y" if suf == "ies" else "")
    return w


def _tokens(text: str) -> List[str]:
    text = text.lower().translate(str.maketrans({c: " " for c in string.punctuation}))
    return [t for t in re.split(r"\s+", text) if t]


class Blocklist(ContentSafetyGuardrail):
    def __init__(self, checkpoint_dir: Optional[str] = None, guardrail_partial_match_min_chars: int = 6,
                 guardrail_partial_match_letter_count: float = 0.4, terms: Optional[Iterable[str]] = None):
        self.min_chars = guardrail_partial_match_min_chars
        self.letter_frac = guardrail_partial_match_letter_count
        block: List[str] = list(terms) if terms is not None else []
        white: List[str] = []
        if checkpoint_dir and os.path.isdir(checkpoint_dir):
            for sub, dst in (("exact_match", block), ("custom", block), ("whitelist", white)):
                d = os.path.join(checkpoint_dir, sub)
                if os.path.isdir(d):
                    for f in sorted(os.listdir(d)):
                        with open(os.path.join(d, f), errors="ignore") as fh:
                            dst += [ln.strip() for ln in fh if ln.strip() and not ln.startswith("#")]
        if not block:
            block = list(_BUILTIN)
        self.whitelist: Set[str] = {" ".join(_stem(t) for t in _tokens(w)) for w in white}
        self.phrases: List[Tuple[str, ...]] = sorted({tuple(_stem(t) for t in _tokens(p)) for p in block if _tokens(p)})

    def censor_prompt(self, prompt: str) -> Tuple[bool, str]:
        toks = [_stem(t) for t in _tokens(prompt)]
        hits = []
        for ph in self.phrases:
            n = len(ph)
            for i in range(len(toks) - n + 1):
                if tuple(toks[i:i + n]) == ph and " ".join(ph) not in self.whitelist:
                    hits.append(" ".join(ph))
                    break
        if hits:
            return True, f"prompt blocked by the word blocklist ({len(hits)} term(s))"
        return False, ""

    def is_safe(self, prompt: str) -> Tuple[bool, str]:
        blocked, msg = self.censor_prompt(prompt or "")
        return (not blocked), msg
