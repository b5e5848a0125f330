"""Side-by-side comparison of tokenizers on a text: compression (characters / bytes per token), what kinds of tokens each
uses, where the segmentations differ, and a coloured per-token rendering for the terminal.

Counterpart of scripts/compare_tokenizers.py (summary, token categories, distinctive examples, validation).  Works with
anything that has ``encode(str) -> ids`` and ``decode(ids) -> str`` (``tokenizers.Tokenizer``, HF tokenizers, the
framework's ``Tokenizer``)."""
from __future__ import annotations

import re
import unicodedata
from collections import Counter
from typing import Sequence

_ANSI = ["\033[48;5;153m", "\033[48;5;223m", "\033[48;5;194m", "\033[48;5;225m"]
_RESET = "\033[0m"
_INTERESTING = re.compile(r"\d[\d.,]*\d|\\[a-zA-Z]+|[A-Za-z_]+\(|https?://\S+|[^\x00-\x7f]+|\s{2,}|[=<>!+\-*/]{2,}")


def encode_ids(tok, text: str) -> list:
    out = tok.encode(text)
    if hasattr(out, "ids"):
        return list(out.ids)
    return out.tolist() if hasattr(out, "tolist") else list(out)


def pieces(tok, text: str) -> list:
    """The surface string of every token (decoded one id at a time)."""
    return [tok.decode([i]) for i in encode_ids(tok, text)]


def categorize_token(piece: str) -> str:
    s = piece.strip()
    if not s:
        return "whitespace"
    if s.isdigit():
        return "digits"
    if all(unicodedata.category(c).startswith("P") or unicodedata.category(c).startswith("S") for c in s):
        return "symbols"
    if all(ord(c) < 128 for c in s):
        return "ascii-word" if s.isalpha() else "ascii-mixed"
    return "non-ascii"


def analyze(tok, text: str) -> dict:
    ps = pieces(tok, text)
    n = max(len(ps), 1)
    cats = Counter(categorize_token(p) for p in ps)
    return {"tokens": len(ps), "chars_per_token": len(text) / n, "bytes_per_token": len(text.encode()) / n,
            "mean_piece_len": sum(len(p) for p in ps) / n, "categories": dict(cats),
            "longest": sorted(set(ps), key=len, reverse=True)[:5]}


def interesting_sequences(text: str, limit: int = 20) -> list:
    seen, out = set(), []
    for m in _INTERESTING.finditer(text):
        s = m.group(0)
        if s not in seen:
            seen.add(s)
            out.append(s)
        if len(out) == limit:
            break
    return out


def render(tok, text: str, color: bool = True) -> str:
    ps = pieces(tok, text)
    if not color:
        return "|".join(ps)
    return "".join(_ANSI[i % len(_ANSI)] + p + _RESET for i, p in enumerate(ps))


def strip_ansi(text: str) -> str:
    return re.sub(r"\033\[[0-9;]*m", "", text)


def compare(text: str, tokenizers: Sequence, labels: Sequence[str], num_sequences: int = 20, color: bool = False) -> dict:
    """Statistics per tokenizer, the relative token counts, and the sub-strings they segment differently."""
    stats = {lab: analyze(t, text) for t, lab in zip(tokenizers, labels)}
    base = stats[labels[0]]["tokens"]
    diffs = []
    for seq in interesting_sequences(text, num_sequences):
        segs = {lab: pieces(t, seq) for t, lab in zip(tokenizers, labels)}
        if len({tuple(v) for v in segs.values()}) > 1:
            diffs.append({"text": seq, **{lab: v for lab, v in segs.items()}})
    return {"stats": stats, "relative_tokens": {lab: stats[lab]["tokens"] / max(base, 1) for lab in labels},
            "differences": diffs,
            "rendered": {lab: render(t, text[:400], color) for t, lab in zip(tokenizers, labels)}}


def summarize(result: dict) -> str:
    lines = []
    for lab, st in result["stats"].items():
        lines.append(f"{lab:>16}: {st['tokens']:7d} tokens  {st['chars_per_token']:.2f} chars/token  "
                     f"x{result['relative_tokens'][lab]:.3f}  {st['categories']}")
    for d in result["differences"][:10]:
        lines.append(f"  {d['text']!r}: " + "  vs  ".join(f"{k}={v}" for k, v in d.items() if k != "text"))
    return "\n".join(lines)


def validate_roundtrip(tok, samples: Sequence[str]) -> list:
    """Samples that do not survive encode -> decode (a tokenizer that drops or alters characters)."""
    return [s for s in samples if tok.decode(encode_ids(tok, s)) != s]
