"""Raw sources -> one ``text`` column: source manifest, row unification (several text features, chat transcripts rendered
with the chat template), text repair, language filter, parquet shards of a target size.

Counterpart of the middle stages of scripts/data_processing_pipeline.py (``DataSource`` manifest :155-188, unifying
formatter :286-324, language filter :329-391, ftfy :393-395, ``save_as_parquet`` :241-266).  The reference relies on
datatrove's fastText language model and on ftfy; neither can be fetched here, so both steps take a plug-in
(``lid=`` / ``fixer=``) and ship self-contained defaults: Unicode-script shares plus stop-word hits for the same list
of thirty non-English languages, and NFC normalisation with the most frequent UTF-8-as-Latin-1 repairs."""
from __future__ import annotations

import os
import re
import unicodedata
from dataclasses import dataclass, field
from typing import Callable, Iterable, Iterator, Optional

ROLE_KEYS = ("role", "from", "speaker", "author")
CONTENT_KEYS = ("content", "value", "text", "message")
ASSISTANT_NAMES = {"assistant", "gpt", "bot", "model", "chatgpt", "bard", "ai"}


@dataclass
class DataSource:
    """One entry of the source manifest (YAML mapping of name -> these fields)."""
    address: str
    features: list = field(default_factory=lambda: ["text"])
    subset: Optional[str] = None
    needs_chat_templating: bool = False
    weight: float = 1.0
    category: str = "generic-text"
    every_token_is_sacred: bool = False
    license: str = "unknown"
    citation: str = ""
    requires_software_heritage_aws_download: bool = False


def load_sources(path: str) -> dict:
    import yaml

    with open(path) as f:
        raw = yaml.safe_load(f) or {}
    known = set(DataSource.__dataclass_fields__)
    return {name: DataSource(**{k: v for k, v in (spec or {}).items() if k in known}) for name, spec in raw.items()}


def default_chat_template(messages: list, bos: str = "<|begin_text|>") -> str:
    """``<|begin_header|>role<|end_header|>\\n\\ncontent<|end_turn|>`` per message, bos before the first."""
    out = []
    for i, m in enumerate(messages):
        turn = f"<|begin_header|>{m['role']}<|end_header|>\n\n{str(m['content']).strip()}<|end_turn|>"
        out.append((bos if i == 0 else "") + turn)
    return "".join(out)


def unify_row(example: dict, source: DataSource, chat_template: Callable[[list], str] = default_chat_template,
              assistant_name: str = "Huginn") -> dict:
    """Map one raw row to ``{"text": ...}``.  Several features are joined by newlines (or become alternating user /
    assistant turns); a single chat feature is a list of messages whose role / content keys vary by dataset; every
    assistant-like role is renamed to ``assistant_name``."""
    feats = source.features
    if source.needs_chat_templating:
        if len(feats) > 1:
            msgs = [{"role": "user" if i == 0 else "assistant", "content": str(example[f])}
                    for i, f in enumerate(feats) if f in example]
        else:
            msgs = [{"role": next((m[k] for k in ROLE_KEYS if k in m), None),
                     "content": next((m[k] for k in CONTENT_KEYS if k in m), None)} for m in example[feats[0]]]
        for m in msgs:
            if str(m["role"]).lower() in ASSISTANT_NAMES:
                m["role"] = assistant_name
        return {"text": chat_template(msgs)}
    if len(feats) > 1:
        return {"text": "\n".join(str(example[f]) for f in feats if f in example)}
    return {"text": str(example[feats[0]]) if feats[0] in example else ""}


# ------------------------------------------------------------------------------------------------------ text repair
_CP1252_EXTRA = "€‚ƒ„…†‡ˆ‰Š‹ŒŽ‘’“”•–—˜™š›œžŸ"
_MOJIBAKE_RUN = re.compile("[\u0080-\u00ff" + _CP1252_EXTRA + "]{2,}")


def _repair_run(m: "re.Match") -> str:
    run = m.group(0)
    for enc in ("cp1252", "latin-1"):
        try:
            fixed = run.encode(enc).decode("utf-8")
        except (UnicodeEncodeError, UnicodeDecodeError):
            continue
        if len(fixed) < len(run):
            return fixed
    return run


def fix_text(text: str) -> str:
    """Undo UTF-8 that was read as Latin-1 / cp1252 (run by run, only where the round trip is lossless and shortens the
    run), drop control characters other than newline and tab, normalise to NFC."""
    text = _MOJIBAKE_RUN.sub(_repair_run, text)
    text = "".join(ch for ch in text if ch in "\n\t" or unicodedata.category(ch) != "Cc")
    return unicodedata.normalize("NFC", text)


# ------------------------------------------------------------------------------------------------------ language id
TARGET_LANGUAGES = ["zh", "es", "ar", "pt", "id", "fr", "ja", "ru", "de", "ko", "tr", "it", "pl", "nl", "hi", "fa", "vi",
                    "th", "sv", "he", "cs", "ro", "el", "da", "fi", "no", "hu", "bn", "uk", "ms"]
_SCRIPTS = {"zh": ("CJK",), "ja": ("HIRAGANA", "KATAKANA"), "ko": ("HANGUL",), "ar": ("ARABIC",), "ru": ("CYRILLIC",),
            "hi": ("DEVANAGARI",), "th": ("THAI",), "he": ("HEBREW",), "el": ("GREEK",), "bn": ("BENGALI",)}
_STOP = {
    "es": "el la de que y en los se del las por un para con no una su al lo como más pero sus le ya o este sí porque",
    "pt": "o a de que e do da em um para é com não uma os no se na por mais as dos como mas foi ao ele das tem à seu",
    "fr": "le la de et les des en un du une que est pour qui dans a par plus pas au sur ne se ce il sont avec ou",
    "de": "der die und in den von zu das mit sich des auf für ist im dem nicht ein eine als auch es an werden aus",
    "it": "il di che e la per un in è non una sono con si da come le dei ma più anche del alla nel lo gli della",
    "nl": "de van het een en in is dat op te zijn voor met die niet aan er om ook als dan maar bij nog uit",
    "pl": "w i na z do się nie że to jest o jak po co tak za od przez ale czy tego już dla są był tym oraz",
    "tr": "ve bir bu da de için ile olarak çok daha gibi en ancak kadar her ne o ama ya sonra olan var ise",
    "id": "yang dan di itu dengan untuk tidak ini dari dalam akan pada juga saya ke karena tersebut bisa ada mereka",
    "ms": "yang dan di itu dengan untuk tidak ini dari dalam akan pada juga saya ke kerana tersebut boleh ada mereka",
    "vi": "và của là có trong được cho không một người này với các đã những để khi đó về như cũng từ",
    "sv": "och i att det som en på är av för med till den har de inte om ett han men var jag sig från så",
    "cs": "a se na je v že to s z do o i ve jako za by pro ale po tak jsem byl jeho které si však",
    "ro": "de și în a la cu că pe care un o este din se nu pentru mai ce să sunt au ca lui fost prin",
    "da": "og i at det er en til af på for med som den de der har ikke et han var jeg sig men fra om",
    "fi": "ja on ei että oli se hän mutta kun niin kuin tai myös ovat joka sen vain jos olla tämä hänen",
    "no": "og i er det som på en til av for med at har de ikke den et om var fra men seg han jeg så",
    "hu": "a az és hogy nem is egy de meg ez volt van el már csak mint még azt vagy ha ki be fel",
    "fa": "و در به از که این را با است برای آن یک خود تا کرد بر هم نیز شد", "uk": "і в на з що не до як це та за але від його",
}
_STOP_SETS = {k: set(v.split()) for k, v in _STOP.items()}
_ENGLISH = set("the of and to in a is that for it as was with be by on not he this are or his from at which but have "
               "an had they you were their one all we can her has there been if more when will would who so no".split())
_WORD = re.compile(r"[^\W\d_]+", re.UNICODE)


def script_of(ch: str) -> str:
    try:
        return unicodedata.name(ch).split(" ")[0]
    except ValueError:
        return ""


def identify_language(text: str, sample: int = 4000) -> tuple[str, float]:
    """(language code, confidence in [0, 1]) by script share, then by stop-word share among Latin / Cyrillic / Arabic
    script languages.  "en" when English stop words dominate or nothing else scores."""
    text = text[:sample]
    letters = [ch for ch in text if ch.isalpha()]
    if not letters:
        return "en", 0.0
    counts: dict = {}
    for ch in letters:
        s = script_of(ch)
        counts[s] = counts.get(s, 0) + 1
    n = len(letters)
    best, share = "en", 0.0
    for lang, names in _SCRIPTS.items():
        sh = sum(counts.get(nm, 0) for nm in names) / n
        if lang == "ja" and sh > 0.05:
            sh += counts.get("CJK", 0) / n           # kana present: the Han characters are Japanese too
        if sh > share:
            best, share = lang, sh
    words = [w.lower() for w in _WORD.findall(text)]
    if share >= 0.5:
        if best in ("ru", "ar") and words:           # Cyrillic: ru vs uk; Arabic script: ar vs fa
            alt = "uk" if best == "ru" else "fa"
            hit = sum(w in _STOP_SETS[alt] for w in words) / len(words)
            if hit > 0.08 and (alt == "fa" or any(ch in "іїєґ" for ch in text.lower())):
                return alt, share
        return best, share
    if not words:
        return "en", 0.0
    en = sum(w in _ENGLISH for w in words) / len(words)
    top, top_score = "en", en
    for lang, stop in _STOP_SETS.items():
        if lang in ("fa", "uk"):
            continue
        sc = sum(w in stop for w in words) / len(words)
        if sc > top_score:
            top, top_score = lang, sc
    if top == "en":
        return "en", min(1.0, en * 3)
    return top, min(1.0, top_score * 3 * (1.0 if top_score > 1.5 * en else 0.5))


def language_filter(example: dict, non_english_threshold: float = 0.5,
                    lid: Callable[[str], tuple] = identify_language) -> bool:
    """False (drop the row) when the text is confidently one of the thirty listed non-English languages."""
    if example.get("text") is not None:
        text = example["text"]
    elif example.get("messages"):
        text = "\n".join(m["content"] for m in example["messages"] if m.get("content") is not None)
    else:
        text = " "
    lang, score = lid(text)
    return not (lang in TARGET_LANGUAGES and score > non_english_threshold)


# ------------------------------------------------------------------------------------------------------ driver
def process_source(rows: Iterable[dict], source: DataSource, *, filter_language: bool = False, run_fix: bool = False,
                   lid=identify_language, fixer=fix_text, chat_template=default_chat_template) -> Iterator[dict]:
    for ex in rows:
        row = unify_row(ex, source, chat_template)
        if not row["text"].strip():
            continue
        if run_fix:
            row["text"] = fixer(row["text"])
        if filter_language and not language_filter(row, lid=lid):
            continue
        yield row


def save_as_parquet(rows: Iterable[dict], out_dir: str, name: str, target_shard_bytes: int = 2 * 1024 ** 3,
                    resume: bool = True) -> list:
    """Write ``{name}_{i:05d}.parquet`` shards of about ``target_shard_bytes`` of text each; an existing shard is kept
    when ``resume`` (only new files are written).  Returns the shard paths."""
    import pyarrow as pa
    import pyarrow.parquet as pq

    os.makedirs(out_dir, exist_ok=True)
    paths, buf, size, idx = [], [], 0, 0

    def flush():
        nonlocal buf, size, idx
        if not buf:
            return
        path = os.path.join(out_dir, f"{name}_{idx:05d}.parquet")
        if not (resume and os.path.exists(path)):
            tmp = path + ".tmp"
            pq.write_table(pa.table({"text": buf}), tmp)
            os.replace(tmp, path)
        paths.append(path)
        buf, size, idx = [], 0, idx + 1

    for row in rows:
        buf.append(row["text"])
        size += len(row["text"].encode("utf-8", "ignore"))
        if size >= target_shard_bytes:
            flush()
    flush()
    return paths
