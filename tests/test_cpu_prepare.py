"""Offline data-preparation stages on CPU: unify / repair / language filter, MinHash and sentence dedup, downloads with
an injected transport, tokenizer comparison, the loop-depth probe."""
import gzip
import os

import torch

from recurrent_pretraining_b200.data.prepare import compare_tokenizers as ct
from recurrent_pretraining_b200.data.prepare import dedup, download, loop_probe
from recurrent_pretraining_b200.data.prepare import unify_filter as uf


def test_unify_repair_and_language_filter(tmp_path):
    plain = uf.DataSource(address="x", features=["title", "body"])
    assert uf.unify_row({"title": "T", "body": "B", "other": 1}, plain) == {"text": "T\nB"}
    chat = uf.DataSource(address="x", features=["conversations"], needs_chat_templating=True)
    row = uf.unify_row({"conversations": [{"from": "human", "value": " hi "}, {"from": "gpt", "value": "hello"}]}, chat)
    assert row["text"] == ("<|begin_text|><|begin_header|>human<|end_header|>\n\nhi<|end_turn|>"
                           "<|begin_header|>Huginn<|end_header|>\n\nhello<|end_turn|>")
    pair = uf.DataSource(address="x", features=["q", "a"], needs_chat_templating=True)
    assert "<|begin_header|>user<|end_header|>\n\nQ" in uf.unify_row({"q": "Q", "a": "A"}, pair)["text"]
    # repair: UTF-8 read as Latin-1, a control character, decomposed accents
    broken = "cafÃ© dâ€™Ã©tÃ©\x07 é"
    assert uf.fix_text(broken) == "café d’été é"
    # language id on the listed languages and on English
    samples = {
        "en": "The quick brown fox jumps over the lazy dog and it was not happy that they were all there with him.",
        "de": "Der schnelle braune Fuchs springt über den faulen Hund und das ist nicht gut für die Tiere in dem Wald.",
        "fr": "Le renard brun rapide saute par-dessus le chien paresseux et il est dans la forêt avec les autres.",
        "es": "El rápido zorro marrón salta sobre el perro perezoso y no se va de la casa por la noche con los otros.",
        "ru": "Быстрая коричневая лиса перепрыгивает через ленивую собаку, и это не нравится никому в лесу.",
        "zh": "敏捷的棕色狐狸跳过了懒狗，然后跑进了森林里面，再也没有回来。",
        "ja": "素早い茶色の狐はのろまな犬を飛び越えて、森の中へ走っていきました。",
        "ko": "빠른 갈색 여우가 게으른 개를 뛰어넘어 숲속으로 달려갔습니다.",
        "ar": "الثعلب البني السريع يقفز فوق الكلب الكسول ويذهب إلى الغابة مع الآخرين.",
    }
    for lang, text in samples.items():
        got, score = uf.identify_language(text)
        assert got == lang, (lang, got, score)
        assert uf.language_filter({"text": text}) == (lang == "en"), lang
    assert uf.language_filter({"messages": [{"content": samples["de"]}]}) is False
    assert uf.language_filter({"text": "x = 3 + 4  # 12345 ()"}) is True        # code / numbers are kept
    # driver + sharded parquet output with resume
    rows = [{"title": "A", "body": samples["en"]}, {"title": "B", "body": samples["de"]}, {"title": "", "body": ""}]
    out = list(uf.process_source(rows, plain, filter_language=True, run_fix=True))
    assert len(out) == 1 and out[0]["text"].startswith("A\n")
    paths = uf.save_as_parquet(({"text": "x" * 100} for _ in range(10)), str(tmp_path), "src", target_shard_bytes=350)
    assert len(paths) == 3
    import pyarrow.parquet as pq

    assert sum(pq.read_table(p).num_rows for p in paths) == 10
    mtime = os.path.getmtime(paths[0])
    uf.save_as_parquet(({"text": "x" * 100} for _ in range(10)), str(tmp_path), "src", target_shard_bytes=350)
    assert os.path.getmtime(paths[0]) == mtime          # resume: existing shards are not rewritten
    # manifest
    (tmp_path / "sources.yaml").write_text("wiki:\n  address: org/wiki\n  features: [text]\n  weight: 2\n  extra: 1\n"
                                           "code:\n  address: org/code\n  requires_software_heritage_aws_download: true\n")
    src = uf.load_sources(str(tmp_path / "sources.yaml"))
    assert src["wiki"].weight == 2 and src["code"].requires_software_heritage_aws_download


def test_minhash_and_sentence_dedup(tmp_path):
    base = ("Recurrent depth models iterate a shared block of layers several times before decoding the next token. "
            "The number of iterations can be chosen at test time. This gives a knob for compute per token. ")
    docs = [base + "Appendix A lists the shapes.", base + "Appendix A lists the shapes!",      # near duplicates
            "A completely different document about parquet files and row groups and how they are shuffled on disk.",
            base.replace("Recurrent", "Looped") + "Appendix A lists the shapes.",              # still a near duplicate
            "Short."]
    hasher = dedup.MinHasher(num_buckets=20, hashes_per_bucket=4, n_grams=3)
    clusters = dedup.minhash_clusters(docs, hasher)
    assert clusters[0] == clusters[1] == clusters[3] and clusters[2] != clusters[0] and clusters[4] not in clusters[:4]
    assert dedup.minhash_dedup(docs, hasher) == [0, 2, 4]
    sig = hasher.signature(docs[0])
    assert sig.shape == (80,) and (hasher.signature(docs[0]) == sig).all()
    # estimated Jaccard tracks the true one
    a, b = dedup.shingles(docs[0], 3), dedup.shingles(docs[3], 3)
    true_j = len(a & b) / len(a | b)
    est = float((hasher.signature(docs[0]) == hasher.signature(docs[3])).mean())
    assert abs(true_j - est) < 0.25
    # sentence-level: the repeated three-sentence passage disappears from the second document only
    intro = "First unique sentence here. "
    d1 = intro + base
    d2 = "Another opening line. " + base + "And a unique ending."
    out = dedup.sentence_dedup([d1, d2], span=3)
    assert out[0] == d1.strip() and "iterate a shared block" not in out[1] and "unique ending" in out[1]
    # parquet driver
    import pyarrow as pa
    import pyarrow.parquet as pq

    f1, f2 = str(tmp_path / "a.parquet"), str(tmp_path / "b.parquet")
    pq.write_table(pa.table({"text": docs[:2]}), f1)
    pq.write_table(pa.table({"text": docs[2:]}), f2)
    rep = dedup.dedup_parquet([f1, f2], str(tmp_path / "out"), num_buckets=20, hashes_per_bucket=4, n_grams=3)
    assert rep == {"documents_in": 5, "documents_out": 3}
    assert pq.read_table(str(tmp_path / "out" / "a.parquet")).num_rows == 1


def test_download_with_injected_transport(tmp_path):
    blobs = {"b1": gzip.compress("print('hi')\n".encode()), "b2": "raw text é".encode("latin-1")}

    def fetch(blob_id):
        if blob_id not in blobs:
            raise KeyError(blob_id)
        return blobs[blob_id]

    rows = list(download.attach_blob_contents([{"blob_id": "b1"}, {"blob_id": "b2", "src_encoding": "latin-1"},
                                               {"blob_id": "missing"}], fetch, max_workers=2, batch=2))
    assert rows[0]["content"] == "print('hi')\n" and rows[1]["content"] == "raw text é"
    assert rows[2]["content"] == "" and "KeyError" in rows[2]["download_error"]
    sources = {"wiki": uf.DataSource(address="org/wiki", features=["text"]),
               "code": uf.DataSource(address="org/code", requires_software_heritage_aws_download=True)}
    data = {"org/wiki": [{"text": "alpha"}, {"text": "beta"}], "org/code": [{"blob_id": "b1"}]}
    calls = []

    def open_source(src):
        calls.append(src.address)
        return iter(data[src.address])

    done = download.download_sources(sources, str(tmp_path), open_source, fetch)
    import pyarrow.parquet as pq

    assert pq.read_table(done["wiki"][0]).column("text").to_pylist() == ["alpha", "beta"]
    assert pq.read_table(done["code"][0]).column("text").to_pylist() == ["print('hi')\n"]
    download.download_sources(sources, str(tmp_path), open_source, fetch)
    assert calls == ["org/wiki", "org/code"]            # second call: everything already on disk


class _CharTok:
    def encode(self, s):
        return [ord(c) for c in s]

    def decode(self, ids):
        return "".join(chr(i) for i in ids)


class _WordTok:
    def __init__(self):
        self.vocab, self.inv = {}, {}

    def encode(self, s):
        import re

        out = []
        for piece in re.findall(r"\s*\S+|\s+", s):
            if piece not in self.vocab:
                self.vocab[piece] = len(self.vocab)
                self.inv[self.vocab[piece]] = piece
            out.append(self.vocab[piece])
        return out

    def decode(self, ids):
        return "".join(self.inv[i] for i in ids)


def test_tokenizer_comparison_and_manual_tokens():
    from recurrent_pretraining_b200.data.prepare.tokenizer_train import manual_tokens

    text = "Compute 3.1415 * radius**2 with \\alpha = 10 and visit https://example.org for naïve cafés."
    res = ct.compare(text, [_CharTok(), _WordTok()], ["chars", "words"], color=False)
    assert res["stats"]["chars"]["tokens"] == len(text) and res["relative_tokens"]["words"] < 0.3
    assert res["stats"]["chars"]["chars_per_token"] == 1.0
    assert any(d["text"] == "3.1415" for d in res["differences"])
    assert "words" in ct.summarize(res)
    assert ct.strip_ansi(ct.render(_WordTok(), "a b", color=True)) == "a b"
    assert ct.validate_roundtrip(_CharTok(), ["ok", "é"]) == []
    assert ct.categorize_token(" 123") == "digits" and ct.categorize_token("=>") == "symbols"
    man = manual_tokens()
    assert len(man) == len(set(man)) and " " * 16 in man and "\n" * 3 in man and "Huginn" in man and "∑" in man


def test_loop_probe_learns_depth_on_a_tiny_model():
    from recurrent_pretraining_b200.config import ModelConfig
    from recurrent_pretraining_b200.models.hf import RavenForCausalLM
    from recurrent_pretraining_b200.models.hf_config import RavenConfig

    torch.manual_seed(0)
    cfg = ModelConfig.from_name("nebel-raven-3.5b", block_size=32, vocab_size=128, padding_multiple=64, n_embd=32,
                                num_attention_heads=2, num_key_value_heads=2, intermediate_size=48,
                                n_layers_in_recurrent_block=1, n_layers_in_prelude=1, n_layers_in_coda=1,
                                mean_recurrence=4, mean_backprop_depth=2)
    model = RavenForCausalLM(RavenConfig.from_model_config(cfg)).eval()
    ids = torch.randint(0, 100, (2, 16))
    lat = loop_probe.capture_latents(model, ids, 4)
    assert lat.shape == (4, 2, 16, 32)
    res = loop_probe.train_probe(model, [ids] * 40, 4, lr=3e-3)
    assert res["chance"] == 0.25 and res["accuracy"][-1] > res["accuracy"][0]
    pair = loop_probe.train_probe(model, [ids] * 5, 4, classes=torch.tensor([0, 3]))
    assert pair["chance"] == 0.5 and len(pair["accuracy"]) == 5


def test_category_report_sums_and_shares():
    from recurrent_pretraining_b200.data.prepare.count_tokens import category_report, format_category_report
    from recurrent_pretraining_b200.data.prepare.unify_filter import DataSource

    sources = {"web-a": DataSource("org/web-a", category="generic-web"), "web-b": DataSource("org/web-b", category="generic-web"),
               "code": DataSource("org/code", category="code"), "empty": DataSource("org/none", category="math")}
    rep = category_report(sources, {"web-a": (600, 800), "web-b": (200, 200), "code": (200, 250)})
    assert rep["total_kept"] == 1000
    assert rep["categories"]["generic-web"]["kept"] == 800 and rep["categories"]["generic-web"]["share_pct"] == 80.0
    assert rep["categories"]["generic-web"]["datasets"] == ["web-a", "web-b"]
    assert rep["datasets"]["web-a"]["dropped_pct"] == 25.0 and rep["datasets"]["empty"]["kept"] == 0
    text = format_category_report(rep)
    assert "generic-web" in text and "Total tokens" in text
