"""Data path, settings loader, schedules, goldfish masking."""
import os
import random

import pytest
import torch

from recurrent_pretraining_b200.data import (DataScheduler, DataSchedulerTracker, ParquetStream, RandomTokens,
                                             StatefulLoader, apply_tld, generic_collate_fn)
from recurrent_pretraining_b200.data.goldfish import hashint
from recurrent_pretraining_b200.optim.schedules import get_batch_size, get_lr
from recurrent_pretraining_b200.settings import DataEntry, GoldfishConfig, parse_cli

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _write_shards(tmp_path, n_files=3, groups=2, rows=5, width=9):
    import pyarrow as pa
    import pyarrow.parquet as pq

    counter = 0
    for f in range(n_files):
        tables = []
        for _ in range(groups):
            data = [[counter * 100 + j for j in range(width)] for counter in range(counter, counter + rows)]
            counter += rows
            tables.append(pa.table({"input_ids": data}))
        with pq.ParquetWriter(str(tmp_path / f"shard_{f:03d}.parquet"), tables[0].schema) as w:
            for t in tables:
                w.write_table(t)
    return n_files * groups * rows


def test_parquet_stream_covers_everything_once_and_resumes(tmp_path):
    total = _write_shards(tmp_path)
    ds = ParquetStream(str(tmp_path), seed=1, plan_for_later_rank_expansion_to=0)
    rows = [tuple(r.tolist()) for r in ds]
    assert len(rows) == total and len(set(rows)) == total
    # resume in the middle of a row group: the continuation equals the uninterrupted stream
    ds1 = ParquetStream(str(tmp_path), seed=1, plan_for_later_rank_expansion_to=0)
    it = iter(ds1)
    head = [tuple(next(it).tolist()) for _ in range(7)]
    state = ds1.state_dict()
    ds2 = ParquetStream(str(tmp_path), seed=1, plan_for_later_rank_expansion_to=0)
    ds2.load_state_dict(state)
    tail = [tuple(r.tolist()) for r in ds2]
    assert head + tail == rows
    # rank sharding is disjoint
    a = ParquetStream(str(tmp_path), seed=1, num_processes=3, process_rank=0, plan_for_later_rank_expansion_to=0)
    b = ParquetStream(str(tmp_path), seed=1, num_processes=3, process_rank=1, plan_for_later_rank_expansion_to=0)
    assert not set(a.parquet_files) & set(b.parquet_files)
    # fingerprint mismatch restarts from the beginning instead of indexing out of bounds
    bad = dict(state, fingerprint=["deadbeef"])
    ds3 = ParquetStream(str(tmp_path), seed=1, plan_for_later_rank_expansion_to=0)
    ds3.load_state_dict(bad)
    assert ds3._file_idx == 0


def test_collate_shift_and_padding_rules():
    class Tok:
        pad_id, eos_id = 9, 7

    rows = [torch.arange(10), torch.tensor([1, 2, 9, 9, 9, 9, 9, 9, 9, 9])]
    x, y, meta = generic_collate_fn(rows, tokenizer=Tok(), all_block_size_tensors=True)
    assert x.shape == (2, 9) and y.shape == (2, 9) and x.dtype == torch.int64
    assert torch.equal(y[0], torch.arange(1, 10))
    assert x[1].tolist() == [1, 2, 7, 7, 7, 7, 7, 7, 7]  # pad -> eos in inputs only
    assert y[1].tolist() == [2, 9, 9, 9, 9, 9, 9, 9, 9]
    x2, y2, _ = generic_collate_fn([torch.arange(5), torch.arange(3)], tokenizer=Tok(), block_size=8)
    assert x2.shape == (2, 4) and x2[1].tolist() == [0, 1, 2, 7]
    with pytest.raises(StopIteration):
        generic_collate_fn([torch.full((4,), 9)], tokenizer=Tok(), block_size=8)


def test_stateful_loader_batches_and_random_tokens():
    ds = RandomTokens(100, 17, seed=3)
    loader = StatefulLoader(ds, 4, lambda rows: generic_collate_fn(rows, all_block_size_tensors=True), prefetch=2)
    it = iter(loader)
    x, y, _ = next(it)
    assert x.shape == (4, 16) and int(x.max()) < 100 and torch.equal(x[:, 1:], y[:, :-1])
    again = RandomTokens(100, 17, seed=3)
    assert torch.equal(next(iter(again)), torch.cat([x[0, :1], y[0]]))


@pytest.mark.parametrize("kind", ["random", "parquet"])
def test_loader_resume_with_prefetch_is_exact(tmp_path, kind):
    """Stop after k batches while the producer thread is several batches ahead, save, reload into a fresh loader: the
    continuation equals the uninterrupted stream (nothing skipped, nothing repeated)."""
    import time

    if kind == "parquet":
        _write_shards(tmp_path, n_files=3, groups=3, rows=7)

    def make():
        ds = RandomTokens(100, 9, seed=5, length=60) if kind == "random" else \
            ParquetStream(str(tmp_path), seed=2, plan_for_later_rank_expansion_to=0)
        return StatefulLoader(ds, 2, lambda rows: generic_collate_fn(rows, all_block_size_tensors=True), prefetch=4)

    full = [x.clone() for x, _, _ in make()]
    assert len(full) >= 12
    for k in (1, 5, 8):
        loader = make()
        it = iter(loader)
        head = [next(it)[0].clone() for _ in range(k)]
        time.sleep(0.3)                      # let the producer fill its queue: it is now 4-5 batches ahead
        state = loader.state_dict()
        resumed = make()
        resumed.load_state_dict(state)
        tail = [x.clone() for x, _, _ in resumed]
        got = head + tail
        assert len(got) == len(full), (k, len(got), len(full))
        assert all(torch.equal(a, b) for a, b in zip(got, full)), k
        it.close()
    # the same loader object can also go on after its iterator was closed early
    loader = make()
    it = iter(loader)
    head = [next(it)[0].clone() for _ in range(3)]
    time.sleep(0.2)
    it.close()
    rest = [x.clone() for x, _, _ in loader]
    assert all(torch.equal(a, b) for a, b in zip(head + rest, full)) and len(head + rest) == len(full)


def test_goldfish_masks():
    labels = torch.randint(1, 1000, (2, 64))
    out, idx = apply_tld(labels, GoldfishConfig(4, 1, 13, "static"))
    assert (out[:, 1::4] == -100).all() and (out[:, 0] == labels[:, 0]).all()
    for strat in ("hash-table", "hash-avalanche"):
        a, da = apply_tld(labels, GoldfishConfig(4, 0, 5, strat))
        b, _ = apply_tld(labels, GoldfishConfig(4, 0, 5, strat))
        assert torch.equal(a, b)  # deterministic function of the context
        assert (a[:, :4] == labels[:, :4]).all()  # the first context_width-1 labels are never dropped
        assert 0 < int((a == -100).sum()) < labels.numel() // 2
    # the hash is a bijection on 32 bits: distinct keys stay distinct
    keys = torch.arange(0, 5000, dtype=torch.int64)
    assert hashint(keys).unique().numel() == 5000


def test_data_scheduler_weights():
    entries = [DataEntry("rngds", "a", weight=30, scheduler=["linear", 10, 50, 10]), DataEntry("rngds", "b", scheduler=["base"]),
               DataEntry("rngds", "c", weight=5, max_epoch=1)]
    tracker = DataSchedulerTracker([e.weight for e in entries])
    sched = DataScheduler(tracker, entries, max_steps=100)
    sched.step(0)
    assert tracker.weights == [10, 85.0, 5]
    sched.step(5)
    assert tracker.weights[0] == 30 and tracker.weights[1] == 65.0
    tracker.epoch_count[2] = 1
    sched.step(10)
    assert tracker.weights == [50, 50.0, 0]


def test_lr_and_batch_schedules():
    kw = dict(warmup_steps=10, max_steps=100, cooldown_steps=20, min_lr=1e-5)
    assert get_lr(1e-3, 5, schedule="cosine", **kw) == pytest.approx(5e-4)
    assert get_lr(1e-3, 50, schedule="trapezoid", **kw) == 1e-3
    assert get_lr(1e-3, 90, schedule="trapezoid", **kw) == pytest.approx(5e-4)
    assert get_lr(1e-3, 100, schedule="trapezoid", **kw) == 1e-5
    assert get_lr(1e-3, 55, schedule="cosine", warmup_steps=10, max_steps=100) == pytest.approx(5e-4, rel=1e-6)
    with pytest.raises(ValueError):
        get_lr(1e-3, 50, schedule="nope", **kw)
    assert get_batch_size(0, 100, 8) == 1 and get_batch_size(50, 100, 8) == 4 and get_batch_size(200, 100, 8) == 8
    assert get_batch_size(30, 100, 8) == 3      # ceil, as train.py:856-862 of the reference


def test_settings_yaml_overrides_and_derivations(tmp_path, monkeypatch):
    monkeypatch.setenv("WORLD_SIZE", "8")
    monkeypatch.delenv("SLURM_NTASKS", raising=False)
    cfg = parse_cli([f"--config={ROOT}/launch_configs/nebel_zero_8xb200.yaml", f"--out_dir={tmp_path}",
                     "--optim_config.lr=1e-3", "--fabric.optim_sharding=true", "--model_overwrite.mean_recurrence=16"])
    assert cfg.gradient_accumulation_steps == 8 and cfg.devices == 8 and cfg.loader_block_size == 4097
    assert cfg.optim_config["lr"] == 1e-3 and cfg.fabric.optim_sharding and cfg.model_config.mean_recurrence == 16
    assert cfg.model_config.n_embd == 5280 and cfg.model_config.sampling_scheme == "fixed"
    cfg.dump(str(tmp_path / "run_config.json"))
    with pytest.raises(SystemExit):
        parse_cli([f"--out_dir={tmp_path}", "--no_such_flag=1"])
    with pytest.raises(ValueError):  # world batch must factor into micro-batch x accumulation x devices
        parse_cli([f"--out_dir={tmp_path}", "--world_batch_size=12", "--micro_batch_size=5", "--max_steps=3", "--max_tokens=0"])


def test_reference_yaml_loads(monkeypatch, tmp_path):
    monkeypatch.setenv("WORLD_SIZE", "4096")
    monkeypatch.setenv("SLURM_JOB_NUM_NODES", "512")
    monkeypatch.setenv("SLURM_NTASKS_PER_NODE", "8")
    monkeypatch.setenv("RUN_DIR", str(tmp_path))
    cfg = parse_cli([f"--config={ROOT}/launch_configs/frontier_nebel_512_nodes.yaml"])
    assert cfg.optimizer == "ELLISAdam" and cfg.optim_config["atan_adam"] and cfg.gradient_accumulation_steps == 1
    assert cfg.partial_depth_eval == [1, 4, 8, 16, 64] and cfg.model_config.lockstep_n


def test_offline_pipeline_tokenizer_pack_shuffle_count(tmp_path):
    """Raw text -> tokenizer -> packed shards -> reshuffle -> counts -> readable by the training loader."""
    import json as _json

    import pyarrow.parquet as pq

    from recurrent_pretraining_b200.data.datasets import ParquetStream
    from recurrent_pretraining_b200.data.prepare import count_tokens, shuffle_shards, tokenize_pack, tokenizer_train
    from recurrent_pretraining_b200.data.prepare.special_tokens import special_token_ids

    assert special_token_ids(65536)["<|begin_text|>"] == 65504 and special_token_ids(65536)["<|end_text|>"] == 65505
    assert special_token_ids(65536)["<|end_turn|>"] == 65508 and special_token_ids(65536)["<|pad|>"] == 65509
    raw = tmp_path / "raw.jsonl"
    with open(raw, "w") as f:
        for i in range(200):
            f.write(_json.dumps({"text": f"Document {i}: the quick brown fox jumps over {i * 7} lazy dogs.\n\\alpha == 3"}) + "\n")
    V = 512
    tok = tokenizer_train.train_tokenizer([str(raw)], vocab_size=V, out_dir=str(tmp_path / "tok"))
    assert tok.get_vocab_size() == V
    ids = special_token_ids(V)
    assert tok.token_to_id("<|begin_text|>") == ids["<|begin_text|>"] == V - 32
    text = "the quick brown fox 123"
    assert tok.decode(tok.encode(text).ids) == text
    info = tokenize_pack.prepare([str(raw)], lambda s: tok.encode(s).ids, ids["<|begin_text|>"], ids["<|end_text|>"],
                                 str(tmp_path / "data"), block_size=32, num_shards=4, val_fraction=0.1, row_group_size=8)
    assert info["documents"] == 200 and info["rows"] == info["tokens"] // 33 and len(info["train"]) == 4
    before = count_tokens.count_folder(str(tmp_path / "data" / "train"), track_ids=[ids["<|begin_text|>"]])
    first_rows = pq.read_table(info["train"][0]).column("input_ids").to_pylist()
    assert all(len(r) == 33 for r in first_rows)
    assert shuffle_shards.shuffle_shards(str(tmp_path / "data" / "train"), rounds=2, group_size=2) == 4
    after = count_tokens.count_folder(str(tmp_path / "data" / "train"), track_ids=[ids["<|begin_text|>"]])
    assert after["rows"] == before["rows"] and after["tokens"] == before["tokens"] and after["tracked"] == before["tracked"]
    assert pq.read_table(info["train"][0]).column("input_ids").to_pylist() != first_rows
    ds = ParquetStream(str(tmp_path / "data" / "train"), num_processes=1, process_rank=0, broadcast_glob=False,
                       plan_for_later_rank_expansion_to=0)
    rows = list(ds)
    assert len(rows) == after["rows"] and rows[0].shape == (33,)


def test_every_launch_config_parses_and_names_a_known_model(tmp_path):
    import glob

    from recurrent_pretraining_b200.config import ModelConfig
    from recurrent_pretraining_b200.settings import parse_cli

    files = sorted(glob.glob(f"{ROOT}/launch_configs/*.yaml"))
    assert len(files) >= 7
    for f in files:
        cfg = parse_cli([f"--config={f}", f"--out_dir={tmp_path}"])
        mc = ModelConfig.from_name(cfg.model_name, **(cfg.model_overwrite or {}))
        assert mc.n_embd % mc.num_attention_heads == 0 and cfg.micro_batch_size >= 1, f
        assert cfg.optimizer and cfg.fabric_strategy, f


def test_buffer_shuffled_parquet_covers_everything_and_resumes_exactly(tmp_path):
    from recurrent_pretraining_b200.data import BufferShuffledParquet

    total = _write_shards(tmp_path, n_files=3, groups=2, rows=11)
    make = lambda **kw: BufferShuffledParquet(str(tmp_path), seed=4, buffer_size=8, read_batch=4, **kw)  # noqa: E731
    rows = [tuple(r.tolist()) for r in make()]
    assert len(rows) == total and len(set(rows)) == total
    plain = [tuple(r.tolist()) for r in make(shuffle=False, shuffle_filenames=False)]
    assert rows != plain and sorted(rows) == sorted(plain)
    for k in (1, 9, 20, 37):
        ds = make()
        it = iter(ds)
        head = [tuple(next(it).tolist()) for _ in range(k)]
        state = ds.state_dict()
        again = make()
        again.load_state_dict(state)
        assert head + [tuple(r.tolist()) for r in again] == rows, k
    a, b = make(num_processes=2, process_rank=0), make(num_processes=2, process_rank=1)
    assert not set(a.parquet_files) & set(b.parquet_files)
    assert sum(t.shape[0] for t in make().iter_batches(16)) == total


def test_text_rows_are_dealt_over_ranks_and_workers_and_resume(tmp_path):
    """The row-sharded text source: shard ``rank * workers + worker`` of ``ranks * workers`` takes every n-th row of the
    (repeated) table, keeps only the signature's keys, and resumes at its saved row (recpre/huggingface_dataset.py:341-441)."""
    import pyarrow as pa
    import pyarrow.parquet as pq
    from torch.utils.data import DataLoader

    from recurrent_pretraining_b200.data import HuggingfaceDataset, TextRows

    assert HuggingfaceDataset is TextRows
    rows = [{"text": f"row {i}", "extra": i} for i in range(23)]
    pq.write_table(pa.Table.from_pylist(rows), tmp_path / "part.parquet")
    sig = {"keys": ["text"], "format_fn": "pass_text"}
    seen = []
    for rank in range(2):
        ds = TextRows(str(tmp_path), sig, num_processes=2, process_rank=rank, repetitions=2, data_id="d")
        assert len(ds) == 23
        got = list(ds)
        assert all(set(r) == {"text", "data_signature", "data_id"} for r in got)
        seen += [r["text"] for r in got]
        assert ds.fingerprint is not None and ds.index_range[0] == rank
    assert sorted(seen) == sorted([f"row {i}" for i in range(23)] * 2)          # two repetitions, nothing lost
    # with loader workers the table is dealt over ranks * workers shards
    ds = TextRows(rows, sig, num_processes=2, process_rank=1)
    via_workers = [r for batch in DataLoader(ds, batch_size=None, num_workers=2) for r in [batch["text"]]]
    assert sorted(via_workers) == sorted(f"row {i}" for i in range(23) if i % 4 in (2, 3))
    # resume
    a = TextRows(rows, sig, num_processes=2, process_rank=0)
    it = iter(a)
    head = [next(it)["text"] for _ in range(5)]
    state = a.state_dict()
    b = TextRows(rows, sig, num_processes=2, process_rank=0)
    b.load_state_dict(state)
    assert head + [r["text"] for r in b] == [f"row {i}" for i in range(0, 23, 2)]


def test_data_classes_accept_the_reference_constructor_keywords(tmp_path):
    """Scripts written against the reference pass its argument names (recpre/huggingface_dataset.py:35-51,128-145,
    298-309,445; recpre/data_scheduler_utils.py:131; recpre/tokenizer.py:11)."""
    import types

    import pyarrow as pa
    import pyarrow.parquet as pq

    from recurrent_pretraining_b200.data.datasets import (BufferShuffledParquet, ParquetStream, RandomTokens, TextRows,
                                                          WeightedMixture)
    from recurrent_pretraining_b200.data.scheduler import DataScheduler, DataSchedulerTracker, GetScheduler
    from recurrent_pretraining_b200.data.tokenizer import Tokenizer
    from recurrent_pretraining_b200.settings import DataEntry

    pq.write_table(pa.table({"tokens": [[1, 2, 3, 4], [5, 6, 7, 8]]}), tmp_path / "a_0.parquet")
    kw = dict(dataset_folder_path=str(tmp_path), seed=1, shuffle=False, num_processes=1, process_rank=0, prefix="a_",
              verbose=False, shuffle_filenames=True, data_signature={"keys": ["tokens"]}, repetitions=None,
              return_data_id=False, data_id=None, broadcast_glob=False, stateful=True)
    rows = [list(map(int, r)) for r in ParquetStream(plan_for_later_rank_expansion_to=0, **kw)]
    assert sorted(rows) == [[1, 2, 3, 4], [5, 6, 7, 8]]
    assert sorted(list(map(int, r)) for r in BufferShuffledParquet(**kw)) == sorted(rows)
    text = TextRows(ds_name_or_path=[{"text": "a"}, {"text": "b"}, {"text": "c"}], num_processes=1, process_rank=0)
    assert [r["text"] for r in text] == ["a", "b", "c"] and text.sig["format_fn"] == "pass_text" and text.seed == 12345
    assert RandomTokens().block_size == 4096 and RandomTokens().vocab_size == 1024
    mix = WeightedMixture(datasets=[[1, 1, 1], [2, 2, 2]], seed=3)                # uniform weights
    assert sorted(mix) == [1, 1, 1, 2, 2, 2] and mix.weights == [0.5, 0.5]
    mix = WeightedMixture([[1], [2]], 7, [1.0, 0.0])                               # (datasets, seed, weights)
    assert mix.weights == [1.0, 0.0] and list(mix) == [1]
    entries = [DataEntry(type="rngds", prefix="", weight=60, scheduler=["linear", 60, 20]),
               DataEntry(type="rngds", prefix="", weight=40)]
    tracker = DataSchedulerTracker([60, 40])
    sched = DataScheduler(data_scheduler_tracker=tracker, data_config=entries, args=types.SimpleNamespace(max_steps=10))
    sched.step(5)
    assert tracker.weights == [40.0, 40]
    assert GetScheduler(["linear", 60, 20], 0, types.SimpleNamespace(max_steps=10)).get_weight(10) == 20
    assert Tokenizer(tmp_path / "missing", broken_state_load_fallback=True).processor is None
    with pytest.raises(NotADirectoryError):
        Tokenizer(tmp_path / "missing", broken_state_load_fallback=False)


def test_goldfish_strategies_against_the_reference_and_their_definitions():
    """``static`` and ``hash-table`` equal the reference's masks bit for bit; the random strategies drop about 1/k of
    the positions of EVERY row (the reference blanks rows 0 and 1 instead); ``hash-legacy`` and the micro-batch-seeded
    form are functions of the labels alone."""
    import refload

    from recurrent_pretraining_b200.data.goldfish import apply_tld
    from recurrent_pretraining_b200.settings import GoldfishConfig

    torch.manual_seed(0)
    labels = torch.randint(1, 500, (4, 96))
    if refload.available():
        ref_tld = refload.module("utils").apply_tld
        for strat in ("static", "hash-table"):
            for k, start, ctx in ((2, 0, 3), (4, 5, 13), (3, 1, 4)):
                cfg = GoldfishConfig(strategy=strat, k_token_loss_dropout=k, start_position=start, context_width=ctx)
                want, _ = ref_tld(labels.clone(), cfg, ignore_index=-100)
                got, _ = apply_tld(labels.clone(), cfg, ignore_index=-100)
                assert torch.equal(got, want), (strat, k, start, ctx)
    for strat in ("seeded_random", "pure_random", "random_but_consisent_for_given_micro_batch", "hash-legacy"):
        cfg = GoldfishConfig(strategy=strat, k_token_loss_dropout=4, context_width=3)
        out, drop = apply_tld(labels, cfg)
        frac = (out == -100).float().mean(dim=1)
        assert bool(((frac > 0.05) & (frac < 0.5)).all()), (strat, frac)
        assert torch.equal((out == -100), drop.bool()) and torch.equal(out[out != -100], labels[out != -100])
    for strat in ("random_but_consisent_for_given_micro_batch", "hash-legacy", "hash-avalanche"):
        cfg = GoldfishConfig(strategy=strat, k_token_loss_dropout=3, context_width=3)
        assert torch.equal(apply_tld(labels, cfg)[0], apply_tld(labels.clone(), cfg)[0])
    with pytest.raises(NotImplementedError):
        apply_tld(labels, GoldfishConfig(strategy="nope"))


def test_collate_matches_the_reference_collate_function():
    """Tensor rows (fast and general path, pad replaced by eos in the inputs only) and text rows with every format
    function, against recpre/data_loading_utils.py:generic_collate_fn on the same batches."""
    import copy

    import refload

    if not refload.available():
        pytest.skip("reference not installed under baseline/_ref")
    ref_collate = refload.module("data_loading_utils").generic_collate_fn
    from recurrent_pretraining_b200.data.collate import generic_collate_fn

    class Tok:
        pad_id, eos_id, bos_id = 0, 2, 1

        def encode(self, s, bos=False, eos=False, device=None, max_length=-1):
            ids = [3 + (ord(c) % 50) for c in s]
            ids = ([self.bos_id] if bos else []) + ids + ([self.eos_id] if eos else [])
            return torch.tensor(ids[:max_length] if max_length > 0 else ids, dtype=torch.int)

    def same(x, y):
        if torch.is_tensor(x):
            return torch.is_tensor(y) and x.shape == y.shape and torch.equal(x.long(), y.long())
        if isinstance(x, (list, tuple)):
            return len(x) == len(y) and all(same(i, j) for i, j in zip(x, y))
        return x == y

    tok = Tok()
    torch.manual_seed(0)
    rows = [torch.randint(3, 60, (17,)) for _ in range(3)]
    rows[0][5] = 0
    batches = [(rows, kw) for kw in (dict(block_size=16, all_block_size_tensors=True),
                                     dict(block_size=16, pad_to_block_size=True), dict(block_size=16))]
    for fmt, keys in (("pass_text", ["text"]), ("concat_input_target", ["input", "target"]),
                      ("condition_input_supervise_target", ["input", "target"])):
        sig = {"keys": keys, "format_fn": fmt}
        text = [dict({k: ("hello world " * (i + 1))[:7 * (i + 1) + j] for j, k in enumerate(keys)}, data_signature=sig)
                for i in range(3)]
        batches += [(text, kw) for kw in (dict(block_size=24, pad_to_block_size=True), dict(block_size=24),
                                          dict(block_size=12, add_bos=False))]
    for batch, kw in batches:
        want = ref_collate(copy.deepcopy(batch), tok, **kw)
        got = generic_collate_fn(copy.deepcopy(batch), tok, **kw)
        assert same(want, got), kw


def test_parquet_stream_yields_rows_in_the_reference_order(tmp_path, capsys):
    """File shuffle, per-rank file striding (with the later-expansion plan) and the per-row-group shuffle give the same
    row sequence as recpre/huggingface_dataset.py:ParquetStreamPure on the same shards."""
    import random

    import pyarrow as pa
    import pyarrow.parquet as pq
    import refload

    if not refload.available():
        pytest.skip("reference not installed under baseline/_ref")
    ref_cls = refload.module("huggingface_dataset").ParquetStreamPure
    from recurrent_pretraining_b200.data.datasets import ParquetStream

    rng = random.Random(0)
    for f in range(40):
        rows = [[f * 1000 + g * 100 + i, rng.randrange(100)] for g in range(3) for i in range(7)]
        pq.write_table(pa.table({"input_ids": rows}), tmp_path / f"train_{f:03d}.parquet", row_group_size=7)

    def take(ds, n):
        it = iter(ds)
        return [[int(v) for v in next(it)] for _ in range(n)]

    base = dict(dataset_folder_path=str(tmp_path), seed=7, prefix="train_", broadcast_glob=False)
    for kw in (dict(num_processes=1, process_rank=0), dict(num_processes=2, process_rank=1),
               dict(num_processes=2, process_rank=0, shuffle=False),
               dict(num_processes=1, process_rank=0, shuffle_filenames=False),
               dict(num_processes=3, process_rank=2, plan_for_later_rank_expansion_to=0),
               dict(num_processes=16, process_rank=9)):
        assert take(ref_cls(**base, **kw), 30) == take(ParquetStream(**base, **kw), 30), kw
    capsys.readouterr()


@pytest.mark.parametrize("name", ["recurrent.yaml", "frontier_nebel_512_nodes.yaml", "frontier_baseline_256_nodes.yaml"])
def test_derived_settings_match_the_reference_settings_class(name, monkeypatch):
    """The reference's launch configs through the reference's ``CLISettings`` and through ours, under the same SLURM
    environment: every derived attribute (batch arithmetic, loader block size, dataset prefixes, environment fields)
    and every field both classes have agree."""
    import dataclasses

    import refload
    import yaml

    if not refload.available():
        pytest.skip("reference not installed under baseline/_ref")
    theirs_mod = refload.module("settings")
    from recurrent_pretraining_b200 import settings as ours_mod

    for k, v in {"SLURM_JOB_NUM_NODES": "4", "SLURM_NTASKS": "32", "SLURM_NTASKS_PER_NODE": "8", "WORLD_SIZE": "32",
                 "SLURM_JOB_ID": "77", "SLURM_ARRAY_TASK_ID": "2", "SLURM_ARRAY_TASK_COUNT": "5",
                 "SLURM_ARRAY_JOB_ID": "70", "SLURM_PROCID": "3", "MASTER_ADDR": "node0", "MASTER_PORT": "29400",
                 "OUTPUT_DIR": "/tmp/out"}.items():
        monkeypatch.setenv(k, v)
    path = os.path.join(os.path.dirname(__file__), "..", "launch_configs", name)

    def build(mod):
        y = yaml.safe_load(open(path))
        if "fabric" in y:
            y["fabric"] = mod.FabricConfig(**y["fabric"])
        if "goldfish" in y:
            y["goldfish"] = mod.GoldfishConfig(**y["goldfish"])
        if isinstance(y.get("data_config"), dict):
            y["data_config"] = {k: [mod.DataEntry(**e) for e in v] for k, v in y["data_config"].items()}
        return mod.CLISettings(**y)

    a, b = build(theirs_mod), build(ours_mod)
    def plain(v):
        if dataclasses.is_dataclass(v):
            return dataclasses.asdict(v)
        if isinstance(v, dict):
            return {k: plain(x) for k, x in v.items()}
        if isinstance(v, (list, tuple)):
            return [plain(x) for x in v]
        return v

    # derived later over there / a site-specific default path
    skipped = {"model_config", "max_steps", "max_tokens_per_device", "tokens_per_step", "tokenizer_path"}
    for key, want in vars(a).items():
        if key in skipped:
            continue
        assert hasattr(b, key), key
        assert plain(getattr(b, key)) == plain(want), (key, getattr(b, key), want)
    # the step budget the reference derives at start-up (train.py:268-271)
    world = a.devices * a.num_nodes
    assert b.max_steps == (a.max_tokens // world) // (a.micro_batch_size * a.block_size)
    for key in ("n_embd", "intermediate_size", "mean_recurrence", "mean_backprop_depth", "sampling_scheme",
                "injection_type", "block_class_name", "norm_class_name", "init_strategy", "padded_vocab_size"):
        if hasattr(a.model_config, key):
            assert getattr(b.model_config, key) == getattr(a.model_config, key), key


def test_tokenizer_wrapper_matches_the_reference_wrapper(tmp_path):
    """A small BPE tokenizer trained on the spot, loaded through the reference's wrapper and through ours: special ids,
    vocabulary size, encodings with every bos / eos / max_length combination, decoding, pickling."""
    import json
    import pickle

    import refload
    from tokenizers import Tokenizer as RawTokenizer
    from tokenizers import models, pre_tokenizers, trainers

    from recurrent_pretraining_b200.data.tokenizer import Tokenizer

    raw = RawTokenizer(models.BPE(unk_token="<unk>"))
    raw.pre_tokenizer = pre_tokenizers.Whitespace()
    trainer = trainers.BpeTrainer(vocab_size=200, special_tokens=["<unk>", "<|begin_text|>", "<|end_text|>", "<|pad|>"])
    raw.train_from_iterator(["hello world this is a test of the tokenizer", "another line of text for training"] * 20,
                            trainer)
    raw.save(str(tmp_path / "tokenizer.json"))
    special = {"bos_token": "<|begin_text|>", "eos_token": "<|end_text|>", "pad_token": "<|pad|>"}
    (tmp_path / "tokenizer_config.json").write_text(json.dumps(dict(special, tokenizer_class="PreTrainedTokenizerFast")))
    (tmp_path / "special_tokens_map.json").write_text(json.dumps(special))
    ours = Tokenizer(tmp_path)
    assert (ours.bos_id, ours.eos_id, ours.pad_id) == (1, 2, 3) and ours.cache_token_id is None
    text = "hello world this is a test"
    if refload.available():
        theirs = refload.module("tokenizer").Tokenizer(tmp_path)
        assert (theirs.bos_id, theirs.eos_id, theirs.pad_id, theirs.vocab_size) == (1, 2, 3, ours.vocab_size)
        for kw in (dict(), dict(bos=True), dict(eos=True), dict(bos=True, eos=True, max_length=5),
                   dict(bos=False, eos=True, max_length=3)):
            a, b = theirs.encode(text, **kw), ours.encode(text, **kw)
            assert a.dtype == b.dtype and torch.equal(a, b), kw
        ids = theirs.encode("hello world", bos=True, eos=True)
        assert theirs.decode(ids) == ours.decode(ids)
    ids = ours.encode(text, bos=True, eos=True)
    assert int(ids[0]) == 1 and int(ids[-1]) == 2 and "hello" in ours.decode(ids)
    again = pickle.loads(pickle.dumps(ours))
    assert torch.equal(again.encode(text), ours.encode(text))
