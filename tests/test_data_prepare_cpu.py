"""Dataset preparation: shards written from local text are what the native loaders read."""
import json

import numpy as np

from llm_kittens_b200.data import prepare
from llm_kittens_b200.utils import formats
from llm_kittens_b200.utils.dataloader import DataLoader, EvalLoader


def test_text_to_shards_and_loader(tmp_path):
    src = tmp_path / "corpus.txt"
    src.write_text("hello world. " * 400 + "\n<doc>\n" + "second document " * 300)
    tok = prepare.get_tokenizer("bytes")
    paths = prepare.prepare_text(str(src), str(tmp_path / "out"), tok, val_fraction=0.1, doc_separator="\n<doc>\n", shard_size=4096)
    assert any("_val_" in p for p in paths) and sum("_train_" in p for p in paths) >= 2
    train = np.concatenate([formats.read_tokens(p) for p in paths if "_train_" in p])
    val = formats.read_tokens([p for p in paths if "_val_" in p][0])
    allt = np.concatenate([val, train])
    assert allt[0] == tok.eot and (allt == tok.eot).sum() == 2
    assert bytes(allt[1:12].astype(np.uint8)) == b"hello world"
    loader = DataLoader(str(tmp_path / "out" / "corpus_train_*.bin"), 2, 16)
    x, y = loader.next_batch()
    assert x.shape == (2, 16) and (x[0, 1:] == y[0, :-1]).all()
    assert (x.flatten()[:8].numpy() == train[:8]).all()


def test_synthetic_and_eval_files(tmp_path):
    paths = prepare.prepare_synthetic(str(tmp_path / "s"), 10000, vocab_size=1000, seed=1)
    assert len(paths) == 2 and formats.read_tokens(paths[1]).max() < 1000
    jl = tmp_path / "h.jsonl"
    rows = [{"ctx": "the cat sat on the", "endings": ["mat", "moon", "sea", "sun"], "label": i % 4} for i in range(8)]
    jl.write_text("\n".join(json.dumps(r) for r in rows))
    out = tmp_path / "h.bin"
    assert prepare.main(["hellaswag", "--input", str(jl), "--out", str(out), "--tokenizer", "bytes"]) == 0
    ev = EvalLoader(str(out), 8, 32)
    assert ev.num_examples == 8


def test_documents_from_parquet_jsonl_and_json_stream_into_shards(tmp_path):
    """The corpus command (job of the reference's dev/data/fineweb.py and tinystories.py on local files): documents from
    parquet / JSON-lines / JSON files, tokenized by a process pool in document order, first shard = validation."""
    import pyarrow as pa
    import pyarrow.parquet as pq

    docs = [f"document number {i} " * (3 + i % 5) for i in range(60)]
    pq.write_table(pa.table({"text": docs[:25], "id": list(range(25))}), str(tmp_path / "a_000.parquet"), row_group_size=10)
    (tmp_path / "a_001.jsonl").write_text("\n".join(json.dumps({"text": d}) for d in docs[25:45]) + "\n")
    (tmp_path / "a_002.json").write_text(json.dumps([{"text": d} for d in docs[45:]]))
    tok = prepare.get_tokenizer("bytes")
    want = np.concatenate([[tok.eot] + tok.encode(d.strip()) for d in docs])

    out1 = prepare.prepare_documents(str(tmp_path / "a_*"), str(tmp_path / "o1"), "bytes", name="mini", shard_size=2048, workers=0)
    assert out1[0].endswith("mini_val_000000.bin") and out1[1].endswith("mini_train_000000.bin") and len(out1) >= 3
    got = np.concatenate([formats.read_tokens(p) for p in out1])
    assert len(formats.read_tokens(out1[0])) == 2048 and (got == want).all()

    # a pool of two worker processes writes byte-identical shards, through the command line
    assert prepare.main(["docs", "--input", str(tmp_path / "a_*"), "--out-dir", str(tmp_path / "o2"), "--name", "mini", "--tokenizer", "bytes",
                         "--shard-size", "2048", "--workers", "2"]) == 0
    for p in out1:
        q = tmp_path / "o2" / p.split("/")[-1]
        assert q.read_bytes() == open(p, "rb").read()

    # another field name (the TinyStories files hold {"story": ...}); the loader reads what was written
    (tmp_path / "t.json").write_text(json.dumps([{"story": d} for d in docs[:10]]))
    out3 = prepare.prepare_documents(str(tmp_path / "t.json"), str(tmp_path / "o3"), "bytes", name="ts", field="story", shard_size=512)
    loader = DataLoader(str(tmp_path / "o3" / "ts_train_*.bin"), 2, 16)
    x, _ = loader.next_batch()
    assert (x.flatten()[:8].numpy() == formats.read_tokens(out3[1])[:8]).all()
