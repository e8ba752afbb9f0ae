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
