"""Token-shard and evaluation-file preparation from LOCAL files.

Plays the role of the reference's dataset scripts (dev/data/data_common.py:26-143 ``write_datafile`` /
``write_evalfile`` and the per-dataset drivers tinyshakespeare.py, tinystories.py, fineweb.py, hellaswag.py,
mmlu.py). Those scripts download their sources; this module never touches the network: it tokenizes text or
JSON-lines files that are already on disk and writes the same ``.bin`` formats (utils/formats.py).

    python -m llm_kittens_b200.data.prepare text  --input corpus.txt --out-dir data/corpus --tokenizer gpt2
    python -m llm_kittens_b200.data.prepare docs  --input "fineweb/*.parquet" --out-dir data/fineweb10B --name fineweb --workers 32
    python -m llm_kittens_b200.data.prepare docs  --input "TinyStories_all_data/*.json" --field story --out-dir data/tinystories --name TinyStories
    python -m llm_kittens_b200.data.prepare hellaswag --input hellaswag_val.jsonl --out data/hellaswag_val.bin
    python -m llm_kittens_b200.data.prepare synthetic --out-dir data/synth --tokens 2000000

Tokenizers: ``gpt2`` needs a local GPT-2 BPE (``tiktoken`` with its cache, or ``--tokenizer-dir`` holding
vocab.json / merges.txt for ``transformers``); ``llama-3`` needs ``--tokenizer-dir`` with an HF tokenizer;
``bytes`` is a dependency-free byte-level tokenizer (256 byte tokens + end-of-text = 256).
"""
from __future__ import annotations

import argparse
import glob
import json
import multiprocessing
import os

import numpy as np

from ..utils import formats


class ByteTokenizer:
    eot = 256
    vocab_size = 257
    model_desc = "gpt-2"

    def encode(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))


class _HFTokenizer:
    def __init__(self, path: str, model_desc: str):
        from transformers import AutoTokenizer

        self.tok = AutoTokenizer.from_pretrained(path, local_files_only=True)
        self.model_desc = model_desc
        self.eot = self.tok.eos_token_id if model_desc == "gpt-2" else (self.tok.bos_token_id or self.tok.eos_token_id)
        self.vocab_size = len(self.tok)

    def encode(self, text: str) -> list[int]:
        return self.tok.encode(text, add_special_tokens=False)


class _TiktokenGPT2:
    model_desc = "gpt-2"

    def __init__(self):
        import tiktoken

        self.enc = tiktoken.get_encoding("gpt2")
        self.eot = self.enc._special_tokens["<|endoftext|>"]
        self.vocab_size = self.enc.n_vocab

    def encode(self, text: str) -> list[int]:
        return self.enc.encode_ordinary(text)


def get_tokenizer(name: str, tokenizer_dir: str | None = None):
    if name == "bytes":
        return ByteTokenizer()
    if name == "gpt2":
        if tokenizer_dir:
            return _HFTokenizer(tokenizer_dir, "gpt-2")
        try:
            return _TiktokenGPT2()
        except Exception as e:  # no tiktoken or no cached vocabulary
            raise RuntimeError(f"GPT-2 tokenizer unavailable offline ({e}); pass --tokenizer-dir or use --tokenizer bytes") from e
    if name == "llama-3":
        if not tokenizer_dir:
            raise RuntimeError("--tokenizer-dir with a local Llama-3 tokenizer is required")
        return _HFTokenizer(tokenizer_dir, "llama-3")
    raise ValueError(f"unknown tokenizer {name}")


def tokenize_documents(docs, tok) -> np.ndarray:
    """Each document is preceded by the end-of-text token (as the reference's scripts do)."""
    out = []
    for d in docs:
        out.append(tok.eot)
        out.extend(tok.encode(d))
    return np.asarray(out, dtype=np.int64)


def write_shards(tokens: np.ndarray, out_dir: str, name: str, model_desc: str, shard_size: int = 100_000_000,
                 val_tokens: int = 0) -> list[str]:
    """``val_tokens`` leading tokens go to ``<name>_val_000000.bin``, the rest to ``<name>_train_%06d.bin`` shards."""
    os.makedirs(out_dir, exist_ok=True)
    paths = []
    if val_tokens > 0:
        p = os.path.join(out_dir, f"{name}_val_000000.bin")
        formats.write_tokens(p, tokens[:val_tokens], model_desc)
        paths.append(p)
        tokens = tokens[val_tokens:]
    for i, start in enumerate(range(0, len(tokens), shard_size)):
        p = os.path.join(out_dir, f"{name}_train_{i:06d}.bin")
        formats.write_tokens(p, tokens[start:start + shard_size], model_desc)
        paths.append(p)
    return paths


def prepare_text(input_path: str, out_dir: str, tok, name: str | None = None, shard_size: int = 100_000_000,
                 val_fraction: float = 0.05, doc_separator: str | None = None) -> list[str]:
    text = open(input_path, encoding="utf-8").read()
    docs = [d for d in text.split(doc_separator)] if doc_separator else [text]
    tokens = tokenize_documents(docs, tok)
    name = name or os.path.splitext(os.path.basename(input_path))[0]
    return write_shards(tokens, out_dir, name, tok.model_desc, shard_size, int(len(tokens) * val_fraction))


def iter_documents(paths: list[str], field: str = "text"):
    """Texts of the documents in ``paths``, file by file: ``.parquet`` (column ``field``, read row group by row group),
    ``.jsonl`` (one object per line), ``.json`` (a list of objects) or plain text (the whole file is one document)."""
    for path in paths:
        ext = os.path.splitext(path)[1].lower()
        if ext == ".parquet":
            import pyarrow.parquet as pq

            f = pq.ParquetFile(path)
            for g in range(f.num_row_groups):
                for text in f.read_row_group(g, columns=[field]).column(field).to_pylist():
                    yield text
        elif ext == ".jsonl":
            with open(path, encoding="utf-8") as fh:
                for line in fh:
                    if line.strip():
                        yield json.loads(line)[field]
        elif ext == ".json":
            with open(path, encoding="utf-8") as fh:
                for obj in json.load(fh):
                    yield obj[field]
        else:
            with open(path, encoding="utf-8") as fh:
                yield fh.read()


_WORKER_TOK = None


def _worker_init(tokenizer: str, tokenizer_dir: str | None) -> None:
    global _WORKER_TOK
    _WORKER_TOK = get_tokenizer(tokenizer, tokenizer_dir)


def _worker_encode(text: str) -> np.ndarray:
    tok = _WORKER_TOK
    ids = [tok.eot]
    ids.extend(tok.encode(text.strip() if isinstance(text, str) else str(text)))
    return np.asarray(ids, dtype=np.uint32)


class ShardWriter:
    """Streams token arrays into fixed-size shards: the first full shard is the validation shard, the rest are the
    training shards (the split of the reference's dev/data/fineweb.py:60-116); memory stays at one shard. A document that
    does not fit the rest of a shard is cut at the shard boundary."""

    def __init__(self, out_dir: str, name: str, model_desc: str, shard_size: int):
        os.makedirs(out_dir, exist_ok=True)
        self.out_dir, self.name, self.model_desc, self.shard_size = out_dir, name, model_desc, int(shard_size)
        self.buf = np.empty(self.shard_size, dtype=np.uint32)
        self.fill, self.index, self.paths, self.total = 0, 0, [], 0

    def _flush(self) -> None:
        split = "val" if self.index == 0 else "train"
        number = 0 if self.index == 0 else self.index - 1
        p = os.path.join(self.out_dir, f"{self.name}_{split}_{number:06d}.bin")
        formats.write_tokens(p, self.buf[:self.fill], self.model_desc)
        self.paths.append(p)
        self.index += 1
        self.fill = 0

    def add(self, ids: np.ndarray) -> None:
        self.total += len(ids)
        while len(ids):
            n = min(len(ids), self.shard_size - self.fill)
            self.buf[self.fill:self.fill + n] = ids[:n]
            self.fill += n
            ids = ids[n:]
            if self.fill == self.shard_size:
                self._flush()

    def close(self) -> list[str]:
        if self.fill:
            self._flush()
        return self.paths


def prepare_documents(pattern: str, out_dir: str, tokenizer: str, tokenizer_dir: str | None = None, name: str = "corpus",
                      field: str = "text", shard_size: int = 100_000_000, workers: int = 0) -> list[str]:
    """Tokenizes every document of the files matching ``pattern`` with a pool of ``workers`` processes (0: in this
    process) and streams the tokens, each document led by the end-of-text token, into shards."""
    paths = sorted(glob.glob(pattern))
    if not paths:
        raise FileNotFoundError(f"no input file matches {pattern}")
    tok = get_tokenizer(tokenizer, tokenizer_dir)        # fails early, in the parent, when the vocabulary is not on disk
    writer = ShardWriter(out_dir, name, tok.model_desc, shard_size)
    docs = iter_documents(paths, field)
    if workers <= 0:
        _worker_init(tokenizer, tokenizer_dir)
        for text in docs:
            writer.add(_worker_encode(text))
    else:
        with multiprocessing.get_context("spawn").Pool(workers, initializer=_worker_init, initargs=(tokenizer, tokenizer_dir)) as pool:
            for ids in pool.imap(_worker_encode, docs, chunksize=16):     # imap keeps the document order: reruns give identical shards
                writer.add(ids)
    return writer.close()


def prepare_synthetic(out_dir: str, num_tokens: int, vocab_size: int = 50257, seed: int = 0, model_desc: str = "gpt-2",
                      shard_size: int = 100_000_000) -> list[str]:
    rng = np.random.default_rng(seed)
    tokens = rng.integers(0, vocab_size, size=num_tokens, dtype=np.int64)
    return write_shards(tokens, out_dir, "synthetic", model_desc, shard_size, min(num_tokens // 10, shard_size))


def hellaswag_examples(jsonl_path: str, tok):
    """HellaSwag JSON lines (``ctx``, ``endings``, ``label``) -> example dicts; endings get a leading space."""
    for line in open(jsonl_path, encoding="utf-8"):
        if not line.strip():
            continue
        ex = json.loads(line)
        yield {"label": int(ex["label"]), "ctx_tokens": tok.encode(ex["ctx"]),
               "ending_tokens": [tok.encode(" " + e) for e in ex["endings"]]}


def mmlu_examples(jsonl_path: str, tok):
    """MMLU JSON lines (``question``, ``choices``, ``answer`` index) -> the same example layout."""
    for line in open(jsonl_path, encoding="utf-8"):
        if not line.strip():
            continue
        ex = json.loads(line)
        ctx = f"Question: {ex['question']}\n\nAnswer:"
        yield {"label": int(ex["answer"]), "ctx_tokens": tok.encode(ctx), "ending_tokens": [tok.encode(" " + c) for c in ex["choices"]]}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    t = sub.add_parser("text")
    t.add_argument("--input", required=True)
    t.add_argument("--out-dir", required=True)
    t.add_argument("--tokenizer", default="gpt2", choices=["gpt2", "llama-3", "bytes"])
    t.add_argument("--tokenizer-dir")
    t.add_argument("--shard-size", type=int, default=100_000_000)
    t.add_argument("--val-fraction", type=float, default=0.05)
    t.add_argument("--doc-separator")
    d = sub.add_parser("docs")
    d.add_argument("--input", required=True, help="glob of .parquet / .jsonl / .json / text files")
    d.add_argument("--out-dir", required=True)
    d.add_argument("--name", default="corpus")
    d.add_argument("--field", default="text")
    d.add_argument("--tokenizer", default="gpt2", choices=["gpt2", "llama-3", "bytes"])
    d.add_argument("--tokenizer-dir")
    d.add_argument("--shard-size", type=int, default=100_000_000)
    d.add_argument("--workers", type=int, default=max(1, (os.cpu_count() or 2) - 2))
    for name in ("hellaswag", "mmlu"):
        e = sub.add_parser(name)
        e.add_argument("--input", required=True)
        e.add_argument("--out", required=True)
        e.add_argument("--tokenizer", default="gpt2", choices=["gpt2", "llama-3", "bytes"])
        e.add_argument("--tokenizer-dir")
    s = sub.add_parser("synthetic")
    s.add_argument("--out-dir", required=True)
    s.add_argument("--tokens", type=int, default=2_000_000)
    s.add_argument("--vocab-size", type=int, default=50257)
    args = ap.parse_args(argv)
    if args.cmd == "synthetic":
        paths = prepare_synthetic(args.out_dir, args.tokens, args.vocab_size)
    elif args.cmd == "docs":
        paths = prepare_documents(args.input, args.out_dir, args.tokenizer, args.tokenizer_dir, args.name, args.field, args.shard_size,
                                  args.workers)
    else:
        tok = get_tokenizer(args.tokenizer, args.tokenizer_dir)
        if args.cmd == "text":
            paths = prepare_text(args.input, args.out_dir, tok, shard_size=args.shard_size, val_fraction=args.val_fraction,
                                 doc_separator=args.doc_separator)
        else:
            ex = hellaswag_examples(args.input, tok) if args.cmd == "hellaswag" else mmlu_examples(args.input, tok)
            formats.write_evalfile(args.out, ex, tok.model_desc)
            paths = [args.out]
    for p in paths:
        print(p)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
