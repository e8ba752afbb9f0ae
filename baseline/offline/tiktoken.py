"""Offline stand-in for the `tiktoken` package, for the reference arm of bench.py only.

The reference's PyTorch trainer calls `tiktoken.get_encoding("gpt2")` at start-up. The real package fetches
the GPT-2 vocabulary from the network on first use, which a machine without network access cannot do, and
the vocabulary files are not on the image. The trainer uses the encoding only to write a tokenizer file
(`--write_tensors 1`) and to print samples (`--sample_every > 0`); the benchmark runs it with both off, so
nothing in the timed path touches the tokenizer. This module gives the trainer an object with the fields
it reads (`eot_token`, `max_token_value`) so that the unmodified script starts. It is put on PYTHONPATH of
the reference subprocess alone; nothing in the package imports it.
"""


class _Gpt2Ids:
    name = "gpt2"
    eot_token = 50256
    max_token_value = 50256
    n_vocab = 50257

    def decode(self, ids):
        return " ".join(str(int(i)) for i in ids)

    def decode_bytes(self, ids):
        return self.decode(ids).encode()

    def encode(self, text, allowed_special=()):
        raise RuntimeError("the offline stand-in has no vocabulary; it cannot encode text")


def get_encoding(name):
    if name != "gpt2":
        raise ValueError(f"offline stand-in knows only 'gpt2', not {name!r}")
    return _Gpt2Ids()
