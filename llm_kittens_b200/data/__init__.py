"""Dataset preparation: text / JSON-lines sources -> token shards and evaluation files."""
