"""Host-side utilities: file formats, data loaders, tokenizer, RNG, LR schedules, logging, MFU."""
