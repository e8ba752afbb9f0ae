"""ctypes handle to the C++ host runtime (``_lib/libllmk_host.so``, built from ``csrc/host``)."""
from __future__ import annotations

import ctypes
import threading

from .. import build as _build

_LOCK = threading.Lock()
_LIB = None

c_void_p, c_int, c_long, c_float, c_char_p, c_u32 = (ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float,
                                                     ctypes.c_char_p, ctypes.c_uint32)

_SIGNATURES = {
    "llmk_host_last_error": (c_char_p, []),
    "llmk_rng_create": (c_void_p, [c_u32]),
    "llmk_rng_destroy": (None, [c_void_p]),
    "llmk_rng_seed": (None, [c_void_p, c_u32]),
    "llmk_rng_u32": (c_u32, [c_void_p]),
    "llmk_rng_uniform": (None, [c_void_p, c_void_p, c_long, c_float, c_float]),
    "llmk_rng_normal": (None, [c_void_p, c_void_p, c_long, c_float, c_float]),
    "llmk_rng_permutation": (None, [c_void_p, c_void_p, c_int]),
    "llmk_rng_state_bytes": (c_long, []),
    "llmk_rng_save": (None, [c_void_p, c_void_p]),
    "llmk_rng_load": (None, [c_void_p, c_void_p]),
    "llmk_xorshift_u32": (c_u32, [c_void_p]),
    "llmk_xorshift_f32": (c_float, [c_void_p]),
    "llmk_sample_softmax": (c_int, [c_void_p, c_int, c_float]),
    "llmk_loader_create": (c_void_p, [c_char_p, c_long, c_long, c_int, c_int, c_int]),
    "llmk_loader_destroy": (None, [c_void_p]),
    "llmk_loader_next": (c_int, [c_void_p, c_void_p, c_void_p]),
    "llmk_loader_reset": (c_int, [c_void_p]),
    "llmk_loader_resume": (c_int, [c_void_p, c_long, c_long]),
    "llmk_loader_num_tokens": (c_long, [c_void_p]),
    "llmk_loader_shard_idx": (c_long, [c_void_p]),
    "llmk_loader_sample_idx": (c_long, [c_void_p]),
    "llmk_loader_shard_samples": (c_long, [c_void_p]),
    "llmk_loader_num_shards": (c_int, [c_void_p]),
    "llmk_loader_token_bytes": (c_int, [c_void_p]),
    "llmk_loader_shuffle_state_bytes": (c_long, [c_void_p]),
    "llmk_loader_save_shuffle_state": (None, [c_void_p, c_void_p]),
    "llmk_loader_load_shuffle_state": (c_int, [c_void_p, c_void_p, c_long]),
    "llmk_evalloader_create": (c_void_p, [c_char_p, c_long, c_long, c_int, c_int]),
    "llmk_evalloader_destroy": (None, [c_void_p]),
    "llmk_evalloader_reset": (c_int, [c_void_p]),
    "llmk_evalloader_next": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "llmk_evalloader_num_examples": (c_int, [c_void_p]),
    "llmk_evalloader_num_batches": (c_int, [c_void_p]),
    "llmk_evalloader_stat_losses": (c_int, [c_void_p, c_void_p, c_void_p, c_long, c_long]),
    "llmk_tokenizer_create": (c_void_p, [c_char_p]),
    "llmk_tokenizer_destroy": (None, [c_void_p]),
    "llmk_tokenizer_vocab_size": (c_int, [c_void_p]),
    "llmk_tokenizer_eot": (c_int, [c_void_p]),
    "llmk_tokenizer_decode": (c_int, [c_void_p, c_int, c_void_p, c_int]),
    "llmk_lr_get": (c_float, [c_int, c_float, c_int, c_int, c_float, c_int]),
    "llmk_outlier_create": (c_void_p, []),
    "llmk_outlier_destroy": (None, [c_void_p]),
    "llmk_outlier_update": (ctypes.c_double, [c_void_p, ctypes.c_double]),
    "llmk_logger_create": (c_void_p, [c_char_p, c_int, c_int]),
    "llmk_logger_destroy": (None, [c_void_p]),
    "llmk_logger_eval": (None, [c_void_p, c_int, c_float]),
    "llmk_logger_val": (None, [c_void_p, c_int, c_float]),
    "llmk_logger_train": (None, [c_void_p, c_int, c_float, c_float, c_float]),
}


class HostError(RuntimeError):
    pass


def lib():
    global _LIB
    if _LIB is None:
        with _LOCK:
            if _LIB is None:
                path = _build.host_lib_path()
                if not path.exists():
                    _build.build()
                h = ctypes.CDLL(str(path))
                for name, (res, args) in _SIGNATURES.items():
                    fn = getattr(h, name)
                    fn.restype = res
                    fn.argtypes = args
                _LIB = h
    return _LIB


def last_error() -> str:
    return lib().llmk_host_last_error().decode(errors="replace")
