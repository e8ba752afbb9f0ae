"""Binary file formats (all start with a 256 x int32 header) and their readers / writers.

========== =========================== ===================================================
file       header                      payload
========== =========================== ===================================================
GPT model  [0]=20240326 [1]=5 bf16 / 3 fp32, [2..7]=maxT,V,L,NH,C,Vp       tensors in layout order
Llama      [0]=20240803 [1]=5, [2..15]=maxT,V,L,NH,NKVH,C,hidden,multiple_of,-,theta,scaled,genB,major,minor
MoE        [0]=20250301 [1]=5, GPT fields + [8]=E [9]=top_k [10]=capacity*100
state      [0]=20240527 (GPT) / 20240804 (Llama) / 20250302 (MoE) [1]=1, [2]=nproc [3]=rank [4]=use_master
           [5]=shuffle [10]=step [20..21]=rng [22..23]=rng at last update [30..31]=shard idx [32..33]=sample idx;
           then m, v, (master) fp32 shards, then the loader's shuffle state
tokens     [0]=20240520 [1]=1 (uint16) / [0]=20240801 [1]=7 (uint32), [2]=ntok
eval       [0]=20240522 v1 / 20240802 v7, [2]=examples [3]=longest example bytes
tokenizer  [0]=20240328 [1]=2 [2]=n [3]=eot; (uint8 len, bytes) x n
debug      [0]=20240327 [1]=2 [2]=B [3]=T; x,y int32; logits fp32; loss; grads fp32
========== =========================== ===================================================

The GPT / Llama / state / token / eval / tokenizer layouts are those of the reference
(train_gpt2.cu:553-667, 1462-1567; train_llama3.cu:740-867; dev/data/data_common.py:26-143;
train_gpt2.py:479-524) so files are interchangeable; the MoE magic numbers are defined here.
"""
from __future__ import annotations

import os
import struct

import numpy as np
import torch

from ..models.config import ModelConfig, llama_hidden_dim

HEADER_INTS = 256
HEADER_BYTES = HEADER_INTS * 4

GPT_MODEL_MAGIC, LLAMA_MODEL_MAGIC, MOE_MODEL_MAGIC = 20240326, 20240803, 20250301
GPT_STATE_MAGIC, LLAMA_STATE_MAGIC, MOE_STATE_MAGIC = 20240527, 20240804, 20250302
TOKENS_MAGIC_U16, TOKENS_MAGIC_U32 = 20240520, 20240801
EVAL_MAGIC_U16, EVAL_MAGIC_U32 = 20240522, 20240802
TOKENIZER_MAGIC = 20240328
DEBUG_STATE_MAGIC = 20240327

IO_CHUNK_BYTES = 32 << 20


class FormatError(ValueError):
    pass


def _new_header() -> np.ndarray:
    return np.zeros(HEADER_INTS, dtype=np.int32)


def read_header(path: str) -> np.ndarray:
    with open(path, "rb") as f:
        raw = f.read(HEADER_BYTES)
    if len(raw) != HEADER_BYTES:
        raise FormatError(f"{path}: short header")
    return np.frombuffer(raw, dtype=np.int32).copy()


# ------------------------------------------------------------------------------------- model files
def model_header(config: ModelConfig, fp32: bool = False) -> np.ndarray:
    h = _new_header()
    # what the headers cannot express must not be written: a reader would rebuild another geometry from the file
    if config.family == "llama3" and config.padded_vocab_size != config.vocab_size:
        raise FormatError("Llama model files have no padded vocabulary: padded_vocab_size must equal vocab_size")
    if config.family != "llama3" and config.hidden_dim != 4 * config.channels:
        raise FormatError("GPT-2 / MoE model files imply hidden_dim = 4 * channels")
    if config.family == "llama3":
        h[0], h[1] = LLAMA_MODEL_MAGIC, 5
        h[2:10] = [config.max_seq_len, config.vocab_size, config.num_layers, config.num_heads, config.num_kv_heads,
                   config.channels, config.hidden_dim, config.multiple_of]
        h[10] = 1 if config.tied_embeddings else 0
        h[11] = int(config.rope_theta)
        h[12] = int(config.use_scaled_rope)
        h[13] = 4
        h[14], h[15] = config.version_major, config.version_minor
        return h
    h[0] = GPT_MODEL_MAGIC if config.family == "gpt2" else MOE_MODEL_MAGIC
    h[1] = 3 if fp32 else 5
    h[2:8] = [config.max_seq_len, config.vocab_size, config.num_layers, config.num_heads, config.channels,
              config.padded_vocab_size]
    if config.family == "moe":
        h[8], h[9], h[10] = config.num_experts, config.top_k, int(round(config.capacity_factor * 100))
    return h


def config_from_model_header(h: np.ndarray, path: str = "<header>") -> tuple[ModelConfig, bool]:
    """Returns (config, payload_is_fp32)."""
    magic, version = int(h[0]), int(h[1])
    if magic in (GPT_MODEL_MAGIC, MOE_MODEL_MAGIC):
        if version not in (3, 5):
            raise FormatError(f"{path}: unsupported model version {version} (3 = fp32, 5 = bf16)")
        maxT, V, L, NH, C, Vp = (int(x) for x in h[2:8])
        kw = dict(family="gpt2", max_seq_len=maxT, vocab_size=V, padded_vocab_size=Vp, num_layers=L, num_heads=NH,
                  num_kv_heads=NH, channels=C, hidden_dim=4 * C)
        if magic == MOE_MODEL_MAGIC:
            kw.update(family="moe", num_experts=int(h[8]), top_k=int(h[9]), capacity_factor=int(h[10]) / 100.0)
        return ModelConfig(**kw), version == 3
    if magic == LLAMA_MODEL_MAGIC:
        if version != 5:
            raise FormatError(f"{path}: only bf16 Llama checkpoints (version 5) are supported; got version {version}")
        maxT, V, L, NH, NKVH, C, hidden, mult = (int(x) for x in h[2:10])
        mult = mult or 1024
        hidden = hidden or llama_hidden_dim(C, mult)
        return ModelConfig(family="llama3", max_seq_len=maxT, vocab_size=V, padded_vocab_size=V, num_layers=L, num_heads=NH,
                           num_kv_heads=NKVH, channels=C, hidden_dim=hidden, multiple_of=mult,
                           tied_embeddings=bool(h[10]), rope_theta=float(h[11]) if h[11] else 500000.0,
                           use_scaled_rope=bool(h[12]), version_major=int(h[14]), version_minor=int(h[15])), False
    raise FormatError(f"{path}: bad model magic {magic}")


def tensor_to_file(f, t: torch.Tensor) -> None:
    """Stream a (device or host) tensor to an open file in 32 MiB chunks through pinned memory."""
    flat = t.detach().reshape(-1).view(torch.uint8) if t.dtype != torch.uint8 else t.detach().reshape(-1)
    n = flat.numel()
    if n == 0:
        return
    if not flat.is_cuda:
        f.write(flat.numpy().tobytes())
        return
    bufs = [torch.empty(min(IO_CHUNK_BYTES, n), dtype=torch.uint8, pin_memory=True) for _ in range(2)]
    events = [torch.cuda.Event(), torch.cuda.Event()]
    chunks = [(o, min(IO_CHUNK_BYTES, n - o)) for o in range(0, n, IO_CHUNK_BYTES)]
    o, ln = chunks[0]
    bufs[0][:ln].copy_(flat[o:o + ln], non_blocking=True)
    events[0].record()
    for i, (o, ln) in enumerate(chunks):
        if i + 1 < len(chunks):
            o2, ln2 = chunks[i + 1]
            bufs[(i + 1) & 1][:ln2].copy_(flat[o2:o2 + ln2], non_blocking=True)
            events[(i + 1) & 1].record()
        events[i & 1].synchronize()
        f.write(bufs[i & 1][:ln].numpy().tobytes())


def file_to_tensor(f, t: torch.Tensor) -> None:
    """Fill tensor ``t`` (device or host, any dtype) with the next ``t.nbytes`` bytes of the file."""
    flat = t.reshape(-1).view(torch.uint8)
    n = flat.numel()
    for o in range(0, n, IO_CHUNK_BYTES):
        ln = min(IO_CHUNK_BYTES, n - o)
        raw = f.read(ln)
        if len(raw) != ln:
            raise FormatError("unexpected end of file")
        src = torch.frombuffer(bytearray(raw), dtype=torch.uint8)
        flat[o:o + ln].copy_(src)
    if flat.is_cuda:
        torch.cuda.synchronize()


def write_model(path: str, config: ModelConfig, params: torch.Tensor) -> None:
    """``params``: the flat parameter buffer (bf16 -> version 5, fp32 -> version 3)."""
    fp32 = params.dtype == torch.float32
    if params.numel() != config.num_parameters():
        raise FormatError("parameter buffer does not match the model configuration")
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(model_header(config, fp32).tobytes())
        tensor_to_file(f, params)
    os.replace(tmp, path)


def read_model(path: str, device="cpu", dtype=torch.bfloat16) -> tuple[ModelConfig, torch.Tensor]:
    h = read_header(path)
    config, fp32 = config_from_model_header(h, path)
    n = config.num_parameters()
    elem = 4 if fp32 else 2
    expected = HEADER_BYTES + n * elem
    actual = os.path.getsize(path)
    if actual != expected:
        raise FormatError(f"{path}: file size {actual} does not match header ({expected} bytes expected)")
    src_dtype = torch.float32 if fp32 else torch.bfloat16
    buf = torch.empty(n, dtype=src_dtype, device=device)
    with open(path, "rb") as f:
        f.seek(HEADER_BYTES)
        file_to_tensor(f, buf)
    return config, buf.to(dtype)


# ------------------------------------------------------------------------------------- state files
def state_magic(family: str) -> int:
    return {"gpt2": GPT_STATE_MAGIC, "llama3": LLAMA_STATE_MAGIC, "moe": MOE_STATE_MAGIC}[family]


def write_state(path: str, family: str, nproc: int, rank: int, step: int, m: torch.Tensor, v: torch.Tensor,
                master: torch.Tensor | None, rng_state: int, rng_state_last_update: int, shard_idx: int, sample_idx: int,
                shuffle_blob: bytes | None) -> None:
    h = _new_header()
    h[0], h[1], h[2], h[3] = state_magic(family), 1, nproc, rank
    h[4] = 1 if master is not None else 0
    h[5] = 1 if shuffle_blob else 0
    h[10] = step
    raw = bytearray(h.tobytes())
    struct.pack_into("<Q", raw, 20 * 4, rng_state & 0xFFFFFFFFFFFFFFFF)
    struct.pack_into("<Q", raw, 22 * 4, rng_state_last_update & 0xFFFFFFFFFFFFFFFF)
    struct.pack_into("<Q", raw, 30 * 4, shard_idx)
    struct.pack_into("<Q", raw, 32 * 4, sample_idx)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(bytes(raw))
        tensor_to_file(f, m)
        tensor_to_file(f, v)
        if master is not None:
            tensor_to_file(f, master)
        if shuffle_blob:
            f.write(shuffle_blob)
    os.replace(tmp, path)


def read_state(path: str, family: str, nproc: int, rank: int, m: torch.Tensor, v: torch.Tensor,
               master: torch.Tensor | None) -> dict:
    """Fills m / v / master in place and returns the scalar fields plus the loader's shuffle blob."""
    with open(path, "rb") as f:
        raw = f.read(HEADER_BYTES)
        if len(raw) != HEADER_BYTES:
            raise FormatError(f"{path}: short header")
        h = np.frombuffer(raw, dtype=np.int32)
        if h[0] != state_magic(family):
            raise FormatError(f"{path}: bad state magic {h[0]}")
        if h[1] != 1:
            raise FormatError(f"{path}: bad state version {h[1]}")
        if h[2] != nproc or h[3] != rank:
            raise FormatError(f"{path}: state written by rank {h[3]} of {h[2]}, loading as rank {rank} of {nproc}")
        use_master = bool(h[4])
        if use_master != (master is not None):
            raise FormatError(f"{path}: master-weight setting differs from the checkpoint")
        out = {
            "use_master": use_master,
            "shuffle": bool(h[5]),
            "step": int(h[10]),
            "rng_state": struct.unpack_from("<Q", raw, 20 * 4)[0],
            "rng_state_last_update": struct.unpack_from("<Q", raw, 22 * 4)[0],
            "shard_idx": struct.unpack_from("<Q", raw, 30 * 4)[0],
            "sample_idx": struct.unpack_from("<Q", raw, 32 * 4)[0],
        }
        file_to_tensor(f, m)
        file_to_tensor(f, v)
        if master is not None:
            file_to_tensor(f, master)
        out["shuffle_blob"] = f.read() if out["shuffle"] else b""
    return out


def find_max_step(output_dir: str | None) -> int:
    """Largest N such that ``DONE_%08d`` exists in the directory, or -1."""
    if not output_dir or not os.path.isdir(output_dir):
        return -1
    best = -1
    for name in os.listdir(output_dir):
        if name.startswith("DONE_"):
            try:
                best = max(best, int(name[5:]))
            except ValueError:
                pass
    return best


def checkpoint_paths(output_dir: str, step: int, rank: int) -> tuple[str, str, str]:
    return (os.path.join(output_dir, "model_%08d.bin" % step), os.path.join(output_dir, "state_%08d_%05d.bin" % (step, rank)),
            os.path.join(output_dir, "DONE_%08d" % step))


# ------------------------------------------------------------------------------------- token shards
def write_tokens(path: str, tokens, model_desc: str = "gpt-2") -> None:
    """Token shard writer (``gpt-2`` -> uint16, ``llama-3`` -> uint32)."""
    h = _new_header()
    toks = np.asarray(tokens)
    if model_desc == "gpt-2":
        h[0], h[1] = TOKENS_MAGIC_U16, 1
        if toks.size and (toks.min() < 0 or toks.max() >= 2 ** 16):
            raise FormatError("token out of uint16 range")
        data = toks.astype(np.uint16)
    elif model_desc == "llama-3":
        h[0], h[1] = TOKENS_MAGIC_U32, 7
        data = toks.astype(np.uint32)
    else:
        raise FormatError(f"unknown model_desc {model_desc}")
    h[2] = data.size
    with open(path, "wb") as f:
        f.write(h.tobytes())
        f.write(data.tobytes())


def read_tokens(path: str) -> np.ndarray:
    h = read_header(path)
    if h[0] == TOKENS_MAGIC_U16 and h[1] == 1:
        dt = np.uint16
    elif h[0] == TOKENS_MAGIC_U32 and h[1] == 7:
        dt = np.uint32
    else:
        raise FormatError(f"{path}: bad token shard magic/version {h[0]}/{h[1]}")
    data = np.fromfile(path, dtype=dt, offset=HEADER_BYTES)
    if data.size != h[2]:
        raise FormatError(f"{path}: header says {h[2]} tokens, file holds {data.size}")
    return data


def write_evalfile(path: str, examples, model_desc: str = "gpt-2") -> None:
    """``examples``: iterable of dicts with ``label``, ``ctx_tokens``, ``ending_tokens`` (list of lists)."""
    if model_desc == "gpt-2":
        magic, version, dt = EVAL_MAGIC_U16, 1, np.uint16
    elif model_desc == "llama-3":
        magic, version, dt = EVAL_MAGIC_U32, 7, np.uint32
    else:
        raise FormatError(f"unknown model_desc {model_desc}")
    start = np.iinfo(dt).max
    item = np.dtype(dt).itemsize
    streams = []
    longest = 0
    for idx, ex in enumerate(examples):
        body = [ex["label"], len(ex["ending_tokens"]), len(ex["ctx_tokens"]), *ex["ctx_tokens"]]
        for end in ex["ending_tokens"]:
            body += [len(end), *end]
        nbytes = (3 + len(body)) * item
        if nbytes >= 2 ** 16 and dt == np.uint16:
            raise FormatError("example too long for the uint16 stream")
        stream = np.array([start, nbytes, idx, *body], dtype=dt)
        longest = max(longest, nbytes)
        streams.append(stream)
    h = _new_header()
    h[0], h[1], h[2], h[3] = magic, version, len(streams), longest
    with open(path, "wb") as f:
        f.write(h.tobytes())
        for s in streams:
            f.write(s.tobytes())


def write_tokenizer(path: str, token_bytes: list[bytes], eot_token: int) -> None:
    h = _new_header()
    h[0], h[1], h[2], h[3] = TOKENIZER_MAGIC, 2, len(token_bytes), eot_token
    with open(path, "wb") as f:
        f.write(h.tobytes())
        for b in token_bytes:
            if len(b) > 255:
                raise FormatError("token longer than 255 bytes")
            f.write(struct.pack("<B", len(b)))
            f.write(b)


# ------------------------------------------------------------------------------------- debug state
def write_debug_state(path: str, x: np.ndarray, y: np.ndarray, logits: np.ndarray, loss: float, grads: np.ndarray) -> None:
    """Reference activations for whole-model parity checks: inputs, targets, fp32 logits (B,T,V), loss
    and fp32 gradients in parameter order."""
    h = _new_header()
    h[0], h[1], h[2], h[3] = DEBUG_STATE_MAGIC, 2, x.shape[0], x.shape[1]
    with open(path, "wb") as f:
        f.write(h.tobytes())
        f.write(x.astype(np.int32).tobytes())
        f.write(y.astype(np.int32).tobytes())
        f.write(logits.astype(np.float32).tobytes())
        f.write(np.float32(loss).tobytes())
        f.write(grads.astype(np.float32).tobytes())


def read_debug_state(path: str, vocab_size: int, num_parameters: int) -> dict:
    h = read_header(path)
    if h[0] != DEBUG_STATE_MAGIC or h[1] != 2:
        raise FormatError(f"{path}: bad debug-state magic/version")
    B, T = int(h[2]), int(h[3])
    with open(path, "rb") as f:
        f.seek(HEADER_BYTES)
        x = np.frombuffer(f.read(B * T * 4), dtype=np.int32).reshape(B, T)
        y = np.frombuffer(f.read(B * T * 4), dtype=np.int32).reshape(B, T)
        logits = np.frombuffer(f.read(B * T * vocab_size * 4), dtype=np.float32).reshape(B, T, vocab_size)
        loss = float(np.frombuffer(f.read(4), dtype=np.float32)[0])
        grads = np.frombuffer(f.read(num_parameters * 4), dtype=np.float32)
    return {"B": B, "T": T, "x": x, "y": y, "logits": logits, "loss": loss, "grads": grads}
