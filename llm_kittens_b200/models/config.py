"""Model configurations, descriptor parsing and flat parameter layouts.

One :class:`ModelConfig` covers the three families the framework trains:

* ``gpt2`` - GPT-2 / GPT-3 shaped decoders (LayerNorm with bias, learned positions, tanh-GELU MLP,
  MHA, tied embedding / LM head). Descriptors ``dN``, ``gpt2:dN``, ``gpt3:cN``
  (reference train_gpt2.cu:669-734).
* ``llama3`` - Llama-3 shaped decoders (RMSNorm, RoPE, GQA, SwiGLU, no biases). Descriptors
  ``llama3:1B``, ``llama3:8B``, ``llama3.1:8B`` (reference train_llama3.cu:583-629) plus
  ``llama3.2:1B`` (tied embeddings, 32 query / 8 KV heads of size 64).
* ``moe`` - GPT-2 block whose MLP is a top-k mixture of GELU experts. Descriptor
  ``moe:dN[:eE][:kK]`` (``moe:d24`` is the GPT-2-medium shaped 8-expert top-2 model).

The parameter tensors of a model are stored in ONE flat bf16 buffer in a fixed order, each tensor
stacked over layers ``(L, ...)``; that order is also the order in the ``.bin`` checkpoints.
"""
from __future__ import annotations

from dataclasses import dataclass, replace


@dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: tuple          # per-layer shape
    layered: bool         # stacked over num_layers?
    decay: bool           # weight decay applies (2-D tensors)
    init: str             # "normal" | "resid" (normal * 1/sqrt(2L)) | "ones" | "zeros"
    expert: bool = False  # expert-parallel tensor (leading expert dimension inside the layer shape)

    def layers(self, L: int) -> int:
        return L if self.layered else 1

    def per_layer_size(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


@dataclass(frozen=True)
class ModelConfig:
    family: str = "gpt2"
    max_seq_len: int = 1024
    vocab_size: int = 50257
    padded_vocab_size: int = 50304
    num_layers: int = 12
    num_heads: int = 12
    num_kv_heads: int = 12
    channels: int = 768
    hidden_dim: int = 3072
    norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    use_scaled_rope: bool = False
    tied_embeddings: bool = True
    multiple_of: int = 1024
    version_major: int = 3
    version_minor: int = 0
    # mixture of experts
    num_experts: int = 0
    top_k: int = 2
    capacity_factor: float = 1.25
    aux_loss_coef: float = 0.01
    descriptor: str = ""

    @property
    def head_size(self) -> int:
        return self.channels // self.num_heads

    @property
    def qkv_width(self) -> int:
        return (self.num_heads + 2 * self.num_kv_heads) * self.head_size

    # ------------------------------------------------------------------ tensors
    def tensor_specs(self) -> list[TensorSpec]:
        C, L, H = self.channels, self.num_layers, self.hidden_dim
        Vp, T = self.padded_vocab_size, self.max_seq_len
        if self.family in ("gpt2", "moe"):
            specs = [
                TensorSpec("wte", (Vp, C), False, True, "normal"),
                TensorSpec("wpe", (T, C), False, True, "normal"),
                TensorSpec("ln1w", (C,), True, False, "ones"),
                TensorSpec("ln1b", (C,), True, False, "zeros"),
                TensorSpec("qkvw", (3 * C, C), True, True, "normal"),
                TensorSpec("qkvb", (3 * C,), True, False, "zeros"),
                TensorSpec("attprojw", (C, C), True, True, "resid"),
                TensorSpec("attprojb", (C,), True, False, "zeros"),
                TensorSpec("ln2w", (C,), True, False, "ones"),
                TensorSpec("ln2b", (C,), True, False, "zeros"),
            ]
            if self.family == "gpt2":
                specs += [
                    TensorSpec("fcw", (H, C), True, True, "normal"),
                    TensorSpec("fcb", (H,), True, False, "zeros"),
                    TensorSpec("fcprojw", (C, H), True, True, "resid"),
                    TensorSpec("fcprojb", (C,), True, False, "zeros"),
                ]
            else:
                E = self.num_experts
                specs += [
                    TensorSpec("fcw", (E, H, C), True, True, "normal", expert=True),
                    TensorSpec("fcb", (E, H), True, False, "zeros", expert=True),
                    TensorSpec("fcprojw", (E, C, H), True, True, "resid", expert=True),
                    TensorSpec("fcprojb", (E, C), True, False, "zeros", expert=True),
                ]
            specs += [
                TensorSpec("lnfw", (C,), False, False, "ones"),
                TensorSpec("lnfb", (C,), False, False, "zeros"),
            ]
            if self.family == "moe":
                specs.append(TensorSpec("routerw", (self.num_experts, C), True, True, "normal"))
            return specs
        if self.family == "llama3":
            specs = [
                TensorSpec("wte", (Vp, C), False, True, "normal"),
                TensorSpec("ln1w", (C,), True, False, "ones"),
                TensorSpec("qkvw", (self.qkv_width, C), True, True, "normal"),
                TensorSpec("attprojw", (C, C), True, True, "resid"),
                TensorSpec("ln2w", (C,), True, False, "ones"),
                TensorSpec("fcw_up", (H, C), True, True, "normal"),
                TensorSpec("fcw_gate", (H, C), True, True, "normal"),
                TensorSpec("fcprojw", (C, H), True, True, "resid"),
                TensorSpec("lnfw", (C,), False, False, "ones"),
            ]
            if not self.tied_embeddings:
                specs.append(TensorSpec("lm_head", (Vp, C), False, True, "normal"))
            return specs
        raise ValueError(f"unknown model family {self.family}")

    def layout(self) -> "ParamLayout":
        return ParamLayout(self)

    def num_parameters(self) -> int:
        return self.layout().total


@dataclass
class TensorSlot:
    spec: TensorSpec
    index: int
    offset: int      # element offset of layer 0 in the flat buffer
    layers: int
    size: int        # per-layer elements

    @property
    def total(self) -> int:
        return self.size * self.layers


class ParamLayout:
    """Element offsets of every tensor of a model in the flat parameter / gradient buffers."""

    def __init__(self, config: ModelConfig):
        self.config = config
        self.slots: list[TensorSlot] = []
        off = 0
        for i, spec in enumerate(config.tensor_specs()):
            slot = TensorSlot(spec, i, off, spec.layers(config.num_layers), spec.per_layer_size())
            if off % 64 != 0:
                raise ValueError(f"tensor {spec.name} would start at element {off}, not 128-byte aligned")
            self.slots.append(slot)
            off += slot.total
        self.total = off
        self.by_name = {s.spec.name: s for s in self.slots}

    def __getitem__(self, name: str) -> TensorSlot:
        return self.by_name[name]

    def views(self, flat) -> dict:
        """Dict name -> view of ``flat`` shaped (L, *shape) for layered tensors, (*shape) otherwise."""
        out = {}
        for s in self.slots:
            v = flat[s.offset: s.offset + s.total]
            out[s.spec.name] = v.view(s.layers, *s.spec.shape) if s.spec.layered else v.view(*s.spec.shape)
        return out


# ---------------------------------------------------------------------------------- descriptors
_GPT2_DEPTHS = {6: (384, 6), 12: (768, 12), 24: (1024, 16), 36: (1280, 20), 48: (1600, 25), 60: (1920, 30),
                72: (2880, 30), 84: (3456, 36)}
_GPT3_CHANNELS = {384: (6, 64), 768: (12, 64), 1024: (24, 64), 1536: (24, 96), 2048: (24, 128), 2560: (32, 80),
                  4096: (32, 128), 5120: (40, 128), 12288: (96, 128)}


def _gpt2(depth: int, descriptor: str) -> ModelConfig:
    if depth not in _GPT2_DEPTHS:
        raise ValueError(f"Unsupported GPT-2 depth: {depth}")
    C, NH = _GPT2_DEPTHS[depth]
    return ModelConfig(family="gpt2", max_seq_len=1024, num_layers=depth, num_heads=NH, num_kv_heads=NH, channels=C,
                       hidden_dim=4 * C, descriptor=descriptor)


def _gpt3(channels: int, descriptor: str) -> ModelConfig:
    if channels not in _GPT3_CHANNELS:
        raise ValueError(f"Unsupported GPT-3 channels: {channels}")
    depth, hs = _GPT3_CHANNELS[channels]
    return ModelConfig(family="gpt2", max_seq_len=2048, num_layers=depth, num_heads=channels // hs,
                       num_kv_heads=channels // hs, channels=channels, hidden_dim=4 * channels, descriptor=descriptor)


_LLAMA = {
    "llama3:1B": dict(max_seq_len=2048, num_layers=16, num_heads=16, num_kv_heads=8, channels=2048, hidden_dim=8192,
                      tied_embeddings=False, version_minor=0),
    "llama3:8B": dict(max_seq_len=2048, num_layers=32, num_heads=32, num_kv_heads=8, channels=4096, hidden_dim=14336,
                      tied_embeddings=False, version_minor=0),
    "llama3.1:8B": dict(max_seq_len=8192, num_layers=32, num_heads=32, num_kv_heads=8, channels=4096, hidden_dim=14336,
                        tied_embeddings=False, use_scaled_rope=True, version_minor=1),
    "llama3.2:1B": dict(max_seq_len=2048, num_layers=16, num_heads=32, num_kv_heads=8, channels=2048, hidden_dim=8192,
                        tied_embeddings=True, version_minor=2),
}


def config_from_descriptor(descriptor: str) -> ModelConfig:
    """Parse ``dN`` / ``gpt2:dN`` / ``gpt3:cN`` / ``llama3:*`` / ``moe:dN[:eE][:kK]``."""
    d = descriptor.strip()
    try:
        if d.startswith("gpt2:d"):
            return _gpt2(int(d[6:]), d)
        if d.startswith("gpt3:c"):
            return _gpt3(int(d[6:]), d)
        if d.startswith("moe:d"):
            parts = d.split(":")
            base = _gpt2(int(parts[1][1:]), d)
            E, K = 8, 2
            for p in parts[2:]:
                if p.startswith("e"):
                    E = int(p[1:])
                elif p.startswith("k"):
                    K = int(p[1:])
            return replace(base, family="moe", num_experts=E, top_k=K)
        if len(d) > 1 and d[0] == "d":
            return _gpt2(int(d[1:]), d)
    except ValueError as e:
        if "Unsupported" in str(e):
            raise
        raise ValueError(f"Unsupported model descriptor: {descriptor}") from None
    if d in _LLAMA:
        kw = dict(_LLAMA[d])
        return ModelConfig(family="llama3", vocab_size=128256, padded_vocab_size=128256, descriptor=d, **kw)
    raise ValueError(f"Unsupported model descriptor: {descriptor}")


def llama_hidden_dim(channels: int, multiple_of: int = 1024, ffn_dim_multiplier: float = 1.3) -> int:
    """SwiGLU width rule of Llama-3: 4C * 2/3, scaled, rounded up to ``multiple_of``."""
    h = int(2 * (4 * channels) / 3)
    h = int(ffn_dim_multiplier * h)
    return multiple_of * ((h + multiple_of - 1) // multiple_of)
