"""Plain-PyTorch implementation of the same models over the same flat parameter layout.

Used three ways: (1) as the fp32 CPU oracle that the CUDA path is checked against (tests), (2) as
the "library baseline" on the GPU (cuBLAS GEMMs + SDPA attention through autograd, bf16) that the
hand-written kernels are timed against, and (3) under ``gloo`` on CPU to test the ZeRO / trainer
logic without a GPU. It exposes the same surface as ``models.transformer.Transformer``
(``params``, ``grads``, ``forward``, ``backward``, ``zero_grad``, ``acts['loss_acc']``).

Model math follows the reference's PyTorch scripts (train_gpt2.py:40-300: pre-LN blocks, tanh GELU,
tied embedding; train_llama3.py:60-330: RMSNorm, interleaved-pair RoPE, GQA by repeating KV heads,
SwiGLU ``down(silu(gate) * up)``).
"""
from __future__ import annotations

import math
from typing import Callable

import torch
import torch.nn.functional as F

from ..models.config import ModelConfig
from ..utils.rand import Mt19937


def rope_tables(T, HS, theta, scaled, device):
    inv = 1.0 / (theta ** (torch.arange(0, HS, 2, dtype=torch.float64) / HS))
    if scaled:
        factor, low, high, old = 8.0, 1.0, 4.0, 8192.0
        wavelen = 2 * math.pi / inv
        smooth = ((old / wavelen) - low) / (high - low)
        inv = torch.where(wavelen < old / high, inv, torch.where(wavelen > old / low, inv / factor,
                                                                 (1 - smooth) * inv / factor + smooth * inv))
    ang = torch.outer(torch.arange(T, dtype=torch.float64), inv)
    return ang.cos().float().to(device), ang.sin().float().to(device)


def apply_rope(x, cos, sin, interleaved=True):
    """x: (B, T, heads, HS); cos/sin: (T, HS/2)."""
    c, s = cos[None, :, None, :].to(x.dtype), sin[None, :, None, :].to(x.dtype)
    if interleaved:
        x0, x1 = x[..., 0::2], x[..., 1::2]
        return torch.stack([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1).flatten(-2)
    h = x.shape[-1] // 2
    x0, x1 = x[..., :h], x[..., h:]
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)


def causal_attention(q, k, v):
    """q: (B, NH, T, HS); k, v: (B, NKVH, T, HS)."""
    rep = q.shape[1] // k.shape[1]
    if rep > 1:
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
    return F.scaled_dot_product_attention(q, k, v, is_causal=True)


def moe_mlp(cfg: ModelConfig, p: dict, l: int, h: torch.Tensor, aux: list, forced_idx=None) -> torch.Tensor:
    """Top-k mixture of GELU experts with capacity dropping in (token, k) order; appends this layer's
    load-balance loss ``coef * E * sum_e density_e^2`` to ``aux``. ``h``: (B, T, C). ``forced_idx``
    (N, K) replaces the top-k choice (tests use the choices of the implementation under test, so that a
    near-tie decided differently in bf16 does not turn into an O(1) difference)."""
    B, T, C = h.shape
    E, K = cfg.num_experts, cfg.top_k
    x = h.reshape(-1, C)
    N = x.shape[0]
    probs = torch.softmax(F.linear(x.float(), p["routerw"][l].float()), dim=-1)
    if forced_idx is not None:
        top_i = forced_idx.long()
        top_p = probs.gather(1, top_i)
    else:
        top_p, top_i = probs.topk(K, dim=-1)
    w = top_p / top_p.sum(-1, keepdim=True)
    cap = int(-(-cfg.capacity_factor * K * N // E))
    cap = (cap + 7) // 8 * 8
    onehot = F.one_hot(top_i.reshape(-1), E)                       # (N*K, E) in (token, k) order
    slot = (onehot.cumsum(0) - 1)[torch.arange(N * K, device=x.device), top_i.reshape(-1)]
    keep = (slot < cap).reshape(N, K)
    out = torch.zeros_like(x)
    for e in range(E):
        sel = (top_i == e) & keep                                      # (N, K)
        tok = sel.any(-1)
        if tok.any():
            xe = x[tok]
            ye = F.linear(F.gelu(F.linear(xe, p["fcw"][l][e], p["fcb"][l][e]), approximate="tanh"), p["fcprojw"][l][e],
                          p["fcprojb"][l][e])
            we = (w * sel)[tok].sum(-1, keepdim=True).to(ye.dtype)
            out[tok] += we * ye
    density = probs.mean(0)
    aux.append(cfg.aux_loss_coef * E * (density * density).sum())
    return out.view(B, T, C)


def forward_logits(config: ModelConfig, p: dict, tokens: torch.Tensor, rope_interleaved: bool = True,
                   aux: list | None = None, forced_routing=None) -> torch.Tensor:
    """``p``: name -> parameter view (any float dtype); ``tokens``: (B, T) integer; returns (B, T, Vp) logits.
    For the MoE family the per-layer load-balance losses are appended to ``aux``."""
    cfg = config
    B, T = tokens.shape
    C, NH, NKVH, HS = cfg.channels, cfg.num_heads, cfg.num_kv_heads, cfg.head_size
    tok = tokens.long()
    llama = cfg.family == "llama3"
    x = p["wte"][tok]
    if not llama:
        x = x + p["wpe"][:T][None]
    if llama:
        cos, sin = rope_tables(T, HS, cfg.rope_theta, cfg.use_scaled_rope, x.device)

    def norm(h, w, b):
        if llama:
            hf = h.float()
            return (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + cfg.norm_eps)).to(h.dtype) * w
        return F.layer_norm(h, (C,), w, b, 1e-5)

    for l in range(cfg.num_layers):
        h = norm(x, p["ln1w"][l], None if llama else p["ln1b"][l])
        qkv = F.linear(h, p["qkvw"][l], None if llama else p["qkvb"][l]).view(B, T, NH + 2 * NKVH, HS)
        q, k, v = qkv[:, :, :NH], qkv[:, :, NH:NH + NKVH], qkv[:, :, NH + NKVH:]
        if llama:
            q, k = apply_rope(q, cos, sin, rope_interleaved), apply_rope(k, cos, sin, rope_interleaved)
        att = causal_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).reshape(B, T, C)
        x = x + F.linear(att, p["attprojw"][l], None if llama else p["attprojb"][l])
        h = norm(x, p["ln2w"][l], None if llama else p["ln2b"][l])
        if llama:
            m = F.silu(F.linear(h, p["fcw_gate"][l])) * F.linear(h, p["fcw_up"][l])
            x = x + F.linear(m, p["fcprojw"][l])
        elif cfg.family == "moe":
            x = x + moe_mlp(cfg, p, l, h, aux if aux is not None else [], None if forced_routing is None else forced_routing[l])
        else:
            m = F.gelu(F.linear(h, p["fcw"][l], p["fcb"][l]), approximate="tanh")
            x = x + F.linear(m, p["fcprojw"][l], p["fcprojb"][l])
    x = norm(x, p["lnfw"], None if llama else p["lnfb"])
    head = p["wte"] if cfg.tied_embeddings else p["lm_head"]
    return F.linear(x, head)


class TorchTransformer:
    """Autograd-backed model with the surface of ``models.transformer.Transformer``."""

    def __init__(self, config: ModelConfig, device="cpu", dtype=torch.float32, rope_interleaved=True):
        self.config = config
        self.device = torch.device(device)
        self.dtype = dtype
        self.rope_interleaved = rope_interleaved
        self.layout = config.layout()
        self.num_parameters = self.layout.total
        self.params = torch.zeros(self.num_parameters, dtype=dtype, device=self.device)
        self.grads = torch.zeros(self.num_parameters, dtype=dtype, device=self.device)
        self.p = self.layout.views(self.params)
        self.g = self.layout.views(self.grads)
        self.acts = {"loss_acc": torch.zeros(1, dtype=torch.float32, device=self.device)}
        self.param_hook = None
        self._loss = None
        self._leaf = None
        self.B = self.T = 0

    def init_weights(self, seed: int = 42) -> None:
        cfg = self.config
        rng = Mt19937(seed)
        host = torch.zeros(self.num_parameters, dtype=torch.float32)
        resid_scale = 1.0 / math.sqrt(2.0 * cfg.num_layers)
        for slot in self.layout.slots:
            spec = slot.spec
            seg = host[slot.offset: slot.offset + slot.total]
            if spec.init == "ones":
                seg.fill_(1.0)
            elif spec.init != "zeros":
                std = 0.02 * (resid_scale if spec.init == "resid" else 1.0)
                if spec.name in ("wte", "lm_head"):
                    n = cfg.vocab_size * cfg.channels
                    seg[:n] = torch.from_numpy(rng.normal_(n, 0.0, std))
                else:
                    for l in range(slot.layers):
                        seg[l * slot.size:(l + 1) * slot.size] = torch.from_numpy(rng.normal_(slot.size, 0.0, std))
        self.params.copy_(host.to(self.dtype))

    def load_parameters(self, flat: torch.Tensor) -> None:
        self.params.copy_(flat.to(self.dtype))

    def allocate(self, B, T):
        self.B, self.T = B, T

    def zero_grad(self):
        self.grads.zero_()

    def forward(self, tokens, targets=None, grad_accum_steps=1, micro_step=0, compute_dlogits=True):
        cfg = self.config
        tokens = tokens.to(self.device)
        self.B, self.T = tokens.shape
        need_grad = targets is not None and compute_dlogits
        leaf = self.params.detach().clone().requires_grad_(need_grad)
        views = self.layout.views(leaf)
        with torch.set_grad_enabled(need_grad):
            aux = []
            logits = forward_logits(cfg, views, tokens, self.rope_interleaved, aux, getattr(self, "forced_routing", None))
            self.logits = logits.detach()
            if targets is not None:
                tgt = targets.to(self.device).long().view(-1)
                lg = logits.view(-1, cfg.padded_vocab_size)[:, : cfg.vocab_size].float()
                losses = F.cross_entropy(lg, tgt, reduction="none")
                self.acts["losses"] = losses.detach()
                loss = losses.mean() / grad_accum_steps
                if micro_step == 0:
                    self.acts["loss_acc"].zero_()
                    self.acts["aux_acc"] = torch.zeros(1, dtype=torch.float32, device=self.device)
                self.acts["loss_acc"] += loss.detach()
                if aux:   # mixture of experts: the load-balance loss joins the objective, not the reported CE
                    aux_total = torch.stack(aux).sum() / grad_accum_steps
                    self.acts["aux_acc"] += aux_total.detach().float()
                    loss = loss + aux_total.to(loss.dtype)
                self._loss, self._leaf = (loss, leaf) if need_grad else (None, None)

    def backward(self, last_micro_step=True, bucket_ready: Callable | None = None):
        self._loss.backward()
        self.grads += self._leaf.grad.to(self.dtype)
        self._loss = self._leaf = None
        if last_micro_step and bucket_ready is not None:
            for l in range(self.config.num_layers - 1, -1, -1):
                bucket_ready(l)
            bucket_ready(None)

    def mean_loss(self) -> float:
        return float(self.acts["loss_acc"].item())

    def logits_view(self):
        return self.logits
