"""Decoder-only transformer with an explicit forward / backward schedule over flat buffers.

There is no autograd in the hot path: parameters and gradients are two flat bf16 buffers (tensor
order and stacking as in the checkpoint files), activations are preallocated per layer, and
``forward`` / ``backward`` issue the hand-written kernels of ``ops/`` in a fixed order on the current
CUDA stream. The schedule plays the role of gpt2_forward / gpt2_backward_and_reduce
(reference train_gpt2.cu:800-915, 948-1167) and llama_forward / llama_backward_and_reduce
(train_llama3.cu:922-998, 1023-1182) with these differences:

* residual adds are fused into the epilogue of the projection GEMMs (``out = residual + x W^T + b``),
  the GELU and its derivative into the MLP GEMM epilogues; QKV stays packed ``(B, T, (NH+2*NKVH)*HS)``
  end to end, so there are no permute / unpermute kernels;
* every reduction over tokens (bias, norm weight, embedding gradients) is deterministic and runs on
  the GPU - no host-side bucket sort;
* ``recompute``: 0 keeps all activations, 1 recomputes the GELU output, 2 also the normalised
  activations (for both families), 3 keeps only each block's input and re-runs the block forward
  inside backward (activation checkpointing);
* a ``bucket_ready`` callback fires when a block's gradients are final (last micro-step), which is
  where data-parallel reduction of that bucket starts.
"""
from __future__ import annotations

import os

import math
from typing import Callable

import torch

from ..ops import attention as attn_ops
from ..ops import classifier as cls_ops
from ..ops import elementwise as ew
from ..ops import gemm
from ..ops import norm as norm_ops
from ..utils.rand import Mt19937
from .config import ModelConfig

BF16 = torch.bfloat16


class Transformer:
    def __init__(self, config: ModelConfig, device: str | torch.device = "cuda", recompute: int = 1,
                 rope_interleaved: bool = True):
        if config.family not in ("gpt2", "llama3") and type(self) is Transformer:
            raise ValueError("Transformer handles the dense families; use models.moe.MoETransformer for 'moe'")
        self.config = config
        self.device = torch.device(device)
        self.recompute = int(recompute)
        self.rope_interleaved = rope_interleaved
        self.layout = config.layout()
        self.num_parameters = self.layout.total
        self.params = torch.zeros(self.num_parameters, dtype=BF16, device=self.device)
        self.grads = torch.zeros(self.num_parameters, dtype=BF16, device=self.device)
        self.p = self.layout.views(self.params)
        self.g = self.layout.views(self.grads)
        self.B = self.T = 0
        self.acts = None
        self.is_llama = config.family == "llama3"
        # ZeRO-3 style hooks: called with the layer index right before a block's parameters are used
        self.param_hook: Callable[[int | None, str], None] | None = None
        # sharded-gradient communication: called before a block's backward writes its gradients, and
        # block buckets are handed over after every micro-step instead of only the last one
        self.grad_hook: Callable[[int], None] | None = None
        self.reduce_every_micro_step = False
        # Bandwidth-shaped side work of the backward pass (bias-gradient column sums, the D = rowsum(dO * O) pre-pass of
        # attention) runs on a second stream beside the GEMMs that follow it: those are tensor-bound and leave most of
        # the memory system idle. LLMK_SIDE_STREAM=0 keeps everything on one stream.
        self.side = None
        if self.device.type == "cuda" and os.environ.get("LLMK_SIDE_STREAM", "1") != "0":
            self.side = torch.cuda.Stream(device=self.device)
        self._side_busy = False

    # ------------------------------------------------------------------ parameters
    def init_weights(self, seed: int = 42) -> None:
        """N(0, 0.02) from an MT19937 stream in tensor order, residual projections scaled by
        1/sqrt(2L), norm weights 1, biases 0; only the first ``vocab_size`` rows of the embeddings are
        drawn (the padding rows stay 0). Same recipe as the reference (train_gpt2.cu:736-796)."""
        cfg = self.config
        rng = Mt19937(seed)
        host = torch.zeros(self.num_parameters, dtype=torch.float32)
        resid_scale = 1.0 / math.sqrt(2.0 * cfg.num_layers)
        for slot in self.layout.slots:
            spec = slot.spec
            seg = host[slot.offset: slot.offset + slot.total]
            if spec.init == "ones":
                seg.fill_(1.0)
            elif spec.init == "zeros":
                pass
            else:
                std = 0.02 * (resid_scale if spec.init == "resid" else 1.0)
                if spec.name in ("wte", "lm_head"):
                    n = cfg.vocab_size * cfg.channels
                    seg[:n] = torch.from_numpy(rng.normal_(n, 0.0, std))
                else:
                    for l in range(slot.layers):
                        seg[l * slot.size:(l + 1) * slot.size] = torch.from_numpy(rng.normal_(slot.size, 0.0, std))
        self.params.copy_(host.to(BF16))

    def load_parameters(self, flat: torch.Tensor) -> None:
        self.params.copy_(flat.to(BF16))

    # ------------------------------------------------------------------ activations
    def allocate(self, B: int, T: int) -> None:
        if (B, T) == (self.B, self.T) and self.acts is not None:
            return
        cfg = self.config
        if T % 64 != 0:
            raise ValueError("sequence length must be a multiple of 64")
        if T > cfg.max_seq_len:
            raise ValueError(f"sequence length {T} exceeds the model's maximum {cfg.max_seq_len}")
        self.B, self.T = B, T
        BT, C, L, H = B * T, cfg.channels, cfg.num_layers, cfg.hidden_dim
        NH, QW, Vp = cfg.num_heads, cfg.qkv_width, cfg.padded_vocab_size
        dev = self.device
        r = self.recompute
        Lk = 1 if r >= 3 else L        # per-layer activations kept for backward
        Ln = 1 if r >= 2 else L        # normalised activations
        Lg = 1 if r >= 1 else L        # GELU / SwiGLU output

        def e(*shape, dtype=BF16):
            return torch.empty(*shape, dtype=dtype, device=dev)

        a = {}
        a["encoded"] = e(BT, C)
        a["block_in"] = e(L, BT, C) if r >= 3 else None   # inputs of every block (checkpointing)
        a["ln1"] = e(Ln, BT, C)
        a["ln1_rstd"] = e(Lk, BT, dtype=torch.float32)
        a["ln2"] = e(Ln, BT, C)
        a["ln2_rstd"] = e(Lk, BT, dtype=torch.float32)
        if not self.is_llama:
            a["ln1_mean"] = e(Lk, BT, dtype=torch.float32)
            a["ln2_mean"] = e(Lk, BT, dtype=torch.float32)
            a["lnf_mean"] = e(BT, dtype=torch.float32)
        a["qkv"] = e(Lk, BT, QW)
        a["atty"] = e(Lk, BT, C)
        a["lse"] = e(Lk, B, NH, T, dtype=torch.float32)
        a["res2"] = e(Lk, BT, C)
        a["res3"] = e(Lk, BT, C)
        if self.is_llama:
            a["up"] = e(Lk, BT, H)
            a["gate"] = e(Lk, BT, H)
            a["act"] = e(Lg, BT, H)
        elif self._dense_mlp_buffers():
            a["fch"] = e(Lk, BT, H)
            a["act"] = e(Lg, BT, H)
        a["lnf"] = e(BT, C)
        a["lnf_rstd"] = e(BT, dtype=torch.float32)
        a["logits"] = e(BT, Vp)
        a["losses"] = e(BT, dtype=torch.float32)
        # backward scratch
        a["dresidual"] = e(BT, C)
        a["d_btc"] = e(BT, C)
        a["d_wide"] = e(BT, max(H, QW))
        a["d_wide2"] = e(BT, H) if self.is_llama else None
        a["dvec"] = e(B, NH, T, dtype=torch.float32)
        a["loss_acc"] = torch.zeros(1, dtype=torch.float32, device=dev)
        if self.is_llama:
            a["rope"] = ew.rope_tables(T, cfg.head_size, cfg.rope_theta, cfg.use_scaled_rope, device=dev)
        self.acts = a
        self.tokens = torch.zeros(B, T, dtype=torch.int32, device=dev)
        self.targets = torch.zeros(B, T, dtype=torch.int32, device=dev)

    def _dense_mlp_buffers(self) -> bool:
        """Whether the dense-MLP activation buffers are needed (a subclass with another MLP says no)."""
        return True

    def activation_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.acts.values() if isinstance(t, torch.Tensor))

    # ------------------------------------------------------------------ building blocks
    def _norm_fwd(self, x, w, b, out, mean, rstd):
        if self.is_llama:
            norm_ops.rmsnorm_fwd(x, w, self.config.norm_eps, out=out, rstd=rstd)
        else:
            norm_ops.layernorm_fwd(x, w, b, out=out, mean=mean, rstd=rstd)

    def _norm_bwd(self, dinp, dw, db, dout, x, w, mean, rstd, accumulate=True):
        if self.is_llama:
            norm_ops.rmsnorm_bwd(dinp, dw, dout, x, w, rstd, accumulate_dinp=accumulate)
        else:
            norm_ops.layernorm_bwd(dinp, dw, db, dout, x, w, mean, rstd, accumulate_dinp=accumulate)

    def _fork(self, fn) -> None:
        """Run ``fn`` on the side stream, ordered after everything queued so far on the current stream."""
        if self.side is None:
            fn()
            return
        ev = torch.cuda.Event()
        ev.record()
        self.side.wait_event(ev)
        with torch.cuda.stream(self.side):
            fn()
        self._side_busy = True

    def _join(self) -> None:
        """The current stream waits for the side work: before anything overwrites what that work reads, and before its
        results (bias gradients, D) are used."""
        if self._side_busy:
            torch.cuda.current_stream().wait_stream(self.side)
            self._side_busy = False

    def _dweight(self, dout: torch.Tensor, inp: torch.Tensor, gw: torch.Tensor, gb: torch.Tensor | None) -> None:
        """``gw += dout^T inp`` and, for a layer with a bias, ``gb += column sums of dout``: one launch when the
        weight-gradient GEMM can sum its A tiles on the way, else the column sums run on the side stream."""
        if gb is None:
            gemm.gemm_tn(dout, inp, out=gw, accumulate=True)
        elif gemm.fused_dbias_available():
            gemm.gemm_tn(dout, inp, out=gw, accumulate=True, dbias=gb)
        else:
            self._fork(lambda: ew.dbias(gb, dout, accumulate=True))
            gemm.gemm_tn(dout, inp, out=gw, accumulate=True)

    def _fused_rope(self) -> bool:
        """Llama with interleaved pairs on the tcgen05 attention path: RoPE lives in the QKV projection's epilogue and
        its backward in the output tiles of the attention backward kernels; no separate pass over QKV or dQKV. The
        half-split pair convention and sequence lengths that fall back to the warp-level attention kernels keep the
        stand-alone rotation kernel."""
        return (self.is_llama and self.rope_interleaved and attn_ops.fused_rope_available(self.T)
                and self.config.head_size in (64, 128) and os.environ.get("LLMK_FUSED_ROPE", "1") != "0")

    def _idx(self, l: int, kind: str) -> int:
        """Index of layer ``l`` in a per-layer activation given the recompute level."""
        r = self.recompute
        if kind == "k":
            return 0 if r >= 3 else l
        if kind == "n":
            return 0 if r >= 2 else l
        return 0 if r >= 1 else l

    def _block_forward(self, l: int, x: torch.Tensor, phase: str = "forward") -> torch.Tensor:
        """One transformer block; ``x`` is the residual stream input (BT, C); returns the output view.
        ``phase`` is handed to the parameter hook: ``backward`` when the block is re-run for recomputation."""
        cfg, a, p = self.config, self.acts, self.p
        B, T = self.B, self.T
        k, n, gi = self._idx(l, "k"), self._idx(l, "n"), self._idx(l, "g")
        if self.param_hook:
            self.param_hook(l, phase)
        ln1, ln2 = a["ln1"][n], a["ln2"][n]
        mean1 = None if self.is_llama else a["ln1_mean"][k]
        mean2 = None if self.is_llama else a["ln2_mean"][k]
        self._norm_fwd(x, p["ln1w"][l], None if self.is_llama else p["ln1b"][l], ln1, mean1, a["ln1_rstd"][k])
        qkv = a["qkv"][k]
        if self._fused_rope():
            # RoPE in the projection's epilogue: q and k are rotated while still fp32 accumulators
            gemm.gemm_qkv_rope(ln1, p["qkvw"][l], a["rope"], T, (cfg.num_heads + cfg.num_kv_heads) * cfg.head_size, cfg.head_size,
                               out=qkv)
        else:
            gemm.gemm_nt(ln1, p["qkvw"][l], bias=None if self.is_llama else p["qkvb"][l], out=qkv)
            if self.is_llama:
                ew.rope_qk_(qkv, a["rope"], B, T, cfg.num_heads, cfg.num_kv_heads, cfg.head_size, self.rope_interleaved)
        attn_ops.attention_fwd(qkv, B, T, cfg.num_heads, cfg.num_kv_heads, cfg.head_size, out=a["atty"][k], lse=a["lse"][k])
        res2 = a["res2"][k]
        gemm.gemm_nt(a["atty"][k], p["attprojw"][l], bias=None if self.is_llama else p["attprojb"][l], out=res2, add=x)
        self._norm_fwd(res2, p["ln2w"][l], None if self.is_llama else p["ln2b"][l], ln2, mean2, a["ln2_rstd"][k])
        self._mlp_forward(l, k, gi, ln2, res2, a["res3"][k])
        return a["res3"][k]

    def _mlp_forward(self, l: int, k: int, gi: int, ln2: torch.Tensor, res2: torch.Tensor, out: torch.Tensor) -> None:
        """``out = res2 + MLP(ln2)`` for block ``l`` (dense GELU MLP or SwiGLU)."""
        a, p = self.acts, self.p
        act = a["act"][gi]
        if self.is_llama:
            # up, gate and silu(gate) * up from one launch when the fused-epilogue kernel takes the shape
            if os.environ.get("LLMK_FUSED_SWIGLU", "1") == "0" or not gemm.gemm_swiglu(ln2, p["fcw_up"][l], p["fcw_gate"][l], act,
                                                                                   a["up"][k], a["gate"][k]):
                gemm.gemm_nt(ln2, p["fcw_up"][l], out=a["up"][k])
                gemm.gemm_nt(ln2, p["fcw_gate"][l], out=a["gate"][k])
                ew.swiglu_fwd(a["gate"][k], a["up"][k], out=act)
            gemm.gemm_nt(act, p["fcprojw"][l], out=out, add=res2)
        else:
            gemm.gemm_nt(ln2, p["fcw"][l], bias=p["fcb"][l], out=act, gelu_pre_out=a["fch"][k])
            gemm.gemm_nt(act, p["fcprojw"][l], bias=p["fcprojb"][l], out=out, add=res2)

    def _mlp_backward(self, l: int, k: int, gi: int, dres: torch.Tensor, d_ln2: torch.Tensor, ln2: torch.Tensor) -> None:
        """Backward of ``res3 = res2 + MLP(ln2)``: given ``dres`` = d(res3), accumulate the MLP weight
        gradients and write d(ln2) into ``d_ln2`` (the residual path keeps ``dres`` as is)."""
        a, p, g = self.acts, self.p, self.g
        BT, H = self.B * self.T, self.config.hidden_dim
        act = a["act"][gi]
        if self.is_llama:
            if 1 <= self.recompute < 3:
                ew.swiglu_fwd(a["gate"][k], a["up"][k], out=act)
            d_act = a["d_wide"].view(-1)[: BT * H].view(BT, H)
            gemm.gemm_nn(dres, p["fcprojw"][l], out=d_act)
            gemm.gemm_tn(dres, act, out=g["fcprojw"][l], accumulate=True)
            d_gate, d_up = a["d_wide2"], d_act
            ew.swiglu_bwd(d_act, a["gate"][k], a["up"][k], dgate=d_gate, dup=d_up)
            gemm.gemm_nn(d_up, p["fcw_up"][l], out=d_ln2)
            gemm.gemm_nn(d_gate, p["fcw_gate"][l], out=d_ln2, add=d_ln2)
            gemm.gemm_tn(d_up, ln2, out=g["fcw_up"][l], accumulate=True)
            gemm.gemm_tn(d_gate, ln2, out=g["fcw_gate"][l], accumulate=True)
        else:
            if 1 <= self.recompute < 3:
                ew.gelu_fwd(a["fch"][k], out=act)
            d_fch = a["d_wide"].view(-1)[: BT * H].view(BT, H)
            self._dweight(dres, act, g["fcprojw"][l], g["fcprojb"][l])
            gemm.gemm_nn(dres, p["fcprojw"][l], out=d_fch, dgelu_of=a["fch"][k])
            gemm.gemm_nn(d_fch, p["fcw"][l], out=d_ln2)
            self._dweight(d_fch, ln2, g["fcw"][l], g["fcb"][l])

    # ------------------------------------------------------------------ forward
    def forward(self, tokens: torch.Tensor, targets: torch.Tensor | None = None, grad_accum_steps: int = 1,
                micro_step: int = 0, compute_dlogits: bool = True) -> None:
        """Runs the forward pass on (B, T) int32 token tensors (device or pinned host). With targets,
        the per-token losses land in ``acts['losses']``, their mean (scaled by 1/grad_accum_steps and
        accumulated over micro-steps) in ``acts['loss_acc']``, and - when ``compute_dlogits`` - the
        logits buffer is overwritten by dlogits, ready for :meth:`backward`."""
        cfg, a, p = self.config, self.acts, self.p
        B, T = tokens.shape
        self.allocate(B, T)
        a = self.acts
        self.tokens.copy_(tokens, non_blocking=True)
        if self.param_hook:
            self.param_hook(None, "forward")
        ew.encoder_fwd(self.tokens, p["wte"], None if self.is_llama else p["wpe"], out=a["encoded"].view(B, T, -1))
        x = a["encoded"]
        for l in range(cfg.num_layers):
            if self.recompute >= 3:
                a["block_in"][l].copy_(x)
            x = self._block_forward(l, x)
        if self.param_hook:
            self.param_hook(None, "head")
        self._norm_fwd(x, p["lnfw"], None if self.is_llama else p["lnfb"], a["lnf"], None if self.is_llama else a["lnf_mean"],
                       a["lnf_rstd"])
        self._final_residual = x
        head = p["wte"] if cfg.tied_embeddings else p["lm_head"]
        gemm.gemm_nt(a["lnf"], head, out=a["logits"])
        if targets is not None:
            self.targets.copy_(targets, non_blocking=True)
            BT = B * T
            dloss = 1.0 / (BT * grad_accum_steps)
            if micro_step == 0:
                a["loss_acc"].zero_()
            cls_ops.fused_classifier(a["logits"], self.targets.view(-1), cfg.vocab_size, dloss, losses=a["losses"],
                                     write_dlogits=compute_dlogits)
            cls_ops.sum_scaled(a["loss_acc"], a["losses"], dloss, accumulate=True)

    # ------------------------------------------------------------------ backward
    def zero_grad(self) -> None:
        self.grads.zero_()

    def backward(self, last_micro_step: bool = True, bucket_ready: Callable[[int | None], None] | None = None) -> None:
        """Backward of the last :meth:`forward` (which must have written dlogits). Gradients are
        accumulated (``+=``) into ``self.grads``; call :meth:`zero_grad` before the first micro-step."""
        cfg, a, p, g = self.config, self.acts, self.p, self.g
        B, T = self.B, self.T
        BT, C, H, QW = B * T, cfg.channels, cfg.hidden_dim, cfg.qkv_width
        L = cfg.num_layers
        dres, d_btc = a["dresidual"], a["d_btc"]
        if self.param_hook:
            self.param_hook(None, "head")
        head_name = "wte" if cfg.tied_embeddings else "lm_head"
        # LM head: d(lnf) and d(head weight)
        gemm.gemm_nn(a["logits"], p[head_name], out=d_btc)
        gemm.gemm_tn(a["logits"], a["lnf"], out=g[head_name], accumulate=True)
        self._norm_bwd(dres, g["lnfw"], None if self.is_llama else g["lnfb"], d_btc, self._final_residual, p["lnfw"],
                       None if self.is_llama else a["lnf_mean"], a["lnf_rstd"], accumulate=False)
        for l in range(L - 1, -1, -1):
            if self.recompute >= 3:
                x_in = a["block_in"][l]
                self._block_forward(l, x_in, phase="backward")
            else:
                x_in = a["encoded"] if l == 0 else a["res3"][l - 1]
                if self.param_hook:
                    self.param_hook(l, "backward")
            if self.grad_hook:
                self.grad_hook(l)
            k, n, gi = self._idx(l, "k"), self._idx(l, "n"), self._idx(l, "g")
            ln1, ln2 = a["ln1"][n], a["ln2"][n]
            mean1 = None if self.is_llama else a["ln1_mean"][k]
            mean2 = None if self.is_llama else a["ln2_mean"][k]
            res2 = a["res2"][k]
            # ---- MLP
            if self.recompute == 2:
                self._norm_fwd(res2, p["ln2w"][l], None if self.is_llama else p["ln2b"][l], ln2, mean2, a["ln2_rstd"][k])
            self._mlp_backward(l, k, gi, dres, d_btc, ln2)
            self._join()   # the column sums over dres are done before the norm backward adds to it
            self._norm_bwd(dres, g["ln2w"][l], None if self.is_llama else g["ln2b"][l], d_btc, res2, p["ln2w"][l], mean2,
                           a["ln2_rstd"][k], accumulate=True)
            # ---- attention
            # dO, and with 64-wide heads D = rowsum(dO * O) from the same epilogue; else D is a pass of its own on the side stream
            prep = [False]
            if (gemm.fused_drow_available(cfg.head_size) and attn_ops.fused_rope_available(T)
                    and gemm.gemm_nn(dres, p["attprojw"][l], out=d_btc, drow_of=(a["atty"][k], a["dvec"], T)) is not False):
                prep[0] = True
            else:
                gemm.gemm_nn(dres, p["attprojw"][l], out=d_btc)

                def attention_side_work():
                    prep[0] = attn_ops.attention_bwd_prep(d_btc, a["atty"][k], a["dvec"], B, T, cfg.num_heads, cfg.head_size)

                self._fork(attention_side_work)
            self._dweight(dres, a["atty"][k], g["attprojw"][l], None if self.is_llama else g["attprojb"][l])
            self._join()   # D is needed now, and the next kernel overwrites the buffer that the MLP's column sum read
            dqkv = a["d_wide"].view(-1)[: BT * QW].view(BT, QW)
            fused_rope = self._fused_rope()
            attn_ops.attention_bwd(d_btc, a["qkv"][k], a["atty"][k], a["lse"][k], B, T, cfg.num_heads, cfg.num_kv_heads,
                                   cfg.head_size, dqkv=dqkv, dvec=a["dvec"], rope=a["rope"] if fused_rope else None,
                                   prep_done=prep[0])
            if self.is_llama and not fused_rope:
                ew.rope_qk_(dqkv, a["rope"], B, T, cfg.num_heads, cfg.num_kv_heads, cfg.head_size, self.rope_interleaved,
                            inverse=True)
            if self.recompute == 2:
                self._norm_fwd(x_in, p["ln1w"][l], None if self.is_llama else p["ln1b"][l], ln1, mean1, a["ln1_rstd"][k])
            gemm.gemm_nn(dqkv, p["qkvw"][l], out=d_btc)
            self._dweight(dqkv, ln1, g["qkvw"][l], None if self.is_llama else g["qkvb"][l])
            self._join()   # bias gradients of this block are complete before its bucket is handed over
            self._norm_bwd(dres, g["ln1w"][l], None if self.is_llama else g["ln1b"][l], d_btc, x_in, p["ln1w"][l], mean1,
                           a["ln1_rstd"][k], accumulate=True)
            if (last_micro_step or self.reduce_every_micro_step) and bucket_ready is not None:
                bucket_ready(l)
        if self.param_hook:
            self.param_hook(None, "embedding")
        ew.encoder_bwd(g["wte"], None if self.is_llama else g["wpe"], dres.view(B, T, C), self.tokens)
        if last_micro_step and bucket_ready is not None:
            bucket_ready(None)

    # ------------------------------------------------------------------ conveniences
    def mean_loss(self) -> float:
        """Host value of the accumulated mean loss (synchronises)."""
        return float(self.acts["loss_acc"].item())

    def logits_view(self) -> torch.Tensor:
        return self.acts["logits"].view(self.B, self.T, -1)
