"""GPT-2 shaped transformer whose MLP is a top-k mixture of GELU experts, with expert parallelism.

The reference has no MoE model, only un-wired primitives (llmc/moe.cuh, llmc/gemm_ext.cuh:132-158,
llmc/distributed_ext.cuh:27-48, llmc/losses.cuh:522-559); the model is defined here from their
semantics:

* router ``logits = ln2 . Wr^T`` (fp32), softmax over E, top-k, weights renormalised to sum 1;
* capacity ``cap = ceil(capacity_factor * k * tokens_per_rank / E)`` rows per (source rank, expert);
  assignments beyond it are dropped in deterministic (token, k) order;
* dispatch / combine are direct row stores / loads through a table of peer pointers: rank r owns
  experts ``[r*E/P, (r+1)*E/P)`` and receives rows in ``recv[e_local][src][cap][C]``; padded slots are
  zeroed by the sender. With one process the same kernels run on a single-entry table;
* no barrier separates dispatch, expert GEMMs, return and combine: each producer publishes its blocks
  in the consumer's arrival table and each consumer waits inside its kernel for exactly what it reads
  (the grouped GEMM per M tile, i.e. per source rank; the combine for its owners);
* expert ``y = GELU(x W1^T + b1) W2^T + b2`` = two tcgen05 GEMMs per local expert on its row block;
* output ``res3 = res2 + sum_k w_k y_k``; auxiliary loss ``coef * E * sum_e density_e^2`` (density =
  mean router probability per expert on this rank) is added to the reported loss and to the router
  gradient.

Dense parameters (attention, norms, router, embeddings) are data-parallel (ZeRO like the dense
models); expert parameters are owned by one rank each and are neither reduced nor gathered.
"""
from __future__ import annotations

import os

import torch

from ..ops import elementwise as ew
from ..ops import gemm
from ..ops import moe as moe_ops
from .config import ModelConfig
from .transformer import BF16, Transformer


class LocalExchange:
    """Single-process stand-in for the expert-parallel exchange: buffers are ordinary tensors, the
    pointer tables have one entry, and the signal / wait steps are no-ops."""

    world_size, rank = 1, 0

    limit_ns = int(2e9)

    def alloc(self, numel: int, device) -> tuple[torch.Tensor, object]:
        t = torch.zeros(numel, dtype=BF16, device=device)
        return t, moe_ops.ptr_table([t])

    def arrival_table(self, entries: int, device=None):
        t = torch.zeros(entries, dtype=torch.int32, device=device)
        return t, moe_ops.ptr_table([t])

    def sync(self, tag: int) -> None:
        pass


class MoETransformer(Transformer):
    def __init__(self, config: ModelConfig, device="cuda", recompute: int = 0, exchange=None, **kw):
        if config.family != "moe":
            raise ValueError("MoETransformer needs a 'moe' configuration")
        super().__init__(config, device=device, recompute=min(int(recompute), 2), **kw)
        self.exchange = exchange if exchange is not None else LocalExchange()
        self.E, self.K = config.num_experts, config.top_k
        self.P, self.ep_rank = self.exchange.world_size, self.exchange.rank
        if self.E % self.P != 0:
            raise ValueError(f"{self.E} experts cannot be split over {self.P} expert-parallel ranks")
        self.Eloc = self.E // self.P

    # ------------------------------------------------------------------ activations
    def allocate(self, B: int, T: int) -> None:
        if (B, T) == (self.B, self.T) and self.acts is not None:
            return
        super().allocate(B, T)
        cfg, a, dev = self.config, self.acts, self.device
        N, C, H, L = B * T, cfg.channels, cfg.hidden_dim, cfg.num_layers
        E, K, P, Eloc = self.E, self.K, self.P, self.Eloc
        cap = int(-(-cfg.capacity_factor * K * N // E))
        self.cap = cap = (cap + 7) // 8 * 8
        rows = Eloc * P * cap                      # rows this rank's experts process per layer
        self.rows = rows
        f32, i32 = torch.float32, torch.int32
        a["probs"] = torch.empty(L, N, E, dtype=f32, device=dev)
        a["top_idx"] = torch.empty(L, N, K, dtype=i32, device=dev)
        a["top_w"] = torch.empty(L, N, K, dtype=f32, device=dev)
        a["slot"] = torch.empty(L, N, K, dtype=i32, device=dev)
        a["counts"] = torch.empty(L, E, dtype=i32, device=dev)
        a["density"] = torch.empty(L, E, dtype=f32, device=dev)
        a["aux_acc"] = torch.zeros(1, dtype=f32, device=dev)
        a["dw"] = torch.empty(N, K, dtype=f32, device=dev)
        a["dlogits"] = torch.empty(N, (E + 7) // 8 * 8, dtype=BF16, device=dev)
        if E % 8:
            a["routerw_pad"] = torch.zeros((E + 7) // 8 * 8, C, dtype=BF16, device=dev)
            a["grouter_pad"] = torch.zeros((E + 7) // 8 * 8, C, dtype=BF16, device=dev)
        Lg = 1 if self.recompute >= 1 else L
        a["hid_pre"] = torch.empty(L, rows, H, dtype=BF16, device=dev)
        a["hid_act"] = torch.empty(Lg, rows, H, dtype=BF16, device=dev)
        # expert outputs / input grads of this rank's experts, [e_local][source rank][slot]: peers fetch their rows from
        # here (pull-style way back), so it lives in the exchange's (symmetric) memory
        t, self.y_loc_ptrs = self.exchange.alloc(rows * C, dev)
        a["y_loc"] = t.view(rows, C)
        a["d_hid"] = torch.empty(rows, H, dtype=BF16, device=dev)
        # exchange buffers (symmetric memory when expert-parallel)
        self.recv_x, self.recv_x_ptrs = [], []
        self.back_y, self.back_y_ptrs = [], []
        for _ in range(L):
            t, p = self.exchange.alloc(rows * C, dev)
            self.recv_x.append(t.view(rows, C))
            self.recv_x_ptrs.append(p)
            t, p = self.exchange.alloc(E * cap * C, dev)
            self.back_y.append(t.view(E * cap, C))
            self.back_y_ptrs.append(p)
        t, self.recv_dy_ptrs = self.exchange.alloc(rows * C, dev)
        self.recv_dy = t.view(rows, C)
        t, self.back_dx_ptrs = self.exchange.alloc(E * cap * C, dev)
        self.back_dx = t.view(E * cap, C)
        # arrival tables: E entries per (layer, exchange), exchange 0 = tokens out, 1 = expert outputs back,
        # 2 = output gradients out, 3 = input gradients back; the values are exchange numbers that only grow
        # (2 * E entries per exchange: [0, E) block / expert flags, [E, E + P) "source rank is ready" flags of the pull-style dispatch)
        self.arrive, self.arrive_ptrs = self.exchange.arrival_table(L * 4 * 2 * E, dev)
        # pull-style dispatch: a peer-readable copy of the token rows and, per layer, the inverse slot maps
        self.dispatch_mode = os.environ.get("LLMK_MOE_DISPATCH", "pull")
        t, x_ptrs = self.exchange.alloc(N * C, dev)
        self.x_sym, self.x_sym_ptrs = t.view(N, C), x_ptrs
        t, tok_ptrs = self.exchange.alloc(2 * L * E * cap, dev)       # int32 viewed through a bf16 allocation
        self.inv_tok = t.view(torch.int32).view(L, E * cap)
        t, w_ptrs = self.exchange.alloc(2 * L * E * cap, dev)
        self.inv_w = t.view(torch.float32).view(L, E * cap)
        per_layer = E * cap * 4
        self.inv_tok_ptrs = [moe_ops.ptr_table([int(q) + l * per_layer for q in tok_ptrs]) for l in range(L)]
        self.inv_w_ptrs = [moe_ops.ptr_table([int(q) + l * per_layer for q in w_ptrs]) for l in range(L)]
        self.done = torch.zeros(1 + Eloc * P, dtype=i32, device=dev)
        # the second GEMM stores its rows straight into the source ranks' buffers when the row blocks are whole tiles
        self.scatter = (P * cap) % gemm.tile_rows() == 0 and cap >= 32 and H % 64 == 0
        # the way back: "pull" (default: plain local GEMM epilogue, the combine fetches its rows from the owners by peer
        # loads), "scatter" (the GEMM's epilogue stores into the senders' buffers) or "push" (a return kernel does)
        self.way_back = os.environ.get("LLMK_MOE_RETURN", "pull")
        if self.way_back == "scatter" and not self.scatter:
            self.way_back = "push"
        self._epoch = 0
        self.library = bool(getattr(self.exchange, "library", False))
        if self.library:
            # baseline route: a packed send buffer [E][cap][C] and a receive buffer in the collective's order
            self.a2a_send = torch.zeros(E * cap, C, dtype=BF16, device=dev)
            self.a2a_recv = torch.zeros(rows, C, dtype=BF16, device=dev)
            self.a2a_send_ptrs = moe_ops.ptr_table([self.a2a_send])

    def _dense_mlp_buffers(self) -> bool:
        return False

    # ------------------------------------------------------------------ MLP = mixture of experts
    # ---- baseline route through all_to_all_single (LibraryExchange) -------------------------------------------------
    def _library_out(self, x, idx, slot, w, counts, recv_rows, scale_by_weight):
        """rows of ``x`` -> this rank's packed [E][cap][C] send buffer -> all-to-all -> ``recv_rows`` [el][src][cap][C]."""
        E, P, cap, Eloc = self.E, self.P, self.cap, self.Eloc
        moe_ops.dispatch(self.a2a_send_ptrs, x, idx, slot, w, counts, E, cap, 0, 1, scale_by_weight=scale_by_weight)
        if Eloc == 1:
            self.exchange.all_to_all(recv_rows, self.a2a_send)           # [src][1][cap] is [1][src][cap]
        else:
            self.exchange.all_to_all(self.a2a_recv, self.a2a_send)       # [src][el][cap][C]
            recv_rows.view(Eloc, P, cap, -1).copy_(self.a2a_recv.view(P, Eloc, cap, -1).transpose(0, 1))

    def _library_back(self, y_rows, back):
        """``y_rows`` [el][src][cap][C] -> all-to-all -> ``back`` [e][cap][C] on the source ranks."""
        P, cap, Eloc = self.P, self.cap, self.Eloc
        if Eloc == 1:
            self.exchange.all_to_all(back, y_rows)
        else:
            self.a2a_recv.view(P, Eloc, cap, -1).copy_(y_rows.view(Eloc, P, cap, -1).transpose(0, 1))
            self.exchange.all_to_all(back, self.a2a_recv)

    def _mlp_forward(self, l, k, gi, ln2, res2, out):
        a, p, cfg = self.acts, self.p, self.config
        E, K, P, cap = self.E, self.K, self.P, self.cap
        moe_ops.router_fwd(ln2, p["routerw"][l], K, a["probs"][l], a["top_idx"][l], a["top_w"][l])
        moe_ops.assign_slots(a["top_idx"][l], E, cap, a["slot"][l], a["counts"][l])
        moe_ops.density(a["probs"][l], cfg.aux_loss_coef * self._loss_scale, a["density"][l], a["aux_acc"], accumulate=True)
        ep, lim = self._epoch, self.exchange.limit_ns
        r_out, r_back = (4 * l + 0) * 2 * E, (4 * l + 1) * 2 * E
        lib = self.library
        if lib:
            self._library_out(ln2, a["top_idx"][l], a["slot"][l], a["top_w"][l], a["counts"][l], self.recv_x[l], False)
        elif self.dispatch_mode == "pull":
            # the owners fetch the rows: this rank only exposes its tokens and the inverse of its slot assignment
            self.x_sym.copy_(ln2)
            moe_ops.inverse_map(self.inv_tok[l], self.inv_w[l], a["top_idx"][l], a["slot"][l], a["top_w"][l], E, cap)
            moe_ops.source_ready(self.arrive_ptrs, r_out, E, self.ep_rank, P, ep)
            moe_ops.dispatch_pull(self.recv_x[l], self.x_sym_ptrs, self.inv_tok_ptrs[l], self.inv_w_ptrs[l], cfg.channels, E, cap,
                                  self.ep_rank, P, False, self.arrive[r_out:], self.done[1:], ep, lim)
        else:
            moe_ops.dispatch_signal(self.recv_x_ptrs[l], ln2, a["top_idx"][l], a["slot"][l], a["top_w"][l], a["counts"][l], E, cap,
                                    self.ep_rank, P, False, self.arrive_ptrs, r_out, self.done[0:1], ep)
        per = P * cap
        act_l = a["hid_act"][0 if self.recompute >= 1 else l]
        # the local experts have equal row counts (P * capacity): one grouped launch per projection
        G, loc = self.Eloc, slice(self.ep_rank * self.Eloc, (self.ep_rank + 1) * self.Eloc)
        rows = slice(0, G * per)
        # every M tile of the first GEMM waits only for the source rank whose rows it loads
        gemm.gemm_nt(self.recv_x[l][rows], p["fcw"][l][loc], bias=p["fcb"][l][loc], out=act_l[rows],
                     gelu_pre_out=a["hid_pre"][l][rows], groups=G,
                     a_ready=None if lib else (self.arrive[r_out:], cap, ep, lim, ((self.ep_rank + 1) % P) * cap))
        if lib:
            gemm.gemm_nt(act_l[rows], p["fcprojw"][l][loc], bias=p["fcprojb"][l][loc], out=a["y_loc"][rows], groups=G)
            self._library_back(a["y_loc"], self.back_y[l])
            moe_ops.combine(out, res2, self.back_y[l], a["top_idx"][l], a["slot"][l], a["top_w"][l], cap)
            return
        if self.way_back == "pull":
            gemm.gemm_nt(act_l[rows], p["fcprojw"][l][loc], bias=p["fcprojb"][l][loc], out=a["y_loc"][rows], groups=G)
            moe_ops.publish(self.arrive_ptrs, r_back, E, self.ep_rank, P, ep)
            moe_ops.combine_pull(out, res2, self.y_loc_ptrs, self.back_y[l], a["top_idx"][l], a["slot"][l], a["top_w"][l], E, cap,
                                 self.ep_rank, P, self.arrive[r_back:], ep, lim)
            return
        if self.way_back == "scatter":
            # the GEMM's epilogue IS the way back: rows go to the senders' buffers, blocks are published as they complete
            gemm.gemm_grouped_scatter(act_l[rows], p["fcprojw"][l][loc], p["fcprojb"][l][loc], a["y_loc"][rows], G,
                                      self.back_y_ptrs[l], self.arrive_ptrs, r_back, self.done[1:], cap, P, self.ep_rank, ep)
        else:
            gemm.gemm_nt(act_l[rows], p["fcprojw"][l][loc], bias=p["fcprojb"][l][loc], out=a["y_loc"][rows], groups=G)
            moe_ops.return_signal(self.back_y_ptrs[l], a["y_loc"], cfg.channels, E, cap, self.ep_rank, P, self.arrive_ptrs, r_back,
                                  self.done[1:], ep)
        moe_ops.combine_wait(out, res2, self.back_y[l], a["top_idx"][l], a["slot"][l], a["top_w"][l], cap,
                             self.arrive[r_back:], E, ep, lim)

    def _mlp_backward(self, l, k, gi, dres, d_ln2, ln2):
        a, p, g, cfg = self.acts, self.p, self.g, self.config
        E, K, P, cap, C = self.E, self.K, self.P, self.cap, cfg.channels
        N = self.B * self.T
        idx, slot, w = a["top_idx"][l], a["slot"][l], a["top_w"][l]
        moe_ops.combine_dweight(dres, self.back_y[l], idx, slot, cap, dw=a["dw"])
        ep, lim = self._epoch, self.exchange.limit_ns
        r_out, r_back = (4 * l + 2) * 2 * E, (4 * l + 3) * 2 * E
        lib = self.library
        if lib:
            self._library_out(dres, idx, slot, w, a["counts"][l], self.recv_dy, True)
        elif self.dispatch_mode == "pull":
            self.x_sym.copy_(dres)
            moe_ops.source_ready(self.arrive_ptrs, r_out, E, self.ep_rank, P, ep)
            moe_ops.dispatch_pull(self.recv_dy, self.x_sym_ptrs, self.inv_tok_ptrs[l], self.inv_w_ptrs[l], C, E, cap, self.ep_rank, P,
                                  True, self.arrive[r_out:], self.done[1:], ep, lim)
        else:
            moe_ops.dispatch_signal(self.recv_dy_ptrs, dres, idx, slot, w, a["counts"][l], E, cap, self.ep_rank, P, True,
                                    self.arrive_ptrs, r_out, self.done[0:1], ep)
        per = P * cap
        act_l = a["hid_act"][0 if self.recompute >= 1 else l]
        G, loc = self.Eloc, slice(self.ep_rank * self.Eloc, (self.ep_rank + 1) * self.Eloc)
        rows = slice(0, G * per)
        dy, x, d_hid = self.recv_dy[rows], self.recv_x[l][rows], a["d_hid"][rows]
        if self.recompute >= 1:
            ew.gelu_fwd(a["hid_pre"][l][rows], out=act_l[rows])
        # the first consumer of dy waits tile by tile for its source ranks; the products after it find dy complete
        gemm.gemm_nn(dy, p["fcprojw"][l][loc], out=d_hid, dgelu_of=a["hid_pre"][l][rows], groups=G,
                     a_ready=None if lib else (self.arrive[r_out:], cap, ep, lim, ((self.ep_rank + 1) % P) * cap))
        # weight and bias gradients of all local experts: one grouped launch per projection
        gemm.gemm_tn(dy, act_l[rows], out=g["fcprojw"][l][loc], accumulate=True, groups=G, dbias=g["fcprojb"][l][loc])
        gemm.gemm_tn(d_hid, x, out=g["fcw"][l][loc], accumulate=True, groups=G, dbias=g["fcb"][l][loc])
        fused_back = self.way_back == "scatter" and not lib
        if fused_back:
            gemm.gemm_grouped_scatter(d_hid, p["fcw"][l][loc], None, a["y_loc"][rows], G, self.back_dx_ptrs, self.arrive_ptrs, r_back,
                                      self.done[1:], cap, P, self.ep_rank, ep, nn=True)
        else:
            gemm.gemm_nn(d_hid, p["fcw"][l][loc], out=a["y_loc"][rows], groups=G)
        if lib:
            self._library_back(a["y_loc"], self.back_dx)
            moe_ops.combine(d_ln2, None, self.back_dx, idx, slot, None, cap)
        elif self.way_back == "pull":
            moe_ops.publish(self.arrive_ptrs, r_back, E, self.ep_rank, P, ep)
            moe_ops.combine_pull(d_ln2, None, self.y_loc_ptrs, None, idx, slot, None, E, cap, self.ep_rank, P, self.arrive[r_back:],
                                 ep, lim)
        else:
            if not fused_back:
                moe_ops.return_signal(self.back_dx_ptrs, a["y_loc"], C, E, cap, self.ep_rank, P, self.arrive_ptrs, r_back,
                                      self.done[1:], ep)
            moe_ops.combine_wait(d_ln2, None, self.back_dx, idx, slot, None, cap, self.arrive[r_back:], E, ep, lim)
        # router: gradient through the renormalised top-k weights plus the load-balance term
        aux_scale = cfg.aux_loss_coef * E * 2.0 / N * self._loss_scale
        dlog = moe_ops.router_bwd(a["probs"][l], idx, w, a["dw"], slot, a["density"][l], aux_scale, dlogits=a["dlogits"])
        if E % 8 == 0:
            gemm.gemm_tn(dlog, ln2, out=g["routerw"][l], accumulate=True)
            gemm.gemm_nn(dlog, p["routerw"][l], out=d_ln2, add=d_ln2)
        else:
            # expert counts that are not a multiple of 8: the same tcgen05 GEMMs on a router matrix padded with zero
            # rows up to the next multiple of 8 (dlogits is already that wide, with zero columns)
            wr_pad, gr_pad = a["routerw_pad"], a["grouter_pad"]
            wr_pad[:E].copy_(p["routerw"][l])
            gemm.gemm_tn(dlog, ln2, out=gr_pad)
            ew.add(g["routerw"][l], gr_pad[:E], out=g["routerw"][l])
            gemm.gemm_nn(dlog, wr_pad, out=d_ln2, add=d_ln2)

    # ------------------------------------------------------------------ forward wrapper: aux-loss bookkeeping
    def forward(self, tokens, targets=None, grad_accum_steps: int = 1, micro_step: int = 0, compute_dlogits: bool = True):
        self.allocate(*tokens.shape)
        self._epoch += 1          # number of this micro-step's exchanges (forward and backward)
        self._loss_scale = 1.0 / grad_accum_steps
        if micro_step == 0:
            self.acts["aux_acc"].zero_()
        super().forward(tokens, targets, grad_accum_steps, micro_step, compute_dlogits)
        if targets is not None:
            # reported loss = cross-entropy + auxiliary load-balance loss (both already scaled by 1/accum)
            self.acts["loss_total"] = self.acts["loss_acc"] + self.acts["aux_acc"]

    def mean_loss(self) -> float:
        return float(self.acts["loss_acc"].item())

    def aux_loss(self) -> float:
        return float(self.acts["aux_acc"].item())
