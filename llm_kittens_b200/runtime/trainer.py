"""Training step orchestration: gradient accumulation, data-parallel reduction, global-norm
clipping, AdamW on this rank's ZeRO shard, parameter all-gather, loss / norm read-back.

Plays the role of the inner loop of the reference trainers (train_gpt2.cu:2227-2316: micro-steps,
gpt2_calculate_grad_norm, gpt2_update) with these differences: the clip coefficient is computed on
the device and consumed by the AdamW kernel through a pointer (no host sync between norm and
update), one AdamW launch covers the whole shard via a segment table, and the only device-to-host
traffic per step is one small read-back of (loss, grad-norm, overflow flag) after everything has been
queued.

The optimizer has two back-ends with the same semantics: the CUDA kernels of ``ops/optim.py`` (with
stochastic rounding and optional fp32 master weights) and a PyTorch one used when the model lives on
the CPU (oracle / gloo tests).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parallel.comm import SingleProcessComm
from ..parallel.zero import ZeroPlan
from ..utils.nvtx import nvtx_range
from ..utils.rand import Xorshift


@dataclass
class StepResult:
    loss: float
    grad_norm: float
    lr: float
    skipped: bool = False


class Trainer:
    def __init__(self, model, *, zero_stage: int = 0, use_master_weights: bool = True, learning_rate: float = 3e-4,
                 weight_decay: float = 0.0, beta1: float = 0.9, beta2: float = 0.95, eps: float = 1e-8, grad_clip: float = 1.0,
                 comm=None, num_processes: int = 1, rank: int = 0, rng_state: int = 13371337):
        self.model = model
        self.device = model.device
        self.native = self.device.type == "cuda" and hasattr(model, "recompute")
        self.cuda = self.device.type == "cuda"
        self.plan = ZeroPlan(model.config, num_processes, rank, zero_stage)
        self.comm = comm if comm is not None else SingleProcessComm(self.plan)
        self.sharded_state = getattr(self.comm, "sharded_state", False)   # real ZeRO-2/3: the comm owns shard buffers
        param_dtype = model.params.dtype if model.params is not None else torch.bfloat16
        self.use_master = use_master_weights and param_dtype != torch.float32
        self.lr, self.wd, self.beta1, self.beta2, self.eps, self.grad_clip = learning_rate, weight_decay, beta1, beta2, eps, grad_clip
        self.step_count = 0
        self.use_cuda_graph = False
        self._graph, self._graph_key, self._graph_acts, self._steps_begun = None, None, None, 0
        self.rng = Xorshift(rng_state)
        self.rng_state_last_update = rng_state
        n = self.plan.state_elements
        dev = self.device
        self.m = torch.zeros(n, dtype=torch.float32, device=dev)
        self.v = torch.zeros(n, dtype=torch.float32, device=dev)
        self.master = torch.zeros(n, dtype=torch.float32, device=dev) if self.use_master else None
        self._master_ready = False
        self.rows = self.plan.segment_rows()
        # expert-parallel tensors: the owner's gradient is a SUM over the tokens of all ranks, while dense
        # gradients are averaged over ranks; dividing by P puts both on the same (global mean) scale
        lay = self.plan.layout
        self.expert_ranges = [(sg.param_off, sg.length) for sg in self.plan.segments if lay[sg.tensor].spec.expert] \
            if num_processes > 1 else []
        self.num_processes = num_processes
        # device scalars: [norm2], [scale], [norm], flag
        self.norm2 = torch.zeros(1, dtype=torch.float32, device=dev)
        self.scale = torch.ones(1, dtype=torch.float32, device=dev)
        self.norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self.flag = torch.zeros(1, dtype=torch.int32, device=dev)
        self.readback = torch.zeros(4, dtype=torch.float32, device=dev)
        self.readback_host = torch.zeros(4, dtype=torch.float32)
        if self.cuda:
            self.readback_host = self.readback_host.pin_memory()
        if self.native:
            from ..ops import optim

            self.segs, self.max_len = optim.make_segments(self.rows, device=dev)
            self.partials = torch.empty(int(self.segs.shape[0]) * 1024, dtype=torch.float32, device=dev)

    # ------------------------------------------------------------------ optimizer pieces
    def _local_norm2(self) -> None:
        g = self.model.grads
        if self.native:
            from ..ops import optim

            optim.global_norm2(g, self.segs, self.max_len, out=self.norm2, partials=self.partials)
        else:
            acc = torch.zeros((), dtype=torch.float32, device=self.device)
            for p_off, g_off, s_off, n, wd in self.rows:
                acc += g[g_off:g_off + n].float().pow(2).sum()
            self.norm2[0] = acc

    def _clip(self) -> None:
        if self.native:
            from ..ops import optim

            optim.clip_scale(self.norm2, self.grad_clip, self.scale, self.norm, self.flag)
        else:
            n = torch.sqrt(self.norm2[0])
            self.norm[0] = n
            finite = torch.isfinite(n)
            self.flag[0] = 0 if finite else 1
            self.scale[0] = (self.grad_clip / n if (self.grad_clip > 0 and n > self.grad_clip) else 1.0) if finite else 0.0

    def _ensure_master(self) -> None:
        if self.use_master and not self._master_ready:
            if self.sharded_state:
                self.comm.master_from_shard(self.master)
            elif self.native:
                from ..ops import optim

                optim.master_from_params(self.master, self.model.params, self.segs, self.max_len)
            else:
                for p_off, g_off, s_off, n, wd in self.rows:
                    self.master[s_off:s_off + n] = self.model.params[p_off:p_off + n].float()
            self._master_ready = True

    def _adamw(self, lr: float, seed: int) -> None:
        t = self.step_count + 1
        if self.native:
            from ..ops import optim

            optim.adamw(self.model.params, self.master, self.model.grads, self.m, self.v, self.segs, self.max_len, lr,
                        self.beta1, self.beta2, t, self.eps, self.wd, grad_scale_ptr=self.scale, seed=seed)
            return
        if int(self.flag[0]) != 0:
            return   # non-finite gradient norm: same as the kernels, state and parameters stay as they are
        b1c, b2c = 1.0 - self.beta1 ** t, 1.0 - self.beta2 ** t
        gs = self.scale[0]
        P, G = self.model.params, self.model.grads
        for p_off, g_off, s_off, n, wd in self.rows:
            g = G[g_off:g_off + n].float() * gs
            m, v = self.m[s_off:s_off + n], self.v[s_off:s_off + n]
            m.mul_(self.beta1).add_(g, alpha=1 - self.beta1)
            v.mul_(self.beta2).addcmul_(g, g, value=1 - self.beta2)
            old = self.master[s_off:s_off + n] if self.use_master else P[p_off:p_off + n].float()
            new = old - lr * ((m / b1c) / ((v / b2c).sqrt() + self.eps) + (self.wd if wd else 0.0) * old)
            if self.use_master:
                self.master[s_off:s_off + n] = new
            P[p_off:p_off + n] = new.to(P.dtype)

    # ------------------------------------------------------------------ the step
    def accumulate(self, micro_batches) -> int:
        """zero grads, run forward/backward over the micro-batches, start bucket reductions."""
        self.begin_step()
        batches = list(micro_batches)
        accum = len(batches)
        for i, (x, y) in enumerate(batches):
            self.micro_step(x, y, i, accum)
        return accum

    def micro_step(self, x, y, index: int, accum: int) -> None:
        """Forward + backward of micro-batch ``index`` of ``accum`` (after :meth:`begin_step`). Loops that drive the
        micro-steps themselves must go through here: the sharded communication path counts micro-steps. With CUDA
        graphs enabled (and a communication path that can be captured) the first optimizer step runs eagerly, the
        second one captures its micro-steps and every later one replays them."""
        if index == 0:
            self._steps_begun = getattr(self, "_steps_begun", 0) + 1
        if self.use_cuda_graph and self._steps_begun > 1 and self._graph_usable([(x, y)]):
            self._micro_step_graph(x, y, index, accum)
            return
        if self.sharded_state:
            self.comm.start_micro_step(index)
        with nvtx_range("forward"):
            self.model.forward(x, y, grad_accum_steps=accum, micro_step=index)
        with nvtx_range("backward_and_reduce"):
            self.model.backward(last_micro_step=(index == accum - 1), bucket_ready=self._bucket_ready)

    # ------------------------------------------------------------------ CUDA graph of one micro-step
    def enable_cuda_graph(self, on: bool = True) -> None:
        """Replay captured forward+backward graphs per micro-step instead of launching ~370 kernels from Python: one
        graph for the micro-steps that only accumulate, one for the last micro-step of a step, which also holds the
        per-bucket "ready" signals and reduce-scatter kernels of the fused ZeRO-1 path (they read the step's epoch
        from device memory). One process, or several with ``FusedComm``; the first step with a given
        (B, T, accumulation) runs eagerly, the second one is captured."""
        self.use_cuda_graph = bool(on)

    def _graph_usable(self, batches) -> bool:
        comm_ok = isinstance(self.comm, SingleProcessComm) or getattr(self.comm, "graph_capturable", False)
        return (self.native and comm_ok and type(self.model).__name__ == "Transformer"
                and len({tuple(x.shape) for x, _ in batches}) == 1)

    def _micro_step_graph(self, x, y, index: int, accum: int) -> None:
        from ..ops import _native

        model = self.model
        key = (tuple(x.shape), accum)
        with_comm = not isinstance(self.comm, SingleProcessComm)
        if self._graph_key != key or self._graph_acts is not model.acts:
            # (re)capture: first use, another shape, or the model's activation buffers were reallocated since (a
            # forward of another shape ran in between): the old graphs point at the old buffers
            B, T = key[0]
            model.allocate(B, T)          # outside the capture: these buffers outlive the graph's own pool
            self._gx = torch.zeros(B, T, dtype=torch.int32, device=self.device)
            self._gy = torch.zeros(B, T, dtype=torch.int32, device=self.device)
            torch.cuda.synchronize(self.device)

            def capture(last: bool):
                graph = torch.cuda.CUDAGraph()
                before = _native.launch_count()
                with torch.cuda.graph(graph):
                    # micro_step=1: the loss accumulator is cleared outside the graph, before the first micro-step
                    model.forward(self._gx, self._gy, grad_accum_steps=accum, micro_step=1)
                    model.backward(last_micro_step=last, bucket_ready=self._bucket_ready if (last and with_comm) else None)
                    if last and with_comm:
                        self.comm.join_buckets()
                # the capture recorded the kernels without running them; gradients and loss are still untouched
                kernels = _native.launch_count() - before
                _native.count_replayed(-kernels)   # they were recorded, not launched
                return graph, kernels

            self._graph_last, self._graph_last_kernels = capture(True)
            if with_comm and accum > 1:
                self._graph, self._graph_kernels = capture(False)
            else:
                self._graph, self._graph_kernels = self._graph_last, self._graph_last_kernels
            self._graph_key, self._graph_acts = key, model.acts
        self._gx.copy_(x, non_blocking=True)
        self._gy.copy_(y, non_blocking=True)
        if index == 0:
            model.acts["loss_acc"].zero_()
        last = index == accum - 1
        (self._graph_last if last else self._graph).replay()
        _native.count_replayed(self._graph_last_kernels if last else self._graph_kernels)

    def begin_step(self) -> None:
        """Start of an optimizer step: wait for the peers (fused communication) and zero the gradients."""
        if getattr(self.comm, "fused", False):
            self.comm.begin_step()
        self.model.zero_grad()

    def _bucket_ready(self, layer) -> None:
        self.comm.reduce_bucket(self.model.grads, layer)

    def update(self, lr: float | None = None, skip: bool = False) -> None:
        """Queue reduction -> norm -> clip -> AdamW -> parameter gather on the current stream (no host
        sync). With ``skip`` the optimizer part is left out; :meth:`apply_update` can run it later."""
        with nvtx_range("reduce_and_grad_norm"):
            for off, n in self.expert_ranges:
                self.model.grads[off:off + n].mul_(1.0 / self.num_processes)
            self.comm.finish_reduce()
            if getattr(self.comm, "fused", False):
                # the bucket kernels already left the norm partials of the averaged shard; the mean loss of the ranks
                # travels with the norm exchange (no library collective in the step)
                self.comm.norm_and_clip(self.grad_clip, self.scale, self.norm, self.flag, loss=self.model.acts["loss_acc"])
            else:
                self.comm.all_reduce_scalar(self.model.acts["loss_acc"], "avg")
                self._local_norm2()
                if self.plan.sharded:
                    self.comm.all_reduce_scalar(self.norm2, "sum")
                self._clip()
        if not skip:
            self.apply_update(lr)

    def skip_update(self) -> None:
        """The caller decided to leave the optimizer out of this step (after ``update(skip=True)``): tell the
        communication path, whose peers otherwise wait for this rank's parameter push."""
        hook = getattr(self.comm, "skip_update", None)
        if hook is not None:
            hook()

    def apply_update(self, lr: float | None = None) -> None:
        with nvtx_range("optimizer_update_and_gather"):
            self._apply_update(lr)

    def _apply_update(self, lr: float | None = None) -> None:
        lr = self.lr if lr is None else lr
        self._ensure_master()
        self.rng_state_last_update = self.rng.state
        seed = self.rng.u32()
        if self.sharded_state:
            self.comm.adamw_shard(self.master, self.m, self.v, lr, self.beta1, self.beta2, self.step_count + 1, self.eps,
                                  self.wd, self.scale, seed)
        elif getattr(self.comm, "fused", False):
            self.comm.adamw_push(self.master, self.m, self.v, lr, self.beta1, self.beta2, self.step_count + 1, self.eps,
                                 self.wd, self.scale, seed)
        else:
            self._adamw(lr, seed)
            self.comm.gather_params(self.model.params)
        self.step_count += 1

    def read_scalars(self) -> tuple[float, float, bool]:
        """(mean loss, grad norm, non-finite flag): one device-to-host copy of 16 bytes, then a sync."""
        self.readback[0:1].copy_(self.model.acts["loss_acc"])
        self.readback[1:2].copy_(self.norm)
        self.readback[2:3].copy_(self.flag.float())
        if self.native:
            from ..ops import _native

            # the kernels' bounded-wait status travels with the same copy: a recorded failure raises here
            self.readback[3:4].copy_(_native.status_word()[0:1].float())
        self.readback_host.copy_(self.readback, non_blocking=True)
        if self.cuda:
            torch.cuda.current_stream().synchronize()
        loss, norm, flag, status = self.readback_host.tolist()
        if status != 0.0:
            from ..ops import _native

            _native.check_status()
        return loss, norm, flag != 0.0

    def train_step(self, micro_batches, lr: float | None = None) -> StepResult:
        """One optimizer step over an iterable of (tokens, targets) micro-batches (pinned-host or device
        int32 tensors of shape (B, T)). Returns loss / grad-norm read back from the device."""
        lr = self.lr if lr is None else lr
        self.accumulate(micro_batches)
        self.update(lr)
        loss, norm, bad = self.read_scalars()
        # a non-finite gradient norm makes the AdamW kernels leave state and parameters untouched
        return StepResult(loss=loss, grad_norm=norm, lr=lr, skipped=bad)

    # ------------------------------------------------------------------ evaluation
    @torch.no_grad()
    def validate(self, tokens, targets) -> float:
        self.model.forward(tokens, targets, grad_accum_steps=1, micro_step=0, compute_dlogits=False)
        return self.model.mean_loss()

    def full_params(self) -> torch.Tensor:
        """The complete bf16 parameter vector in checkpoint order (a collective when parameters are sharded)."""
        if self.model.params is None:
            return self.comm.materialize_params()
        gather_experts = getattr(self.comm, "gather_expert_params", None)
        if gather_experts is not None and self.plan._has_experts():
            gather_experts(self.model.params)      # back-ends that keep another rank's experts stale between steps
        return self.model.params

    def restore_params_from_master(self) -> None:
        """Re-derive the bf16 parameters of this rank's shard from the fp32 master copy with the
        rounding noise of the last update (bit-exact resume), then gather the other shards."""
        if not self.use_master:
            return
        rng = Xorshift(self.rng_state_last_update)
        seed = rng.u32()
        if self.sharded_state:
            self.comm.shard_from_master(self.master, seed)
            self._master_ready = True
            return
        if self.native:
            from ..ops import optim

            optim.params_from_master(self.model.params, self.master, self.segs, self.max_len, seed)
        else:
            for p_off, g_off, s_off, n, wd in self.rows:
                self.model.params[p_off:p_off + n] = self.master[s_off:s_off + n].to(self.model.params.dtype)
        self._master_ready = True
        self.comm.gather_params(self.model.params)
