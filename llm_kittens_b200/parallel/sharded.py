"""ZeRO stages 2 and 3 with real sharding, on top of the peer-memory kernels of ``csrc/comm_fused.cu``.

The reference's stages 2 and 3 keep the full gradient and parameter buffers allocated and gather all
parameters right after the optimizer step (llmc/zero.cuh:543-620, train_gpt2.cu:448-480, 1352-1361),
so they save no memory. Here:

* **stage 2 (gradients sharded)**: a block's gradients live in one of two rotating bucket slots. As
  soon as a block's backward is done (every micro-step) the bucket is reduce-scattered straight into
  the rank's fp32 gradient shard (peer loads, ``rs_bucket``; later micro-steps accumulate), and the slot
  is reused two blocks later - after every peer has signalled that it finished reading it. No full
  gradient buffer exists; only the non-block tensors (embeddings, final norm) keep a full-size
  gradient, reduced once per step. After AdamW on the shard the replicated parameters are refreshed
  by one gather kernel (peer loads of the P shards).
* **stage 3 (parameters sharded too)**: the only persistent copy of the block parameters is the
  rank's bf16 shard (symmetric memory). A block's parameters are gathered just in time into one of
  two staging slots by ``ag_bucket`` on a side stream, one block ahead of the compute in forward,
  backward and recompute; AdamW updates the shard in place and nothing is pushed. The non-block
  tensors are gathered once per optimizer step into a persistent buffer. The gather of a block's weight
  MATRICES is tile-granular: the gather kernel publishes one flag per chunk of each matrix as the chunk
  lands (``ag_bucket_flags``), and the GEMMs that consume the matrix poll only the flags covering the
  tile they are about to load (``llmk_gemm_b_ready``), so the compute stream never waits for a whole
  bucket; only the small tensors of a block (norm weights, biases) are waited for with an event.
  ``LLMK_AG_FLAGS=0`` restores the bucket-granular gather (one event per bucket).

The model sees none of this except through its ``p`` / ``g`` dictionaries (per-layer views into the
slots) and the ``param_hook`` / ``grad_hook`` / ``bucket_ready`` callbacks.

Ordering rules that make the peer accesses safe (every wait is bounded, see ``wait_flags_block``):

* a gradient slot is zeroed for block ``l`` only after all ranks raised the "done reading" flag of the
  block that used the slot before;
* the non-block gradient buffer is zeroed at the start of a step, which follows the norm exchange of
  the previous step, and every rank enters that exchange only after its own reads are complete;
* a rank starts AdamW on its shard only after the norm exchange, i.e. after every rank has consumed
  all the parameter gathers of the step; gathers of the next step wait for the "parameters ready"
  flag of every rank.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import _native as N
from ..ops import optim
from .zero import ZeroPlan


class ShardedComm:
    fused = True
    sharded_state = True   # the trainer updates ``param_shard`` / reads ``gshard`` instead of full buffers

    def __init__(self, plan: ZeroPlan, model, device: torch.device, timeout_ms: int | None = None):
        stage = plan.stage
        if not plan.sharded or stage < 2:
            raise RuntimeError("ShardedComm implements ZeRO stages 2 and 3 on more than one rank")
        if any(s.spec.expert for s in plan.layout.slots):
            raise RuntimeError("expert-parallel models use ZeRO stage 1 (their expert tensors are not replicated)")
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        self._symm = symm_mem
        self.plan, self.model, self.device, self.stage = plan, model, device, stage
        self.world_size, self.rank = plan.P, plan.rank
        self.group = dist.group.WORLD
        self.limit_ns = int((timeout_ms if timeout_ms is not None else int(os.environ.get("LLMK_PEER_TIMEOUT_MS", "30000"))) * 1e6)
        self._keep = []
        cfg, lay = plan.config, plan.layout
        L = self.L = cfg.num_layers

        # ---- bucket geometry: offset of every tensor inside a block bucket / the non-block bucket
        self.block_names = [s.spec.name for s in lay.slots if s.spec.layered]
        self.global_names = [s.spec.name for s in lay.slots if not s.spec.layered]
        self.block_off, self.block_size = self._pack(self.block_names)
        self.global_off, self.global_size = self._pack(self.global_names)

        # ---- symmetric buffers (peers read them)
        self.ctrl, self.ctrl_ptrs = self._symmetric(int(N.lib().llmk_comm_ctrl_ints()), torch.int32)
        self.ctrl.zero_()
        self.grad_slots, self.grad_slot_ptrs = self._symmetric(2 * self.block_size, torch.bfloat16)
        self.grad_globals, self.grad_global_ptrs = self._symmetric(self.global_size, torch.bfloat16)
        self.grad_slots.zero_()
        self.grad_globals.zero_()
        self.param_shard, self.param_shard_ptrs = self._symmetric(plan.state_elements, torch.bfloat16)
        self.gshard = torch.zeros(plan.state_elements, dtype=torch.float32, device=device)

        # ---- this rank's shard, from the model's (replicated) initial parameters
        full = model.params
        for s in plan.segments:
            self.param_shard[s.state_off: s.state_off + s.length].copy_(full[s.param_off: s.param_off + s.length])

        # ---- segment tables: reduce-scatter (grad offset of my slice, state offset, length) and
        #      all-gather (state offset, offset of rank 0's slice in the destination, length)
        by_key = {}
        for s in plan.segments:
            by_key.setdefault((s.tensor, s.layer), []).append(s)
        self.rs_tables, self.ag_tables = {}, {}
        ag_full_rows = []
        for layer in list(range(L)) + [None]:
            rs_rows, ag_rows = [], []
            names = self.global_names if layer is None else self.block_names
            for nme in names:
                lidx = 0 if layer is None else layer
                base = self.global_off[nme] if layer is None else (lidx % 2) * self.block_size + self.block_off[nme]
                for s in by_key[(nme, lidx)]:
                    rs_rows.append((base + self.rank * s.length, s.state_off, s.length))
                    ag_rows.append((s.state_off, base, s.length))
                    ag_full_rows.append((s.state_off, s.param_off - self.rank * s.length, s.length))
            self.rs_tables[layer] = torch.tensor(rs_rows, dtype=torch.int64, device=device)
            self.ag_tables[layer] = torch.tensor(ag_rows, dtype=torch.int64, device=device)
        self.ag_full_table = torch.tensor(ag_full_rows, dtype=torch.int64, device=device)
        from .fused import comm_grid_x

        self.grid_x = comm_grid_x(max(s.length for s in plan.segments))
        max_rows = max(int(t.shape[0]) for t in self.rs_tables.values())
        self.partials = torch.zeros(max_rows * self.grid_x, dtype=torch.float32, device=device)  # unused by-product of rs_bucket
        rows = []
        for s in plan.segments:   # a tensor's layers are contiguous in the state buffers: one row per tensor
            if rows and rows[-1][2] + rows[-1][3] == s.state_off and rows[-1][4] == int(s.decay):
                o, _, _, n, d = rows[-1]
                rows[-1] = (o, o, o, n + s.length, d)
            else:
                rows.append((s.state_off, s.state_off, s.state_off, s.length, int(s.decay)))
        self.shard_segs, self.shard_max_len = optim.make_segments(rows, device=device)
        self.norm_partials = torch.empty(int(self.shard_segs.shape[0]) * 1024, dtype=torch.float32, device=device)
        self.norm2 = torch.zeros(8, dtype=torch.float32, device=device)

        # ---- what the model sees
        self.flagged = False
        if stage >= 3:
            self.param_slots = torch.empty(2 * self.block_size, dtype=torch.bfloat16, device=device)
            self.param_globals = torch.empty(self.global_size, dtype=torch.bfloat16, device=device)
            model.p = self._views(self.param_slots, self.param_globals)
            model.params = None           # no full parameter buffer any more
            model.param_hook = self._param_hook
            if os.environ.get("LLMK_AG_FLAGS", "1") != "0":
                self._setup_flagged_gather(model, by_key)
        del full
        model.g = self._views(self.grad_slots, self.grad_globals)
        model.grads = None
        model.zero_grad = self.grad_globals.zero_
        model.grad_hook = self._grad_hook
        model.reduce_every_micro_step = True

        # ---- protocol state
        self.epoch = 0           # optimizer steps
        self.micro = 0           # micro-steps since start (block buckets are reduced every micro-step)
        self.slot_globals, self.slot_params, self.slot_norm = L, L + 1, L + 2
        self.slot_done = L + 3   # + layer: "I have finished reading your gradient bucket of this layer"
        if (self.slot_done + L) * int(N.lib().llmk_comm_max_ranks()) > 2048:
            raise RuntimeError("too many layers for the control buffer of the fused communication path")
        self.stream = torch.cuda.Stream(device=device)       # reduce-scatter kernels
        # parameter gathers: high priority, so that a gather which GEMMs are already polling for gets the next free
        # thread slots of every SM (a GEMM CTA leaves most of an SM's thread and register budget unused)
        self.ag_stream = torch.cuda.Stream(device=device, priority=-1)
        self._gathered = {}                # layer -> event of a queued gather not yet consumed
        self._resident = [None, None]      # layer whose parameters sit in each slot
        self._globals_stale = True
        self._params_pending = 0           # step whose shard updates the peers may still be running
        self._first_micro = True
        torch.cuda.synchronize(device)
        dist.barrier()

    # ------------------------------------------------------------------ helpers
    def _pack(self, names):
        off, table = 0, {}
        for nme in names:
            table[nme] = off
            off += self.plan.layout[nme].size
        return table, off

    def _symmetric(self, numel, dtype):
        t = self._symm.empty(numel, dtype=dtype, device=self.device)
        hdl = self._symm.rendezvous(t, self.group)
        self._keep.append(hdl)
        ptrs = (ctypes.c_longlong * self.world_size)(*[int(p) for p in hdl.buffer_ptrs])
        return t, ptrs

    def _views(self, slots: torch.Tensor, globals_: torch.Tensor) -> dict:
        lay = self.plan.layout
        out = {}
        for nme in self.block_names:
            sl = lay[nme]
            views = []
            for l in range(self.L):
                base = (l % 2) * self.block_size + self.block_off[nme]
                views.append(slots[base: base + sl.size].view(*sl.spec.shape))
            out[nme] = views
        for nme in self.global_names:
            sl = lay[nme]
            out[nme] = globals_[self.global_off[nme]: self.global_off[nme] + sl.size].view(*sl.spec.shape)
        return out

    def _wait(self, slot: int, epoch: int) -> None:
        N.call("llmk_comm_wait", self.ctrl, slot, epoch, self.world_size, self.limit_ns, N.status_word())

    def _signal(self, slot: int, epoch: int) -> None:
        N.call("llmk_comm_signal", self.ctrl_ptrs, slot, self.rank, self.world_size, epoch)

    # ------------------------------------------------------------------ parameters (stage 3)
    def _setup_flagged_gather(self, model, by_key) -> None:
        """Split every block bucket into its weight matrices (gathered chunk by chunk with one flag per chunk, consumed
        by GEMMs that poll those flags) and the small rest (norm weights, biases: gathered first, waited for with an
        event). A matrix of ``size`` elements arrives as P shards of ``size / P``; each shard is cut into ``cps`` chunks
        of about ``LLMK_AG_CHUNK_BYTES`` (default 1 MiB), so flag ``f`` of a matrix covers its elements
        ``[f * chunk, (f + 1) * chunk)`` and a GEMM maps a tile to flags by one division."""
        from ..ops import gemm

        lay, P = self.plan.layout, self.world_size
        target = max(4096, int(os.environ.get("LLMK_AG_CHUNK_BYTES", str(1 << 20)))) // 2   # elements
        self.matrix_names, geometry, nflags = [], {}, 0
        for nme in self.block_names:
            spec = lay[nme].spec
            per_layer = lay[nme].size
            segs = by_key[(nme, 0)]
            if len(spec.shape) != 2 or per_layer < 16384 or len(segs) != 1 or segs[0].length * P != per_layer:
                continue
            length = segs[0].length
            cps = max(1, min(8, length // target))
            while cps > 1 and length % (cps * 8):
                cps -= 1
            self.matrix_names.append(nme)
            geometry[nme] = (cps, length // cps)
        if not self.matrix_names:
            return
        for q in range(2):
            for nme in self.matrix_names:
                geometry[(q, nme)] = nflags
                nflags += P * geometry[nme][0]
        self.ag_flags = torch.zeros(nflags, dtype=torch.int32, device=self.device)
        self.ag_arrivals = torch.zeros(nflags, dtype=torch.int32, device=self.device)
        # blocks per chunk: about 600 blocks per gather, so that enough peer loads are in flight to fill the links
        self.ag_bpc = max(1, min(16, 600 // max(1, P * sum(geometry[n][0] for n in self.matrix_names))))
        self.ag_small_tables, self.ag_flag_tables = {}, {}
        for layer in range(self.L):
            small, flagged = [], []
            for nme in self.block_names:
                base = (layer % 2) * self.block_size + self.block_off[nme]
                for sg in by_key[(nme, layer)]:
                    if nme in self.matrix_names:
                        flagged.append((sg.state_off, base, sg.length, geometry[(layer % 2, nme)], geometry[nme][0]))
                    else:
                        small.append((sg.state_off, base, sg.length))
            self.ag_small_tables[layer] = torch.tensor(small, dtype=torch.int64, device=self.device) if small else None
            self.ag_flag_tables[layer] = torch.tensor(flagged, dtype=torch.int64, device=self.device)
        self.ag_max_cps = max(geometry[n][0] for n in self.matrix_names)
        # the consumers: one registry entry per (slot, matrix); layers l and l + 2 share the slot and its entry
        self._ready_entries = {}
        for q in range(min(2, self.L)):
            for nme in self.matrix_names:
                self._ready_entries[(q, nme)] = gemm.register_b_ready(model.p[nme][q], self.ag_flags, geometry[(q, nme)],
                                                                     geometry[nme][1], self.limit_ns)
        self._tick = 0
        self._gathers_in_flight = []
        self.flagged = True

    def _gather(self, layer, after: torch.cuda.Event) -> None:
        """Queue the gather of one bucket on the gather stream, after the compute recorded in ``after``."""
        table = self.ag_tables[layer]
        dst = self.param_globals if layer is None else self.param_slots
        with torch.cuda.stream(self.ag_stream):
            self.ag_stream.wait_event(after)
            if self.flagged and layer is not None:
                small, flagged = self.ag_small_tables[layer], self.ag_flag_tables[layer]
                if small is not None:
                    N.call("llmk_comm_ag_bucket", self.param_shard_ptrs, dst, small, int(small.shape[0]), 2, self.world_size)
                ev = torch.cuda.Event()
                ev.record()           # the compute stream waits for the small tensors only
                self._tick += 1
                N.call("llmk_comm_ag_bucket_flags", self.param_shard_ptrs, dst, flagged, int(flagged.shape[0]), self.ag_max_cps,
                       self.world_size, self.ag_flags, self.ag_arrivals, self.ag_bpc, self._tick)
                done = torch.cuda.Event()
                done.record()
                self._gathers_in_flight.append(done)
                for nme in self.matrix_names:
                    self._ready_entries[(layer % 2, nme)][3] = self._tick
            else:
                N.call("llmk_comm_ag_bucket", self.param_shard_ptrs, dst, table, int(table.shape[0]), self.grid_x, self.world_size)
                ev = torch.cuda.Event()
                ev.record()
        self._gathered[layer] = ev
        if layer is not None:
            self._resident[layer % 2] = layer

    def _param_hook(self, layer, phase: str) -> None:
        """Called by the model right before it uses the parameters of ``layer`` (None = non-block tensors);
        ``phase`` tells the direction of travel (``forward`` or ``backward``)."""
        cur = torch.cuda.current_stream()
        if layer is None:
            if phase == "forward" and self._globals_stale:
                if self._params_pending:
                    self._wait(self.slot_params, self._params_pending)
                    self._params_pending = 0
                now = torch.cuda.Event()
                now.record()
                self._gather(None, now)
                cur.wait_event(self._gathered.pop(None))
                self._globals_stale = False
            return
        now = torch.cuda.Event()
        now.record()
        if self._resident[layer % 2] != layer:
            self._gather(layer, now)
        if layer in self._gathered:
            cur.wait_event(self._gathered.pop(layer))
        nxt = layer + 1 if phase == "forward" else layer - 1
        if 0 <= nxt < self.L and self._resident[nxt % 2] != nxt:
            # one block ahead: the slot was last read by the block before this one, all queued before `now`
            self._gather(nxt, now)

    # ------------------------------------------------------------------ gradients
    def _grad_hook(self, layer: int) -> None:
        """Before block ``layer`` writes gradients: wait until every rank has finished reading what the
        slot held before, then clear it."""
        if layer + 2 < self.L:
            user, when = layer + 2, self.micro
        else:
            user, when = layer % 2, self.micro - 1
        if when > 0:
            self._wait(self.slot_done + user, when)
        base = (layer % 2) * self.block_size
        self.grad_slots[base: base + self.block_size].zero_()

    def begin_step(self) -> None:
        self.epoch += 1
        self._first_micro = True

    def start_micro_step(self, index: int) -> None:
        self.micro += 1
        self._first_micro = index == 0

    def reduce_bucket(self, grads, layer) -> None:
        """Reduce-scatter one bucket into the fp32 gradient shard; block buckets every micro-step (adding to
        the shard after the first), the non-block bucket once per step."""
        if self.micro == 0 or self.epoch == 0:
            raise RuntimeError("ShardedComm: begin_step() / start_micro_step() were not called (drive micro-steps through "
                               "Trainer.micro_step)")
        if layer is None:
            slot, epoch, ptrs, acc = self.slot_globals, self.epoch, self.grad_global_ptrs, 0
        else:
            slot, epoch, ptrs, acc = layer, self.micro, self.grad_slot_ptrs, 0 if self._first_micro else 1
        self._signal(slot, epoch)
        ev = torch.cuda.Event()
        ev.record()
        table = self.rs_tables[layer]
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(ev)
            N.call("llmk_comm_rs_bucket", ptrs, self.ctrl, slot, epoch, table, int(table.shape[0]), self.gshard, self.partials,
                   self.grid_x, self.world_size, acc, self.limit_ns, N.status_word())
            if layer is not None:
                self._signal(self.slot_done + layer, self.micro)

    def finish_reduce(self) -> None:
        torch.cuda.current_stream().wait_stream(self.stream)

    def norm_and_clip(self, clip, scale, norm, flag, loss=None) -> None:
        if self.flagged:
            # every gather of this step has been consumed tile by tile; before this rank tells the others (through the
            # norm exchange) that its reads of their shards are over, the gather kernels themselves must have ended
            cur = torch.cuda.current_stream()
            for ev in self._gathers_in_flight:
                cur.wait_event(ev)
            self._gathers_in_flight.clear()
        optim.global_norm2(self.gshard, self.shard_segs, self.shard_max_len, out=self.norm2[:1], partials=self.norm_partials)
        N.call("llmk_comm_norm_exchange", self.ctrl_ptrs, self.norm2, 1, self.slot_norm, self.rank, self.world_size, self.epoch,
               float(clip), scale, norm, flag, loss, 1.0, self.limit_ns, N.status_word())

    # ------------------------------------------------------------------ optimizer
    def adamw_shard(self, master, m, v, lr, beta1, beta2, step, eps, wd, scale, seed) -> None:
        optim.adamw(self.param_shard, master, self.gshard, m, v, self.shard_segs, self.shard_max_len, lr, beta1, beta2, step, eps,
                    wd, grad_scale_ptr=scale, seed=seed)
        self._signal(self.slot_params, self.epoch)
        if self.stage >= 3:
            self._params_pending = self.epoch
            self._invalidate()
        else:
            self._wait(self.slot_params, self.epoch)
            self._refresh_replicated()

    def _invalidate(self) -> None:
        self._globals_stale = True
        self._resident = [None, None]
        self._gathered.clear()

    def _refresh_replicated(self) -> None:
        """Stage 2: rebuild the replicated parameter buffer from the P shards (one kernel, peer loads)."""
        t = self.ag_full_table
        N.call("llmk_comm_ag_bucket", self.param_shard_ptrs, self.model.params, t, int(t.shape[0]), self.grid_x, self.world_size)

    def master_from_shard(self, master: torch.Tensor) -> None:
        master.copy_(self.param_shard)

    def shard_from_master(self, master: torch.Tensor, seed: int) -> None:
        """Re-derive the bf16 shard from fp32 master weights with the rounding noise of ``seed`` (resume)."""
        optim.params_from_master(self.param_shard, master, self.shard_segs, self.shard_max_len, seed)
        self._publish()

    def _publish(self) -> None:
        """After a host-driven change of the shards: make it visible to every rank's next gather."""
        torch.cuda.current_stream().synchronize()
        dist.barrier(group=self.group)
        if self.stage >= 3:
            self._invalidate()
        else:
            self._refresh_replicated()
            torch.cuda.current_stream().synchronize()
            dist.barrier(group=self.group)

    # ------------------------------------------------------------------ library-style helpers
    def all_reduce_scalar(self, t: torch.Tensor, op: str = "sum") -> None:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        if op == "avg":
            t.div_(self.world_size)

    def gather_params(self, params) -> None:
        pass

    def materialize_params(self) -> torch.Tensor:
        """Full bf16 parameter vector in checkpoint order (collective: every rank must call it)."""
        torch.cuda.current_stream().synchronize()
        dist.barrier(group=self.group)
        full = torch.empty(self.plan.layout.total, dtype=torch.bfloat16, device=self.device)
        t = self.ag_full_table
        N.call("llmk_comm_ag_bucket", self.param_shard_ptrs, full, t, int(t.shape[0]), self.grid_x, self.world_size)
        torch.cuda.current_stream().synchronize()
        dist.barrier(group=self.group)
        return full

    def load_params(self, full: torch.Tensor) -> None:
        """Take this rank's shard from a full parameter vector (checkpoint load)."""
        for s in self.plan.segments:
            self.param_shard[s.state_off: s.state_off + s.length].copy_(full[s.param_off: s.param_off + s.length])
        self._publish()

    def barrier(self) -> None:
        dist.barrier(group=self.group)
