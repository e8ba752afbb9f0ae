"""Tensor-, sequence-, pipeline-, context- and expert-parallel building blocks.

The reference ships these as un-wired primitives (llmc/distributed_ext.cuh:27-191: equal-count all-to-all,
column / row parallel weight slicing with the matching all-reduces, the sequence-parallel all-gather,
send / recv wrappers for pipeline stages, the ring exchange for context parallelism; local ring-attention
steps in llmc/attention_ext.cuh:433-481 and llmc/tk/ring_attention_sm120.cuh:55-189, forward only and
without causal masking across shards). Here they are functions over ``torch.distributed`` process groups
(NCCL on GPUs, gloo on CPU - the same code runs in the CPU test tier), plus two things the reference only
describes: a 1F1B pipeline schedule with an executor, and a causal ring attention with backward.

The data-parallel / ZeRO / expert-parallel paths of the trainers do not go through this module: they use
the fused peer-memory kernels (parallel/fused.py, parallel/sharded.py, parallel/expert.py).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist


def _world(group=None) -> tuple[int, int]:
    return dist.get_rank(group), dist.get_world_size(group)


# ------------------------------------------------------------------------------------------ expert parallel
def all_to_all_equal(x: torch.Tensor, group=None) -> torch.Tensor:
    """Equal-count all-to-all: ``x`` is [P * n, ...]; block r goes to rank r, block r of the result came from rank r."""
    out = torch.empty_like(x)
    dist.all_to_all_single(out, x.contiguous(), group=group)
    return out


# ------------------------------------------------------------------------------------------ tensor parallel
def tp_slice_columns(weight: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Column-parallel shard of a [OC, C] weight: a contiguous block of output channels."""
    oc = weight.shape[0]
    assert oc % world == 0, "output channels must divide by the tensor-parallel size"
    n = oc // world
    return weight[rank * n:(rank + 1) * n].contiguous()


def tp_slice_rows(weight: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Row-parallel shard of a [OC, C] weight: a contiguous block of input channels."""
    c = weight.shape[1]
    assert c % world == 0, "input channels must divide by the tensor-parallel size"
    n = c // world
    return weight[:, rank * n:(rank + 1) * n].contiguous()


def _matmul_nt(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """a @ w^T with the tcgen05 GEMM on CUDA bf16 inputs, torch otherwise."""
    if a.is_cuda and a.dtype == torch.bfloat16 and a.dim() == 2:
        from ..ops import gemm

        return gemm.gemm_nt(a.contiguous(), w.contiguous())
    return a @ w.t()


def column_parallel_forward(x: torch.Tensor, w_shard: torch.Tensor, b_shard: torch.Tensor | None = None) -> torch.Tensor:
    """y_shard = x W_shard^T (+ b_shard): no communication in forward (x is replicated)."""
    y = _matmul_nt(x, w_shard)
    return y if b_shard is None else y + b_shard


def column_parallel_backward(dy_shard: torch.Tensor, x: torch.Tensor, w_shard: torch.Tensor, group=None):
    """Returns (dx, dW_shard, db_shard); dx is summed over the tensor-parallel group (llmc/distributed_ext.cuh:85-88)."""
    dx = dy_shard @ w_shard
    dist.all_reduce(dx, group=group)
    return dx, dy_shard.t() @ x, dy_shard.sum(0)


def row_parallel_forward(x_shard: torch.Tensor, w_shard: torch.Tensor, bias: torch.Tensor | None = None, group=None) -> torch.Tensor:
    """y = sum over ranks of x_shard W_shard^T (+ bias once): all-reduce of the partial outputs (distributed_ext.cuh:123-126)."""
    y = _matmul_nt(x_shard, w_shard)
    dist.all_reduce(y, group=group)
    return y if bias is None else y + bias


def row_parallel_backward(dy: torch.Tensor, x_shard: torch.Tensor, w_shard: torch.Tensor):
    """Returns (dx_shard, dW_shard): no communication (dy is replicated)."""
    return dy @ w_shard, dy.t() @ x_shard


# ------------------------------------------------------------------------------------------ sequence parallel
def sp_all_gather(x_shard: torch.Tensor, dim: int = 1, group=None) -> torch.Tensor:
    """[B, S/P, D] shards -> [B, S, D] on every rank (entering a tensor-parallel region; distributed_ext.cuh:142-154)."""
    _, world = _world(group)
    parts = [torch.empty_like(x_shard) for _ in range(world)]
    dist.all_gather(parts, x_shard.contiguous(), group=group)
    return torch.cat(parts, dim=dim)


def sp_reduce_scatter(x: torch.Tensor, dim: int = 1, group=None) -> torch.Tensor:
    """The reverse: sum over ranks, keep this rank's sequence shard (leaving a tensor-parallel region)."""
    rank, world = _world(group)
    chunks = [c.contiguous() for c in x.chunk(world, dim=dim)]
    out = torch.empty_like(chunks[rank])
    dist.reduce_scatter(out, chunks, group=group)
    return out


# ------------------------------------------------------------------------------------------ pipeline parallel
def pp_send(t: torch.Tensor, dst: int, group=None) -> None:
    dist.send(t.contiguous(), dst, group=group)


def pp_recv(like: torch.Tensor, src: int, group=None) -> torch.Tensor:
    out = torch.empty_like(like)
    dist.recv(out, src, group=group)
    return out


@dataclass(frozen=True)
class PipeOp:
    kind: str        # "F" or "B"
    micro: int


def one_f_one_b_schedule(num_stages: int, num_micro: int, stage: int) -> list[PipeOp]:
    """The 1F1B order of one stage: warm-up forwards, steady one-forward-one-backward, cool-down backwards.
    At most ``num_stages - stage`` activations are alive on a stage."""
    warm = min(num_stages - stage - 1, num_micro)
    ops = [PipeOp("F", i) for i in range(warm)]
    f, b = warm, 0
    while f < num_micro:
        ops.append(PipeOp("F", f))
        ops.append(PipeOp("B", b))
        f += 1
        b += 1
    while b < num_micro:
        ops.append(PipeOp("B", b))
        b += 1
    return ops


def run_pipeline(stage_module: torch.nn.Module, micro_inputs, loss_fn, act_shape, dtype=torch.float32, device="cpu", group=None):
    """Executes one 1F1B step for this rank's stage (rank = stage index, world = number of stages).

    ``micro_inputs``: list of per-micro-batch inputs (used by stage 0) or targets (used by the last stage);
    ``loss_fn(output, micro_input)`` runs on the last stage. Activations of shape ``act_shape`` travel forward,
    their gradients backward. Returns the summed loss on the last stage, None elsewhere; parameter gradients are
    accumulated into ``stage_module``.
    """
    stage, stages = _world(group)
    first, last = stage == 0, stage == stages - 1
    saved = {}
    total = 0.0
    pending = []   # sends are asynchronous: a forward send of this stage may cross a backward send of the next one

    def send(t, dst):
        t = t.contiguous()
        pending.append((dist.isend(t, dst, group=group), t))
    for op in one_f_one_b_schedule(stages, len(micro_inputs), stage):
        if op.kind == "F":
            if first:
                x = micro_inputs[op.micro]
            else:
                x = pp_recv(torch.empty(act_shape, dtype=dtype, device=device), stage - 1, group).requires_grad_(True)
            y = stage_module(x)
            if last:
                loss = loss_fn(y, micro_inputs[op.micro])
                total += float(loss.detach())
                saved[op.micro] = (x, loss)
            else:
                send(y.detach(), stage + 1)
                saved[op.micro] = (x, y)
        else:
            x, y = saved.pop(op.micro)
            if last:
                y.backward()
            else:
                y.backward(pp_recv(torch.empty(act_shape, dtype=dtype, device=device), stage + 1, group))
            if not first:
                send(x.grad, stage - 1)
    for work, _ in pending:
        work.wait()
    return total if last else None


# ------------------------------------------------------------------------------------------ context parallel
def cp_ring_send_recv(t: torch.Tensor, group=None) -> torch.Tensor:
    """Send ``t`` to the next rank of the ring, return what the previous rank sent (distributed_ext.cuh:184-191)."""
    rank, world = _world(group)
    out = torch.empty_like(t)
    ops = [dist.P2POp(dist.isend, t.contiguous(), (rank + 1) % world, group), dist.P2POp(dist.irecv, out, (rank - 1) % world, group)]
    for r in dist.batch_isend_irecv(ops):
        r.wait()
    return out


def _block_attention(q, k, v, scale, mask):
    """softmax-free pieces of one (query shard, key shard) block: (unnormalised output, row max, row sum)."""
    s = torch.einsum("bhqd,bhkd->bhqk", q, k) * scale
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    m = s.amax(-1, keepdim=True)
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    p = torch.exp(s - m)
    return torch.einsum("bhqk,bhkd->bhqd", p, v), m, p.sum(-1, keepdim=True)


class _RingAttention(torch.autograd.Function):
    """Causal attention over a sequence split into contiguous shards (rank r holds tokens [r*S/P, (r+1)*S/P)).

    K/V shards travel round the ring; a visiting shard from an earlier rank is attended without mask, the own shard
    with the causal mask, later ranks' shards are skipped. Partial results are merged with their log-sum-exp. The
    backward sends dK/dV round the ring together with K/V so that every shard's gradient ends on its owner.
    """

    @staticmethod
    def forward(ctx, q, k, v, group):
        rank, world = _world(group)
        B, H, S, D = q.shape
        scale = 1.0 / math.sqrt(D)
        causal = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
        acc = torch.zeros_like(q, dtype=torch.float32)
        m_run = torch.full((B, H, S, 1), float("-inf"), device=q.device)
        l_run = torch.zeros(B, H, S, 1, device=q.device)
        kk, vv = k, v
        for step in range(world):
            src = (rank - step) % world
            if src <= rank:
                o, m, l = _block_attention(q.float(), kk.float(), vv.float(), scale, causal if src == rank else None)
                m_new = torch.maximum(m_run, m)
                a, b = torch.exp(m_run - m_new), torch.exp(m - m_new)
                acc = acc * a + o * b
                l_run = l_run * a + l * b
                m_run = m_new
            if step + 1 < world:
                kk, vv = cp_ring_send_recv(kk, group), cp_ring_send_recv(vv, group)
        out = (acc / l_run).to(q.dtype)
        ctx.save_for_backward(q, k, v, out, m_run + torch.log(l_run))
        ctx.group = group
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        group = ctx.group
        rank, world = _world(group)
        B, H, S, D = q.shape
        scale = 1.0 / math.sqrt(D)
        causal = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
        dvec = (dout.float() * out.float()).sum(-1, keepdim=True)
        dq = torch.zeros_like(q, dtype=torch.float32)
        kk, vv = k, v
        dk_t, dv_t = torch.zeros_like(k, dtype=torch.float32), torch.zeros_like(v, dtype=torch.float32)
        for step in range(world):
            src = (rank - step) % world
            if src <= rank:
                s = torch.einsum("bhqd,bhkd->bhqk", q.float(), kk.float()) * scale
                if src == rank:
                    s = s.masked_fill(~causal, float("-inf"))
                p = torch.exp(s - lse)
                dp = torch.einsum("bhqd,bhkd->bhqk", dout.float(), vv.float())
                ds = p * (dp - dvec) * scale
                dq += torch.einsum("bhqk,bhkd->bhqd", ds, kk.float())
                dk_t += torch.einsum("bhqk,bhqd->bhkd", ds, q.float())
                dv_t += torch.einsum("bhqk,bhqd->bhkd", p, dout.float())
            # the gradient buffers travel with their K/V shard; after `world` hops they are back at the owner
            kk, vv = cp_ring_send_recv(kk, group), cp_ring_send_recv(vv, group)
            dk_t, dv_t = cp_ring_send_recv(dk_t, group), cp_ring_send_recv(dv_t, group)
        return dq.to(q.dtype), dk_t.to(k.dtype), dv_t.to(v.dtype), None


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group=None) -> torch.Tensor:
    """Causal attention for [B, H, S_local, D] shards of a sequence distributed over the ranks of ``group``."""
    return _RingAttention.apply(q, k, v, group)
