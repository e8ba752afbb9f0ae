"""Run-validation commands: ``python -m llm_kittens_b200.cli.check <command> …``.

* ``log MAIN_LOG [--final-step N] [--max-train-loss X] [--max-val-loss X] [--no-decrease]`` — the threshold /
  decrease checks of the reference's ``dev/validate_training_log.py`` (1-179) on a ``main.log``.
* ``compare LOG_A LOG_B [--rel-tol R] [--abs-tol A]`` — curve comparison of two runs, as in
  ``dev/compare_training_logs.py`` (1-125): how "N GPUs == 1 GPU" is checked.
* ``zero-layout [--models …] [--world …]`` — recomputes the ZeRO shard intervals of every model descriptor at every
  world size and checks that they tile each tensor exactly (``dev/validate_zero_layout.py:1-174``).
* ``checkpoint DIR [--step N]`` — header / size / DONE-marker checks of a checkpoint directory
  (``dev/validate_llama_checkpoint_artifacts.py``).

* ``write-debug-state MODEL_BIN OUT [--batch B] [--seq T] [--seed S]`` — runs the fp32 PyTorch model on one batch of
  seeded tokens and writes inputs, targets, logits, loss and every gradient (the artefact that the reference's
  ``train_gpt2.py`` writes for its C tests, train_gpt2.py:395-524).
* ``debug-state MODEL_BIN DEBUG_STATE [--device cuda|cpu] [--logit-tol X] [--loss-tol X]`` — the whole-model gate on
  exported artefacts (jobs of ``dev/cuda/gpt2_validate.cu:12-101`` and ``test_gpt2.cu:168-229``): loads the model file,
  runs forward + backward of the framework's model (the CUDA path on a GPU, else the PyTorch model) on the stored
  batch and compares logits, loss and every gradient tensor with the stored values, tensor by tensor.

* ``device [--peers]`` — preflight of the machine (job of ``dev/cuda/cuda_runtime_check.cu:53-133`` for this
  framework's one target): driver / runtime versions, every visible GPU with its compute capability, SM count and
  memory; fails unless all of them are sm_100 (B200 / GB200: the kernels are built for ``sm_100a`` only), the CUDA
  library loads and reports resident CTA pairs, and a 1-byte allocate / memset / synchronise works; ``--peers`` also
  requires peer access between every pair of GPUs (the fused communication kernels need it).

Every command prints its findings and exits 1 if there are any.
"""
from __future__ import annotations

import argparse
import os
import sys

from ..models.config import config_from_descriptor
from ..parallel import zero
from ..utils import formats
from ..utils.logger import compare_logs, validate_log

DEFAULT_MODELS = ["d12", "d24", "d36", "d48", "gpt3:c768", "gpt3:c1024", "gpt3:c2048", "gpt3:c4096", "gpt3:c12288",
                  "llama3.2:1B", "llama3:8B", "llama3.1:8B"]
DEFAULT_WORLDS = [1, 2, 4, 8, 16]


def check_zero_layout(models=DEFAULT_MODELS, worlds=DEFAULT_WORLDS) -> list[str]:
    """Every non-expert tensor's per-layer shard intervals are equal-sized, ordered by rank, disjoint, and cover
    exactly [offset + l*size, offset + (l+1)*size); a world size that does not divide a tensor must be reported by
    ``validate_sharding`` instead of producing a layout."""
    problems = []
    for desc in models:
        cfg = config_from_descriptor(desc)
        layout = cfg.layout()
        for world in worlds:
            refused = zero.validate_sharding(cfg, world, 3)
            if refused:
                # a refusal is right when a tensor does not divide, or a shard would not be a whole number of 16-byte units
                unsplittable = [s.spec.name for s in layout.slots if not s.spec.expert and s.size % (8 * world)]
                if not unsplittable:
                    problems.append(f"{desc} P={world}: refused ({refused[0]}) although every tensor splits")
                continue
            table = zero.shard_intervals_table(cfg, world)
            for slot in layout.slots:
                if slot.spec.expert:
                    continue
                rows = table[slot.spec.name]
                if len(rows) != slot.layers * world:
                    problems.append(f"{desc} P={world} {slot.spec.name}: {len(rows)} intervals, expected {slot.layers * world}")
                    continue
                for l in range(slot.layers):
                    cursor = slot.offset + l * slot.size
                    for r in range(world):
                        layer, rank, start, end = rows[l * world + r]
                        if (layer, rank) != (l, r) or start != cursor or end - start != slot.size // world:
                            problems.append(f"{desc} P={world} {slot.spec.name} layer {l} rank {r}: [{start},{end}) breaks the tiling at {cursor}")
                        cursor = end
                    if cursor != slot.offset + (l + 1) * slot.size:
                        problems.append(f"{desc} P={world} {slot.spec.name} layer {l}: shards end at {cursor}")
    return problems


def check_checkpoint(directory: str, step: int | None = None) -> list[str]:
    """The model file's header describes a known configuration and its payload has exactly the size the layout gives;
    every rank's state file is present with a matching header; the DONE marker exists."""
    problems = []
    if step is None:
        step = formats.find_max_step(directory)
        if step < 0:
            return [f"no finished checkpoint (DONE_*) in {directory}"]
    model_path, _, done_path = formats.checkpoint_paths(directory, step, 0)
    if not os.path.exists(done_path):
        problems.append(f"missing {os.path.basename(done_path)}")
    if not os.path.exists(model_path):
        return problems + [f"missing {os.path.basename(model_path)}"]
    try:
        cfg, fp32 = formats.config_from_model_header(formats.read_header(model_path), model_path)
    except formats.FormatError as e:
        return problems + [str(e)]
    want = 1024 + cfg.num_parameters() * (4 if fp32 else 2)
    have = os.path.getsize(model_path)
    if have != want:
        problems.append(f"{os.path.basename(model_path)}: {have} bytes, the header's configuration needs {want}")
    _, state0, _ = formats.checkpoint_paths(directory, step, 0)
    if not os.path.exists(state0):
        return problems + [f"missing {os.path.basename(state0)}"]
    h = formats.read_header(state0)
    if int(h[0]) != formats.state_magic(cfg.family):
        problems.append(f"{os.path.basename(state0)}: magic {int(h[0])} is not the {cfg.family} state magic")
    nproc = int(h[2])
    for rank in range(nproc):
        _, sp, _ = formats.checkpoint_paths(directory, step, rank)
        if not os.path.exists(sp):
            problems.append(f"missing {os.path.basename(sp)} (the checkpoint was written by {nproc} processes)")
            continue
        hr = formats.read_header(sp)
        if int(hr[2]) != nproc or int(hr[3]) != rank or int(hr[10]) != step:
            problems.append(f"{os.path.basename(sp)}: header says nproc {int(hr[2])} rank {int(hr[3])} step {int(hr[10])}")
    return problems


def write_debug_state(model_path: str, out_path: str, B: int = 4, T: int = 64, seed: int = 1337) -> None:
    import numpy as np
    import torch

    from ..oracle.torch_model import TorchTransformer

    cfg, params = formats.read_model(model_path, device="cpu", dtype=torch.float32)
    model = TorchTransformer(cfg, device="cpu", dtype=torch.float32)
    model.load_parameters(params)
    g = torch.Generator().manual_seed(seed)
    x = torch.randint(0, cfg.vocab_size, (B, T), generator=g, dtype=torch.int32)
    y = torch.randint(0, cfg.vocab_size, (B, T), generator=g, dtype=torch.int32)
    model.zero_grad()
    model.forward(x, y)
    model.backward()
    logits = model.logits_view().reshape(B, T, -1)[..., : cfg.vocab_size].float().numpy()
    formats.write_debug_state(out_path, x.numpy(), y.numpy(), np.ascontiguousarray(logits), model.mean_loss(), model.grads.float().numpy())


def check_debug_state(model_path: str, state_path: str, device: str = "", logit_tol: float = 0.0, loss_tol: float = 0.0) -> list[str]:
    """Problems found when the framework's model, loaded from ``model_path``, is run on the batch of ``state_path``.
    Default tolerances: bf16 CUDA path logits 0.25 / loss 0.05 (the reference accepts 25.0 on bf16 logits and 0.05 on
    the loss, test_gpt2.cu:223-229, 326-347), fp32 path 1e-3 / 1e-4; gradients per tensor ``thr + 0.079 * |ref|`` on at
    least 99.5 % of the elements, ``thr`` by tensor kind as in test_gpt2.cu:9-50."""
    import torch

    cfg, params = formats.read_model(model_path, device="cpu", dtype=torch.float32)
    layout = cfg.layout()
    state = formats.read_debug_state(state_path, cfg.vocab_size, layout.total)
    cuda = (device or ("cuda" if torch.cuda.is_available() else "cpu")).startswith("cuda")
    x, y = torch.from_numpy(state["x"].copy()), torch.from_numpy(state["y"].copy())
    if cuda:
        from ..models.moe import MoETransformer
        from ..models.transformer import Transformer

        cls = MoETransformer if cfg.family == "moe" else Transformer
        model = cls(cfg, device="cuda", recompute=0)
        model.params.copy_(params.to(torch.bfloat16))
        x, y = x.cuda(), y.cuda()
    else:
        from ..oracle.torch_model import TorchTransformer

        model = TorchTransformer(cfg, device="cpu", dtype=torch.float32)
        model.load_parameters(params)
    logit_tol = logit_tol or (0.25 if cuda else 1e-3)
    loss_tol = loss_tol or (0.05 if cuda else 1e-4)
    problems = []
    model.forward(x, y, compute_dlogits=False)
    logits = model.logits_view().reshape(state["B"], state["T"], -1)[..., : cfg.vocab_size].float().cpu()
    err = (logits - torch.from_numpy(state["logits"].copy())).abs().max().item()
    if not err <= logit_tol:
        problems.append(f"logits differ by up to {err:.4g} (tolerance {logit_tol})")
    model.zero_grad()
    model.forward(x, y)
    loss = model.mean_loss()
    if not abs(loss - state["loss"]) <= loss_tol:
        problems.append(f"loss {loss:.6f} vs stored {state['loss']:.6f} (tolerance {loss_tol})")
    model.backward()
    grads = model.grads.float().cpu()
    ref = torch.from_numpy(state["grads"].copy())
    for slot in layout.slots:
        g, r = grads[slot.offset: slot.offset + slot.total], ref[slot.offset: slot.offset + slot.total]
        thr = (5e-3 if slot.spec.name in ("wte", "lm_head") else 2e-2) if cuda else 1e-5
        bad = ((g - r).abs() > thr + (0.079 if cuda else 1e-3) * r.abs()).float().mean().item()
        if not bad <= (5e-3 if cuda else 0.0):
            problems.append(f"gradient of {slot.spec.name}: {100 * bad:.2f} % of the elements are outside {thr} + 0.079*|ref| "
                            f"(max abs diff {(g - r).abs().max().item():.4g})")
    return problems


class _TorchProbe:
    """What ``check_device`` asks of the machine; tests pass a stand-in."""

    def versions(self) -> tuple[str, str]:
        import torch

        drv = "?"
        try:
            import pynvml

            pynvml.nvmlInit()
            drv = pynvml.nvmlSystemGetDriverVersion()
            drv = drv.decode() if isinstance(drv, bytes) else str(drv)
        except Exception:      # NVML is optional here: the runtime version is enough to go on
            pass
        return drv, str(torch.version.cuda)

    def devices(self) -> list[dict]:
        import torch

        out = []
        for i in range(torch.cuda.device_count() if torch.cuda.is_available() else 0):
            p = torch.cuda.get_device_properties(i)
            out.append({"name": p.name, "major": p.major, "minor": p.minor, "sms": p.multi_processor_count, "memory": p.total_memory})
        return out

    def can_access_peer(self, a: int, b: int) -> bool:
        import torch

        return bool(torch.cuda.can_device_access_peer(a, b))

    def touch(self, dev: int) -> None:
        import torch

        t = torch.zeros(1, dtype=torch.uint8, device=f"cuda:{dev}")
        torch.cuda.synchronize(dev)
        del t

    def pair_clusters(self, dev: int) -> int:
        import torch

        from ..ops import _native

        with torch.cuda.device(dev):
            return int(_native.lib().llmk_gemm_pair_clusters())


def check_device(peers: bool = False, probe=None, out=print) -> list[str]:
    probe = probe or _TorchProbe()
    problems: list[str] = []
    drv, rt = probe.versions()
    out(f"CUDA driver version: {drv}")
    out(f"CUDA runtime version: {rt}")
    devs = probe.devices()
    out(f"CUDA visible devices: {len(devs)}")
    if not devs:
        return ["no CUDA devices visible to the runtime"]
    for i, d in enumerate(devs):
        out(f"CUDA device {i}: {d['name']} (sm_{d['major']}{d['minor']}), {d['sms']} SMs, {d['memory'] / 2**30:.0f} GiB")
        if (d["major"], d["minor"]) != (10, 0):
            problems.append(f"device {i} is {d['name']} (sm_{d['major']}{d['minor']}): the kernels are built for sm_100a (B200 / GB200) only")
    if problems:
        return problems
    for i in range(len(devs)):
        try:
            probe.touch(i)
            pairs = probe.pair_clusters(i)
        except Exception as e:      # report, do not crash: this command exists to explain a broken machine
            problems.append(f"device {i}: {type(e).__name__}: {e}")
            continue
        out(f"CUDA device {i}: library loaded, {pairs} resident CTA pairs for the tcgen05 GEMM")
        if pairs <= 0:
            problems.append(f"device {i}: the CTA-pair GEMM kernel cannot be resident (LLMK_GEMM_PAIR=0 set, or shared memory opt-in refused)")
    if peers:
        for a in range(len(devs)):
            for b in range(len(devs)):
                if a != b and not probe.can_access_peer(a, b):
                    problems.append(f"no peer access from device {a} to device {b}: the fused communication kernels need it "
                                    f"(the trainers then fall back to library collectives)")
    return problems


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="llm_kittens_b200.cli.check", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)
    p = sub.add_parser("log")
    p.add_argument("path")
    p.add_argument("--final-step", type=int)
    p.add_argument("--max-train-loss", type=float)
    p.add_argument("--max-val-loss", type=float)
    p.add_argument("--no-decrease", action="store_true")
    p = sub.add_parser("compare")
    p.add_argument("a")
    p.add_argument("b")
    p.add_argument("--rel-tol", type=float, default=0.02)
    p.add_argument("--abs-tol", type=float, default=0.02)
    p = sub.add_parser("zero-layout")
    p.add_argument("--models", nargs="*", default=DEFAULT_MODELS)
    p.add_argument("--world", nargs="*", type=int, default=DEFAULT_WORLDS)
    p = sub.add_parser("checkpoint")
    p.add_argument("directory")
    p.add_argument("--step", type=int)
    p = sub.add_parser("write-debug-state")
    p.add_argument("model")
    p.add_argument("out")
    p.add_argument("--batch", type=int, default=4)
    p.add_argument("--seq", type=int, default=64)
    p.add_argument("--seed", type=int, default=1337)
    p = sub.add_parser("debug-state")
    p.add_argument("model")
    p.add_argument("state")
    p.add_argument("--device", default="")
    p.add_argument("--logit-tol", type=float, default=0.0)
    p.add_argument("--loss-tol", type=float, default=0.0)
    p = sub.add_parser("device")
    p.add_argument("--peers", action="store_true")
    args = ap.parse_args(argv)

    if args.command == "device":
        problems = check_device(args.peers)
    elif args.command == "log":
        problems = validate_log(args.path, args.final_step, args.max_train_loss, args.max_val_loss, not args.no_decrease)
    elif args.command == "compare":
        problems = compare_logs(args.a, args.b, args.rel_tol, args.abs_tol)
    elif args.command == "zero-layout":
        problems = check_zero_layout(args.models, args.world)
    elif args.command == "write-debug-state":
        write_debug_state(args.model, args.out, args.batch, args.seq, args.seed)
        problems = []
    elif args.command == "debug-state":
        problems = check_debug_state(args.model, args.state, args.device, args.logit_tol, args.loss_tol)
    else:
        problems = check_checkpoint(args.directory, args.step)
    for line in problems:
        print("FAIL:", line)
    if not problems:
        print("ok")
    return 1 if problems else 0


if __name__ == "__main__":
    sys.exit(main())
