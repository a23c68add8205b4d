#!/usr/bin/env python
"""Headline benchmark: training throughput (tokens/s) of Llama-3-8B, bf16 with fp32
AdamW master weights, sequence length 8192, micro-batch 1 per GPU, activation
checkpointing; FSDP over the mesh dim ``gpus`` when run on more than one GPU.

    python bench.py --gpus 1 --steps 8 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 8 --warmup 3

The step is driven the way a user of the framework drives it: the processes of the launch
form a proc mesh (``attach_proc_mesh``), rank 0 is the controller, a ``TrainerActor`` is
spawned on every proc and the controller sends endpoint calls.

* ``value``: device-timed whole-job tokens/s -- one ``timed_steps`` call; inside it every
  rank runs ``warmup`` untimed steps and then exactly ``steps`` optimizer steps between two
  CUDA events with a barrier + synchronize on both sides; the maximum over the ranks counts.
* ``e2e``: the same metric through ``trainers.step.call(i).get()`` once per step: every step
  copies its batch from pinned host memory, runs, and reads the loss back to the host, and
  the reply travels over the actor mesh to the controller, whose clock times the loop.
* ``vs_baseline``: ``value`` divided by the same measurement of the library arm in the same
  run (``baseline``: stock torch modules, cuBLAS, SDPA, fused torch AdamW, ``fully_shard`` over
  NCCL for more than one GPU) -- what the reference's tensor worker would execute for this
  program.  The reference itself cannot be built offline (``--impl reference`` says why).

Prints ONE JSON line on rank 0.  Synthetic token ids, random-init weights.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "aten"])
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--parallelism", default="auto")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--recompute-layers", type=int, default=None,
                    help="activation checkpointing: recompute only the first N layers and keep "
                         "the activations of the rest (default: recompute every layer)")
    ap.add_argument("--schedule", default="1f1b", choices=["gpipe", "1f1b", "zb-h1"],
                    help="pipeline schedule (ppPxtpT only)")
    ap.add_argument("--microbatches", type=int, default=8,
                    help="micro-batches per step of a pipeline-parallel run (ppPxtpT)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--cpu", action="store_true",
                    help="run the same flow on CPU ranks (gloo, library collectives): a check of "
                         "the harness, not a benchmark")
    ap.add_argument("--no-baseline", action="store_true",
                    help="skip the library arm (vs_baseline stays null)")
    return ap.parse_args()


def reference_unavailable():
    print(json.dumps({
        "impl": "reference",
        "unavailable": "pytorch-labs/monarch needs cargo + Rust nightly + crates.io and "
                       "setuptools_rust to build; none is installed offline here (pip install "
                       "of the reference tree fails at metadata: No module named 'setuptools_rust')",
    }))
    return 0


def run_arm(mesh, impl: str, args, e2e: bool):
    """Spawn the trainers of one arm on ``mesh``, measure, release them."""
    from monarch_b200.parallel.trainer_actor import TrainerActor
    spec = {"impl": impl, "model": args.model, "seq_len": args.seq, "micro_batch": args.micro_batch,
            "parallelism": args.parallelism, "comm": args.comm,
            "recompute_layers": args.recompute_layers, "microbatches": args.microbatches,
            "schedule": args.schedule, "cuda": not args.cpu}
    trainers = mesh.spawn(f"trainer_{impl}", TrainerActor, spec)
    info = [v for _, v in trainers.info.call().get(timeout=1800).items()]
    timed = [v for _, v in trainers.timed_steps.call(args.warmup, args.steps).get(timeout=3600).items()]
    ms = max(t["ms"] for t in timed)
    tokens_per_step = info[0]["tokens_per_step"]
    r0 = next(t for t in timed if t["rank"] == 0)
    out = {"impl": impl, "value": tokens_per_step * args.steps / (ms / 1e3),
           "ms_per_step": ms / args.steps, "clocks": r0["clocks"], "launches": r0["launches"],
           "loss": next((t["loss"] for t in timed if t["loss"] is not None), None),
           "max_mem_gb": max(t["max_mem_gb"] for t in timed), "info": info[0],
           "tokens_per_step": tokens_per_step, "e2e": None}
    if e2e:
        for i in range(2):
            trainers.step.call(i).get(timeout=1800)
        trainers.sync.call().get(timeout=600)
        t0 = time.perf_counter()
        for i in range(args.steps):
            trainers.step.call(i).get(timeout=1800)
        trainers.sync.call().get(timeout=600)
        wall = time.perf_counter() - t0
        out["e2e"] = {"value": tokens_per_step * args.steps / wall, "unit": "tokens/s",
                      "ms_per_step": wall * 1e3 / args.steps,
                      "h2d_bytes_per_step": info[0]["h2d_bytes_per_step"],
                      "d2h_bytes_per_step": info[0]["d2h_bytes_per_step"],
                      "api": "attach_proc_mesh -> ProcMesh.spawn(TrainerActor) -> "
                             "trainers.step.call(i).get() per step (controller wall clock)"}
    trainers.release.call().get(timeout=600)
    return out


def main():
    args = parse()
    if args.impl == "reference":
        return reference_unavailable()

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not args.cpu:
        torch.cuda.set_device(local_rank)
        dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if args.cpu:
            dist.init_process_group("gloo")
        else:
            dist.init_process_group("nccl", device_id=dev)

    from monarch_b200.actor import attach_proc_mesh
    mesh, hosted = attach_proc_mesh({"gpus": world}, rank=rank, world=world)
    if mesh is None:
        # this rank hosts its proc of the mesh: its trainer actors run here until the
        # controller stops the mesh
        hosted.join()
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return 0

    from monarch_b200.models import PRESETS
    import re
    m_pp = re.fullmatch(r"pp(\d+)xtp(\d+)", args.parallelism)
    res = run_arm(mesh, args.impl, args, e2e=not args.no_e2e)
    base = None
    if args.impl == "ours" and not args.no_baseline and not m_pp and args.parallelism != "ep":
        base = run_arm(mesh, "aten", args, e2e=False)
    mesh.stop().get()
    hosted.join(timeout=60)

    cfg = PRESETS[args.model]
    S, B = args.seq, args.micro_batch
    par = res["info"]["parallelism"]
    if world > 1 and not m_pp:
        par = f"{par}{world}"
    per_gpu = res["tokens_per_step"] / world * args.steps / (res["ms_per_step"] * args.steps / 1e3)
    out = {
        "metric": "tokens/s Llama-3-8B FSDP-on-mesh" if args.model == "llama3-8b"
                  else f"tokens/s {args.model}",
        "value": res["value"], "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": (res["value"] / base["value"]) if base else None,
        "dtype": "bf16", "data": "synthetic", "impl": args.impl,
        "config": {"model": args.model,
                   "global_batch": args.microbatches * B if m_pp else B * world, "seq_len": S,
                   "parallelism": par,
                   "activation_checkpointing": True if args.recompute_layers is None else
                   f"first {args.recompute_layers} layers recomputed, the rest kept",
                   "optimizer": "AdamW fp32 master",
                   # what the parameter store actually runs (CPU ranks fall back to the library)
                   "comm": res["info"].get("comm") or args.comm,
                   **({"fsdp_gather": res["info"]["fsdp_gather"]} if par.startswith("fsdp") else {}),
                   "driven_by": "actor mesh over the launch's processes (attach_proc_mesh); "
                                "TrainerActor.timed_steps",
                   "l2": "per-step working set (>100 GB of weights and optimizer state) "
                         "is far larger than the 126 MB L2"},
        "clocks": res["clocks"], "e2e": res["e2e"], "gpu_launches": res["launches"],
        "loss": res["loss"], "max_mem_gb": res["max_mem_gb"],
        # model FLOPs (3x forward; recomputation not counted) and what the hardware executed
        "model_tflops_per_gpu": cfg.flops_per_token(S) * per_gpu / 1e12,
        "hardware_tflops_per_gpu": cfg.flops_per_token(S, recompute=True) * per_gpu / 1e12
        if args.recompute_layers is None else None,
        "baseline": None if base is None else {
            "impl": "aten: stock torch modules (cuBLAS, SDPA), autograd checkpointing, fused "
                    "torch AdamW on fp32 masters" + ("; fully_shard over NCCL" if world > 1 else ""),
            "value": base["value"], "unit": "tokens/s", "ms_per_step": base["ms_per_step"],
            "clocks": base["clocks"], "max_mem_gb": base["max_mem_gb"], "loss": base["loss"],
            "note": "same run, same processes, same steps/warm-up, measured after this "
                    "package's arm released its memory"},
    }
    print(json.dumps(out))
    sys.stdout.flush()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
