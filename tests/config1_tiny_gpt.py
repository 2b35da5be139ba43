"""Runner of the plumbing benchmark as written: GPT-2-style tiny decoder (2 layers, d_model 64, 4 heads, GELU FFN 256,
LayerNorm, learned positions, vocab 512, tied embeddings), CPU / gloo world size 2, DP + ZeRO-1, fp32, sequence 64,
micro-batch 4 per rank, tokens uniform in [0, 512) from ``torch.manual_seed(0 + rank)``, AdamW lr 1e-3 wd 0.01, gradient
accumulation 2, clipping 1.0. Launched by ``tests/test_config1_tiny_gpt.py`` under ``torch.distributed.run``:

    python -m torch.distributed.run --nproc-per-node 2 tests/config1_tiny_gpt.py --impl ours|reference --steps 10 \
        [--save-at 6 --ckpt DIR] [--resume DIR/step_00000006]

``--impl reference`` runs the SAME model file under the reference's runtime (its ``RuntimeCore`` / ``Zero1Plugin`` from
the tree given by ``--reference-root``), which accepts any loss-returning module. Rank 0 prints one JSON line of losses.
"""
import argparse
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--reference-root", default=str(ROOT / "baseline" / "_ref"))
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--save-at", type=int, default=None)
    ap.add_argument("--ckpt", default=None)
    ap.add_argument("--resume", default=None)
    args = ap.parse_args()
    if args.impl == "reference":
        sys.path.insert(0, args.reference_root)           # `runtime`, `state`, ... resolve to the reference's packages
    sys.path.insert(1, str(ROOT))
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    from maltos_b200.models.gpt import GPTConfig, TinyGPT   # the model file is this framework's in both arms

    if args.impl == "reference":
        from runtime import MeshConfig, RuntimeCore
        from runtime.plugins.zero1 import Zero1Plugin
        from state import save_sharded_checkpoint
    else:
        from maltos_b200.runtime import MeshConfig, RuntimeCore
        from maltos_b200.runtime.plugins.zero1 import Zero1Plugin
        from maltos_b200.state import save_sharded_checkpoint

    torch.manual_seed(1234)                                 # identical initial weights on both ranks
    model = TinyGPT(GPTConfig())
    core = RuntimeCore(model=model, mesh=MeshConfig(dp=world), plugins=[Zero1Plugin(bucket_mb_size=25)], grad_accum_steps=2,
                       grad_clip_max_norm=1.0, optimizer_factory=lambda ps: torch.optim.AdamW(ps, lr=1e-3, weight_decay=0.01))
    core.setup(checkpoint_path=args.resume) if args.resume else core.setup()
    core.model.train()
    gen = torch.Generator().manual_seed(0 + rank)
    start = int(core.state.step_context.step)
    losses = []
    for step in range(args.steps):
        for _ in range(2):
            toks = torch.randint(0, 512, (4, 65), generator=gen)          # drawn for every step, so a resumed run sees the same stream
            if step < start:
                continue
            core.run_step({"input_ids": toks[:, :-1].contiguous(), "labels": toks[:, 1:].contiguous()})
        if step < start:
            continue
        core.step_optimizer()
        losses.append(float(core.collect_metrics()["loss"]))       # mean over the accumulation window
        if args.save_at is not None and step + 1 == args.save_at:
            save_sharded_checkpoint(core.state_manager, os.path.join(args.ckpt, f"step_{step + 1:08d}"))
    core.close()
    if rank == 0:
        print("LOSSES " + json.dumps(losses), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
