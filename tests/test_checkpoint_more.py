"""More of the checkpoint contract: weights-only (evaluation) load, buffers, logical vs physical shapes and source ranks
under tensor parallelism, ZeRO-3 bucket entries and their round trip on two ranks (the kinds of the reference's
``tests/tiny_transformer_tp_checkpoint_manifest.py`` and ``tests/tiny_model_zero3_checkpoint_roundtrip.py``)."""
import json

import torch
import torch.nn as nn

import maltos_b200  # noqa: F401
from maltos_b200.runtime import RuntimeCore
from maltos_b200.state import load_sharded_checkpoint, save_sharded_checkpoint
from tests.dist_utils import run_distributed


class _WithBuffer(nn.Module):
    def __init__(self):
        super().__init__()
        self.lin = nn.Linear(8, 8)
        self.register_buffer("seen", torch.zeros(3))

    def forward(self, x):
        self.seen += 1
        return self.lin(x).pow(2).mean()


def _rt():
    torch.manual_seed(1)
    rt = RuntimeCore(model=_WithBuffer(), optimizer_factory=lambda p: torch.optim.AdamW(p, lr=1e-2))
    rt.setup()
    return rt


def test_weights_only_load_restores_parameters_and_buffers_but_no_training_state(tmp_path):
    rt = _rt()
    for _ in range(2):
        rt.run_step(torch.randn(4, 8))
        rt.step_optimizer()
    ckpt = tmp_path / "step_00000002"
    save_sharded_checkpoint(rt.state_manager, ckpt)
    manifest = json.loads((ckpt / "manifest.json").read_text())
    keys = [e["state_key"] for e in manifest["ranks"][0]["entries"]]
    assert "seen" in keys and "lin.weight" in keys                                  # buffers are part of the model state

    evaluator = _rt()
    load_sharded_checkpoint(evaluator.state_manager, ckpt, weights_only=True)
    assert torch.equal(evaluator.model.lin.weight, rt.model.lin.weight)
    assert torch.equal(evaluator.model.seen, rt.model.seen) and float(evaluator.model.seen[0]) == 2.0
    assert evaluator.state.step_context.step == 0                                    # trainer state untouched
    opt, _ = evaluator.get_optimizer_and_scheduler()
    assert len(opt.state) == 0                                                       # optimizer state untouched

    resumed = _rt()
    load_sharded_checkpoint(resumed.state_manager, ckpt)
    assert resumed.state.step_context.step == 2
    opt, _ = resumed.get_optimizer_and_scheduler()
    assert len(opt.state) == 2 and all(int(s["step"]) == 2 for s in opt.state.values())
    # both continue identically from here
    x = torch.randn(4, 8)
    a, _ = rt.run_step(x.clone())
    b, _ = resumed.run_step(x.clone())
    assert torch.equal(a.detach(), b.detach())


def _sharded_case(rank, world, flags, root):
    from maltos_b200.train import cli, flags as F

    argv = ["--model", "llama", "--dim", "32", "--n-heads", "4", "--n-kv-heads", "2", "--hidden-size", "64", "--n-layers", "2", "--vocab-size", "64",
            "--seq-len", "16", "--micro-batch-size", "2", "--lr", "1e-2", "--seed", "3", "--precision", "fp32", "--disable-metrics", *flags]
    a = F.parse_args_from(argv, require_data=False)
    cli.validate_args(a, world)
    torch.manual_seed(a.seed)
    core = cli._build_runtime(a, cli._build_model(a), torch.device("cpu"))
    core.setup()
    core.model.train()
    g = torch.Generator().manual_seed(7)
    ids = torch.randint(0, 64, (2, 16), generator=g)
    batch = {"input_ids": ids, "labels": ids.roll(-1, 1)}
    losses = []
    for _ in range(2):
        loss, _ = core.run_step({k: v.clone() for k, v in batch.items()})
        core.step_optimizer()
        losses.append(float(loss.detach()))
    ckpt = f"{root}/step_00000002"
    save_sharded_checkpoint(core.state_manager, ckpt)
    loss3, _ = core.run_step({k: v.clone() for k, v in batch.items()})
    core.close()

    torch.manual_seed(99)                                                          # different init: everything must come from the checkpoint
    again = cli._build_runtime(a, cli._build_model(a), torch.device("cpu"))
    again.setup(checkpoint_path=ckpt)
    again.model.train()
    loss3_again, _ = again.run_step({k: v.clone() for k, v in batch.items()})
    again.close()
    manifest = json.loads(open(f"{ckpt}/manifest.json").read())
    return losses, float(loss3.detach()), float(loss3_again.detach()), manifest


def test_tensor_parallel_manifest_has_logical_and_physical_shapes(tmp_path):
    results = run_distributed(_sharded_case, 2, ["--tp-size", "2"], str(tmp_path))
    for losses, l3, l3_again, manifest in results:
        assert abs(l3 - l3_again) < 1e-6                                              # resume == continuous
    manifest = results[0][3]
    assert manifest["world_size"] == 2 and manifest["optimizer_source_ranks"] == [0, 1]
    for rank_entry in manifest["ranks"]:
        by_key = {e["state_key"]: e for e in rank_entry["entries"]}
        q = next(e for k, e in by_key.items() if k.endswith("q_proj.weight") or k.endswith("wq.weight"))
        assert q["logical_shapes"] == [[32, 32]] and q["physical_shape"] == [16, 32]  # column parallel: rows split
        o = next(e for k, e in by_key.items() if k.endswith("o_proj.weight") or k.endswith("wo.weight"))
        assert o["logical_shapes"] == [[32, 32]] and o["physical_shape"] == [32, 16]  # row parallel: columns split
        assert q["source_rank"] == rank_entry["rank"] and o["source_rank"] == rank_entry["rank"]   # shards: every rank writes its own
        norm = next(e for k, e in by_key.items() if "norm" in k and k.endswith("weight"))
        assert norm["source_rank"] == 0 and norm["logical_shapes"] == [norm["physical_shape"]]     # replicated: rank 0 writes


def test_zero3_checkpoint_roundtrip_on_two_ranks(tmp_path):
    results = run_distributed(_sharded_case, 2, ["--dp-size", "2", "--zero-stage", "3"], str(tmp_path))
    for losses, l3, l3_again, manifest in results:
        assert abs(l3 - l3_again) < 1e-6
    manifest = results[0][3]
    keys = [e["state_key"] for e in manifest["ranks"][0]["entries"]]
    buckets = [k for k in keys if k.startswith("zero3_bucket_")]
    assert buckets == [f"zero3_bucket_{i}" for i in range(len(buckets))] and buckets
    bucket = next(e for e in manifest["ranks"][1]["entries"] if e["state_key"] == "zero3_bucket_0")
    assert len(bucket["logical_names"]) == len(bucket["logical_shapes"]) >= 1
    assert len(bucket["physical_shape"]) == 1 and bucket["source_rank"] == 1          # a flat shard, written by its owner
    assert manifest["optimizer_source_ranks"] == [0, 1]


def _buffer_case(rank, world, zero_stage):
    from maltos_b200.train import cli, flags as F

    a = F.parse_args_from(["--model", "olmo2", "--dim", "16", "--n-heads", "4", "--hidden-size", "32", "--n-layers", "2", "--vocab-size", "32", "--seq-len", "8",
                           "--dp-size", "2", "--zero-stage", str(zero_stage), "--precision", "bf16"], require_data=False)
    core = cli._build_runtime(a, cli._build_model(a), torch.device("cpu"))
    core.setup()
    buffers = {n: (b.dtype, b.device.type) for n, b in core.model.named_buffers()}
    params = {p.dtype for p in core.model.parameters()}
    core.close()
    return buffers, params


def test_buffers_after_zero3_setup():
    """Buffers outside the sharded modules are materialised with the model (kind of the reference's
    ``tests/zero3_buffer_materialization.py``); the rotary tables stay fp32 here by design, the parameters are bf16."""
    for zero_stage in (0, 3):
        buffers, params = run_distributed(_buffer_case, 2, zero_stage)[0]
        rotary = {n: v for n, v in buffers.items() if n.endswith(("cos", "sin"))}
        assert len(rotary) >= 2 and all(v == (torch.float32, "cpu") for v in rotary.values()), rotary
        assert params == {torch.bfloat16}
