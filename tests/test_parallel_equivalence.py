"""Data/pipeline/context/expert parallel runs on gloo ranks must reproduce single-process full-batch training
(loss, then parameters after two optimizer steps with gradient accumulation), fp32."""
import pytest
import torch

from tests.dist_utils import run_distributed

VOCAB, SEQ, ROWS = 96, 16, 4     # ROWS sequences per rank and micro-step
ACCUM, STEPS = 2, 2


def _model(kind: str):
    import maltos_b200  # noqa: F401
    from maltos_b200 import models

    torch.manual_seed(4321)
    if kind == "moe":
        return models.TinyMoETransformer(64, 4, 2, 128, 1e-5, 2, VOCAB, SEQ, 4, moe_aux_loss_coef=0.01)
    return models.TinyTransformer(64, 4, 2, 128, 1e-5, 2, VOCAB, SEQ)


def _data(n_shards: int):
    """[step][micro][shard] -> batch dict; identical in every process."""
    g = torch.Generator().manual_seed(99)
    out = []
    for _ in range(STEPS):
        micro = []
        for _ in range(ACCUM):
            ids = torch.randint(0, VOCAB, (n_shards * ROWS, SEQ), generator=g)
            labels = ids.roll(-1, 1)
            micro.append([{"input_ids": ids[i * ROWS:(i + 1) * ROWS], "labels": labels[i * ROWS:(i + 1) * ROWS]} for i in range(n_shards)])
        out.append(micro)
    return out


def _opt(params):
    return torch.optim.AdamW(params, lr=1e-2, weight_decay=0.01)


def _single(kind: str, n_shards: int, clip=None):
    model = _model(kind)
    opt = _opt(model.parameters())
    losses = []
    for step in _data(n_shards):
        opt.zero_grad(set_to_none=True)
        acc = 0.0
        for shards in step:
            for b in shards:
                out = model(b)
                loss = out.loss if hasattr(out, "loss") else out
                (loss / (ACCUM * n_shards)).backward()
                acc += float(loss.detach())
        if clip is not None:
            torch.nn.utils.clip_grad_norm_(model.parameters(), clip)
        opt.step()
        losses.append(acc / (ACCUM * n_shards))
    return losses, {n: p.detach().clone() for n, p in model.named_parameters()}


def _worker(rank, world, kind, mode, mesh_kw, clip):
    import maltos_b200  # noqa: F401
    from maltos_b200.parallel import ParallelPlan, PipelineScheduleConfig
    from maltos_b200.parallel.context_interfaces import ContextParallelAttentionCoreType
    from maltos_b200.runtime import MeshConfig, RuntimeCore
    from maltos_b200.runtime.plugins import cp, ddp, ep, grad_clip, pp, zero1, zero3

    model = _model(kind)
    mesh = MeshConfig(**mesh_kw)
    plan_kw = {}
    plugins = []
    grad_clip_max = None
    if mode in ("ddp_sync", "ddp_async"):
        plugins.append(ddp.DataParallelPlugin(async_op=mode == "ddp_async"))
    elif mode == "ddp_bucket":
        plugins.append(ddp.BucketDataParallelPlugin(bucket_mb_size=1))
    elif mode == "zero1":
        plugins.append(zero1.Zero1Plugin(bucket_mb_size=1))
    elif mode == "zero2":
        plugins.append(zero1.Zero2Plugin(bucket_mb_size=1))
    elif mode == "zero3":
        import torch.nn as nn

        from maltos_b200.models.tiny_transformer import RmsNorm

        plugins.append(zero3.Zero3Plugin(wrap_cls={nn.Linear, nn.Embedding, RmsNorm}))
    elif mode in ("pp_afab", "pp_1f1b"):
        plugins.append(pp.PipelineParallelPlugin(schedule="afab" if mode == "pp_afab" else "1f1b"))
        plan_kw["pp_schedule"] = PipelineScheduleConfig(microbatches=2)
    elif mode in ("cp_allgather", "cp_ring"):
        plugins.append(cp.ContextParallelPlugin())
        plan_kw["cp_attn_core"] = ContextParallelAttentionCoreType.RING if mode == "cp_ring" else ContextParallelAttentionCoreType.ALL_GATHER_KV
    elif mode == "ep":
        plugins += [ep.ExpertParallelPlugin(bucket_mb_size=1), ddp.DataParallelPlugin()]
    elif mode == "ep_zero2":
        plugins += [ep.ExpertParallelPlugin(), zero1.Zero2Plugin(bucket_mb_size=1)]
    if clip is not None:
        if mode.startswith("zero") or mode == "ep_zero2":
            grad_clip_max = clip
        else:
            plugins.append(grad_clip.GradClipPlugin(clip))
    rt = RuntimeCore(model=model, mesh=mesh, plan=ParallelPlan(**plan_kw), plugins=plugins, optimizer_factory=_opt,
                     grad_accum_steps=ACCUM, grad_clip_max_norm=grad_clip_max)
    rt.setup()
    dp_idx = mesh.rank_coordinates(rank)[0]
    losses = []
    for step in _data(mesh.dp):
        for shards in step:
            loss, should = rt.run_step(shards[dp_idx])
        assert should
        rt.step_optimizer()
        losses.append(rt.collect_metrics()["loss"])
    z3 = next((p for p in rt.plugins if isinstance(p, zero3.Zero3Plugin)), None)
    if z3 is not None:
        z3.materialize_model()
    params = {}
    for name, p in rt.model.named_parameters():
        entry = rt.state_manager.params.get(name)
        logical = entry.meta.logical_names[0] if entry is not None and len(entry.meta.logical_names) == 1 else name
        params[logical] = p.detach().clone()
    rt.close()
    return losses, params


CASES = [
    ("dense", "ddp_sync", dict(dp=2), None), ("dense", "ddp_async", dict(dp=2), 0.5), ("dense", "ddp_bucket", dict(dp=2), None),
    ("dense", "zero1", dict(dp=2), None), ("dense", "zero2", dict(dp=2), 0.5), ("dense", "zero3", dict(dp=2), None),
    ("dense", "pp_afab", dict(pp=2), None), ("dense", "pp_1f1b", dict(pp=2), None),
    ("dense", "cp_allgather", dict(cp=2), None), ("dense", "cp_ring", dict(cp=2), None),
    ("moe", "ep", dict(dp=2, ep=2), None), ("moe", "ep_zero2", dict(dp=2, ep=2), None),
]


@pytest.mark.parametrize("kind,mode,mesh_kw,clip", CASES, ids=[c[1] + ("_clip" if c[3] else "") for c in CASES])
def test_matches_single_process(kind, mode, mesh_kw, clip):
    n_shards = mesh_kw.get("dp", 1)
    ref_losses, ref_params = _single(kind, n_shards, clip)
    world = 1
    for v in (mesh_kw.get(k, 1) for k in ("dp", "tp", "pp", "cp")):
        world *= v
    results = run_distributed(_worker, world, kind, mode, mesh_kw, clip)
    # the reported loss is the mean over the accumulation window of this rank's micro-batches; PP/CP ranks see the global one
    if mesh_kw.get("cp", 1) > 1:
        # every CP rank differentiates its share (local mean x local/global targets) and reports cp x share, so that the mean
        # over the ranks is the loss of the whole rows
        total = [sum(r[0][i] for r in results) / len(results) for i in range(STEPS)]
        assert max(abs(a - b) for a, b in zip(total, ref_losses)) < 2e-4, (total, ref_losses)
    elif n_shards == 1:
        for losses, _ in results:
            assert max(abs(a - b) for a, b in zip(losses, ref_losses)) < 2e-4, (losses, ref_losses)
    seen = set()
    for rank, (_, params) in enumerate(results):
        for name, value in params.items():
            assert name in ref_params, name
            seen.add(name)
            diff = (value - ref_params[name]).abs().max().item()
            assert diff < 5e-4, f"{mode}: {name} on rank {rank} differs by {diff}"
    assert seen == set(ref_params), sorted(set(ref_params) - seen)
