"""Unit tests of framework components that need neither a GPU nor several processes: data loaders and their resume
state, the buffer pool, metric aggregation and formatting, master-weights optimizer, plugin ordering, losses."""
import json

import numpy as np
import pytest
import torch
import torch.nn as nn

from maltos_b200.data.prefetch import PrefetchDataLoader
from maltos_b200.data.pretrain import PretrainingDataLoader, TokenShardDataset
from maltos_b200.data.simple import SimpleTensorDataLoader
from maltos_b200.runtime.buffer_allocator import BufferPolicy, BufferPool
from maltos_b200.runtime.optim import MasterWeightsOptimizer
from maltos_b200.utils import metrics as M
from maltos_b200.utils.constants import IGNORE_INDEX
from maltos_b200.utils.losses import causal_cross_entropy


@pytest.fixture()
def shards(tmp_path):
    rng = np.random.default_rng(0)
    sizes = [1000, 777, 1303]
    for i, n in enumerate(sizes):
        rng.integers(0, 5000, size=n, dtype=np.uint32).tofile(tmp_path / f"tokens_{i:05d}.bin")
    return sorted(tmp_path.glob("*.bin"))


# ------------------------------------------------------------------------------------------------ data loaders
def test_token_shard_loader_dp_interleave_and_wraparound(shards):
    flat = np.concatenate([np.fromfile(p, dtype=np.uint32) for p in shards]).astype(np.int64)
    seq, mb, world = 16, 2, 2
    loaders = [PretrainingDataLoader(TokenShardDataset(shards), seq_len=seq, micro_batch_size=mb, dp_rank=r, dp_world_size=world) for r in range(world)]
    sample = seq + 1
    for step in range(60):          # more than one pass over 3080 tokens -> wraps around
        for r, ld in enumerate(loaders):
            b = ld.next_batch()
            for i in range(mb):
                k = (step * mb + i) * world + r            # global sample index: ranks interleave sample by sample
                want = flat[np.arange(k * sample, (k + 1) * sample) % flat.size]
                assert torch.equal(b["input_ids"][i], torch.from_numpy(want[:-1]))
                assert torch.equal(b["labels"][i], torch.from_numpy(want[1:]))
    assert loaders[0].consumed_tokens == 60 * mb * seq


def test_token_shard_loader_resume_and_validation(shards):
    ds = TokenShardDataset(shards)
    a = PretrainingDataLoader(ds, seq_len=32, micro_batch_size=3, dp_rank=1, dp_world_size=2)
    for _ in range(7):
        a.next_batch()
    state = json.loads(json.dumps(a.state_dict().__dict__))      # survives a JSON round trip
    b = PretrainingDataLoader(ds, seq_len=32, micro_batch_size=3, dp_rank=1, dp_world_size=2)
    b.load_state_dict(state)
    for _ in range(5):
        x, y = a.next_batch(), b.next_batch()
        assert torch.equal(x["input_ids"], y["input_ids"]) and torch.equal(x["labels"], y["labels"])
    with pytest.raises(ValueError):
        b.load_state_dict({**state, "shard_idx": 9})
    with pytest.raises(ValueError):
        PretrainingDataLoader(ds, seq_len=0, micro_batch_size=1)
    with pytest.raises(ValueError):
        PretrainingDataLoader(ds, seq_len=8, micro_batch_size=1, dp_rank=2, dp_world_size=2)
    with pytest.raises(RuntimeError):
        a.next_batch(cp_rank=0)          # CP-local batches need a sharder


def test_prefetch_loader_is_transparent_and_resumable(shards):
    ds = TokenShardDataset(shards)
    plain = PretrainingDataLoader(ds, seq_len=16, micro_batch_size=2)
    pre = PrefetchDataLoader(PretrainingDataLoader(ds, seq_len=16, micro_batch_size=2))
    for _ in range(4):
        assert torch.equal(plain.next_batch()["input_ids"], pre.next_batch()["input_ids"])
    state = pre.state_dict()             # must describe the batches CONSUMED, not the one already prefetched
    state = state if isinstance(state, dict) else state.__dict__
    again = PrefetchDataLoader(PretrainingDataLoader(ds, seq_len=16, micro_batch_size=2))
    again.load_state_dict(dict(state))
    for _ in range(3):
        want = plain.next_batch()["input_ids"]
        assert torch.equal(pre.next_batch()["input_ids"], want) and torch.equal(again.next_batch()["input_ids"], want)
    pre.close()
    again.close()


def test_simple_loader_epochs_and_resume():
    data = torch.arange(10 * 3).view(10, 3)
    a = SimpleTensorDataLoader(data, batch_size=4)
    seen = [a.next_batch() for _ in range(5)]
    assert all(b.shape[0] == 4 for b in seen)
    st = a.state_dict()
    b = SimpleTensorDataLoader(data, batch_size=4)
    b.load_state_dict(st.__dict__ if not isinstance(st, dict) else st)
    assert torch.equal(a.next_batch(), b.next_batch())


# ------------------------------------------------------------------------------------------------ buffer pool
def test_buffer_pool_policies_alignment_and_coalescing():
    pool = BufferPool()
    h1 = pool.acquire(shape=(10,), dtype=torch.float32, device="cpu", policy=BufferPolicy.PINNED, key="k")
    h2 = pool.acquire(shape=(10,), dtype=torch.float32, device="cpu", policy="pinned", key="k")
    assert h1 is h2                                   # keyed buffers persist
    with pytest.raises(ValueError):
        pool.acquire(shape=(1,), dtype=torch.float32, device="cpu", policy=BufferPolicy.PINNED)
    with pytest.raises(ValueError):
        pool.acquire(shape=(1,), dtype=torch.float32, device="cpu", policy=BufferPolicy.TEMPORARY, key="x")
    a = pool.acquire(shape=(100,), dtype=torch.float32, device="cpu", policy=BufferPolicy.TEMPORARY)
    b = pool.acquire(shape=(3, 5), dtype=torch.bfloat16, device="cpu", policy=BufferPolicy.TEMPORARY)
    c = pool.acquire(shape=(7,), dtype=torch.int64, device="cpu", policy=BufferPolicy.TEMPORARY)
    assert a.start % 256 == b.start % 256 == c.start % 256 == 0 and len({a.start, b.start, c.start}) == 3
    assert b.tensor.shape == (3, 5) and b.tensor.dtype == torch.bfloat16
    reserved = pool.reserved_bytes()
    for h in (a, c, b):                               # out of order: free segments must merge again
        pool.release(h)
    with pytest.raises(ValueError):
        pool.release(a)
    big = pool.acquire(shape=(a.alloc_numel + b.alloc_numel + c.alloc_numel,), dtype=torch.uint8, device="cpu", policy=BufferPolicy.TEMPORARY)
    assert big.start == 0 and pool.reserved_bytes() == reserved      # served from the same slab, nothing new reserved
    pool.clear()
    assert pool.reserved_bytes() == 0


# ------------------------------------------------------------------------------------------------ metrics
def test_metric_rules_and_console_format(tmp_path):
    agg = M.MetricAggregator()
    agg.update({"loss": 2.0, "lr": 1e-3, "step": 1, "tokens": 100, "overflow": False})
    agg.update({"loss": 4.0, "lr": 5e-4, "step": 2, "tokens": 50, "overflow": True})
    out = agg.flush(step_delta=2)
    assert out["loss"] == pytest.approx(3.0) and out["lr"] == 5e-4 and out["step"] == 2
    assert not agg.has_values()
    line = M._format_metrics({"step": 7, "loss": 1.234567, "lr": 3e-4, "perf/step_sec": 34.0181, "train/tokens_per_sec": 7706.0,
                              "perf/tflops_per_gpu": 86.0, "memory/allocated_gb": 53.0, "memory/max_allocated_gb": 64.6})
    assert line == "[step 00007] loss 1.23457 | lr 3.00e-04 | step 34.02s | throughput 7,706 tok/s | compute 86.0 TF/GPU | memory 53.0/64.6 GiB"
    assert M._format_metrics({"b": 1, "a": 0.5}) == "a=0.5 b=1"
    sink = M.JsonlMetricLogger(tmp_path / "m.jsonl")
    sink.log({"step": 1, "loss": 0.5})
    sink.log({"step": 2, "loss": 0.25})
    rows = [json.loads(l) for l in (tmp_path / "m.jsonl").read_text().splitlines()]
    assert [r["step"] for r in rows] == [1, 2]


# ------------------------------------------------------------------------------------------------ optimizer wrapper
def test_master_weights_optimizer_keeps_fp32_masters_and_roundtrips_state():
    torch.manual_seed(0)
    lin = nn.Linear(8, 4).to(torch.bfloat16)
    ref = nn.Linear(8, 4)
    ref.load_state_dict({k: v.float() for k, v in lin.state_dict().items()})
    opt = MasterWeightsOptimizer(lin.parameters(), optimizer_factory=lambda ps: torch.optim.AdamW(ps, lr=1e-2, weight_decay=0.0))
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.0)
    x = torch.randn(16, 8)
    for _ in range(3):
        lin(x.bfloat16()).float().pow(2).mean().backward()
        opt.step()
        opt.zero_grad()
        g = [p.grad for p in lin.parameters()]
        assert all(gi is None or float(gi.abs().sum()) == 0 for gi in g)
    masters = [p for group in opt.inner.param_groups for p in group["params"]]
    assert all(p.dtype == torch.float32 for p in masters)
    for p, m in zip(lin.parameters(), masters):
        assert torch.equal(p.detach(), m.detach().to(torch.bfloat16))       # the model weight is the rounded master
    state = opt.state_dict()
    assert {"inner_optimizer", "master_params"} <= set(state)
    lin2 = nn.Linear(8, 4).to(torch.bfloat16)
    opt2 = MasterWeightsOptimizer(lin2.parameters(), optimizer_factory=lambda ps: torch.optim.AdamW(ps, lr=1e-2, weight_decay=0.0))
    opt2.load_state_dict(state)
    m2 = [p for group in opt2.inner.param_groups for p in group["params"]]
    assert all(torch.equal(a, b) for a, b in zip(masters, m2))
    del ropt


# ------------------------------------------------------------------------------------------------ plugin ordering, loss
def test_plugin_topological_order_and_cycle_detection():
    from maltos_b200.runtime.core import order_plugins
    from maltos_b200.runtime.plugin import PluginId, RuntimePlugin

    a = RuntimePlugin(id=PluginId.DP, runs_after={PluginId.TP})
    b = RuntimePlugin(id=PluginId.TP)
    c = RuntimePlugin(id=PluginId.METRICS, runs_after={PluginId.DP})
    assert [p.id for p in order_plugins([c, a, b])] == [PluginId.TP, PluginId.DP, PluginId.METRICS]
    with pytest.raises(ValueError):
        order_plugins([RuntimePlugin(id=PluginId.DP, runs_after={PluginId.TP}), RuntimePlugin(id=PluginId.TP, runs_after={PluginId.DP})])
    with pytest.raises(ValueError):
        order_plugins([RuntimePlugin(id=PluginId.DP, requires={PluginId.TP})])


def test_causal_cross_entropy_ignores_and_normalises():
    torch.manual_seed(0)
    logits = torch.randn(2, 5, 11)
    labels = torch.randint(0, 11, (2, 5))
    labels[0, :2] = IGNORE_INDEX
    want = torch.nn.functional.cross_entropy(logits.view(-1, 11), labels.view(-1), ignore_index=IGNORE_INDEX, reduction="sum") / 8
    assert torch.allclose(causal_cross_entropy(logits, labels), want)
    assert float(causal_cross_entropy(logits, torch.full((2, 5), IGNORE_INDEX))) == 0.0
