"""A micro-step (forward + backward) recorded into a CUDA graph replays with the same loss and gradients as eager
execution, accumulates gradients across replays, and costs fewer host launches."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def _model():
    import maltos_b200  # noqa: F401
    from maltos_b200.models import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=2048, hidden_size=256, intermediate_size=704, num_hidden_layers=4, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=256, rms_norm_eps=1e-5)
    return cfg, LlamaForCausalLM(cfg).cuda().bfloat16()


def _batch(cfg, seed):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, cfg.vocab_size, (2, 256), generator=g)
    return {"input_ids": ids.cuda(), "labels": ids.roll(-1, 1).cuda()}


def _loss(model, batch):
    out = model(batch)
    return out.loss if hasattr(out, "loss") else out


def test_graphed_micro_step_matches_eager_and_accumulates():
    from maltos_b200.ops import _lib
    from maltos_b200.utils.cuda_graph import GraphedMicroStep

    cfg, model = _model()
    params = list(model.parameters())
    b1, b2 = _batch(cfg, 1), _batch(cfg, 2)
    # eager: two micro-steps accumulated
    for p in params:
        p.grad = None
    l1 = _loss(model, b1)
    (l1 * 0.5).backward()
    l2 = _loss(model, b2)
    (l2 * 0.5).backward()
    eager = [p.grad.detach().float().clone() for p in params]
    eager_losses = (l1.item(), l2.item())
    del l1, l2           # a live eager graph keeps its gradient-accumulation nodes bound to the stream they ran on
    for p in params:
        p.grad = None
    step = GraphedMicroStep(lambda batch: _loss(model, batch), params, b1, loss_scale=0.5)
    assert all(p.grad is None for p in params)                          # warm-up and capture left no trace
    g1 = float(step(b1))
    g2 = float(step(b2))
    torch.cuda.synchronize()
    assert abs(g1 - eager_losses[0]) < 1e-3 and abs(g2 - eager_losses[1]) < 1e-3
    for p, e in zip(params, eager):
        assert (p.grad.float() - e).abs().max().item() <= 2e-2 * max(1e-3, e.abs().max().item())
    assert _lib.fetch_status(raise_on_error=False)[0] == 0
    with pytest.raises(ValueError):
        step({"input_ids": b1["input_ids"][:1], "labels": b1["labels"][:1]})

    # host cost: one replay against a few hundred launches
    def timed(fn, n=10):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / n * 1e3

    def eager_step():
        (_loss(model, b1) * 0.5).backward()

    t_eager, t_graph = timed(eager_step), timed(lambda: step(b1))
    print(f"micro-step wall time: eager {t_eager:.2f} ms, graph replay {t_graph:.2f} ms")
    assert t_graph < t_eager * 1.2


def test_cuda_graph_plugin_reproduces_eager_training():
    """Same model, data and optimizer with and without the plugin: losses agree, and after the eager lead-in every
    micro-step is a replay."""
    import maltos_b200  # noqa: F401
    from maltos_b200.models import LlamaConfig, LlamaForCausalLM
    from maltos_b200.runtime import RuntimeCore
    from maltos_b200.runtime.optim import FusedAdamW
    from maltos_b200.runtime.plugins.cuda_graph import CudaGraphPlugin

    def train(graphed):
        torch.manual_seed(0)
        cfg = LlamaConfig(vocab_size=2048, hidden_size=256, intermediate_size=704, num_hidden_layers=2, num_attention_heads=4,
                          num_key_value_heads=2, max_position_embeddings=128, rms_norm_eps=1e-5)
        plugin = CudaGraphPlugin(eager_steps=2) if graphed else None
        rt = RuntimeCore(model=LlamaForCausalLM(cfg), device=torch.device("cuda", 0), dtype=torch.bfloat16, grad_accum_steps=2,
                         plugins=[plugin] if plugin else [], optimizer_factory=lambda p: FusedAdamW(p, lr=1e-3, betas=(0.9, 0.95)))
        rt.setup()
        g = torch.Generator().manual_seed(5)
        losses = []
        for _ in range(4):
            for _ in range(2):
                ids = torch.randint(0, cfg.vocab_size, (2, 128), generator=g)
                rt.run_step({"input_ids": ids, "labels": ids.roll(-1, 1)})
            rt.step_optimizer()
            losses.append(float(rt.collect_metrics()["loss"]))
        replays = plugin.runner.replays if plugin else 0
        rt.close()
        return losses, replays

    eager, _ = train(False)
    graphed, replays = train(True)
    assert replays == 6                                     # 8 micro-steps, the first two eager
    assert max(abs(a - b) for a, b in zip(eager, graphed)) < 3e-2, (eager, graphed)
