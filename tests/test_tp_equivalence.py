"""TP and TP+SP on 2 gloo ranks must reproduce the single-process loss and gradients (fp32)."""
import pytest
import torch

from tests.dist_utils import run_distributed


def _make_model(kind: str, variant: str):
    import maltos_b200  # noqa: F401
    from maltos_b200 import models

    torch.manual_seed(1234)
    if kind == "tiny":
        cls = {"base": models.TinyTransformer, "tp": models.TinyTransformerTp, "sp": models.TinyTransformerTpSp}[variant]
        return cls(64, 4, 2, 128, 1e-5, 2, 96, 32)
    if kind == "llama":
        cls = {"base": models.LlamaForCausalLM, "tp": models.LlamaForCausalLMTp, "sp": models.LlamaForCausalLMTpSp}[variant]
        return cls(models.LlamaConfig(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32))
    cls = {"base": models.OlmoForCausalLM, "tp": models.OlmoForCausalLMTp, "sp": models.OlmoForCausalLMTpSp}[variant]
    return cls(models.OlmoConfig(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                 num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32))


def _batch():
    g = torch.Generator().manual_seed(7)
    ids = torch.randint(0, 96, (2, 16), generator=g)
    labels = ids.roll(-1, 1).clone()
    labels[0, :3] = -100
    return {"input_ids": ids, "labels": labels}


def _worker(rank, world, kind, variant):
    import maltos_b200  # noqa: F401
    from maltos_b200.runtime import MeshConfig, RuntimeCore
    from maltos_b200.runtime.plugins.tp import TensorParallelPlugin
    from maltos_b200.runtime.plugins.tp_sp import TpSpPlugin

    model = _make_model(kind, variant)
    plugin = TensorParallelPlugin() if variant == "tp" else TpSpPlugin()
    rt = RuntimeCore(model=model, mesh=MeshConfig(tp=world), plugins=[plugin], optimizer_factory=lambda p: torch.optim.SGD(p, lr=0.0))
    rt.setup()
    loss, should = rt.run_step(_batch())
    rt._run_step_phase(__import__("maltos_b200").runtime.types.RuntimePhase.PRE_STEP)
    grads = {}
    for name, entry in rt.state_manager.params.items():
        grads[name] = (entry.param.grad.detach().clone(), entry.meta.logical_shapes[0], entry.meta.physical_shape)
    out = (float(loss), grads)
    rt.close()
    return out


@pytest.mark.parametrize("kind", ["tiny", "llama", "olmo"])
@pytest.mark.parametrize("variant", ["tp", "sp"])
def test_tp_matches_single_process(kind, variant):
    base = _make_model(kind, "base")
    loss = base(_batch())
    loss.backward()
    ref = {n: p.grad.detach().clone() for n, p in base.named_parameters()}
    results = run_distributed(_worker, 2, kind, variant)
    for rank, (l, grads) in enumerate(results):
        assert abs(l - float(loss)) < 1e-5, (l, float(loss))
        for name, (g, logical, physical) in grads.items():
            full = ref[name]
            if tuple(logical) != tuple(physical):
                dim = [i for i, (a, b) in enumerate(zip(logical, physical)) if a != b][0]
                per = physical[dim]
                full = full.narrow(dim, rank * per, per)
            assert torch.allclose(g, full, atol=2e-5, rtol=1e-4), f"{name} rank {rank} max diff {(g - full).abs().max()}"
