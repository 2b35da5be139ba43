"""Distributed layers: differentiable collectives, TP/SP linears, sharded norms, MoE and context-parallel cores."""
