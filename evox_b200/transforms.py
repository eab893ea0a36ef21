"""Fitness transforms that plug into `StdWorkflow(fitness_transform=...)`
(the reference's plug point: evox/workflows/std_workflow.py:57-58, 102-115)."""

from __future__ import annotations

import torch


class CenteredRank(torch.nn.Module):
    """Replace fitness by its rank scaled to [-0.5, 0.5] (lowest fitness -> -0.5).

    The reference feeds raw fitness into the ES gradient (open_es.py:70, virtual_lora_es.py:115);
    the benchmark configuration asks for centred ranks, which this module adds without touching
    the algorithms. Ties keep index order (stable sort)."""

    def forward(self, fitness: torch.Tensor) -> torch.Tensor:
        n = fitness.numel()
        order = torch.argsort(fitness, stable=True)
        ranks = torch.empty_like(order)
        ranks[order] = torch.arange(n, device=fitness.device)
        return ranks.to(torch.float32) / max(n - 1, 1) - 0.5
