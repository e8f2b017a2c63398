"""Helpers shared by the session-level metrics: rank of every example inside its session."""
from __future__ import annotations

import torch


def ranking_within_session(predictions: torch.Tensor, session: torch.Tensor) -> torch.Tensor:
    """0-based rank (0 = highest prediction) of every example among the examples with the same session id.
    ``predictions`` and ``session`` are 1-D (or ``[1, n]``)."""
    p = predictions.view(-1).double()
    s = session.view(-1)
    n = p.numel()
    # sort by (session, -prediction), then rank = position - start of the session's run
    order = torch.argsort(-p, stable=True)
    order = order[torch.argsort(s[order], stable=True)]
    ss = s[order]
    new_run = torch.ones(n, dtype=torch.bool, device=p.device)
    new_run[1:] = ss[1:] != ss[:-1]
    pos = torch.arange(n, device=p.device)
    run_start = torch.cummax(torch.where(new_run, pos, torch.zeros_like(pos)), 0).values
    ranks = torch.empty(n, dtype=torch.long, device=p.device)
    ranks[order] = pos - run_start
    return ranks.view(predictions.shape)
