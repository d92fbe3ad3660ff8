"""Golden state transitions of pipeline-mode self-speculation, produced by the reference's
AsyncSpeculativeRunner._pipeline_step (vllm_rlt/worker/async_speculative.py:502-584).

    PYTHONPATH=<reference checkout> python tests/golden/make_golden_pipeline.py

The method is called unmodified on CPU tensors with stand-ins for the model (a seeded embedding,
a deterministic recurrent step and a small LM head, so that drafts are sometimes right and
sometimes wrong); every call's inputs — the per-request device state, the widths, the LM-head
choices and the hidden rows the step produced — and the state and wire buffer it left behind are
stored in `pipeline.pt`.
"""

from pathlib import Path
from types import SimpleNamespace

import torch

from vllm_rlt.worker.async_speculative import (AsyncSpeculativeRunner, DevicePipelineState,
                                               SpeculativeRequestState)

HERE = Path(__file__).resolve().parent


def main():
    torch.manual_seed(5)
    n, width, hidden_size, vocab, draft_loops, target_loops = 6, 4, 8, 6, 2, 4
    embedding = torch.randn(vocab, hidden_size)
    head = torch.randn(vocab, hidden_size)
    record = {}

    def forward(batch):
        return SimpleNamespace(hidden=embedding[batch.tokens])

    mix = torch.randn(8, hidden_size)

    def recurrent(hidden, positions, tables, depth, allocations, active):
        return torch.tanh(hidden * 0.7 + 0.25 * torch.roll(hidden, 1, dims=1) + 0.05 * mix[depth])

    def coda(hidden):
        record["step_hidden"] = hidden.clone()
        logits = hidden @ head.T
        record["choices"] = logits.argmax(-1).clone()
        return logits

    runner = SimpleNamespace(device=torch.device("cpu"),
                             config=SimpleNamespace(draft_loops=draft_loops, target_loops=target_loops),
                             runtime=SimpleNamespace(forward=forward), _execute_recurrent_step=recurrent, _coda=coda)
    prompts = [3, 9, 2, 5, 7, 4]
    max_tokens = [9, 4, 30, 2, 12, 6]
    states, spans = [], []
    for i in range(n):
        request = SimpleNamespace(prompt_token_ids=list(range(prompts[i])),
                                  sampling_params=SimpleNamespace(max_tokens=max_tokens[i]))
        pipeline = DevicePipelineState(tokens=torch.zeros(width, dtype=torch.long), depths=torch.zeros(width, dtype=torch.long),
                                       hidden=torch.zeros(width, hidden_size), candidates=torch.zeros(width, dtype=torch.long),
                                       active=torch.zeros(width, dtype=torch.bool))
        pipeline.tokens[0] = int(torch.randint(0, vocab, ()))
        pipeline.active[0] = True
        states.append(SpeculativeRequestState(request=request, allocation=None, token=pipeline.tokens[0].clone(),
                                              position=torch.tensor(prompts[i]), pipeline=pipeline))
        spans.append(SimpleNamespace(token_count=width, request=request))
    tables = torch.zeros(n, target_loops, 4, dtype=torch.int32)
    steps = []
    budgets = [4, 4, 3, 4, 2, 4, 4, 1, 4, 4, 4, 4, 4, 4, 4, 4, 4, 4, 4, 4, 4, 4, 4, 4]
    for budget in budgets:
        for span in spans:
            span.token_count = budget
        before = dict(
            tokens=torch.stack([s.pipeline.tokens for s in states]).clone(),
            depths=torch.stack([s.pipeline.depths for s in states]).clone(),
            hidden=torch.stack([s.pipeline.hidden for s in states]).clone(),
            candidates=torch.stack([s.pipeline.candidates for s in states]).clone(),
            active=torch.stack([s.pipeline.active for s in states]).clone(),
            token=torch.stack([s.token for s in states]).clone(),
            position=torch.stack([s.position for s in states]).clone())
        buffer = SimpleNamespace(result=torch.zeros(6 * n, dtype=torch.long))
        AsyncSpeculativeRunner._pipeline_step(runner, spans, states, tables, None, buffer)
        after = dict(
            tokens=torch.stack([s.pipeline.tokens for s in states]).clone(),
            depths=torch.stack([s.pipeline.depths for s in states]).clone(),
            hidden=torch.stack([s.pipeline.hidden for s in states]).clone(),
            candidates=torch.stack([s.pipeline.candidates for s in states]).clone(),
            active=torch.stack([s.pipeline.active for s in states]).clone(),
            token=torch.stack([s.token for s in states]).clone(),
            position=torch.stack([s.position for s in states]).clone(),
            result=buffer.result.clone())
        widths = torch.tensor([min(budget, width)] * n, dtype=torch.int32)
        steps.append(dict(before=before, after=after, widths=widths, choices=record["choices"],
                          step_hidden=record["step_hidden"]))
    limits = torch.tensor([prompts[i] + max_tokens[i] - 1 for i in range(n)])
    torch.save(dict(steps=steps, limits=limits, draft_loops=draft_loops, target_loops=target_loops), HERE / "pipeline.pt")
    emitted = sum(int(s["after"]["result"].view(n, 6)[:, 2].sum()) for s in steps)
    accepted = sum(int(s["after"]["result"].view(n, 6)[:, 1].sum()) for s in steps)
    print("steps", len(steps), "emitted", emitted, "accepted", accepted, (HERE / "pipeline.pt").stat().st_size)


if __name__ == "__main__":
    main()
