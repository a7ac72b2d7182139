"""Shared by tests/golden/make_golden.py and tests/test_plain.py: one golden case."""
import torch

import plain_gpt2 as P
from tiny_configs import make_model

WORKLOADS = {
    # workloads of the two tiny configurations: prompt lengths and greedy steps
    "A": ([5, 9, 13], 8),
    "B": ([1, 17], 12),
}


def prompts_for(name, vocab):
    g = torch.Generator().manual_seed({"A": 101, "B": 202}[name])
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in WORKLOADS[name][0]]


def build_case(name, root):
    d = make_model(root, name)
    W = P.PlainWeights(d)
    prompts = prompts_for(name, W.cfg["vocab_size"])
    n_new = WORKLOADS[name][1]
    logits = P.forward_logits(W, prompts[-1])[-1]
    return {
        "config": name, "prompts": prompts,
        "greedy": [P.greedy_generate(W, p, n_new) for p in prompts],
        "argmax": int(torch.argmax(logits)),
        "last_logits_head": [float(v) for v in logits[:4]],
        "last_logits_tail": [float(v) for v in logits[-4:]],
        "last_logits_sum": float(logits.sum()),
    }
