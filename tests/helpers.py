"""Input generators shared by the tests (distributions follow the reference's tests and the benchmark
configurations: uniform top-k without replacement, softmax or |N(0,1)| weights, optional -1 masks)."""
import random

import torch


def make_routing(num_tokens, num_experts, num_topk, device, seed=0, masked_fraction=0.0, zipf_s=None):
    g = torch.Generator(device="cpu").manual_seed(seed)
    if zipf_s is None:
        scores = torch.rand(num_tokens, num_experts, generator=g)
    else:
        p = 1.0 / torch.arange(1, num_experts + 1, dtype=torch.float64) ** zipf_s
        scores = torch.log(p / p.sum()).float() - torch.log(-torch.log(torch.rand(num_tokens, num_experts, generator=g)))
    topk_idx = scores.topk(num_topk, dim=-1).indices.to(torch.int64)
    logits = torch.randn(num_tokens, num_topk, generator=g)
    topk_weights = torch.softmax(logits, dim=-1).float()
    if masked_fraction > 0:
        m = torch.rand(num_tokens, num_topk, generator=g) < masked_fraction
        topk_idx[m] = -1
    return topk_idx.to(device), topk_weights.to(device)


def make_tokens(num_tokens, hidden, device, seed=0):
    g = torch.Generator(device="cpu").manual_seed(1000 + seed)
    return torch.randn(num_tokens, hidden, generator=g).to(torch.bfloat16).to(device)
