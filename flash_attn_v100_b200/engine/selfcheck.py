"""Consistency check of the tensor-parallel decoder on the GPUs of a running job.

`tp_consistency_check` generates a few tokens with a small model split over all ranks (decode step on the
library's peer-memory collectives, replayed from one CUDA graph) and compares this rank's vocabulary shard of
the logits with a single-rank run of the same weights on the same GPU.  It is the check the reference makes in
test_multi_gpu.py:672-727 (tensor-parallel result == single-GPU result), sized to run in seconds so that a
multi-GPU benchmark run can carry its outcome."""
from __future__ import annotations

import torch

from .config import ModelConfig
from .model import TPDecoder
from .runner import GenerationRunner
from .weights import make_rank_weights


def check_config() -> ModelConfig:
    """Two layers, eight KV heads: divisible by every tensor-parallel size up to 8."""
    return ModelConfig(num_layers=2, hidden_size=512, num_heads=16, num_kv_heads=8, head_dim=64,
                       intermediate_size=1024, vocab_size=2048)


def tp_consistency_check(rank: int, world: int, device, tol: float = 3e-2, new_tokens: int = 8) -> dict:
    import torch.distributed as dist
    cfg = check_config()
    dev = torch.device(device)
    prompts = torch.randint(0, cfg.vocab_size, (4, 21), generator=torch.Generator().manual_seed(17))
    w_tp = make_rank_weights(cfg, rank, world, 9, dev, gen_device="cpu")
    tp = GenerationRunner(TPDecoder(cfg, w_tp, rank, world, None, dev), 4, 64, peer_collectives=True)
    logs_tp = []
    toks_eager = tp.generate(prompts, new_tokens, logits_out=logs_tp)     # eager, logits kept
    toks_graph = tp.generate(prompts, new_tokens)                         # captured, then replayed
    toks_again = tp.generate(prompts, new_tokens)
    torch.cuda.synchronize(dev)
    tp.model.comm.check()
    tp.close()
    replay_equal = bool(torch.equal(toks_graph, toks_eager) and torch.equal(toks_again, toks_eager))
    w_1 = make_rank_weights(cfg, 0, 1, 9, dev, gen_device="cpu")
    one = GenerationRunner(TPDecoder(cfg, w_1, 0, 1, None, dev), 4, 64, use_cuda_graph=False)
    logs_1 = []
    toks_1 = one.generate(prompts, new_tokens, logits_out=logs_1)
    torch.cuda.synchronize(dev)
    vl = cfg.vocab_size // world
    err = (logs_tp[0][2] - logs_1[0][2][:, rank * vl:(rank + 1) * vl]).abs().max().item()
    # decode steps: only while the two runs still feed the same tokens (a random model has near-ties)
    same_prefix = (toks_eager == toks_1).long().cumprod(dim=1)
    err_dec = 0.0
    for i in range(1, len(logs_tp)):
        keep = same_prefix[:, i - 1].bool()
        if keep.any():
            a = logs_tp[i][2][keep]
            b = logs_1[i][2][keep][:, rank * vl:(rank + 1) * vl]
            err_dec = max(err_dec, (a - b).abs().max().item())
    ok = replay_equal and err < tol and err_dec < tol
    stats = torch.tensor([1.0 if ok else 0.0, -err, -err_dec], device=dev)
    dist.all_reduce(stats, op=dist.ReduceOp.MIN)
    return {"ok": bool(stats[0].item() == 1.0), "tp": world, "first_token_logit_err": -stats[1].item(),
            "decode_logit_err": -stats[2].item(), "tolerance": tol, "graph_replay_equals_eager": replay_equal,
            "token_agreement_with_one_gpu": (toks_eager == toks_1).float().mean().item(),
            "model": "2 layers, hidden 512, 16/8 heads of 64, vocabulary 2048; 4 prompts of 21 tokens, "
                     f"{new_tokens} new tokens; decode step on the peer-memory collectives in one CUDA graph"}
