"""GPU: the decoder engine slice against the eager fp32 restatement of the same block on the same
seeded weights (tiny shape).  Logits of every step are compared with teacher forcing on the engine's
own tokens (tolerance 3e-2 absolute: bf16 GEMMs and bf16 activations against fp32); the greedy token
must agree wherever the oracle's top-2 margin exceeds twice that tolerance.  CUDA-graph replay must
reproduce the eager tokens exactly."""
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 3e-2


def _setup(seed=5):
    from flash_attn_v100_b200.engine import GenerationRunner, TPDecoder, make_rank_weights, tiny_config
    cfg = tiny_config()
    w = make_rank_weights(cfg, 0, 1, seed, "cuda", gen_device="cpu")
    model = TPDecoder(cfg, w)
    return cfg, model, GenerationRunner


def test_engine_matches_oracle_logits_and_tokens():
    from oracle import model_oracle as mo
    cfg, model, Runner = _setup()
    g = torch.Generator().manual_seed(3)
    B, P, N = 3, 21, 12
    prompts = torch.randint(0, cfg.vocab_size, (B, P), generator=g)
    logs = []
    runner = Runner(model, max_batch=4, max_seq_len=64, use_cuda_graph=False)
    toks = runner.generate(prompts, N, prefill_chunk=2, logits_out=logs).cpu()
    torch.cuda.synchronize()
    # engine logits per generated position
    pre = torch.cat([lg for kind, _, lg in logs if kind == "prefill"]).cpu()            # [B, vocab]
    dec = [lg.cpu() for kind, _, lg in logs if kind == "decode"]                         # N-1 x [B, vocab]
    eng = torch.stack([pre] + dec, dim=1)                                                # [B, N, vocab]
    full = torch.cat([prompts, toks[:, :-1]], dim=1)
    ref = mo.forward_logits(cfg, 5, full)[:, P - 1:]                                     # teacher forcing
    assert eng.shape == ref.shape
    err = (eng - ref).abs().max().item()
    assert err < TOL, err
    top2 = ref.topk(2, dim=-1).values
    confident = (top2[..., 0] - top2[..., 1]) > 2 * TOL
    assert (toks[confident] == ref.argmax(-1)[confident]).all()
    assert confident.float().mean().item() > 0.2        # the check is not vacuous
    import flash_attn_v100_b200 as pkg
    pkg.check_async_errors(); pkg.check_prefill_errors()


def test_engine_with_bfloat16_attention_matches_oracle_logits():
    """The same comparison with q / k / v and the KV pages in bfloat16 (the library's *_bf16 twins): no cast to
    fp16 anywhere in the block."""
    from oracle import model_oracle as mo
    cfg, model, Runner = _setup()
    model.attn_dtype = torch.bfloat16
    g = torch.Generator().manual_seed(3)
    B, P, N = 3, 21, 12
    prompts = torch.randint(0, cfg.vocab_size, (B, P), generator=g)
    logs = []
    runner = Runner(model, max_batch=4, max_seq_len=64, use_cuda_graph=False)
    assert runner.kv.k_pools[0].dtype == torch.bfloat16
    toks = runner.generate(prompts, N, prefill_chunk=2, logits_out=logs).cpu()
    torch.cuda.synchronize()
    pre = torch.cat([lg for kind, _, lg in logs if kind == "prefill"]).cpu()
    dec = [lg.cpu() for kind, _, lg in logs if kind == "decode"]
    eng = torch.stack([pre] + dec, dim=1)
    full = torch.cat([prompts, toks[:, :-1]], dim=1)
    ref = mo.forward_logits(cfg, 5, full)[:, P - 1:]
    err = (eng - ref).abs().max().item()
    assert err < TOL, err
    top2 = ref.topk(2, dim=-1).values
    confident = (top2[..., 0] - top2[..., 1]) > 2 * TOL
    assert (toks[confident] == ref.argmax(-1)[confident]).all()
    # graph replay reproduces the eager tokens in this mode too
    r2 = Runner(model, max_batch=4, max_seq_len=64, use_cuda_graph=True)
    assert torch.equal(r2.generate(prompts, N, prefill_chunk=2).cpu(), toks)
    import flash_attn_v100_b200 as pkg
    pkg.check_async_errors(); pkg.check_prefill_errors()


def test_fused_qkv_kernel_is_bit_identical_to_the_two_kernels_it_replaces():
    """QK-norm + cast + rotary + append in one launch against the norm kernel followed by the rotary/append
    kernel: the same tokens and bit-identical logits, prompts (packed) and decode steps, and bit-identical
    cache pages."""
    cfg, model, Runner = _setup(seed=11)
    g = torch.Generator().manual_seed(6)
    prompts = torch.randint(0, cfg.vocab_size, (3, 37), generator=g)
    out = {}
    for fused in (True, False):
        model.fused_qkv = fused
        logs = []
        r = Runner(model, max_batch=4, max_seq_len=64, use_cuda_graph=False)
        toks = r.generate(prompts, 9, prefill_chunk=2, logits_out=logs)
        torch.cuda.synchronize()
        out[fused] = (toks.clone(), [lg.clone() for _, _, lg in logs], [kp.clone() for kp in r.kv.k_pools],
                      [vp.clone() for vp in r.kv.v_pools])
    model.fused_qkv = True
    assert torch.equal(out[True][0], out[False][0])
    for a, b in zip(out[True][1], out[False][1]):
        assert torch.equal(a, b)
    for a, b in zip(out[True][2] + out[True][3], out[False][2] + out[False][3]):
        assert torch.equal(a, b)
    import flash_attn_v100_b200 as pkg
    pkg.check_async_errors(); pkg.check_prefill_errors()


def test_cuda_graph_replay_reproduces_eager_tokens():
    cfg, model, Runner = _setup(seed=7)
    g = torch.Generator().manual_seed(4)
    prompts = torch.randint(0, cfg.vocab_size, (4, 33), generator=g)
    eager = Runner(model, max_batch=4, max_seq_len=80, use_cuda_graph=False).generate(prompts, 24)
    r = Runner(model, max_batch=4, max_seq_len=80, use_cuda_graph=True)
    graphed = r.generate(prompts, 24)
    again = r.generate(prompts, 24)                 # second call replays the cached graph only
    torch.cuda.synchronize()
    assert torch.equal(eager, graphed) and torch.equal(eager, again)
    import flash_attn_v100_b200 as pkg
    pkg.check_async_errors(); pkg.check_prefill_errors()


def test_two_rank_tensor_parallel_matches_single_rank():
    """TP=2 over NCCL (two GPUs) produces the same tokens as TP=1; skipped on a single-GPU box."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import os, subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29541", os.path.join(root, "tests", "tp_engine_check.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "TP_ENGINE_OK" in res.stdout
