"""GPU parity of the INT8-QK decode: int32 QK^T accumulators bit-exact against the
CPU restatement, outputs within 2e-3."""
import pytest
import torch

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu


def _scales(q, k):
    qs = q.abs().amax(-1).float().squeeze(-1) / 127          # [B,H_Q]
    ks = k.abs().amax(-1).float() / 127                      # [B,H_KV,N]
    return qs.contiguous(), ks.contiguous()


@pytest.mark.parametrize("B,H_Q,H_KV,N,D,cache_len", [
    (2, 8, 2, 70, 64, 69), (1, 32, 8, 257, 128, 256), (2, 16, 16, 33, 128, 20), (1, 8, 1, 129, 256, 128),
    (3, 32, 8, 1000, 128, 999), (1, 40, 2, 50, 64, 49),
])
def test_int8_scores_bit_exact_and_output_close(B, H_Q, H_KV, N, D, cache_len):
    import flash_attn_v100 as fa
    import flash_attn_v100_b200
    g = torch.Generator().manual_seed(N * 7 + D)
    q = torch.randn(B, H_Q, 1, D, generator=g).half()
    k = torch.randn(B, H_KV, N, D, generator=g).half()
    v = torch.randn(B, H_KV, N, D, generator=g).half()
    qs, ks = _scales(q, k)
    out, scores = fa.forward_decode_int8_gqa(q.cuda(), k.cuda(), v.cuda(), qs.cuda(), ks.cuda(), cache_len,
                                             return_scores=True)
    ref_out, ref_dots = orc.decode_int8_gqa(q, k, v, qs, ks, cache_len, final_cast=False)
    n_vis = cache_len + 1
    assert torch.equal(scores.cpu()[:, :, :n_vis], ref_dots[:, :, :n_vis])     # bit-exact int32
    assert (scores.cpu()[:, :, n_vis:] == 0).all()
    assert (out.float().cpu() - ref_out).abs().max().item() < 2e-3
    out2 = fa.forward_decode_int8_gqa(q.cuda(), k.cuda(), v.cuda(), qs.cuda(), ks.cuda(), cache_len)
    assert torch.equal(out2, out)
    torch.cuda.synchronize()
    flash_attn_v100_b200.check_async_errors()


def test_int8_rounding_ties_and_clamp():
    """Values engineered to land on .5 ties and beyond +-127 after division."""
    import flash_attn_v100 as fa
    B, H_Q, H_KV, N, D = 1, 4, 1, 32, 64
    q = torch.zeros(B, H_Q, 1, D).half()
    k = torch.zeros(B, H_KV, N, D).half()
    base = torch.tensor([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5, -126.5, 127.5, 200.0, -200.0, 0.25, 63.5, -63.5])
    k[0, 0, :, : base.numel()] = base.half()
    k[0, 0, :, 20] = torch.arange(N).half()
    q[0, :, 0, : base.numel()] = torch.tensor([1.0, -1.0, 2.0, 3.0, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0, 1.0, 5.0, 2.0, 2.0]).half()
    q[0, :, 0, 20] = 1.0
    v = torch.randn(B, H_KV, N, D).half()
    qs = torch.ones(B, H_Q)
    ks = torch.ones(B, H_KV, N)
    _, scores = fa.forward_decode_int8_gqa(q.cuda(), k.cuda(), v.cuda(), qs.cuda(), ks.cuda(), N - 1, return_scores=True)
    ref = orc.int8_scores(q, k, qs, ks)
    assert torch.equal(scores.cpu(), ref)


def test_int8_benchmark_shape_scores_bit_exact_on_sampled_rows():
    """The INT8 benchmark configuration at full size (B=32, 32/8 heads, D=128, N=4096, cache_len 4095):
    the int32 accumulators of sampled (batch, head) rows against the CPU restatement, bit for bit, and the
    outputs of those rows within 2e-3."""
    import flash_attn_v100 as fa
    import flash_attn_v100_b200
    B, H_Q, H_KV, D, N = 32, 32, 8, 128, 4096
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(4)
    q = torch.randn(B, H_Q, 1, D, generator=g, device=dev, dtype=torch.float16)
    k = torch.randn(B, H_KV, N, D, generator=g, device=dev, dtype=torch.float16)
    v = torch.randn(B, H_KV, N, D, generator=g, device=dev, dtype=torch.float16)
    qs = (q.abs().amax(-1).float().squeeze(-1) / 127).contiguous()
    ks = (k.abs().amax(-1).float() / 127).contiguous()
    out, scores = fa.forward_decode_int8_gqa(q, k, v, qs, ks, N - 1, return_scores=True)
    torch.cuda.synchronize()
    flash_attn_v100_b200.check_async_errors()
    for b in (0, 13, 31):
        sl = slice(b, b + 1)
        ref_out, ref_dots = orc.decode_int8_gqa(q[sl].cpu(), k[sl].cpu(), v[sl].cpu(), qs[sl].cpu(), ks[sl].cpu(), N - 1,
                                                final_cast=False)
        assert torch.equal(scores[sl].cpu(), ref_dots), b
        assert (out[sl].float().cpu() - ref_out).abs().max().item() < 2e-3, b
