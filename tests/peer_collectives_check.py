"""Run under torchrun with >= 2 ranks: the peer-memory all-reduce / all-gather against torch.distributed,
eagerly and replayed from a CUDA graph, and the bounded wait when a rank stays away."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flash_attn_v100_b200 import _lib  # noqa: E402
from flash_attn_v100_b200.comm import PeerCollectives  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    pc = PeerCollectives(dist.group.WORLD, dev, 8 << 20)
    ok = True
    g = torch.Generator(device=dev).manual_seed(100 + rank)

    def expected_sum(x):
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x)
        acc = torch.zeros(x.shape, dtype=torch.float32, device=dev)
        for p in parts:                       # rank order, fp32, one rounding: what the kernel computes
            acc += p.float()
        return acc.bfloat16()

    # ---- all-reduce: several sizes, exact against the fp32 rank-order sum, identical on all ranks ----
    for rows, cols in [(1, 8 * world), (256, 4096), (3, 64 * world), (512, 4096)]:
        x = torch.randn(rows, cols, generator=g, device=dev).bfloat16()
        want = expected_sum(x)
        v = pc.view(0, (rows, cols), torch.bfloat16)
        v.copy_(x)
        pc.all_reduce_(v)
        torch.cuda.synchronize()
        same = torch.equal(v, want)
        allr = [torch.empty_like(v) for _ in range(world)]
        dist.all_gather(allr, v.clone())
        ident = all(torch.equal(allr[0], a) for a in allr)
        ok &= same and ident
        if rank == 0:
            print(f"all-reduce {rows}x{cols}: exact {same}, identical across ranks {ident}", flush=True)

    # ---- all-reduce + residual add + RMS norm in one kernel: bit-identical to the separate kernels ----
    lib = _lib.load()
    for rows, cols in [(world, 8), (8 * world, 4096), (4 * world, 1032), (32 * world, 2048 + 64)]:
        n = rows * cols * 2
        reg = (n + 255) // 256 * 256
        part = pc.view(0, (rows, cols), torch.bfloat16)
        xr = pc.view(reg, (rows, cols), torch.bfloat16)
        hr = pc.view(2 * reg, (rows, cols), torch.bfloat16)
        gs = torch.Generator(device=dev).manual_seed(7)          # the residual stream is the same on every rank
        x0 = torch.randn(rows, cols, generator=gs, device=dev).bfloat16()
        wn = (1.0 + 0.1 * torch.randn(cols, generator=gs, device=dev)).bfloat16()
        p0 = torch.randn(rows, cols, generator=g, device=dev).bfloat16()
        # separate kernels
        part.copy_(p0)
        pc.all_reduce_(part)
        x_ref = x0.clone()
        h_ref = torch.empty_like(x_ref)
        _lib.check(lib.fa_add_rmsnorm_bf16(x_ref.data_ptr(), part.data_ptr(), wn.data_ptr(), h_ref.data_ptr(), rows, cols,
                                           1e-6, torch.cuda.current_stream(dev).cuda_stream))
        torch.cuda.synchronize()
        dist.barrier()
        # one kernel
        part.copy_(p0)
        xr.copy_(x0)
        hr.zero_()
        pc.all_reduce_add_rmsnorm_(part, xr, hr, wn, 1e-6)
        torch.cuda.synchronize()
        okf = torch.equal(xr, x_ref) and torch.equal(hr, h_ref) and torch.equal(part, p0)
        ok &= okf
        if rank == 0:
            print(f"all-reduce + add + rmsnorm {rows}x{cols}: bit-identical to the separate kernels {okf}", flush=True)
        dist.barrier()

    # ---- all-gather ----
    src = torch.randn(64, 2, generator=g, device=dev)
    out = pc.view(4 << 20, (world, 64, 2), torch.float32)
    pc.all_gather_into(out, src)
    torch.cuda.synchronize()
    want = torch.empty(world, 64, 2, device=dev)
    dist.all_gather_into_tensor(want, src)
    okg = torch.equal(out, want)
    ok &= okg
    if rank == 0:
        print(f"all-gather: {okg}", flush=True)

    # ---- a step with two all-reduces and an all-gather, captured once and replayed ----
    w = torch.randn(512, 256, generator=g, device=dev).bfloat16() * 0.05
    a_in = torch.empty(32, 256, device=dev, dtype=torch.bfloat16)
    buf = pc.view(0, (32, 512), torch.bfloat16)
    gat = pc.view(1 << 20, (world, 32), torch.float32)
    res = torch.empty(32, 512, device=dev, dtype=torch.bfloat16)

    def step():
        torch.mm(a_in, w.t(), out=buf)
        pc.all_reduce_(buf)
        h = torch.tanh(buf.float()).bfloat16()
        buf.copy_(h * 0.5)
        pc.all_reduce_(buf)
        res.copy_(buf)
        pc.all_gather_into(gat, buf.float().sum(dim=1).contiguous())

    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        a_in.copy_(torch.randn(32, 256, generator=g, device=dev).bfloat16())
        step()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
            step()
        okr = True
        for it in range(20):
            a_in.copy_(torch.randn(32, 256, generator=g, device=dev).bfloat16())
            graph.replay()
            side.synchronize()
            got, got_g = res.clone(), gat.clone()
            # the same step with torch.distributed collectives
            t = expected_sum(a_in @ w.t())
            t = expected_sum((torch.tanh(t.float()).bfloat16() * 0.5))
            rows = torch.empty(world, 32, device=dev)
            dist.all_gather_into_tensor(rows, t.float().sum(dim=1).contiguous())
            okr &= torch.equal(got, t) and torch.equal(got_g, rows)
    torch.cuda.current_stream(dev).wait_stream(side)
    ok &= okr
    if rank == 0:
        print(f"graph replay x20 equal to torch.distributed: {okr}", flush=True)
    pc.check()

    # ---- bounded wait: rank 0 calls an all-reduce that the others never join ----
    dist.barrier()
    _lib.check(_lib.load().fa_peer_set_max_polls(1 << 20))
    timed_out = True
    if rank == 0:
        pc.all_reduce_(pc.view(0, (1, 8 * world), torch.bfloat16))
        try:
            pc.check()
            timed_out = False
        except RuntimeError as e:
            print(f"bounded wait reported: {e}", flush=True)
    ok &= timed_out
    torch.cuda.synchronize()
    # ---- the way back: every rank resets its flags / epoch / status, then collectives work again ----
    pc.reset()
    _lib.check(_lib.load().fa_peer_set_max_polls(1 << 26))
    x = torch.randn(64, 8 * world, generator=g, device=dev).bfloat16()
    want = expected_sum(x)
    v = pc.view(0, (64, 8 * world), torch.bfloat16)
    v.copy_(x)
    pc.all_reduce_(v)
    torch.cuda.synchronize()
    recovered = torch.equal(v, want)
    try:
        pc.check()
    except RuntimeError:
        recovered = False
    ok &= recovered
    if rank == 0:
        print(f"all-reduce after reset: {recovered}", flush=True)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    pc.close()
    if rank == 0 and int(flag) == 1:
        print("PEER_COLLECTIVES_OK", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
