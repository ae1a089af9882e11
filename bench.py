#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--workload paged_decode|varlen_prefill|int8_decode|contig_decode|int8_kv_decode|sliding_window_decode]

Default workload (the headline): paged GQA decode, B=64, 32 query / 8 KV heads,
D=128, fp16, 16-token pages, seq_lens uniform in [512, 8192], block table a
seeded random permutation of the pool.  One "step" is one decode call over the
whole batch (one new token per sequence).  Under torchrun every rank owns an
independent batch of the same shape (weak scaling, no collective on the data
path); the timed region is bracketed by a barrier and a device synchronise and
the reported time is the maximum over ranks.

One JSON line is printed on stdout by rank 0.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# DRAM bytes per launch of the split-KV decode kernel on the headline workload, from
# the ncu capture summarised in profiles/ (dram__bytes_read.sum + dram__bytes_write.sum).
# The paged-decode figure is the B=16 capture (304.8 MB for 73,364 tokens) scaled by tokens to
# the benchmark launch (275,479 tokens); the INT8 figure is the B=16 capture (274.8 MB) scaled to
# B=32; traffic grows in proportion to tokens.  None = no DRAM-traffic figure (tensor-bound kernel
# or no capture).
NCU_TRAFFIC_BYTES = {"paged_decode": 1_146_000_000, "int8_decode": 549_700_000, "contig_decode": None,
                     "varlen_prefill": None,
                     # B=16 capture (272.8 + 4.6 MB) scaled by 2 to the B=32 launch (traffic grows with the tokens)
                     "int8_kv_decode": 554_800_000, "sliding_window_decode": None}

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {k: float(d[k]) for k in FALLBACK_PEAKS if k in d}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


# ----------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.tmp = None

    def start(self):
        try:
            self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=self.tmp, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.tmp.flush()
        self.tmp.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.tmp.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.unlink(self.tmp.name)
        except OSError:
            pass
        if sm:
            sm.sort()
            out.update(sm_mhz=sm[len(sm) // 2], sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


# ----------------------------------------------------------------------------
# workloads
# ----------------------------------------------------------------------------
def decode_algorithmic_bytes(tokens_attended: int, pages: int, B: int, H_Q: int, H_KV: int, D: int) -> int:
    """K and V read once per KV head, Q read and O written once, block table and lengths."""
    return tokens_attended * (2 * H_KV * D * 2) + 2 * (B * H_Q * D * 2) + 4 * pages + 4 * B


class PagedDecode:
    name = "paged_decode"
    metric = "paged_gqa_decode_tokens_per_s"
    unit = "tokens/s"
    bound = "hbm"
    dtype = "fp16"
    B, H_Q, H_KV, D = 64, 32, 8, 128

    def __init__(self, device, seed):
        from flash_attn_v100_b200.synthetic import make_paged_decode_batch
        self.device = device
        # lengths and page placement are the same on every rank (table seed 0), so that the work per GPU
        # is fixed exactly under weak scaling; the tensor values are seeded by the rank.  Everything is
        # drawn on the host from seeded CPU generators: the reference arm (`--impl reference`) rebuilds
        # exactly the batch of rank 0 and runs the CPU implementation on it.
        t = make_paged_decode_batch(self.B, self.H_Q, self.H_KV, self.D, 512, 8192, table_seed=0, value_seed=seed)
        self.seq_lens_h, self.block_table_h, self.n_pages = t["seq_lens"], t["block_table"], t["n_pages"]
        self.max_blocks = t["max_num_blocks"]
        self.k_cache = t["k_cache"].to(device)
        self.v_cache = t["v_cache"].to(device)
        q_host = t["q"]
        del t
        # the per-step inputs live in ONE pinned host allocation (q | block_table | seq_lens), so that the
        # end-to-end step moves them with a single host-to-device copy
        q_bytes, bt_bytes = self.B * self.H_Q * self.D * 2, self.block_table_h.numel() * 4
        self._in_off = (0, q_bytes, q_bytes + bt_bytes, q_bytes + bt_bytes + self.B * 4)
        self.in_h = torch.empty(self._in_off[3], dtype=torch.uint8).pin_memory()
        self.q_h = self.in_h[:q_bytes].view(torch.float16).view(self.B, self.H_Q, 1, self.D)
        self.bt_h = self.in_h[q_bytes:q_bytes + bt_bytes].view(torch.int32).view(self.block_table_h.shape)
        self.sl_h = self.in_h[q_bytes + bt_bytes:].view(torch.int32)
        self.q_h.copy_(q_host)
        self.bt_h.copy_(self.block_table_h)
        self.sl_h.copy_(self.seq_lens_h)
        self.in_d = torch.empty(self._in_off[3], dtype=torch.uint8, device=device)
        self.q = self.q_h.to(device)
        self.bt = self.bt_h.to(device)
        self.sl = self.sl_h.to(device)
        self.out_h = torch.empty(self.B, self.H_Q, 1, self.D, dtype=torch.float16).pin_memory()
        self.units_per_step = self.B  # one new token per sequence
        tokens = int(self.seq_lens_h.sum())
        pages = int(((self.seq_lens_h + 15) // 16).sum())
        self.alg_bytes = decode_algorithmic_bytes(tokens, pages, self.B, self.H_Q, self.H_KV, self.D)
        self.alg_flops = 4 * self.H_Q * self.D * tokens
        self.launches_per_step = 1  # one fused split-KV kernel (scan + work + merge)

    @classmethod
    def config_of(cls, seq_lens, n_pages):
        """The `config` of the headline line; both arms (GPU and CPU reference) print exactly this."""
        return {"workload": "paged_gqa_decode B=64 H_Q=32 H_KV=8 D=128 page=16 seq_lens~U[512,8192] (BASELINE configs[1])",
                "batch_per_gpu": cls.B, "tokens_attended_per_gpu": int(seq_lens.sum()),
                "kv_bytes_per_gpu": int(n_pages) * cls.H_KV * 16 * cls.D * 2 * 2,
                "l2": "inputs larger than L2 (KV pool >> 126 MB), no flush",
                "partition": "independent batch per rank (same lengths on every rank, values seeded by rank)"}

    def config(self):
        return self.config_of(self.seq_lens_h, self.n_pages)

    def step(self, fa):
        return fa.forward_paged_decode_gqa_fp16(self.q, self.k_cache, self.v_cache, self.bt, self.sl, self.max_blocks)

    def step_e2e(self, fa):
        # per-step inputs of a decode iteration: the new queries, the block table and the lengths;
        # the KV pool is resident state (it lives on the device in the reference as well)
        o = self._in_off
        self.in_d.copy_(self.in_h, non_blocking=True)
        q = self.in_d[:o[1]].view(torch.float16).view(self.B, self.H_Q, 1, self.D)
        bt = self.in_d[o[1]:o[2]].view(torch.int32).view(self.block_table_h.shape)
        sl = self.in_d[o[2]:].view(torch.int32)
        out = fa.forward_paged_decode_gqa_fp16(q, self.k_cache, self.v_cache, bt, sl, self.max_blocks)
        self.out_h.copy_(out, non_blocking=True)
        return out

    def e2e_bytes(self):
        return (self.q_h.numel() * 2 + self.bt_h.numel() * 4 + self.sl_h.numel() * 4, self.out_h.numel() * 2)

    def host_copy(self):
        return dict(q=self.q_h.clone(), k_cache=self.k_cache.cpu(), v_cache=self.v_cache.cpu(),
                    block_table=self.block_table_h, seq_lens=self.seq_lens_h)

    @staticmethod
    def cpu_reference(host, seqs):
        from oracle import attention_oracle as orc
        idx = torch.tensor(seqs)
        return orc.paged_decode(host["q"][idx], host["k_cache"], host["v_cache"], host["block_table"][idx],
                                host["seq_lens"][idx])


class ContigDecode(PagedDecode):
    """Continuous-batching decode over a padded contiguous cache (same sizes as the paged workload)."""
    name = "contig_decode"
    metric = "continuous_batching_decode_tokens_per_s"

    def __init__(self, device, seed):
        g = torch.Generator().manual_seed(0)   # same lengths on every rank
        self.device = device
        self.B = 32
        self.max_N = 8192
        self.cache_lens_h = torch.randint(511, 8192, (self.B,), generator=g, dtype=torch.int32)
        gd = torch.Generator(device=device).manual_seed(seed)
        self.k = torch.randn(self.B, self.H_KV, self.max_N, self.D, generator=gd, device=device, dtype=torch.float16)
        self.v = torch.randn(self.B, self.H_KV, self.max_N, self.D, generator=gd, device=device, dtype=torch.float16)
        self.q = torch.randn(self.B, self.H_Q, 1, self.D, generator=gd, device=device, dtype=torch.float16)
        self.cl = self.cache_lens_h.to(device)
        self.units_per_step = self.B
        tokens = int((self.cache_lens_h + 1).sum())
        self.alg_bytes = decode_algorithmic_bytes(tokens, 0, self.B, self.H_Q, self.H_KV, self.D)
        self.alg_flops = 4 * self.H_Q * self.D * tokens
        self.launches_per_step = 1

    def config(self):
        return {"workload": "continuous_batching_decode B=32 H_Q=32 H_KV=8 D=128 max_N=8192 cache_lens~U[511,8191]",
                "l2": "inputs larger than L2, no flush"}

    def step(self, fa):
        return fa.forward_continuous_batching_fp16(self.q, self.k, self.v, self.cl, True)

    step_e2e = None


class Int8Decode:
    name = "int8_decode"
    metric = "int8_gqa_decode_tokens_per_s"
    unit = "tokens/s"
    bound = "hbm"
    dtype = "int8 QK^T (int32 accumulate), fp16 PV"
    B, H_Q, H_KV, D, N = 32, 32, 8, 128, 4096

    def __init__(self, device, seed):
        self.device = device
        gd = torch.Generator(device=device).manual_seed(seed)
        self.q = torch.randn(self.B, self.H_Q, 1, self.D, generator=gd, device=device, dtype=torch.float16)
        self.k = torch.randn(self.B, self.H_KV, self.N, self.D, generator=gd, device=device, dtype=torch.float16)
        self.v = torch.randn(self.B, self.H_KV, self.N, self.D, generator=gd, device=device, dtype=torch.float16)
        self.qs = (self.q.abs().amax(-1).float().squeeze(-1) / 127).contiguous()
        self.ks = (self.k.abs().amax(-1).float() / 127).contiguous()
        self.units_per_step = self.B
        self.alg_bytes = (self.B * self.H_KV * self.N * self.D * 2 * 2 + self.ks.numel() * 4 +
                          2 * self.B * self.H_Q * self.D * 2 + self.qs.numel() * 4)
        self.alg_flops = 4 * self.H_Q * self.D * self.N * self.B
        self.launches_per_step = 1

    def config(self):
        return {"workload": "int8_gqa_decode B=32 H_Q=32 H_KV=8 D=128 N=4096 cache_len=4095 (BASELINE configs[3])",
                "l2": "inputs larger than L2 (K/V 537 MB), no flush"}

    def step(self, fa):
        return fa.forward_decode_int8_gqa(self.q, self.k, self.v, self.qs, self.ks, self.N - 1)

    step_e2e = None


class Int8KVDecode:
    """Decode over an INT8 KV cache with per-token fp16 scales (same shape as the int8 score workload)."""
    name = "int8_kv_decode"
    metric = "int8_kv_cache_gqa_decode_tokens_per_s"
    unit = "tokens/s"
    bound = "hbm"
    dtype = "int8 cache dequantised to fp16 in registers, fp32 accumulate"
    B, H_Q, H_KV, D, N = 32, 32, 8, 128, 8192

    def __init__(self, device, seed):
        self.device = device
        gd = torch.Generator(device=device).manual_seed(seed)
        self.q = torch.randn(self.B, self.H_Q, 1, self.D, generator=gd, device=device, dtype=torch.float16)
        shape = (self.B, self.H_KV, self.N, self.D)
        self.k8 = torch.randint(-127, 128, shape, generator=gd, device=device, dtype=torch.int8)
        self.v8 = torch.randint(-127, 128, shape, generator=gd, device=device, dtype=torch.int8)
        # absmax/127 scales of N(0,1) rows of 128 values: about 3/127
        self.ks = (torch.rand(shape[:3], generator=gd, device=device) * 0.01 + 0.02).half()
        self.vs = (torch.rand(shape[:3], generator=gd, device=device) * 0.01 + 0.02).half()
        self.units_per_step = self.B
        self.alg_bytes = (2 * self.B * self.H_KV * self.N * self.D + 2 * self.ks.numel() * 2 +
                          2 * self.B * self.H_Q * self.D * 2)
        self.alg_flops = 4 * self.H_Q * self.D * self.N * self.B
        self.launches_per_step = 1

    def config(self):
        return {"workload": "int8_kv_cache_gqa_decode B=32 H_Q=32 H_KV=8 D=128 N=8192 cache_len=8191",
                "l2": "inputs larger than L2 (K/V 537 MB), no flush"}

    def step(self, fa):
        return fa.forward_decode_int8_kv_cache_gqa(self.q, self.k8, self.v8, self.ks, self.vs, self.N - 1)

    step_e2e = None


class SlidingWindowDecode:
    """Sliding-window + sink decode: the window and the sink are read, the rest of the cache is not."""
    name = "sliding_window_decode"
    metric = "sliding_window_gqa_decode_tokens_per_s"
    unit = "tokens/s"
    bound = "hbm"
    dtype = "fp16"
    B, H_Q, H_KV, D, N, WINDOW, SINK = 128, 32, 8, 128, 8192, 4096, 4

    def __init__(self, device, seed):
        self.device = device
        gd = torch.Generator(device=device).manual_seed(seed)
        self.q = torch.randn(self.B, self.H_Q, 1, self.D, generator=gd, device=device, dtype=torch.float16)
        self.k = torch.randn(self.B, self.H_KV, self.N, self.D, generator=gd, device=device, dtype=torch.float16)
        self.v = torch.randn(self.B, self.H_KV, self.N, self.D, generator=gd, device=device, dtype=torch.float16)
        self.units_per_step = self.B
        pages = (self.SINK + 15) // 16 + self.WINDOW // 16      # window ends at N, page aligned
        self.alg_bytes = self.B * self.H_KV * pages * 16 * self.D * 2 * 2 + 2 * self.B * self.H_Q * self.D * 2
        self.alg_flops = 4 * self.H_Q * self.D * (self.WINDOW + self.SINK) * self.B
        self.launches_per_step = 1

    def config(self):
        return {"workload": "sliding_window_gqa_decode B=128 H_Q=32 H_KV=8 D=128 N=8192 cache_len=8191 window=4096 sink=4",
                "l2": "pages read per step (2.15 GB) larger than L2, no flush",
                "bytes": "whole 16-token pages that hold an attended key"}

    def step(self, fa):
        return fa.forward_decode_sliding_window_gqa(self.q, self.k, self.v, True, self.N - 1, self.WINDOW, self.SINK)

    step_e2e = None


class VarlenPrefill:
    name = "varlen_prefill"
    metric = "varlen_causal_gqa_prefill_tflops"
    unit = "TFLOP/s"
    bound = "tensor"
    dtype = "fp16"
    H_Q, H_KV, D = 32, 8, 128

    def __init__(self, device, seed):
        self.device = device
        g = torch.Generator().manual_seed(0)   # same lengths on every rank
        self.lens = torch.randint(128, 4097, (16,), generator=g).tolist()
        cu = [0]
        for n in self.lens:
            cu.append(cu[-1] + n)
        self.total = cu[-1]
        self.cu = torch.tensor(cu, dtype=torch.int32, device=device)
        gd = torch.Generator(device=device).manual_seed(seed)
        self.q = torch.randn(self.total, self.H_Q, self.D, generator=gd, device=device, dtype=torch.float16)
        self.k = torch.randn(self.total, self.H_KV, self.D, generator=gd, device=device, dtype=torch.float16)
        self.v = torch.randn(self.total, self.H_KV, self.D, generator=gd, device=device, dtype=torch.float16)
        self.alg_flops = sum(4 * self.H_Q * self.D * n * (n + 1) // 2 for n in self.lens)
        self.alg_bytes = (self.q.numel() * 2 + self.k.numel() * 2) * 2
        self.units_per_step = self.alg_flops / 1e12   # TFLOP per step
        self.launches_per_step = 1
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def config(self):
        return {"workload": "varlen_causal_gqa_prefill 16 seqs L~U[128,4096] H_Q=32 H_KV=8 D=128 (BASELINE configs[2])",
                "total_tokens": self.total, "flops": "causal-exact 4*H_Q*D*L(L+1)/2 per sequence",
                "l2": "256 MB buffer written between timed iterations"}

    def step(self, fa):
        return fa.forward_varlen_prefill_fp16(self.q, self.k, self.v, self.cu, max(self.lens), True)

    step_e2e = None


class VarlenPrefillBF16(VarlenPrefill):
    """configs[2] through the bfloat16 twin of the operator."""
    name = "varlen_prefill_bf16"
    dtype = "bf16"

    def __init__(self, device, seed):
        super().__init__(device, seed)
        self.q, self.k, self.v = self.q.bfloat16(), self.k.bfloat16(), self.v.bfloat16()

    def config(self):
        c = super().config()
        c["workload"] = c["workload"].replace("varlen_causal_gqa_prefill", "varlen_causal_gqa_prefill (bfloat16 twin)")
        return c

    def step(self, fa):
        return fa.forward_varlen_prefill_bf16(self.q, self.k, self.v, self.cu, max(self.lens), True)


class HeadShardedPagedDecode:
    """ONE paged-decode batch of the headline shape split over the ranks by KV-head group (the reference's
    multi-GPU partition, tensor_parallel.py:435-457 and :553-571): rank r holds KV heads
    [r*8/N, (r+1)*8/N) of every page and the 32/N query heads that map to them; block_table and seq_lens are
    replicated; no collective.  Strong scaling: the bytes per rank shrink with N (141 MB at N=8, about the size
    of L2), so the step rotates over N distinct K/V pools of the same shape."""
    name = "paged_decode_head_sharded"
    metric = "paged_gqa_decode_tokens_per_s"
    unit = "tokens/s"
    bound = "hbm"
    dtype = "fp16"
    B, H_Q, H_KV, D = 64, 32, 8, 128

    def __init__(self, device, rank, world):
        from flash_attn_v100_b200.sharding import head_shard
        from flash_attn_v100_b200.synthetic import make_paged_tables
        self.shard = head_shard(self.H_Q, self.H_KV, rank, world)
        self.hq = self.shard.q_heads[1] - self.shard.q_heads[0]
        self.hkv = self.shard.kv_heads[1] - self.shard.kv_heads[0]
        t = make_paged_tables(self.B, 512, 8192, 0)      # the global batch: same tables on every rank
        self.max_blocks, self.n_pages = t["max_num_blocks"], t["n_pages"]
        self.bt, self.sl = t["block_table"].to(device), t["seq_lens"].to(device)
        g = torch.Generator(device=device).manual_seed(977 + rank)
        self.pools = []
        for _ in range(max(world, 1)):
            k = torch.empty(self.n_pages, self.hkv, 16, self.D, dtype=torch.float16, device=device)
            v = torch.empty_like(k)
            for s0 in range(0, self.n_pages, 4096):
                e = min(s0 + 4096, self.n_pages)
                k[s0:e] = torch.randn(e - s0, self.hkv, 16, self.D, generator=g, device=device).half()
                v[s0:e] = torch.randn(e - s0, self.hkv, 16, self.D, generator=g, device=device).half()
            self.pools.append((k, v))
        self.q = torch.randn(self.B, self.hq, 1, self.D, generator=g, device=device, dtype=torch.float16)
        self.turn = 0
        tokens = int(t["seq_lens"].sum())
        pages = int(((t["seq_lens"] + 15) // 16).sum())
        self.alg_bytes = decode_algorithmic_bytes(tokens, pages, self.B, self.hq, self.hkv, self.D)   # per rank
        self.alg_flops = 4 * self.hq * self.D * tokens
        self.units_per_step = self.B
        self.launches_per_step = 1

    def config(self):
        return {"workload": "paged_gqa_decode B=64 H_Q=32 H_KV=8 D=128 (BASELINE configs[1]), ONE batch split by "
                            "KV-head group", "kv_heads_per_rank": self.hkv, "q_heads_per_rank": self.hq,
                "kv_bytes_per_rank": int(self.pools[0][0].numel() * 4), "pools_rotated": len(self.pools),
                "l2": "the step rotates over as many distinct K/V pools as there are ranks (1.13 GB in all), so no "
                      "launch finds its pages in L2"}

    def step(self, fa):
        k, v = self.pools[self.turn % len(self.pools)]
        self.turn += 1
        return fa.forward_paged_decode_gqa_fp16(self.q, k, v, self.bt, self.sl, self.max_blocks)

    def graph_of_one_rotation(self, fa, device):
        """One launch per pool, captured into a CUDA graph (how a serving loop replays its decode step): at 8 ranks
        a launch is short enough for the eager call's host time to show in `step`."""
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            for _ in range(len(self.pools)):
                self.step(fa)
            self.turn = 0
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                for _ in range(len(self.pools)):
                    self.step(fa)
        torch.cuda.current_stream(device).wait_stream(side)
        return graph, len(self.pools)


class PagedDecodeBF16(PagedDecode):
    """The headline workload through the bfloat16 twin of the operator (the same bytes, bfloat16 q / pages / out)."""
    name = "paged_decode_bf16"
    dtype = "bf16"

    def __init__(self, device, seed):
        super().__init__(device, seed)
        self.k_cache = self.k_cache.bfloat16()
        self.v_cache = self.v_cache.bfloat16()
        self.q = self.q.bfloat16()
        self.step_e2e = None

    def step(self, fa):
        return fa.forward_paged_decode_gqa_bf16(self.q, self.k_cache, self.v_cache, self.bt, self.sl, self.max_blocks)

    def config(self):
        c = super().config()
        c["workload"] = c["workload"].replace("paged_gqa_decode", "paged_gqa_decode (bfloat16 twin)")
        return c


WORKLOADS = {w.name: w for w in (PagedDecode, PagedDecodeBF16, ContigDecode, Int8Decode, Int8KVDecode,
                                 SlidingWindowDecode, VarlenPrefill, VarlenPrefillBF16)}


def run_engine(args):
    """BASELINE.json configs[4]: Qwen3-8B-shaped decoder, random-init bf16 weights, 256 requests x 1024-token
    prompts, greedy generation of 256 tokens, paged KV, tensor parallel over all ranks (by KV-head group).
    One step = the whole generation (prefill + 255 decode steps)."""
    rank, world, local = dist_setup(args.gpus)
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    from flash_attn_v100_b200.engine import GenerationRunner, TPDecoder, make_rank_weights, qwen3_8b_shaped, tiny_config
    import flash_attn_v100_b200
    peaks, peak_src = load_peaks()
    cfg = tiny_config() if args.engine_tiny else qwen3_8b_shaped()
    B, P, N = (8, 64, 16) if args.engine_tiny else (args.engine_requests, 1024, 256)
    w = make_rank_weights(cfg, rank, world, 0, device)
    model = TPDecoder(cfg, w, rank, world, None, device)
    runner = GenerationRunner(model, max_batch=B, max_seq_len=P + N, use_cuda_graph=True,
                              peer_collectives=not args.engine_nccl_decode)
    prompts = torch.randint(0, cfg.vocab_size, (B, P), generator=torch.Generator().manual_seed(0))
    times = []
    for it in range(max(args.warmup, 1) + args.steps):
        torch.cuda.synchronize(); barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        toks = runner.generate(prompts, N, prefill_chunk=args.engine_prefill_chunk)
        e1.record()
        torch.cuda.synchronize()
        ms = max_over_ranks(e0.elapsed_time(e1), world, device)
        if it >= max(args.warmup, 1):
            times.append(ms)
            phases = runner.last_timing_ms()
    flash_attn_v100_b200.check_async_errors(); flash_attn_v100_b200.check_prefill_errors()
    if model.comm is not None:
        model.comm.check()
    if rank != 0:
        return
    ms = sum(times) / len(times)
    wbytes = sum(t.numel() * t.element_size() for lw in w["layers"] for t in lw.values()) + w["lm_head"].numel() * 2
    kv_bytes_mid = B * (P + N // 2) * cfg.num_layers * model.kl * 2 * cfg.head_dim * 2
    line = {
        "metric": "qwen3_8b_shaped_generation_tokens_per_s", "value": B * N / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16 weights and activations, fp16 attention operators", "data": "synthetic (seeded random weights, uniform random token ids)",
        "config": {"workload": "Qwen3-8B-shaped decoder end to end (BASELINE configs[4])" if not args.engine_tiny else "tiny decoder (smoke)",
                   "layers": cfg.num_layers, "hidden": cfg.hidden_size, "heads": f"{cfg.num_heads}/{cfg.num_kv_heads}",
                   "requests": B, "prompt_len": P, "new_tokens": N, "parallelism": f"tp{world}", "page": 16,
                   "decode": "one CUDA graph per step" if world == 1 else "chain of CUDA graphs per step, NCCL collectives eager in between", "prefill_chunk": args.engine_prefill_chunk},
        "prefill_ms": phases[0], "decode_ms": phases[1], "decode_ms_per_token_step": phases[1] / max(N - 1, 1),
        "prefill_tokens_per_s": B * P / (phases[0] * 1e-3), "decode_tokens_per_s": B * (N - 1) / (phases[1] * 1e-3),
        "per_rank_weight_bytes": wbytes, "per_rank_kv_bytes_mid_generation": kv_bytes_mid,
        "roofline": None, "cpu_baseline": None, "e2e": None, "gpu_launches": None, "impl": "b200",
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------
# timing
# ----------------------------------------------------------------------------
def dist_setup(n_gpus):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")   # plain NVLink paths only (see collectives_record)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        torch.cuda.set_device(local)
        # NCCL announces its version on stdout at the first communicator set-up; stdout carries the
        # one JSON line only, so point fd 1 at stderr until the communicator exists.
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)
    return rank, world, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()


def max_over_ranks(x, world, device):
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_steps(fn, steps, world, device, flush=None):
    """Device time of `steps` calls: CUDA events on the launching (current) stream,
    barrier + synchronise on both sides.  With `flush`, each step is timed separately
    and an L2-sized write runs between steps outside the events."""
    torch.cuda.synchronize()
    barrier(world)
    torch.cuda.synchronize()
    if flush is None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
    else:
        evs = []
        for _ in range(steps):
            flush.fill_(1)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            evs.append((a, b))
        torch.cuda.synchronize()
        ms = sum(a.elapsed_time(b) for a, b in evs)
    barrier(world)
    return max_over_ranks(ms, world, device)


def measure(fn, steps, world, device, flush=None, min_seconds=0.5, max_blocks=400):
    """Repeat the block of exactly `steps` timed steps until the blocks add up to `min_seconds` of device
    time (every block is bracketed and reduced over the ranks as in time_steps).  The reported step time
    is the median block; the fastest block and the number of blocks are kept beside it."""
    blocks = []
    while True:
        blocks.append(time_steps(fn, steps, world, device, flush))   # the same number on every rank
        if sum(blocks) >= min_seconds * 1e3 or len(blocks) >= max_blocks:
            break
    ordered = sorted(blocks)
    return {"ms_block": ordered[len(ordered) // 2], "ms_block_min": ordered[0], "blocks": len(blocks),
            "timed_seconds": sum(blocks) * 1e-3}


def roofline_of(wl, ms_per_step, peaks, peak_src):
    if wl.bound == "hbm":
        achieved, peak, unit = wl.alg_bytes / (ms_per_step * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s"
    else:
        achieved, peak, unit = wl.alg_flops / (ms_per_step * 1e-3) / 1e12, peaks["bf16_tflops"], "TFLOP/s"
    extra = {}
    if wl.bound != "hbm" and peaks.get("bf16_tflops_sustained"):
        # `peak` is the burst figure; a step timed inside blocks that add up to half a second runs under the
        # power cap, where the library GEMM itself settles at the sustained figure
        extra = {"peak_sustained": peaks["bf16_tflops_sustained"],
                 "frac_of_sustained": achieved / peaks["bf16_tflops_sustained"]}
    return {"bound": wl.bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak, **extra,
            "traffic": NCU_TRAFFIC_BYTES.get(wl.name), "peak_source": peak_src,
            "algorithmic_bytes_per_launch": wl.alg_bytes, "algorithmic_flops_per_launch": wl.alg_flops,
            "frac_of_nominal": achieved / (8000.0 if wl.bound == "hbm" else 2250.0),
            "duration": "CUDA-event time of one step on the launching stream (median block of `steps` steps)"}


MIN_SECONDS = 0.5   # device time covered by the repeated blocks of one measurement (--min-seconds)


def timed_record(wl, fa, steps, warmup, world, device, rank, local, peaks, peak_src):
    """Warm up, then time `wl.step` in blocks of `steps` with the clocks sampled across the timed blocks."""
    import flash_attn_v100_b200
    for _ in range(max(warmup, 3)):
        wl.step(fa)
    torch.cuda.synchronize()
    flash_attn_v100_b200.check_async_errors()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.15)
    m = measure(lambda: wl.step(fa), steps, world, device, getattr(wl, "flush", None), min_seconds=MIN_SECONDS)
    clocks = sampler.stop() if rank == 0 else None
    flash_attn_v100_b200.check_async_errors()
    ms_per_step = m["ms_block"] / steps
    return {"workload": wl.name, "metric": wl.metric, "value": wl.units_per_step * world / (ms_per_step * 1e-3),
            "unit": wl.unit, "ms_per_step": ms_per_step, "ms_per_step_min": m["ms_block_min"] / steps,
            "steps": steps, "blocks": m["blocks"], "timed_seconds": m["timed_seconds"], "dtype": wl.dtype,
            "roofline": roofline_of(wl, ms_per_step, peaks, peak_src), "clocks": clocks, "config": wl.config(),
            "gpu_launches": wl.launches_per_step * steps * m["blocks"]}


def collectives_record(rank, world, device, iters=200):
    """The decode step's all-reduce message (256 x 4096 bf16 = 2 MB) through the library's peer-memory kernel
    and through NCCL: exactness against the fp32 rank-order sum, device time (max over ranks), algorithmic
    NVLink bytes per rank 2*(N-1)/N*n*2 over that time, and the kernel's status word."""
    import torch.distributed as dist
    from flash_attn_v100_b200.comm import PeerCollectives
    rows, cols = 256, 4096
    n = rows * cols
    pc = PeerCollectives(dist.group.WORLD, device, n * 2)
    g = torch.Generator(device=device).manual_seed(4242 + rank)
    x = torch.randn(rows, cols, generator=g, device=device).bfloat16()
    parts = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(parts, x)
    acc = torch.zeros(rows, cols, dtype=torch.float32, device=device)
    for part in parts:                         # rank order, fp32, one rounding: what the kernel computes
        acc += part.float()
    want = acc.bfloat16()
    v = pc.view(0, (rows, cols), torch.bfloat16)
    v.copy_(x)
    pc.all_reduce_(v)
    torch.cuda.synchronize()
    exact = bool(torch.equal(v, want))
    y = torch.zeros(rows, cols, dtype=torch.bfloat16, device=device)
    v.zero_()                                  # zeros stay zeros however often they are summed

    def timed(fn):
        for _ in range(10):
            fn()
        return time_steps(fn, iters, world, device) / iters * 1e3   # microseconds, max over ranks

    us_peer = timed(lambda: pc.all_reduce_(v))
    us_nccl = timed(lambda: dist.all_reduce(y))
    status_ok = True
    try:
        pc.check()
    except RuntimeError:
        status_ok = False
    flag = torch.tensor([1 if (exact and status_ok) else 0], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    pc.close()
    link_bytes = 2.0 * (world - 1) / world * n * 2
    return {"message": "256 x 4096 bf16 (2 MB), sum all-reduce, in place", "peer_us": us_peer, "nccl_us": us_nccl,
            "nvlink_bytes_per_rank": link_bytes, "peer_gbs_per_rank": link_bytes / us_peer / 1e3,
            "nccl_gbs_per_rank": link_bytes / us_nccl / 1e3, "exact_vs_fp32_rank_order_sum_all_ranks": bool(flag.item()),
            "peer_status_clean": status_ok, "nvls": "off (NCCL_NVLS_ENABLE=0); peer kernel uses plain peer loads/stores",
            "link_peak_gbs": 770.0}


def run_b200(args):
    rank, world, local = dist_setup(args.gpus)
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    import flash_attn_v100 as fa
    import flash_attn_v100_b200
    peaks, peak_src = load_peaks()

    wl = WORKLOADS[args.workload](device, seed=rank)
    head = timed_record(wl, fa, args.steps, args.warmup, world, device, rank, local, peaks, peak_src)
    headline = args.workload == "paged_decode"

    e2e = None
    if wl.step_e2e is not None:
        for _ in range(3):
            wl.step_e2e(fa)
        m = measure(lambda: wl.step_e2e(fa), args.steps, world, device, min_seconds=MIN_SECONDS)
        ms_e2e = m["ms_block"] / args.steps
        h2d, d2h = wl.e2e_bytes()
        e2e = {"value": wl.units_per_step * world / (ms_e2e * 1e-3), "unit": wl.unit,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e, "blocks": m["blocks"],
               "note": "q, block_table and seq_lens copied from pinned host memory and the output read back every "
                       "step through the Python operator API; the KV pool is resident device state"}
    flash_attn_v100_b200.check_async_errors()

    cpu_baseline = None
    if rank == 0 and world == 1 and headline and not args.no_cpu_baseline:
        host = wl.host_copy()
        torch.set_num_threads(os.cpu_count() or 1)
        seqs = list(range(wl.B))          # the whole batch, repeated for about ten seconds of CPU work
        PagedDecode.cpu_reference(host, seqs[:2])
        passes, dt, ref = 0, 0.0, None
        while passes < 40 and dt < 10.0:
            t0 = time.perf_counter()
            ref = PagedDecode.cpu_reference(host, seqs)
            dt += time.perf_counter() - t0
            passes += 1
        got = wl.step(fa).float().cpu()
        err = (got - ref.float()).abs().max().item()
        cpu_baseline = {"value": passes * len(seqs) / dt, "unit": "tokens/s", "cores": torch.get_num_threads(),
                        "kind": "port",
                        "sample": f"all {wl.B} sequences of the same batch, {passes} passes, {dt:.1f} s; PyTorch fp32 "
                                  f"CPU restatement of the reference's SDPA decode oracle",
                        "max_abs_err_vs_gpu": err}
        del host, ref

    extra = {}
    if headline and not args.headline_only:
        t1_ms = head["ms_per_step"]       # one GPU holding all eight KV heads of a batch of this shape
        del wl
        torch.cuda.empty_cache()
        # (1) the same batch shape split by KV-head group over the ranks: strong scaling, no collective
        if 8 % world == 0:
            hs = HeadShardedPagedDecode(device, rank, world)
            rec = timed_record(hs, fa, args.steps, args.warmup, world, device, rank, local, peaks, peak_src)
            ms = rec["ms_per_step"]       # max over ranks: the step of the global batch ends with the slowest shard
            rec.update(ms_per_step=ms, us_per_rank_step=ms * 1e3, value=hs.B / (ms * 1e-3),
                       hbm_gbs_per_gpu=hs.alg_bytes / (ms * 1e-3) / 1e9, scaling="strong",
                       strong_scaling_efficiency_vs_one_gpu=t1_ms / (world * ms),
                       one_gpu_ms_per_step=t1_ms)
            rec["roofline"] = roofline_of(hs, ms, peaks, peak_src)
            rec["roofline"]["traffic"] = None
            # the same launches replayed from a CUDA graph (one rotation over the pools per replay)
            graph, per_replay = hs.graph_of_one_rotation(fa, device)
            for _ in range(3):
                graph.replay()
            mg = measure(graph.replay, max(args.steps // per_replay, 1), world, device, min_seconds=MIN_SECONDS / 2)
            ms_g = mg["ms_block"] / max(args.steps // per_replay, 1) / per_replay
            flash_attn_v100_b200.check_async_errors()
            rec.update(us_per_rank_step_graph_replay=ms_g * 1e3,
                       hbm_gbs_per_gpu_graph_replay=hs.alg_bytes / (ms_g * 1e-3) / 1e9,
                       strong_scaling_efficiency_graph_replay_vs_one_gpu=t1_ms / (world * ms_g))
            del graph
            extra["head_sharded"] = rec
            del hs
            torch.cuda.empty_cache()
        # (2) the rest of the metric: causal varlen prefill and INT8 decode, on one GPU
        if world == 1:
            sec = []
            for cls in (VarlenPrefill, Int8Decode):
                w2 = cls(device, 0)
                sec.append(timed_record(w2, fa, args.steps, args.warmup, 1, device, rank, local, peaks, peak_src))
                del w2
                torch.cuda.empty_cache()
            flash_attn_v100_b200.check_prefill_errors()
            extra["secondary"] = sec
        # (3) the multi-GPU pieces of the engine slice that only a multi-GPU run can show
        if world > 1:
            extra["collectives"] = collectives_record(rank, world, device)
            try:
                from flash_attn_v100_b200.engine.selfcheck import tp_consistency_check
                extra["tp_engine_check"] = tp_consistency_check(rank, world, device)
            except Exception as ex:   # a failed check is a result, not a crash of the benchmark line
                extra["tp_engine_check"] = {"ok": False, "error": repr(ex)[:300]}

    if rank != 0:
        return
    line = {
        "metric": head["metric"], "value": head["value"], "unit": head["unit"], "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": head["dtype"],
        "data": "synthetic (seeded N(0,1) fp16 drawn on the host, random page permutation)",
        "config": head["config"],
        "timing": {"blocks": head["blocks"], "timed_seconds": head["timed_seconds"],
                   "ms_per_step_median_block": head["ms_per_step"], "ms_per_step_fastest_block": head["ms_per_step_min"],
                   "note": "the block of `steps` steps is repeated until at least 0.5 s of device time is covered; "
                           "value and ms_per_step are the median block; clocks are sampled across all blocks"},
        "hbm_gbs_per_gpu": head["roofline"]["achieved"] if head["roofline"]["bound"] == "hbm" else None,
        "roofline": head["roofline"],
        "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": head["gpu_launches"],
        "clocks": head["clocks"], "impl": "b200",
    }
    line.update(extra)
    print(json.dumps(line), flush=True)


def run_reference(args):
    """The reference's CPU implementation of the path: its PyTorch eager fp32 oracle
    (restated in oracle/, since the reference tree is not present on a GPU box),
    on all host cores.  One step = the WHOLE headline batch, rebuilt from the same
    seeds as the batch rank 0 of the GPU arm runs (identical tensors)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    from flash_attn_v100_b200.synthetic import make_paged_decode_batch
    from oracle import attention_oracle as orc
    torch.set_num_threads(os.cpu_count() or 1)
    B, H_Q, H_KV, D = PagedDecode.B, PagedDecode.H_Q, PagedDecode.H_KV, PagedDecode.D
    w = make_paged_decode_batch(B, H_Q, H_KV, D, 512, 8192, table_seed=0, value_seed=0)
    q, kc, vc, bt, sl = w["q"], w["k_cache"], w["v_cache"], w["block_table"], w["seq_lens"]
    for _ in range(max(min(args.warmup, 2), 1)):
        orc.paged_decode(q[:4], kc, vc, bt[:4], sl[:4])
    # bounded: about a minute of CPU work at most (one pass over the batch takes under a second)
    steps = args.steps
    t0 = time.perf_counter()
    done = 0
    for _ in range(steps):
        orc.paged_decode(q, kc, vc, bt, sl)
        done += 1
        if time.perf_counter() - t0 > 90.0:
            break
    dt = (time.perf_counter() - t0) / done
    value = B / dt
    cores = torch.get_num_threads()
    desc = (f"all {B} sequences of the paged-decode batch per step (same seeded tensors as rank 0 of the GPU arm), "
            f"{done} steps timed; PyTorch fp32 CPU restatement of the reference's SDPA decode oracle "
            "(test_decode.py:9-19)")
    line = {
        "impl": "reference", "metric": PagedDecode.metric, "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": done, "warmup": max(min(args.warmup, 2), 1), "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp32 (CPU)",
        "data": "synthetic (seeded N(0,1) fp16 drawn on the host, random page permutation)",
        "config": PagedDecode.config_of(sl, w["n_pages"]),
        "note": "one CPU process whatever --gpus says: its value does not grow with N",
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="paged_decode", choices=sorted(WORKLOADS) + ["engine"])
    ap.add_argument("--engine-tiny", action="store_true", help="engine workload on the tiny test shape")
    ap.add_argument("--engine-nccl-decode", action="store_true",
                    help="engine workload: NCCL collectives in the decode step (chain of CUDA graphs) instead of "
                         "the library's peer-memory collectives (one CUDA graph per step)")
    ap.add_argument("--engine-requests", type=int, default=256)
    ap.add_argument("--engine-prefill-chunk", type=int, default=16)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--headline-only", action="store_true",
                    help="skip the head-sharded, secondary (prefill, INT8) and multi-GPU records of the default run")
    ap.add_argument("--min-seconds", type=float, default=0.5,
                    help="repeat the block of --steps timed steps until this much device time is covered "
                         "(0: one block; used for the profiler's launch list)")
    args = ap.parse_args()
    global MIN_SECONDS
    MIN_SECONDS = args.min_seconds
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "engine":
        run_engine(args)
    else:
        run_b200(args)
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 and torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
