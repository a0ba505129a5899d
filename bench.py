#!/usr/bin/env python
"""Benchmark of the per-token hot path (default: benchmark configuration 5, the token-sharded chain).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload chain5|chain4|route3|rope2|next6|part1]
                    [--eager] [--verify]

A step is one pass of the chain over the rank's token shard:
    chain5 : add+RMSNorm+int8 quant -> softmax top-2 of 8 -> scatter with per-row int8 quant -> weighted gather
For N > 1 launch with torchrun (one rank per GPU); tokens are split evenly by rank, there is no collective on
the data path, and the step time is the maximum over ranks of the device time between CUDA events.
Rank 0 prints ONE JSON line.  The default run (one GPU, chain5) then also times the other configurations briefly
(key `other_configs`).  `--verify` checks, off the clock, every rank's outputs against the CPU oracle (key `verify`).
`--impl reference` times the CPU restatement of the reference path (oracle/) on the host cores instead; it is a
reported baseline, not a target.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

NOMINAL_HBM_GBS = 8000.0
L2_BYTES = 126 * 1024 * 1024
FALLBACK_HBM_GBS = 6650.0
METRIC = "fused_chain_tokens_per_s"
# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) per token of the norm+quant kernel at hidden 7168, from
# an ncu capture of a 32,768-token launch (939.8 MB read + 651.5 MB written); traffic grows in proportion to the
# tokens (every row is touched exactly once).
NORM_QUANT_DRAM_BYTES_PER_TOKEN = (939_755_520 + 651_474_432) / 32768


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs (and, when that region is
    shorter than the sampler's start-up, while the same replays continue off the clock: time_graph_replays)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc = gpu_index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons),
                "window": "the timed replays and, where they take less than 0.5 s, the same replays continued off the clock"}


# ------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------
class Chain5:
    """Configuration 5: T tokens x hidden 7168, softmax top-2 of 8 experts."""
    name = "config5 token_sharded_chain_262144: add+rmsnorm+int8 quant -> softmax top2/8 -> scatter+int8 quant -> weighted gather"
    kernels = ["norm_quant", "softmax_topk", "scatter", "gather"]
    launches_per_step = 5  # norm, softmax, scatter bitmaps + quant, gather (tok2row given: no inversion pass)

    def __init__(self, tokens, hidden=7168, experts=8, topk=2, t0=0, device="cuda", gen_device="cuda", pinned_host=False):
        from mcoplib_b200 import workloads as W
        self.T, self.H, self.E, self.k, self.W = tokens, hidden, experts, topk, W
        self.dev = device
        d = W.norm_quant_inputs(tokens, hidden, t0, 0, gen_device, device)
        self.x, self.res, self.w = d["x"], d["residual"], d["weight"]
        self.logits = W.router_inputs(tokens, experts, t0, 0, gen_device, device)["logits"]
        dd = W.dispatch_inputs(tokens, hidden, experts, topk, t0, 0, gen_device, device, with_hidden=False)
        self.smooth, self.y = dd["smooth"], dd["y"]
        R = tokens * topk
        o = dict(device=device)
        self.codes = torch.empty(tokens, hidden, dtype=torch.int8, **o)
        self.scales = torch.empty(tokens, 1, dtype=torch.float32, **o)
        self.topk_w = torch.empty(tokens, topk, dtype=torch.float32, **o)
        self.topk_ids = torch.empty(tokens, topk, dtype=torch.int32, **o)
        self.rows = torch.empty(R, hidden, dtype=torch.int8, **o)
        self.row_scales = torch.empty(R, dtype=torch.float32, **o)
        self.row2tok = torch.empty(R, dtype=torch.int32, **o)
        self.counts = torch.empty(experts, dtype=torch.int32, **o)
        self.starts = torch.empty(experts, dtype=torch.int32, **o)
        self.tok2row = torch.empty(tokens, topk, dtype=torch.int32, **o)
        self.out = torch.empty(tokens, hidden, dtype=torch.bfloat16, **o)

    def bytes_per_kernel(self):
        return self.W.chain5_bytes(self.T, self.H, self.E, self.k)

    def l2_side_bytes(self):
        # what the SMs take in and put out for the scatter: a token row is read once per expert that consumes it,
        # the first time from DRAM and the other k - 1 times from L2 (the algorithmic bytes count it once)
        return {"scatter": self.W.scatter_bytes(self.T, self.H, self.E, self.k) + (self.k - 1) * self.T * self.H * 2}

    def stages(self, ops):
        return [
            lambda: ops.rms_norm_dynamic_per_token_quant_custom(self.codes, self.x, self.w, self.scales, 1e-6, None, self.res),
            lambda: ops.moe_softmax_topk(self.topk_w, self.topk_ids, self.logits, False),
            lambda: ops.moe_scatter_dynamic_quant(self.x, self.topk_ids, self.topk_w, self.smooth, self.rows, self.row_scales,
                                                  self.row2tok, self.counts, self.starts, self.E, 0, 0, self.tok2row),
            lambda: ops.moe_gather_weighted(self.y, self.row2tok, self.topk_ids, self.topk_w, self.starts, self.out, False, self.tok2row),
        ]

    def inputs(self):
        return [self.x, self.res, self.logits, self.y]

    def outputs(self):
        return [self.codes, self.scales, self.res, self.topk_w, self.topk_ids, self.rows, self.row_scales, self.row2tok,
                self.counts, self.starts, self.out]


class Chain4:
    """Configuration 4: add+RMSNorm+quant at hidden 8192, then RoPE (64 Q / 8 KV heads) + int8 paged KV store."""
    name = "config4 llama70b_prefill_chunk_32768: add+rmsnorm+int8 quant -> neox rope + int8 paged kv store"
    kernels = ["norm_quant", "rope_kv_store"]
    launches_per_step = 2

    def __init__(self, tokens, t0=0, device="cuda", gen_device="cuda", **_):
        from mcoplib_b200 import op as ops
        from mcoplib_b200 import workloads as W
        self.T, self.H, self.W = tokens, 8192, W
        d = W.norm_quant_inputs(tokens, 8192, t0, 0, gen_device, device)
        self.x, self.res, self.w = d["x"], d["residual"], d["weight"]
        nb = max(2048, (tokens + 15) // 16)
        self.r = W.rope_kv_inputs(tokens, 64, 8, 128, 131072, 500000.0, 16, nb, t0, 0, gen_device, device)
        self.codes = torch.empty(tokens, 8192, dtype=torch.int8, device=device)
        self.scales = torch.empty(tokens, 1, dtype=torch.float32, device=device)
        kr = self.r["key"].clone()
        ops.vllm_rotary_embedding(self.r["positions"], self.r["query"].clone(), kr, 128, self.r["cos_sin_cache"], True)
        self.ks, self.vs = W.kv_scales(kr, self.r["value"], 8, 128)

    def bytes_per_kernel(self):
        return {"norm_quant": self.W.norm_quant_bytes(self.T, self.H), "rope_kv_store": self.W.rope_kv_bytes(self.T, 64, 8, 128)}

    def stages(self, ops):
        r = self.r
        return [
            lambda: ops.rms_norm_dynamic_per_token_quant_custom(self.codes, self.x, self.w, self.scales, 1e-6, None, self.res),
            lambda: ops.rope_kv_store_int8(r["positions"], r["query"], r["key"], r["value"], 128, r["cos_sin_cache"], True,
                                           r["key_cache"], r["value_cache"], r["slot_mapping"], self.ks, self.vs),
        ]


class Route3:
    """Configuration 3: DeepSeek-V3-shaped gate (256 experts, 8 groups, top-8) + scatter + weighted gather, hidden 7168."""
    name = "config3 deepseek_route_dispatch_8192: grouped sigmoid gate -> scatter+int8 quant -> weighted gather"
    kernels = ["gate", "scatter", "gather"]
    launches_per_step = 4  # gate, scatter bitmaps + quant, gather

    def __init__(self, tokens, t0=0, device="cuda", gen_device="cuda", **_):
        from mcoplib_b200 import workloads as W
        self.T, self.H, self.E, self.k, self.W = tokens, 7168, 256, 8, W
        r = W.router_inputs(tokens, 256, t0, 0, gen_device, device)
        self.logits, self.bias = r["logits"], r["bias"]
        d = W.dispatch_inputs(tokens, 7168, 256, 8, t0, 0, gen_device, device)
        self.hidden, self.smooth, self.y = d["hidden"], d["smooth"], d["y"]
        R = tokens * 8
        o = dict(device=device)
        self.topk_w = torch.empty(tokens, 8, dtype=torch.float32, **o)
        self.topk_ids = torch.empty(tokens, 8, dtype=torch.int32, **o)
        self.rows = torch.empty(R, 7168, dtype=torch.int8, **o)
        self.row_scales = torch.empty(R, dtype=torch.float32, **o)
        self.row2tok = torch.empty(R, dtype=torch.int32, **o)
        self.counts = torch.empty(256, dtype=torch.int32, **o)
        self.starts = torch.empty(256, dtype=torch.int32, **o)
        self.tok2row = torch.empty(tokens, 8, dtype=torch.int32, **o)
        self.out = torch.empty(tokens, 7168, dtype=torch.bfloat16, **o)

    def bytes_per_kernel(self):
        W = self.W
        return {"gate": W.gate_bytes(self.T, 256, 8), "scatter": W.scatter_bytes(self.T, 7168, 256, 8),
                "gather": W.gather_bytes(self.T, 7168, 8, False)}

    def l2_side_bytes(self):
        return {"scatter": self.W.scatter_bytes(self.T, 7168, 256, 8) + 7 * self.T * 7168 * 2}

    def stages(self, ops):
        return [
            lambda: ops.fused_moe_gate_deepseek(self.logits, self.bias, self.topk_w, self.topk_ids, 8, True, 8, 4, None, 2.5, 0),
            lambda: ops.moe_scatter_dynamic_quant(self.hidden, self.topk_ids, self.topk_w, self.smooth, self.rows, self.row_scales,
                                                  self.row2tok, self.counts, self.starts, 256, 0, 0, self.tok2row),
            lambda: ops.moe_gather_weighted(self.y, self.row2tok, self.topk_ids, self.topk_w, self.starts, self.out, False, self.tok2row),
        ]


class Rope2:
    """Configuration 2: NeoX RoPE + int8 paged KV store, 32 Q / 8 KV heads."""
    name = "config2 rope_kv_4096: neox rope + int8 paged kv store"
    kernels = ["rope_kv_store"]
    launches_per_step = 1

    def __init__(self, tokens, t0=0, device="cuda", gen_device="cuda", **_):
        from mcoplib_b200 import op as ops
        from mcoplib_b200 import workloads as W
        self.T, self.W = tokens, W
        nb = max(2048, (tokens + 15) // 16)
        self.r = W.rope_kv_inputs(tokens, 32, 8, 128, 8192, 500000.0, 16, nb, t0, 0, gen_device, device)
        kr = self.r["key"].clone()
        ops.vllm_rotary_embedding(self.r["positions"], self.r["query"].clone(), kr, 128, self.r["cos_sin_cache"], True)
        self.ks, self.vs = W.kv_scales(kr, self.r["value"], 8, 128)

    def bytes_per_kernel(self):
        return {"rope_kv_store": self.W.rope_kv_bytes(self.T, 32, 8, 128)}

    def stages(self, ops):
        r = self.r
        return [lambda: ops.rope_kv_store_int8(r["positions"], r["query"], r["key"], r["value"], 128, r["cos_sin_cache"], True,
                                               r["key_cache"], r["value_cache"], r["slot_mapping"], self.ks, self.vs)]


class Next6:
    """The operators either side of the path (alternate output formats of part 1, the activation-quant steps after the
    expert up-projection, vLLM's softmax router, its token-major combine and its block-aligned index preparation), each
    timed on its own: hidden 7168, expert intermediate size 2048."""
    name = ("next rows: padded-record norm+quant, norm+quant with norm output, per-token int8 quant, swiglu+quant, "
            "silu_mul+quant, topk_softmax, moe_sum, moe_align_block_size")
    kernels = ["norm_quant_padded", "norm_quant_norm_out", "dynamic_int8_quant", "swiglu_quant", "silu_mul_quant", "topk_softmax",
               "moe_sum", "moe_align_block_size"]
    launches_per_step = 10   # one kernel each, three (rank, scan, fill) for moe_align_block_size at this size

    def __init__(self, tokens, t0=0, device="cuda", gen_device="cuda", **_):
        from mcoplib_b200 import workloads as W
        self.T, self.H, self.I, self.E, self.W = tokens, 7168, 2048, 8, W
        d = W.norm_quant_inputs(tokens, 7168, t0, 0, gen_device, device)
        self.x, self.res, self.w = d["x"], d["residual"], d["weight"]
        o = dict(device=device)
        self.pad = 3840
        self.packed = torch.empty(tokens, 2 * self.pad, dtype=torch.int8, **o)
        self.norm = torch.empty(tokens, 7168, dtype=torch.bfloat16, **o)
        self.codes = torch.empty(tokens, 7168, dtype=torch.int8, **o)
        self.scales = torch.empty(tokens, 1, dtype=torch.float32, **o)
        R = 2 * tokens                                   # rows after a top-2 dispatch
        self.R = R
        self.gu = W.per_token("randn", 80, 2 * t0, 2 * t0 + R, 2 * self.I, torch.bfloat16, 0, gen_device, device)
        self.smooth = torch.ones(self.E, self.I, dtype=torch.float32, **o)
        per = R // self.E
        self.counts = torch.full((self.E,), per, dtype=torch.int32, **o)
        self.counts[-1] += R - per * self.E
        self.starts = (torch.cumsum(self.counts, 0) - self.counts).to(torch.int32)
        self.act = torch.empty(R, self.I, dtype=torch.int8, **o)
        self.act_scale = torch.empty(R, dtype=torch.float32, **o)
        self.row_ids = (torch.arange(R, device=device, dtype=torch.int64) % self.E)
        self.logits = W.router_inputs(tokens, 8, t0, 0, gen_device, device)["logits"]
        self.tw = torch.empty(tokens, 2, dtype=torch.float32, **o)
        self.ti = torch.empty(tokens, 2, dtype=torch.int32, **o)
        self.tsrc = torch.empty(tokens, 2, dtype=torch.int32, **o)
        self.none = torch.empty(0)
        # token-major expert outputs [T, 2, H] (the same bytes as the gather input of configuration 5) and their sum
        self.y3 = W.per_token("randn", 81, 2 * t0, 2 * t0 + R, 7168, torch.bfloat16, 1, gen_device, device).view(tokens, 2, 7168)
        self.ysum = torch.empty(tokens, 7168, dtype=torch.bfloat16, **o)
        # block-aligned index preparation of a DeepSeek-V3-shaped routing: top-8 of 256, blocks of 64
        g = torch.Generator(device="cpu").manual_seed(5)
        self.align_ids = torch.rand(tokens, 256, generator=g).topk(8, dim=-1).indices.to(torch.int32).to(device)
        cap = tokens * 8 + 256 * 64
        self.sorted_ids = torch.empty(cap, dtype=torch.int32, **o)
        self.block_experts = torch.empty(cap // 64, dtype=torch.int32, **o)
        self.post_pad = torch.empty(1, dtype=torch.int32, **o)

    def bytes_per_kernel(self):
        T, H, R, I = self.T, self.H, self.R, self.I
        nq = self.W.norm_quant_bytes(T, H)
        return {"norm_quant_padded": nq + T * H * (2 + 1) + 4 * T,        # + norm output, plain codes and the packed scale
                "norm_quant_norm_out": nq + T * H * 2,
                "dynamic_int8_quant": T * H * (2 + 1) + 4 * T,
                "swiglu_quant": R * I * (4 + 1) + 4 * R + self.E * I * 4,
                "silu_mul_quant": R * I * (4 + 1) + 4 * R + 8 * R,
                "topk_softmax": self.W.gate_bytes(T, 8, 2) - 8 * 4 + 8 * T,
                "moe_sum": T * H * 2 * (2 + 1),
                # ids read, sorted positions and block experts written (the byte count of the reference's own runner)
                "moe_align_block_size": T * 8 * 4 + self.sorted_ids.numel() * 4 + self.block_experts.numel() * 4 + 4}

    def stages(self, ops):
        return [
            lambda: ops.fused_add_rms_norm_dynamic_per_token_quant_padding_output(self.packed, self.norm, self.codes, self.scales, self.x,
                                                                                  self.res, self.w, self.pad, 1e-6),
            lambda: ops.sgl_rms_norm_dynamic_per_token_quant_custom(self.codes, self.norm, self.x, self.w, self.scales, 1e-6, None, self.res),
            lambda: ops.dynamic_scaled_int8_quant(self.codes, self.x, self.scales, None),
            lambda: ops.moe_swiglu_dynamic_quantize(self.gu, self.smooth, self.starts, self.counts, self.act, self.act_scale, self.E),
            lambda: ops.fused_silu_mul_dq_reorder_quant(self.act, self.act_scale, self.gu, self.row_ids, self.none, 0, self.E - 1),
            lambda: ops.topk_softmax(self.tw, self.ti, self.tsrc, self.logits, True),
            lambda: ops.moe_sum(self.y3, self.ysum),
            lambda: ops.moe_align_block_size(self.align_ids, 256, 64, self.sorted_ids, self.block_experts, self.post_pad, None),
        ]


class Part1:
    """The other entry points of parts 1 and 2, each timed on its own on bf16 rows of 7168: fused_add_rms_norm (in place), rms_norm
    with a residual, the 9-argument norm + smooth quant, scale_dynamic_quant, head_rms_norm (56 heads of 128), the unpaged
    int8 store of packed K/V (64 Q + 8 + 8 KV heads of 128, one sequence per 4096 tokens) and sglang's RoPE with the save of the
    rotated K and of V into token-indexed buffers (same heads, positions below 8192, a random permutation of rows), the packed
    rotary_embedding of mcoplib.op (positions from the sequence bounds, output to a second tensor) and the two paged copies of
    K / V rows (8 heads of 128, blocks of 16; flash layout with scattered slots, split layout with the consecutive slots of a
    prefill - scattered slots cost the split layout one 2-byte store per element by construction)."""
    name = ("other entry points: fused_add_rms_norm, rms_norm (+residual), 9-argument rms_norm_dynamic_per_token_quant, "
            "scale_dynamic_quant, head_rms_norm, store_kv_cache_cuda_interface, apply_rope_pos_ids_cos_sin_cache with save, "
            "rotary_embedding (packed), reshape_and_cache_flash, reshape_and_cache")
    kernels = ["fused_add_rms_norm", "rms_norm", "norm_smooth_quant", "scale_dynamic_quant", "head_rms_norm", "store_kv", "rope_kv_save",
               "rotary_embedding_packed", "reshape_and_cache_flash", "reshape_and_cache"]
    launches_per_step = 10

    def __init__(self, tokens, t0=0, device="cuda", gen_device="cuda", **_):
        from mcoplib_b200 import workloads as W
        self.T, self.H = tokens, 7168
        d = W.norm_quant_inputs(tokens, 7168, t0, 0, gen_device, device)
        self.x, self.res, self.w = d["x"], d["residual"], d["weight"]
        o = dict(device=device)
        # the in-place operator gets buffers of its own: it rewrites both of its inputs every step
        self.x_io, self.res_io = self.x.clone(), self.res.clone()
        self.smooth = torch.ones(7168, dtype=torch.bfloat16, **o)
        self.smooth32 = torch.ones(7168, dtype=torch.float32, **o)
        self.out = torch.empty(tokens, 7168, dtype=torch.bfloat16, **o)
        self.after_res = torch.empty_like(self.out)
        self.after_norm = torch.empty_like(self.out)
        self.codes = torch.empty(tokens, 7168, dtype=torch.int8, **o)
        self.scales = torch.empty(tokens, dtype=torch.float32, **o)
        self.head_w = torch.ones(56, 128, dtype=torch.bfloat16, **o)
        # packed qkv for the unpaged store: 64 Q heads (not read), 8 K + 8 V heads of 128; sequences of 4096 tokens
        self.Hq, self.Hkv, self.D, seq = 64, 8, 128, 4096
        self.qkv = W.per_token("randn", 70, t0, t0 + tokens, (self.Hq + 2 * self.Hkv) * self.D, torch.bfloat16, 0, gen_device, device)
        self.qkv = self.qkv.view(tokens, self.Hq + 2 * self.Hkv, self.D)
        nseq = max(1, tokens // seq)
        self.q_lens = torch.full((nseq,), tokens // nseq, dtype=torch.int32, **o)
        self.accum = (torch.arange(nseq + 1, **o) * (tokens // nseq)).to(torch.int32)
        self.cache_lens = torch.zeros(nseq, dtype=torch.int32, **o)
        self.slot_ids = torch.arange(nseq, dtype=torch.int32, **o)
        self.k_cache = torch.empty(nseq, self.Hkv, tokens // nseq, self.D, dtype=torch.int8, **o)
        self.v_cache = torch.empty_like(self.k_cache)
        self.kv_scale = torch.full((self.Hkv, self.D), 30.0, dtype=torch.float32, **o)
        self.nseq = nseq
        # sglang's rope + save: an fp32 cos || sin cache of 8192 positions, buffers of one row per token
        g = torch.Generator(device=device).manual_seed(71 + t0)
        self.rope_pos = torch.randint(0, 8192, (tokens,), generator=g, device=device, dtype=torch.int64)
        inv = 1.0 / (10000.0 ** (torch.arange(0, self.D, 2, dtype=torch.float32, device=device) / self.D))
        f = torch.outer(torch.arange(8192, dtype=torch.float32, device=device), inv)
        self.rope_cache = torch.cat([f.cos(), f.sin()], dim=-1).contiguous()
        self.kv_loc = torch.randperm(tokens, generator=g, device=device).to(torch.int64)
        self.k_buffer = torch.empty(tokens, self.Hkv, self.D, dtype=torch.bfloat16, **o)
        self.v_buffer = torch.empty_like(self.k_buffer)
        # packed rotary_embedding: cos / sin halves of the same table, an output tensor of the packed shape
        self.cos_half = self.rope_cache[:, :self.D // 2].contiguous()
        self.sin_half = self.rope_cache[:, self.D // 2:].contiguous()
        self.packed_out = torch.empty_like(self.qkv)
        # paged copies: blocks of 16 slots
        self.bs = 16
        nb = (tokens + self.bs - 1) // self.bs
        self.flash_k = torch.empty(nb, self.bs, self.Hkv, self.D, dtype=torch.bfloat16, **o)
        self.flash_v = torch.empty_like(self.flash_k)
        self.split_k = torch.empty(nb, self.Hkv, self.D // 8, self.bs, 8, dtype=torch.bfloat16, **o)
        self.split_v = torch.empty(nb, self.Hkv, self.D, self.bs, dtype=torch.bfloat16, **o)
        self.slots_seq = torch.arange(tokens, dtype=torch.int64, **o)
        self.one = torch.ones(1, **o)

    def bytes_per_kernel(self):
        n = self.T * self.H
        kv = self.T * self.Hkv * self.D
        return {"fused_add_rms_norm": 8 * n + 2 * self.H,          # x, residual read and written
                "rms_norm": 8 * n + 2 * self.H,                    # x, residual read; out, after_res written
                "norm_smooth_quant": 9 * n + 4 * self.H + 4 * self.T,  # + after_norm, codes, scale
                "scale_dynamic_quant": 3 * n + 4 * self.H + 4 * self.T,  # x read, codes + scale written
                "head_rms_norm": 4 * n + 2 * self.H,               # every head read and written
                "store_kv": 2 * kv * 2 + 2 * kv + 8 * self.Hkv * self.D,   # K, V heads read, two int8 caches written
                # q, k, v read; q, k written in place; rotated k and v written to the buffers; cos || sin row, position, row id
                "rope_kv_save": self.T * ((self.Hq + 2 * self.Hkv) * self.D * 2 + (self.Hq + self.Hkv) * self.D * 2
                                          + 2 * self.Hkv * self.D * 2 + 4 * self.D + 16),
                # q, k heads read and written to the output tensor, the cos and sin half rows
                "rotary_embedding_packed": self.T * (2 * (self.Hq + self.Hkv) * self.D * 2 + 4 * self.D),
                # K and V rows read, written to the caches, the slot
                "reshape_and_cache_flash": self.T * (4 * self.Hkv * self.D * 2 + 8),
                "reshape_and_cache": self.T * (4 * self.Hkv * self.D * 2 + 8)}

    def stages(self, ops):
        x3 = self.x.view(self.T, 56, 128)
        out3 = self.out.view(self.T, 56, 128)
        q, k = self.qkv[:, :self.Hq], self.qkv[:, self.Hq:self.Hq + self.Hkv]   # rotated in place: norms are kept, values stay put
        v = self.qkv[:, self.Hq + self.Hkv:]
        cache_ops = getattr(torch.ops, ops.torch_namespace + "_cache_ops")
        return [
            lambda: ops.fused_add_rms_norm(self.x_io, self.res_io, self.w, 1e-6),
            lambda: ops.rms_norm(self.out, self.x, self.w, 1e-6, self.after_res, self.res, False),
            lambda: ops.rms_norm_dynamic_per_token_quant(self.codes, self.x, self.w, self.smooth, self.scales, 1e-6, self.after_res,
                                                         self.after_norm, self.res),
            lambda: ops.scale_dynamic_quant(self.x, self.smooth32),
            lambda: ops.head_rms_norm(out3, x3, self.head_w, 1e-6, 0, 56),
            lambda: ops.store_kv_cache_cuda_interface(self.qkv, self.q_lens, self.accum, self.cache_lens, self.slot_ids, self.k_cache,
                                                      self.v_cache, self.kv_scale, self.kv_scale, self.nseq, self.Hq, self.Hkv),
            lambda: ops.apply_rope_pos_ids_cos_sin_cache(q, k, q, k, self.rope_cache, self.rope_pos, False, False, v=v,
                                                         k_buffer=self.k_buffer, v_buffer=self.v_buffer, kv_cache_loc=self.kv_loc),
            lambda: ops.rotary_embedding(self.qkv, self.q_lens, self.accum, self.cache_lens, self.cos_half, self.sin_half, self.packed_out,
                                         self.Hq, self.Hkv, 0),
            lambda: cache_ops.reshape_and_cache_flash(k, v, self.flash_k, self.flash_v, self.kv_loc, "auto", self.one, self.one),
            lambda: cache_ops.reshape_and_cache(k, v, self.split_k, self.split_v, self.slots_seq, "auto", self.one, self.one),
        ]


WORKLOADS = {"chain5": (Chain5, 262144), "chain4": (Chain4, 32768), "route3": (Route3, 8192), "rope2": (Rope2, 4096),
             "next6": (Next6, 65536), "part1": (Part1, 65536)}


# ------------------------------------------------------------------------------------------------
# CPU arm: the oracle restatement of the reference path on the host cores
# ------------------------------------------------------------------------------------------------
def cpu_chain5(sample_tokens: int, reps: int = 1, warm: bool = True):
    """Times the CPU restatement (oracle/ref_ops.py) of configuration 5's chain on `sample_tokens` tokens."""
    from mcoplib_b200 import workloads as W
    from oracle import ref_ops as R
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)

    def make(n):
        d = W.norm_quant_inputs(n, 7168)
        d["logits"] = W.router_inputs(n, 8)["logits"]
        d.update(W.dispatch_inputs(n, 7168, 8, 2, with_hidden=False))
        return d

    def run(d, n):
        R.rms_norm_dynamic_per_token_quant(d["x"], d["weight"], 1e-6, residual=d["residual"])
        w, ids = R.moe_softmax_topk(d["logits"], 2)
        _, _, row2tok, _, starts, _ = R.moe_scatter_dynamic_quant(d["x"], ids, w, d["smooth"], 8)
        R.moe_gather_weighted(d["y"], row2tok, ids, w, starts, torch.empty(n, 7168, dtype=torch.bfloat16), False)

    if warm:
        run(make(512), 512)
    d = make(sample_tokens)
    times = []
    for _ in range(reps):
        t = time.perf_counter()
        run(d, sample_tokens)
        times.append(time.perf_counter() - t)
    return {"seconds": times, "tokens": sample_tokens, "threads": threads}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    sample = args.cpu_sample
    r = cpu_chain5(sample, reps=max(1, args.steps), warm=args.warmup > 0)
    total = sum(r["seconds"])
    value = sample * len(r["seconds"]) / total
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * total / len(r["seconds"]), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": Chain5.name, "tokens_per_step_sample": sample, "hidden": 7168, "experts": 8, "topk": 2},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": r["threads"], "kind": "port",
                         "sample": f"{sample} tokens of the config-5 chain per step, torch CPU oracle, {r['threads']} threads"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), file=_RESULT_OUT or sys.stdout, flush=True)
    return 0


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def e2e_chain5(ops, tokens_rank, chunk, steps, warmup, device):
    """The same chain driven from HOST buffers: the rank's batch is streamed in `chunk`-token pieces from pinned
    host memory (H2D), through the operators, and every output is copied back (D2H), on two alternating streams.
    Returns (seconds per step, h2d bytes per step, d2h bytes per step, the host-side inputs of a chunk, the host-side
    outputs of the last chunk)."""
    chunk = min(chunk, tokens_rank)
    nchunks = (tokens_rank + chunk - 1) // chunk
    slots = []
    host_in = None
    for s in range(2):
        c = Chain5(chunk, device=device, gen_device=device)
        if host_in is None:
            host_in = [t.cpu().pin_memory() for t in c.inputs()]
        host_out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in c.outputs()]
        slots.append((c, host_out, torch.cuda.Stream(device=device)))
    h2d = sum(t.numel() * t.element_size() for t in host_in) * nchunks
    d2h = sum(t.numel() * t.element_size() for t in slots[0][1]) * nchunks
    main = torch.cuda.current_stream()

    def one_step():
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        start.record(main)
        for _, _, st in slots:
            st.wait_event(start)
        for i in range(nchunks):
            c, host_out, st = slots[i % 2]
            with torch.cuda.stream(st):
                for dst, src in zip(c.inputs(), host_in):
                    dst.copy_(src, non_blocking=True)
                for f in c.stages(ops):
                    f()
                for dst, src in zip(host_out, c.outputs()):
                    dst.copy_(src, non_blocking=True)
        for _, _, st in slots:
            ev = torch.cuda.Event()
            ev.record(st)
            main.wait_event(ev)
        stop.record(main)
        return start, stop

    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    evs = [one_step() for _ in range(steps)]
    torch.cuda.synchronize()
    secs = sum(a.elapsed_time(b) for a, b in evs) / 1e3 / steps
    last = slots[(nchunks - 1) % 2]
    return secs, h2d, d2h, host_in, last[1]


_ORIG_AFFINITY = []  # the CPU set of the process before bind_near_gpu narrowed it


def bind_near_gpu(local: int):
    """Runs this process (and therefore the first touch of its pinned host buffers) on the CPUs that share a NUMA node
    with GPU `local`, as listed by sysfs for the GPU's PCI function.  Only the end-to-end leg depends on it: host
    memory on the far socket costs PCIe copy bandwidth.  Returns the CPU list used, or None when sysfs has no answer."""
    try:
        p = torch.cuda.get_device_properties(local)
        bdf = "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
        with open(f"/sys/bus/pci/devices/{bdf}/local_cpulist") as fh:
            text = fh.read().strip()
        cpus = set()
        for part in text.split(","):
            if "-" in part:
                a, b = part.split("-")
                cpus.update(range(int(a), int(b) + 1))
            elif part:
                cpus.add(int(part))
        orig = os.sched_getaffinity(0)
        cpus &= orig
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        _ORIG_AFFINITY.append(orig)
        return text
    except Exception:  # no sysfs entry, no permission, unknown attribute: run unbound
        return None


def build_sets(cls, tokens_rank, t0, device, kw):
    """The workload plus, when its traffic per step is below twice the L2 size, enough identical buffer sets that a
    set has left L2 before its turn comes again.  Returns (first workload, list of stage lists, footprint, nsets)."""
    wl = cls(tokens_rank, t0=t0, device=device, gen_device=device, **kw)
    footprint = sum(wl.bytes_per_kernel().values())
    nsets = 1 if footprint >= 2 * L2_BYTES else int(min(8, -(-2 * L2_BYTES // footprint)))
    sets = [wl] + [cls(tokens_rank, t0=t0, device=device, gen_device=device, **kw) for _ in range(nsets - 1)]
    return wl, sets, footprint, nsets


def time_steps(stage_sets, steps, warmup, world, device, dist):
    """`warmup` untimed steps, then `steps` timed ones between a barrier + synchronize on both sides; CUDA events on the
    launching stream around the region and around every stage.  Returns (elapsed ms, per-stage ms), max over ranks."""
    nsets, nst = len(stage_sets), len(stage_sets[0])
    turn = [0]

    def step(events=None):
        stages = stage_sets[turn[0] % nsets]
        turn[0] += 1
        if events is not None:
            events[0].record()
        for i, f in enumerate(stages):
            f()
            if events is not None:
                events[i + 1].record()

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(nst + 1)] for _ in range(steps)]
    t_start = torch.cuda.Event(enable_timing=True)
    t_stop = torch.cuda.Event(enable_timing=True)
    t_start.record()
    for s in range(steps):
        step(evs[s])
    t_stop.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    elapsed_ms = t_start.elapsed_time(t_stop)
    per_kernel_ms = [sum(evs[s][i].elapsed_time(evs[s][i + 1]) for s in range(steps)) / steps for i in range(nst)]
    if world > 1:
        t = torch.tensor([elapsed_ms] + per_kernel_ms, device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, per_kernel_ms = float(t[0]), [float(v) for v in t[1:]]
    return elapsed_ms, per_kernel_ms, step, turn


def time_graph_replays(step, turn, nsets, steps, warmup, world, device, dist, on_start=None):
    """The same steps as replays of ONE captured step per buffer set (a CUDA graph: same kernels, same buffers, no event
    records and no host launch gaps between the kernels - how a serving engine runs a fixed-shape step).  `warmup` steps of
    replays warm up; barrier + synchronize on both sides of the timed replays; maximum over ranks.
    Returns (total ms, steps replayed)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    turn[0] = 0
    with torch.cuda.graph(g):
        for _ in range(nsets):  # one step per buffer set
            step()
    for _ in range(max(1, -(-warmup // nsets))):
        g.replay()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if on_start:
        on_start()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(1, -(-steps // nsets))
    g0.record()
    for _ in range(reps):
        g.replay()
    g1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    total = g0.elapsed_time(g1)
    if on_start:
        # A clock sampler is running (nvidia-smi needs a few hundred ms for its first line, a short timed region would get no
        # sample at all): the SAME replays continue off the clock until the sampler has seen about 0.5 s of this load.
        t_end = time.time() + max(0.0, 0.5 - total * 1e-3)
        while time.time() < t_end:
            for _ in range(reps):
                g.replay()
            torch.cuda.synchronize()
    if world > 1:
        t = torch.tensor([total], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total = float(t[0])
    return total, reps * nsets


def kernel_table(wl, per_kernel_ms, peak):
    bpk = wl.bytes_per_kernel()
    out = {}
    for name, ms in zip(wl.kernels, per_kernel_ms):
        gbs = bpk[name] / (ms * 1e-3) / 1e9
        out[name] = {"ms": ms, "algorithmic_bytes": bpk[name], "gb_per_s": gbs, "frac_of_measured_copy_peak": gbs / peak,
                     "frac_of_8TBps_nominal": gbs / NOMINAL_HBM_GBS}
    # where a kernel re-reads rows from L2, the rate at which bytes cross between L2 and the SMs is given beside the
    # algorithmic rate (it is not a roofline fraction: the denominator above is a DRAM copy)
    side = wl.l2_side_bytes() if hasattr(wl, "l2_side_bytes") else {}
    for name, b in side.items():
        if name in out:
            out[name]["l2_side_bytes"] = b
            out[name]["l2_side_gb_per_s"] = b / (out[name]["ms"] * 1e-3) / 1e9
    return out


def l2_note(footprint, nsets):
    if nsets == 1:
        return "per-step traffic (%.2f GB) exceeds twice the 126 MB L2; no explicit flush" % (footprint / 1e9)
    return ("per-step traffic %.0f MB: steps rotate through %d identical buffer sets so that no step finds its data in L2"
            % (footprint / 1e6, nsets))


# ------------------------------------------------------------------------------------------------
# verification of the sharded run against the CPU oracle (off the clock; the oracle is the checker, never the product)
# ------------------------------------------------------------------------------------------------
VERIFY_SAMPLE = 1024          # tokens per rank whose rows are recomputed by the oracle
DIGEST_MOD = (1 << 61) - 1


def _digest(per_token: torch.Tensor, t0: int) -> int:
    """Additive digest of a per-token integer tensor [tokens, n]: sum over tokens of (global token index + 1) * (sum over
    j of (j + 1) * value), modulo a prime.  The digests of the shards of a token range add up to the digest of the range."""
    v = per_token.to(torch.int64).reshape(per_token.shape[0], -1)
    col = torch.arange(1, v.shape[1] + 1, device=v.device, dtype=torch.int64)
    h = (v * col).sum(dim=1) % 1_000_003
    tok = torch.arange(t0 + 1, t0 + 1 + v.shape[0], device=v.device, dtype=torch.int64) % 1_000_033
    return int((h * tok % DIGEST_MOD).sum() % DIGEST_MOD)


def verify_chain5(ops, tokens_rank, t0, device, hidden):
    """One step of configuration 5 on FRESH inputs of this rank's shard, every output held against the CPU oracle:
    softmax top-k ids / weights on all tokens; counts, starts, row2tok, tok2row bit-exact on all rows (recomputed from the
    kernel's own ids); norm+quant codes / scales / residual, scatter rows / scales and weighted-gather rows on a fixed
    sample of tokens.  Returns a dict with the number of mismatching checks and the digests of the per-token outputs."""
    from oracle import compare as C
    from oracle import ref_ops as R
    wl = Chain5(tokens_rank, hidden=hidden, t0=t0, device=device, gen_device=device)
    T, H, E, k = wl.T, wl.H, wl.E, wl.k
    n = min(VERIFY_SAMPLE, T)
    idx = torch.arange(n, device=device, dtype=torch.int64) * (T // n)          # evenly spread sample of tokens
    x_s, res_s = wl.x[idx].cpu(), wl.res[idx].cpu()                             # before the step: res is updated in place
    for f in wl.stages(ops):
        f()
    torch.cuda.synchronize()
    bad = []

    def check(name, fn):
        try:
            fn()
        except AssertionError as e:
            bad.append(f"{name}: {str(e)[:200]}")

    # part 1 on the sample
    q_ref, s_ref, r_ref = R.rms_norm_dynamic_per_token_quant(x_s, wl.w.cpu(), 1e-6, residual=res_s)
    check("norm codes", lambda: C.assert_codes(wl.codes[idx], q_ref))
    check("norm scales", lambda: C.assert_close(wl.scales[idx], s_ref))
    check("residual", lambda: C.assert_equal(wl.res[idx].cpu().view(torch.int16), r_ref.view(torch.int16)))
    # router on every token
    logits = wl.logits.cpu()
    w_ref, ids_ref = R.moe_softmax_topk(logits, k)
    ids, tw = wl.topk_ids.cpu(), wl.topk_w.cpu()
    def router():
        excused = C.assert_ids_with_margin(ids, ids_ref, R.softmax_topk_margin(logits, k), logits.abs().amax(-1), "top-k ids")
        assert excused <= max(1, T // 10000), f"{excused} rows excused"
        same = (ids == ids_ref).all(-1)
        C.assert_close(tw[same], w_ref[same], "top-k weights", rel=1e-4, abs_=1e-6)
    check("router", router)
    # permutation on every row, from the kernel's own ids
    r2t_ref, cnt_ref, st_ref, t2r_ref = R.moe_scatter_permutation(ids, E)
    check("counts", lambda: C.assert_equal(wl.counts, cnt_ref))
    check("starts", lambda: C.assert_equal(wl.starts, st_ref))
    nrows = int(cnt_ref.sum())
    check("row2tok", lambda: C.assert_equal(wl.row2tok[:nrows], r2t_ref[:nrows]))
    check("tok2row", lambda: C.assert_equal(wl.tok2row, t2r_ref))
    # scatter rows and gather rows of the sampled tokens: the oracle runs on the sub-problem made of these tokens; a
    # token's rows keep their arithmetic and their relative order, only their row numbers differ
    ci = idx.cpu()
    sub = R.moe_scatter_dynamic_quant(x_s, ids[ci], tw[ci], wl.smooth.cpu(), E)
    rows_sub, sc_sub, _, _, st_sub, t2r_sub = sub
    full_rows = t2r_ref[ci].reshape(-1).long()
    sub_rows = t2r_sub.reshape(-1).long()
    keep = (full_rows >= 0) & (sub_rows >= 0)
    fr, sr = full_rows[keep].to(device), sub_rows[keep]
    check("scatter rows", lambda: C.assert_codes(wl.rows[fr], rows_sub[sr]))
    check("scatter scales", lambda: C.assert_close(wl.row_scales[fr], sc_sub[sr], rel=1e-5, abs_=1e-9))
    y_sub = torch.zeros(n * k, H, dtype=torch.bfloat16)
    y_sub[sr] = wl.y[fr].cpu()
    r2t_sub = torch.full((n * k,), -1, dtype=torch.int32)
    r2t_sub[sr] = torch.arange(n).repeat_interleave(k)[keep].to(torch.int32)
    out_ref = R.moe_gather_weighted(y_sub, r2t_sub, ids[ci], tw[ci], st_sub, torch.zeros(n, H, dtype=torch.bfloat16), False)
    check("gather rows", lambda: C.assert_equal(wl.out[idx].cpu().view(torch.int16), out_ref.view(torch.int16)))
    res = {"mismatches": len(bad), "detail": bad, "sampled_tokens": n, "tokens": T, "rows": nrows,
           "digest_codes": _digest(wl.codes.view(T, -1), t0), "digest_ids": _digest(wl.topk_ids, t0)}
    del wl
    torch.cuda.empty_cache()
    return res


def verify_e2e_chunk(host_in, host_out, chunk):
    """The end-to-end leg drives the chain chunk by chunk, so its outputs are those of one call per chunk: the last chunk's
    host-side outputs are held against the oracle run on that chunk's host-side inputs."""
    from oracle import compare as C
    from oracle import ref_ops as R
    x, res, logits, y = host_in
    codes, scales, res_out, tw, ids, rows, row_scales, row2tok, counts, starts, out = host_out
    bad = []
    from mcoplib_b200 import workloads as W
    w = W.norm_weight(x.shape[1], torch.bfloat16)   # the seeded replicated parameter every chunk was run with
    n = min(2048, chunk)            # the oracle's row arithmetic on the first tokens, its permutation on the whole chunk
    q_ref, s_ref, r_ref = R.rms_norm_dynamic_per_token_quant(x[:n], w, 1e-6, residual=res[:n])
    try:
        C.assert_codes(codes[:n], q_ref); C.assert_close(scales[:n], s_ref)
        C.assert_equal(res_out[:n].view(torch.int16), r_ref.view(torch.int16))
        r2t_ref, cnt_ref, st_ref, _ = R.moe_scatter_permutation(ids, 8)
        C.assert_equal(counts, cnt_ref); C.assert_equal(starts, st_ref)
        C.assert_equal(row2tok[:int(cnt_ref.sum())], r2t_ref[:int(cnt_ref.sum())])
    except AssertionError as e:
        bad.append(str(e)[:200])
    return {"mismatches": len(bad), "detail": bad, "tokens": chunk}


OTHER_CONFIGS = ["chain4", "route3", "rope2", "part1"]


def run_ours(args):
    import torch.distributed as dist
    from mcoplib_b200 import op as ops  # raises if the extension is not built: there is no fallback

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py --impl ours needs a CUDA device (the kernels have no CPU fallback)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    numa = None if args.no_numa_bind else bind_near_gpu(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    n = max(world, 1)

    cls, tokens_global = WORKLOADS[args.workload]
    if args.tokens:
        tokens_global = args.tokens
    if args.scaling == "weak":
        tokens_rank, t0 = tokens_global, rank * tokens_global
        tokens_total = tokens_global * n
    else:
        tokens_rank = tokens_global // n
        t0 = rank * tokens_rank
        tokens_total = tokens_rank * n
    kw = {"hidden": args.hidden} if (args.hidden and args.workload == "chain5") else {}
    wl, sets, footprint, nsets = build_sets(cls, tokens_rank, t0, device, kw)
    stage_sets = [w.stages(ops) for w in sets]

    # Region 1: K eagerly launched steps with CUDA events around every operator - the per-kernel table and the roofline.
    eager_ms, per_kernel_ms, step, turn = time_steps(stage_sets, args.steps, args.warmup, world, device, dist)
    elapsed_ms, timed_as = eager_ms, "eager"
    steps_timed = args.steps

    # Region 2 (the headline unless --eager): the same K steps as CUDA-graph replays of the captured step.
    graph = None
    sampler = ClockSampler(local) if rank == 0 else None
    if not args.eager:
        try:
            gms_total, gsteps = time_graph_replays(step, turn, nsets, args.steps, args.warmup, world, device, dist,
                                                   on_start=(sampler.start if sampler else None))
            graph = {"ms_per_step": gms_total / gsteps, "steps": gsteps}
            elapsed_ms, timed_as, steps_timed = gms_total, "cuda_graph_replay", gsteps
        except Exception as e:  # capture refused: the eager region stays the headline
            graph = None
            print(f"bench: CUDA-graph capture failed ({e}); reporting the eager region", file=sys.stderr)
    if graph is None:
        # eager headline: sample the clocks over a repeat of the eager region
        if sampler:
            sampler.start()
        eager_ms, per_kernel_ms, step, turn = time_steps(stage_sets, args.steps, args.warmup, world, device, dist)
        elapsed_ms = eager_ms
    clocks = sampler.stop() if sampler else None

    e2e = None
    e2e_check = None
    if args.workload == "chain5" and not args.no_e2e:
        secs, h2d, d2h, host_in, host_out = e2e_chain5(ops, tokens_rank, args.e2e_chunk, args.steps, args.warmup, device)
        rank_secs = [secs]
        if world > 1:
            t = torch.zeros(world, device=device, dtype=torch.float64)
            t[rank] = secs
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
            rank_secs = [float(v) for v in t]
            secs = max(rank_secs)
        e2e = {"value": tokens_total / secs, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": secs * 1e3, "steps": args.steps, "warmup": args.warmup, "host_cpus": numa or "unbound",
               # both directions run at once; per rank, bytes of the rank's own step over the rank's own step time
               "h2d_gb_per_s_per_rank": [h2d / s / 1e9 for s in rank_secs],
               "d2h_gb_per_s_per_rank": [d2h / s / 1e9 for s in rank_secs],
               "how": f"host pinned buffers -> H2D -> operators -> D2H of every output, streamed in {min(args.e2e_chunk, tokens_rank)}-token "
                      "chunks on two streams per rank (one operator call per chunk: counts, starts and the row order are per chunk)"}
        if args.verify:
            e2e_check = verify_e2e_chunk(host_in, host_out, min(args.e2e_chunk, tokens_rank))
        del host_in, host_out

    verify = None
    if args.verify and args.workload == "chain5":
        v = verify_chain5(ops, tokens_rank, t0, device, wl.H)
        if e2e_check is not None:
            v["mismatches"] += e2e_check["mismatches"]
            v["detail"] += ["e2e chunk: " + d for d in e2e_check["detail"]]
        mine = torch.tensor([[v["mismatches"], v["sampled_tokens"], v["digest_codes"], v["digest_ids"], v["rows"]]], dtype=torch.int64,
                            device=device)
        if world > 1:
            from mcoplib_b200 import sharding
            allv = sharding.gather_for_verification(mine, world)   # one row per rank, over NCCL
        else:
            allv = mine
        allv = allv.cpu()
        verify = {"ranks": n, "sampled_tokens": int(allv[:, 1].sum()), "mismatches": int(allv[:, 0].sum()),
                  "rows_checked_bit_exact": int(allv[:, 4].sum()),
                  "per_rank_mismatches": [int(x) for x in allv[:, 0]],
                  "digest_codes": int(allv[:, 2].sum() % DIGEST_MOD), "digest_ids": int(allv[:, 3].sum() % DIGEST_MOD),
                  "detail": v["detail"][:4],
                  "what": "every rank: one step on fresh inputs of its shard against the CPU oracle - router ids/weights and the "
                          "scatter permutation on all tokens/rows, norm+quant, scatter rows and weighted-gather rows on the "
                          "sampled tokens" + ("; one end-to-end chunk from its host-side outputs" if e2e_check is not None else "")}
        if args.record_digest and n == 1 and rank == 0:
            with open(args.record_digest, "w") as fh:
                json.dump({f"{tokens_total}x{wl.H}": {"codes": verify["digest_codes"], "ids": verify["digest_ids"]}}, fh)
        ref_digest = known_digest(tokens_total, wl.H)
        if ref_digest is not None:
            verify["digest_matches_single_gpu_run"] = (verify["digest_codes"] == ref_digest["codes"] and verify["digest_ids"] == ref_digest["ids"])
            if not verify["digest_matches_single_gpu_run"]:
                verify["mismatches"] += 1
    if world > 1:
        dist.barrier()

    other = None
    if args.workload == "chain5" and n == 1 and not args.no_other_configs and not args.tokens and not args.hidden:
        # the other benchmark configurations, each timed briefly on its own (same rules: warm-up, CUDA events, buffer
        # rotation below twice the L2 size), so that one run records every per-kernel figure
        del sets, stage_sets, step
        wl_keep = wl
        torch.cuda.empty_cache()
        other = {}
        peak, _ = measured_peak()
        for name in OTHER_CONFIGS:
            ocls, otok = WORKLOADS[name]
            owl, osets, ofoot, onsets = build_sets(ocls, otok, 0, device, {})
            sm = ClockSampler(local)
            sm.start()
            steps_o = min(args.steps, 10)
            oms, opk, ostep, oturn = time_steps([w.stages(ops) for w in osets], steps_o, 3, 1, device, dist)
            oeager = oms / steps_o
            try:
                # (on_start given: the replays continue off the clock until the sampler above has seen 0.5 s of this load)
                gtot, gst = time_graph_replays(ostep, oturn, onsets, steps_o, 3, 1, device, dist, on_start=lambda: None)
                oms, steps_o = gtot, gst
            except Exception:
                pass
            oclk = sm.stop()
            del ostep
            other[name] = {"workload": owl.name, "tokens": otok, "ms_per_step": oms / steps_o, "steps": steps_o, "warmup": 3,
                           "eager_ms_per_step": oeager,
                           "kernels": kernel_table(owl, opk, peak), "l2": l2_note(ofoot, onsets),
                           "gpu_launches": owl.launches_per_step * steps_o, "clocks": oclk}
            del owl, osets
            torch.cuda.empty_cache()
        wl = wl_keep

    if rank == 0:
        ms_per_step = elapsed_ms / steps_timed
        peak, peak_kind = measured_peak()
        bpk = wl.bytes_per_kernel()
        kernels = kernel_table(wl, per_kernel_ms, peak)
        dom = max(wl.kernels, key=lambda k: bpk[k])
        traffic = None
        if dom == "norm_quant" and NORM_QUANT_DRAM_BYTES_PER_TOKEN is not None and wl.H == 7168:
            traffic = NORM_QUANT_DRAM_BYTES_PER_TOKEN * tokens_rank
        line = {
            "metric": METRIC, "value": tokens_total / (ms_per_step * 1e-3), "unit": "tokens/s", "n_gpus": n, "steps": steps_timed,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling,
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": wl.name, "hidden": getattr(wl, "H", None), "tokens_global": tokens_total, "tokens_per_gpu": tokens_rank,
                       "parallelism": f"token-sharded x{n}, no collective on the data path", "l2": l2_note(footprint, nsets)},
            "roofline": {"bound": "hbm", "kernel": dom, "achieved": kernels[dom]["gb_per_s"], "peak": peak, "peak_kind": f"of {peak_kind}",
                         "unit": "GB/s", "frac": kernels[dom]["gb_per_s"] / peak, "traffic": traffic},
            "kernels": kernels,
            "gpu_launches": wl.launches_per_step * steps_timed,
            "clocks": clocks,
            "impl": "ours",
            "timed_region": ("K replays of one captured step (CUDA graph): the same kernels on the same buffers without event records "
                             "or host launch gaps between them" if timed_as == "cuda_graph_replay"
                             else "K eagerly launched steps"),
            "kernels_from": "a region of K eagerly launched steps with CUDA events around every operator (same buffers, same run)",
            "eager": {"ms_per_step": eager_ms / args.steps, "value": tokens_total / (eager_ms / args.steps * 1e-3), "unit": "tokens/s",
                      "steps": args.steps},
        }
        if args.csv:
            # performance history in the manner of the reference's benchmark driver (benchmark/README.md:84-103); the report
            # goes to stderr, stdout stays one JSON line
            from mcoplib_b200 import perf_csv
            mode = "generate" if args.generate else ("update" if args.update else "compare")
            recs = [perf_csv.make_record(torch.cuda.get_device_name(local), f"{args.workload}/{k}", "bf16", f"tokens={tokens_rank}",
                                         args.steps, v["ms"] * 1e3, v["gb_per_s"], peak) for k, v in kernels.items()]
            print(perf_csv.format_report(perf_csv.apply(args.csv, recs, mode)), file=sys.stderr, flush=True)
        if e2e is not None:
            line["e2e"] = e2e
        if verify is not None:
            line["verify"] = verify
        if other is not None:
            line["other_configs"] = other
        if n == 1 and args.workload == "chain5" and not args.no_cpu_baseline:
            if _ORIG_AFFINITY:
                os.sched_setaffinity(0, _ORIG_AFFINITY[0])  # the CPU baseline uses every host core again
            r = cpu_chain5(args.cpu_sample, reps=args.cpu_reps)
            total = sum(r["seconds"])
            v = r["tokens"] * len(r["seconds"]) / total
            line["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": r["threads"], "kind": "port",
                                    "sample": f"{len(r['seconds'])} passes over {r['tokens']} tokens of the same chain, torch CPU "
                                              f"oracle, {r['threads']} threads, {total:.1f} s of CPU work"}
        print(json.dumps(line), file=_RESULT_OUT or sys.stdout, flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


def known_digest(tokens_total, hidden):
    """Digests of the per-token outputs (int8 codes of part 1, expert ids of the router) of a single-GPU run on the same
    seeded inputs, recorded by `bench.py --verify --record-digest FILE` and kept in tests/golden/chain5_digest.json.  The inputs are
    generated per 4096-token chunk from chunk-indexed seeds, so every sharding must reproduce them."""
    try:
        with open(os.path.join(ROOT, "tests", "golden", "chain5_digest.json")) as fh:
            return json.load(fh).get(f"{tokens_total}x{hidden}")
    except Exception:
        return None


_RESULT_OUT = None  # the process's original standard output, kept for the one result line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="chain5", choices=sorted(WORKLOADS))
    ap.add_argument("--tokens", type=int, default=0, help="override the global token count of the workload")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="strong: the configuration's tokens are split across ranks (as configuration 5 states); weak: each rank gets all of them")
    ap.add_argument("--e2e-chunk", type=int, default=16384)
    ap.add_argument("--cpu-sample", type=int, default=0,
                    help="tokens per CPU sample (default 16384 for the cpu_baseline of the GPU arm, 8192 per step of --impl reference)")
    ap.add_argument("--cpu-reps", type=int, default=8, help="passes over the CPU sample for the cpu_baseline of the GPU arm")
    ap.add_argument("--hidden", type=int, default=0, help="chain5 only: another row length than 7168 (per-kernel study)")
    ap.add_argument("--csv", default="", help="performance history file; with --generate, --update or --compare (default)")
    ap.add_argument("--generate", action="store_true", help="add records that the history does not hold yet")
    ap.add_argument("--update", action="store_true", help="replace stored records that the run beats by more than 5 %%")
    ap.add_argument("--compare", action="store_true", help="report the run against the stored records")
    ap.add_argument("--no-numa-bind", action="store_true", help="do not bind the process to the CPUs local to its GPU")
    ap.add_argument("--eager", action="store_true", help="headline from the eagerly launched steps instead of CUDA-graph replays of the step")
    ap.add_argument("--graph", action="store_true", help=argparse.SUPPRESS)  # (replays are the default now)
    ap.add_argument("--verify", action="store_true",
                    help="after the timed regions, every rank checks one step of its shard (and one end-to-end chunk) against the CPU oracle")
    ap.add_argument("--record-digest", default="", metavar="FILE",
                    help="with --verify on one GPU: write the output digests to FILE (kept in tests/golden/chain5_digest.json for sharded runs)")
    ap.add_argument("--no-other-configs", action="store_true", help="one GPU, chain5: do not time the other configurations afterwards")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    # Standard output carries exactly one JSON line.  Libraries print there too (NCCL's version banner on the first
    # collective), so file descriptor 1 is pointed at standard error for everything but that line.
    global _RESULT_OUT
    sys.stdout.flush()
    _RESULT_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3  # timing rule: at least three untimed steps
    if args.impl == "reference":
        args.cpu_sample = args.cpu_sample or 8192
        return run_reference(args)
    args.cpu_sample = args.cpu_sample or 16384
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
