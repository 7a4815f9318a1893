#!/usr/bin/env python
"""Benchmark of the speculative-decoding hot path on B200: tree verify + accept, then accepted-path KV compaction.

Workload (BASELINE.json configs[4], "8-GPU sharded speculative step"): 512 independent sequences
split over the N GPUs of one box.  Each sequence owns a 64-node draft tree and target logits
bf16 [64, 152064] ~ N(0, 3^2) with one drafted child boosted by +6 at 60 % of the internal nodes,
and a paged bf16 KV region of 28 layers x 4 KV heads x 128 dim x 4096 tokens (page 16, random page
table).  One "step" of a sequence = greedy (exact) verify, lossy verify (entropy gate 0.3, window 6)
and compaction of the accepted path's KV rows.  Sequences are processed in waves of `--wave`
sequences (one launch per kernel per wave); there is no collective on the hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W]            # N > 1: launched by torchrun
    python bench.py --impl reference ...                            # the CPU restatement of the reference path

Prints ONE JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

VOCAB = 152064
NODES = 64
KV_LAYERS, KV_HEADS, KV_DIM, KV_TOKENS, PAGE_LEN = 28, 4, 128, 4096, 16
LOSSY_KW = {"threshold_method": "entropy", "threshold": 0.3, "window_size": 6}
METRIC = "tree verify+accept steps/s"
CPU_SAMPLE = 16  # sequences per pass of the CPU path: ~0.5 s on 16 cores, so three passes or twenty steps stay short


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--seqs", type=int, default=512, help="sequences in the whole job (split over the GPUs)")
    ap.add_argument("--wave", type=int, default=64, help="sequences per kernel launch")
    ap.add_argument("--variant", default="literal", choices=["literal", "peaked"],
                    help="literal: +6 boost as BASELINE.json states; peaked: boosted child = row max + 4")
    ap.add_argument("--kv-tokens", type=int, default=KV_TOKENS)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--two-pass", action="store_true",
                    help="verify greedily and lossily in two launches (two passes over the logits) instead of one")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the side measurements of the other kernels")
    ap.add_argument("--extras-only", choices=["step", "expand", "attention", "stochastic", "gemm", "lmhead", "lmhead-small"], default=None,
                    help="run one of the side measurements alone on GPU 0 and print it as one JSON line")
    ap.add_argument("--cpu-sample", type=int, default=CPU_SAMPLE,
                    help="sequences per pass of the CPU path (the cpu_baseline leg and the reference arm use the same)")
    return ap.parse_args()


# --------------------------------------------------------------------------------------
# inputs
# --------------------------------------------------------------------------------------
def make_wave_inputs(seq_ids, variant: str, device, with_logits=True):
    """Trees (host) and logits (device) for the given global sequence ids; everything seeded by the id."""
    from subspec_b200 import synthetic

    return synthetic.config5_wave(seq_ids, variant, device, nodes=NODES, vocab=VOCAB, with_logits=with_logits)


def flats_of(trees):
    from subspec_b200.tree import Tree
    from subspec_b200.verify import flatten_tree

    out = []
    for st in trees:
        t = Tree.from_arrays(st.token_ids.tolist(), st.parents.tolist())
        tok, off, idx = flatten_tree(t, 0, limit=st.n, restrict=True)
        out.append((tok, off, idx, st.n, 0))
    return out


# --------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, device_index: int, period_s: float = 0.0005):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            uuid = torch.cuda.get_device_properties(device_index).uuid
            self._nv = pynvml
            try:
                self._h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(uuid)).encode())
            except Exception:
                self._h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
            self._period = period_s
        except Exception as e:  # NVML missing: report that instead of numbers
            self._nv = None
            self.error = repr(e)

    def _loop(self):
        nv = self._nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self._period)

    def sample_now(self):
        """One sample from the calling thread (the timed region's launches are queued and still running)."""
        if self._nv is None:
            return
        nv = self._nv
        try:
            self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
        except Exception:
            pass

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if self._nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "error": self.error}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# --------------------------------------------------------------------------------------
# CPU restatement of the reference path (oracle), used as baseline and as the reference arm
# --------------------------------------------------------------------------------------
def cpu_step(trees, logits_cpu, pools, beams_out=None):
    """One pass of the reference's CPU path over a list of sequences: verify exact, verify lossy, KV reorder."""
    from oracle import kv_oracle as ko
    from oracle import verify_oracle as vo

    accepted = 0
    for i, st in enumerate(trees):
        lg = logits_cpu[i]
        tok, ch = st.token_ids.tolist(), st.children()
        vo.verify(logits=lg, token_ids=tok, children=ch, method="exact")
        r = vo.verify(logits=lg, token_ids=tok, children=ch, method="lossy", threshold=LOSSY_KW["threshold"],
                      window=LOSSY_KW["window_size"], threshold_method="entropy")
        accepted += len(r.tokens)
        if pools is not None:
            ko.paged_reorder(pools[i % len(pools)], torch.tensor(r.hidden), KV_TOKENS - NODES)
    return accepted


def cpu_baseline(sample: int, reps: int, variant: str):
    """Times `reps` passes of the CPU path over `sample` sequences; returns (seq-steps/s, description)."""
    torch.set_num_threads(os.cpu_count() or 1)
    seq_ids = list(range(sample))
    trees, _ = make_wave_inputs(seq_ids, variant, "cpu", with_logits=False)
    gen = torch.Generator().manual_seed(123)
    logits = (torch.randn(sample, NODES, VOCAB, generator=gen) * 3.0).to(torch.bfloat16)
    # one identity-table pool per sequence in flight, as the reference's FlashInferCache allocates it
    pool = (torch.randn(KV_LAYERS, KV_TOKENS // PAGE_LEN, 2, PAGE_LEN, KV_HEADS, KV_DIM, generator=gen)
            .to(torch.bfloat16))
    cpu_step(trees[:1], logits[:1], [pool])  # warm-up
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        cpu_step(trees, logits, [pool])
        times.append(time.perf_counter() - t0)
    times.sort()
    med = times[len(times) // 2]
    return sample / med, (f"{sample} sequences x {reps} passes (median): torch-CPU softmax/entropy/argmax + Python walk "
                          f"(exact, then lossy) on bf16 [64,{VOCAB}] logits, then clone-whole-pool KV reorder of a "
                          f"{pool.numel() * 2 / 1e6:.1f} MB pool, as the reference does per sequence")


def moved_row_count(out) -> int:
    """Accepted-path rows whose source differs from their destination (beam[i] != i): the rows compaction moves."""
    moved = 0
    for b in range(out["out_meta"].shape[0]):
        L = int(out["out_meta"][b, 0])
        moved += int((out["out_hidden"][b, :L] != np.arange(L)).sum())
    return moved


def profiled_traffic(wave: int):
    """DRAM bytes per verify launch (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture at a wave of
    64 sequences), read from the summary of that capture; None when the summary does not state it."""
    import re

    path = ROOT / "profiles" / "verify_rows_kernel_bf16_wave64.md"
    if not path.exists():
        return None
    m = re.search(r"dram_bytes_per_launch_wave64:\s*([0-9.eE+]+)", path.read_text())
    return float(m.group(1)) * wave / 64 if m else None


def spot_check(spot):
    """The GPU's lossy-verify results of a few sequences against the CPU restatement; raises on a mismatch."""
    from oracle import verify_oracle as vo

    for seq_id, logits, st, tokens, hidden in spot:
        r = vo.verify(logits=logits, token_ids=st.token_ids.tolist(), children=st.children(), method="lossy",
                      threshold=LOSSY_KW["threshold"], window=LOSSY_KW["window_size"], threshold_method="entropy",
                      upcast=True)
        if (tokens, hidden) != (r.tokens, r.hidden):
            raise SystemExit(f"parity check failed on sequence {seq_id}: {(tokens, hidden)} vs {(r.tokens, r.hidden)}")
    return len(spot)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    sample = args.cpu_sample
    torch.set_num_threads(cores)
    seq_ids = list(range(sample))
    trees, _ = make_wave_inputs(seq_ids, args.variant, "cpu", with_logits=False)
    gen = torch.Generator().manual_seed(123)
    logits = (torch.randn(sample, NODES, VOCAB, generator=gen) * 3.0).to(torch.bfloat16)
    pool = (torch.randn(KV_LAYERS, KV_TOKENS // PAGE_LEN, 2, PAGE_LEN, KV_HEADS, KV_DIM, generator=gen)
            .to(torch.bfloat16))
    accepted = 0
    for _ in range(args.warmup):
        cpu_step(trees[:1], logits[:1], [pool])
    t0 = time.perf_counter()
    for _ in range(args.steps):
        accepted += cpu_step(trees, logits, [pool])
    dt = time.perf_counter() - t0
    value = sample * args.steps / dt
    desc = (f"each step = {sample} sequences of the workload through the CPU restatement of the reference path "
            f"(oracle/verify_oracle.py + oracle/kv_oracle.py), {cores} torch threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "steps/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, args.seqs, max(1, args.gpus), args.seqs // max(1, args.gpus)),
        "accepted_tok_per_s": accepted / dt,
        "cpu_baseline": {"value": value, "unit": "steps/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, total_seqs, world, per_rank):
    return {
        "workload": "BASELINE.json configs[4]: sharded speculative step (greedy + lossy verify of 64-node trees, "
                    "vocab 152064, bf16 logits; accepted-path KV compaction, 28x4x128x4096 bf16 paged cache, page 16, "
                    "random page table)",
        "sequences": total_seqs, "sequences_per_gpu": per_rank, "wave": args.wave, "variant": args.variant,
        "lossy": LOSSY_KW, "kv_tokens": args.kv_tokens, "parallelism": f"dp{world}",
        "verify_launches": ("two (greedy, then lossy: two passes over the logits)" if args.two_pass else
                            "one (greedy and lossy results from one pass over the logits)"),
        "l2": "inputs larger than L2 (each wave streams 1.25 GB of logits per verify pass; no flush needed)",
    }


# --------------------------------------------------------------------------------------
# side measurements: the other kernels of the path on their own configs (not part of `value`)
# --------------------------------------------------------------------------------------
def _spin_up(device, ms=60.0):
    """Keep the GPU busy for a while so that short kernels are timed at boost clocks, not during the ramp from idle."""
    a = torch.empty(64 << 20, dtype=torch.float32, device=device)
    t0 = time.perf_counter()
    while (time.perf_counter() - t0) * 1e3 < ms:
        for _ in range(20):
            a.add_(1.0)
        torch.cuda.synchronize()


def _time_ms(fn, iters=10, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def extras(device, peak_gbs, peak_tf, peak_tf_sustained=None):
    """The secondary kernels at their full configurations: one expansion step (config 3), one stochastic
    verification batch (config 2), the W4A16 GEMM shapes (config 4), tree attention, and the lm_head product fused
    with the verification of a wave; each on inputs larger than L2."""
    out = {}
    out.update(extra_step_peaked(device, peak_gbs))
    out.update(extra_expand(device, peak_gbs))
    out.update(extra_attention(device, peak_gbs, peak_tf))
    out.update(extra_stochastic(device, peak_gbs))
    out.update(extra_gemm(device, peak_gbs, peak_tf))
    torch.cuda.empty_cache()
    out.update(extra_lm_head(device, peak_gbs, peak_tf, peak_tf_sustained or peak_tf))
    return out


def extra_step_peaked(device, peak_gbs, wave=64):
    """One wave of the sharded step on the "peaked" inputs (boosted child = row maximum + 4), where the walks
    accept tokens, the lossy gate opens and compaction moves real rows; the literal inputs accept next to
    nothing, so their compaction launch finds every kept row already in place."""
    from subspec_b200 import synthetic
    from subspec_b200.step import SpeculativeStepBatch

    pages_per_seq = KV_TOKENS // PAGE_LEN
    ids = list(range(wave))
    trees, logits = make_wave_inputs(ids, "peaked", device)
    sb = SpeculativeStepBatch(wave, NODES, device, kv_layers=KV_LAYERS, kv_heads=KV_HEADS, head_dim=KV_DIM,
                              page_len=PAGE_LEN, pages_per_seq=pages_per_seq,
                              page_table=synthetic.random_page_table(wave, pages_per_seq,
                                                                     torch.Generator().manual_seed(31)))
    for layer in range(KV_LAYERS):
        sb.pool[layer].normal_()
    sb.set_trees(flats_of(trees))
    sb.set_kv_offsets([KV_TOKENS - NODES] * wave)

    def step():
        sb.verify(logits, verify_method="exact+lossy", verify_kwargs=LOSSY_KW)
        sb.compact_kv()

    _spin_up(device)
    ms_step = _time_ms(step, iters=50, warm=5)
    res = sb.results()
    kept, moved = int(res["out_meta"][:, 0].sum()), moved_row_count(res)
    # the compaction launch alone: its inputs (the verify outputs) stay as the last step left them, and a
    # repeated compaction moves the same rows again, so every launch does the same work
    ms_kv = _time_ms(sb.compact_kv, iters=200, warm=10)
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        for _ in range(20):
            sb.compact_kv()
    ms_kv_graph = _time_ms(gr.replay, iters=20, warm=3) / 20
    sb.results()
    moved_bytes = 2 * moved * sb.kv_row_bytes
    floor_us = moved_bytes / (peak_gbs * 1e9) * 1e6
    out = {"step_peaked_wave64": {
        "ms_verify_plus_compact": ms_step, "sequence_steps_per_s": wave / (ms_step * 1e-3),
        "accepted_tokens_per_sequence": (kept - wave) / wave, "tokens_emitted_per_s": kept / (ms_step * 1e-3),
        "kv_compact": {"us_per_launch_eager": ms_kv * 1e3, "us_per_launch_in_graph": ms_kv_graph * 1e3,
                       "rows_kept": kept, "rows_moved": moved, "bytes_read_plus_written": moved_bytes,
                       "GB/s": moved_bytes / (ms_kv_graph * 1e-3) / 1e9,
                       "frac_of_measured_peak": moved_bytes / (ms_kv_graph * 1e-3) / 1e9 / peak_gbs,
                       "floor_us_at_peak": floor_us,
                       "bound": "launch and latency: one dependent chain (counts, beam, page table, bulk load, "
                                "bulk store) per CTA; the bytes alone would take floor_us_at_peak"}}}
    sb.pool = None
    del sb, logits
    torch.cuda.empty_cache()
    return out


def extra_attention(device, peak_gbs, peak_tf, batch=64):
    """Tree attention of one layer at the sharded-step shape: 64 requests, a 64-node tree behind 4032 cached
    rows each (4096 in all, page 16, random page table), 28 query heads on 4 KV heads of dim 128."""
    from subspec_b200 import synthetic
    from subspec_b200.attention import tree_attention_paged

    QL, HQ, HKV, D, page_len, kv = 64, 28, 4, 128, PAGE_LEN, KV_TOKENS
    pages = kv // page_len
    gen = torch.Generator().manual_seed(77)
    table = synthetic.random_page_table(batch, pages, gen).to(device)
    pool = torch.empty(1, batch * pages, 2, page_len, HKV, D, dtype=torch.bfloat16, device=device).normal_()
    q = torch.randn(batch, QL, HQ, D, device=device).to(torch.bfloat16)
    kv_len = torch.full((batch,), kv, dtype=torch.int32, device=device)
    mask = torch.zeros(batch, QL, kv, dtype=torch.bool, device=device)
    mask[:, :, :kv - QL] = True
    mask[:, :, kv - QL:] = torch.tril(torch.ones(QL, QL, dtype=torch.bool, device=device))  # a chain: the densest tree
    _spin_up(device)
    ms = _time_ms(lambda: tree_attention_paged(q, pool, 0, page_table=table, kv_len=kv_len, mask=mask), iters=20, warm=3)
    flops = 4.0 * batch * QL * HQ * kv * D
    nbytes = batch * (2 * kv * HKV * D * 2 + 2 * QL * HQ * D * 2)
    t_roof = max(nbytes / (peak_gbs * 1e9), flops / (peak_tf * 1e12))
    res = {"tree_attention_layer_config5": {
        "ms": ms, "TFLOP/s": flops / (ms * 1e-3) / 1e12, "GB/s": nbytes / (ms * 1e-3) / 1e9,
        "roofline_ms": t_roof * 1e3, "frac": t_roof / (ms * 1e-3), "bound": "tensor",
        "path": "tcgen05 (S and O in tensor memory, K/V tiles by tensor copies)", "requests": batch}}
    del pool, table
    # the same problem on the static caches of the reference's default path, with the additive mask, and what
    # that path itself runs there: torch's scaled_dot_product_attention (repeat_kv done beforehand, not timed)
    from subspec_b200.attention import tree_attention_static
    qh = q.permute(0, 2, 1, 3).contiguous()
    kc = torch.empty(batch, HKV, kv, D, dtype=torch.bfloat16, device=device).normal_()
    vc = torch.empty(batch, HKV, kv, D, dtype=torch.bfloat16, device=device).normal_()
    add = (~mask[:1, None]).to(torch.bfloat16) * torch.finfo(torch.bfloat16).min
    ms_s = _time_ms(lambda: tree_attention_static(qh, kc, vc, kv_len=kv_len, mask=add), iters=20, warm=3)
    kk, vv = kc.repeat_interleave(HQ // HKV, dim=1), vc.repeat_interleave(HQ // HKV, dim=1)
    sdpa = torch.nn.functional.scaled_dot_product_attention
    ms_t = _time_ms(lambda: sdpa(qh, kk, vv, attn_mask=add), iters=10, warm=3)
    # one request alone (the reference's own setting): device time inside a CUDA graph of ten calls; the cache
    # rows are cut into ranges for several CTAs and merged (the wrapper's default for few requests)
    def graph_us(fn):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for _ in range(10):
                fn()
        gr.replay()
        torch.cuda.synchronize()
        return _time_ms(gr.replay, iters=5, warm=1) * 100.0  # us per call

    one = {}
    q1, k1, v1, len1, o1 = qh[:1], kc[:1], vc[:1], kv_len[:1], torch.empty_like(qh[:1])
    for name, sp in (("whole_cache_per_cta_us", 1), ("split_ranges_us", None)):
        one[name] = graph_us(lambda: tree_attention_static(q1, k1, v1, kv_len=len1, mask=add, out=o1, kv_splits=sp))
    kk1, vv1 = kk[:1], vv[:1]
    one["torch_sdpa_us"] = graph_us(lambda: sdpa(q1, kk1, vv1, attn_mask=add))
    res["tree_attention_layer_config5"]["one_request"] = one
    res["tree_attention_layer_config5"]["static_caches"] = {
        "ms": ms_s, "TFLOP/s": flops / (ms_s * 1e-3) / 1e12, "mask": "additive bf16 [1,1,q,kv]",
        "torch_sdpa_ms": ms_t, "note": "torch_sdpa_ms is the library call the reference's default path makes, beside ours"}
    return res


def extra_expand(device, peak_gbs):
    from subspec_b200.draft import topk_sampling_from_logits

    out = {}
    gen = torch.Generator(device=device).manual_seed(3)
    # config 3: 32 sequences x 16 leaves x 128256 bf16 draft logits, k = 16
    B, L, V, k = 32, 16, 128256, 16
    logits = (torch.randn(B, L, V, generator=gen, device=device) * 3.0).to(torch.bfloat16)
    pp = torch.rand(B, L, generator=gen, device=device).to(torch.bfloat16)
    _spin_up(device)
    ms = _time_ms(lambda: topk_sampling_from_logits(logits, pp, k, 1.0), iters=300, warm=50)
    gbs = logits.numel() * 2 / (ms * 1e-3) / 1e9
    out["expand_step_config3"] = {"ms": ms, "GB/s": gbs, "frac_of_measured_peak": gbs / peak_gbs,
                                  "bytes": logits.numel() * 2}
    return out


def extra_stochastic(device, peak_gbs):
    from subspec_b200 import _lib, synthetic
    from subspec_b200.tree import Tree
    from subspec_b200.verify import flatten_tree, get_workspace

    out = {}
    gen = torch.Generator(device=device).manual_seed(5)
    # config 2: 64 sequences x 128-node trees, bf16 logits N(0, 2.5^2), T = 1, top-p 0.9, injected uniforms
    B, N, V = 64, 128, 152064
    cgen = torch.Generator().manual_seed(4)
    flats = []
    for _ in range(B):
        st = synthetic.random_tree(N, 10, 8, V, cgen)
        t = Tree.from_arrays(st.token_ids.tolist(), st.parents.tolist())
        tok, off, idx = flatten_tree(t, 0, limit=N, restrict=False)
        flats.append((tok, off, idx, N, 0))
    logits = torch.empty(B, N, V, dtype=torch.bfloat16, device=device)
    for b in range(B):
        logits[b] = (torch.randn(N, V, generator=gen, device=device) * 2.5).to(torch.bfloat16)
    ws = get_workspace(B, N, device)
    ws.set_trees(flats)
    ws.uniforms.uniform_(generator=gen)

    def timed(mode, draft=None):
        ms_ = _time_ms(lambda: ws.run(logits, input_kind=_lib.IN_LOGITS, method=_lib.VERIFY_EXACT, do_sample=mode,
                                      temperature=1.0, top_p=0.9, draft_logits=draft), iters=5, warm=2)
        return ms_, ws.fetch()

    # every decoded row draws its target (what the lossy verifier needs): all 2.49 GB are read
    ms, _ = timed(1)
    gbs = logits.numel() * 2 / (ms * 1e-3) / 1e9
    out["stochastic_verify_config2"] = {"ms": ms, "GB/s": gbs, "frac_of_measured_peak": gbs / peak_gbs,
                                        "bytes": logits.numel() * 2, "draws": "every decoded row"}
    # sample-and-match as the reference walks it: a draw only at the contexts the walk stands on.  With the
    # config's unboosted logits no draft token is ever drawn (one context per sequence); the second figure
    # boosts the first child of every node so that walks run down the tree.
    ms_lazy, res = timed(2)
    out["stochastic_verify_config2_walk"] = {"ms": ms_lazy, "contexts_visited_per_sequence":
                                             float((res["node_target"] >= 0).sum(axis=1).mean()),
                                             "draws": "only where the walk stands (default)"}
    for b in range(B):
        tok, off, idx = flats[b][:3]
        first = idx[off[:-1][off[1:] > off[:-1]]]          # first child of every inner node
        parent = np.nonzero(off[1:] > off[:-1])[0]
        logits[b, torch.as_tensor(parent, device=device), torch.as_tensor(tok[first], device=device)] = 16.0
    ms_deep, res = timed(2)
    visited = (res["node_target"] >= 0).sum(axis=1)
    out["stochastic_verify_config2_walk_boosted"] = {"ms": ms_deep, "contexts_visited_per_sequence":
                                                     float(visited.mean()), "most_contexts_in_a_sequence":
                                                     int(visited.max()),
                                                     "accepted_per_sequence": float(res["out_meta"][:, 1].mean())}
    # residual (p - q) acceptance on the same boosted inputs, with draft logits that resemble the target's
    draft = torch.empty_like(logits)
    for b in range(B):
        draft[b] = (logits[b].float() * 0.7 + torch.randn(N, V, generator=gen, device=device)).to(torch.bfloat16)
    ws.accept_uniforms.uniform_(generator=gen)
    ms_res, res = timed(2, draft)
    visited = (res["node_target"] >= 0).sum(axis=1)
    out["stochastic_verify_config2_residual_boosted"] = {"ms": ms_res, "contexts_visited_per_sequence":
                                                         float(visited.mean()), "most_contexts_in_a_sequence":
                                                         int(visited.max()),
                                                         "accepted_per_sequence": float(res["out_meta"][:, 1].mean())}
    del draft, logits
    # fp32 logits (config 1's type: one 64-node tree, V = 152064) have no 16-bit histogram; the filters'
    # boundaries are searched with counting passes over the L2-resident row
    B1, N1 = 1, 64
    st = synthetic.random_tree(N1, 10, 8, V, cgen)
    t = Tree.from_arrays(st.token_ids.tolist(), st.parents.tolist())
    tok, off, idx = flatten_tree(t, 0, limit=N1, restrict=False)
    ws1 = get_workspace(B1, N1, device)
    ws1.set_trees([(tok, off, idx, N1, 0)])
    ws1.uniforms.uniform_(generator=gen)
    # inputs cycled through a set larger than L2
    sets = [torch.randn(B1, N1, V, generator=gen, device=device) * 2.5 for _ in range(5)]
    for mode, name in ((1, "every_row"), (2, "walk")):
        it = iter(range(10 ** 9))
        ms1 = _time_ms(lambda: ws1.run(sets[next(it) % len(sets)], input_kind=_lib.IN_LOGITS,
                                       method=_lib.VERIFY_EXACT, do_sample=mode, temperature=1.0, top_p=0.9),
                       iters=10, warm=3)
        out["stochastic_verify_fp32_config1_" + name] = {"ms": ms1, "rows_sampled": N1 if mode == 1 else int(
            (ws1.fetch()["node_target"] >= 0).sum())}
    return out


def extra_gemm(device, peak_gbs, peak_tf):
    # config 4: HQQ W4A16 GEMM on the Qwen2.5-7B linear shapes; roofline time = max(bytes / HBM, flops / tensor)
    from subspec_b200 import quant
    from subspec_b200.synthetic import w4a16_case

    out = {}
    gen = torch.Generator(device=device).manual_seed(7)
    gemm = {}
    reps = 20
    for name, (n, k) in {"qo": (3584, 3584), "kv": (512, 3584), "gate_up": (18944, 3584),
                         "down": (3584, 18944)}.items():
        qweight, scale, zero, _ = w4a16_case(n, k, 1, seed=n + k)
        # a set of distinct weight copies larger than L2, cycled, so that every call streams from HBM
        copies = max(2, int(200e6 // (n * k * 0.5625)) + 1)
        packed = [quant.pack(qweight.cuda(), scale.cuda(), zero.cuda()) for _ in range(copies)]
        for m in (16, 64, 256):
            x = torch.randn(m, k, generator=gen, device=device).to(torch.bfloat16)
            state = {"i": 0}

            def call():
                quant.w4a16_matmul(x, packed[state["i"] % copies], n, k)
                state["i"] += 1

            call()
            torch.cuda.synchronize()
            graph_ok = True
            try:
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    for _ in range(reps):
                        call()
                _spin_up(device, 30.0)
                ms = _time_ms(gr.replay, iters=40, warm=10) / reps
            except Exception:
                graph_ok = False
                torch.cuda.synchronize()
                ms = _time_ms(call, iters=reps, warm=3)
            nbytes = n * k * 0.5625 + 2 * m * k + 2 * m * n
            flops = 2.0 * m * n * k
            t_roof = max(nbytes / (peak_gbs * 1e9), flops / (peak_tf * 1e12))
            gemm[f"{name}_m{m}"] = {"us": ms * 1e3, "roofline_us": t_roof * 1e6, "frac": t_roof / (ms * 1e-3),
                                    "TFLOP/s": flops / (ms * 1e-3) / 1e12, "GB/s": nbytes / (ms * 1e-3) / 1e9,
                                    "timed": "cuda graph of %d calls" % reps if graph_ok else "eager"}
        del packed
    out["w4a16_gemm_config4"] = gemm
    return out


def extra_lm_head(device, peak_gbs, peak_tf, peak_tf_sustained, wave=64, vocab=VOCAB):
    """The target's last projection and the verification of one wave ([wave * nodes, hidden] x [hidden, vocab] bf16,
    Qwen2.5-7B's 3584 x 152064): this repository's fused call (tcgen05 GEMM whose epilogue keeps the row statistics,
    no logits written) beside the library GEMM writing the logits followed by the streaming verify launch that
    reads them.  Each variant is timed twice: as a loop of back-to-back calls (the state a GPU is in behind a
    target forward: power-capped) and as single calls after a pause.  Not part of the default run (milliseconds
    per call).  `vocab` below the model's: a short case of the same kernels (weights still larger than L2) for a
    profiler capture."""
    from subspec_b200 import synthetic
    from subspec_b200.step import SpeculativeStepBatch

    hidden = 3584
    rows = wave * NODES
    gen = torch.Generator(device=device).manual_seed(5)
    h = (torch.randn(wave, NODES, hidden, generator=gen, device=device) * 0.5).to(torch.bfloat16)
    w = (torch.randn(vocab, hidden, generator=gen, device=device) * 0.02).to(torch.bfloat16)
    logits = torch.empty(wave, NODES, vocab, dtype=torch.bfloat16, device=device)
    trees, _ = synthetic.config5_wave(list(range(wave)), "literal", device, nodes=NODES, vocab=vocab, with_logits=False)
    sb = SpeculativeStepBatch(wave, NODES, device, kv_layers=1, kv_heads=KV_HEADS, head_dim=KV_DIM,
                              pages_per_seq=KV_TOKENS // PAGE_LEN, page_len=PAGE_LEN)
    sb.set_trees(flats_of(trees))
    _spin_up(device)
    flops = 2.0 * rows * hidden * vocab

    def single_ms(fn, n=5):  # one call at a time, the device idle for a moment before each
        fn()
        torch.cuda.synchronize(device)
        ts = []
        for _ in range(n):
            time.sleep(0.05)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize(device)
            ts.append(e0.elapsed_time(e1))
        return sorted(ts)[len(ts) // 2]

    out = {"flop_per_wave": flops, "vocab": vocab, "logits_bytes": rows * vocab * 2,
           "gemm_roofline_ms": {"burst_peak": flops / (peak_tf * 1e12) * 1e3,
                                "sustained_peak": flops / (peak_tf_sustained * 1e12) * 1e3}}
    gemm = lambda: torch.matmul(h.view(rows, hidden), w.t(), out=logits.view(rows, vocab))
    out["library_gemm_ms"] = {"loop": _time_ms(gemm, iters=5, warm=2), "single": single_ms(gemm)}
    for name, method, kw in (("greedy", "exact", None), ("lossy", "lossy", LOSSY_KW)):
        def pair():
            gemm()
            sb.verify(logits, verify_method=method, verify_kwargs=kw)
        fused = lambda: sb.verify_from_hidden(h, w, verify_method=method, verify_kwargs=kw)
        r = {"library_gemm_then_verify_ms": {"loop": _time_ms(pair, iters=5, warm=2), "single": single_ms(pair)},
             "fused_ms": {"loop": _time_ms(fused, iters=5, warm=2), "single": single_ms(fused)}}
        r["fused_TFLOP/s_single"] = flops / (r["fused_ms"]["single"] * 1e-3) / 1e12
        r["fused_frac_of_burst_peak"] = r["fused_TFLOP/s_single"] / peak_tf
        out[name] = r
    # End to end from the host for the fused call: the wave's hidden states from pinned memory (29 MB instead of
    # 1.25 GB of logits), the call, the results back to pinned memory.
    host_h = h.cpu().pin_memory()
    dev_h = torch.empty_like(h)

    def e2e_step():
        dev_h.copy_(host_h, non_blocking=True)
        sb.verify_from_hidden(dev_h, w, verify_method="exact+lossy", verify_kwargs=LOSSY_KW)
        sb.results()

    for _ in range(2):
        e2e_step()
    torch.cuda.synchronize(device)
    t0 = time.perf_counter()
    for _ in range(5):
        e2e_step()
    torch.cuda.synchronize(device)
    ms = (time.perf_counter() - t0) / 5 * 1e3
    out["e2e_from_hidden_states"] = {"ms_per_wave": ms, "sequence_steps_per_s": wave / (ms * 1e-3),
                                     "h2d_bytes_per_step": host_h.numel() * 2, "method": "exact+lossy",
                                     "note": "includes the lm_head GEMM, which the logits-in end-to-end number does not"}
    return {"lm_head_verify_wave64": out}


def run_extras_only(args):
    from subspec_b200 import build as _build

    _build.build()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    pk = ROOT / "MEASURED_PEAKS.json"
    peaks = json.loads(pk.read_text()) if pk.exists() else {}
    peak_gbs, peak_tf = float(peaks.get("hbm_gbs", 6650.0)), float(peaks.get("bf16_tflops", 1590.0))
    if args.extras_only == "step":
        out = extra_step_peaked(device, peak_gbs)
    elif args.extras_only == "expand":
        out = extra_expand(device, peak_gbs)
    elif args.extras_only == "attention":
        out = extra_attention(device, peak_gbs, peak_tf)
    elif args.extras_only == "stochastic":
        out = extra_stochastic(device, peak_gbs)
    elif args.extras_only in ("lmhead", "lmhead-small"):
        out = extra_lm_head(device, peak_gbs, peak_tf, float(peaks.get("bf16_tflops_sustained", peak_tf)),
                            vocab=VOCAB if args.extras_only == "lmhead" else 32768)
    else:
        out = extra_gemm(device, peak_gbs, peak_tf)
    print(json.dumps(out), flush=True)


# --------------------------------------------------------------------------------------
# native arm
# --------------------------------------------------------------------------------------
def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.extras_only:
        run_extras_only(args)
        return

    import torch.distributed as dist

    from subspec_b200 import build as _build
    from subspec_b200 import synthetic
    from subspec_b200.step import SpeculativeStepBatch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    from subspec_b200.shard import device_for_rank

    local_world = int(os.environ.get("LOCAL_WORLD_SIZE", str(world)))
    dev_index = device_for_rank(local, local_world, torch.cuda.device_count())
    torch.cuda.set_device(dev_index)
    device = torch.device("cuda", dev_index)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    if rank == 0:
        _build.build()
    if world > 1:
        dist.barrier()

    total = args.seqs
    from subspec_b200.shard import reduce_stats, shard_sequences

    shard = shard_sequences(total, world, rank, args.wave)
    per_rank, wave, n_waves, total = shard.count, shard.wave, shard.n_waves, shard.total
    pages_per_seq = args.kv_tokens // PAGE_LEN
    kv_bytes_seq = KV_LAYERS * pages_per_seq * 2 * PAGE_LEN * KV_HEADS * KV_DIM * 2
    need = per_rank * (NODES * VOCAB * 2 + kv_bytes_seq) + (6 << 30)
    free, _ = torch.cuda.mem_get_info(device)
    if need > free:
        raise SystemExit(f"rank {rank}: needs {need / 2**30:.1f} GiB, {free / 2**30:.1f} GiB free; "
                         f"use --kv-tokens to shrink the per-sequence cache")

    # ---- build the waves ----
    waves = []
    for w in range(n_waves):
        ids = shard.wave_ids(w)
        trees, logits = make_wave_inputs(ids, args.variant, device)
        pgen = torch.Generator().manual_seed(31 + ids[0])
        sb = SpeculativeStepBatch(wave, NODES, device, kv_layers=KV_LAYERS, kv_heads=KV_HEADS, head_dim=KV_DIM,
                                  page_len=PAGE_LEN, pages_per_seq=pages_per_seq,
                                  page_table=synthetic.random_page_table(wave, pages_per_seq, pgen))
        for layer in range(KV_LAYERS):
            sb.pool[layer].normal_()
        sb.set_trees(flats_of(trees))
        sb.set_kv_offsets([args.kv_tokens - NODES] * wave)
        waves.append((sb, logits, trees, ids))
    torch.cuda.synchronize()

    def one_step(events=None):
        last = None  # the event behind the previous wave's compaction is the one in front of this wave's verify
        for sb, logits, _, _ in waves:
            if events is not None:
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
                if last is None:
                    ev[0].record()
                else:
                    ev[0] = last
            if args.two_pass:
                sb.verify(logits, verify_method="exact")
                if events is not None:
                    ev[1].record()
            elif events is not None:
                ev[1] = ev[0]  # no separate greedy launch: nothing to bracket, one command fewer in the stream
            # greedy and lossy results of the step; by default from one launch = one pass over the logits
            sb.verify(logits, verify_method="lossy" if args.two_pass else "exact+lossy", verify_kwargs=LOSSY_KW)
            if events is not None:
                ev[2].record()
            sb.compact_kv()
            if events is not None:
                ev[3].record()
                events.append(ev)
                last = ev[3]

    def barrier():
        if world > 1:
            dist.barrier()

    # ---- device-resident timing ----
    for _ in range(args.warmup):
        one_step()
    torch.cuda.synchronize()
    barrier()
    kernel_events = []
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(dev_index) as clocks:
        torch.cuda.synchronize()
        t_start.record()
        for _ in range(args.steps):
            one_step(kernel_events)
        t_end.record()
        clocks.sample_now()  # the launches above are still executing: a short region gets its sample under load
        torch.cuda.synchronize()
    barrier()
    ms_total = t_start.elapsed_time(t_end)
    ms_exact = sum(e[0].elapsed_time(e[1]) for e in kernel_events) / len(kernel_events)
    ms_lossy = sum(e[1].elapsed_time(e[2]) for e in kernel_events) / len(kernel_events)
    ms_kv = sum(e[2].elapsed_time(e[3]) for e in kernel_events) / len(kernel_events)

    # ---- results of the last step: acceptance statistics + parity spot check ----
    accepted_tokens, kept_rows, moved_rows = 0, 0, 0
    outs = []
    for sb, _, _, _ in waves:
        out = sb.results()
        outs.append(out)
        accepted_tokens += int(out["out_meta"][:, 0].sum())
        kept_rows += int(out["out_meta"][:, 0].sum())
        moved_rows += moved_row_count(out)
    # a few sequences of the first wave, kept on the host for the CPU-baseline leg, which checks the GPU
    # results against the CPU restatement (the only place this script runs it)
    spot = []
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sb, logits, trees, ids = waves[0]
        for b in range(min(4, wave)):
            L = int(outs[0]["out_meta"][b, 0])
            spot.append((ids[b], logits[b].cpu(), trees[b], outs[0]["out_tokens"][b, :L].tolist(),
                         outs[0]["out_hidden"][b, :L].tolist()))

    # ---- end-to-end: logits start in pinned host memory, results end in host memory ----
    e2e = None
    if not args.no_e2e:
        e2e_steps = max(2, min(args.steps, 5))
        host_logits = torch.empty(wave, NODES, VOCAB, dtype=torch.bfloat16).pin_memory()
        host_logits.copy_(waves[0][1])
        stage = [torch.empty_like(waves[0][1]) for _ in range(2)]
        copy_stream, comp_stream = torch.cuda.Stream(device), torch.cuda.Stream(device)
        ready = [torch.cuda.Event() for _ in range(2)]
        freed = [torch.cuda.Event() for _ in range(2)]

        wave_flats = [flats_of(trees) for _, _, trees, _ in waves]
        tree_bytes = sum(sb.ws._in_host.numel() * 4 for sb, _, _, _ in waves)

        def e2e_step():
            for i, (sb, _, _, _) in enumerate(waves):
                s = i % 2
                with torch.cuda.stream(copy_stream):
                    copy_stream.wait_event(freed[s])
                    stage[s].copy_(host_logits, non_blocking=True)
                    ready[s].record(copy_stream)
                with torch.cuda.stream(comp_stream):
                    # the step's trees: checked, packed into the pinned block and copied (runs on the host while
                    # the logits copy above is in flight)
                    sb.set_trees(wave_flats[i])
                    comp_stream.wait_event(ready[s])
                    if args.two_pass:
                        sb.verify(stage[s], verify_method="exact")
                    sb.verify(stage[s], verify_method="lossy" if args.two_pass else "exact+lossy",
                              verify_kwargs=LOSSY_KW)
                    sb.compact_kv()
                    freed[s].record(comp_stream)
                    sb.ws._out_host.copy_(sb.ws._out_dev, non_blocking=True)
            comp_stream.synchronize()

        for _ in range(2):
            e2e_step()
        torch.cuda.synchronize()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        torch.cuda.synchronize()
        dt_e2e = time.perf_counter() - t0
        barrier()
        e2e = {"dt": dt_e2e, "steps": e2e_steps,
               "h2d": n_waves * host_logits.numel() * 2 + tree_bytes,
               "d2h": n_waves * waves[0][0].ws._out_host.numel()}

    # ---- gather (max over ranks of the times; sums of the counts) ----
    red = reduce_stats({"ms_total": ms_total, "ms_exact": ms_exact, "ms_lossy": ms_lossy, "ms_kv": ms_kv,
                        "dt_e2e": e2e["dt"] if e2e else 0.0},
                       {"accepted_tokens": accepted_tokens, "kept_rows": kept_rows, "moved_rows": moved_rows},
                       device=device)
    ms_total, ms_exact, ms_lossy, ms_kv, dt_e2e = (red[k] for k in ("ms_total", "ms_exact", "ms_lossy", "ms_kv",
                                                                     "dt_e2e"))
    accepted_tokens, kept_rows, moved_rows = red["accepted_tokens"], red["kept_rows"], red["moved_rows"]

    if rank == 0:
        peaks = {}
        pk = ROOT / "MEASURED_PEAKS.json"
        if pk.exists():
            peaks = json.loads(pk.read_text())
        peak_gbs = float(peaks.get("hbm_gbs", 6650.0))
        peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)" if peaks else "fallback 6650 GB/s"
        rows_bytes = wave * NODES * VOCAB * 2  # algorithmic bytes of one verify launch
        achieved = rows_bytes / (ms_lossy * 1e-3) / 1e9
        secs = ms_total * 1e-3
        line = {
            "metric": METRIC, "value": total * args.steps / secs, "unit": "steps/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_total / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args, total, world, per_rank),
            "accepted_tok_per_s": accepted_tokens * args.steps / secs,
            "mean_tokens_per_step": accepted_tokens / total,
            "kernels_ms": ({"verify_exact": ms_exact, "verify_lossy": ms_lossy, "kv_compact": ms_kv,
                            "per": f"launch over a wave of {wave} sequences"} if args.two_pass else
                           {"verify_exact_and_lossy": ms_lossy, "kv_compact": ms_kv,
                            "per": f"launch over a wave of {wave} sequences"}),
            "roofline": {"bound": "hbm",
                         "kernel": "verify_rows_kernel<bf16, logits, softmax+entropy>" +
                                   (" (lossy verify)" if args.two_pass else " (greedy + lossy verify, one pass)"),
                         "achieved": achieved, "peak": peak_gbs, "unit": "GB/s", "frac": achieved / peak_gbs,
                         "peak_source": peak_src,
                         "traffic": profiled_traffic(wave), "algorithmic_bytes": rows_bytes,
                         "exact_kernel_gbs": rows_bytes / (ms_exact * 1e-3) / 1e9 if args.two_pass else None},
            # the compaction launch of this workload: rows that really move (beam[i] != i), read + written
            "kv_compact": {"us_per_launch": ms_kv * 1e3, "rows_kept_per_launch": kept_rows / (world * n_waves),
                           "rows_moved_per_launch": moved_rows / (world * n_waves),
                           "GB/s": 2 * (moved_rows / (world * n_waves)) * waves[0][0].kv_row_bytes
                           / (ms_kv * 1e-3) / 1e9},
            "gpu_launches": args.steps * n_waves * (3 if args.two_pass else 2),
            "clocks": clocks.summary(),
        }
        if e2e:
            line["e2e"] = {"value": total * e2e["steps"] / dt_e2e, "unit": "steps/s",
                           "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                           "steps": e2e["steps"],
                           "h2d_GBps_per_rank": e2e["h2d"] * e2e["steps"] / dt_e2e / 1e9,
                           "gpus_used": [device_for_rank(r, local_world, torch.cuda.device_count())
                                         for r in range(local_world)],
                           "note": "bytes are per GPU and step; per wave the logits are copied from pinned host "
                                   "memory (double-buffered), the trees are checked, packed and copied, and the "
                                   "results are read back to pinned host memory"}
        if world == 1 and not args.no_extras:
            for w in waves:
                w[0].pool = None
            del waves[:]
            torch.cuda.empty_cache()
            line["other_kernels"] = extras(device, peak_gbs, float(peaks.get("bf16_tflops", 1590.0)),
                                           float(peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops", 1590.0))))
        if world == 1 and not args.no_cpu_baseline:
            v, desc = cpu_baseline(args.cpu_sample, 5, args.variant)
            line["cpu_baseline"] = {"value": v, "unit": "steps/s", "cores": os.cpu_count(), "kind": "port",
                                    "sample": desc, "gpu_results_checked_sequences": spot_check(spot)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
