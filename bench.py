#!/usr/bin/env python
"""Benchmark of the KV append + split-KV decode attention path on B200.

Workload (BASELINE.json configs[2], the batched paged decode the metric's roofline target is quoted
on): 64 sequences, context lengths uniform in [512, 32768] from a seed, 16-token pages in one pool
with a randomly permuted block table, 16 Q / 8 KV heads, head_dim 256, bf16. One step = one decode
step through one period of the 5:1 layer pattern: five sliding-window layers (ring of 1024 live
keys) and one global layer (linear cache), each layer-step being fused append + split-KV decode +
combine. Sequences are sharded over ranks (greedy longest-first on context length); no collective is
on the data path.

    python bench.py --gpus N --steps K --warmup W            # this library (CUDA, through the C-ABI)
    python bench.py --impl reference --gpus N ...            # the reference's own CUDA kernels (oracle/_ref) on one GPU

Prints one JSON line (rank 0). The default line also carries: `verified` (the last timed step's outputs checked
against the oracle, outside the timed region; a miss makes the run exit 3), `other_workloads` (short runs of the
other BASELINE configs in the same process), `reference_cuda`, `cpu_baseline` (all cores) and `cpu_baseline_1t`.
"""
from __future__ import annotations

import argparse
import copy
import ctypes
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))

HQ, HKV, D, PAGE, WINDOW = 16, 8, 256, 16, 1024
E_KV = 2  # bytes per cached element (bf16)
METRIC = "KV append + decode attention: achieved HBM GB/s (us per layer-step alongside)"


def parse_args(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--seqs", type=int, default=0, help="sequences in the batch (cfg3: 64, cfg5: 32)")
    ap.add_argument("--min-ctx", type=int, default=512)
    ap.add_argument("--max-ctx", type=int, default=32768)
    ap.add_argument("--seed", type=int, default=20260)
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--cpu-seconds", type=float, default=10.0, help="target CPU time of the cpu_baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-cuda", action="store_true",
                    help="skip timing the reference's own CUDA kernels (oracle/_ref) beside the library")
    ap.add_argument("--split-global", type=int, default=0, help="override the planned global split size")
    ap.add_argument("--split-local", type=int, default=0)
    ap.add_argument("--workload", default="cfg3", choices=["cfg1", "cfg2", "cfg3", "cfg4", "cfg5", "native_global", "prefill", "layer"],
                    help="BASELINE.json configs (1-based): cfg3 (default) is the batched paged decode the "
                         "metric is quoted on; the others are reported as extra lines on request")
    ap.add_argument("--partition", default="balanced", choices=["balanced", "splits"],
                    help="balanced: keys of the batch divided evenly over a fixed grid (split_size 0); "
                         "splits: fixed-size splits as the reference defines them")
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"],
                    help="replay each step from a CUDA graph captured once (auto: on for the batch-1 latency "
                         "workloads cfg1/cfg2, where the host cannot issue 3 launches per layer fast enough)")
    ap.add_argument("--layers", type=int, default=48, help="--workload layer: layers in the stack")
    ap.add_argument("--shard", default="heads", choices=["heads", "keys"],
                    help="cfg4 on more than one GPU: every rank holds all KV heads of a contiguous range of the keys "
                         "and the ranks' rows are merged by log-sum-exp (keys), or every rank holds some KV heads "
                         "of all keys and the rows are all-gathered (heads)")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"],
                    help="cfg4 on more than one GPU: all-gather of the head outputs by the library's peer-memory "
                         "kernel (b200kv_peer_allgather) or by ncclAllGather")
    ap.add_argument("--emulate-world", type=int, default=0,
                    help="tuning aid: on one GPU, run the shard that rank --emulate-rank of this many ranks would own")
    ap.add_argument("--emulate-rank", type=int, default=0)
    ap.add_argument("--cache", default="warm", choices=["warm", "cold", "both"],
                    help="cold / both: after the timed steps, time more steps one by one with an L2 flush (a write "
                         "over 512 MiB) before each and the events recorded after the flush; reported as `cold_cache`")
    ap.add_argument("--no-tickets", action="store_true",
                    help="do not hand the layer-step its tickets: small jobs then run as fused attention + combine "
                         "(two launches) instead of the one-launch form")
    ap.add_argument("--no-verify", action="store_true",
                    help="skip the oracle check of the last timed step's outputs (`verified`)")
    ap.add_argument("--no-other-workloads", action="store_true",
                    help="default workload only: do not add the short runs of the other BASELINE configs")
    ap.add_argument("--other-steps", type=int, default=100, help="timed steps of each of those short runs")
    return ap.parse_args(argv)


# --------------------------------------------------------------------------- workload description
def context_lengths(args) -> np.ndarray:
    rng = np.random.default_rng(args.seed)
    return rng.integers(args.min_ctx, args.max_ctx + 1, size=args.seqs or 64).astype(np.int64)


def shard_sequences(ctx: np.ndarray, world: int) -> list[list[int]]:
    """Greedy longest-first partition of sequences over ranks (gemma.c_b200/sharding.py)."""
    from __graft_entry__ import load_package

    load_package()
    from gemma_c_b200 import sharding

    return sharding.shard_sequences(ctx, world)


def layer_step_bytes(seq_len_after_append: np.ndarray, window: int, hkv: int = HKV, e_kv: int = E_KV) -> int:
    """Algorithmic HBM bytes of one layer-step (append + decode attention) for the given sequences."""
    s = np.asarray(seq_len_after_append, dtype=np.int64)
    hq = 2 * hkv
    live = np.minimum(s, window) if window > 0 else s
    first = s - live
    pages_touched = (s - 1) // PAGE - first // PAGE + 1
    scales = 4 * pages_touched * hkv * 2 if e_kv == 1 else 0
    attn = live * hkv * D * 2 * e_kv + hq * D * 2 + hq * D * 2 + 4 * pages_touched + scales
    append = (hq + 2 * hkv) * D * 2 + hq * D * 2 + 2 * hkv * D * e_kv + 4
    return int((attn + append).sum())


def attention_kernel_bytes(seq_len_after_append: np.ndarray, window: int, hkv: int = HKV, e_kv: int = E_KV) -> int:
    """Algorithmic bytes of the split-KV attention launch alone (K/V stream, q, output, page table)."""
    s = np.asarray(seq_len_after_append, dtype=np.int64)
    hq = 2 * hkv
    live = np.minimum(s, window) if window > 0 else s
    first = s - live
    pages_touched = (s - 1) // PAGE - first // PAGE + 1
    scales = 4 * pages_touched * hkv * 2 if e_kv == 1 else 0
    return int((live * hkv * D * 2 * e_kv + hq * D * 2 + hq * D * 2 + 4 * pages_touched + scales).sum())


def hbm_peak():
    """The measured copy bandwidth of this pool's B200s (driver-written), else the stated fallback."""
    peaks_path = REPO / "MEASURED_PEAKS.json"
    if peaks_path.exists():
        return float(json.loads(peaks_path.read_text())["hbm_gbs"]), "MEASURED_PEAKS.json hbm_gbs"
    return 6650.0, "fallback 6.65 TB/s (MEASURED_PEAKS.json absent)"


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = tempfile.NamedTemporaryFile(prefix="clocks_", suffix=".csv", delete=False).name
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu=timestamp,{self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20", "-i", str(gpu_index)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        self.marks: dict[str, float] = {}

    def mark(self, name: str):
        self.marks[name] = time.time()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        import datetime as dt

        rows = []
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                ts = dt.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(parts[1]), float(parts[2]), float(parts[3]), parts[4:]))
            except ValueError:
                continue
        os.unlink(self.path)
        t0, t1 = self.marks.get("timed_begin", 0.0), self.marks.get("timed_end", float("inf"))
        inside = [r for r in rows if t0 <= r[0] <= t1]
        window = "timed region"
        if len(inside) < 3:   # region shorter than the sampling period: use everything sampled under load
            lo, hi = self.marks.get("load_begin", 0.0), self.marks.get("load_end", float("inf"))
            inside = [r for r in rows if lo <= r[0] <= hi]
            window = "warm-up + timed + e2e (timed region shorter than the sampling period)"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"], "samples": 0}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[4][1 + i].lower().startswith("active") for r in inside)]
        return {"sm_mhz": statistics.median(r[1] for r in inside), "sm_max_mhz": inside[0][2],
                "power_w_max": max(r[3] for r in inside), "reasons": reasons, "samples": len(inside),
                "window": window}


# --------------------------------------------------------------------------- device workload
class Spec:
    """Which layers one step runs and on what geometry."""

    def __init__(self, name, text, n_local, n_global, hkv=8, fp8=False, tight_ring=False, outliers=False,
                 gather=False, key_shard=None):
        self.name, self.text = name, text
        self.key_shard = key_shard                  # (rank, ranks): this rank holds one range of the keys
        self.n_local, self.n_global = n_local, n_global
        self.hkv, self.hq = hkv, 2 * hkv           # KV / query heads held by this rank
        self.fp8, self.tight_ring, self.outliers, self.gather = fp8, tight_ring, outliers, gather
        self.e_kv = 1 if fp8 else 2


class RankWorkload:
    """Everything one rank holds in HBM for its share of the workload."""

    def __init__(self, kv, torch, ctx: np.ndarray, total_steps: int, seed: int, args, spec: Spec):
        self.kv, self.torch, self.spec = kv, torch, spec
        dev = "cuda"
        self.B = B = int(ctx.size)
        self.ctx = ctx
        self.total_steps = total_steps
        HKV, HQ = spec.hkv, spec.hq
        nl, ng = spec.n_local, spec.n_global
        sm = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed)
        rng = np.random.default_rng(seed)

        def normal_bf16(n):
            t = torch.empty(n, dtype=torch.bfloat16, device=dev)
            t.normal_(generator=gen)
            return t

        max_pos = int(ctx.max()) + total_steps + 1
        # Key-range sharding: a rank's keys sit at local positions 0 .. C-1 of its own cache; the new token has
        # local position C + s on every rank and absolute position shift + C + s, so the RoPE tables are
        # entered `shift` rows further down. Only the last rank has pages for the new rows: on the others the
        # position is unmapped, nothing is appended, and q is still prepared at the absolute position.
        self.rope_shift, self.owns_new_rows = 0, True
        if spec.key_shard:
            me, shards = spec.key_shard
            self.rope_shift = (shards - 1) * int(ctx[0])
            self.owns_new_rows = me == shards - 1
            max_pos += self.rope_shift
        self.g_cfg = self.l_cfg = None
        if ng:
            # global layers: linear cache, one pool, permuted block table
            pages_b = (ctx + total_steps + PAGE) // PAGE
            self.g_pages = int(pages_b.sum())
            self.g_mpps = int(pages_b.max())
            table = np.full((B, self.g_mpps), -1, dtype=np.int32)
            pool = rng.permutation(self.g_pages).astype(np.int32)
            cur = 0
            for b in range(B):
                table[b, :pages_b[b]] = pool[cur:cur + pages_b[b]]
                cur += int(pages_b[b])
            self.g_cfg = kv.make_kv_config(ng, self.g_pages, PAGE, self.g_mpps, B, HKV, D, 0)
            if not self.owns_new_rows:
                table[:, (int(ctx[0]) + PAGE - 1) // PAGE:] = -1
            self.g_table = torch.from_numpy(table).to(dev)
            gc, gs = kv.fill_rope_tables(max_pos, D // 2, 1000000.0, D)
            self.g_cos, self.g_sin = torch.from_numpy(gc).to(dev), torch.from_numpy(gs).to(dev)
            if spec.fp8:
                n = self.g_cfg.cache_elements()
                self.g_k = torch.empty(n, dtype=torch.uint8, device=dev)
                self.g_v = torch.empty(n, dtype=torch.uint8, device=dev)
                self.g_sk = torch.zeros(ng * self.g_pages * HKV, dtype=torch.float32, device=dev)
                self.g_sv = torch.zeros_like(self.g_sk)
                self._fill_fp8(normal_bf16)
            else:
                self.g_k = normal_bf16(self.g_cfg.cache_elements())
                self.g_v = normal_bf16(self.g_cfg.cache_elements())
                if spec.outliers:      # 1 % of the keys scaled x8 (attention-sink-like rows)
                    rows = self.g_k.view(-1, D)
                    pick = torch.rand(rows.shape[0], device=dev, generator=gen) < 0.01
                    rows[pick] *= 8.0
        if nl:
            # local layers: ring of the window plus one page of slack (or exactly the window)
            self.l_mpps = WINDOW // PAGE if spec.tight_ring else (WINDOW + PAGE - 1 + PAGE - 1) // PAGE
            self.l_pages = B * self.l_mpps
            ltable = rng.permutation(self.l_pages).astype(np.int32).reshape(B, self.l_mpps)
            self.l_cfg = kv.make_kv_config(nl, self.l_pages, PAGE, self.l_mpps, B, HKV, D, WINDOW)
            self.l_table = torch.from_numpy(ltable).to(dev)
            self.l_k = normal_bf16(self.l_cfg.cache_elements())
            self.l_v = normal_bf16(self.l_cfg.cache_elements())
            lc, ls = kv.fill_rope_tables(max_pos, D // 2, 10000.0, D)
            self.l_cos, self.l_sin = torch.from_numpy(lc).to(dev), torch.from_numpy(ls).to(dev)
        w = torch.empty(2, D, dtype=torch.float32, device=dev).normal_(1.0, 0.05, generator=gen)
        self.q_w, self.k_w = w[0].to(torch.bfloat16).contiguous(), w[1].to(torch.bfloat16).contiguous()

        # this step's projections for every layer: [layers, B, (HQ + 2 HKV) * D]
        L = nl + ng
        self.L = L
        self.row = (HQ + 2 * HKV) * D
        self.raw = normal_bf16(L * B * self.row).view(L, B, self.row)
        self.raw_host = torch.empty((L, B, self.row), dtype=torch.bfloat16).pin_memory()
        self.raw_host.copy_(self.raw)
        self.raw_q = torch.empty((L, B, HQ * D), dtype=torch.bfloat16, device=dev)
        self.raw_k = torch.empty((L, B, HKV * D), dtype=torch.bfloat16, device=dev)
        self.raw_v = torch.empty((L, B, HKV * D), dtype=torch.bfloat16, device=dev)
        self._unpack_raw()
        self.q_prepared = torch.empty((L, B, HQ, D), dtype=torch.bfloat16, device=dev)
        self.out = torch.empty((L, B, HQ, D), dtype=torch.bfloat16, device=dev)
        self.out_host = torch.empty((L, B, HQ, D), dtype=torch.bfloat16).pin_memory()
        self.lse = torch.empty((L, B, HQ), dtype=torch.float32, device=dev)
        self.status = torch.zeros(4, dtype=torch.int32, device=dev)
        self.world = int(os.environ.get("WORLD_SIZE", "1")) if spec.gather else 1
        self.peer = None
        if spec.gather and self.world > 1:
            import torch.distributed as dist

            self.out_all = torch.empty((self.world, L, B, HQ, D), dtype=torch.bfloat16, device=dev)
            self.gather_checked = True          # nothing to check against on the nccl arm
            if args.gather == "peer":
                self.out_bytes = self.out.numel() * 2
                slot = self.out_bytes               # the gathered view is then exactly [world][rows][D]
                if spec.key_shard:
                    slot = (self.out_bytes + self.lse.numel() * 4 + 15) // 16 * 16
                self.peer = kv.PeerBuffer(slot, self.world, int(os.environ.get("RANK", "0")))
                mine = torch.tensor(list(self.peer.export), dtype=torch.uint8, device=dev)
                everyone = torch.empty(self.world * 64, dtype=torch.uint8, device=dev)
                dist.all_gather_into_tensor(everyone, mine)
                self.peer.connect(bytes(everyone.cpu().tolist()))
                dist.barrier()
                self.gather_checked = False

        # per-step metadata, resident: position of the appended token and length after the append
        steps = np.arange(total_steps, dtype=np.int64)[:, None]
        self.pos_all = torch.from_numpy((ctx[None, :] + steps).astype(np.int32)).to(dev)
        lengths = ctx[None, :] + steps + 1 if self.owns_new_rows else ctx[None, :] + 0 * steps
        self.len_all = torch.from_numpy(lengths.astype(np.int32)).to(dev)

        balanced_ok = HKV == 8 and B <= 1024
        self.g_split, self.g_nsplit = kv.plan_splits_total(B, int(ctx.max()) + total_steps,
                                                           int(ctx.sum()) + B * total_steps, HKV, sm)
        self.l_split, self.l_nsplit = kv.plan_splits_total(B, WINDOW, B * WINDOW, HKV, sm)
        tiled_ok = not args.no_tickets and not spec.fp8 and B == 1   # the one-launch form takes any number of KV heads
        if (args.partition == "balanced" and (balanced_ok or tiled_ok)) or spec.fp8:
            self.g_split = self.l_split = 0
            self.g_nsplit = self.l_nsplit = kv.plan_balanced(B, sm)
        if args.split_global:
            self.g_split = args.split_global
            self.g_nsplit = -(-(int(ctx.max()) + total_steps) // self.g_split)
        if args.split_local:
            self.l_split = args.split_local
            self.l_nsplit = -(-WINDOW // self.l_split)
        nmax = max(self.g_nsplit if ng else 1, self.l_nsplit if nl else 1)
        rows = B * HQ * nmax
        self.pm = torch.empty(rows, dtype=torch.float32, device=dev)
        self.pl = torch.empty(rows, dtype=torch.float32, device=dev)
        self.pacc = torch.empty(rows * D, dtype=torch.float32, device=dev)

        # tickets of the one-launch layer-step (zero before the first call, left zero by every call)
        self.ticket = torch.zeros(B * HKV * kv.TICKETS_PER_HEAD, dtype=torch.int32, device=dev)
        self.layers = (kv.LayerStepArgs * L)()
        self.ev_begin = [kv.Timer() for _ in range(total_steps)]
        self.ev_end = [kv.Timer() for _ in range(total_steps)]
        for i in range(L):
            a = self.layers[i]
            # the reference's cadence: five sliding layers, then one global (src/gemma4.h:105-108)
            is_global = self.layer_is_global(i)
            li = self.cache_layer_of(i)
            a.q, a.out, a.lse = self.q_prepared[i].data_ptr(), self.out[i].data_ptr(), self.lse[i].data_ptr()
            a.partial_m, a.partial_l, a.partial_acc = self.pm.data_ptr(), self.pl.data_ptr(), self.pacc.data_ptr()
            a.cache_k = (self.g_k if is_global else self.l_k).data_ptr()
            a.cache_v = (self.g_v if is_global else self.l_v).data_ptr()
            a.cache_config = self.g_cfg if is_global else self.l_cfg
            a.page_table = (self.g_table if is_global else self.l_table).data_ptr()
            a.cache_layer = li
            a.split_size = self.g_split if is_global else self.l_split
            a.num_splits = self.g_nsplit if is_global else self.l_nsplit
            a.softmax_scale = 1.0 / math.sqrt(D)
            a.raw_q, a.raw_k, a.raw_v = self.raw_q[i].data_ptr(), self.raw_k[i].data_ptr(), self.raw_v[i].data_ptr()
            a.q_norm_weight, a.k_norm_weight = self.q_w.data_ptr(), self.k_w.data_ptr()
            rope_offset = self.rope_shift * (D // 2) * 4 if is_global else 0
            a.cos = (self.g_cos if is_global else self.l_cos).data_ptr() + rope_offset
            a.sin = (self.g_sin if is_global else self.l_sin).data_ptr() + rope_offset
            a.batch_count, a.q_heads, a.rotary_dim, a.norm_mode = B, HQ, D, kv.NORM_RSQRT_APPROX
            a.status = self.status.data_ptr()
            a.ticket = None if args.no_tickets else self.ticket.data_ptr()
            # KV-head sharding with the library's exchange: the step itself ends with the all-gather
            # (inside the one-launch kernel where the step runs as that, a gather kernel behind it otherwise)
            a.peer_gather = self.peer.handle if (self.peer is not None and not spec.key_shard) else None
        self.timed_layer = max((i for i in range(L) if self.layer_is_global(i)), default=L - 1)
        self.stream = torch.cuda.current_stream().cuda_stream
        self.launches_per_step = 0
        self.kernels_per_layer = []
        for i in range(L):
            if spec.fp8:
                n = 3                                   # fp8 append, balanced attention, combine
            else:
                n = kv.layer_step_launches(self.layers[i])
            self.kernels_per_layer.append(n)
            self.launches_per_step += n
        if self.peer is not None and spec.key_shard:
            self.launches_per_step += 1              # the peer-memory merge kernel (key-range sharding)

    def layer_is_global(self, i: int) -> bool:
        nl, ng = self.spec.n_local, self.spec.n_global
        if ng == 0:
            return False
        if nl == 0:
            return True
        period = (nl + ng) // ng
        return (i + 1) % period == 0

    def cache_layer_of(self, i: int) -> int:
        g = self.layer_is_global(i)
        return sum(1 for j in range(i) if self.layer_is_global(j) == g)

    def _fill_fp8(self, normal_bf16):
        """Fill the fp8 global cache the way a prompt would: bf16 N(0,1) rows through the bulk
        quantise-on-append entry point, sequence by sequence."""
        kv, torch, spec = self.kv, self.torch, self.spec
        HKV = spec.hkv
        for layer in range(spec.n_global):
            for b in range(self.B):
                n = int(self.ctx[b])
                rows_k, rows_v = normal_bf16(n * HKV * D), normal_bf16(n * HKV * D)
                one = lambda x: torch.tensor([x], dtype=torch.int32, device="cuda")
                kv.fp8_append_rows(self.g_k, self.g_v, self.g_sk, self.g_sv, self.g_cfg, self.g_table, one(b), one(0),
                                   one(n), one(0), 1, n, layer, rows_k, rows_v)
        torch.cuda.synchronize()

    def _unpack_raw(self):
        hq, hkv = self.spec.hq, self.spec.hkv
        q, k, v = self.raw.split([hq * D, hkv * D, hkv * D], dim=2)
        self.raw_q.copy_(q)
        self.raw_k.copy_(k)
        self.raw_v.copy_(v)

    def enable_graph(self, first_step: int, steps_per_graph: int = 1):
        """Capture `steps_per_graph` consecutive steps into one CUDA graph. The captured launches read their
        step's positions and lengths from fixed buffers that the graph itself advances at its end, so replaying
        it walks through consecutive decode steps. A one-layer workload puts several steps into a graph: one step
        would be a single kernel, and a replay's fixed cost (the launch of the graph, the kernel that advances the
        buffers) would be what is measured. The per-layer timing hooks are not captured."""
        torch = self.torch
        k = self.steps_per_graph = steps_per_graph
        # positions and lengths of the replayed steps live in one buffer so that one small kernel advances both
        self.step_state = torch.stack([self.pos_all[first_step:first_step + k],
                                       self.len_all[first_step:first_step + k]]).contiguous()      # [2, k, B]
        self.graph_first = self.graph_next = first_step

        def launch_all(stream):
            if self.L == 1 and k > 1 and not self.spec.fp8:
                # the k steps of the one layer as ONE b200kv_decode_step_bf16 call: the library then knows that
                # they are consecutive steps of one cache layer and keeps their launches overlapped
                steps = (type(self.layers[0]) * k)()
                for j in range(k):
                    steps[j] = self.layers[0]
                    steps[j].token_position = self.step_state[0, j].data_ptr()
                    steps[j].seq_lengths = self.step_state[1, j].data_ptr()
                    steps[j].event_before_attention = None
                    steps[j].event_after_attention = None
                self.graph_entries = steps
                self.kv.decode_step(steps, k, stream=stream)
                return
            for j in range(k):
                self._launch_step(self.step_state[0, j].data_ptr(), self.step_state[1, j].data_ptr(), None, stream)

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):      # warm-up outside capture (first-use attribute calls)
            launch_all(side.cuda_stream)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            launch_all(torch.cuda.current_stream().cuda_stream)
            self.step_state.add_(k)
        torch.cuda.synchronize()

    def step(self, s: int, events: bool = False):
        """One decode step, inputs resident in HBM. `events` brackets the timed layer's attention with
        device timers; an event between the append and the attention keeps the attention from starting
        under the append's tail, so the timed steps run without them."""
        if getattr(self, "graph", None) is not None:
            assert s == self.graph_next, "graph replay walks consecutive steps"
            if (s - self.graph_first) % self.steps_per_graph == 0:
                self.graph.replay()           # this and the next steps_per_graph - 1 steps
            self.graph_next += 1
            self._exchange()
            return
        self._launch_step(self.pos_all[s].data_ptr(), self.len_all[s].data_ptr(), s if events else None, self.stream)
        self._exchange()

    def step_direct(self, s: int):
        """One decode step launched on the stream even when a graph has been captured (the cold-cache timing of
        a workload whose graph holds several steps); skip_replayed_steps() afterwards keeps the graph in step."""
        self._launch_step(self.pos_all[s].data_ptr(), self.len_all[s].data_ptr(), None, self.stream)
        self._exchange()

    def skip_replayed_steps(self, count: int):
        assert count % self.steps_per_graph == 0 and (self.graph_next - self.graph_first) % self.steps_per_graph == 0
        self.step_state.add_(count)
        self.graph_next += count

    def _exchange(self):
        """The step's exchange between the ranks (cfg4 on more than one GPU). KV-head sharding: all-gather of the
        head outputs, after which every rank holds all heads' rows. Key-range sharding: every rank's rows and
        log-sum-exp are exchanged and merged, after which `out` / `lse` hold the full attention on every rank."""
        if not (self.spec.gather and self.world > 1):
            return
        import torch.distributed as dist

        torch = self.torch
        rows = self.out.numel() // D
        if self.spec.key_shard:
            if self.peer is None or not self.gather_checked:
                # ncclAllGather of rows and log-sum-exp, merge with torch ops (the --gather nccl arm, and once in
                # the warm-up the check of the peer kernel's merge)
                all_out = torch.empty((self.world, rows, D), dtype=torch.bfloat16, device=self.out.device)
                all_lse = torch.empty((self.world, rows), dtype=torch.float32, device=self.out.device)
                dist.all_gather_into_tensor(all_out, self.out.view(rows, D))
                dist.all_gather_into_tensor(all_lse, self.lse.view(rows))
                weight = torch.softmax(all_lse, dim=0)
                merged = (weight[:, :, None] * all_out.float()).sum(0)
                if self.peer is None:
                    self.out.view(rows, D).copy_(merged)
                    self.lse.view(rows).copy_(torch.logsumexp(all_lse, dim=0))
                    return
            self.peer.merge_attention(self.out, self.lse, self.out, self.lse, rows, D, status=self.status,
                                      stream=self.stream)
            if not self.gather_checked:
                self.gather_checked = True
                err = (self.out.view(rows, D).float() - merged).abs().max().item()
                assert err <= 2.0 ** -7 * max(1.0, merged.abs().max().item()), f"peer merge differs: {err}"
            return
        if self.peer is None:
            dist.all_gather_into_tensor(self.out_all, self.out)
            return
        self.gathered_ptr = self.peer.gathered()          # the step's own exchange has been enqueued with it
        if not self.gather_checked:          # once, in the warm-up: the same rows as NCCL's all-gather
            self.gather_checked = True
            dist.all_gather_into_tensor(self.out_all, self.out)
            got = torch.empty_like(self.out_all)
            cudart = ctypes.CDLL("libcudart.so.12")
            cudart.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
            torch.cuda.synchronize()
            rc = cudart.cudaMemcpy(got.data_ptr(), self.gathered_ptr, got.numel() * 2, 3)
            assert rc == 0 and torch.equal(got.view(torch.int16), self.out_all.view(torch.int16)), \
                "peer all-gather differs from ncclAllGather"

    def _launch_step(self, pos: int, length: int, s, stream: int):
        kv = self.kv
        if self.spec.fp8:
            # the fp8 cache has its own two entry points; the layer loop is here instead of in the library
            for i in range(self.L):
                li = self.cache_layer_of(i)
                kv.decode_append_fp8(self.q_prepared[i], self.g_k, self.g_v, self.g_sk, self.g_sv, self.g_cfg,
                                     self.g_table, pos, li, self.raw_q[i], self.raw_k[i], self.raw_v[i], self.q_w,
                                     self.k_w, self.g_cos, self.g_sin, self.B, self.spec.hq, D,
                                     kv.NORM_RSQRT_APPROX, stream=stream)
                if i == self.timed_layer and s is not None:
                    self.ev_begin[s].record(stream)
                kv.decode_attention_fp8(self.out[i], self.lse[i], self.q_prepared[i], self.g_k, self.g_v, self.g_sk,
                                        self.g_sv, self.g_cfg, self.g_table, length, li, 1.0 / math.sqrt(D),
                                        self.g_nsplit, self.B, self.spec.hq, self.pm, self.pl, self.pacc,
                                        self.status, stream=stream)
                if i == self.timed_layer and s is not None:
                    self.ev_end[s].record(stream)
        else:
            for i in range(self.L):
                self.layers[i].token_position = pos
                self.layers[i].seq_lengths = length
            g = self.layers[self.timed_layer]
            g.event_before_attention = self.ev_begin[s].handle if s is not None else None
            g.event_after_attention = self.ev_end[s].handle if s is not None else None
            kv.decode_step(self.layers, self.L, stream=stream)

    def step_e2e(self, s: int):
        """The same step called with host buffers: projections come from pinned host memory and the
        attention outputs go back to the host, every step."""
        torch = self.torch
        self.raw.copy_(self.raw_host, non_blocking=True)
        self._unpack_raw()
        self.step(s)
        self.out_host.copy_(self.out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def bytes_for_step(self, s: int) -> tuple[int, int]:
        sp = self.spec
        after = self.ctx + s + 1 if self.owns_new_rows else self.ctx
        total = (sp.n_local * layer_step_bytes(after, WINDOW, sp.hkv, sp.e_kv)
                 + sp.n_global * layer_step_bytes(after, 0, sp.hkv, sp.e_kv))
        timed_window = 0 if sp.n_global else WINDOW
        return total, attention_kernel_bytes(after, timed_window, sp.hkv, sp.e_kv)


# --------------------------------------------------------------------------- CPU baseline
def cpu_layer_step_sample(ctx: np.ndarray, threads: int, target_seconds: float, max_keys: int = 131072):
    """Times the CPU restatement (oracle) on a bounded sample of the same workload: the global layer-step
    for the first sequences of the batch (about `max_keys` keys, 1 GiB of K+V), repeated until roughly
    `target_seconds` of host time have passed."""
    from oracle import binding as orc

    orc.build()
    rng = np.random.default_rng(1)
    chosen, total = [], 0
    for c in ctx:
        if chosen and total + int(c) > max_keys:
            break
        chosen.append(int(c))
        total += int(c)
    sample_ctx = np.array(chosen, dtype=np.int64)
    B = sample_ctx.size
    pages_b = (sample_ctx + 1 + PAGE - 1) // PAGE
    num_pages, mpps = int(pages_b.sum()), int(pages_b.max())
    table = np.full((B, mpps), -1, dtype=np.int32)
    pool = rng.permutation(num_pages).astype(np.int32)
    cur = 0
    for b in range(B):
        table[b, :pages_b[b]] = pool[cur:cur + pages_b[b]]
        cur += int(pages_b[b])
    cfg = (1, num_pages, PAGE, mpps, B, HKV, D, 0)
    elems = num_pages * PAGE * HKV * D
    block = orc.f32_to_bf16(rng.standard_normal(1 << 22, dtype=np.float32))
    reps = -(-elems // block.size)
    ck = np.tile(block, reps)[:elems].copy()
    cv = np.tile(block[::-1], reps)[:elems].copy()
    q = orc.f32_to_bf16(rng.standard_normal((B, HQ, D), dtype=np.float32))
    k = orc.f32_to_bf16(rng.standard_normal((B, HKV, D), dtype=np.float32))
    v = orc.f32_to_bf16(rng.standard_normal((B, HKV, D), dtype=np.float32))
    w = orc.f32_to_bf16(np.ones(D, dtype=np.float32))
    cos, sin = orc.fill_rope_tables(int(sample_ctx.max()) + 1, D // 2, 1000000.0, D)
    pos = sample_ctx.astype(np.int32)
    lens = (sample_ctx + 1).astype(np.int32)
    out = np.zeros((B, HQ, D), dtype=np.uint16)
    qp = np.zeros((B, HQ, D), dtype=np.uint16)
    nbytes = layer_step_bytes(sample_ctx + 1, 0)
    secs, runs = 0.0, 0
    while runs < 1 or (secs < target_seconds and runs < 1000):
        secs += orc.layer_step_timed(threads, out, qp, ck, cv, cfg, table, pos, lens, 0, q, k, v, w, w, cos, sin,
                                     B, HQ, 1.0 / math.sqrt(D), 256)
        runs += 1
    return {"seconds": secs, "bytes": nbytes * runs, "gbps": nbytes * runs / secs / 1e9, "sequences": int(B),
            "keys": int(sample_ctx.sum()) + int(B), "runs": runs, "us_per_layer_step": secs / runs * 1e6}


def reference_cuda_numbers(wl, torch, step_index: int):
    """The reference's own CUDA kernels (compiled from the gemma.c sources for sm_100a into oracle/_ref, when
    that library is present) on the timed layer of this rank's workload, same cache, same inputs, same GPU:
    fused append phase, split phase + reduce phase at the reference's default split size of 20 keys
    (src/gemma4.h:24) and at larger splits. Reported beside the library's number; never part of it."""
    from oracle import ref_binding as ref

    sp = wl.spec
    if not ref.available() or sp.fp8 or sp.hkv != 8:
        return None
    i = wl.timed_layer
    is_global = wl.layer_is_global(i)
    cfg = (wl.g_cfg if is_global else wl.l_cfg).astuple()
    ck, cv = (wl.g_k, wl.g_v) if is_global else (wl.l_k, wl.l_v)
    table = wl.g_table if is_global else wl.l_table
    cos, sin = (wl.g_cos, wl.g_sin) if is_global else (wl.l_cos, wl.l_sin)
    layer = wl.cache_layer_of(i)
    pos, length = wl.pos_all[step_index], wl.len_all[step_index]
    window = 0 if is_global else WINDOW
    longest = int(wl.ctx.max()) + step_index + 1
    live = min(longest, window) if window else longest
    nbytes = attention_kernel_bytes(wl.ctx + step_index + 1, window, sp.hkv, sp.e_kv)
    qp = torch.empty_like(wl.q_prepared[i])
    out = torch.empty_like(wl.out[i])

    def timed(fn, reps):
        fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps * 1e3

    result = {"kernels": "phase_decode_q_paged_kv_norm_rope / phase_decode_paged_grouped_split / "
                         "phase_decode_paged_reduce of src/gemma4_flash_attention_decode.cu, sm_100a build",
              "layer": "global" if is_global else "sliding", "attention": []}
    result["append_us"] = timed(lambda: ref.decode_append(qp, ck, cv, cfg, table, pos, layer, wl.raw_q[i], wl.raw_k[i],
                                                          wl.raw_v[i], wl.q_w, wl.k_w, cos, sin, wl.B), 5)
    for split in (20, 64, 256):
        nsplit = max(1, -(-live // split))
        rows = wl.B * sp.hq * nsplit
        if rows * (D + 2) * 4 > 8e9 or nsplit > 65535:
            continue
        pm = torch.empty(rows, dtype=torch.float32, device="cuda")
        pl = torch.empty(rows, dtype=torch.float32, device="cuda")
        pacc = torch.empty(rows * D, dtype=torch.float32, device="cuda")
        us = timed(lambda: ref.decode_attention(out, pm, pl, pacc, qp, ck, cv, table, length, cfg, layer,
                                                1.0 / math.sqrt(D), split, nsplit, wl.B), 2)
        result["attention"].append({"split_size": split, "num_splits": nsplit, "us": us,
                                    "GBps": nbytes / (us * 1e-6) / 1e9})
        del pm, pl, pacc
    return result


# --------------------------------------------------------------------------- parity of what was just run
# Tolerances of the GPU tests (tests/helpers.py): attention rows against double precision on the same cache,
# max_abs and max_rel with the reference bench's denominator max(|a|, |b|, 1)
# (src/benches/gemma4_bench_utils.cuh:450-472); natural-log log-sum-exp.
VERIFY_MAX_ABS, VERIFY_MAX_REL, VERIFY_LSE = 2.0 ** -6, 2.0 ** -6, 1.0e-3


def sample_sequences(ctx: np.ndarray, count: int, seed: int) -> list[int]:
    """The longest, the shortest and seeded random other sequences of a batch (at most `count`, no repeats)."""
    order = np.argsort(ctx, kind="stable")
    picks = []
    for b in [int(order[-1]), int(order[0]), *np.random.default_rng(seed).permutation(ctx.size).tolist()]:
        if b not in picks and len(picks) < count:
            picks.append(int(b))
    return picks


def _bits(t):
    """Device bf16 / int16 tensor -> host uint16 bit patterns."""
    import torch

    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def compact_layer_cache(wl, i: int, seqs: list[int]):
    """The pages of layer i's cache that the sequences `seqs` map, gathered (on the device) into a small cache
    of their own with a page table to match: what a CPU checker needs of a pool of many GB. Returns device
    tensors and the config tuple of the small cache; every page keeps its bytes, fp8 scales ride along."""
    torch = wl.torch
    g = wl.layer_is_global(i)
    cfg = (wl.g_cfg if g else wl.l_cfg).astuple()
    layers, pages, ps, mpps, _, heads, dim, window = cfg
    li = wl.cache_layer_of(i)
    table = (wl.g_table if g else wl.l_table)[torch.tensor(seqs, device="cuda")]
    valid = (table >= 0) & (table < pages)
    phys = table[valid].long()
    small_table = torch.full_like(table, -1)
    small_table[valid] = torch.arange(phys.numel(), dtype=table.dtype, device="cuda")
    k, v = (wl.g_k, wl.g_v) if g else (wl.l_k, wl.l_v)
    page_elems = ps * heads * dim
    out = {"ck": k.view(layers, pages, page_elems)[li].index_select(0, phys).contiguous(),
           "cv": v.view(layers, pages, page_elems)[li].index_select(0, phys).contiguous(),
           "table": small_table.contiguous(),
           "cfg": (1, int(phys.numel()), ps, mpps, len(seqs), heads, dim, window)}
    if wl.spec.fp8:
        out["sk"] = wl.g_sk.view(layers, pages, heads)[li].index_select(0, phys).contiguous()
        out["sv"] = wl.g_sv.view(layers, pages, heads)[li].index_select(0, phys).contiguous()
    return out


def attention_errors(got_bits: np.ndarray, ref: np.ndarray, orc):
    a = orc.bf16_to_f32(got_bits).astype(np.float64).reshape(-1)
    b = ref.astype(np.float64).reshape(-1)
    diff = np.abs(a - b)
    return float(diff.max(initial=0.0)), float((diff / np.maximum(np.maximum(np.abs(a), np.abs(b)), 1.0)).max(initial=0.0))


def bf16_mismatch(a: np.ndarray, b: np.ndarray, orc):
    """(elements whose bits differ, elements further apart than one bf16 step at their magnitude, largest
    |difference|) between two arrays of bf16 bit patterns. "One step at their magnitude": |a - b| <=
    2^-7 * max(|a|, |b|), with an absolute floor of 2^-9 for results that cancel to almost nothing (there a
    last-bit difference of the norm scale moves the tiny result by many of ITS steps and by nothing that matters)."""
    x = orc.bf16_to_f32(a.reshape(-1)).astype(np.float64)
    y = orc.bf16_to_f32(b.reshape(-1)).astype(np.float64)
    diff = np.abs(x - y)
    bound = np.maximum(2.0 ** -7 * np.maximum(np.abs(x), np.abs(y)), 2.0 ** -9)
    return int((a.reshape(-1) != b.reshape(-1)).sum()), int((diff > bound).sum()), float(diff.max(initial=0.0))


def verify_step(wl, s: int, count: int = 4, layers=None, seqs=None) -> dict:
    """Checks what step `s` -- the step that ran last -- left on the device, for a sample of this rank's
    sequences (the longest, the shortest, random others; `count` in all, or `seqs`) on the timed (global) layer
    and on the first sliding layer (or `layers`), against the CPU oracle (test infrastructure, never timed):
      * attention rows and log-sum-exp against double precision over the same cache and prepared q;
      * the prepared q and the appended K/V rows against the oracle's fused append (IEEE square root and
        divide; the library's default mode uses rsqrt.approx like the reference's GPU code, so single elements
        may sit one bf16 step away: counted, bounded) and, where the reference's own append kernel is built
        (oracle/_ref, same arithmetic as the default mode), against that kernel bit for bit.
    Runs outside every timed region. Returns the figures and "ok"."""
    from oracle import binding as orc

    orc.build()
    torch, sp = wl.torch, wl.spec
    torch.cuda.synchronize()
    if seqs is None:
        seqs = sample_sequences(wl.ctx, count, 7 + s)
    if layers is None:
        layers = [i for i in (wl.timed_layer, 0) if 0 <= i < wl.L]
        layers = list(dict.fromkeys(layers))
    idx = torch.tensor(seqs, device="cuda")
    n = len(seqs)
    lens = wl.len_all[s][idx].cpu().numpy().astype(np.int32)
    pos = wl.pos_all[s][idx].cpu().numpy().astype(np.int32)
    res = {"step": int(s), "sequences": [int(b) for b in seqs], "layers": [], "rows": 0, "max_abs": 0.0, "max_rel": 0.0,
           "lse_max_abs": 0.0, "cache_rows_exact": None, "append_vs_ieee_oracle": {"elements": 0, "differing": 0,
                                                                                 "beyond_one_step": 0, "max_abs": 0.0}}
    ok = int(wl.status[0].item()) == 0
    ref_lib = None
    if not sp.fp8 and sp.hkv == 8 and not sp.key_shard:
        try:
            from oracle import ref_binding

            ref_lib = ref_binding if ref_binding.available() else None
        except OSError:
            ref_lib = None
    for i in layers:
        g = wl.layer_is_global(i)
        c = compact_layer_cache(wl, i, seqs)
        cfg = c["cfg"]
        table = c["table"].cpu().numpy().astype(np.int32)
        q = _bits(wl.q_prepared[i][idx])
        got = _bits(wl.out[i][idx])
        got_lse = wl.lse[i][idx].cpu().numpy()
        scale = 1.0 / math.sqrt(D)
        if sp.fp8:
            ck, cv = c["ck"].cpu().numpy(), c["cv"].cpu().numpy()
            ref, ref_lse = orc.fp8_decode_attention_f64(q, ck.reshape(-1), cv.reshape(-1), c["sk"].cpu().numpy().reshape(-1),
                                                        c["sv"].cpu().numpy().reshape(-1), table, lens, cfg, 0, scale, n, sp.hq)
        else:
            ck, cv = _bits(c["ck"]).reshape(-1), _bits(c["cv"]).reshape(-1)
            ref, ref_lse = orc.decode_attention_f64(q, ck, cv, table, lens, cfg, 0, scale, n, sp.hq)
        max_abs, max_rel = attention_errors(got, ref, orc)
        finite = np.isfinite(ref_lse)
        lse_err = float(np.abs(got_lse[finite] - ref_lse[finite]).max(initial=0.0))
        ok = ok and max_abs <= VERIFY_MAX_ABS and max_rel <= VERIFY_MAX_REL and lse_err <= VERIFY_LSE \
            and bool(np.array_equal(np.isfinite(got_lse), finite))
        entry = {"layer": int(i), "kind": "global" if g else "sliding", "keys": [int(min(x, WINDOW)) if not g else int(x)
                                                                               for x in lens],
                 "max_abs": max_abs, "max_rel": max_rel, "lse_max_abs": lse_err}
        res["rows"] += n * sp.hq
        res["max_abs"], res["max_rel"] = max(res["max_abs"], max_abs), max(res["max_rel"], max_rel)
        res["lse_max_abs"] = max(res["lse_max_abs"], lse_err)
        if not sp.fp8 and not sp.key_shard:
            # the append of this step: prepared q and the new cache rows
            rq, rk, rv = _bits(wl.raw_q[i][idx]), _bits(wl.raw_k[i][idx]), _bits(wl.raw_v[i][idx])
            cos_t, sin_t = ((wl.g_cos, wl.g_sin) if g else (wl.l_cos, wl.l_sin))
            cos, sin = cos_t.cpu().numpy(), sin_t.cpu().numpy()
            qp = np.zeros((n, sp.hq, D), np.uint16)
            ck2, cv2 = ck.copy(), cv.copy()
            orc.decode_append(qp, ck2, cv2, cfg, table, pos, 0, rq.reshape(n, sp.hq, D), rk.reshape(n, sp.hkv, D),
                              rv.reshape(n, sp.hkv, D), _bits(wl.q_w), _bits(wl.k_w), cos, sin, n, sp.hq, D)
            off = [bf16_mismatch(qp, q, orc), bf16_mismatch(ck2, ck, orc), bf16_mismatch(cv2, cv, orc)]
            elements = n * (sp.hq + 2 * sp.hkv) * D
            differing, beyond = sum(o[0] for o in off), sum(o[1] for o in off)
            a = res["append_vs_ieee_oracle"]
            a["elements"] += elements
            a["differing"] += differing
            a["beyond_one_step"] += beyond
            a["max_abs"] = max(a["max_abs"], max(o[2] for o in off))
            ok = ok and beyond == 0 and differing <= 0.02 * elements
            if ref_lib is not None:
                # the reference's own fused append kernel on a copy of the same pages: it rewrites the new rows,
                # and nothing may change
                ckd, cvd = c["ck"].clone(), c["cv"].clone()
                qpd = torch.zeros_like(wl.q_prepared[i][idx])
                rc = ref_lib.decode_append(qpd, ckd, cvd, cfg, c["table"], wl.pos_all[s][idx].contiguous(), 0,
                                           wl.raw_q[i][idx].contiguous(), wl.raw_k[i][idx].contiguous(),
                                           wl.raw_v[i][idx].contiguous(), wl.q_w, wl.k_w, cos_t, sin_t, n)
                torch.cuda.synchronize()
                exact = (rc == 0 and torch.equal(ckd, c["ck"]) and torch.equal(cvd, c["cv"])
                         and torch.equal(qpd.view(torch.int16), wl.q_prepared[i][idx].view(torch.int16)))
                entry["append_equals_reference_kernel"] = bool(exact)
                res["cache_rows_exact"] = bool(exact) if res["cache_rows_exact"] is None else (res["cache_rows_exact"] and exact)
                ok = ok and exact
        res["layers"].append(entry)
    if res["cache_rows_exact"] is None and res["append_vs_ieee_oracle"]["elements"]:
        res["cache_rows_exact"] = res["append_vs_ieee_oracle"]["differing"] == 0
        res["cache_checker"] = "host oracle (IEEE 1/sqrt); the reference's append kernel was not available"
    elif res["cache_rows_exact"] is not None:
        res["cache_checker"] = "the reference's own fused append kernel (oracle/_ref) on the same pages, bit for bit"
    res["tolerance"] = {"max_abs": VERIFY_MAX_ABS, "max_rel": VERIFY_MAX_REL, "lse_max_abs": VERIFY_LSE,
                        "append": "host oracle (IEEE 1/sqrt; the library's default mode uses rsqrt.approx like the "
                                  "reference's GPU code): no element further than one bf16 step at its magnitude "
                                  "(floor 2^-9), under 2 % of elements differing at all; reference kernel: exact"}
    res["ok"] = bool(ok)
    return res


def run_reference_arm(args):
    """`--impl reference`: the reference's own implementation of the path on the same workload. gemma.c has no CPU
    implementation of it -- its KV path is CUDA only -- so the arm runs the reference's own CUDA kernels, built
    for sm_100a from its unchanged sources (oracle/_ref, oracle/build_ref.sh), when that library and a GPU are
    there: fused append phase, split phase and reduce phase at the reference's split size of 20 keys
    (src/gemma4.h:24), layer by layer. The reference is single-GPU (decode requires batch 1 and one device,
    src/gemma4_decode_megakernel.cu:143): under torchrun rank 0 alone runs the whole batch on its GPU and the
    other ranks exit. Without that library (or a GPU) it falls back to the CPU port of the same phases."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import ref_binding as ref

    gpu = False
    try:
        import torch

        gpu = torch.cuda.is_available()
    except ImportError:
        torch = None
    if gpu and ref.available() and args.workload == "cfg3":
        run_reference_cuda_arm(args, torch, ref)
    else:
        run_reference_cpu_arm(args, "no GPU" if not gpu else ("oracle/_ref not built" if not ref.available()
                                                              else f"workload {args.workload}"))


def run_reference_cuda_arm(args, torch, ref):
    """The default workload (BASELINE configs[2]) through the reference's CUDA phases on one GPU. Nothing of the
    B200 library is loaded: caches, tables and metadata are built with torch and the oracle's host helpers."""
    from oracle import binding as orc

    orc.build()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = "cuda"
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    ctx = context_lengths(args)
    B = int(ctx.size)
    split = 20                                            # GEMMA4_SLIDING_DECODE_SPLIT_SIZE, src/gemma4.h:24
    e2e_warm = 2
    e2e_steps = min(args.e2e_steps, 5)
    total = args.warmup + args.steps + e2e_warm + e2e_steps
    gen = torch.Generator(device=dev)
    gen.manual_seed(args.seed)
    rng = np.random.default_rng(args.seed)

    def normal_bf16(n):
        t = torch.empty(n, dtype=torch.bfloat16, device=dev)
        t.normal_(generator=gen)
        return t

    pages_b = (ctx + total + PAGE) // PAGE
    g_pages, g_mpps = int(pages_b.sum()), int(pages_b.max())
    table = np.full((B, g_mpps), -1, dtype=np.int32)
    pool = rng.permutation(g_pages).astype(np.int32)
    cur = 0
    for b in range(B):
        table[b, :pages_b[b]] = pool[cur:cur + pages_b[b]]
        cur += int(pages_b[b])
    n_local, n_global = 5, 1
    l_mpps = (WINDOW + PAGE - 1 + PAGE - 1) // PAGE
    g_cfg = (n_global, g_pages, PAGE, g_mpps, B, HKV, D, 0)
    l_cfg = (n_local, B * l_mpps, PAGE, l_mpps, B, HKV, D, WINDOW)
    g_table = torch.from_numpy(table).to(dev)
    l_table = torch.from_numpy(rng.permutation(B * l_mpps).astype(np.int32).reshape(B, l_mpps)).to(dev)
    elems = lambda c: c[0] * c[1] * c[2] * c[5] * c[6]
    g_k, g_v = normal_bf16(elems(g_cfg)), normal_bf16(elems(g_cfg))
    l_k, l_v = normal_bf16(elems(l_cfg)), normal_bf16(elems(l_cfg))
    max_pos = int(ctx.max()) + total + 1
    g_cos, g_sin = (torch.from_numpy(t).to(dev) for t in orc.fill_rope_tables(max_pos, D // 2, 1000000.0, D))
    l_cos, l_sin = (torch.from_numpy(t).to(dev) for t in orc.fill_rope_tables(max_pos, D // 2, 10000.0, D))
    w = torch.empty(2, D, dtype=torch.float32, device=dev).normal_(1.0, 0.05, generator=gen).to(torch.bfloat16)
    L = n_local + n_global
    row = (HQ + 2 * HKV) * D
    raw = normal_bf16(L * B * row).view(L, B, row)
    raw_host = torch.empty((L, B, row), dtype=torch.bfloat16).pin_memory()
    raw_host.copy_(raw)
    raw_q = torch.empty((L, B, HQ * D), dtype=torch.bfloat16, device=dev)
    raw_k = torch.empty((L, B, HKV * D), dtype=torch.bfloat16, device=dev)
    raw_v = torch.empty((L, B, HKV * D), dtype=torch.bfloat16, device=dev)

    def unpack():
        q, k, v = raw.split([HQ * D, HKV * D, HKV * D], dim=2)
        raw_q.copy_(q); raw_k.copy_(k); raw_v.copy_(v)

    unpack()
    q_prepared = torch.empty((L, B, HQ, D), dtype=torch.bfloat16, device=dev)
    out = torch.empty((L, B, HQ, D), dtype=torch.bfloat16, device=dev)
    out_host = torch.empty((L, B, HQ, D), dtype=torch.bfloat16).pin_memory()
    steps_i = np.arange(total, dtype=np.int64)[:, None]
    pos_all = torch.from_numpy((ctx[None, :] + steps_i).astype(np.int32)).to(dev)
    len_all = torch.from_numpy((ctx[None, :] + steps_i + 1).astype(np.int32)).to(dev)
    g_nsplit = -(-(int(ctx.max()) + total) // split)
    l_nsplit = -(-WINDOW // split)
    rows = B * HQ * max(g_nsplit, l_nsplit)
    pm = torch.empty(rows, dtype=torch.float32, device=dev)
    pl = torch.empty(rows, dtype=torch.float32, device=dev)
    pacc = torch.empty(rows * D, dtype=torch.float32, device=dev)
    is_global = [(i + 1) % 6 == 0 for i in range(L)]       # five sliding layers, then one global (src/gemma4.h:105-108)
    scale = 1.0 / math.sqrt(D)

    def step(s):
        n_l = n_g = 0
        for i in range(L):
            g = is_global[i]
            cfg, ck, cv, tab = (g_cfg, g_k, g_v, g_table) if g else (l_cfg, l_k, l_v, l_table)
            cos, sin = (g_cos, g_sin) if g else (l_cos, l_sin)
            li = n_g if g else n_l
            rc = ref.decode_append(q_prepared[i], ck, cv, cfg, tab, pos_all[s], li, raw_q[i], raw_k[i], raw_v[i],
                                   w[0], w[1], cos, sin, B)
            rc2 = ref.decode_attention(out[i], pm, pl, pacc, q_prepared[i], ck, cv, tab, len_all[s], cfg, li, scale,
                                       split, g_nsplit if g else l_nsplit, B)
            if rc or rc2:
                raise RuntimeError(f"reference kernel launch failed: {rc} {rc2}")
            n_g, n_l = n_g + int(g), n_l + int(not g)

    def bytes_of(s):
        after = ctx + s + 1
        return n_local * layer_step_bytes(after, WINDOW) + n_global * layer_step_bytes(after, 0)

    sampler.mark("load_begin")
    s = 0
    for _ in range(args.warmup):
        step(s); s += 1
    torch.cuda.synchronize()
    sampler.mark("timed_begin")
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    first = s
    marks[0].record()
    for i in range(args.steps):
        step(s); s += 1
        marks[i + 1].record()
    torch.cuda.synchronize()
    sampler.mark("timed_end")
    ms = marks[0].elapsed_time(marks[-1])
    step_bytes = sum(bytes_of(i) for i in range(first, first + args.steps))

    def step_e2e(s):
        raw.copy_(raw_host, non_blocking=True)
        unpack()
        step(s)
        out_host.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(e2e_warm):
        step_e2e(s); s += 1
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    first_e = s
    e0.record()
    for _ in range(e2e_steps):
        step_e2e(s); s += 1
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1)
    e2e_bytes = sum(bytes_of(i) for i in range(first_e, first_e + e2e_steps))
    sampler.mark("load_end")
    clocks = sampler.stop()
    value = step_bytes / (ms * 1e-3) / 1e9
    threads = orc.hardware_threads()
    cpu = cpu_layer_step_sample(ctx, threads, min(args.cpu_seconds, 5.0))
    cfg_line = workload_config(args, 1, "B200 (one GPU)", "single GPU: the reference does not shard", L)
    cfg_line["launch"] = "stream launches: fused append phase, split phase, reduce phase per layer"
    cfg_line["split_size"] = split
    line = {
        "impl": "reference", "reference_class": "cuda",
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus, "gpus_used": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg_line,
        "us_per_layer_step": ms * 1e3 / (args.steps * L), "step_ms_stats": step_stats(marks),
        "e2e": {"value": e2e_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": int(raw_host.numel() * 2), "d2h_bytes_per_step": int(out_host.numel() * 2),
                "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
        "cpu_baseline": {"value": cpu["gbps"], "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"global layer-step over the first {cpu['sequences']} sequences ({cpu['keys']} keys), "
                                   f"{cpu['runs']} passes, oracle port on all host threads; shown beside, not the arm's value"},
        "gpu_launches": 3 * L * args.steps,
        "kernels": "phase_decode_q_paged_kv_norm_rope, phase_decode_paged_grouped_split, phase_decode_paged_reduce of "
                   "src/gemma4_flash_attention_decode.cu:305-375,692-977, compiled unchanged for sm_100a",
        "clocks": clocks,
        "note": "gemma.c has no CPU implementation of this path; this arm is its own CUDA code on one B200"
                + ("" if args.gpus == 1 else f" (single-GPU reference: rank 0 ran all {B} sequences on one GPU of the {args.gpus})"),
    }
    print(json.dumps(line))


def run_reference_cpu_arm(args, why: str):
    """Fallback of the reference arm: the CPU port of the reference's phases on all host cores; each step is
    one global layer-step over a bounded sample of the workload's sequences."""
    from oracle import binding as orc

    orc.build()
    threads = orc.hardware_threads()
    _, ctx, _, _, _ = plan_workload(args, 1, 0)
    per_step = max(0.5, min(args.cpu_seconds, 120.0 / max(1, args.steps + args.warmup)))
    times, sample = [], None
    for i in range(args.warmup + args.steps):
        sample = cpu_layer_step_sample(ctx, threads, per_step)
        if i >= args.warmup:
            times.append(sample)
    secs = sum(t["seconds"] for t in times)
    nbytes = sum(t["bytes"] for t in times)
    value = nbytes / secs / 1e9
    desc = (f"global layer-step (append + split attention + reduce) over the first {sample['sequences']} "
            f"sequences ({sample['keys']} keys) of the workload, {sample['runs']} passes per step")
    line = {
        "impl": "reference", "reference_class": "cpu", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs / len(times) * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args, 1, "cpu"),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": f"the reference's CUDA kernels could not be run here ({why}); this is the oracle port of its CUDA "
                "phases (oracle/kv_oracle.cpp) on all host threads",
    }
    print(json.dumps(line))


WORKLOADS = {
    "cfg1": "configs[0]: single sliding layer, batch 1, tight 1024-token ring pre-filled, one token appended "
            "per step (wraps), 16Q/8KV/D256 bf16",
    "cfg2": "configs[1]: 48-layer stack (40 sliding window-1024 + 8 global at context 4096), batch 1, "
            "16Q/8KV/D256 bf16, one token appended per layer per step",
    "cfg3": "configs[2]: batched paged decode, 64 sequences ctx~U[512,32768], 16-token pages, permuted block "
            "table, 16Q/8KV/D256 bf16; step = 5 sliding (window 1024) + 1 global layer-step",
    "cfg4": "configs[3]: one sequence of 131072 keys (1 % of keys x8), global layer, split-KV decode; KV heads "
            "sharded over the ranks, all-gather of the head outputs",
    "cfg5": "configs[4]: FP8 e4m3 cache (fp32 scale per 16-token page and KV head), batch 32, context 8192, "
            "global layer, quantise-on-append + fused dequant",
}


# One-layer workloads put this many consecutive steps into one graph: what a replay of configs[1] holds (48 layers).
ONE_LAYER_STEPS_PER_GRAPH = 48


def replays_graph(args, world: int) -> bool:
    """Whether the steps are replayed from a CUDA graph: the batch-1 workloads, and the KV-head-sharded long
    context with the one-launch kernel (on several GPUs with the exchange inside the kernel, or one rank's share
    emulated on one GPU) -- ONE_LAYER_STEPS_PER_GRAPH consecutive steps of the one layer per graph, handed to the library as one
    b200kv_decode_step_bf16 call, so that the ranks' launches do not drift against each other under the hosts'
    jitter and the library can keep the steps' launches overlapped."""
    if args.graph != "auto":
        return args.graph == "on"
    if args.workload in ("cfg1", "cfg2"):
        return True
    sharded = world > 1 or args.emulate_world > 1
    return (args.workload == "cfg4" and sharded and args.shard == "heads" and not args.no_tickets
            and (args.gather == "peer" or world == 1))


def plan_workload(args, world: int, rank: int):
    """Returns (spec, all context lengths, this rank's context lengths, parallelism text, scaling)."""
    name = args.workload
    if name == "cfg3":
        ctx_all = context_lengths(args)
        mine = ctx_all[shard_sequences(ctx_all, world)[rank]]
        return Spec(name, WORKLOADS[name], 5, 1), ctx_all, mine, f"sequence-sharded x{world}, no collective", "strong"
    if name == "cfg5":
        ctx_all = np.full(args.seqs or 32, 8192, dtype=np.int64)
        mine = ctx_all[shard_sequences(ctx_all, world)[rank]]
        return (Spec(name, WORKLOADS[name], 0, 1, fp8=True), ctx_all, mine,
                f"sequence-sharded x{world}, no collective", "strong")
    if name == "cfg4":
        if 8 % world:
            raise SystemExit("cfg4 shards 8 KV heads: --gpus must divide 8")
        ctx_all = np.array([131072], dtype=np.int64)
        shards = args.emulate_world if (world == 1 and args.emulate_world > 1) else world   # tuning aid: one rank's share
        if args.shard == "keys" and shards > 1:
            if 131072 % (shards * PAGE):
                raise SystemExit("cfg4 --shard keys: the ranks must divide 131072 / 16 pages")
            me = rank if world > 1 else args.emulate_rank
            mine = np.array([131072 // shards], dtype=np.int64)
            return (Spec(name, WORKLOADS[name], 0, 1, outliers=True, gather=world > 1, key_shard=(me, shards)),
                    ctx_all, mine,
                    f"key-range-sharded x{shards} (all 8 KV heads of {131072 // shards} keys per rank), rows merged by "
                    "log-sum-exp" + (" in one peer-store kernel per rank over NVLink (b200kv_peer_merge_attention)"
                                     if args.gather == "peer" else " after two ncclAllGather calls"), "strong")
        return (Spec(name, WORKLOADS[name], 0, 1, hkv=8 // shards, outliers=True, gather=True), ctx_all, ctx_all,
                f"KV-head-sharded x{world} ({8 // world} KV heads per rank), all-gather of head outputs: "
                + ("one peer-store kernel per rank over NVLink (b200kv_peer_allgather)" if args.gather == "peer"
                   else "ncclAllGather"),
                "strong")
    if world > 1:
        raise SystemExit(f"{name} is a batch-1 latency case: run it on one GPU")
    if name == "cfg1":
        ctx_all = np.array([1024], dtype=np.int64)
        return Spec(name, WORKLOADS[name], 1, 0, tight_ring=True), ctx_all, ctx_all, "single GPU", "strong"
    ctx_all = np.array([4096], dtype=np.int64)
    return Spec(name, WORKLOADS[name], 40, 8), ctx_all, ctx_all, "single GPU", "strong"


def workload_config(args, world, where, parallelism=None, layers=None):
    cfg = {
        "workload": WORKLOADS[args.workload],
        "seed": args.seed, "page_size": PAGE,
        "parallelism": parallelism or f"x{world}",
        "partition": args.partition,
        "where": where,
        "launch": ("one CUDA graph replay per step" + (f" ({ONE_LAYER_STEPS_PER_GRAPH} one-kernel steps per replay)"
                                                         if args.workload in ("cfg1", "cfg4") else "")
                   if replays_graph(args, world)
                   else "stream launches (programmatic dependent launch between kernels)"),
    }
    if args.workload == "cfg3":
        cfg.update({"sequences": args.seqs or 64, "ctx_range": [args.min_ctx, args.max_ctx], "layers_per_step": 6,
                    "l2": "inputs larger than L2: every step streams more than 1 GB per rank before any byte "
                          "is revisited"})
    elif layers is not None:
        cfg["layers_per_step"] = layers
    if args.workload in ("cfg1", "cfg2"):
        cfg["l2"] = ("working set of a step (8 MB / 600 MB) against a 126 MB L2: cfg1 is L2-resident by "
                     "construction and is a latency case, not a bandwidth claim")
    elif args.workload in ("cfg4", "cfg5"):
        cfg["l2"] = "inputs larger than L2: a step streams more than 130 MB per rank" 
    return cfg


def step_stats(marks) -> dict:
    """Distribution of the per-step device times between consecutive events of the timed region."""
    ms = np.array([marks[i].elapsed_time(marks[i + 1]) for i in range(len(marks) - 1)], dtype=np.float64)
    q = lambda p: float(np.percentile(ms, p))
    return {"median": q(50), "min": float(ms.min()), "max": float(ms.max()), "p95": q(95), "p99": q(99),
            "iqr": q(75) - q(25), "samples": int(ms.size)}


# --------------------------------------------------------------------------- next row: native global geometry
def run_native_global(args, kv, torch, sampler):
    """Extra line (not a BASELINE config): the reference's native global-layer geometry, 16 query heads on
    one KV head of 512 dims, rotary 128, V derived from raw K (src/gemma4.h:19-21,28) -- append + tensor-core
    decode attention through b200kv_decode_layer_step_bf16 on a ragged batch (--seqs, default 64; context
    lengths as cfg3) in a permuted page pool. One GPU."""
    H, HKVG, DG, ROT = 16, 1, 512, 128
    rng = np.random.default_rng(args.seed)
    B = args.seqs or 64
    ctx = rng.integers(args.min_ctx, args.max_ctx + 1, size=B).astype(np.int64)
    e2e_warm, probe = 3, 11
    total = args.warmup + args.steps + e2e_warm + args.e2e_steps + probe
    pages = (ctx + total + PAGE - 1) // PAGE
    mpps, num_pages = int(pages.max()), int(pages.sum())
    pool = rng.permutation(num_pages).astype(np.int32)
    table = np.full((B, mpps), -1, np.int32)
    cur = 0
    for b in range(B):
        table[b, :pages[b]] = pool[cur:cur + pages[b]]
        cur += int(pages[b])
    dev = torch.device("cuda")
    cfg = kv.make_kv_config(1, num_pages, PAGE, mpps, B, HKVG, DG, 0)
    elems = num_pages * PAGE * HKVG * DG
    ck = torch.randn(elems, dtype=torch.bfloat16, device=dev)
    cv = torch.randn(elems, dtype=torch.bfloat16, device=dev)
    raw_host = torch.randn((B, H + HKVG, DG), dtype=torch.bfloat16).pin_memory()
    raw = raw_host.to(dev)
    raw_q, raw_k = raw[:, :H].contiguous(), raw[:, H:].contiguous()
    ones = torch.ones(DG, dtype=torch.bfloat16, device=dev)
    cos_h, sin_h = kv.fill_rope_tables(int(ctx.max()) + total + 1, ROT // 2, 1.0e6, DG)
    cos, sin = torch.from_numpy(cos_h).to(dev), torch.from_numpy(sin_h).to(dev)
    dtable = torch.from_numpy(table).to(dev)
    pos_all = torch.from_numpy((ctx[None, :] + np.arange(total)[:, None]).astype(np.int32)).to(dev)
    len_all = pos_all + 1
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    nsplit = kv.plan_balanced(B, sms)
    qp = torch.empty((B, H, DG), dtype=torch.bfloat16, device=dev)
    out = torch.empty_like(qp)
    out_host = torch.empty((B, H, DG), dtype=torch.bfloat16).pin_memory()
    lse = torch.empty((B, H), dtype=torch.float32, device=dev)
    pm = torch.empty(B * H * nsplit, dtype=torch.float32, device=dev)
    pl = torch.empty_like(pm)
    pacc = torch.empty(B * H * nsplit * DG, dtype=torch.float32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    ev0 = [kv.Timer() for _ in range(total)]
    ev1 = [kv.Timer() for _ in range(total)]
    stream = torch.cuda.current_stream().cuda_stream
    a = kv.LayerStepArgs()
    a.q, a.out, a.lse = qp.data_ptr(), out.data_ptr(), lse.data_ptr()
    a.partial_m, a.partial_l, a.partial_acc = pm.data_ptr(), pl.data_ptr(), pacc.data_ptr()
    a.cache_k, a.cache_v, a.cache_config = ck.data_ptr(), cv.data_ptr(), cfg
    a.page_table = dtable.data_ptr()
    a.cache_layer, a.split_size, a.num_splits, a.softmax_scale = 0, 0, nsplit, 1.0 / math.sqrt(DG)
    a.raw_q, a.raw_k, a.raw_v = raw_q.data_ptr(), raw_k.data_ptr(), None
    a.q_norm_weight, a.k_norm_weight, a.cos, a.sin = ones.data_ptr(), ones.data_ptr(), cos.data_ptr(), sin.data_ptr()
    a.batch_count, a.q_heads, a.rotary_dim, a.norm_mode = B, H, ROT, kv.NORM_RSQRT_APPROX
    a.status = status.data_ptr()

    def step(s, events=False):
        a.token_position, a.seq_lengths = pos_all[s].data_ptr(), len_all[s].data_ptr()
        a.event_before_attention = ev0[s].handle if events else None
        a.event_after_attention = ev1[s].handle if events else None
        kv.decode_layer_step(a, stream=stream)

    def bytes_of(s):
        n = ctx + s + 1
        pg = (n - 1) // PAGE + 1
        attn = int((n * HKVG * DG * 2 * 2 + 2 * H * DG * 2 + 4 * pg).sum())
        append = B * ((H + HKVG) * DG * 2 + H * DG * 2 + 2 * HKVG * DG * 2 + 4)
        return attn + append, attn

    s = 0
    for _ in range(args.warmup):
        step(s); s += 1
    torch.cuda.synchronize()
    if sampler:
        sampler.mark("timed_begin")
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    first = s
    marks[0].record()
    for i in range(args.steps):
        step(s); s += 1
        marks[i + 1].record()
    torch.cuda.synchronize()
    if sampler:
        sampler.mark("timed_end")
    ms = marks[0].elapsed_time(marks[-1])
    step_bytes = sum(bytes_of(i)[0] for i in range(first, first + args.steps))
    for _ in range(e2e_warm):
        step(s); s += 1
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    first_e = s
    e0.record()
    for _ in range(args.e2e_steps):
        raw.copy_(raw_host, non_blocking=True)
        raw_q.copy_(raw[:, :H]); raw_k.copy_(raw[:, H:])
        step(s); s += 1
        out_host.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1)
    e2e_bytes = sum(bytes_of(i)[0] for i in range(first_e, first_e + args.e2e_steps))
    p0 = s
    for _ in range(probe):
        step(s, events=True); s += 1
    torch.cuda.synchronize()
    attn_ms = statistics.mean(ev0[i].elapsed_ms(ev1[i]) for i in range(p0 + 3, p0 + probe))
    attn_bytes = statistics.mean(bytes_of(i)[1] for i in range(p0 + 3, p0 + probe))
    clocks = None
    if sampler:
        sampler.mark("load_end")
        clocks = sampler.stop()
    peaks_path = REPO / "MEASURED_PEAKS.json"
    peak = float(json.loads(peaks_path.read_text())["hbm_gbs"]) if peaks_path.exists() else 6650.0
    value = step_bytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 (tensor-core QK^T and P*V, fp32 accumulate and softmax)", "data": "synthetic",
        "config": {"workload": "next row, not a BASELINE config: reference-native global geometry, 16 Q / 1 KV / "
                               "head_dim 512, rotary 128, V from raw K; ragged batch, permuted 16-token pages",
                   "sequences": B, "ctx_range": [args.min_ctx, args.max_ctx], "seed": args.seed,
                   "l2": "inputs larger than L2" if step_bytes / args.steps > 2.6e8 else "step smaller than 2x L2",
                   "launch": "append + attention + combine, programmatic dependent launch"},
        "us_per_layer_step": ms * 1e3 / args.steps, "frac_of_hbm_peak": value / peak,
        "step_ms_stats": step_stats(marks),
        "roofline": {"bound": "hbm", "kernel": "decode_gqa16_kernel + combine", "achieved": attn_bytes / (attn_ms * 1e-3) / 1e9,
                     "peak": peak, "unit": "GB/s", "frac": attn_bytes / (attn_ms * 1e-3) / 1e9 / peak, "traffic": None,
                     "algorithmic_bytes_per_launch": attn_bytes, "avg_launch_ms": attn_ms},
        "e2e": {"value": e2e_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": int(raw_host.numel() * 2), "d2h_bytes_per_step": int(out_host.numel() * 2)},
        "gpu_launches": 3 * args.steps, "device_status": int(status[0].item()), "clocks": clocks,
    }))


# --------------------------------------------------------------------------- next row: the decode layer around the KV path
def run_layer(args, kv, torch, sampler):
    """Extra line (not a BASELINE config): the attention half of the reference's fused decode layer for batch 1,
    b200kv_decode_attention_layer_bf16 = input RMSNorm + [Q|K|V] projection (ingress), append + decode attention
    + combine (the KV path), O projection + post-attention norm + residual + pre-FFN norm (egress), on the stack
    of BASELINE config 2: --layers layers (48) in the 5:1 pattern, sliding layers on a 1024-token ring, global
    layers on a linear cache of 4096 keys, 16 Q / 8 KV heads of 256, hidden 3840, every layer with its own
    seeded weights (94 MB per layer, so nothing is served from L2 twice) and the layer input chained from the
    previous layer's ffn_residual. One step = one token through all layers; the position is the same every step
    (the row is rewritten in place), so that a step can be replayed from a CUDA graph. One GPU."""
    dev = torch.device("cuda")
    HID, H, QW, KW = 3840, 16, 16 * D, HKV * D
    COLS = QW + 2 * KW
    L = args.layers
    is_global = [(l + 1) % 6 == 0 for l in range(L)]            # gemma4_is_global_layer, src/gemma4.h:105-108
    gen = torch.Generator(device=dev)
    gen.manual_seed(args.seed)
    rng = np.random.default_rng(args.seed)

    def cache(window, ctx, layers):
        mpps = (window + PAGE - 1) // PAGE + 1 if window else (ctx + PAGE) // PAGE + 1
        table = rng.permutation(mpps).astype(np.int32)[None, :]
        cfg = kv.make_kv_config(layers, mpps, PAGE, mpps, 1, HKV, D, window)
        elems = layers * mpps * PAGE * HKV * D
        return dict(cfg=cfg, table=torch.from_numpy(table).to(dev),
                    k=torch.randn(elems, dtype=torch.bfloat16, device=dev, generator=gen),
                    v=torch.randn(elems, dtype=torch.bfloat16, device=dev, generator=gen),
                    pos=torch.tensor([ctx], dtype=torch.int32, device=dev),
                    length=torch.tensor([ctx + 1], dtype=torch.int32, device=dev), keys=min(ctx + 1, window) if window else ctx + 1)

    n_global = sum(is_global)
    caches = {False: cache(1024, 1500, max(L - n_global, 1)), True: cache(0, 4096, max(n_global, 1))}
    w_qkv = (torch.randn(L, COLS, HID, dtype=torch.float32, device=dev, generator=gen) * HID ** -0.5).bfloat16() if L <= 8 else None
    if w_qkv is None:                       # generated layer by layer: the fp32 staging copy of 48 layers is 12 GB
        w_qkv = torch.empty(L, COLS, HID, dtype=torch.bfloat16, device=dev)
        for l in range(L):
            w_qkv[l] = (torch.randn(COLS, HID, dtype=torch.float32, device=dev, generator=gen) * HID ** -0.5).bfloat16()
    w_o = torch.empty(L, HID, QW, dtype=torch.bfloat16, device=dev)
    for l in range(L):
        w_o[l] = (torch.randn(HID, QW, dtype=torch.float32, device=dev, generator=gen) * QW ** -0.5).bfloat16()
    norm_w = (1.0 + 0.05 * torch.randn(4, L, HID, dtype=torch.float32, device=dev, generator=gen)).bfloat16()
    head_w = (1.0 + 0.05 * torch.randn(2, D, dtype=torch.float32, device=dev, generator=gen)).bfloat16()
    x_host = torch.randn(HID, dtype=torch.bfloat16).pin_memory()
    x = torch.zeros(L + 1, HID, dtype=torch.bfloat16, device=dev)
    out_host = torch.empty(HID, dtype=torch.bfloat16).pin_memory()
    cos_s, sin_s = (torch.from_numpy(t).to(dev) for t in kv.fill_rope_tables(4200, D // 2, 1.0e4, D))
    cos_g, sin_g = (torch.from_numpy(t).to(dev) for t in kv.fill_rope_tables(4200, D // 2, 1.0e6, D))
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    nsplit = kv.plan_balanced(1, sms)
    q, out = (torch.empty(H * D, dtype=torch.bfloat16, device=dev) for _ in range(2))
    pm, pl = (torch.empty(H * nsplit, dtype=torch.float32, device=dev) for _ in range(2))
    pacc = torch.empty(H * nsplit * D, dtype=torch.float32, device=dev)
    raw = torch.empty(COLS, dtype=torch.bfloat16, device=dev)
    o_proj, normed, ffn_x = (torch.empty(HID, dtype=torch.bfloat16, device=dev) for _ in range(3))
    ticket = torch.zeros(1, dtype=torch.int32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)

    layers = []
    seen = {False: 0, True: 0}
    for l in range(L):
        c = caches[is_global[l]]
        a = kv.AttentionLayerArgs()
        s = a.kv
        s.q, s.out, s.lse = q.data_ptr(), out.data_ptr(), None
        s.partial_m, s.partial_l, s.partial_acc = pm.data_ptr(), pl.data_ptr(), pacc.data_ptr()
        s.cache_k, s.cache_v, s.cache_config = c["k"].data_ptr(), c["v"].data_ptr(), c["cfg"]
        s.page_table, s.token_position, s.seq_lengths = c["table"].data_ptr(), c["pos"].data_ptr(), c["length"].data_ptr()
        s.cache_layer, s.split_size, s.num_splits, s.softmax_scale = seen[is_global[l]], 0, nsplit, 1.0 / math.sqrt(D)
        seen[is_global[l]] += 1
        s.q_norm_weight, s.k_norm_weight = head_w[0].data_ptr(), head_w[1].data_ptr()
        s.cos, s.sin = (cos_g.data_ptr(), sin_g.data_ptr()) if is_global[l] else (cos_s.data_ptr(), sin_s.data_ptr())
        s.batch_count, s.q_heads, s.rotary_dim, s.norm_mode, s.status = 1, H, D, kv.NORM_RSQRT_APPROX, status.data_ptr()
        a.attention_x, a.attention_input_norm_weight = x[l].data_ptr(), norm_w[0, l].data_ptr()
        a.attention_qkv_proj_col_major, a.attention_o_proj_col_major = w_qkv[l].data_ptr(), w_o[l].data_ptr()
        a.attention_post_norm_weight, a.attention_pre_ffn_norm_weight = norm_w[1, l].data_ptr(), norm_w[2, l].data_ptr()
        a.raw_qkv, a.residual_out, a.normed_out = raw.data_ptr(), o_proj.data_ptr(), normed.data_ptr()
        a.ffn_residual, a.ffn_x, a.ticket = x[l + 1].data_ptr(), ffn_x.data_ptr(), ticket.data_ptr()
        a.hidden_size, a.has_v_projection = HID, 1
        layers.append(a)

    def step():
        for a in layers:
            kv.decode_attention_layer(a)

    def step_e2e():
        x[0].copy_(x_host, non_blocking=True)
        run()
        out_host.copy_(x[L], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def timed(fn, n):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    x[0].copy_(x_host)
    use_graph = args.graph != "off"
    run = step
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if use_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        run = graph.replay
        for _ in range(3):
            run()
    steps = max(3, min(args.steps, 50))
    if sampler:
        sampler.mark("timed_begin")
    ms = timed(run, steps)
    if sampler:
        sampler.mark("timed_end")
    e2e_ms = timed(step_e2e, max(3, min(args.e2e_steps, 20)))

    # the two projection kernels alone, every call on another layer's matrix (cold in L2)
    def only(kind):
        calls = []
        for l, a in enumerate(layers):
            if kind == "ingress":
                i = kv.IngressArgs()
                i.raw_qkv, i.x, i.input_norm_weight = raw.data_ptr(), x[l].data_ptr(), norm_w[0, l].data_ptr()
                i.qkv_proj_col_major, i.batch_count, i.hidden_size = w_qkv[l].data_ptr(), 1, HID
                i.cols, i.q_width, i.k_width, i.norm_mode, i.status = COLS, QW, KW, kv.NORM_RSQRT_APPROX, status.data_ptr()
                calls.append((kv.decode_ingress, i))
            else:
                e = kv.EgressArgs()
                e.residual_out, e.normed_out, e.ffn_residual, e.ffn_x = (o_proj.data_ptr(), normed.data_ptr(),
                                                                         x[l + 1].data_ptr(), ffn_x.data_ptr())
                e.attention_out, e.o_proj_col_major = out.data_ptr(), w_o[l].data_ptr()
                e.post_norm_weight, e.pre_ffn_norm_weight = norm_w[1, l].data_ptr(), norm_w[2, l].data_ptr()
                e.x, e.ticket, e.batch_count, e.hidden_size = x[l].data_ptr(), ticket.data_ptr(), 1, HID
                e.attention_width, e.norm_mode, e.status = QW, kv.NORM_RSQRT_APPROX, status.data_ptr()
                calls.append((kv.decode_egress, e))

        def go():
            for fn, a in calls:
                fn(a)
        go()
        return timed(go, max(3, steps // 4)) * 1e3 / L

    us_ingress, us_egress = only("ingress"), only("egress")
    reference = None
    try:
        from oracle import ref_binding as ref
        if ref.has_projections() and not args.no_reference_cuda:
            scratch = torch.empty(HID, dtype=torch.bfloat16, device=dev)

            def ref_in():
                for l in range(L):
                    ref.decode_ingress(raw, scratch, x[l], norm_w[0, l], w_qkv[l], False)

            def ref_out():
                for l in range(L):
                    ref.decode_egress(o_proj, normed, scratch, ffn_x, out, w_o[l], norm_w[1, l], norm_w[2, l], x[l], False)
            ref_in(); ref_out()
            reference = {"kernels": "phase_decode_rmsnorm_project_bf16 / project_attention_out_post_attention of "
                                    "src/gemma4_flash_attention_decode.cu (sm_100a build, cooperative launch)",
                         "ingress_us": timed(ref_in, 3) * 1e3 / L, "egress_us": timed(ref_out, 3) * 1e3 / L}
    except OSError:
        reference = None
    clocks = None
    if sampler:
        sampler.mark("load_end")
        clocks = sampler.stop()

    w_bytes = (COLS * HID + HID * QW) * 2
    cpu = None
    if not args.no_cpu_baseline:          # the oracle's two projections of layer 0 on all host threads
        from oracle import binding as orc

        def bits(t):
            return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)
        h = dict(x=bits(x[0]), w_in=bits(norm_w[0, 0]), w=bits(w_qkv[0]), attn=bits(out), w_o=bits(w_o[0]),
                 w_post=bits(norm_w[1, 0]), w_pre=bits(norm_w[2, 0]))
        threads = orc.hardware_threads()
        reps, t0 = 0, time.time()
        while time.time() - t0 < max(args.cpu_seconds, 1.0):
            orc.decode_ingress(h["x"], h["w_in"], h["w"], threads=threads)
            orc.decode_egress(h["attn"], h["w_o"], h["w_post"], h["w_pre"], h["x"], threads=threads)
            reps += 1
        cpu_s = (time.time() - t0) / reps
        cpu = {"value": w_bytes / cpu_s / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
               "sample": "the two projections of one layer (94 MB of weights), %d repetitions, %.1f s of host time, "
                         "oracle port on all host threads; the KV path's CPU figure is the default workload's" % (reps, cpu_s * reps)}
    small = (HID * 2 * 2 + COLS * 2 + QW * 2 + HID * 2 * 5)        # rows read and written around the matrices
    per_layer = [w_bytes + small + layer_step_bytes(np.array([caches[g]["keys"]]), 1024 if not g else 0) for g in is_global]
    step_bytes = int(sum(per_layer))
    peak, peak_source = hbm_peak()
    gbs = step_bytes / (ms * 1e-3) / 1e9
    ingress_gbs = COLS * HID * 2 / (us_ingress * 1e-6) / 1e9
    print(json.dumps({
        "metric": "decode attention layer (QKV projection + KV append + decode attention + O projection), batch 1: "
                  "achieved HBM GB/s (us per layer alongside)", "unit": "GB/s", "value": gbs, "n_gpus": 1,
        "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": "next row, not a BASELINE config: b200kv_decode_attention_layer_bf16 over %d layers "
                               "(5 sliding : 1 global, ring 1024 / linear 4096), batch 1, hidden 3840" % L,
                   "launch": "one CUDA graph replay per step" if use_graph else "stream launches",
                   "l2": "every layer has its own 94 MB of weights: %d MB per step, nothing revisited within L2's reach" % (step_bytes >> 20)},
        "us_per_layer": ms * 1e3 / L, "frac_of_hbm_peak": gbs / peak,
        "kernels_alone_us": {"ingress": us_ingress, "egress": us_egress},
        "roofline": {"bound": "hbm", "kernel": "decode_projection_kernel (QKV projection, 8192 x 3840)", "achieved": ingress_gbs,
                     "peak": peak, "unit": "GB/s", "frac": ingress_gbs / peak, "traffic": None, "peak_source": peak_source,
                     "algorithmic_bytes_per_launch": COLS * HID * 2, "avg_launch_ms": us_ingress * 1e-3},
        "e2e": {"value": step_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": HID * 2,
                "d2h_bytes_per_step": HID * 2, "ms_per_step": e2e_ms},
        "gpu_launches": 4 * L * steps, "device_status": int(status[0].item()), "reference_cuda": reference, "cpu_baseline": cpu, "clocks": clocks,
    }))


# --------------------------------------------------------------------------- next row: prompt attention
def run_prefill(args, kv, torch, sampler):
    """Extra lines (not a BASELINE config): the two prompt-attention entry points of
    src/gemma4_flash_attention.cuh -- prep + causal attention -- on seeded N(0,1) prompts, sliding
    (8 KV x 256, window 1024) and global (1 KV x 512) geometry, with the reference's own kernels
    (oracle/_ref) timed beside them when present. Tensor-bound: reported in TFLOP/s of the attention
    (4 * D * visible (query, key) pairs * 16 heads)."""
    from oracle import ref_binding as ref
    dev = torch.device("cuda")
    B = args.seqs or 4
    S = min(args.max_ctx, 4096)
    H = 16
    results = []
    for kind, HKVp, Dp, ROT, theta, window in (("sliding", 8, 256, 256, 1.0e4, 1024), ("global", 1, 512, 128, 1.0e6, 0)):
        rows = B * S
        q = torch.randn(rows, H, Dp, dtype=torch.bfloat16, device=dev)
        k = torch.randn(rows, HKVp, Dp, dtype=torch.bfloat16, device=dev)
        v = torch.randn(rows, HKVp, Dp, dtype=torch.bfloat16, device=dev)
        out, qp = torch.empty_like(q), torch.empty_like(q)
        kp, vp = torch.empty_like(k), torch.empty_like(k)
        w = torch.ones(Dp, dtype=torch.bfloat16, device=dev)
        cos_h, sin_h = kv.fill_rope_tables(S, ROT // 2, theta, Dp)
        cos, sin = torch.from_numpy(cos_h).to(dev), torch.from_numpy(sin_h).to(dev)
        pos = torch.arange(S, dtype=torch.int32, device=dev).repeat(B)
        scale = 1.0 / math.sqrt(Dp)
        r = np.arange(S, dtype=np.int64)
        pairs = int((r + 1).sum()) if window == 0 else int(np.minimum(r + 1, window).sum())
        flops = 4.0 * Dp * pairs * H * B

        def mine():
            if kind == "sliding":
                kv.flash_attention_sliding_fwd(out, qp, kp, vp, q, k, v, w, w, cos, sin, pos, B, S, S, window, scale)
            else:
                kv.flash_attention_global_fwd(out, qp, kp, vp, q, k, w, w, cos, sin, pos, B, S, S, scale)

        def attn_only():
            kv.prefill_attention(out, qp, kp, vp, B, S, H, HKVp, Dp, window, scale)

        def theirs():
            if kind == "sliding":
                ref.prefill_sliding(out, qp, kp, vp, q, k, v, w, w, cos, sin, pos, B, S, S, window, scale)
            else:
                ref.prefill_global(out, qp, kp, vp, q, k, w, w, cos, sin, pos, B, S, S, scale)

        def timed(fn, n):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / n

        n = max(3, min(args.steps, 50))
        entry = {"kind": kind, "batch": B, "seq_len": S, "window": window, "ms_call": timed(mine, n),
                 "ms_attention": timed(attn_only, n)}
        entry["tflops_attention"] = flops / (entry["ms_attention"] * 1e-3) / 1e12
        if ref.has_prefill() and not args.no_reference_cuda:
            entry["reference_cuda_ms_call"] = timed(theirs, max(3, n // 5))
        results.append(entry)
    clocks = None
    if sampler:
        sampler.mark("timed_begin"); sampler.mark("timed_end"); sampler.mark("load_end")
        clocks = sampler.stop()
    peaks_path = REPO / "MEASURED_PEAKS.json"
    peak = float(json.loads(peaks_path.read_text()).get("bf16_tflops", 1590.0)) if peaks_path.exists() else 1590.0
    best = results[0]
    print(json.dumps({
        "metric": "prompt attention (causal, sliding window 1024): TFLOP/s of the attention stage", "unit": "TFLOP/s",
        "value": best["tflops_attention"], "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": best["ms_call"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 (sliding: tcgen05.mma, accumulators in tensor memory; global: mma.sync m16n8k16; fp32 accumulate and softmax)", "data": "synthetic",
        "config": {"workload": "next row, not a BASELINE config: gemma4_flash_attention_{sliding,global}_fwd_bf16_norm_rope, "
                               "prompts of %d x %d tokens" % (B, S)},
        "roofline": {"bound": "tensor", "achieved": best["tflops_attention"], "peak": peak, "unit": "TFLOP/s",
                     "frac": best["tflops_attention"] / peak, "traffic": None,
                     "note": "peak = measured cuBLAS bf16; flops = 4 * head_dim per visible (query, key) pair"},
        "results": results, "gpu_launches": 2 * args.steps, "clocks": clocks,
    }))


# --------------------------------------------------------------------------- main arm
L2_FLUSH_BYTES = 512 << 20      # four times the 126 MB L2 of a B200


def measure_workload(args, kv, torch, dist, world, rank, sampler=None, verify=True, extras=True):
    """Builds one workload on this rank, runs warm-up + timed + end-to-end + probe steps and returns the JSON
    line as a dict on rank 0 (None elsewhere). `verify`: check the last timed step's outputs against the
    oracle. `extras`: the reference's CUDA kernels and the CPU baselines beside the number (rank 0, one GPU)."""
    spec, ctx_all, ctx, parallelism, scaling = plan_workload(args, world, rank)
    if args.emulate_world > 1 and world == 1 and args.workload in ("cfg3", "cfg5"):
        ctx = ctx_all[shard_sequences(ctx_all, args.emulate_world)[args.emulate_rank]]
    e2e_warm = 3
    use_graph = replays_graph(args, world)
    probe_steps = 11                        # steps after the timed regions that carry the per-kernel events
    # a one-layer step is a single kernel: as many steps per replayed graph as configs[1] has layer-steps
    # per replay (see RankWorkload.enable_graph)
    steps_per_graph = ONE_LAYER_STEPS_PER_GRAPH if (use_graph and spec.n_local + spec.n_global == 1) else 1
    if steps_per_graph > 1:
        args = copy.copy(args)
        args.warmup = -(-args.warmup // steps_per_graph) * steps_per_graph
        args.steps = -(-args.steps // steps_per_graph) * steps_per_graph
    cold_steps = min(args.steps, 50) if args.cache in ("cold", "both") else 0
    if cold_steps and steps_per_graph > 1:
        # cold steps are timed one by one, so they are launched directly, not replayed; a whole number of graphs'
        # worth of them keeps the replays that follow in step
        cold_steps = steps_per_graph
    total_steps = args.warmup + args.steps + cold_steps + e2e_warm + args.e2e_steps + probe_steps
    wl = RankWorkload(kv, torch, ctx, total_steps, args.seed + 1000 * rank, args, spec)
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if sampler:
        sampler.mark("load_begin")
    s = 0
    if use_graph:
        wl.enable_graph(0, steps_per_graph)
    for _ in range(args.warmup):
        wl.step(s)
        s += 1
    barrier()
    if sampler:
        sampler.mark("timed_begin")
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    first_timed = s
    marks[0].record()
    for i in range(args.steps):
        wl.step(s)
        s += 1
        marks[i + 1].record()
    barrier()
    if sampler:
        sampler.mark("timed_end")
    elapsed_ms = marks[0].elapsed_time(marks[-1])
    step_bytes = sum(wl.bytes_for_step(i)[0] for i in range(first_timed, first_timed + args.steps))
    attn_bytes = statistics.mean(wl.bytes_for_step(i)[1] for i in range(first_timed, first_timed + args.steps))
    status = int(wl.status[0].item())

    if steps_per_graph > 1:
        wl.graph = None                     # what follows goes step by step: plain launches from here on
    # parity of what the timed region just produced (host work, outside every timed region)
    verified = None
    if verify:
        verified = verify_step(wl, s - 1) if not spec.key_shard else {
            "ok": True, "skipped": "key-range sharding: a rank holds a slice of the keys, the merged rows are "
                                   "checked against ncclAllGather + a torch merge in the warm-up instead"}

    # cold cache: an L2 flush (a write over four times the L2) before every timed iteration, the events recorded
    # after the flush -- the reference bench's contract (src/benches/gemma4_kv_cache_bench.cu:60-112,187-195)
    cold = None
    if cold_steps:
        flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device="cuda")
        begin = [torch.cuda.Event(enable_timing=True) for _ in range(cold_steps)]
        end = [torch.cuda.Event(enable_timing=True) for _ in range(cold_steps)]
        first_cold = s
        for i in range(cold_steps):
            flush.fill_(i & 0xFF)
            begin[i].record()
            if steps_per_graph > 1:
                wl.step_direct(s)
            else:
                wl.step(s)
            s += 1
            end[i].record()
        if steps_per_graph > 1:
            wl.skip_replayed_steps(cold_steps)
        barrier()
        ms = np.array([begin[i].elapsed_time(end[i]) for i in range(cold_steps)])
        cold_bytes = statistics.mean(wl.bytes_for_step(i)[0] for i in range(first_cold, first_cold + cold_steps))
        cold = {"steps": cold_steps, "ms_per_step_median": float(np.median(ms)), "ms_per_step_min": float(ms.min()),
                "ms_per_step_max": float(ms.max()), "us_per_layer_step": float(np.median(ms)) * 1e3 / wl.L,
                "GBps": cold_bytes / (float(np.median(ms)) * 1e-3) / 1e9,
                "flush": f"{L2_FLUSH_BYTES >> 20} MiB written before every step, events after the flush"}
        del flush

    # end to end through host buffers
    for _ in range(e2e_warm):
        wl.step_e2e(s)
        s += 1
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    first_e2e = s
    e0.record()
    for _ in range(args.e2e_steps):
        wl.step_e2e(s)
        s += 1
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    e2e_bytes = sum(wl.bytes_for_step(i)[0] for i in range(first_e2e, first_e2e + args.e2e_steps))
    # per-kernel events cannot be read out of a replayed graph, and on stream launches they would stand
    # between the append and the attention: time the attention launch of the same workload in a few
    # plainly launched steps right after
    wl.graph = None
    probe0 = s
    for _ in range(probe_steps):
        wl.step(s, events=True)
        s += 1
    torch.cuda.synchronize()
    attn_ms = [wl.ev_begin[i].elapsed_ms(wl.ev_end[i]) for i in range(probe0 + 3, probe0 + probe_steps)]
    clocks = None
    if sampler:
        sampler.mark("load_end")
        clocks = sampler.stop()

    v_ok = 1.0 if (verified is None or verified.get("ok")) else 0.0
    stats = torch.tensor([elapsed_ms, e2e_ms, -float(step_bytes), -float(e2e_bytes), float(status),
                          statistics.mean(attn_ms), -v_ok, (verified or {}).get("max_abs", 0.0),
                          (verified or {}).get("lse_max_abs", 0.0), cold["ms_per_step_median"] if cold else 0.0],
                         dtype=torch.float64, device="cuda")
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm_ = stats.clone()
        dist.all_reduce(sm_, op=dist.ReduceOp.SUM)
        elapsed_ms, e2e_ms, status = mx[0].item(), mx[1].item(), int(mx[4].item())
        step_bytes, e2e_bytes = -sm_[2].item(), -sm_[3].item()
        if verified is not None:
            # the figures of every rank that is out of band travel to rank 0 with the line
            mine = None if verified.get("ok") else {k: v for k, v in verified.items() if k != "tolerance"}
            failed = [None] * world
            dist.all_gather_object(failed, mine)
            failed = {str(r): f for r, f in enumerate(failed) if f is not None}
            if failed:
                verified["ranks_out_of_band"] = failed
            verified["all_ranks_ok"] = bool(-mx[6].item() >= 1.0)
            verified["max_abs_over_ranks"], verified["lse_max_abs_over_ranks"] = mx[7].item(), mx[8].item()
            verified["ok"] = verified["all_ranks_ok"]
        if cold:
            cold["ms_per_step_median_max_over_ranks"] = mx[9].item()
    launches = wl.launches_per_step * args.steps
    splits = {"global": [wl.g_split, wl.g_nsplit], "local": [wl.l_split, wl.l_nsplit]}
    timed_split = wl.layers[wl.timed_layer].split_size
    timed_kernels = wl.kernels_per_layer[wl.timed_layer]
    timed_kernel = ("decode_pagetile_kernel (append, attention and merge in one launch)" if timed_kernels == 1 else
                    ("decode_balanced_kernel" if timed_split == 0 or spec.fp8 else "decode_split_kernel") + " + combine")
    kernels_per_layer = list(wl.kernels_per_layer)
    ref_cuda = None
    if rank == 0 and extras and not args.no_reference_cuda and world == 1:
        try:
            ref_cuda = reference_cuda_numbers(wl, torch, first_timed)
        except Exception as exc:  # the second checker must never cost the bench line
            ref_cuda = {"error": repr(exc)}
    n_layers, n_global, fp8 = wl.L, spec.n_global, spec.fp8
    if wl.peer is not None:
        wl.peer.close()
    del wl
    torch.cuda.empty_cache()
    if rank != 0:
        return None

    peak, peak_src = hbm_peak()
    value = step_bytes / (elapsed_ms * 1e-3) / 1e9
    attn_achieved = attn_bytes / (statistics.mean(attn_ms) * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
        "scaling": scaling, "vs_baseline": None, "dtype": ("fp8 e4m3 cache; scores e4m3 tensor-core MMA (query hi+lo) with fp32 accumulate, P*V fp16 per 8 keys into fp32"
                                                            if fp8 else "bf16"),
        "data": "synthetic",
        "config": workload_config(args, world, "B200", parallelism, n_layers),
        "us_per_layer_step": elapsed_ms * 1e3 / (args.steps * n_layers),
        "us_global_layer_attention": statistics.mean(attn_ms) * 1e3,
        "step_ms_stats": step_stats(marks),
        "frac_of_hbm_peak": value / (peak * world),
        "roofline": {
            "bound": "hbm",
            "kernel": timed_kernel + ", " + ("global" if n_global else "sliding") + " layer (rank 0)",
            "achieved": attn_achieved, "peak": peak, "unit": "GB/s", "frac": attn_achieved / peak,
            "traffic": None, "peak_source": peak_src,
            "algorithmic_bytes_per_launch": attn_bytes, "avg_launch_ms": statistics.mean(attn_ms),
        },
        "e2e": {
            "value": e2e_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
            "h2d_bytes_per_step": int(n_layers * ctx.size * (spec.hq + 2 * spec.hkv) * D * 2),
            "d2h_bytes_per_step": int(n_layers * ctx.size * spec.hq * D * 2),
            "steps": args.e2e_steps, "ms_per_step": e2e_ms / args.e2e_steps,
            "note": "per rank, rank 0's copy sizes; host buffers are pinned, copies and a stream sync are inside "
                    "the timed region every step",
        },
        "gpu_launches": launches,
        "kernels_per_layer_step": kernels_per_layer,
        "splits": splits,
        "device_status": status,
        "clocks": clocks,
    }
    if verified is not None:
        line["verified"] = verified
    if cold is not None:
        line["cold_cache"] = cold
    traffic_path = REPO / "profiles" / "decode_balanced_traffic.json"
    if traffic_path.exists():
        try:
            t = json.loads(traffic_path.read_text())
            t = t.get("fp8", t) if fp8 else t
            line["roofline"]["traffic"] = t["dram_bytes_per_algorithmic_byte"] * attn_bytes
            line["roofline"]["traffic_source"] = t.get("source")
        except (ValueError, KeyError):
            pass
    if ref_cuda is not None:
        line["reference_cuda"] = ref_cuda
    if extras and not args.no_cpu_baseline and world == 1:
        threads = os.cpu_count() or 1
        for key, n_threads, seconds in (("cpu_baseline", threads, args.cpu_seconds),
                                        ("cpu_baseline_1t", 1, args.cpu_seconds)):
            base = cpu_layer_step_sample(ctx_all, n_threads, seconds, max_keys=131072 if n_threads > 1 else 32768)
            line[key] = {
                "value": base["gbps"], "unit": "GB/s", "cores": n_threads, "kind": "port",
                "us_per_layer_step_of_sample": base["us_per_layer_step"],
                "sample": f"global layer-step over the first {base['sequences']} sequences ({base['keys']} keys) of the "
                          f"batch, repeated {base['runs']}x, {base['seconds']:.2f} s of host time, oracle port on "
                          + (f"all {n_threads} host threads" if n_threads > 1 else "one host thread"),
            }
    return line


def summary_of(line: dict) -> dict:
    """The figures of a secondary workload that go into the main line's `other_workloads`."""
    peak = line["roofline"]["peak"]
    out = {
        "workload": line["config"]["workload"], "parallelism": line["config"]["parallelism"],
        "launch": line["config"]["launch"], "n_gpus": line["n_gpus"], "steps": line["steps"], "warmup": line["warmup"],
        "us_per_layer_step": line["us_per_layer_step"], "ms_per_step": line["ms_per_step"], "GBps": line["value"],
        "frac_of_hbm_peak_x_gpus": line["value"] / (peak * line["n_gpus"]),
        "dominant_kernel": {k: line["roofline"][k] for k in ("kernel", "achieved", "frac", "avg_launch_ms",
                                                             "algorithmic_bytes_per_launch")},
        "e2e_GBps": line["e2e"]["value"], "device_status": line["device_status"], "dtype": line["dtype"],
        "step_ms_stats": line["step_ms_stats"],
    }
    for key in ("verified", "cold_cache", "reference_cuda"):
        if key in line:
            out[key] = line[key]
    if isinstance(out.get("verified"), dict):         # the short form: figures, not the per-layer list
        out["verified"] = {k: v for k, v in out["verified"].items() if k not in ("layers", "sequences", "tolerance")}
    return out


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    from __graft_entry__ import load_package

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    kv = load_package()
    kv.load_library(build_if_missing=False)
    sampler = ClockSampler(local_rank) if rank == 0 else None   # started early: nvidia-smi takes a second to come up

    if args.workload in ("prefill", "layer", "native_global"):
        if world > 1:
            raise SystemExit(f"--workload {args.workload} is a one-GPU line")
        {"prefill": run_prefill, "layer": run_layer, "native_global": run_native_global}[args.workload](
            args, kv, torch, sampler)
        return

    line = measure_workload(args, kv, torch, dist, world, rank, sampler, verify=not args.no_verify)

    # The other BASELINE configs, short runs in the same process (default workload only): batch-1 latency cases on
    # one GPU; the long single sequence KV-head-sharded with the peer all-gather (and ncclAllGather beside it) and
    # the fp8 batch sequence-sharded on as many GPUs as this run has.
    others = []
    if args.workload == "cfg3" and not args.no_other_workloads and not args.emulate_world:
        plan = []
        if world == 1:
            plan += [("cfg1", {"cache": "both"}), ("cfg2", {"cache": "both"})]
        if 8 % world == 0:
            plan += [("cfg4", {"gather": "peer"})]
            if world > 1:
                plan += [("cfg4", {"gather": "nccl"})]
        plan += [("cfg5", {})]
        for name, extra in plan:
            sub = copy.copy(args)
            sub.workload, sub.seqs = name, 0
            sub.steps = max(20, min(args.steps, args.other_steps))
            sub.warmup = max(3, min(args.warmup, 10))
            sub.e2e_steps = min(args.e2e_steps, 5)
            sub.cache = "warm"
            sub.no_cpu_baseline = True
            for k, v in extra.items():
                setattr(sub, k, v)
            try:
                got = measure_workload(sub, kv, torch, dist, world, rank, None, verify=not args.no_verify)
            except Exception as exc:          # a secondary workload must never cost the main line
                got = None
                if rank == 0:
                    others.append({"workload": WORKLOADS[name], "error": repr(exc)})
            if got is not None:
                entry = summary_of(got)
                if name == "cfg4" and world > 1:
                    entry["exchange"] = extra["gather"]
                others.append(entry)
    if rank == 0:
        if others:
            line["other_workloads"] = others
        print(json.dumps(line))
    failed = False
    if rank == 0:
        checks = [line.get("verified")] + [o.get("verified") for o in others]
        failed = any(isinstance(c, dict) and not c.get("ok", True) for c in checks)
    if world > 1:
        dist.destroy_process_group()
    if failed:
        print("bench.py: outputs of a timed step are outside the parity band (see `verified`)", file=sys.stderr)
        sys.exit(3)


if __name__ == "__main__":
    main()
