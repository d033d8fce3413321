#!/usr/bin/env python
"""Benchmark of the NVFP4 linear op (OP_GEMM_F4) on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--case NAME]

One "step" is one pass of the hot path over one batch of synthetic input:

  N = 1   the decode sweep: M in {1,2,4,8,16} on gate+up (K=5120 -> N=34816) and
          down (K=17408 -> N=5120); ten ops, each on its own copy of the weights
          (750 MB per step, larger than L2), replayed as one captured graph (the
          engine runs the ten independent ops as one persistent group launch).
          value = packed weight bytes (payload + block scales) / time, GB/s: the
          median of REPEATS timed regions of --steps steps each, min and max beside it.
  N > 1   the same ten ops, every one split along N over the ranks (strong scaling):
          per rank one group launch whose epilogue stores every output tile into
          all ranks' copies, then a barrier kernel.  value = whole-weight bytes /
          time, GB/s.  The tensor-parallel linears of config 4 (gate+up and the LM
          head at M=32 and M=8192) are in "tp" at every N.

The JSON line also carries the prefill GEMM sweep ("prefill": TFLOP/s against
the dense bf16 tensor roofline), the 64-layer decode step ("decode_step"), the
like-for-like tensor-parallel series at every N ("tp"), the end-to-end number
through the host-buffer C-ABI call ("e2e"), the roofline of the dominant
kernel and the reference CPU kernel timed on this host ("cpu_baseline").  In "tp"
the prefill exchange is timed in both forms the library has (the epilogue's peer
stores, the copy engines) and the faster one is the figure ("prefill_exchange").

--case NAME runs one workload alone and prints its own line: single kernels for
profiling (decode, group, sweep, prefill, prefill_tail, ...), "tp" (the
tensor-parallel series at any number of ranks), "planner_layers8" (eight layers
in the reference planner's op order) and "chain_timeline" (time stamps from inside
dependent launches; needs a library built with -DMMB_MEASURE_MODES).

Synthetic data: weights N(0, 0.02) seed 0 packed by the library's packer,
activations N(0, 1) seed 1 rounded to bf16.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "NVFP4 linear: decode GEMV weight GB/s vs HBM peak (prefill GEMM TFLOP/s in 'prefill')"
SHAPES = {  # name: (K, N)
    "gate_up": (5120, 34816), "down": (17408, 5120), "q": (5120, 6144), "k": (5120, 1024),
    "v": (5120, 1024), "o": (6144, 5120), "lm_head": (5120, 151936), "qkv": (5120, 8192),
}
DECODE_M = (1, 2, 4, 8, 16)
PREFILL_M = (512, 2048, 8192)
HBM_FALLBACK_GBS, TENSOR_FALLBACK_TFS = 6650.0, 1590.0
REPEATS = 7          # timed regions per headline number
# dram__bytes_read + dram__bytes_write over algorithmic bytes, from an ncu capture of the group
# kernel on two gate+up ops at M=1 and M=16; traffic grows with the weight bytes, so the
# per-launch figure of the sweep is this ratio times its algorithmic bytes.
GROUP_TRAFFIC_RATIO = 1.03


def wbytes(K, N):
    """packed payload + block scales"""
    return N * K // 2 + N * K // 16


def alg_bytes(M, K, N):
    """algorithmic bytes of one op: W (payload + scales + global scale) + x + y"""
    return wbytes(K, N) + 4 + 2 * M * K + 2 * M * N


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm": d["hbm_gbs"], "tensor_burst": d["bf16_tflops"],
                "tensor_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "src": "measured"}
    return {"hbm": HBM_FALLBACK_GBS, "tensor_burst": TENSOR_FALLBACK_TFS,
            "tensor_sustained": 1400.0, "src": "fallback"}


class Clocks:
    """Samples nvidia-smi every 200 ms while a timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path, self.t0 = index, None, None, None

    def __enter__(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.t0 = time.time()
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def samples(self):
        """(seconds since the sampler started, SM MHz, board W) per 200 ms sample."""
        out = []
        if not self.path or not os.path.exists(self.path):
            return out
        for i, line in enumerate(open(self.path)):
            f = [x.strip() for x in line.split(",")]
            try:
                out.append((0.2 * i, float(f[0]), float(f[2])))
            except (ValueError, IndexError):
                continue
        return out

    def summary(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "power_w_max": None, "samples": 0}
        if not self.path or not os.path.exists(self.path):
            return out
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1])); pw.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        os.unlink(self.path)
        if sm:
            busy = [s for s, p in zip(sm, pw) if p > 0.5 * max(pw)] or sm
            out.update(sm_mhz=statistics.median(busy), sm_max_mhz=max(mx), power_w_max=max(pw),
                       reasons=sorted(reasons), samples=len(sm))
        return out


# --------------------------------------------------------------------------- our arm
class Bench:
    def __init__(self, args):
        import torch
        import torch.distributed as dist
        import mimfer_b200 as mm
        self.torch, self.dist, self.mm, self.args = torch, dist, mm, args
        self.rank = int(os.environ.get("RANK", 0))
        self.world = int(os.environ.get("WORLD_SIZE", 1))
        self.local = int(os.environ.get("LOCAL_RANK", 0))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the NVFP4 kernels have no CPU path")
        torch.cuda.set_device(self.local)
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
        self.rt = mm.Runtime.get(self.local)
        self.dev = self.rt.device
        self._wcache = {}

    # -- helpers ---------------------------------------------------------------
    def weight(self, name, rows=None):
        """Host weight (cached), optionally a row shard; device copies are made per use."""
        K, N = SHAPES[name]
        if name not in self._wcache:
            self._wcache[name] = self.mm.make_weight(N, K, seed=0, std=0.02)
        w = self._wcache[name]
        return w if rows is None else w.rows(*rows)

    def dev_weight(self, w):
        return self.mm.NvFp4Weight(w.payload, w.scales, w.gs, w.N, w.K).to_device(self.dev)

    def acts(self, M, K):
        return self.rt.to_device_bf16(self.mm.make_activations(M, K, seed=1))

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def timed(self, fn, steps, warmup, repeats=1, stats=None):
        """ms per step: events on the compute stream, max over ranks.  With repeats > 1 the
        timed region of `steps` steps runs that many times and the median is returned;
        `stats` (a dict) receives median, min and max."""
        for _ in range(max(warmup, 3)):
            fn()
        vals = []
        for _ in range(max(1, repeats)):
            self.rt.sync()
            self.barrier()
            self.rt.time_begin()
            for _ in range(steps):
                fn()
            ms = self.rt.time_end()
            self.barrier()
            if self.world > 1:
                t = self.torch.tensor([ms], device=self.dev)
                self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
                ms = float(t.item())
            vals.append(ms / steps)
        status = self.rt.device_status()
        if status:
            raise RuntimeError(f"device status 0x{status:x} after timed region")
        med = statistics.median(vals)
        if stats is not None:
            stats.update(median=med, min=min(vals), max=max(vals), regions=len(vals), steps_per_region=steps)
        return med

    def engine(self, ops, overlap=False, group=True):
        """ops: list of (x, w_dev, y). Captured into one graph.  group: independent decode
        ops as persistent group launches (the engine's default); off, with `overlap`, the
        op-by-op forms."""
        eng = self.mm.LinearEngine(self.rt, max_ops=len(ops) + 1)
        eng.overlap(overlap)
        eng.group(group)
        for x, w, y in ops:
            eng.add(x, w, y)
        eng.launch()                  # direct dispatch once: errors surface per op
        self.rt.sync()
        eng.capture()
        return eng

    def empty(self, M, N):
        return self.torch.empty((M, N), dtype=self.torch.bfloat16, device=self.dev)

    # -- workloads -------------------------------------------------------------
    def decode_sweep(self, steps, warmup, ms_list=DECODE_M, names=("gate_up", "down"), per_op=False,
                     repeats=REPEATS, other_orders=True):
        ops, wb, ab = [], 0, 0
        for name in names:
            K, N = SHAPES[name]
            hw = self.weight(name)
            for M in ms_list:
                ops.append((self.acts(M, K), self.dev_weight(hw), self.empty(M, N)))
                wb += wbytes(K, N)
                ab += alg_bytes(M, K, N)
        pk = peaks()["hbm"]
        ms_serial = ms_ahead = float("nan")
        if other_orders:
            serial = self.engine(ops, group=False)          # op by op in list order, one kernel each
            ms_serial = self.timed(serial.launch, steps, warmup, repeats=3)
            serial.close()
            ahead = self.engine(ops, overlap=2, group=False)  # op by op, independent ops run ahead
            ms_ahead = self.timed(ahead.launch, steps, warmup, repeats=3)
            ahead.close()
        table = []
        if per_op:
            # one (op, M) at a time: as many ops of that shape as the sweep holds weight copies
            # of it (5 x 100 MB or 5 x 50 MB per step: larger than L2), one group launch
            for name in names:
                K, N = SHAPES[name]
                same = [o for o in ops if (o[1].K, o[1].N) == (K, N)]
                for M in ms_list:
                    x = self.acts(M, K)
                    grp = [(x, w, self.empty(M, N)) for _, w, _ in same]
                    e = self.engine(grp)
                    ms1 = self.timed(e.launch, steps, warmup, repeats=3) / len(grp)
                    e.close()
                    table.append({"op": name, "M": M, "us": round(ms1 * 1e3, 2),
                                  "weight_gbs": round(wbytes(K, N) / ms1 / 1e6),
                                  "frac": round(alg_bytes(M, K, N) / ms1 / 1e6 / pk, 3)})
        self.rt.lib.mm_f4_launch_count(1)
        eng = self.engine(ops)                            # the default: one persistent group launch
        per_capture = int(self.rt.lib.mm_f4_launch_count(1)) // 2      # issued once directly, once captured
        st = {}
        ms = self.timed(eng.launch, steps, warmup, repeats=repeats, stats=st)
        res = {"ms_per_step": ms, "weight_gbs": wb / ms / 1e6, "alg_gbs": ab / ms / 1e6,
               "ms_per_step_min": st["min"], "ms_per_step_max": st["max"], "timed_regions": st["regions"],
               "weight_gbs_min": wb / st["max"] / 1e6, "weight_gbs_max": wb / st["min"] / 1e6,
               "ops": len(ops), "weight_bytes": wb, "alg_bytes": ab, "group_launches": eng.n_group_launches(),
               "kernel_launches_per_step": per_capture,
               "serial_order": {"ms_per_step": ms_serial, "weight_gbs": wb / ms_serial / 1e6,
                                "what": "one kernel pair per op, in list order"},
               "run_ahead": {"ms_per_step": ms_ahead, "weight_gbs": wb / ms_ahead / 1e6,
                             "what": "one kernel per op, independent ops launched ahead of their predecessors"}}
        if table:
            res["per_op"] = table
        return res, ops, eng

    def decode_e2e(self, ops, eng, steps, warmup):
        """The same step through the host-buffer call of the engine: pinned host x
        in for every op, one graph replay, pinned host y out for every op, one
        synchronisation (mm_lin_engine_launch_host)."""
        torch = self.torch
        x_host = [x.cpu().pin_memory() for x, _, _ in ops]
        y_host = [torch.empty(y.shape, dtype=y.dtype).pin_memory() for _, _, y in ops]
        h2d = sum(t.numel() * 2 for t in x_host)
        d2h = sum(t.numel() * 2 for t in y_host)
        for _ in range(max(warmup, 3)):
            eng.launch_host(x_host, y_host)
        self.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            eng.launch_host(x_host, y_host)
        sec_unbound = (time.perf_counter() - t0) / steps
        # the same step with the copies captured into the graph (bound pinned buffers)
        bound = self.mm.LinearEngine(self.rt, max_ops=len(ops) + 1)
        for x, w, y in ops:
            bound.add(x, w, y)
        bound.upload_group((len(ops) + 2) // 3)    # three launches: copies of one overlap the kernels of the next
        bound.bind_host(x_host, y_host)
        bound.capture()
        for _ in range(max(warmup, 3)):
            bound.step_bound()
        self.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            bound.step_bound()
        sec = (time.perf_counter() - t0) / steps
        bound.close()
        # per-op form (mm_f4_linear_host: copy, op, copy, sync for every op), for the record
        per_op = [(xh, x, w, y, yh) for (x, w, y), xh, yh in zip(ops, x_host, y_host)]
        for xh, xd, w, yd, yh in per_op:
            self.rt.linear_host(xh, xd, w, yd, yh)
        t1 = time.perf_counter()
        for _ in range(max(2, steps // 4)):
            for xh, xd, w, yd, yh in per_op:
                self.rt.linear_host(xh, xd, w, yd, yh)
        sec_op = (time.perf_counter() - t1) / max(2, steps // 4)
        wb = sum(wbytes(w.K, w.N) for _, w, _ in ops)
        return {"value": wb / sec / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": sec * 1e3,
                "call": "mm_lin_engine_step_bound: one graph replay that uploads every op's activations "
                        "from pinned host memory on the transfer stream (one gather kernel per four ops), "
                        "runs the ten ops as three group launches (a launch per upload group, so that the "
                        "copies of one overlap the kernels of the next) and downloads every launch's outputs "
                        "to pinned host memory with one kernel; one sync",
                "copies_outside_graph": {"value": wb / sec_unbound / 1e9, "ms_per_step": sec_unbound * 1e3,
                                         "call": "mm_lin_engine_launch_host"},
                "per_op_sync": {"value": wb / sec_op / 1e9, "ms_per_step": sec_op * 1e3,
                                "call": "mm_f4_linear_host per op"},
                "timing": "host wall clock around synchronous calls"}

    def prefill_sweep(self, steps, warmup, ms_list=PREFILL_M, names=("gate_up", "down", "q", "k", "v", "o")):
        per, ops, flops = [], [], 0
        for name in names:
            K, N = SHAPES[name]
            w = self.dev_weight(self.weight(name))
            for M in ms_list:
                x, y = self.acts(M, K), self.empty(M, N)
                ops.append((x, w, y))
                f = 2.0 * M * N * K
                flops += f
                ms = self.timed(lambda: self.rt.linear_async(x, w, y), max(2, steps // 4), 3)
                per.append({"op": name, "M": M, "ms": round(ms, 4), "tflops": round(f / ms / 1e9, 1)})
        eng = self.engine(ops)
        ms = self.timed(eng.launch, max(2, steps // 4), 3)
        eng.close()
        return {"ms_per_step": ms, "tflops": flops / ms / 1e9, "ops": len(ops), "per_op": per}

    def decode_step_64(self, steps, warmup, layers=64, M=16, names=("q", "k", "v", "o", "gate_up", "down")):
        base = {n: self.weight(n) for n in names}
        ops, wb = [], 0
        for layer in range(layers):
            for n in names:
                K, N = SHAPES[n]
                # every op has its own weights and its own output: 384 independent linears
                ops.append((self.acts(M, K) if layer == 0 else ops[names.index(n)][0],
                            self.dev_weight(base[n]), self.empty(M, N)))
                wb += wbytes(K, N)
        eng = self.engine(ops, group=False)
        ms_serial = self.timed(eng.launch, max(2, steps // 2), 3)
        eng.close()
        eng = self.engine(ops, overlap=2, group=False)
        ms_ahead = self.timed(eng.launch, max(2, steps // 2), 3)
        ind = eng.n_independent()
        eng.close()
        self.rt.lib.mm_f4_launch_count(1)
        eng = self.engine(ops)
        launches = int(self.rt.lib.mm_f4_launch_count(1)) // 2
        st = {}
        ms = self.timed(eng.launch, max(2, steps // 2), 3, repeats=5, stats=st)
        groups = eng.n_group_launches()
        eng.close()
        return {"layers": layers, "M": M, "ops": len(ops), "weight_bytes": wb,
                "sum_linear_ms_per_step": ms, "weight_gbs": wb / ms / 1e6,
                "ms_min": st["min"], "ms_max": st["max"], "timed_regions": st["regions"],
                "group_launches": groups, "kernel_launches_per_step": launches,
                "serial_order": {"sum_linear_ms_per_step": ms_serial, "weight_gbs": wb / ms_serial / 1e6},
                "run_ahead": {"sum_linear_ms_per_step": ms_ahead, "weight_gbs": wb / ms_ahead / 1e6,
                              "independent_ops": ind}}

    def decode_step_planner(self, steps, warmup, layers=64, M=16):
        """The 64-layer decode step with the op sequence of the reference planner
        (src/plan/plan.c:223-247, 386-473): per layer q, k, v, o, gate, up,
        SILU_MUL, down - gate and up as separate tensors - run as emitted (8 ops
        per layer) and with the engine's MLP fusion (6 per layer).  down reads the
        SILU_MUL output."""
        K, inter = SHAPES["gate_up"][0], SHAPES["gate_up"][1] // 2
        full = self.weight("gate_up")
        lin = ("q", "k", "v", "o", "down")
        base = {n: self.weight(n) for n in lin}
        x = self.acts(M, K)
        xo = self.acts(M, SHAPES["o"][0])
        g, u, h = self.empty(M, inter), self.empty(M, inter), self.empty(M, inter)
        ys = {n: self.empty(M, SHAPES[n][1]) for n in lin}
        layer_w, keep, wb = [], [], 0
        for _ in range(layers):
            ws = {n: self.dev_weight(base[n]) for n in lin}
            wg, wu = full.rows(0, inter), full.rows(inter, 2 * inter)
            keep.append(self.mm.place_weights([wg, wu], self.dev))
            ws["gate"], ws["up"] = wg, wu
            layer_w.append(ws)
            wb += sum(wbytes(*SHAPES[n]) for n in lin) + 2 * wbytes(K, inter)
        res = {"layers": layers, "M": M, "weight_bytes": wb}
        for fuse, overlap, group, tag in ((False, 0, False, "as_emitted"), (True, 0, False, "fused_mlp"),
                                          (True, 2, False, "fused_mlp_overlap"), (True, 0, True, "fused_mlp_groups")):
            eng = self.mm.LinearEngine(self.rt, max_ops=8 * layers)
            eng.fuse_mlp(fuse)
            eng.overlap(overlap)
            eng.group(group)
            for ws in layer_w:
                for n in ("q", "k", "v"):
                    eng.add(x, ws[n], ys[n])
                eng.add(xo, ws["o"], ys["o"])
                eng.add(x, ws["gate"], g, note=b"gate")
                eng.add(x, ws["up"], u, note=b"up")
                eng.add_silu_mul(g, u, h)
                eng.add(h, ws["down"], ys["down"])
            n_ops = eng.n_ops()
            eng.launch()
            self.rt.sync()
            eng.capture()
            ms = self.timed(eng.launch, max(2, steps // 2), 3)
            groups = eng.n_group_launches()
            eng.close()
            res[tag] = {"ops": n_ops, "ms_per_step": ms, "weight_gbs": wb / ms / 1e6, "group_launches": groups}
        del layer_w, keep
        self.torch.cuda.empty_cache()
        return res

    def mlp_front(self, steps, warmup, layers=4):
        """The MLP front half (gate and up projections 5120 -> 17408 each, then
        silu(gate) * up) as the reference planner emits it - three ops - against
        the fused kernel, `layers` weight pairs per step so the weights of a step
        (100 MB per pair) exceed L2.  Same engine, fusion off and on."""
        K, inter = SHAPES["gate_up"][0], SHAPES["gate_up"][1] // 2
        full = self.weight("gate_up")
        out = {}
        for tag, M, st in (("decode_m16", 16, steps), ("prefill_m2048", 2048, max(2, steps // 4))):
            pairs, keep = [], []
            for _ in range(layers):
                wg, wu = full.rows(0, inter), full.rows(inter, 2 * inter)
                keep.append(self.mm.place_weights([wg, wu], self.dev))
                pairs.append((wg, wu))
            x = self.acts(M, K)
            g, u, y = self.empty(M, inter), self.empty(M, inter), self.empty(M, inter)
            res = {}
            for fuse in (False, True):
                eng = self.mm.LinearEngine(self.rt, max_ops=3 * layers)
                eng.fuse_mlp(fuse)
                for wg, wu in pairs:
                    eng.add(x, wg, g, note=b"gate")
                    eng.add(x, wu, u, note=b"up")
                    eng.add_silu_mul(g, u, y)
                n_ops = eng.n_ops()
                eng.launch()
                self.rt.sync()
                eng.capture()
                ms = self.timed(eng.launch, st, warmup)
                eng.close()
                res["fused" if fuse else "three_ops"] = {"ops": n_ops, "ms_per_step": ms}
            wb = layers * 2 * wbytes(K, inter)
            fl = layers * 2 * 2.0 * M * K * inter
            f = res["fused"]["ms_per_step"]
            res.update(M=M, layers=layers, weight_gbs=wb / f / 1e6, tflops=fl / f / 1e9,
                       speedup=res["three_ops"]["ms_per_step"] / f)
            out[tag] = res
            del pairs, keep
            self.torch.cuda.empty_cache()
        return out

    def decode_parts(self, secs=1.5):
        """Where a decode launch spends its time: gate+up and down at M = 1 and 16,
        as shipped and in the kernel's measurement modes (mm_f4_tune key 4: 1 = the
        weight stream alone, 2 = the arithmetic alone, 4 = split-K without the
        exchange), each as a short burst (20 graph replays after a pause) and
        sustained for `secs` seconds with SM clock and board power sampled."""
        if self.rt.lib.mm_f4_tune(4, 0) == -1:
            raise SystemExit("decode_parts needs a library built with MMB_EXTRA_DEFS=-DMMB_MEASURE_MODES")
        self.rt.lib.mm_f4_tune(5, 0)                  # the modes belong to the streaming kernel
        rows = []
        for name, copies in (("gate_up", 5), ("down", 8)):
            K, N = SHAPES[name]
            hw = self.weight(name)
            ws = [self.dev_weight(hw) for _ in range(copies)]
            for M in (1, 16):
                x = self.acts(M, K)
                ys = [self.empty(M, N) for _ in ws]
                for mode, tag in ((0, "as shipped"), (1, "weight stream alone"), (2, "arithmetic alone"),
                                  (4, "no split-K exchange")):
                    if mode == 4 and name == "gate_up":
                        continue                      # gate+up runs unsplit
                    self.rt.lib.mm_f4_tune(4, mode)
                    eng = self.engine([(x, w, y) for w, y in zip(ws, ys)], overlap=True, group=False)
                    time.sleep(0.3)
                    burst = self.timed(eng.launch, 20, 3)
                    with Clocks(self.local) as clk:
                        t0, n = time.time(), 0
                        self.rt.sync()
                        self.rt.time_begin()
                        while time.time() - t0 < secs:
                            for _ in range(50):
                                eng.launch()
                            self.rt.sync()
                            n += 50
                        sustained = self.rt.time_end() / n
                    eng.close()
                    self.rt.lib.mm_f4_tune(4, 0)
                    c = clk.summary()
                    rows.append({"op": name, "M": M, "mode": tag, "burst_us": round(burst * 1e3 / copies, 2),
                                 "sustained_us": round(sustained * 1e3 / copies, 2), "sm_mhz": c["sm_mhz"],
                                 "power_w_max": c["power_w_max"], "reasons": c["reasons"],
                                 "weight_gbs_burst": round(wbytes(K, N) / (burst / copies) / 1e6)})
            del ws
            self.torch.cuda.empty_cache()
        self.rt.lib.mm_f4_tune(5, 1)
        return {"rows": rows}

    def decode_sustained(self, secs=4.0, chunk=50):
        """The decode sweep replayed for `secs` seconds in chunks of `chunk` steps, each chunk
        timed with CUDA events, SM clock and board power sampled every 200 ms beside it: step
        time binned by the clock the chunk ran at.  Shows whether the time follows the clock
        (an SM-side bound), the power cap, or neither (memory-side)."""
        _, ops, eng = self.decode_sweep(5, 3, repeats=1, other_orders=False)
        wb = sum(wbytes(w.K, w.N) for _, w, _ in ops)
        torch = self.torch
        stream = self.rt.torch_stream()
        marks, stamps = [], []
        with Clocks(self.local) as clk:
            t0 = time.time()
            with torch.cuda.stream(stream):
                while time.time() - t0 < secs:
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(stream)
                    for _ in range(chunk):
                        eng.launch()
                    b.record(stream)
                    b.synchronize()
                    marks.append(a.elapsed_time(b) / chunk)
                    stamps.append(time.time() - t0)
        samples = clk.samples()          # (seconds since start, sm MHz, watts)
        eng.close()
        bins = {}
        for t, ms in zip(stamps, marks):
            near = min(samples, key=lambda q: abs(q[0] - t)) if samples else (0.0, 0.0, 0.0)
            key = int(round(near[1] / 30.0) * 30)
            bins.setdefault(key, []).append((ms, near[2]))
        rows = [{"sm_mhz": k, "chunks": len(v), "us_per_step": round(statistics.median(m for m, _ in v) * 1e3, 2),
                 "weight_gbs": round(wb / statistics.median(m for m, _ in v) / 1e6),
                 "us_x_ghz": round(statistics.median(m for m, _ in v) * k, 1),
                 "board_w": round(statistics.median(w for _, w in v))} for k, v in sorted(bins.items())]
        return {"seconds": secs, "chunk_steps": chunk, "chunks": len(marks),
                "us_per_step_median": round(statistics.median(marks) * 1e3, 2),
                "us_per_step_first": round(marks[0] * 1e3, 2), "us_per_step_last": round(marks[-1] * 1e3, 2),
                "by_clock": rows, "reasons": clk.summary()["reasons"]}

    def chain_timeline(self, M=16):
        """Where the time of dependent launches goes: globaltimer stamps taken inside the
        slicing kernel and the group kernel of every launch of one captured step (first and last
        CTA in, past the grid-dependency wait, MMAs done, epilogues done).  Needs a library
        built with -DMMB_MEASURE_MODES (MIMFER_B200_LIB points at it); two workloads: four down
        ops that write the same output, and three layers in the reference planner's order."""
        import ctypes as C
        from mimfer_b200 import _lib as L
        raw = C.CDLL(L.LIB_PATH)
        if not hasattr(raw, "mmb_trace_read"):
            raise SystemExit("chain_timeline needs a build with -DMMB_MEASURE_MODES")
        raw.mmb_trace_read.argtypes = [C.c_void_p, C.POINTER(C.c_uint32)]
        names = {"slice": ("in_first", "dep_first", "dep_last", "loads_first", "done_last", "in_last", "loads_last",
                           "sync1_last", None, "sync2_last", "done_first", "sliced_last"),
                 "group": ("in_first", "dep_first", "dep_last", "unit1_mma_first", "done_last", "in_last",
                           "unit1_mma_last", "mma_last", "done_first", "producer_last", "stage1_first", None)}

        def run(eng):
            eng.launch()
            self.rt.sync()
            eng.capture()
            for _ in range(5):
                eng.launch()
            self.rt.sync()
            assert raw.mmb_trace_clear() == 0
            eng.launch()
            self.rt.sync()
            buf = np.zeros((1024, 16), dtype=np.uint64)
            n = C.c_uint32()
            assert raw.mmb_trace_read(buf.ctypes.data, C.byref(n)) == 0
            rows = [buf[i] for i in range(n.value) if buf[i][4] != 0]
            t0 = min(int(r[0]) for r in rows)
            out = []
            for r in rows:
                kind = "group" if int(r[15]) == 1 else "slice"
                rec = {"kernel": kind}
                for k, name in enumerate(names[kind]):
                    if name and int(r[k]) not in (0, 2 ** 64 - 1):
                        rec[name] = round((int(r[k]) - t0) / 1e3, 2)
                out.append(rec)
            ms = self.timed(eng.launch, 20, 3)
            groups = eng.n_group_launches()
            eng.close()
            return {"us_per_step": ms * 1e3, "group_launches": groups, "launches_us_from_first_entry": out}

        assert raw.mmb_trace_reset() == 0
        K, N = SHAPES["down"]
        x, y = self.acts(M, K), self.empty(M, N)
        eng = self.mm.LinearEngine(self.rt, max_ops=8)
        for _ in range(4):
            eng.add(x, self.dev_weight(self.weight("down")), y)
        res = {"four_downs_one_output": run(eng)}
        assert raw.mmb_trace_reset() == 0
        K, inter = SHAPES["gate_up"][0], SHAPES["gate_up"][1] // 2
        full = self.weight("gate_up")
        lin = ("q", "k", "v", "o", "down")
        xx, xo = self.acts(M, K), self.acts(M, SHAPES["o"][0])
        g, u, h = self.empty(M, inter), self.empty(M, inter), self.empty(M, inter)
        ys = {n: self.empty(M, SHAPES[n][1]) for n in lin}
        keep = []
        eng = self.mm.LinearEngine(self.rt, max_ops=32)
        eng.fuse_mlp(True)
        for _ in range(3):
            ws = {n: self.dev_weight(self.weight(n)) for n in lin}
            wg, wu = full.rows(0, inter), full.rows(inter, 2 * inter)
            keep.append((ws, self.mm.place_weights([wg, wu], self.dev)))
            for n in ("q", "k", "v"):
                eng.add(xx, ws[n], ys[n])
            eng.add(xo, ws["o"], ys["o"])
            eng.add(xx, wg, g, note=b"gate")
            eng.add(xx, wu, u, note=b"up")
            eng.add_silu_mul(g, u, h)
            eng.add(h, ws["down"], ys["down"])
        res["planner_order_three_layers"] = run(eng)
        return res

    def _shard_rows(self, name):
        per = SHAPES[name][1] // self.world
        return (self.rank * per, (self.rank + 1) * per)

    def tp_e2e(self, steps, warmup, M=32):
        """The tensor-parallel decode step with host buffers: every rank copies the
        replicated activations up from pinned memory, runs both sharded linears
        (fused mode, one closing barrier), and rank 0 reads both full outputs back;
        one synchronisation per step, host wall clock, max over ranks."""
        from mimfer_b200.tp import TpLinear
        torch = self.torch
        lins = {n: TpLinear(self.weight(n), self.rank, self.world, rt=self.rt, mode="fused")
                for n in ("gate_up", "lm_head")}
        xd = {n: self.acts(M, SHAPES[n][0]) for n in lins}
        xh = {n: xd[n].cpu().pin_memory() for n in lins}
        yh = {n: torch.empty((M, SHAPES[n][1]), dtype=torch.bfloat16).pin_memory() for n in lins}
        last = list(lins.values())[-1]
        stream = self.rt.torch_stream()

        def step():
            with torch.cuda.stream(stream):
                for n in lins:
                    xd[n].copy_(xh[n], non_blocking=True)
            ys = {n: lin.forward(xd[n], barrier=False) for n, lin in lins.items()}
            last.barrier()
            if self.rank == 0:
                with torch.cuda.stream(stream):
                    for n in lins:
                        yh[n].copy_(ys[n], non_blocking=True)
            self.rt.sync()
        for _ in range(max(warmup, 3)):
            step()
        self.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            step()
        self.barrier()
        sec = torch.tensor([(time.perf_counter() - t0) / steps], dtype=torch.float64, device=self.dev)
        self.dist.all_reduce(sec, op=self.dist.ReduceOp.MAX)
        sec = float(sec.item())
        status = self.rt.device_status()
        if status:
            raise RuntimeError(f"device status 0x{status:x} after the end-to-end region")
        wb = sum(wbytes(*SHAPES[n]) for n in lins)
        res = {"value": wb / sec / 1e9, "unit": "GB/s", "ms_per_step": sec * 1e3,
               "h2d_bytes_per_step": sum(t.numel() * 2 for t in xh.values()) * self.world,
               "d2h_bytes_per_step": sum(t.numel() * 2 for t in yh.values()),
               "call": "TpLinear.forward (fused) on host activations, both outputs read back on rank 0",
               "timing": "host wall clock around a synchronous step, max over ranks"}
        for lin in lins.values():
            lin._symm.clear()
        del lins
        torch.cuda.empty_cache()
        return res

    def tp_sweep(self, steps, warmup, repeats=REPEATS):
        """The N=1 headline workload, tensor-parallel: the ten ops of the decode sweep, every
        one sharded along N over the ranks, as ONE group launch per rank whose epilogue stores
        every output tile into all ranks' copies, closed by the barrier kernel (TpGroupStep).
        Strong scaling of the same 752 MB step.  While a rank's share of the weights is at
        least twice the 126 MB L2 (two ranks: 376 MB) the steps run back to back like the
        one-GPU sweep; below that (four ranks: 188 MB, eight: 94 MB) L2 is flushed before every
        step (a 256 MiB fill) and the steps are timed one by one with CUDA events.  Max over
        ranks either way; MMB_TP_SWEEP_FLUSH=0/1 forces one form."""
        from mimfer_b200.tp import TpGroupStep
        torch = self.torch
        weights, xs, wb = [], [], 0
        for name in ("gate_up", "down"):
            K, N = SHAPES[name]
            for M in DECODE_M:
                weights.append(self.weight(name))       # TpGroupStep makes a device copy of every shard
                xs.append(self.acts(M, K))
                wb += wbytes(K, N)
        step = TpGroupStep(weights, xs, self.rank, self.world, self.rt)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.dev)
        stream = self.rt.torch_stream()
        do_flush = wb // self.world < 2 * (126 << 20)
        if os.environ.get("MMB_TP_SWEEP_FLUSH") in ("0", "1"):
            do_flush = os.environ["MMB_TP_SWEEP_FLUSH"] == "1"
        for _ in range(max(warmup, 3)):
            step.replay()
        self.rt.sync()
        regions = []
        for _ in range(repeats):
            self.barrier()
            evs = []
            with torch.cuda.stream(stream):
                if do_flush:
                    for _ in range(steps):
                        flush.fill_(1)
                        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        a.record(stream)
                        step.replay()
                        b.record(stream)
                        evs.append((a, b))
                else:
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(stream)
                    for _ in range(steps):
                        step.replay()
                    b.record(stream)
                    evs.append((a, b))
            self.rt.sync()
            ms = sum(a.elapsed_time(b) for a, b in evs) / steps
            t = torch.tensor([ms], device=self.dev)
            if self.world > 1:
                self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            regions.append(float(t.item()))
        status = self.rt.device_status()
        if status:
            raise RuntimeError(f"device status 0x{status:x} after the tensor-parallel sweep")
        # parity: this rank's copy of every output against the CPU oracle, windows at shard edges
        from oracle.pyoracle import Oracle
        orc = Oracle()
        ys = step.replay()
        self.rt.sync()
        self.barrier()
        worst = 0.0
        for w, x, y in zip(weights, xs, ys):
            xb = self.rt.from_device_bf16(x)
            ns = w.N // self.world
            for e in sorted({0, ns * (self.world // 2), ns * (self.world - 1)}):
                a = max(0, e - 128)
                got = self.rt.from_device_bf16(y[:, a:a + 256].contiguous())
                want = orc.gemm_f4(xb, w.payload, w.scales, w.gs, n_begin=a, n_end=a + 256)
                g = (got.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
                r = (want.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
                den = np.sqrt((r ** 2).sum(axis=1))
                worst = max(worst, float((np.sqrt(((g - r) ** 2).sum(axis=1)) / np.where(den == 0, 1.0, den)).max()))
        t = torch.tensor([worst], dtype=torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        worst = float(t.item())
        launches = step.engines[0].n_group_launches()
        # the same step with host buffers: every rank brings the (replicated) activations up from
        # pinned memory, rank 0 reads all ten full outputs back; one synchronisation per step
        xh = [x.cpu().pin_memory() for x in xs]
        yh = [torch.empty(y.shape, dtype=y.dtype).pin_memory() for y in ys]

        def host_step():
            with torch.cuda.stream(stream):
                for x, h in zip(xs, xh):
                    x.copy_(h, non_blocking=True)
            out = step.replay()
            if self.rank == 0:
                with torch.cuda.stream(stream):
                    for h, y in zip(yh, out):
                        h.copy_(y, non_blocking=True)
            self.rt.sync()
        for _ in range(max(warmup, 3)):
            host_step()
        self.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            host_step()
        self.barrier()
        sec = torch.tensor([(time.perf_counter() - t0) / steps], dtype=torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(sec, op=self.dist.ReduceOp.MAX)
        sec = float(sec.item())
        e2e = {"value": wb / sec / 1e9, "unit": "GB/s", "ms_per_step": sec * 1e3,
               "h2d_bytes_per_step": sum(t.numel() * 2 for t in xh) * self.world,
               "d2h_bytes_per_step": sum(t.numel() * 2 for t in yh),
               "call": "TpGroupStep.replay on host activations (every rank uploads them), all ten outputs read "
                       "back on rank 0",
               "timing": "host wall clock around a synchronous step, max over ranks"}
        step.close()
        del flush
        torch.cuda.empty_cache()
        med = statistics.median(regions)
        return {"ms_per_step": med, "ms_per_step_min": min(regions), "ms_per_step_max": max(regions),
                "timed_regions": len(regions), "weight_bytes": wb, "weight_gbs": wb / med / 1e6,
                "weight_gbs_min": wb / max(regions) / 1e6, "weight_gbs_max": wb / min(regions) / 1e6,
                "group_launches_per_rank": launches, "e2e": e2e,
                "l2": "flushed before every step (256 MiB fill), steps timed one by one" if do_flush
                      else f"every rank reads {wb // self.world >> 20} MB of weights per step, more than twice L2; steps back to back",
                "parity": {"max_row_rel_l2": worst, "tolerance": 2.0 ** -8, "ok": worst <= 2.0 ** -8,
                           "checked": "every rank's copy of all ten outputs, 256-column windows at shard edges, "
                                      "against the CPU oracle"}}

    def tp_parity(self, lins, xs, M):
        """The outputs of one more tensor-parallel step against the CPU oracle (checker only):
        every rank's copy of both full outputs, on column windows inside and across the shard
        edges, sampled rows at prefill size.  Worst per-row relative L2 over ranks and windows."""
        from oracle.pyoracle import Oracle
        orc = Oracle()
        ys = {n: lin.forward(xs[n], barrier=False) for n, lin in lins.items()}
        list(lins.values())[-1].barrier()
        self.rt.sync()
        self.barrier()
        rows = None if M <= 32 else sorted({0, 255, M // 2, M - 1})
        worst = 0.0
        for n, lin in lins.items():
            hw = self.weight(n)
            xb = self.rt.from_device_bf16(xs[n])
            ns = SHAPES[n][1] // self.world
            edges = sorted({0, ns * (self.world // 2), ns * (self.world - 1)})
            y = ys[n]
            for e in edges:
                a = max(0, e - 128)
                b = a + 256
                got = self.rt.from_device_bf16(y[:, a:b].contiguous() if rows is None
                                               else y[rows][:, a:b].contiguous())
                want = orc.gemm_f4(xb, hw.payload, hw.scales, hw.gs, rows=rows, n_begin=a, n_end=b)
                g = (got.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
                r = (want.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
                den = np.sqrt((r ** 2).sum(axis=1))
                err = float((np.sqrt(((g - r) ** 2).sum(axis=1)) / np.where(den == 0, 1.0, den)).max())
                worst = max(worst, err)
        t = self.torch.tensor([worst], dtype=self.torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        worst = float(t.item())
        return {"max_row_rel_l2": worst, "tolerance": 2.0 ** -8, "ok": worst <= 2.0 ** -8,
                "checked": "every rank's outputs, 256-column windows at shard edges, against the CPU oracle"}

    def tp_series(self, steps, warmup):
        """config 5: gate+up and LM head, sharded along N over all ranks, M=32 and M=8192."""
        from mimfer_b200.tp import TpGroupStep, TpLinear, TpStep
        out = {"world": self.world}
        modes = ("gather",) if self.world == 1 else ("fused", "push", "gather")
        for mode in modes:
            lins = {n: TpLinear(self.weight(n), self.rank, self.world, rt=self.rt, mode=mode)
                    for n in ("gate_up", "lm_head")}
            res = {}
            for tag, M, st in (("decode_m32", 32, steps), ("prefill_m8192", 8192, max(2, steps // 4))):
                if mode == "push" and M <= 32:      # the copy engines' form is for prefill-size outputs
                    continue
                xs = {n: self.acts(M, SHAPES[n][0]) for n in lins}

                last = list(lins.values())[-1]

                def step():                     # the linears of a step share one closing barrier
                    for n, lin in lins.items():
                        lin.forward(xs[n], barrier=False)
                    last.barrier()
                ms_eager = ms = self.timed(step, st, warmup)
                captured = (mode == "fused" or self.world == 1) and M <= 32   # launch cost matters at decode sizes only
                ms_two = None
                if captured:
                    # the same step captured once and replayed: one launch per step and rank
                    graph = TpStep(list(lins.values()), [xs[n] for n in lins])
                    ms_two = ms = self.timed(graph.replay, st, warmup)
                    del graph
                    # ... and as one group launch per rank instead of a kernel pair per linear
                    gstep = TpGroupStep([self.weight(n) for n in lins], [xs[n] for n in lins], self.rank,
                                        self.world, self.rt)
                    ms = self.timed(gstep.replay, st, warmup)
                    gstep.close()
                    del gstep
                wb = sum(wbytes(*SHAPES[n]) for n in lins)
                fl = sum(2.0 * M * SHAPES[n][0] * SHAPES[n][1] for n in lins)
                res[tag] = {"ms_per_step": ms, "weight_gbs": wb / ms / 1e6, "tflops": fl / ms / 1e9,
                            "issue": "one group launch + barrier per rank, captured" if captured else "op by op",
                            "op_by_op_ms_per_step": ms_eager}
                if ms_two is not None:
                    res[tag]["kernel_pair_per_linear_ms_per_step"] = ms_two
                if mode in ("fused", "push") or self.world == 1:
                    res[tag]["parity"] = self.tp_parity(lins, xs, M)
                for lin in lins.values():
                    lin._bufs.clear()
                    lin._symm.clear()
                self.torch.cuda.empty_cache()
            out[mode] = res
            del lins
        if self.world > 1:
            out["e2e"] = self.tp_e2e(max(2, steps // 2), warmup)
        # the sharded kernels alone, no exchange: what the GEMM itself scales like
        shards = {n: self.dev_weight(self.weight(n, rows=self._shard_rows(n))) for n in ("gate_up", "lm_head")}
        res = {}
        for tag, M, st in (("decode_m32", 32, steps), ("prefill_m8192", 8192, max(2, steps // 4))):
            ops = [(self.acts(M, SHAPES[n][0]), w, self.empty(M, w.N)) for n, w in shards.items()]

            def step():
                for x, w, y in ops:
                    self.rt.linear_async(x, w, y)
            ms = self.timed(step, st, warmup)
            wb = sum(wbytes(*SHAPES[n]) for n in shards)
            fl = sum(2.0 * M * SHAPES[n][0] * SHAPES[n][1] for n in shards)
            res[tag] = {"ms_per_step": ms, "weight_gbs": wb / ms / 1e6, "tflops": fl / ms / 1e9}
            del ops
            self.torch.cuda.empty_cache()
        out["local_only"] = res
        # like-for-like efficiency: the same two linears unsharded on one GPU, timed in this run
        # (at one rank that is the series itself)
        if self.world > 1:
            whole = {n: self.dev_weight(self.weight(n)) for n in ("gate_up", "lm_head")}
            one = {}
            for tag, M, st in (("decode_m32", 32, steps), ("prefill_m8192", 8192, max(2, steps // 4))):
                ops = [(self.acts(M, SHAPES[n][0]), w, self.empty(M, w.N)) for n, w in whole.items()]
                if M <= 32:
                    eng = self.engine(ops)
                    one[tag] = self.timed(eng.launch, st, warmup)
                    eng.close()
                else:
                    def step():
                        for x, w, y in ops:
                            self.rt.linear_async(x, w, y)
                    one[tag] = self.timed(step, st, warmup)
                del ops
                self.torch.cuda.empty_cache()
            del whole
            self.torch.cuda.empty_cache()
        else:
            one = {tag: out[modes[0]][tag]["ms_per_step"] for tag in ("decode_m32", "prefill_m8192")}
        out["one_gpu_ms_per_step"] = one
        best = modes[0]
        out["mode"] = best + (" (kernel epilogue stores to peers)" if best == "fused" else " (single GPU)")
        out.update(out[best])
        if "push" in out:
            # prefill: the exchange by the epilogue's stores or by the copy engines, whichever is faster here
            out["prefill_exchange"] = {"epilogue_stores_ms": out["fused"]["prefill_m8192"]["ms_per_step"],
                                       "copy_engines_ms": out["push"]["prefill_m8192"]["ms_per_step"]}
            if out["push"]["prefill_m8192"]["ms_per_step"] < out["fused"]["prefill_m8192"]["ms_per_step"]:
                out["prefill_m8192"] = dict(out["push"]["prefill_m8192"],
                                            issue="row chunks; each chunk's slice pushed to the peers by the copy "
                                                  "engines while the next chunk is multiplied")
        out["efficiency"] = {tag: one[tag] / (self.world * out[tag]["ms_per_step"])
                             for tag in ("decode_m32", "prefill_m8192")}
        return out


def cpu_baseline(threads=None, target_s=12.0):
    """The reference CPU kernel (oracle/_ref, else the oracle port) on this
    host's cores, on a bounded sample of the decode sweep: the first R rows of
    gate+up and of down at every M of the sweep, R sized by a short probe so
    the sample takes about target_s seconds.  Same metric as the GPU arm:
    packed weight bytes processed / time.  Inputs come from the host-only
    generator beside the checkers (numpy; the same packing recipe), so this leg
    loads nothing of the product library."""
    from oracle import inputs
    from oracle.pyoracle import Oracle, Reference, host_threads
    threads = threads or host_threads()
    ref = Reference()
    kind = "reference" if ref.available else "port"
    orc = None if ref.available else Oracle()
    cache = {}

    def weights(name, rows):
        if cache.get(name, (0,))[0] < rows:
            K = SHAPES[name][0]
            cache[name] = (rows, *inputs.make_weight(rows, K, seed=0)[:2])
        _, payload, scales = cache[name]
        return payload[:rows], scales[:rows]

    def run(x, payload, scales):
        t0 = time.perf_counter()
        if ref.available:
            rc, _ = ref.gemm_f4(x, payload, scales, threads=threads)
            assert rc == 0
        else:
            orc.gemm_f4(x, payload, scales, 1.0, threads=threads)
        return time.perf_counter() - t0

    def sweep(rows):
        dt, nbytes = 0.0, 0
        for name in ("gate_up", "down"):
            K, N = SHAPES[name]
            r = min(rows, N)
            payload, scales = weights(name, r)
            for M in DECODE_M:
                dt += run(inputs.make_activations(M, K, seed=1), payload, scales)
                nbytes += wbytes(K, r)
        return dt, nbytes

    probe_rows = 16 * threads
    dt, _ = sweep(probe_rows)
    rows = int(min(34816, max(probe_rows, probe_rows * target_s / max(dt, 1e-6))))
    dt, nbytes, passes = *sweep(rows), 1
    while dt < 0.8 * target_s:                     # few rows left to add: repeat the sweep instead
        d2, n2 = sweep(rows)
        dt, nbytes, passes = dt + d2, nbytes + n2, passes + 1
    return {"value": nbytes / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": kind,
            "seconds": dt, "passes": passes,
            "sample": f"decode sweep M in {{1,2,4,8,16}} on the first {rows} rows of gate+up and of down, "
                      f"{dt:.1f} s of CPU time"}


def run_b200(args):
    b = Bench(args)
    b.rt.lib.mm_f4_force_variant(args.variant)
    for kv in args.tune:
        k, v = kv.split("=")
        b.rt.lib.mm_f4_tune(int(k), int(v))
    pk = peaks()
    steps, warmup = args.steps, max(args.warmup, 3)
    line = {"metric": METRIC, "unit": "GB/s", "n_gpus": b.world, "steps": steps, "warmup": warmup,
            "higher_is_better": True, "vs_baseline": None, "dtype": "bf16 x nvfp4 -> f32 accumulate",
            "data": "synthetic"}
    with Clocks(b.local) as clk:
        if args.case != "default":
            res = run_case(b, args.case, steps, warmup)
            if b.rank == 0:
                print(json.dumps({"case": args.case, **res}))
            if b.world > 1:
                b.dist.destroy_process_group()
            return
        if b.world == 1:
            dec, ops, eng = b.decode_sweep(steps, warmup, per_op=True)
            line.update(value=dec["weight_gbs"], ms_per_step=dec["ms_per_step"], scaling="strong",
                        value_min=dec["weight_gbs_min"], value_max=dec["weight_gbs_max"],
                        timed_regions=dec["timed_regions"],
                        gpu_launches=dec["kernel_launches_per_step"] * steps,
                        config={"workload": "decode GEMV sweep M in {1,2,4,8,16} x {gate+up 5120->34816, "
                                            "down 17408->5120}, 10 ops per step, one CUDA graph: one slicing "
                                            "kernel and one persistent group launch of the block-scaled kernel",
                                "l2": "every op reads its own weight copy: 750 MB per step, larger than L2",
                                "timing": f"median of {dec['timed_regions']} timed regions of {steps} steps",
                                "quant": "NVFP4 e2m1 + e4m3/16 + fp32 global scale", "peaks": pk["src"]})
            line["decode_sweep"] = {k: dec[k] for k in ("ops", "weight_bytes", "alg_bytes", "group_launches",
                                                        "kernel_launches_per_step", "ms_per_step_min",
                                                        "ms_per_step_max", "serial_order", "run_ahead", "per_op")}
            line["roofline"] = {"bound": "hbm", "kernel": "f4_mxg_kernel",
                                "achieved": dec["alg_gbs"], "peak": pk["hbm"], "unit": "GB/s",
                                "frac": dec["alg_gbs"] / pk["hbm"], "of": pk["src"],
                                "alg_bytes_per_launch": dec["alg_bytes"],
                                "launch_us": dec["ms_per_step"] * 1e3,
                                "launch_includes": "the step's slicing kernel (activations to digit planes)",
                                "traffic": GROUP_TRAFFIC_RATIO * dec["alg_bytes"],
                                "traffic_src": "ncu capture of a group launch on two gate+up ops, "
                                               "scaled by algorithmic bytes"}
            line["e2e"] = b.decode_e2e(ops, eng, max(2, steps // 2), warmup)
            eng.close()
            del ops
            b.torch.cuda.empty_cache()
            pre = b.prefill_sweep(steps, warmup)
            pre["roofline"] = {"bound": "tensor", "kernel": "f4_umma_kernel", "achieved": pre["tflops"],
                               "peak": pk["tensor_sustained"], "peak_burst": pk["tensor_burst"],
                               "unit": "TFLOP/s", "frac": pre["tflops"] / pk["tensor_sustained"],
                               "frac_of_burst": pre["tflops"] / pk["tensor_burst"], "of": pk["src"]}
            line["prefill"] = pre
            b.torch.cuda.empty_cache()
            line["decode_step"] = b.decode_step_64(steps, warmup)
            b.torch.cuda.empty_cache()
            # same weights with q, k and v as one fused op (the reference planner's OP_QKV layout)
            fused = b.decode_step_64(steps, warmup, names=("qkv", "o", "gate_up", "down"))
            line["decode_step"]["fused_qkv"] = {k: fused[k] for k in ("ops", "sum_linear_ms_per_step", "weight_gbs",
                                                                      "group_launches", "serial_order", "run_ahead")}
            b.torch.cuda.empty_cache()
            line["mlp_front"] = b.mlp_front(steps, warmup)
            line["decode_step"]["planner_sequence"] = b.decode_step_planner(steps, warmup)
        tp = b.tp_series(steps, warmup)
        line["tp"] = tp
        if b.world > 1:
            sw = b.tp_sweep(steps, warmup)
            line["tp_sweep"] = sw
            line.update(value=sw["weight_gbs"], ms_per_step=sw["ms_per_step"], scaling="strong",
                        value_min=sw["weight_gbs_min"], value_max=sw["weight_gbs_max"],
                        timed_regions=sw["timed_regions"], gpu_launches=3 * steps,
                        config={"workload": f"the decode GEMV sweep of the one-GPU line (M in {{1,2,4,8,16}} x "
                                            f"{{gate+up, down}}, 752 MB of weights per step), every op split along N "
                                            f"over {b.world} GPUs: per rank one slicing kernel, one group launch whose "
                                            f"epilogue stores every output tile to all ranks (symmetric memory), one "
                                            f"barrier kernel",
                                "l2": sw["l2"], "timing": f"median of {sw['timed_regions']} timed regions of {steps} steps",
                                "peaks": pk["src"]})
            line["roofline"] = {"bound": "hbm", "kernel": "f4_mxg_kernel", "achieved": sw["weight_gbs"],
                                "peak": pk["hbm"] * b.world, "unit": "GB/s",
                                "frac": sw["weight_gbs"] / (pk["hbm"] * b.world), "of": pk["src"], "traffic": None}
            line["prefill"] = {"tflops": tp["prefill_m8192"]["tflops"],
                               "ms_per_step": tp["prefill_m8192"]["ms_per_step"]}
            line["e2e"] = sw.pop("e2e")
    line["clocks"] = clk.summary()
    if b.rank == 0:
        if b.world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline()
        print(json.dumps(line))
    if b.world > 1:
        b.dist.destroy_process_group()


def run_case(b, case, steps, warmup):
    """Single small cases, used for profiling one kernel at a time."""
    if case == "decode":           # gate+up at M=1 and M=16, two weight copies each
        res, _, eng = b.decode_sweep(steps, warmup, ms_list=(1, 16), names=("gate_up",))
        eng.close()
        return res
    if case == "group":            # one group launch: gate+up and down at M=1 and M=16 (300 MB of weights)
        res, _, eng = b.decode_sweep(steps, warmup, ms_list=(1, 16), repeats=1, other_orders=False)
        eng.close()
        return res
    if case == "sweep":            # the headline workload alone: the ten-op sweep as one group launch
        res, _, eng = b.decode_sweep(steps, warmup, repeats=1, other_orders=False)
        eng.close()
        return res
    if case == "sustained":        # the sweep for four seconds, step time binned by SM clock
        return b.decode_sustained()
    if case == "decode_parts":     # the decode kernel's time split into stream / arithmetic / exchange
        return b.decode_parts()
    if case == "e2e":              # the default sweep and its host-buffer step
        res, ops, eng = b.decode_sweep(steps, warmup)
        res["e2e"] = b.decode_e2e(ops, eng, max(2, steps // 2), warmup)
        eng.close()
        return res
    if case == "decode_m32":       # gate+up at M=32, two weight copies
        res, _, eng = b.decode_sweep(steps, warmup, ms_list=(32, 32), names=("gate_up",))
        eng.close()
        return res
    if case == "decode_m16":
        res, _, eng = b.decode_sweep(steps, warmup, ms_list=(16, 16), names=("gate_up", "down"))
        eng.close()
        return res
    if case == "mlp_front":        # gate + up + silu, three ops against the fused kernel
        return b.mlp_front(steps, warmup)
    if case == "decode_down":
        res, _, eng = b.decode_sweep(steps, warmup, ms_list=(1, 16), names=("down",))
        eng.close()
        return res
    if case == "decode_layers":    # two layers of the 64-layer decode step (12 ops)
        return b.decode_step_64(steps, warmup, layers=2)
    if case == "decode_layers8":   # eight layers (48 ops: one group launch)
        return b.decode_step_64(steps, warmup, layers=8)
    if case == "prefill":          # one 2048 x 5120 x 34816 GEMM
        return b.prefill_sweep(steps, warmup, ms_list=(2048,), names=("gate_up",))
    if case == "chain_down":       # eight down ops at M=16 that write the same output: eight dependent launches
        K, N = SHAPES["down"]
        x, y = b.acts(16, K), b.empty(16, N)
        ops = [(x, b.dev_weight(b.weight("down")), y) for _ in range(8)]
        eng = b.engine(ops, group=os.environ.get("MMB_CHAIN_GROUP", "1") != "0")
        ms = b.timed(eng.launch, steps, warmup, repeats=3)
        groups = eng.n_group_launches()
        eng.close()
        return {"ms_per_step": ms, "us_per_op": ms * 1e3 / 8, "group_launches": groups,
                "weight_gbs": 8 * wbytes(K, N) / ms / 1e6}
    if case == "prefill_tail":     # down at M=2048: 148 whole tiles + 12 tiles in 10 K slices + the tail kernel
        return b.prefill_sweep(steps, warmup, ms_list=(2048,), names=("down",))
    if case == "prefill_kv":       # k at M=2048: 32 tiles, all of them split
        return b.prefill_sweep(steps, warmup, ms_list=(2048,), names=("k",))
    if case == "chain_timeline":   # measurement build only: time stamps inside dependent launches
        return b.chain_timeline()
    if case == "planner_layers8":  # eight layers in the reference planner's op order, with their dependencies
        return b.decode_step_planner(steps, warmup, layers=8)
    if case == "tp":               # the tensor-parallel series alone (any number of ranks)
        return b.tp_series(steps, warmup)
    if case == "prefill_small":
        return b.prefill_sweep(steps, warmup, ms_list=(512,), names=("q",))
    raise SystemExit(f"unknown case {case}")


# --------------------------------------------------------------------------- reference arm
def run_reference(args):
    """The reference's own CPU implementation of the path on this host's cores.  A step is
    one pass over the bounded sample; --warmup passes are untimed, the median of --steps
    (at most 5) timed passes is the value."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 5))
    per = max(4.0, min(12.0, 40.0 / steps))
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_baseline(target_s=2.0)                   # builds the checker, warms the thread pool
    runs = [cpu_baseline(target_s=per) for _ in range(steps)]
    vals = [r["value"] for r in runs]
    v = statistics.median(vals)
    base = runs[vals.index(sorted(vals)[len(vals) // 2])]
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": max(1, min(args.warmup, 2)),
            "ms_per_step": statistics.median(r["seconds"] / r["passes"] for r in runs) * 1e3,
            "value_min": min(vals), "value_max": max(vals),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 x nvfp4 -> f32 accumulate", "data": "synthetic",
            "config": {"workload": "reference CPU kx_op_gemm_f4 on a bounded sample of the decode workload: "
                                   + base["sample"]},
            "cpu_baseline": {**base, "value": v},
            "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--case", default="default")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--tune", action="append", default=[], metavar="KEY=VALUE",
                    help="set a library tuning knob (mm_f4_tune), e.g. 2=1; experiments only")
    ap.add_argument("--variant", type=int, default=-1,
                    help="force a kernel variant for every op (experiments; -1 = selector)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
