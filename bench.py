#!/usr/bin/env python
"""Benchmark of the ug hot path on B200 through the C ABI.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One JSON line on rank 0.  A "step" is one pass of the hot path over one batch
of seeded synthetic input.  Timing: CUDA events on the library's own stream
(the stream its kernels run on), W warm-up steps, K timed steps bracketed by a
barrier and a device synchronisation, maximum over ranks.  The default workload
is the Llama-1.1B-shape decode of ONE batch of 64 sequences: with N ranks every
rank owns a contiguous range of 64 / N sequences and a full replica of the
weights, there is no data-path collective, and the value is 64 sequences per
step of the slowest rank (strong scaling).  At N > 1 the same line also carries
the 64-sequences-per-GPU figure (key "weak") and the head-sharded
tensor-parallel variant (key "tp"); at N = 1 it carries one sub-record per
other benchmark configuration (key "configs").  Rows (softmax, rms_norm) and
GEMM batches are partitioned the same way when chosen with --workload.

``--impl reference`` times the reference's CPU path (the oracle restatement of
ug-core's CPU backend; the Rust sources cannot be compiled in this image) on a
bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return {"hbm": float(d["hbm_gbs"]), "bf16": float(d["bf16_tflops"]),
                    "bf16_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    "source": "measured"}
        except Exception:
            pass
    return {"hbm": FALLBACK_HBM_GBS, "bf16": FALLBACK_BF16_TFLOPS, "bf16_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi during the timed region."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 6:
                continue
            try:
                mhz.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(mhz)) if mhz else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(mhz)}


# ----------------------------------------------------------------- workloads
class RmsSiluWorkload:
    """Config 2: out = rms_norm(x) * w * silu(gate), f32 [8192, 4096] per GPU."""
    name = "rms_norm_silu_gate f32 [8192,4096] (config 2), rows partitioned across GPUs"
    metric = "effective HBM GB/s, fused rms_norm*silu(gate) (row-op bandwidth as in the softmax GB/s metric)"
    unit = "GB/s"
    dtype = "f32"
    bound = "hbm"
    rows, cols = 8192, 4096
    # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this workload's kernel, from an ncu capture
    # of this shape (the output's tail is still in L2 when the counters stop)
    ncu_traffic_bytes = 268_462_080 + 96_574_464

    def __init__(self, rank):
        from ug_b200 import synth
        # every rank owns its own 8192-row partition, seeded by rank
        self.x = synth.normal(1 + 1000 * rank, (self.rows, self.cols))
        self.gate = synth.normal(2 + 1000 * rank, (self.rows, self.cols))
        self.w = synth.uniform(3, (self.cols,), 0.5, 1.5)
        self.eps = 1e-5
        # x + gate read, w read, out written (bytes); GB/s = bytes / time
        self.bytes_per_step = 3 * self.rows * self.cols * 4 + self.cols * 4
        self.h2d_bytes = 2 * self.rows * self.cols * 4 + self.cols * 4
        self.d2h_bytes = self.rows * self.cols * 4
        self.launches_per_step = 1

    def setup(self, dev):
        from ug_b200 import DType
        self.dev = dev
        self.xs = dev.slice_from_values(self.x)
        self.gs = dev.slice_from_values(self.gate)
        self.ws = dev.slice_from_values(self.w)
        self.out = dev.allocate_uninit(DType.F32, self.rows * self.cols)

    def step(self):
        self.dev.rms_norm_silu_gate(self.xs, self.ws, self.gs, self.out, self.rows, self.cols, self.eps)

    def units(self, step_seconds, n_ranks):
        return n_ranks * self.bytes_per_step / step_seconds / 1e9

    def setup_e2e(self):
        import ctypes as C
        from ug_b200._lib import lib
        self._pin = []
        def pinned(arr):
            p = C.c_void_p()
            assert lib.ugb_host_alloc(arr.nbytes, C.byref(p)) == 0
            buf = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=(arr.size,))
            buf[:] = arr.ravel()
            self._pin.append(p)
            return p, buf
        self.px, _ = pinned(self.x)
        self.pg, _ = pinned(self.gate)
        self.pw, _ = pinned(self.w)
        self.po, self.out_host = pinned(np.zeros(self.rows * self.cols, np.float32))

    def e2e_step(self):
        from ug_b200 import DType
        from ug_b200._lib import lib
        d, f32 = self.dev, int(DType.F32)
        d._check(lib.ugb_h2d_async(self.xs._h, self.px, self.rows * self.cols, f32))
        d._check(lib.ugb_h2d_async(self.gs._h, self.pg, self.rows * self.cols, f32))
        d._check(lib.ugb_h2d_async(self.ws._h, self.pw, self.cols, f32))
        self.step()
        d._check(lib.ugb_d2h_async(self.out._h, self.po, self.rows * self.cols, f32))
        d.synchronize()

    def teardown_e2e(self):
        from ug_b200._lib import lib
        for p in self._pin:
            lib.ugb_host_free(p)

    def check(self):
        """Parity of the timed kernel's output against the oracle on a row subset."""
        import oracle
        got = self.out.to_vec().reshape(self.rows, self.cols)[:16]
        ref = oracle.gen_rms_norm_silu_gate(self.x, self.w, self.gate, self.eps, rows=(0, 16))[:16]
        return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 1e-20)))

    def cpu_sample(self, budget_s):
        """ug CPU backend (emitted C, one thread) on a bounded row sample; returns GB/s."""
        import oracle
        rows = 64
        t0 = time.perf_counter()
        oracle.gen_rms_norm_silu_gate(self.x, self.w, self.gate, self.eps, rows=(0, rows))
        per_row = (time.perf_counter() - t0) / rows
        rows = int(max(64, min(self.rows, budget_s / per_row)))
        t0 = time.perf_counter()
        oracle.gen_rms_norm_silu_gate(self.x, self.w, self.gate, self.eps, rows=(0, rows))
        dt = time.perf_counter() - t0
        gbs = rows * self.cols * 12 / dt / 1e9
        return gbs, 1, f"{rows} of {self.rows} rows, emitted-C kernel of ug's CPU backend, 1 thread, {dt:.1f} s"

    def config(self):
        return {"workload": self.name, "rows_per_gpu": self.rows, "cols": self.cols,
                "l2": "inputs larger than L2 (403 MB touched per step vs 126 MB L2)"}


class SoftmaxWorkload(RmsSiluWorkload):
    """Config 1 scaled to HBM size: softmax f32 rows of 4096, 32768 rows per GPU."""
    name = "custom_softmax f32 [32768,4096] (config 1 row shape, 32x rows so the batch exceeds L2)"
    metric = "softmax effective GB/s (rows*cols*8 bytes / time)"
    rows, cols = 32768, 4096
    ncu_traffic_bytes = 536_986_880 + 484_354_048      # ncu capture of this shape, read + write

    def __init__(self, rank):
        from ug_b200 import synth
        self.x = synth.normal(0 + 1000 * rank, (self.rows, self.cols), 2.0)
        self.bytes_per_step = 2 * self.rows * self.cols * 4
        self.h2d_bytes = self.d2h_bytes = self.rows * self.cols * 4
        self.launches_per_step = 1

    def setup(self, dev):
        from ug_b200 import DType
        self.dev = dev
        self.xs = dev.slice_from_values(self.x)
        self.out = dev.allocate_uninit(DType.F32, self.rows * self.cols)

    def step(self):
        self.dev.custom_softmax(self.xs, self.out, self.rows, self.cols)

    def setup_e2e(self):
        import ctypes as C
        from ug_b200._lib import lib
        self._pin = []
        for attr, arr in (("px", self.x), ("po", np.zeros(self.rows * self.cols, np.float32))):
            p = C.c_void_p()
            assert lib.ugb_host_alloc(arr.nbytes, C.byref(p)) == 0
            np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=(arr.size,))[:] = arr.ravel()
            setattr(self, attr, p)
            self._pin.append(p)

    def e2e_step(self):
        from ug_b200 import DType
        from ug_b200._lib import lib
        d, f32 = self.dev, int(DType.F32)
        d._check(lib.ugb_h2d_async(self.xs._h, self.px, self.rows * self.cols, f32))
        self.step()
        d._check(lib.ugb_d2h_async(self.out._h, self.po, self.rows * self.cols, f32))
        d.synchronize()

    def check(self):
        import oracle
        got = self.out.to_vec().reshape(self.rows, self.cols)[:64]
        ref = oracle.custom_softmax(self.x[:64])
        return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 1e-30)))

    def reference_cuda_gbs(self, steps=20):
        """The reference's own softmax.cu (one warp per row, three passes; oracle/_ref) on the same buffers."""
        import oracle
        from ug_b200._lib import lib
        ref = oracle.reference_cuda()
        if ref is None:
            return None
        stream = lib.ugb_device_stream(self.dev._h)
        run = lambda: ref.ugref_softmax_f32(self.xs.device_ptr, self.out.device_ptr, self.rows, self.cols, stream)
        for _ in range(3):
            run()
        self.dev.synchronize()
        self.dev.timer_begin()
        for _ in range(steps):
            run()
        self.dev.timer_end()
        return self.bytes_per_step * steps / (self.dev.timer_elapsed_ms() / 1e3) / 1e9

    def cpu_sample(self, budget_s):
        import oracle
        rows = 32
        t0 = time.perf_counter()
        oracle.gen_softmax(self.x, rows=(0, rows))
        per_row = (time.perf_counter() - t0) / rows
        rows = int(max(32, min(self.rows, budget_s / per_row)))
        t0 = time.perf_counter()
        oracle.gen_softmax(self.x, rows=(0, rows))
        dt = time.perf_counter() - t0
        return rows * self.cols * 8 / dt / 1e9, 1, \
            f"{rows} of {self.rows} rows, two emitted-C kernels of ug's CPU backend, 1 thread, {dt:.1f} s"

    def config(self):
        return {"workload": self.name, "rows_per_gpu": self.rows, "cols": self.cols,
                "l2": "inputs larger than L2 (1.07 GB touched per step vs 126 MB L2)"}


class SoftmaxC1Workload(SoftmaxWorkload):
    """Config 1 at its own size: softmax f32 [1024, 4096].  One launch touches 33.5 MB, which fits the
    126 MB L2, so a step works on the next of 16 distinct input / output buffer pairs (537 MB in all): every
    launch finds its rows in HBM.  `resident_gbs` times the same launch on one pair, i.e. out of L2."""
    name = "custom_softmax f32 [1024,4096] (config 1), rotated over 16 buffer pairs (537 MB) so that no launch finds its rows in L2"
    rows, cols, pairs = 1024, 4096, 16
    ncu_traffic_bytes = (536_986_880 + 484_354_048) // 32     # the 32768-row capture scaled by rows (traffic grows with rows)

    def setup(self, dev):
        from ug_b200 import DType, synth
        self.dev = dev
        self.ins = [dev.slice_from_values(self.x if i == 0 else synth.normal(7000 + i, (self.rows, self.cols), 2.0))
                    for i in range(self.pairs)]
        self.outs = [dev.allocate_uninit(DType.F32, self.rows * self.cols) for _ in range(self.pairs)]
        self.xs, self.out = self.ins[0], self.outs[0]
        self.i = 0

    def step(self):
        j = self.i % self.pairs
        self.i += 1
        self.dev.custom_softmax(self.ins[j], self.outs[j], self.rows, self.cols)

    def resident_gbs(self, steps=200):
        for _ in range(5):
            self.dev.custom_softmax(self.xs, self.out, self.rows, self.cols)
        self.dev.synchronize()
        self.dev.timer_begin()
        for _ in range(steps):
            self.dev.custom_softmax(self.xs, self.out, self.rows, self.cols)
        self.dev.timer_end()
        return self.bytes_per_step * steps / (self.dev.timer_elapsed_ms() / 1e3) / 1e9

    def config(self):
        return {"workload": self.name, "rows_per_gpu": self.rows, "cols": self.cols,
                "l2": "16 buffer pairs of 33.5 MB, one per step in turn (537 MB vs 126 MB L2)"}


class GraphRowWorkload:
    """The UNMODIFIED graph forms of ug-llama (softmax, model.rs:94-101; rms_norm, model.rs:65-78) on f32
    [8192, 4096] through the lazy graph -> schedule -> compile -> run path of the host layer: what the drop-in
    backend makes of ug-core's own op graph (the reference lowers the same graphs to scalar code, two kernels
    for softmax)."""
    unit = "GB/s"
    dtype = "f32"
    bound = "hbm"
    rows, cols = 8192, 4096
    ncu_traffic_bytes = None
    kernel_only = True

    def __init__(self, which):
        from ug_b200 import synth
        self.which = which
        self.name = f"graph {which} f32 [8192,4096] through LazyBuffer / Schedule (unmodified ug-llama graph form)"
        self.metric = f"effective HBM GB/s, graph-form {which} (rows*cols*8 bytes / time)"
        self.x = synth.normal(31, (self.rows, self.cols), 2.0 if which == "softmax" else 1.0)
        self.w = synth.uniform(32, (self.cols,), 0.5, 1.5)
        self.bytes_per_step = 2 * self.rows * self.cols * 4
        self.launches_per_step = 1

    def setup(self, dev):
        from ug_b200 import llama_graph as G
        from ug_b200.lazy import LB, HostDevice, Schedule
        self.dev = dev
        self.hd = HostDevice(dev)
        lx = LB.copy(self.x, (self.rows, self.cols), self.hd)
        self.y = G.softmax(lx) if self.which == "softmax" else G.rms_norm(lx, LB.copy(self.w, (self.cols,), self.hd), 1e-5)
        self.sched = Schedule.create_one(self.y)
        self.compiled = self.sched.compile()
        self.launches_per_step = len(self.compiled)

    def step(self):
        self.compiled.run()

    def units(self, step_seconds, n_ranks):
        return n_ranks * self.bytes_per_step / step_seconds / 1e9

    def check(self):
        import oracle
        got = self.y.data_vec().reshape(self.rows, self.cols)[:32]
        ref = oracle.custom_softmax(self.x[:32]) if self.which == "softmax" else oracle.gen_rms_norm(self.x[:32], self.w, 1e-5)
        return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 1e-30)))

    def config(self):
        return {"workload": self.name, "rows_per_gpu": self.rows, "cols": self.cols,
                "l2": "inputs larger than L2 (268 MB touched per step vs 126 MB L2)"}


class LlamaOpsWorkload:
    """The operators of ug_llama::Device and the small map kernels, each alone at HBM size (f32): rope and rope_i
    (ug-llama/src/cpu_ops.rs:58-127) on [32, 32, 512, 64], cat (cpu_ops.rs:129-167) of two [8192, 4096] along the
    last axis, causal_mask (cpu_ops.rs:33-56) on [32, 1024, 1024], index_select (model.rs:32-63) of 16384 rows of a
    [32000, 2048] table, add and silu(gate) * up on 2^25 elements.  One value per operator: algorithmic bytes
    (every input element read once, every output element written once) / time; parity bit-exact or 1e-6."""
    unit = "GB/s"
    dtype = "f32"
    bound = "hbm"
    kernel_only = True
    ncu_traffic_bytes = None
    name = "rope, rope_i, cat, causal_mask, index_select, add, silu_mul f32, each alone on 134-402 MB per launch"
    metric = "effective HBM GB/s per operator (algorithmic bytes / time)"

    def __init__(self, rank=0):
        self.launches_per_step = 1

    def setup(self, dev):
        from ug_b200 import DType, synth
        self.dev = dev
        A = lambda n: dev.allocate_uninit(DType.F32, n)
        b, h, t, d = 32, 32, 512, 64
        n = b * h * t * d                                   # 2^25 elements = 134 MB
        self.x = synth.normal(41, (n,))
        self.y = synth.normal(42, (n,))
        xs, ys, out = dev.slice_from_values(self.x), dev.slice_from_values(self.y), A(n)
        pos_max = 1024
        ang = np.outer(np.arange(pos_max, dtype=np.float32), (1.0 / 10000.0 ** (np.arange(0, d, 2, dtype=np.float32) / d)))
        self.cos, self.sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
        cs, sn = dev.slice_from_values(self.cos), dev.slice_from_values(self.sin)
        self.pos = np.array([7], np.int32)
        ps = dev.slice_from_values(self.pos)
        vocab, hid, n_ids = 32000, 2048, 16384
        self.emb = synth.normal(43, (vocab, hid))
        self.ids = synth.tokens(44, (n_ids,), vocab)
        es, ids = dev.slice_from_values(self.emb), dev.slice_from_values(self.ids)
        self.out = out
        self.shape = (b, h, t, d)
        self.ops = {
            "rope": (lambda: dev.rope(xs, cs, sn, ps, out, b, h, t, d), 8 * n),
            "rope_i": (lambda: dev.rope_i(xs, cs, sn, ps, out, b, h, t, d), 8 * n),
            "cat": (lambda: dev.cat(xs, ys, self.big, 8192, 4096, 4096), 16 * n),
            "causal_mask": (lambda: dev.causal_mask(xs, out, 32, 1024, 1024), 8 * n),
            "index_select": (lambda: dev.index_select(es, ids, out, n_ids, hid, vocab), 8 * n_ids * hid),
            "add": (lambda: dev.add(xs, ys, out, n), 12 * n),
            "silu_mul": (lambda: dev.silu_mul(xs, ys, out, n), 12 * n),
        }
        self.big = A(2 * n)                                  # cat output: [8192, 8192]
        self._keep = (xs, ys, cs, sn, ps, es, ids)

    def step(self):
        for f, _ in self.ops.values():
            f()

    def _check(self, name):
        import oracle
        b, h, t, d = self.shape
        n = b * h * t * d
        if name in ("rope", "rope_i"):
            got = self.out.to_vec().reshape(b, h, t, d)[:1, :2]
            fn = oracle.rope if name == "rope" else oracle.rope_i
            return float(np.max(np.abs(got - fn(self.x.reshape(b, h, t, d)[:1, :2], self.cos, self.sin, self.pos))))
        if name == "cat":
            got = self.big.to_vec().reshape(8192, 8192)[:16]
            want = oracle.cat(self.x.reshape(8192, 4096)[:16], self.y.reshape(8192, 4096)[:16], 1)
            return float(np.max(np.abs(got - want)))
        if name == "causal_mask":
            got = self.out.to_vec().reshape(1, 32, 1024, 1024)[:, :1]
            want = oracle.causal_mask(self.x.reshape(1, 32, 1024, 1024)[:, :1])
            return 0.0 if np.array_equal(got, want) else 1.0
        if name == "index_select":
            got = self.out.to_vec().reshape(-1, 2048)[:64]
            return float(np.max(np.abs(got - oracle.index_select(self.emb, self.ids[:64]))))
        if name == "add":
            return float(np.max(np.abs(self.out.to_vec()[:65536] - oracle.gen_add(self.x[:65536], self.y[:65536]))))
        got, want = self.out.to_vec()[:65536], oracle.gen_silu_mul(self.x[:65536], self.y[:65536])
        return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-30)))

    def record(self, dev, warmup, steps, peaks):
        ops = {}
        for name, (f, nbytes) in self.ops.items():
            for _ in range(max(warmup, 3)):
                f()
            dev.synchronize()
            dev.timer_begin()
            for _ in range(steps):
                f()
            dev.timer_end()
            sec = dev.timer_elapsed_ms() / 1e3 / steps
            ops[name] = {"value": round(nbytes / sec / 1e9, 1), "frac": round(nbytes / sec / 1e9 / peaks["hbm"], 4),
                         "us_per_launch": round(sec * 1e6, 2), "bytes_per_launch": nbytes,
                         "parity_max_err": self._check(name)}
        worst = min(ops, key=lambda k: ops[k]["frac"])
        return {"workload": self.name, "metric": self.metric, "unit": self.unit, "dtype": self.dtype, "steps": steps,
                "value": ops[worst]["value"], "value_of": worst, "operators": ops,
                "parity_max_rel_err": max(o["parity_max_err"] for o in ops.values()),
                "roofline": {"bound": "hbm", "achieved": ops[worst]["value"], "peak": peaks["hbm"], "unit": "GB/s",
                             "frac": ops[worst]["frac"], "traffic": None, "peak_source": peaks["source"],
                             "note": "the slowest of the operators; inputs larger than L2"}}

    def config(self):
        return {"workload": self.name}


class GraphDecodeWorkload:
    """ug-llama's own generation loop (ug-llama/src/main.rs:127-169: build the graph of one forward pass, schedule,
    compile_with_cache, run, read the logits, pick the next token) for ONE sequence of the 1.1B shape in f32, exactly
    as the reference runs it, on this backend: the drop-in path a user of ug-core gets without touching the model.
    A step is one generated token, timed on the host around the whole loop body (the graph is rebuilt per token,
    as in the reference); the phases are reported beside it the way main.rs -v prints them."""
    unit = "tokens/s"
    dtype = "f32"
    bound = "hbm"
    kernel_only = True
    ncu_traffic_bytes = None
    prompt_len = 16
    name = ("ug-llama generation loop through LazyBuffer / Schedule / compile_with_cache (unmodified graph, f32 weights), "
            "Llama-1.1B shape, 1 sequence, 16-token prompt")
    metric = "tokens/s, one sequence, graph rebuilt / scheduled / compiled / run per token (host time included)"

    def __init__(self, rank=0):
        from ug_b200 import synth
        from ug_b200.llama import Config
        self.cfg = Config.llama_1b()
        self.w = synth.llama_weights_f32(_weights(self.cfg))
        self.prompt = synth.tokens(21, (1, self.prompt_len), self.cfg.vocab_size)
        # every f32 matrix once per token (the embedding table is read whole as the output projection)
        self.bytes_per_step = sum(v.nbytes for k, v in self.w.items() if v.ndim == 2)
        self.launches_per_step = 1

    def setup(self, dev):
        from ug_b200 import llama_graph as G
        from ug_b200.lazy import CompilationCache, HostDevice
        self.dev = dev
        self.hd = HostDevice(dev)
        self.model = G.Model(self.cfg, self.w, self.hd, custom_softmax_op=False)
        self.cache, self.kv = CompilationCache(), self.model.new_cache()
        self.pos, self.phases, self.trace = 0, [], []
        self._forward(self.prompt)

    def _forward(self, ids):
        from ug_b200.lazy import LB, Schedule
        n = ids.shape[1]
        t = [time.perf_counter()]
        out = self.model.fwd(LB.copy(ids, (1, n), self.hd), LB.copy(np.array([[self.pos]], np.int32), (1, 1), self.hd),
                             self.kv)
        t.append(time.perf_counter())
        sched = Schedule.create_one(out)
        t.append(time.perf_counter())
        misses = self.cache.misses
        compiled = sched.compile(self.cache)
        t.append(time.perf_counter())
        compiled.run()
        self.dev.synchronize()
        t.append(time.perf_counter())
        logits = out.data_vec().reshape(n, self.cfg.vocab_size)[-1]
        self.tok = int(np.argmax(logits))
        t.append(time.perf_counter())
        self.trace.append((ids.copy(), self.pos, logits))
        self.pos += n
        self.compiled = compiled
        self.launches_per_step = len(compiled)
        self.phases.append([1e3 * (b - a) for a, b in zip(t, t[1:])] + [self.cache.misses - misses])

    def step(self):
        self._forward(np.array([[self.tok]], np.int32))

    def units(self, step_seconds, n_ranks):
        return n_ranks / step_seconds

    def check(self):
        """The prompt's last logits and the first two generated tokens' logits against the CPU oracle."""
        import oracle
        from oracle import llama_ref as R
        oracle.set_threads(os.cpu_count())
        ref = R.Model(R.Config(**self.cfg.__dict__), self.w, custom_softmax_op=False)
        cache, worst = ref.new_cache(), 0.0
        for ids, pos, got in self.trace[:3]:
            want = ref.fwd(ids, pos, cache)[0, -1]
            worst = max(worst, float(np.max(np.abs(got - want)) / np.max(np.abs(want))))
        return worst

    def record(self, dev, warmup, steps, peaks):
        for _ in range(max(warmup, 4)):          # the KV-dependent kernels become size-generic on their second sighting
            self.step()
        self.phases = []
        dev.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            self.step()
        step_s = (time.perf_counter() - t0) / steps
        ph = np.array(self.phases, np.float64)
        origins = {}
        for o in self.compiled.origins():
            origins[o] = origins.get(o, 0) + 1
        rec = {"workload": self.name, "metric": self.metric, "value": round(1.0 / step_s, 2), "unit": self.unit,
               "ms_per_step": round(step_s * 1e3, 3), "ms_per_step_median": round(float(np.median(ph[:, :5].sum(axis=1))), 3),
               "steps": steps, "dtype": self.dtype,
               "phases_ms": dict(zip(["build_graph", "schedule", "compile_with_cache", "run", "read_logits"],
                                     [round(float(x), 3) for x in np.median(ph[:, :5], axis=0)])),
               "compile_misses_in_timed_steps": int(ph[:, 5].sum()), "poly_hits_total": int(self.cache.poly_hits),
               "launches_per_step": self.launches_per_step, "kernels": origins,
               "cached_positions": [self.pos - steps, self.pos],
               "roofline": {"bound": "hbm", "achieved": round(self.bytes_per_step / step_s / 1e9, 1), "peak": peaks["hbm"],
                            "unit": "GB/s", "frac": round(self.bytes_per_step / step_s / 1e9 / peaks["hbm"], 4),
                            "traffic": None, "peak_source": peaks["source"],
                            "note": "f32 weight bytes per token / whole loop-body time; the loop is host- and launch-bound"},
               "parity_max_rel_err": self.check()}
        return rec

    def config(self):
        return {"workload": self.name, "sequences": 1, "prompt": self.prompt_len}


class F32MatmulWorkload:
    """f32 matmul_t on the FP32 pipe (the dtype ug-llama casts every weight to, model.rs:118,140,313): the
    128 x 128 register-blocked kernel on 4096^3 ("gemm_f32", FP32-pipe bound) or the warp-per-column kernel on one
    activation row against the [32000, 2048] embedding ("gemv_f32", HBM bound on the weight)."""
    dtype = "f32"
    kernel_only = True
    ncu_traffic_bytes = None
    FP32_PEAK_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12       # SMs x FP32 lanes x 2 flop x max SM clock

    def __init__(self, which):
        from ug_b200 import synth
        self.which = which
        self.m, self.n, self.k = (4096, 4096, 4096) if which == "gemm_f32" else (1, 32000, 2048)
        self.name = f"f32 matmul_t [{self.m},{self.k}] x [{self.n},{self.k}]^T on the FP32 pipe"
        self.a = synth.normal(41, (1, self.m, self.k), 0.5)
        self.b = synth.normal(42, (1, self.n, self.k), 0.5)
        self.flops_per_step = 2 * self.m * self.n * self.k
        self.bytes_per_step = 4 * (self.n * self.k + self.m * self.k + self.m * self.n)
        self.launches_per_step = 1
        self.bound = "fp32" if which == "gemm_f32" else "hbm"
        self.unit = "TFLOP/s" if which == "gemm_f32" else "GB/s"
        self.metric = "f32 GEMM TFLOP/s (FP32 pipe, fp32 products and sums)" if which == "gemm_f32" else \
            "effective HBM GB/s of the f32 weight stream (decode-shaped matmul_t)"

    def setup(self, dev):
        from ug_b200 import DType
        self.dev = dev
        self.sa, self.sb = dev.slice_from_values(self.a), dev.slice_from_values(self.b)
        self.dst = dev.allocate_uninit(DType.F32, self.m * self.n)
        m, n, k = self.m, self.n, self.k
        self.args = (self.dst, self.sa, self.sb, (1, m, n, k), ([1, m, k], [m * k, k, 1], 0), ([1, k, n], [n * k, 1, k], 0))

    def step(self):
        self.dev.matmul(*self.args)

    def units(self, step_seconds, n_ranks):
        if self.which == "gemm_f32":
            return n_ranks * self.flops_per_step / step_seconds / 1e12
        return n_ranks * self.bytes_per_step / step_seconds / 1e9

    def check(self):
        import oracle
        rows = slice(0, min(self.m, 8))
        got = self.dst.to_vec().reshape(self.m, self.n)[rows]
        ref = oracle.matmul(self.a[0, rows], self.b[0], transpose_rhs=True)
        return float(np.max(np.abs(got - ref)) / (np.sqrt(self.k) * 0.25))

    def config(self):
        return {"workload": self.name, "m": self.m, "n": self.n, "k": self.k,
                "l2": "operands of 64 MB or more per launch" if self.which == "gemm_f32" else "262 MB weight read per launch vs 126 MB L2"}


class GemmWorkload:
    """Config 3: A bf16 [16,512,4096] x B bf16 [4096,4096] ([k,n]), fp32 accumulate, bf16 out."""
    name = "bf16 matmul [16,512,4096] x [4096,4096] (config 3), batch partitioned across GPUs"
    metric = "bf16 GEMM TFLOP/s (2*b*m*n*k / time), fp32 accumulate"
    unit = "TFLOP/s"
    dtype = "bf16"
    bound = "tensor"
    bs, m, n, k = 16, 512, 4096, 4096
    ncu_traffic_bytes = 111_407_616 + 47_598_336       # ncu capture of this shape (each operand once; part of C still in L2)

    def __init__(self, rank):
        from ug_b200 import synth
        self.a = synth.to_bf16_bits(synth.normal(4 + 1000 * rank, (self.bs, self.m, self.k), 0.02))
        self.b = synth.to_bf16_bits(synth.normal(5, (self.k, self.n), 0.02))
        self.flops_per_step = 2 * self.bs * self.m * self.n * self.k
        self.h2d_bytes = self.a.nbytes + self.b.nbytes
        self.d2h_bytes = self.bs * self.m * self.n * 2
        self.launches_per_step = 1
        # operands + result (201 MB) exceed L2 only marginally: rotate over 3 A / C buffers
        self.rot = 3

    def setup(self, dev):
        from ug_b200 import DType
        self.dev = dev
        self.a_s = [dev.slice_from_values(self.a, bf16=True) for _ in range(self.rot)]
        self.b_s = dev.slice_from_values(self.b, bf16=True)
        self.c_s = [dev.allocate_uninit(DType.BF16, self.bs * self.m * self.n) for _ in range(self.rot)]
        self.i = 0
        bs, m, n, k = self.bs, self.m, self.n, self.k
        self.lhs_l = ([bs, m, k], [m * k, k, 1], 0)
        self.rhs_l = ([bs, k, n], [0, n, 1], 0)

    def step(self):
        j = self.i % self.rot
        self.i += 1
        self.dev.matmul(self.c_s[j], self.a_s[j], self.b_s, (self.bs, self.m, self.n, self.k),
                        self.lhs_l, self.rhs_l)

    def units(self, step_seconds, n_ranks):
        return n_ranks * self.flops_per_step / step_seconds / 1e12

    def setup_e2e(self):
        import ctypes as C
        from ug_b200._lib import lib
        self._pin = []
        def pinned(arr):
            p = C.c_void_p()
            assert lib.ugb_host_alloc(arr.nbytes, C.byref(p)) == 0
            np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint16)), shape=(arr.size,))[:] = arr.ravel()
            self._pin.append(p)
            return p
        self.pa, self.pb = pinned(self.a), pinned(self.b)
        self.pc = pinned(np.zeros(self.bs * self.m * self.n, np.uint16))

    def e2e_step(self):
        from ug_b200 import DType
        from ug_b200._lib import lib
        d, bf = self.dev, int(DType.BF16)
        d._check(lib.ugb_h2d_async(self.a_s[0]._h, self.pa, self.a.size, bf))
        d._check(lib.ugb_h2d_async(self.b_s._h, self.pb, self.b.size, bf))
        self.dev.matmul(self.c_s[0], self.a_s[0], self.b_s, (self.bs, self.m, self.n, self.k),
                        self.lhs_l, self.rhs_l)
        d._check(lib.ugb_d2h_async(self.c_s[0]._h, self.pc, self.bs * self.m * self.n, bf))
        d.synchronize()

    def teardown_e2e(self):
        from ug_b200._lib import lib
        for p in self._pin:
            lib.ugb_host_free(p)

    def check(self):
        import oracle
        from ug_b200 import synth
        got = synth.bf16_bits_to_f32(self.c_s[0].to_vec()).reshape(self.bs * self.m, self.n)[:32]
        ref = oracle.matmul(synth.bf16_bits_to_f32(self.a).reshape(-1, self.k)[:32],
                            synth.bf16_bits_to_f32(self.b))
        return float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 0.05 * np.abs(ref).max())))

    def cpu_sample(self, budget_s):
        """f32 GEMM stand-in for crate gemm 0.18.0 on bf16-rounded inputs, all host threads."""
        import oracle
        from ug_b200 import synth
        a = synth.bf16_bits_to_f32(self.a).reshape(-1, self.k)
        b = synth.bf16_bits_to_f32(self.b)
        threads = oracle.set_threads(os.cpu_count())
        rows = 64
        t0 = time.perf_counter()
        oracle.matmul(a[:rows], b)
        per_row = (time.perf_counter() - t0) / rows
        rows = int(max(64, min(a.shape[0], budget_s / per_row)))
        t0 = time.perf_counter()
        oracle.matmul(a[:rows], b)
        dt = time.perf_counter() - t0
        return 2 * rows * self.n * self.k / dt / 1e12, threads, \
            f"{rows} of {a.shape[0]} lhs rows, f32 GEMM stand-in for crate gemm, {threads} threads, {dt:.1f} s"

    def config(self):
        return {"workload": self.name, "batch_per_gpu": self.bs, "m": self.m, "n": self.n, "k": self.k,
                "l2": "rotates over 3 lhs/result buffer pairs (604 MB) so that no operand tile is L2-resident from the previous step"}


class DecodeWorkload:
    """Config 5: Llama-1.1B shape, ONE batch of 64 sequences whose KV cache is pre-filled to 2048 positions
    from seeded random prompts, greedy decoding.  `seqs = (lo, hi)`: this rank owns sequences lo .. hi - 1 of
    that batch (strong scaling, no collective).  `seqs = None`: the rank owns a full batch of 64 of its own
    (weak scaling; rank-seeded prompts).  `tp = (rank, size)`: head-sharded tensor-parallel variant, every
    rank sees all 64 sequences."""
    metric = "tokens/s, Llama-1.1B-shape decode (batch 64, KV depth 2048+)"
    unit = "tokens/s"
    dtype = "bf16"
    bound = "hbm"
    total_batch, prefill = 64, 2048
    step_is_graph = True

    def __init__(self, rank, prefill=None, layers=None, fast_prefill=False, tp=None, seqs=None):
        self.fast_prefill = fast_prefill
        self.tp = tp
        self.seqs = seqs
        from ug_b200 import synth
        from ug_b200.llama_config import Config
        self.cfg = Config.llama_1b()
        if layers:
            self.cfg.num_hidden_layers = layers
        if prefill is not None:
            self.prefill = prefill
        self.rank = rank
        self.weights = _weights(self.cfg)                       # replicated on every GPU
        if tp is not None or seqs is not None:                  # one global batch, the same on every rank
            prompts = synth.tokens(8, (self.total_batch, self.prefill), self.cfg.vocab_size)
            self.prompts = prompts if seqs is None else np.ascontiguousarray(prompts[seqs[0]:seqs[1]])
        else:
            self.prompts = synth.tokens(8 + 1000 * rank, (self.total_batch, self.prefill), self.cfg.vocab_size)
        self.batch = self.prompts.shape[0]
        c = self.cfg
        per_layer = (c.hidden_size * (c.hidden_size + 2 * c.num_key_value_heads * c.head_dim())
                     + c.hidden_size * c.hidden_size + 3 * c.hidden_size * c.intermediate_size)
        self.weight_bytes = 2 * (per_layer * c.num_hidden_layers + c.vocab_size * c.hidden_size)
        self.kv_bytes_per_pos = c.num_hidden_layers * 2 * c.num_key_value_heads * c.head_dim() * 2
        self.h2d_bytes = self.batch * 4
        self.d2h_bytes = self.batch * 4
        self.launches_per_step = 1 + 7 * c.num_hidden_layers + 3

    @property
    def name(self):
        how = ("64 sequences per GPU" if self.seqs is None and self.tp is None else
               "ONE batch of 64 sequences" + (", heads / FFN columns / vocabulary sharded" if self.tp is not None
                                              else ", sequences sharded across the GPUs"))
        return ("Llama-1.1B-shape greedy decode (dim 2048, 22 layers, 32q/4kv heads, ffn 5632, vocab 32000, "
                "bf16 weights + bf16 KV), %s, cache pre-filled to %d positions" % (how, self.prefill))

    def setup(self, dev, total_steps=256, group=None):
        from ug_b200.llama import Model
        self.dev = dev
        self.t_max = self.prefill + total_steps + 16
        self.model = Model.new(self.cfg, self.weights, dev, self.batch, self.t_max, tp=self.tp, group=group)
        if self.tp is not None:
            # per-rank bytes of a step: the rank's share of the layer weights, the embedding slice it
            # multiplies by, and its KV heads
            n = self.tp[1]
            c = self.cfg
            self.weight_bytes = (self.weight_bytes - 2 * c.vocab_size * c.hidden_size) // n + 2 * c.vocab_size * c.hidden_size // n
            self.kv_bytes_per_pos = self.kv_bytes_per_pos * self.model.kv_heads_local // c.num_key_value_heads
        self.model.reset(0)
        if self.fast_prefill:
            self.model.fwd(self.prompts[:, 0])
            self.model.reset(self.prefill)
        else:
            # pre-fill (untimed): the prompts go through the causal prefill path
            self.model.prefill(self.prompts)
        dev.synchronize()
        self.steps_done = 0

    def close(self):
        self.model.close()

    def step(self):
        self.model.decode(1)
        self.steps_done += 1

    def mean_depth(self, first_pos, n_steps):
        return first_pos + (n_steps - 1) / 2.0 + 1

    def step_bytes(self, depth):
        """Algorithmic HBM bytes of one step on this GPU: its weight replica (or share) + its sequences' KV."""
        return self.weight_bytes + self.kv_bytes_per_pos * depth * self.batch

    def setup_e2e(self):
        import ctypes as C
        from ug_b200 import DType
        from ug_b200._lib import lib
        self._pin = []
        for attr in ("p_in", "p_out"):
            p = C.c_void_p()
            assert lib.ugb_host_alloc(self.batch * 4, C.byref(p)) == 0
            setattr(self, attr, p)
            self._pin.append(p)
        self.tok_slice = self.dev.allocate_uninit(DType.I32, self.batch)
        self.host_in = np.ctypeslib.as_array(C.cast(self.p_in, C.POINTER(C.c_int32)), shape=(self.batch,))
        self.host_out = np.ctypeslib.as_array(C.cast(self.p_out, C.POINTER(C.c_int32)), shape=(self.batch,))
        self.host_in[:] = self.model.next_tokens()

    def e2e_step(self):
        """One step the way a caller with host buffers drives it: token ids host -> device,
        the decode step, chosen ids device -> host, every step."""
        from ug_b200 import DType
        from ug_b200._lib import lib
        d = self.dev
        d._check(lib.ugb_h2d_async(self.tok_slice._h, self.p_in, self.batch, int(DType.I32)))
        d._check(lib.ugb_llama_decode(self.model._h, self.tok_slice._h, 1))
        d._check(lib.ugb_llama_read(self.model._h, 1, self.p_out, self.batch))     # blocking D2H
        self.host_in[:] = self.host_out
        self.steps_done += 1

    def teardown_e2e(self):
        from ug_b200._lib import lib
        for p in self._pin:
            lib.ugb_host_free(p)

    def check(self):
        """Logit parity at the depth the run ended at (2048 + the steps taken), against the CPU oracle of
        ug-llama on the same weights: for the first and the last sequence of this GPU, the oracle takes the KV
        cache as the GPU holds it (bf16 widened to f32), decodes the GPU's next greedy token through all layers
        and its logits are compared with the GPU's next step (max |diff| / max |logit|).  The tensor-parallel
        variant, whose ranks hold a share of the KV heads each, keeps the shallow form: 4 teacher-forced
        positions from an empty cache."""
        if self.tp is not None:
            return self.check_shallow(), "4 teacher-forced positions from an empty cache, 2 sequences"
        from ug_b200 import synth
        ref = self._oracle()
        c, m = self.cfg, self.model
        depth = m.position
        seqs = sorted({0, self.batch - 1})
        tok = m.next_tokens()
        caches = {b: [] for b in seqs}
        for l in range(c.num_hidden_layers):
            k, v = m.kv_cache(l, 0), m.kv_cache(l, 1)
            for b in seqs:
                caches[b].append([synth.bf16_bits_to_f32(k[b:b + 1, :, :depth]).copy(),
                                  synth.bf16_bits_to_f32(v[b:b + 1, :, :depth]).copy()])
        m.decode(1)
        got = m.logits()
        worst = 0.0
        for b in seqs:
            want = ref.fwd(np.array([[tok[b]]], np.int32), depth, caches[b])[0, 0]
            worst = max(worst, float(np.max(np.abs(got[b] - want)) / np.max(np.abs(want))))
        return worst, ("one greedy step at cache depth %d, %d sequence(s), all %d layers, oracle fed the cache "
                       "read back from the GPU" % (depth, len(seqs), c.num_hidden_layers))

    def check_shallow(self):
        ref = self._oracle()
        caches = {b: ref.new_cache() for b in (0, self.batch - 1)}
        worst = 0.0
        self.model.reset(0)
        for i in range(4):
            self.model.fwd(self.prompts[:, i])
            got = self.model.logits()                       # a tensor-parallel rank holds its vocabulary slice
            v0, nv = self.model.vocab_offset, self.model.vocab_local
            for b, cache in caches.items():
                want = ref.fwd(self.prompts[b:b + 1, i:i + 1], i, cache)[0, 0]
                worst = max(worst, float(np.max(np.abs(got[b] - want[v0:v0 + nv])) / np.max(np.abs(want))))
        return worst

    def _oracle(self):
        if getattr(self, "_ref", None) is None:
            import oracle
            from oracle import llama_ref as R
            self.cpu_threads = oracle.set_threads(os.cpu_count())
            from ug_b200 import synth
            self._ref = R.Model(R.Config(**self.cfg.__dict__), synth.llama_weights_f32(self.weights))
        return self._ref

    def cpu_sample(self, budget_s):
        """ug-llama's forward on the CPU oracle: one sequence, one new token per step, against a
        cache of `prefill` positions filled with N(0,1) keys/values (the cost of a step does not
        depend on the cached values); tokens/s of that single sequence.  One sequence because that is
        all the reference model runs (batch 1: ug-core/src/lazy_buffer.rs:432-436, ug-llama/src/model.rs:192-193)."""
        from ug_b200 import synth
        c = self.cfg
        ref = self._oracle()
        cache = [[synth.normal(50 + l, (1, c.num_key_value_heads, self.prefill, c.head_dim())),
                  synth.normal(90 + l, (1, c.num_key_value_heads, self.prefill, c.head_dim()))]
                 for l in range(c.num_hidden_layers)]
        tok = np.array([[1]], np.int32)
        ref.fwd(tok, self.prefill, cache)                       # warm-up
        n, t0 = 0, time.perf_counter()
        while True:
            logits = ref.fwd(tok, self.prefill + 1 + n, cache)
            tok = np.array([[int(logits[0, 0].argmax())]], np.int32)
            n += 1
            dt = time.perf_counter() - t0
            if dt > budget_s or n >= 64:
                break
        return n / dt, self.cpu_threads, (f"{n} greedy tokens of 1 sequence (the reference model runs batch 1 only) at KV depth "
                                          f"{self.prefill}+, oracle of ug-llama's CPU path (f32, GEMM stand-in on "
                                          f"{self.cpu_threads} threads), {dt:.1f} s")

    def config(self, world=1):
        if self.tp is not None:
            par = f"tp{self.tp[1]} (heads, FFN columns and vocabulary sharded; cross-rank sums over NVLink peer memory)"
        elif self.seqs is not None:
            par = f"dp{world} (sequences of one batch sharded, weights replicated, no collective)"
        else:
            par = f"dp{world} (a batch of 64 per GPU, no collective)"
        total = self.total_batch * (world if self.seqs is None and self.tp is None else 1)
        return {"workload": self.name, "parallelism": par, "sequences_total": total,
                "sequences_per_gpu": self.batch, "prefill": self.prefill,
                "layers": self.cfg.num_hidden_layers, "fast_prefill": self.fast_prefill,
                "l2": "inputs larger than L2 (2.07 GB weights + 47.6 MB of KV per sequence read per step vs 126 MB L2)"}


_WEIGHTS = {}


def _weights(cfg):
    """Synthetic weights of a configuration, generated once per process."""
    from ug_b200 import synth
    key = tuple(sorted(cfg.__dict__.items()))
    if key not in _WEIGHTS:
        _WEIGHTS[key] = synth.llama_weights(cfg)
    return _WEIGHTS[key]


class PrefillWorkload(DecodeWorkload):
    """Config 4: Llama-1.1B shape, 8 sequences x 512 prompt positions per GPU through the causal
    prefill path (Model::fwd with seq_len > 1), last-position logits and next tokens as the result."""
    name = ("Llama-1.1B-shape prefill (dim 2048, 22 layers, 32q/4kv heads, ffn 5632, vocab 32000, bf16 weights + "
            "bf16 KV), 8 sequences x 512 positions per GPU")
    metric = "tokens/s, Llama-1.1B-shape prefill (8 x 512 per GPU)"
    unit = "tokens/s"
    dtype = "bf16"
    bound = "tensor"
    sustained_peak = True          # ~200 kernels per step, seconds of back-to-back GEMMs: sustained bf16 figure
    total_batch, prefill = 8, 512
    step_is_graph = False

    def __init__(self, rank, prefill=None, layers=None, fast_prefill=False):
        super().__init__(rank, prefill=prefill, layers=layers)
        c = self.cfg
        t = self.prefill
        rows = self.batch * t
        # projections: 2 flops per weight per row (lm_head on the last position only);
        # attention: QK^T and PV over the causal half, 4 * head_dim flops per (query, key, head)
        self.flops_per_step = (2 * rows * (self.weight_bytes // 2 - c.vocab_size * c.hidden_size)
                               + 2 * self.batch * c.vocab_size * c.hidden_size
                               + c.num_hidden_layers * 4 * c.head_dim() * c.num_attention_heads * self.batch * t * (t + 1) // 2)
        self.h2d_bytes = rows * 4
        self.d2h_bytes = self.batch * 4
        self.launches_per_step = 1 + 9 * c.num_hidden_layers + 3

    def setup(self, dev):
        from ug_b200 import DType
        from ug_b200.llama import Model
        self.dev = dev
        self.model = Model.new(self.cfg, self.weights, dev, self.batch, self.prefill)
        for name, value in getattr(self, "options", {}).items():
            self.model.set_option(name, value)
        self.tok_dev = dev.slice_from_values(self.prompts.reshape(-1))
        dev.synchronize()

    def step(self):
        self.model.reset(0)
        self.model.prefill(self.tok_dev)

    def units(self, step_seconds, n_ranks):
        return n_ranks * self.batch * self.prefill / step_seconds

    def setup_e2e(self):
        import ctypes as C
        from ug_b200._lib import lib
        n = self.batch * self.prefill
        self._pin = []
        for attr, cnt in (("p_in", n), ("p_out", self.batch)):
            p = C.c_void_p()
            assert lib.ugb_host_alloc(cnt * 4, C.byref(p)) == 0
            setattr(self, attr, p)
            self._pin.append(p)
        self.host_in = np.ctypeslib.as_array(C.cast(self.p_in, C.POINTER(C.c_int32)), shape=(n,))
        self.host_in[:] = self.prompts.reshape(-1)

    def e2e_step(self):
        """Prompt ids host -> device, the prefill, chosen next ids device -> host."""
        from ug_b200 import DType
        from ug_b200._lib import lib
        d = self.dev
        d._check(lib.ugb_h2d_async(self.tok_dev._h, self.p_in, self.batch * self.prefill, int(DType.I32)))
        self.model.reset(0)
        d._check(lib.ugb_llama_prefill(self.model._h, self.tok_dev._h, self.prefill, 0))
        d._check(lib.ugb_llama_read(self.model._h, 1, self.p_out, self.batch))     # blocking D2H

    def check(self):
        """Last-position logits of a prefill of the first 48 prompt positions against the CPU oracle of
        ug-llama on the same weights, one sequence (max |diff| / max |logit|)."""
        n = min(48, self.prefill)
        ref = self._oracle()
        want = ref.fwd(self.prompts[3:4, :n], 0, ref.new_cache())[0, -1]
        self.model.reset(0)
        self.model.prefill(self.prompts[:, :n])
        got = self.model.logits()
        return float(np.max(np.abs(got[3] - want)) / np.max(np.abs(want)))

    def cpu_sample(self, budget_s):
        """ug-llama's forward on the CPU oracle over the first positions of one prompt; tokens/s."""
        ref = self._oracle()
        n = 32
        ref.fwd(self.prompts[:1, :8], 0, ref.new_cache())          # warm-up
        done, t0 = 0, time.perf_counter()
        while True:
            ref.fwd(self.prompts[:1, :n], 0, ref.new_cache())
            done += n
            dt = time.perf_counter() - t0
            if dt > budget_s or done >= 512:
                break
        return done / dt, self.cpu_threads, (f"{done} prompt positions in blocks of {n} (one sequence), oracle of ug-llama's "
                                             f"CPU path (f32, GEMM stand-in on {self.cpu_threads} threads), {dt:.1f} s")

    def config(self, world=1):
        return {"workload": self.name, "sequences_per_gpu": self.batch, "prompt_positions": self.prefill,
                "layers": self.cfg.num_hidden_layers,
                "l2": "inputs larger than L2 (2.07 GB of weights read per step vs 126 MB L2)"}


WORKLOADS = {"rms_silu": RmsSiluWorkload, "softmax": SoftmaxWorkload, "softmax_c1": SoftmaxC1Workload,
             "gemm": GemmWorkload, "decode": DecodeWorkload, "prefill": PrefillWorkload,
             "graph_softmax": lambda r: GraphRowWorkload("softmax"), "graph_rms_norm": lambda r: GraphRowWorkload("rms_norm"),
             "gemm_f32": lambda r: F32MatmulWorkload("gemm_f32"), "gemv_f32": lambda r: F32MatmulWorkload("gemv_f32"),
             "graph_decode": GraphDecodeWorkload, "llama_ops": LlamaOpsWorkload}
DEFAULT_WORKLOAD = "decode"

# DRAM traffic of the decode step's kernels, from ncu captures of single launches (dram__bytes_read.sum +
# dram__bytes_write.sum): the attention kernel moved 141,193,472 B at 2049 cached positions of 64 sequences
# (1.02x its algorithmic bytes; grows in proportion to positions x sequences), the weight-streaming
# projections 1.01-1.03x their weight bytes.  The step's traffic is put together from these, not captured whole.
ATT_TRAFFIC_AT_2049_X64 = 141_193_472
GEMM_TRAFFIC_OVER_WEIGHTS = 1.02


def _config_of(wl, world):
    try:
        return wl.config(world)
    except TypeError:
        return wl.config()


def measure(wl, dev, group, rank, local_rank, warmup, steps, e2e_steps, clocks=True):
    """W warm-up steps, K timed steps (CUDA events on the library's stream, barrier + synchronise on both
    sides), then the end-to-end loop with host buffers; maxima over ranks."""
    def barrier():
        dev.synchronize()
        group.barrier()

    for _ in range(warmup):
        wl.step()
    barrier()
    sampler = ClockSampler(local_rank) if (rank == 0 and clocks) else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    n0 = dev.launch_count
    first_pos = wl.model.position if isinstance(wl, DecodeWorkload) and not isinstance(wl, PrefillWorkload) else 0
    barrier()
    dev.timer_begin()
    for _ in range(steps):
        wl.step()
    dev.timer_end()
    ms = dev.timer_elapsed_ms()
    barrier()
    launches = dev.launch_count - n0
    # end to end: host buffers in, host buffers out, copies inside the timed region
    wl.setup_e2e()
    for _ in range(2):
        wl.e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        wl.e2e_step()
    dev.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()
    clk = sampler.stop() if sampler else None
    wl.teardown_e2e()
    ms, e2e_s = group.max([ms, e2e_s])      # the slowest rank defines the step
    return {"ms": ms, "e2e_s": e2e_s, "launches": int(launches), "first_pos": first_pos, "clocks": clk,
            "steps": steps, "e2e_steps": e2e_steps}


def roofline_of(wl, step_s, peaks):
    launch_s = step_s / wl.launches_per_step
    if wl.bound == "hbm":
        achieved, peak, unit = wl.bytes_per_step / wl.launches_per_step / launch_s / 1e9, peaks["hbm"], "GB/s"
    elif wl.bound == "fp32":
        r = {"bound": "fp32", "achieved": round(wl.flops_per_step / launch_s / 1e12, 2), "peak": round(wl.FP32_PEAK_TFLOPS, 1),
             "unit": "TFLOP/s", "traffic": None, "peak_source": "nominal: SMs x 128 FP32 lanes x 2 x max SM clock"}
        r["frac"] = round(r["achieved"] / r["peak"], 4)
        return r
    else:
        peak = peaks["bf16_sustained"] if getattr(wl, "sustained_peak", False) else peaks["bf16"]
        achieved, unit = wl.flops_per_step / wl.launches_per_step / launch_s / 1e12, "TFLOP/s"
    return {"bound": wl.bound, "achieved": round(achieved, 1), "peak": peak, "unit": unit,
            "frac": round(achieved / peak, 4), "traffic": getattr(wl, "ncu_traffic_bytes", None),
            "peak_source": peaks["source"]}


def parity_of(wl):
    r = wl.check()
    return r if isinstance(r, tuple) else (r, None)


def config_records(dev, group, peaks):
    """One sub-record per benchmark configuration other than the decode step (N = 1): value, roofline
    fraction, DRAM traffic of the kernel and parity against the oracle."""
    out = {}
    plan = [("config1_softmax_1024x4096", SoftmaxC1Workload, 200), ("config1_row_shape_32768x4096", SoftmaxWorkload, 30),
            ("config2_rms_norm_silu_gate", RmsSiluWorkload, 50), ("config3_gemm", GemmWorkload, 30),
            ("config4_prefill", PrefillWorkload, 10),
            ("graph_softmax_8192x4096", lambda r: GraphRowWorkload("softmax"), 30),
            ("graph_rms_norm_8192x4096", lambda r: GraphRowWorkload("rms_norm"), 30),
            ("f32_gemm_4096", lambda r: F32MatmulWorkload("gemm_f32"), 10),
            ("f32_decode_matmul_1x32000x2048", lambda r: F32MatmulWorkload("gemv_f32"), 50),
            ("llama_operators_f32", LlamaOpsWorkload, 20),
            ("graph_decode_llama_1b_f32", GraphDecodeWorkload, 32)]
    for key, cls, steps in plan:
        wl = cls(0)
        wl.setup(dev)
        if hasattr(wl, "record"):
            out[key] = wl.record(dev, 4, steps, peaks)
            del wl
            continue
        for _ in range(3):
            wl.step()
        dev.synchronize()
        dev.timer_begin()
        for _ in range(steps):
            wl.step()
        dev.timer_end()
        step_s = dev.timer_elapsed_ms() / 1e3 / steps
        err, what = parity_of(wl)
        rec = {"workload": wl.name, "metric": wl.metric, "value": round(wl.units(step_s, 1), 2), "unit": wl.unit,
               "ms_per_step": round(step_s * 1e3, 5), "steps": steps, "roofline": roofline_of(wl, step_s, peaks),
               "parity_max_rel_err": err}
        if hasattr(wl, "resident_gbs"):
            rec["l2_resident_value"] = round(wl.resident_gbs(), 1)
        if isinstance(wl, GraphRowWorkload):
            rec["kernels"] = wl.compiled.origins()
        if hasattr(wl, "reference_cuda_gbs") and cls is SoftmaxWorkload:
            g = wl.reference_cuda_gbs()
            rec["reference_cuda_kernel"] = None if g is None else round(g, 1)
        out[key] = rec
        if hasattr(wl, "close"):
            wl.close()
        del wl
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ug_b200", choices=["ug_b200", "reference"])
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="decode: leave out the extra records (configs at N = 1; weak and tp at N > 1)")
    ap.add_argument("--prefill", type=int, default=None, help="decode: cached positions before timing")
    ap.add_argument("--device-option", action="append", default=[], metavar="NAME=INT",
                    help="device tuning switch set before the run (ugb_device_set_option), e.g. gemm_cta_pairs=1")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=INT",
                    help="engine option set before the run (profiling of kernel variants)")
    ap.add_argument("--layers", type=int, default=None, help="decode: layer count (profiling of small cases)")
    ap.add_argument("--weak", action="store_true",
                    help="decode at N > 1: every rank decodes its own 64 sequences (64 N in all) instead of a share of one batch")
    ap.add_argument("--tp", action="store_true",
                    help="decode: tensor-parallel variant -- the ranks share ONE batch of 64 sequences (heads, FFN "
                         "columns and vocabulary sharded, cross-rank sums inside the engine's kernels over NVLink)")
    ap.add_argument("--sequences", type=int, default=None,
                    help="decode, profiling aid: this GPU decodes the first N sequences of the batch only (the share of "
                         "one GPU of a 64 / N-GPU run, on one GPU)")
    ap.add_argument("--fast-prefill", action="store_true",
                    help="decode, profiling aid: place the cache at --prefill positions without running the "
                         "prompts (the cache then holds zeros); not a valid benchmark configuration")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.steps is None:
        args.steps = 128 if args.workload == "decode" else 50

    from ug_b200.dist import env_rank, shard_range
    rank, local_rank, world = env_rank()
    options = dict((k, int(v)) for k, v in (o.split("=") for o in args.option))

    def make_decode(mode):
        if mode == "tp":
            return DecodeWorkload(rank, prefill=args.prefill, layers=args.layers, fast_prefill=args.fast_prefill,
                                  tp=(rank, world))
        if mode == "weak":
            return DecodeWorkload(rank, prefill=args.prefill, layers=args.layers, fast_prefill=args.fast_prefill)
        return DecodeWorkload(rank, prefill=args.prefill, layers=args.layers, fast_prefill=args.fast_prefill,
                              seqs=(0, args.sequences) if args.sequences else shard_range(DecodeWorkload.total_batch, rank, world))

    def make_workload(r):
        if args.workload == "decode":
            return make_decode("tp" if args.tp else ("weak" if args.weak else "strong"))
        if args.workload == "prefill":
            wl = PrefillWorkload(r, prefill=args.prefill, layers=args.layers)
            wl.options = options
            return wl
        return WORKLOADS[args.workload](r)

    if args.impl == "reference":
        if rank != 0:
            return 0
        wl_ref = make_workload(0)
        if not hasattr(wl_ref, "cpu_sample"):
            # the secondary records (kernel-only workloads) carry their own parity figure and have no CPU arm
            print(json.dumps({"impl": "reference", "unavailable": "workload %s is a secondary record without a CPU arm; "
                              "the reference arm covers decode, prefill, softmax, rms_silu and gemm" % args.workload}), flush=True)
            return 0
        return reference_arm(args, wl_ref)

    from ug_b200.dist import Group
    group = Group(backend="nccl" if world > 1 else None)

    import ug_b200
    dev = ug_b200.Device(local_rank)
    for o in args.device_option:
        name, value = o.split("=")
        dev.set_option(name, int(value))
    decode = args.workload == "decode"
    e2e_steps = max(3, min(args.steps, 10 if not decode else 32))
    total_steps = args.warmup + args.steps + e2e_steps + 16

    def run_decode(mode, clocks=True):
        wl = make_decode(mode)
        wl.setup(dev, total_steps=total_steps, group=group)
        for name, value in options.items():
            wl.model.set_option(name, value)
        return wl, measure(wl, dev, group, rank, local_rank, args.warmup, args.steps, e2e_steps, clocks)

    if decode:
        mode = "tp" if args.tp else ("weak" if args.weak else "strong")
        wl, m = run_decode(mode)
    else:
        mode = None
        wl = make_workload(rank)
        wl.setup(dev)
        if hasattr(wl, "record"):
            rec = wl.record(dev, args.warmup, args.steps, measured_peaks())
            rec.update({"n_gpus": 1, "warmup": max(args.warmup, 4), "config": _config_of(wl, 1),
                        "gpu_launches": int(dev.launch_count)})
            if rank == 0:
                print(json.dumps(rec), flush=True)
            group.close()
            return 0
        if getattr(wl, "kernel_only", False):
            # secondary records (no end-to-end leg, no CPU arm): device-timed value, roofline, parity
            for _ in range(args.warmup):
                wl.step()
            dev.synchronize()
            dev.timer_begin()
            for _ in range(args.steps):
                wl.step()
            dev.timer_end()
            step_s = dev.timer_elapsed_ms() / 1e3 / args.steps
            err, _ = parity_of(wl)
            if rank == 0:
                rec = {"metric": wl.metric, "value": round(wl.units(step_s, 1), 2), "unit": wl.unit, "n_gpus": 1,
                       "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(step_s * 1e3, 5), "dtype": wl.dtype,
                       "config": _config_of(wl, 1), "roofline": roofline_of(wl, step_s, measured_peaks()),
                       "parity_max_rel_err": err, "gpu_launches": int(dev.launch_count)}
                if hasattr(wl, "compiled"):
                    rec["kernels"] = wl.compiled.origins()
                print(json.dumps(rec), flush=True)
            group.close()
            return 0
        m = measure(wl, dev, group, rank, local_rank, args.warmup, args.steps, e2e_steps)

    tp = decode and mode == "tp"
    gemm_timeline = None
    if rank == 0 and decode and options.get("gemm_profile"):
        # CTA 0 of each decode projection on its own clock (%globaltimer), microseconds after the projection's wait
        # for the preceding kernel returned: the last launches of the timed loop (qkv / o / gate|up / down of the
        # last layer, lm_head); taken before the per-kernel timing below overwrites the stamps
        from ug_b200._lib import lib
        buf = np.zeros(5 * 64, np.float32)
        dev._check(lib.ugb_llama_read(wl.model._h, 5, buf.ctypes.data, buf.size))
        gemm_timeline = {}
        for name, t in zip(["qkv", "o", "gate_up", "down", "lm_head"], buf.reshape(5, 64)):
            kb = [round(float(x), 2) for x in t[8:] if x != 0]
            gemm_timeline[name] = {
                "cta_start": round(float(t[0]), 2), "wait_returned": 0.0, "k_blocks_complete_at": kb,
                "ns_per_k_block": round(1e3 * (kb[-1] - kb[0]) / (len(kb) - 1), 1) if len(kb) > 1 else None,
                "last_mma_issued": round(float(t[2]), 2), "accumulator_seen": round(float(t[3]), 2),
                "epilogue_done": round(float(t[4]), 2), "tmem_released": round(float(t[5]), 2)}
    kern, kdepth = {}, 0
    if rank == 0 and decode:
        # per-kernel share of one step, each kernel type timed alone over all layers (CUDA events); no exchange inside
        for name in wl.model.KERNELS:
            kern[name] = round(wl.model.time_kernel(name, 20), 4)
        kdepth = wl.model.position                      # cache depth the kernels were timed at
    step_phases = None
    if rank == 0 and decode and options.get("step_kernel") and options.get("step_profile"):
        # the persistent step kernel's own clock: per layer, mean microseconds CTA 0 spends working in each phase and
        # waiting at the grid barrier that ends it (%globaltimer stamps of the last step)
        import ctypes as C
        from ug_b200._lib import lib
        buf = np.zeros(4 * 512, np.float32)
        dev._check(lib.ugb_llama_read(wl.model._h, 4, buf.ctypes.data, buf.size))
        t = buf.reshape(4, 512)[0]
        n_sync = 7 * wl.cfg.num_hidden_layers
        arrive, done = t[1:1 + 2 * n_sync:2], t[2:2 + 2 * n_sync:2]
        start = np.concatenate([[t[0]], done[:-1]])
        names = ["rows1", "qkv", "attention", "o", "rows2", "gate_up", "down"]
        work = (arrive - start).reshape(-1, 7)[1:].mean(0)
        wait = (done - arrive).reshape(-1, 7)[1:].mean(0)
        step_phases = {"work_us": {n: round(float(v), 2) for n, v in zip(names, work)},
                       "barrier_wait_us": {n: round(float(v), 2) for n, v in zip(names, wait)},
                       "kernel_us": round(float(done[-1] - t[0]), 1)}
    dev.synchronize()
    group.barrier()
    # under tensor parallelism every engine call is collective: all ranks run the parity check
    parity, parity_what = parity_of(wl) if (rank == 0 or tp) else (None, None)

    peaks = measured_peaks()
    step_s = m["ms"] / 1e3 / args.steps
    e2e_step_s = m["e2e_s"] / e2e_steps
    line = None
    if rank == 0:
        extra = {}
        if decode:
            n_seq = args.sequences if args.sequences else wl.total_batch * (world if mode == "weak" else 1)
            value, e2e_value = n_seq / step_s, n_seq / e2e_step_s
            depth = wl.mean_depth(m["first_pos"], args.steps)
            gpu_bytes = wl.step_bytes(depth)             # this GPU's algorithmic bytes per step (rank 0 holds the largest share)
            achieved = gpu_bytes / step_s / 1e9
            att_traffic = ATT_TRAFFIC_AT_2049_X64 * (depth / 2049.0) * (wl.batch / 64.0) * wl.cfg.num_hidden_layers
            traffic = None if tp else int(att_traffic + GEMM_TRAFFIC_OVER_WEIGHTS * wl.weight_bytes)
            roof = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm"], "unit": "GB/s",
                    "frac": round(achieved / peaks["hbm"], 4), "traffic": traffic, "peak_source": peaks["source"],
                    "scope": ("whole decode step on one GPU (one CUDA graph of %d kernels): that GPU's weight bytes + its "
                              "sequences' KV bytes at the mean cache depth %.0f; traffic = the per-kernel ncu captures "
                              "(attention at 2049 positions scaled by depth x sequences, projections 1.02 x weights)"
                              % (m["launches"] // max(args.steps, 1), depth))}
            extra["kernels_ms_per_step"] = kern
            att_bytes = wl.kv_bytes_per_pos * kdepth * wl.batch
            extra["decode_attention_roofline"] = {
                "traffic": int(ATT_TRAFFIC_AT_2049_X64 * kdepth / 2049 * wl.batch / 64) if not tp else None,
                "achieved": round(att_bytes / (kern["decode_attention"] / 1e3) / 1e9, 1), "peak": peaks["hbm"],
                "unit": "GB/s", "frac": round(att_bytes / (kern["decode_attention"] / 1e3) / 1e9 / peaks["hbm"], 4)}
            # the bandwidth bound of this split: every GPU re-reads the whole weight replica, so the step cannot
            # be shorter than (weights + this GPU's KV) / HBM bandwidth, whatever N is
            one_gpu = DecodeWorkload.total_batch * wl.kv_bytes_per_pos * depth + wl.weight_bytes
            extra["bound"] = {"bytes_per_gpu_per_step": int(gpu_bytes),
                              "step_floor_ms_at_measured_hbm": round(gpu_bytes / peaks["hbm"] / 1e6, 4),
                              "speedup_bound_vs_1_gpu": None if tp or mode == "weak" else round(one_gpu / gpu_bytes, 3)}
        else:
            value = wl.units(step_s, world)
            e2e_value = wl.units(e2e_step_s, world)
            roof = roofline_of(wl, step_s, peaks)
        line = {
            "metric": wl.metric, "value": round(value, 2), "unit": wl.unit, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(m["ms"] / args.steps, 5),
            "higher_is_better": True, "scaling": "strong" if (decode and mode != "weak") else "weak",
            "vs_baseline": None, "dtype": wl.dtype,
            "data": "synthetic (seeded Philox, shapes and distributions of the named config)",
            "config": _config_of(wl, world),
            "e2e": {"value": round(e2e_value, 3), "unit": wl.unit,
                    "h2d_bytes_per_step": wl.h2d_bytes, "d2h_bytes_per_step": wl.d2h_bytes,
                    "steps": e2e_steps},
            "gpu_launches": m["launches"],
            "clocks": m["clocks"],
            "roofline": roof,
        }
        line.update(extra)
        if step_phases:
            line["step_kernel_phases"] = step_phases
        if gemm_timeline:
            line["gemm_timeline_us"] = gemm_timeline
        if hasattr(wl, "reference_cuda_gbs"):
            g = wl.reference_cuda_gbs()
            line["reference_cuda_kernel"] = None if g is None else {
                "value": round(g, 1), "unit": "GB/s", "what": "ug-llama/src/softmax.cu compiled as is (fast-math), "
                "launched as ug-llama/src/cuda_ops.rs does, same buffers"}
        if hasattr(wl, "resident_gbs"):
            line["l2_resident_value"] = round(wl.resident_gbs(), 1)
        line["parity_max_rel_err"] = parity
        if parity_what:
            line["parity_what"] = parity_what
        if not args.no_cpu_baseline:
            v, cores, sample = wl.cpu_sample(args.cpu_seconds)
            line["cpu_baseline"] = {"value": round(v, 4), "unit": wl.unit, "cores": cores,
                                    "kind": "port", "sample": sample}
            if decode:
                line["cpu_baseline"]["sequences"] = 1

    # extra records of the default run: the other configurations at N = 1, the other two splits at N > 1
    if decode and mode == "strong" and not args.no_extras:
        wl.close()
        del wl
        if world == 1:
            if rank == 0:
                line["configs"] = config_records(dev, group, peaks)
        else:
            for other in ("weak", "tp"):
                owl, om = run_decode(other, clocks=False)
                o_step = om["ms"] / 1e3 / args.steps
                n_seq = owl.total_batch * (world if other == "weak" else 1)
                if rank == 0:
                    depth = owl.mean_depth(om["first_pos"], args.steps)
                    b = owl.step_bytes(depth)
                    line[other] = {"value": round(n_seq / o_step, 2), "unit": "tokens/s", "sequences_total": n_seq,
                                   "ms_per_step": round(o_step * 1e3, 5),
                                   "e2e_value": round(n_seq / (om["e2e_s"] / e2e_steps), 2),
                                   "config": _config_of(owl, world),
                                   "roofline_frac": round(b / o_step / 1e9 / peaks["hbm"], 4),
                                   "bytes_per_gpu_per_step": int(b)}
                owl.close()
                del owl
                dev.synchronize()
                group.barrier()
    if rank == 0:
        print(json.dumps(line), flush=True)
    group.close()
    return 0


def reference_arm(args, wl):
    """The reference's own CPU implementation of the path (oracle port), bounded sample per step."""
    per_step = max(0.5, min(20.0, 120.0 / (args.steps + args.warmup)))
    vals, cores, sample = [], 1, ""
    for i in range(args.warmup + args.steps):
        v, cores, sample = wl.cpu_sample(per_step)
        if i >= args.warmup:
            vals.append(v)
    value = float(np.mean(vals))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    line = {
        "impl": "reference", "metric": wl.metric, "value": round(value, 4), "unit": wl.unit,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": None,
        "higher_is_better": True, "scaling": "strong" if isinstance(wl, DecodeWorkload) and not isinstance(wl, PrefillWorkload) else "weak",
        "vs_baseline": None, "dtype": wl.dtype,
        "data": "synthetic (seeded Philox, shapes and distributions of the named config)",
        "config": _config_of(wl, world),
        "cpu_baseline": {"value": round(value, 4), "unit": wl.unit, "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": round(value, 4), "unit": wl.unit, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    if isinstance(wl, DecodeWorkload) and not isinstance(wl, PrefillWorkload):
        line["cpu_baseline"]["sequences"] = 1
        line["note"] = ("the reference model decodes one sequence at a time (batch 1 only), so this is tokens/s of ONE "
                        "sequence on the host cores; the GPU arm's value is over the 64 sequences of the batch")
    print(json.dumps(line), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
