#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4|c1|c2|c3|large] [--impl ours|reference]

Prints ONE JSON line.  A "step" is one pass of the hot path over one batch of seeded synthetic input
with the shapes and value distributions of the benchmark configurations:

  c4 (default)  Whisper-large-v3-shaped model (32+32 layers, d_model 1280, 20 heads, FFN 5120, vocabulary
                51866), random weights, every linear layer W4A16 g128 round-to-nearest; a step transcribes a
                batch of 32 thirty-second windows (128-bin log-mel, 3000 frames), 128 greedy tokens each.
                metric: RTFx = seconds of audio / seconds of wall time.
  c1            one W4A16 layer, g128, K=1280 N=5120 M=1500 (+bias).  metric: TFLOP/s of 2*M*N*K.
  c2            one W4A4 layer: online Hadamard-4096 + per-token int4 activations, int4 g128 weights,
                K=4096 N=1024 M=6000.  metric: int TOP/s of 2*M*N*K.
  c3            W4A16/W2A16 decode sweep, hidden 2048 / intermediate 6144 shapes, M in {1,2,4,8,16}, g64.
                metric: GB/s of algorithmic bytes.

Every workload reports ``roofline`` (dominant kernel, timed live with CUDA events), ``cpu_baseline``
(the reference's own code on the host cores where it can run there, else its CPU restatement),
``e2e`` (the same metric through the public API from pinned HOST buffers, copies timed) and
``parity_checked`` (outputs of the timed configuration compared with the CPU oracle before timing).
The default run prints the c4 line with the other workloads under ``also``.

With N > 1 (torchrun) every rank runs the same step on its own replica of the weights and its own
batch (weak scaling, no data-path collective); the time is the maximum over ranks.  c4 additionally
reports the strong-scaling figure (the 32 utterances of ONE batch divided among the ranks).

``--impl reference`` times the reference's CPU implementation on a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024
MIN_TIMED_MS = 50.0     # a timed region shorter than this is repeated until it is not
E2E_CHUNKS = int(os.environ.get("ASRQ_BENCH_E2E_CHUNKS", "4"))  # token chunks of the host-to-host layer call (1: no overlap)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def recorded_traffic(kernel: str):
    """DRAM bytes of one launch of ``kernel`` from the ncu capture summarised under profiles/, or None when
    the kernel's sources have changed since the capture (the figure would be stale)."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(path):
        return None
    ent = json.load(open(path)).get(kernel)
    if not ent:
        return None
    for rel, sha in ent.get("sources", {}).items():
        p = os.path.join(ROOT, rel)
        if not os.path.exists(p) or hashlib.sha256(open(p, "rb").read()).hexdigest()[:16] != sha:
            return None
    return ent


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def event():
    e = torch.cuda.Event(enable_timing=True)
    e.record()
    return e


def capture_graph(fn):
    """Runs ``fn`` once eagerly on a side stream, then captures it there as a CUDA graph."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    return g


class GraphSteps:
    """K consecutive steps of a kernel-only workload as CUDA-graph replays.

    Issued call by call from Python such a step is bound by the host (a ctypes call and a launch cost as
    much as these kernels run), so steps are captured: one graph holds ``group`` consecutive steps, each on
    its own input set (inside it consecutive launches chain with programmatic dependent launch, as they do
    in a model's layer sequence), and single-step graphs serve the remainder, so exactly K steps run."""

    def __init__(self, step_fn, nsets: int, group: int):
        self.nsets, self.group = nsets, max(1, group)
        self.big = capture_graph(lambda: [step_fn(i % nsets) for i in range(self.group)]) if self.group > 1 else None
        self.single = [capture_graph(lambda i=i: step_fn(i)) for i in range(nsets)]

    def run(self, k: int):
        n_big = k // self.group if self.big is not None else 0
        for _ in range(n_big):
            self.big.replay()
        for i in range(k - n_big * self.group):
            self.single[i % self.nsets].replay()


# ------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------


class Workload:
    name = metric = unit = dtype = ""
    launches_per_step = 0
    graph_steps = True      # False: step() is called directly (it manages its own graphs)
    default_group = 1

    def units_scale(self):
        return 1e12 if self.unit in ("TOP/s", "TFLOP/s") else (1e9 if self.unit == "GB/s" else 1.0)

    def value_from(self, ms_per_step: float, world: int) -> float:
        return self.units_per_step() * world / (ms_per_step * 1e-3) / self.units_scale()


def _rows_ok(y, ref, rel=2e-3, extra=None):
    tol = rel * ref.abs().max(dim=-1, keepdim=True).values
    if extra is not None:
        tol = tol + extra
    return bool(((y.float().cpu() - ref).abs() <= tol).all())


class W4A4Layer(Workload):
    """W4A4 layer: online Hadamard-4096, per-token int4 activations, int4 g128 weights; M=6000 K=4096 N=1024."""
    name = "c2"
    metric = "linearq_w4a4_gemm_throughput"
    unit = "TOP/s"
    dtype = "fp8 e4m3 operands holding int4 codes, exact integer group sums in fp32 (tcgen05 kind::f8f6f4); fp16 in/out"
    M, K, N, G = 6000, 4096, 1024, 128
    launches_per_step = 2
    kernels = ["hadamard_quant", "w4a4_gemm"]

    def __init__(self, device, seed):
        import asrq_b200
        from asrq_b200 import _lib
        from oracle import linearq_oracle as O
        self.lib, self.dev = _lib, device
        c = O.make_c2(seed=seed, m=self.M, k=self.K, n=self.N, group_size=self.G)
        self.case = c
        pw, sw = asrq_b200.pack_w4a4(c["w_fp"], self.G, True)
        self.layer = asrq_b200.LinearQQ(self.K, self.N, 4, 4, self.G, bias=True, hadamard=True).to(device)
        self.layer.load_quantized_params(sw, torch.zeros_like(sw), pw)
        self.layer.bias = c["bias"].to(device)
        x = c["x"].to(device)
        nsets = max(2, (2 * L2_BYTES) // x.numel() // 2 + 1)
        gen = torch.Generator(device="cpu").manual_seed(seed + 1)
        self.xs = [x] + [x[torch.randperm(self.M, generator=gen).to(device)].contiguous() for _ in range(nsets - 1)]
        self.a8 = torch.empty(self.M, self.K, dtype=torch.uint8, device=device)
        if self.layer.operand == "int8":
            self.dtype = "int8 operands holding 16x the int4 codes, exact int32 group sums (tcgen05 kind::i8); fp16 in/out"
        self.w8 = self.layer._prepared_weight()  # 8-bit operand form of the weights, derived once at load
        self.sa = torch.empty(self.M, dtype=torch.float32, device=device)
        self.y = torch.empty(self.M, self.N, dtype=torch.float16, device=device)
        self.ws = torch.zeros(_lib.workspace_bytes(_lib.WS_W4A4_GEMM, self.M, self.N, self.K), dtype=torch.uint8,
                              device=device)
        self.nsets = nsets
        self.default_group = nsets
        self.l2_note = f"rotating {nsets} input sets ({nsets * x.numel() * 2 >> 20} MiB > 126 MiB L2)"
        self.x_host = [t.cpu().pin_memory() for t in self.xs[:2]]
        self.y_host = torch.empty(self.M, self.N, dtype=torch.float16).pin_memory()

    def units_per_step(self):
        return 2.0 * self.M * self.N * self.K

    def prologue_bytes(self):  # x in, 8-bit operand out, scales out
        return self.M * self.K * 2 + self.M * self.K + self.M * 4

    def gemm_bytes(self):
        return self.M * self.K + self.N * self.K + self.N * (self.K // self.G) * 2 + self.M * 4 + self.M * self.N * 2

    def run_kernel(self, name, i):
        st = torch.cuda.current_stream().cuda_stream
        L = self.layer
        if name == "hadamard_quant":
            x = self.xs[i % len(self.xs)]
            self.lib.call(L._entry("hadamard_quant"), x.data_ptr(), self.a8.data_ptr(), self.sa.data_ptr(), self.M,
                          self.K, 1, self.lib.F16, st)
        else:
            self.lib.call(L._entry("w4a4_gemm"), self.a8.data_ptr(), self.sa.data_ptr(), self.w8.data_ptr(),
                          L.scales.data_ptr(), L.bias.data_ptr(), self.y.data_ptr(), None, self.M, self.N, self.K,
                          self.G, self.lib.F16, self.ws.data_ptr(), self.ws.numel(), st)

    def step(self, i):
        self.run_kernel("hadamard_quant", i)
        self.run_kernel("w4a4_gemm", i)

    def check_parity(self):
        """Step 0 of the timed configuration against the CPU oracle: every token's codes and scale bit-exact,
        output of a row sample within 2e-3 of the row maximum."""
        from oracle import linearq_oracle as O
        self.step(0)
        torch.cuda.synchronize()
        c = self.case
        qa, sa, _ = O.hadamard_quant_int4(c["x"], True)
        ok = torch.equal(self.sa.cpu(), sa)
        codes_gpu = self.a8.cpu().view(torch.float8_e4m3fn).float() if self.layer.operand == "f8" else \
            (self.a8.cpu().view(torch.int8).to(torch.int32) // 16).float()
        ok = ok and torch.equal(codes_gpu, qa.float())
        rows = torch.arange(0, self.M, max(1, self.M // 96))
        wcodes, sw, _ = O.prepare_w4a4_weight(c["w_fp"], self.G, True)
        ref = O.w4a4_forward_fp32(qa[rows], sa[rows], wcodes, sw, c["bias"], self.G)
        return ok and _rows_ok(self.y[rows.to(self.dev)], ref)

    def e2e_step(self, i):
        import asrq_b200
        xh = self.x_host[i % len(self.x_host)]
        asrq_b200.forward_host(self.layer, xh, self.y_host, chunks=E2E_CHUNKS)
        return xh.numel() * 2, self.y_host.numel() * 2

    e2e_api = (f"asrq_b200.forward_host(LinearQQ, pinned host in, pinned host out, chunks={E2E_CHUNKS}): copies in and "
               "out overlapped with the kernels chunk by chunk")

    def roofline(self, kernel_ms, peaks, int8_tops):
        ach = self.units_per_step() / (kernel_ms["w4a4_gemm"] * 1e-3) / 1e12
        tr = recorded_traffic("w4a4_tc_kernel")
        out = {"kernel": "w4a4_tc_kernel", "bound": "tensor", "achieved": ach, "unit": "TOP/s", "peak": int8_tops,
               "peak_source": "torch._int_mm 8192^3 timed in this run (the 8-bit tensor peak is not in "
                              "MEASURED_PEAKS.json; fp8 and int8 have the same nominal rate)",
               "frac": ach / int8_tops if int8_tops else None,
               "frac_of_2x_bf16_measured": ach / (2 * peaks["bf16_tflops"]),
               "traffic": tr["dram_bytes_per_launch"] if tr else None, "traffic_algorithmic": self.gemm_bytes()}
        pro = self.prologue_bytes() / (kernel_ms["hadamard_quant"] * 1e-3) / 1e9
        out["prologue"] = {"kernel": "hadamard4096_quant_kernel", "bound": "hbm", "achieved": pro, "unit": "GB/s",
                           "peak": peaks["hbm_gbs"], "frac": pro / peaks["hbm_gbs"], "of": peaks["source"]}
        out["library_gemm_same_shape"] = library_gemm_same_shape(self.dev, self.M, self.K, self.N, "int8")
        out["library_f16_gemm_same_shape"] = library_gemm_same_shape(self.dev, self.M, self.K, self.N, "f16")
        return out

    @classmethod
    def cpu_sample(cls, seed, case=None):
        """No executable counterpart exists in the reference for this composite: the oracle's restatement."""
        from oracle import linearq_oracle as O
        ms = 256
        c = case if case is not None else O.make_c2(seed=seed, m=ms, k=cls.K, n=cls.N, group_size=cls.G)
        x = c["x"][:ms]
        codes, sw, _ = O.prepare_w4a4_weight(c["w_fp"], cls.G, True)

        def run():
            qa, sa, _ = O.hadamard_quant_int4(x, True)
            return O.w4a4_forward_fp32(qa, sa, codes, sw, c["bias"], cls.G)
        return run, 2.0 * ms * cls.N * cls.K, f"{ms} of {cls.M} tokens, full K and N; Hadamard + quantisation + grouped integer GEMM", "port"


def _reference_linearq(case, bias):
    """The reference's own LinearQ (staged under oracle/_ref) holding ``case``'s packed parameters, or None."""
    from oracle import ref_loader
    if not ref_loader.available():
        return None
    RQ = ref_loader.linear().LinearQ
    n, k = case["weight"].shape[0], case["x"].shape[-1]
    m = RQ(k, n, case["bits"], case["group_size"], bias=bias is not None)
    m.load_quantized_params(case["scales"], case["zeros"], case["weight"])
    if bias is not None:
        m.bias = bias
    return m


class W4A16Layer(Workload):
    """W4A16 layer, round-to-nearest g128 asymmetric, 0.1 % weight outliers x10, bias; M=1500 K=1280 N=5120."""
    name = "c1"
    metric = "linearq_w4a16_gemm_throughput"
    unit = "TFLOP/s"
    dtype = "f16 (fp32 accumulation)"
    M, K, N, G = 1500, 1280, 5120, 128
    launches_per_step = 1
    kernels = ["gemm_a16_tc"]

    def __init__(self, device, seed):
        from asrq_b200 import _lib
        from oracle import linearq_oracle as O
        import asrq_b200
        self.lib, self.dev = _lib, device
        c = O.make_c1(seed=seed, m=self.M, k=self.K, n=self.N, bits=4, group_size=self.G)
        self.case = c
        self.layer = asrq_b200.LinearQ(self.K, self.N, 4, self.G, bias=True).to(device)
        self.layer.load_quantized_params(c["scales"], c["zeros"], c["weight"])
        self.layer.bias = c["bias"].to(device)
        per_set = self.algorithmic_bytes()  # one layer is 23 MB: rotate enough (x, W, y) sets to exceed L2 twice over
        nsets = (2 * L2_BYTES) // per_set + 1
        gen = torch.Generator().manual_seed(seed + 1)
        self.sets = [dict(x=c["x"].to(device), w=c["weight"].to(device), s=c["scales"].to(device), z=c["zeros"].to(device),
                          b=c["bias"].to(device), y=torch.empty(self.M, self.N, dtype=torch.float16, device=device))]
        for _ in range(nsets - 1):
            perm = torch.randperm(self.N, generator=gen)
            self.sets.append(dict(
                x=c["x"][torch.randperm(self.M, generator=gen)].to(device).contiguous(),
                w=c["weight"][perm].to(device).contiguous(), s=c["scales"][perm].to(device).contiguous(),
                z=c["zeros"][perm].to(device).contiguous(), b=c["bias"][perm].to(device).contiguous(),
                y=torch.empty(self.M, self.N, dtype=torch.float16, device=device)))
        self.ws = torch.zeros(max(1 << 20, _lib.workspace_bytes(_lib.WS_LINEARQ, self.M, self.N, self.K)),
                              dtype=torch.uint8, device=device)
        self.nsets = nsets
        self.default_group = nsets
        self.l2_note = f"rotating {nsets} (x, W, y) sets ({nsets * per_set >> 20} MiB > 126 MiB L2)"
        self.x_host = [c["x"].pin_memory()]
        self.y_host = torch.empty(self.M, self.N, dtype=torch.float16).pin_memory()

    def units_per_step(self):
        return 2.0 * self.M * self.N * self.K

    def algorithmic_bytes(self):
        return (2 * self.M * self.K + self.N * self.K // 2 + 2 * self.N * (self.K // self.G) * 2 + 2 * self.N
                + 2 * self.M * self.N)

    def run_kernel(self, name, i):
        st = torch.cuda.current_stream().cuda_stream
        s = self.sets[i % len(self.sets)]
        self.lib.call("asrq_w4a16_gemm", s["x"].data_ptr(), s["w"].data_ptr(), s["s"].data_ptr(), s["z"].data_ptr(),
                      s["b"].data_ptr(), s["y"].data_ptr(), self.M, self.N, self.K, self.G, self.lib.F16,
                      self.ws.data_ptr(), self.ws.numel(), st)

    def step(self, i):
        self.run_kernel("gemm_a16_tc", i)

    def check_parity(self):
        from oracle import linearq_oracle as O
        self.step(0)
        torch.cuda.synchronize()
        c = self.case
        rows = torch.arange(0, self.M, 6)
        ref = O.linearq_forward_fp32(c["x"][rows], c["weight"], c["scales"], c["zeros"], c["bias"], 4, self.G)
        return _rows_ok(self.sets[0]["y"][rows.to(self.dev)], ref)

    def e2e_step(self, i):
        import asrq_b200
        xh = self.x_host[0]
        asrq_b200.forward_host(self.layer, xh, self.y_host, chunks=E2E_CHUNKS)
        return xh.numel() * 2, self.y_host.numel() * 2

    e2e_api = (f"asrq_b200.forward_host(LinearQ, pinned host in, pinned host out, chunks={E2E_CHUNKS}): copies in and "
               "out overlapped with the kernels chunk by chunk")

    def roofline(self, kernel_ms, peaks, int8_tops):
        ach = self.units_per_step() / (kernel_ms["gemm_a16_tc"] * 1e-3) / 1e12
        tr = recorded_traffic("gemm_a16_tc2_kernel")
        return {"kernel": "gemm_a16_tc2_kernel (CTA pairs)", "bound": "tensor", "achieved": ach, "unit": "TFLOP/s",
                "peak": peaks["bf16_tflops"], "frac": ach / peaks["bf16_tflops"], "of": peaks["source"] + " (burst)",
                "traffic": tr["dram_bytes_per_launch"] if tr else None, "traffic_algorithmic": self.algorithmic_bytes(),
                "library_gemm_same_shape": library_gemm_same_shape(self.dev, self.M, self.K, self.N, "f16")}

    @classmethod
    def cpu_sample(cls, seed, case=None):
        from oracle import linearq_oracle as O
        c = case if case is not None else O.make_c1(seed=seed, m=cls.M, k=cls.K, n=cls.N, bits=4, group_size=cls.G)
        ref = _reference_linearq(c, c["bias"])
        x = c["x"]  # fp16 activations, as the configuration states: the reference computes in the input's dtype
        if ref is not None:
            return (lambda: ref.forward(x)), 2.0 * cls.M * cls.N * cls.K, \
                "the full layer (M=1500) through the reference's LinearQ.forward, fp16 activations: dequantize + torch.matmul", "reference"
        return (lambda: O.linearq_forward(x, c["weight"], c["scales"], c["zeros"], c["bias"], 4, cls.G)), \
            2.0 * cls.M * cls.N * cls.K, "the full layer (M=1500), fp16 activations: dequantize + torch.matmul", "port"


class DecodeSweep(Workload):
    """Decode sweep: (2048->6144, 6144->2048, 2048->4096) x (W4, W2) x M in {1,2,4,8,16}, g64: 30 launches per
    step, each on its own weight copy."""
    name = "c3"
    metric = "linearq_decode_gemv_bandwidth"
    unit = "GB/s"
    dtype = "f16 (fp32 accumulation)"
    SHAPES = [(2048, 6144), (6144, 2048), (2048, 4096)]
    MS = [1, 2, 4, 8, 16]
    G = 64
    kernels = ["gemv_a16 (30 launches)"]
    nsets = 2
    default_group = 2

    def __init__(self, device, seed):
        from asrq_b200 import _lib
        from oracle import linearq_oracle as O
        self.lib, self.dev = _lib, device
        self.items = []
        total = 0
        gen = torch.Generator().manual_seed(seed)
        for (k, n) in self.SHAPES:
            for bits in (4, 2):
                base = O.make_c3(seed=seed + k + bits, m=16, k=k, n=n, bits=bits, group_size=self.G)
                for m in self.MS:
                    perm = torch.randperm(n, generator=gen)
                    it = dict(m=m, k=k, n=n, bits=bits, x=base["x"][:m].to(device).contiguous(), perm=perm, base=base,
                              w=base["weight"][perm].to(device).contiguous(),
                              s=base["scales"][perm].to(device).contiguous(),
                              z=base["zeros"][perm].to(device).contiguous(),
                              y=torch.empty(m, n, dtype=torch.float16, device=device))
                    it["bytes"] = 2 * m * k + n * k * bits // 8 + 2 * n * (k // self.G) * 2 + 2 * m * n
                    total += it["bytes"]
                    self.items.append(it)
        self.total_bytes = total
        # the sweep touches ~143 MB of distinct weights per step; two copies make it > 2x L2
        self.items2 = [dict(it, w=it["w"].clone(), s=it["s"].clone(), z=it["z"].clone()) for it in self.items]
        self.launches_per_step = len(self.items)
        self.ws = torch.zeros(_lib.workspace_bytes(_lib.WS_LINEARQ, 16, 6144, 6144), dtype=torch.uint8, device=device)
        self.l2_note = (f"{len(self.items)} launches per step, each on its own weight copy "
                        f"({2 * total >> 20} MiB over two alternating sets > 126 MiB L2)")

    def units_per_step(self):
        return float(self.total_bytes)

    def _launch_all(self, items):
        st = torch.cuda.current_stream().cuda_stream
        for it in items:
            self.lib.call(f"asrq_w{it['bits']}a16_gemv", it["x"].data_ptr(), it["w"].data_ptr(), it["s"].data_ptr(),
                          it["z"].data_ptr(), None, it["y"].data_ptr(), it["m"], it["n"], it["k"], self.G,
                          self.lib.F16, self.ws.data_ptr(), self.ws.numel(), st)

    def run_kernel(self, name, i):
        self._launch_all(self.items if i % 2 == 0 else self.items2)

    def step(self, i):
        self.run_kernel(self.kernels[0], i)

    def check_parity(self):
        from oracle import linearq_oracle as O
        self.step(0)
        torch.cuda.synchronize()
        ok = True
        cache = {}
        for it in self.items:
            b = it["base"]
            key = (it["k"], it["n"], it["bits"])
            if key not in cache:  # one fp32 dequantisation per layer, shared by its five token counts
                cache[key] = O.dequantize_weight(b["weight"], b["scales"], b["zeros"], it["bits"], self.G, it["k"])
            ref = (b["x"][:it["m"]].float() @ cache[key].t())[:, it["perm"]]
            ok = ok and _rows_ok(it["y"], ref)
        return ok

    def e2e_step(self, i):
        st = torch.cuda.current_stream().cuda_stream
        if not hasattr(self, "_host"):
            self._host = [(it["x"].cpu().pin_memory(), torch.empty(it["m"], it["n"], dtype=torch.float16).pin_memory())
                          for it in self.items]
        h2d = d2h = 0
        for it, (xh, yh) in zip(self.items if i % 2 == 0 else self.items2, self._host):
            xd = xh.to(self.dev, non_blocking=True)
            self.lib.call(f"asrq_w{it['bits']}a16_gemv", xd.data_ptr(), it["w"].data_ptr(), it["s"].data_ptr(),
                          it["z"].data_ptr(), None, it["y"].data_ptr(), it["m"], it["n"], it["k"], self.G,
                          self.lib.F16, self.ws.data_ptr(), self.ws.numel(), st)
            yh.copy_(it["y"], non_blocking=True)
            h2d += xh.numel() * 2
            d2h += yh.numel() * 2
        return h2d, d2h

    e2e_api = "the C-ABI decode calls with pinned host activations in and pinned host outputs back, call by call"

    def roofline(self, kernel_ms, peaks, int8_tops):
        ach = self.total_bytes / (kernel_ms[self.kernels[0]] * 1e-3) / 1e9
        tr = recorded_traffic("gemv_a16_kernel")
        # ncu captures one launch of the sweep; every launch streams its weights exactly once, so the sweep's
        # traffic is its algorithmic bytes scaled by that launch's measured-to-algorithmic ratio
        traffic = self.total_bytes * tr["dram_bytes_per_launch"] / tr["algorithmic_bytes_per_launch"] if tr else None
        return {"kernel": "gemv_a16_kernel", "bound": "hbm", "achieved": ach, "unit": "GB/s", "peak": peaks["hbm_gbs"],
                "frac": ach / peaks["hbm_gbs"], "of": peaks["source"], "traffic": traffic,
                "traffic_algorithmic": self.total_bytes}

    @classmethod
    def cpu_sample(cls, seed, case=None):
        from oracle import linearq_oracle as O
        c = O.make_c3(seed=seed, m=1, k=2048, n=6144, bits=4, group_size=cls.G)
        b = 2 * 2048 + 6144 * 2048 // 2 + 2 * 6144 * 32 * 2 + 2 * 6144
        ref = _reference_linearq(c, None)
        if ref is not None:
            return (lambda: ref.forward(c["x"])), float(b), \
                "one launch of the sweep (W4 g64 K=2048 N=6144 M=1) through the reference's LinearQ.forward, fp16 activations", "reference"
        return (lambda: O.linearq_forward(c["x"], c["weight"], c["scales"], c["zeros"], None, 4, cls.G)), float(b), \
            "one launch of the sweep: W4 g64 K=2048 N=6144 M=1, dequantize + torch.matmul", "port"


class DecodeLargeLayer(Workload):
    """Supplementary (not a named benchmark configuration): the decode kernel on one layer large enough that
    launch and ramp-up latency do not dominate (W4 g128, 8192 -> 28672, M=1; 112 MiB of packed weights)."""
    name = "large"
    metric = "linearq_decode_gemv_bandwidth_large_layer"
    unit = "GB/s"
    dtype = "f16 (fp32 accumulation)"
    M, K, N, G = 1, 8192, 28672, 128
    launches_per_step = 1
    nsets = 3
    default_group = 3
    kernels = ["gemv_a16"]

    def __init__(self, device, seed):
        from asrq_b200 import _lib
        self.lib, self.dev = _lib, device
        gen = torch.Generator(device=device).manual_seed(seed)
        # timing only (parity of this kernel variant is a test): random packed bytes, positive scales
        self.ws_ = [torch.randint(0, 256, (self.N, self.K // 2), dtype=torch.uint8, device=device, generator=gen)
                    for _ in range(3)]
        self.s = (torch.rand(self.N, self.K // self.G, device=device, generator=gen) * 0.01 + 0.001).half()
        self.z = (torch.rand(self.N, self.K // self.G, device=device, generator=gen) * -0.05).half()
        self.x = torch.randn(self.M, self.K, device=device, generator=gen).half()
        self.y = torch.empty(self.M, self.N, dtype=torch.float16, device=device)
        self.ws = torch.zeros(max(1 << 20, _lib.workspace_bytes(_lib.WS_LINEARQ, self.M, self.N, self.K)),
                              dtype=torch.uint8, device=device)
        self.l2_note = "rotating 3 weight copies (336 MiB > 126 MiB L2)"

    def units_per_step(self):
        return float(2 * self.M * self.K + self.N * self.K // 2 + 2 * self.N * (self.K // self.G) * 2 + 2 * self.M * self.N)

    def run_kernel(self, name, i):
        self.lib.call("asrq_w4a16_gemv", self.x.data_ptr(), self.ws_[i % 3].data_ptr(), self.s.data_ptr(),
                      self.z.data_ptr(), None, self.y.data_ptr(), self.M, self.N, self.K, self.G, self.lib.F16,
                      self.ws.data_ptr(), self.ws.numel(), torch.cuda.current_stream().cuda_stream)

    def step(self, i):
        self.run_kernel("gemv_a16", i)

    def check_parity(self):
        from oracle import linearq_oracle as O
        self.step(0)
        torch.cuda.synchronize()
        rows = torch.arange(0, self.N, 97)
        ref = O.linearq_forward_fp32(self.x.cpu(), self.ws_[0][rows.to(self.dev)].cpu(), self.s[rows.to(self.dev)].cpu(),
                                     self.z[rows.to(self.dev)].cpu(), None, 4, self.G)
        got = self.y[:, rows.to(self.dev)]
        tol = 2e-3 * ref.abs().max()
        return bool(((got.float().cpu() - ref).abs() <= tol).all())

    def e2e_step(self, i):
        if not hasattr(self, "x_host"):
            self.x_host = self.x.cpu().pin_memory()
            self.y_host = torch.empty(self.M, self.N, dtype=torch.float16).pin_memory()
        xd = self.x_host.to(self.dev, non_blocking=True)
        self.lib.call("asrq_w4a16_gemv", xd.data_ptr(), self.ws_[i % 3].data_ptr(), self.s.data_ptr(),
                      self.z.data_ptr(), None, self.y.data_ptr(), self.M, self.N, self.K, self.G, self.lib.F16,
                      self.ws.data_ptr(), self.ws.numel(), torch.cuda.current_stream().cuda_stream)
        self.y_host.copy_(self.y, non_blocking=True)
        return self.x_host.numel() * 2, self.y_host.numel() * 2

    e2e_api = "asrq_w4a16_gemv with a pinned host activation row in and the pinned host output row back"

    @classmethod
    def cpu_sample(cls, seed, case=None):
        from oracle import linearq_oracle as O
        rows = 1024
        c = O.make_c3(seed=0, m=1, k=cls.K, n=rows, bits=4, group_size=cls.G)
        b = 2 * cls.K + rows * cls.K // 2 + 2 * rows * (cls.K // cls.G) * 2 + 2 * rows
        ref = _reference_linearq(c, None)
        if ref is not None:
            return (lambda: ref.forward(c["x"])), float(b), f"{rows} of {cls.N} output features, full K, M=1, the reference's LinearQ.forward", "reference"
        return (lambda: O.linearq_forward(c["x"], c["weight"], c["scales"], c["zeros"], None, 4, cls.G)), float(b), \
            f"{rows} of {cls.N} output features, full K, M=1: dequantize + torch.matmul", "port"

    def roofline(self, kernel_ms, peaks, int8_tops):
        ach = self.units_per_step() / (kernel_ms["gemv_a16"] * 1e-3) / 1e9
        return {"kernel": "gemv_a16_kernel (rounds variant)", "bound": "hbm", "achieved": ach, "unit": "GB/s",
                "peak": peaks["hbm_gbs"], "frac": ach / peaks["hbm_gbs"], "of": peaks["source"], "traffic": None}


def whisper_large_v3_config(layers: int = 32, **over):
    import transformers
    kw = dict(vocab_size=51866, num_mel_bins=128, encoder_layers=layers, decoder_layers=layers,
              encoder_attention_heads=20, decoder_attention_heads=20, d_model=1280, encoder_ffn_dim=5120,
              decoder_ffn_dim=5120, max_source_positions=1500, max_target_positions=448, decoder_start_token_id=50258,
              suppress_tokens=None, begin_suppress_tokens=None)
    kw.update(over)
    return transformers.WhisperConfig(**kw)


class WhisperLargeV3(Workload):
    """Whisper-large-v3-shaped model, random weights, all linear layers W4A16 g128 round-to-nearest; a step
    transcribes 32 thirty-second windows (synthetic 128-bin log-mel N(0,1), 3000 frames) with 128 greedy tokens each."""
    name = "c4"
    metric = "whisper_large_v3_w4a16_rtfx"
    unit = "RTFx"
    dtype = "f16 (fp32 accumulation); W4 g128 weights"
    B, STEPS, LAYERS = 32, 128, 32
    graph_steps = False
    nsets = 2
    kernels = ["encoder_linearq"]

    def __init__(self, device, seed, batch=None):
        from asrq_b200 import whisper as W
        self.W, self.dev = W, device
        self.cfg = whisper_large_v3_config(self.LAYERS)
        self.batch = batch or self.B
        self.engine = W.WhisperEngine.random_init(self.cfg, device, seed=seed)
        gen = torch.Generator().manual_seed(seed + 1)
        self.x_host = [torch.randn(self.batch, 128, 3000, generator=gen).half().pin_memory() for _ in range(self.nsets)]
        self.xs = [x.to(device) for x in self.x_host]
        self.ids_host = torch.empty(self.batch, self.STEPS, dtype=torch.long).pin_memory()
        nlin = len(self.engine.linear_layers())
        self.launches_per_step = None  # counted in count_launches()
        self.l2_note = (f"one step streams {sum(l.weight.numel() for l in self.engine.linear_layers()) >> 20} MiB of packed "
                        f"weights, {self.batch * 1500 * 1280 * 2 * 2 * self.LAYERS >> 20} MiB of cross-attention keys and "
                        f"values per token and GBs of activations: far beyond the 126 MiB L2; 2 alternating input batches")
        self.n_linear = nlin

    def units_per_step(self):
        return self.W.audio_seconds(self.cfg, self.batch)   # seconds of audio; value = units / seconds

    def value_from(self, ms_per_step, world):
        return self.units_per_step() * world / (ms_per_step * 1e-3)

    def step(self, i):
        self.last_ids = self.engine.generate(self.xs[i % self.nsets], steps=self.STEPS)

    def count_launches(self):
        """This library's kernel launches in one step, counted: the C-ABI calls of one eager (not graph-replayed) pass
        through encoder, cross-attention key/value projections and one decoder token, the last times the number of
        tokens.  A call is one launch, except that a large-M layer with a fused activation or residual runs that
        step as a second kernel: those calls are counted twice."""
        from asrq_b200 import _lib
        eng, x = self.engine, self.xs[0]
        c0 = _lib.CALLS
        enc = eng.encode(x)
        eng._alloc(self.batch, enc.shape[1], 4)
        eng._cross_kv(enc)
        c1 = _lib.CALLS
        eng.decode(enc, 2, use_graph=False)
        c2 = _lib.CALLS
        torch.cuda.synchronize()
        fused_large = len(eng.enc_layers) * 3 if self.batch * self.cfg.max_source_positions > 64 else 0  # out, fc1, fc2 of a layer
        return (c1 - c0) + fused_large + (c2 - c1) // 2 * self.STEPS

    def phases(self):
        """Device time of the three phases of one step (CUDA events on the launching stream)."""
        eng = self.engine
        x = self.xs[0]
        torch.cuda.synchronize()
        a = event()
        enc = eng.encode(x)
        b = event()
        eng._alloc(self.batch, enc.shape[1], self.STEPS + 1)
        eng._cross_kv(enc)
        c = event()
        eng.decode(enc, self.STEPS)
        d = event()
        torch.cuda.synchronize()
        ckv = b.elapsed_time(c)
        return {"encoder_ms": a.elapsed_time(b), "cross_kv_ms": ckv, "decode_ms": c.elapsed_time(d) - ckv,
                "decode_ms_per_token": (c.elapsed_time(d) - ckv) / self.STEPS}

    def encoder_linear_times(self, reps=4):
        """The four LinearQ shapes of an encoder layer at the encoder's token count, each timed alone with
        CUDA events (one call per weight set, weight sets rotated over the 32 layers)."""
        eng = self.engine
        m = self.batch * self.cfg.max_source_positions
        out = {}
        gen = torch.Generator(device=self.dev).manual_seed(0)
        for key, k in (("qkv", 1280), ("out", 1280), ("fc1", 1280), ("fc2", 5120)):
            x = torch.randn(m, k, device=self.dev, generator=gen).half()
            layers = [L[key] for L in eng.enc_layers]
            for L in layers[:2]:
                L(x)
            torch.cuda.synchronize()
            a = event()
            for _ in range(reps):
                for L in layers:
                    L(x)
            b = event()
            torch.cuda.synchronize()
            n = layers[0].out_features
            ms = a.elapsed_time(b) / (reps * len(layers))
            out[key] = {"M": m, "K": k, "N": n, "ms": ms, "tflops": 2.0 * m * n * k / (ms * 1e-3) / 1e12}
        return out

    def check_parity(self):
        """(1) the encoder's first fused q/k/v projection on the real activations of this batch, a row sample
        against the fp32 CPU oracle; (2) a decode-sized call (M = batch) of the same layer; (3) the captured
        decoder graph against eager stepping: identical tokens."""
        from oracle import linearq_oracle as O
        eng = self.engine
        x = self.xs[0]
        h = torch.nn.functional.gelu(torch.nn.functional.conv1d(x, eng.conv1_w, eng.conv1_b, padding=1))
        h = torch.nn.functional.gelu(torch.nn.functional.conv1d(h, eng.conv2_w, eng.conv2_b, stride=2, padding=1))
        h = (h.permute(0, 2, 1) + eng.enc_pos).contiguous()
        h = eng.enc_layers[0]["ln1"](h).reshape(-1, 1280)
        L = eng.enc_layers[0]["qkv"]
        y = L(h)
        rows = torch.arange(0, h.shape[0], max(1, h.shape[0] // 256))
        w, s, z, b = L.weight.cpu(), L.scales.cpu(), L.zeros.cpu(), L.bias.cpu()
        ok1 = _rows_ok(y[rows.to(self.dev)], O.linearq_forward_fp32(h[rows.to(self.dev)].cpu(), w, s, z, b, 4, 128))
        hb = h[:self.batch].contiguous()
        ok2 = _rows_ok(L(hb), O.linearq_forward_fp32(hb.cpu(), w, s, z, b, 4, 128))
        nb = min(self.batch, 4)
        a_ = eng.generate(x[:nb], steps=6, use_graph=False).clone()
        b_ = eng.generate(x[:nb], steps=6, use_graph=True).clone()
        ok3 = torch.equal(a_, b_)
        if not (ok1 and ok2 and ok3):
            print(f"bench.py c4 parity on {self.dev}: encoder-sized call {ok1}, decode-sized call {ok2}, graph == eager {ok3}",
                  file=sys.stderr, flush=True)
        return ok1 and ok2 and ok3

    def e2e_step(self, i):
        xh = self.x_host[i % self.nsets]
        ids = self.engine.generate(xh.to(self.dev, non_blocking=True), steps=self.STEPS)
        self.ids_host.copy_(ids, non_blocking=True)
        torch.cuda.current_stream().synchronize()   # the caller has its token ids here
        return xh.numel() * 2, self.ids_host.numel() * 8

    e2e_api = ("asrq_b200.whisper.WhisperEngine.generate(pinned host log-mel batch) -> token ids copied to pinned host "
               "memory, synchronised every step")

    def roofline(self, kernel_ms, peaks, int8_tops):
        lin = self.encoder_linear_times()
        flops = sum(2.0 * v["M"] * v["N"] * v["K"] for v in lin.values())
        ms = sum(v["ms"] for v in lin.values())
        ach = flops / (ms * 1e-3) / 1e12
        tr = recorded_traffic("gemm_a16_tc2_kernel@encoder")
        return {"kernel": "gemm_a16_tc2_kernel (CTA pairs) on the encoder's four layer shapes, M = batch x 1500",
                "bound": "tensor", "achieved": ach, "unit": "TFLOP/s", "peak": peaks["bf16_tflops"],
                "frac": ach / peaks["bf16_tflops"], "of": peaks["source"] + " (burst)",
                "frac_of_sustained": ach / peaks["bf16_tflops_sustained"],
                "traffic": tr["dram_bytes_per_launch"] if tr else None, "per_shape": lin}

    # ---- CPU baseline: the reference's own model classes on a bounded sample ----
    @classmethod
    def cpu_sample(cls, seed, case=None):
        """One encoder layer and one decoder layer at full width through the reference's
        WhisperForConditionalGenerationQ (oracle/_ref; its LinearQ dequantizes every weight on every call):
        the encoder layer on 4 utterances, the decoder layer on the full batch of 32 for ``tok`` tokens (the
        first one includes the cross-attention key/value projections of 32 x 1500 encoder states).  The whole
        configuration is 32 + 32 such layers and 128 tokens; its time is extrapolated linearly and says so."""
        from oracle import ref_loader
        import transformers
        tok, enc_b = 3, 4
        cfg = whisper_large_v3_config(1)
        kind = "reference"
        if ref_loader.available("asrq/models/transformers/whisper.py"):
            model = ref_loader.whisper().WhisperForConditionalGenerationQ(cfg).eval()
            is_q = lambda m: type(m).__name__ == "LinearQ"
        else:
            from oracle import linearq_oracle as O
            kind = "port"
            model = transformers.WhisperForConditionalGeneration(cfg).eval()
            O.swap_in_port_linearq(model, 4, 128, skip=("proj_out",))
            is_q = lambda m: type(m).__name__ == "PortLinearQ"
        gen = torch.Generator().manual_seed(seed)
        for m in model.modules():
            if is_q(m):
                m.weight.copy_(torch.randint(0, 256, m.weight.shape, generator=gen, dtype=torch.uint8))
                m.scales.copy_((torch.rand(m.scales.shape, generator=gen) * 0.005 + 0.001).half())
                m.zeros.copy_((torch.rand(m.zeros.shape, generator=gen) * -0.04).half())
        x = torch.randn(enc_b, 128, 3000, generator=gen)
        enc32 = torch.randn(cls.B, 1500, 1280, generator=gen)
        state = {}

        def run():
            with torch.no_grad():
                t0 = time.perf_counter()
                model.model.encoder(x)
                t1 = time.perf_counter()
                ids = torch.full((cls.B, 1), cfg.decoder_start_token_id, dtype=torch.long)
                past, marks = None, []
                for _ in range(tok):
                    out = model(encoder_outputs=(enc32,), decoder_input_ids=ids[:, -1:], past_key_values=past, use_cache=True)
                    past = out.past_key_values
                    ids = torch.cat([ids, out.logits[:, -1].argmax(-1, keepdim=True)], 1)
                    marks.append(time.perf_counter())
            state["enc_layer_per_utterance_s"] = (t1 - t0) / enc_b
            state["dec_layer_token_s"] = (marks[-1] - marks[0]) / (tok - 1)          # batch of 32, one layer, one token
            state["cross_kv_layer_s"] = max(0.0, (marks[0] - t1) - state["dec_layer_token_s"])
        note = (f"1 encoder layer on {enc_b} utterances and 1 decoder layer on the batch of {cls.B} for {tok} tokens, full width, "
                "fp32 activations; the full configuration is extrapolated linearly: 32 x 32 x encoder-layer time per "
                "utterance + 32 x cross-attention key/value time + 32 x 128 x decoder-layer-token time per batch "
                "(convolutions, embeddings and the output head are counted once per layer here, i.e. over-counted)")
        return run, state, note, kind


def qwen3_1p7b_config(layers: int = 28, **over):
    import transformers
    cfg = dict(vocab_size=151936, hidden_size=2048, intermediate_size=6144, num_hidden_layers=layers, num_attention_heads=16,
               num_key_value_heads=8, head_dim=128, max_position_embeddings=4096, rms_norm_eps=1e-6, tie_word_embeddings=True)
    cfg.update(over)
    return transformers.Qwen3Config(**cfg)


class CanaryQwenShape(Workload):
    """Canary-Qwen-2.5B-shaped model, random weights: a FastConformer-shaped stand-in encoder (32 blocks, d_model 1024,
    FFN 4096, 8 heads, 8x subsampling; NeMo's encoder body is not available) whose linear layers are W4A4 with the online
    Hadamard rotation, and a Qwen3-1.7B-shaped decoder (28 layers, hidden 2048, 16 query / 8 key-value heads, FFN 6144,
    vocabulary 151936) W4A16 g128; a step transcribes 64 twenty-second windows (synthetic 80-bin log-mel N(0,1), 2000
    frames -> 250 encoder tokens, 8 prompt tokens) with 200 greedy tokens each."""
    name = "c5"
    metric = "canary_qwen_shape_w4a4_w4a16_rtfx"
    unit = "RTFx"
    dtype = "f16 (fp32 / exact integer accumulation); encoder W4A4 g128, decoder W4 g128"
    B, STEPS, FRAMES, MEL, ENC_LAYERS, DEC_LAYERS = 64, 200, 2000, 80, 32, 28
    graph_steps = False
    nsets = 2
    kernels = ["encoder_linearqq"]

    def __init__(self, device, seed, batch=None):
        from asrq_b200 import conformer as C, qwen3 as Q
        self.C, self.dev = C, device
        self.batch = batch or self.B
        enc = C.FastConformerStandIn(device, n_layers=self.ENC_LAYERS, seed=seed)
        dec = Q.Qwen3Engine.random_init(qwen3_1p7b_config(self.DEC_LAYERS), device, seed=seed + 1)
        self.model = C.SpeechLM(enc, dec, prompt_tokens=8, seed=seed)
        gen = torch.Generator().manual_seed(seed + 1)
        self.x_host = [torch.randn(self.batch, self.MEL, self.FRAMES, generator=gen).half().pin_memory() for _ in range(self.nsets)]
        self.xs = [x.to(device) for x in self.x_host]
        self.ids_host = torch.empty(self.batch, self.STEPS, dtype=torch.long).pin_memory()
        self.n_linear = len(enc.linear_layers()) + len(dec.linear_layers())
        self.l2_note = ("one step streams the packed weights of both models (about 1.3 GB with the fp16 head) per decoded token "
                        "and GBs of activations: far beyond the 126 MiB L2; 2 alternating input batches")

    def units_per_step(self):
        return self.C.audio_seconds(self.batch, self.FRAMES)

    def value_from(self, ms_per_step, world):
        return self.units_per_step() * world / (ms_per_step * 1e-3)

    def step(self, i):
        self.last_ids = self.model.generate(self.xs[i % self.nsets], steps=self.STEPS)

    def count_launches(self):
        """C-ABI calls of one eager pass: encoder and prompt once, one decoded token times the number of tokens (a W4A4
        layer is two calls: prologue and GEMM)."""
        from asrq_b200 import _lib
        m = self.model
        c0 = _lib.CALLS
        emb = m.prompt_embeddings(self.xs[0])
        m.dec.prefill(emb, self.STEPS)
        c1 = _lib.CALLS
        m.dec.decode(2, use_graph=False)
        c2 = _lib.CALLS
        torch.cuda.synchronize()
        return (c1 - c0) + (c2 - c1) // 2 * (self.STEPS - 1)

    def phases(self):
        m = self.model
        torch.cuda.synchronize()
        a = event()
        enc = m.enc.encode(self.xs[0])
        b = event()
        emb = m.prompt_embeddings(self.xs[0])
        m.dec.prefill(emb, self.STEPS)
        c = event()
        m.dec.decode(self.STEPS - 1)
        d = event()
        torch.cuda.synchronize()
        e_ms = a.elapsed_time(b)
        return {"encoder_ms": e_ms, "prompt_ms": b.elapsed_time(c) - e_ms, "decode_ms": c.elapsed_time(d),
                "decode_ms_per_token": c.elapsed_time(d) / (self.STEPS - 1)}

    def encoder_linear_times(self, reps=2):
        """The W4A4 layer shapes of an encoder block at the encoder's token count (prologue + GEMM per call), each timed
        alone with CUDA events, weight sets rotated over the blocks."""
        enc = self.model.enc
        m = self.batch * (self.FRAMES // 8)
        out = {}
        gen = torch.Generator(device=self.dev).manual_seed(0)
        for key, k in (("ff1_a", 1024), ("ff1_b", 4096), ("q", 1024)):
            x = torch.randn(m, k, device=self.dev, generator=gen).half()
            layers = [L[key] for L in enc.layers]
            for L in layers[:2]:
                L(x)
            torch.cuda.synchronize()
            a = event()
            for _ in range(reps):
                for L in layers:
                    L(x)
            b = event()
            torch.cuda.synchronize()
            n = layers[0].out_features
            ms = a.elapsed_time(b) / (reps * len(layers))
            out[key] = {"M": m, "K": k, "N": n, "ms": ms, "tops": 2.0 * m * n * k / (ms * 1e-3) / 1e12}
        return out

    def check_parity(self):
        """(1) every W4A4 call of the first encoder block on this batch's real activations, a row sample against the CPU
        oracle (codes of the prologue recomputed on the CPU, exact integer sums, fp32 epilogue); (2) the decoder's first fused
        q/k/v projection on the prompt's activations against the fp32 oracle; (3) the captured decoding graph against eager
        stepping: identical tokens."""
        from oracle import linearq_oracle as O
        m = self.model
        seen = {}

        def hook(name, layer, inp, out):
            if name not in seen:
                seen[name] = (layer, inp.reshape(-1, inp.shape[-1]), out.reshape(-1, out.shape[-1]))
        x = m.enc.subsample(self.xs[0][:4])
        m.enc.block(m.enc.layers[0], x, m.enc._pos_emb(x.shape[1]), hook)
        ok = True
        for name, (layer, inp, out) in seen.items():
            rows = torch.arange(0, inp.shape[0], max(1, inp.shape[0] // 48))
            xi = inp[rows.to(self.dev)].cpu()
            qa, sa, _ = O.hadamard_quant_int4(xi, True)
            codes = O.unpack_signed_int4(layer.weight.cpu())
            bias = None if layer.bias is None else layer.bias.cpu()
            ref = O.w4a4_forward_fp32(qa, sa, codes, layer.scales.cpu(), bias, layer.group_size)
            ok = ok and _rows_ok(out[rows.to(self.dev)], ref)
        emb = m.prompt_embeddings(self.xs[0][:4])
        from asrq_b200 import add_rmsnorm
        L0 = m.dec.layers[0]
        h = add_rmsnorm(emb.reshape(-1, emb.shape[-1]), None, L0["ln1"], m.dec.eps)[1]
        y = L0["qkv"](h)
        rows = torch.arange(0, h.shape[0], max(1, h.shape[0] // 64))
        q = L0["qkv"]
        ref = O.linearq_forward_fp32(h[rows.to(self.dev)].cpu(), q.weight.cpu(), q.scales.cpu(), q.zeros.cpu(), None, 4, 128)
        ok = ok and _rows_ok(y[rows.to(self.dev)], ref)
        a_ = m.dec.generate(emb, 5, use_graph=False).clone()
        b_ = m.dec.generate(emb, 5, use_graph=True).clone()
        return ok and torch.equal(a_, b_)

    def e2e_step(self, i):
        xh = self.x_host[i % self.nsets]
        ids = self.model.generate(xh.to(self.dev, non_blocking=True), steps=self.STEPS)
        self.ids_host.copy_(ids, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return xh.numel() * 2, self.ids_host.numel() * 8

    e2e_api = ("asrq_b200.conformer.SpeechLM.generate(pinned host log-mel batch) -> token ids copied to pinned host memory, "
               "synchronised every step")

    def roofline(self, kernel_ms, peaks, int8_tops):
        lin = self.encoder_linear_times()
        ops = sum(2.0 * v["M"] * v["N"] * v["K"] for v in lin.values())
        ms = sum(v["ms"] for v in lin.values())
        ach = ops / (ms * 1e-3) / 1e12
        peak = int8_tops or time_int8_peak(self.dev)
        return {"kernel": "hadamard_quant + w4a4_tc_kernel on the encoder's W4A4 layer shapes, M = batch x 250 (prologue included)",
                "bound": "tensor", "achieved": ach, "unit": "TOP/s", "peak": peak,
                "peak_source": "torch._int_mm 8192^3 timed in this run", "frac": ach / peak if peak else None,
                "traffic": None, "per_shape": lin}

    # ---- CPU baseline: the quantized layers of one encoder block and one decoder layer on a bounded sample ----
    @classmethod
    def cpu_sample(cls, seed, case=None):
        """The reference cannot express the W4A4 layers (its LinearQQ.forward returns None) and its encoder body is NeMo's,
        so the CPU figure is a port restricted to the path: the nine W4A4 layers of one encoder block through the oracle
        (Hadamard, int4 codes, integer sums) on 2 utterances, and the four fused W4A16 layer shapes of one decoder layer
        through the reference's LinearQ.forward (oracle/_ref when staged, else the port) on the batch of 64 for one token
        and on 2 utterances' prompts; everything else of the models (attention, convolutions, norms, the head) is left out,
        i.e. the figure is an upper bound of the CPU's RTFx."""
        from oracle import linearq_oracle as O
        gen = torch.Generator().manual_seed(seed)
        enc_u, T, H = 2, cls.FRAMES // 8, 2048
        enc_layers = []
        for n, k in ((4096, 1024), (1024, 4096), (1024, 1024), (1024, 1024), (1024, 1024), (1024, 1024), (1024, 1024), (4096, 1024), (1024, 4096)):
            codes = torch.randint(-7, 8, (n, k), generator=gen, dtype=torch.int8)
            sw = (torch.rand(n, k // 128, generator=gen) * 0.005 + 0.001).half()
            enc_layers.append((codes, sw, torch.randn(enc_u * T, k, generator=gen).half()))
        dec_layers = []
        for n, k in ((4096, 2048), (2048, 2048), (12288, 2048), (2048, 6144)):
            c = O.make_c3(seed=seed + n, m=1, k=k, n=n, bits=4, group_size=128)
            ref = _reference_linearq(c, None)
            dec_layers.append((c, ref, torch.randn(cls.B, k, generator=gen).half(), torch.randn(enc_u * (T + 8), k, generator=gen).half()))
        state = {}
        kind = "reference (decoder layers) + port (encoder layers)" if dec_layers[0][1] is not None else "port"

        def fwd(c, ref, x):
            if ref is not None:
                return ref.forward(x)
            return O.linearq_forward(x, c["weight"], c["scales"], c["zeros"], None, 4, 128)

        def run():
            with torch.no_grad():
                t0 = time.perf_counter()
                for codes, sw, x in enc_layers:
                    qa, sa, _ = O.hadamard_quant_int4(x, True)
                    O.w4a4_forward_fp32(qa, sa, codes, sw, None, 128)
                t1 = time.perf_counter()
                for c, ref, xt, xp in dec_layers:
                    fwd(c, ref, xt)
                t2 = time.perf_counter()
                for c, ref, xt, xp in dec_layers:
                    fwd(c, ref, xp)
                t3 = time.perf_counter()
            state["enc_block_per_utterance_s"] = (t1 - t0) / enc_u
            state["dec_layer_token_s"] = t2 - t1
            state["dec_layer_prompt_per_utterance_s"] = (t3 - t2) / enc_u
        note = (f"quantized layers only: the 9 W4A4 layers of 1 encoder block on {enc_u} utterances (oracle port), the 4 fused W4A16 "
                f"layers of 1 decoder layer on the batch of {cls.B} for 1 token and on {enc_u} prompts (reference LinearQ.forward "
                "where staged); extrapolated linearly to 32 blocks x 64 utterances + 28 layers x (64 prompts + 200 tokens); "
                "attention, convolutions, norms and the head are left out (the figure is an upper bound of the CPU's RTFx)")
        return run, state, note, kind


WORKLOADS = {"c1": W4A16Layer, "c2": W4A4Layer, "c3": DecodeSweep, "c4": WhisperLargeV3, "c5": CanaryQwenShape, "large": DecodeLargeLayer}


def library_gemm_same_shape(device, m, k, n, kind, reps=40):
    """Context for a tensor-bound roofline: the vendor library's plain dense GEMM on this very shape, timed by the
    protocol of the bench (CUDA graphs replayed back to back over rotating operands).  ``kind`` "f16":
    torch.matmul on fp16 operands (what the reference's dequantize-then-matmul path runs after its
    dequantisation); "int8": torch._int_mm.  Not a peak and not this library's code."""
    try:
        nset = 6
        if kind == "f16":
            a = [torch.randn(m, k, device=device).half() for _ in range(nset)]
            b = [torch.randn(n, k, device=device).half().t() for _ in range(nset)]
            fn = lambda i: torch.matmul(a[i], b[i])
        else:
            a = [torch.randint(-8, 8, (m, k), dtype=torch.int8, device=device) for _ in range(nset)]
            b = [torch.randint(-8, 8, (n, k), dtype=torch.int8, device=device).t() for _ in range(nset)]
            fn = lambda i: torch._int_mm(a[i], b[i])
        g = capture_graph(lambda: [fn(i) for i in range(nset)])
        g.replay()
        torch.cuda.synchronize()
        e0 = event()
        for _ in range(reps):
            g.replay()
        e1 = event()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / (reps * nset)
        return {"ms": ms, "rate": 2.0 * m * n * k / (ms * 1e-3) / 1e12,
                "what": ("torch.matmul fp16" if kind == "f16" else "torch._int_mm int8") +
                        f" {m}x{n}x{k}, dense operands, no dequantisation or group scales, same graph-replay protocol"}
    except Exception as e:
        return {"error": repr(e)}


def time_int8_peak(device):
    """Dense int8 tensor throughput of this GPU (library GEMM), used only as a roofline denominator."""
    try:
        a = torch.randint(-8, 8, (8192, 8192), dtype=torch.int8, device=device)
        b = torch.randint(-8, 8, (8192, 8192), dtype=torch.int8, device=device)
        for _ in range(3):
            torch._int_mm(a, b)
        best = 1e9
        for _ in range(5):
            e0 = event()
            torch._int_mm(a, b)
            e1 = event()
            e1.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return 2 * 8192 ** 3 / (best * 1e-3) / 1e12
    except Exception:
        return None


def run_cpu(cls, seed, budget_s, max_runs, min_runs=1, case=None):
    """Times ``cls``'s CPU sample on all host cores.  Returns the cpu_baseline object."""
    torch.set_num_threads(os.cpu_count() or 1)
    run, units, sample, kind = cls.cpu_sample(seed, case)
    run()
    times = []
    t_begin = time.perf_counter()
    while len(times) < max_runs and (len(times) < min_runs or time.perf_counter() - t_begin < budget_s):
        t0 = time.perf_counter()
        run()
        times.append(time.perf_counter() - t0)
    dt = statistics.median(times)
    out = {"unit": cls.unit, "cores": torch.get_num_threads(), "kind": kind, "sample": sample, "runs": len(times),
           "ms_per_sample": dt * 1e3}
    if cls.name == "c4":
        wall = (32 * 32 * units["enc_layer_per_utterance_s"] + 32 * units["cross_kv_layer_s"]
                + 32 * 128 * units["dec_layer_token_s"])                      # seconds per batch of 32 utterances
        out["value"] = 32 * 30.0 / wall
        out["extrapolated"] = dict(units, seconds_per_batch_of_32=wall)
    elif cls.name == "c5":
        wall = (cls.ENC_LAYERS * cls.B * units["enc_block_per_utterance_s"]
                + cls.DEC_LAYERS * (cls.B * units["dec_layer_prompt_per_utterance_s"] + cls.STEPS * units["dec_layer_token_s"]))
        out["value"] = cls.B * cls.FRAMES / 100.0 / wall
        out["extrapolated"] = dict(units, seconds_per_batch_of_64=wall)
    else:
        scale = 1e12 if cls.unit in ("TOP/s", "TFLOP/s") else 1e9
        out["value"] = units / dt / scale
    return out


def run_reference(args, rank):
    """``--impl reference``: the reference's CPU implementation of the workload on the host cores (rank 0 only)."""
    if rank != 0:
        return
    cls = WORKLOADS[args.workload]
    t0 = time.perf_counter()
    cb = run_cpu(cls, args.seed, budget_s=1e9, max_runs=max(1, args.steps), min_runs=max(1, args.steps))
    line = {"impl": "reference", "metric": cls.metric, "value": cb["value"], "unit": cls.unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": cb["ms_per_sample"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "CPU: the activation dtype the sample states", "data": "synthetic",
            "config": {"workload": f"{cls.name}: " + " ".join((cls.__doc__ or "").split()),
                       "note": "the reference's own Python code staged under oracle/_ref where it can express the "
                               "workload (kind: reference), else its CPU restatement (kind: port); each step is a bounded "
                               "sample of the workload, stated in cpu_baseline.sample"},
            "cpu_baseline": cb, "e2e": {"value": cb["value"], "unit": cls.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "wall_s": time.perf_counter() - t0}
    emit(line)


_RESULT_OUT = sys.stdout


def emit(line):
    """Writes the result line to the process's original standard output."""
    _RESULT_OUT.write(json.dumps(line) + "\n")
    _RESULT_OUT.flush()


def measure(name, args, rank, local_rank, world, device, peaks, steps, warmup, full):
    """One workload: parity check, K timed steps (max over ranks), per-kernel times, end-to-end leg, roofline,
    CPU baseline.  Returns the result object (the JSON line of the headline workload)."""
    from asrq_b200 import _lib, dp
    if name == "c4" and (args.c4_layers or args.c4_tokens):
        WhisperLargeV3.LAYERS = args.c4_layers or WhisperLargeV3.LAYERS
        WhisperLargeV3.STEPS = args.c4_tokens or WhisperLargeV3.STEPS
    if name == "c5" and (args.c4_layers or args.c4_tokens):
        CanaryQwenShape.ENC_LAYERS = args.c4_layers or CanaryQwenShape.ENC_LAYERS
        CanaryQwenShape.DEC_LAYERS = args.c4_layers or CanaryQwenShape.DEC_LAYERS
        CanaryQwenShape.STEPS = args.c4_tokens or CanaryQwenShape.STEPS
    wl = WORKLOADS[name](device, args.seed + 1000 * rank)
    parity = bool(wl.check_parity())
    parity_attempts = 1
    if not parity:
        # a second, fresh check tells a reproducible mismatch from a transient one; either way the line says so
        print(f"bench.py: workload {name}: parity check failed on {device}, checking once more", file=sys.stderr, flush=True)
        parity = bool(wl.check_parity())
        parity_attempts = 2
    if not parity:
        raise SystemExit(f"bench.py: workload {name}: the GPU result does not match the CPU oracle; nothing was timed")

    if wl.graph_steps:
        runner = GraphSteps(wl.step, wl.nsets, wl.default_group if not args.no_group else 1)
        run_steps = runner.run
    else:
        counter = [0]

        def run_steps(k):
            for _ in range(k):
                wl.step(counter[0])
                counter[0] += 1
    run_steps(warmup)
    torch.cuda.synchronize()
    # how many times the K steps are repeated inside the timed region so that it lasts >= MIN_TIMED_MS
    a = event()
    run_steps(steps)
    b = event()
    torch.cuda.synchronize()
    reps = max(1, int(MIN_TIMED_MS / max(a.elapsed_time(b), 1e-3)) + 1) if a.elapsed_time(b) < MIN_TIMED_MS else 1
    reps = int(dp.max_over_ranks(reps))
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    dp.barrier()
    torch.cuda.synchronize()
    t_start = event()
    for _ in range(reps):
        run_steps(steps)
    t_end = event()
    torch.cuda.synchronize()
    dp.barrier()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = dp.max_over_ranks(t_start.elapsed_time(t_end))
    ms_step = total_ms / (steps * reps)

    # each kernel alone, the same way (outside the timed region of the step)
    kernel_ms = {}
    if wl.graph_steps:
        if len(wl.kernels) == 1:
            kernel_ms[wl.kernels[0]] = t_start.elapsed_time(t_end) / (steps * reps)
        else:
            for kname in wl.kernels:
                kr = GraphSteps(lambda i, kname=kname: wl.run_kernel(kname, i), wl.nsets,
                                wl.default_group if not args.no_group else 1)
                kr.run(3)
                a = event()
                for _ in range(reps):
                    kr.run(steps)
                b = event()
                torch.cuda.synchronize()
                kernel_ms[kname] = a.elapsed_time(b) / (steps * reps)

    e2e = None
    if full:
        for i in range(2):
            wl.e2e_step(i)
        torch.cuda.synchronize()
        dp.barrier()
        e_steps = steps if not wl.graph_steps else max(steps, 20)
        a = event()
        for i in range(e_steps):
            h2d, d2h = wl.e2e_step(i)
        b = event()
        torch.cuda.synchronize()
        dp.barrier()
        e2e_ms = dp.max_over_ranks(a.elapsed_time(b)) / e_steps
        e2e = {"value": wl.value_from(e2e_ms, world), "unit": wl.unit, "ms_per_step": e2e_ms, "steps": e_steps,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "api": wl.e2e_api}

    launches = wl.count_launches() if hasattr(wl, "count_launches") else wl.launches_per_step
    line = {
        "metric": wl.metric, "value": wl.value_from(ms_step, world), "unit": wl.unit, "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": wl.dtype, "data": "synthetic",
        "config": {"workload": f"{wl.name}: " + " ".join((wl.__doc__ or "").split()),
                   "per_gpu": "every rank runs the full step on its own replica of the weights and its own batch; "
                              "no data-path collective", "l2": wl.l2_note,
                   "launch": ("kernel-only steps are CUDA-graph replays: one graph holds %d consecutive steps, each on its "
                              "own input set, single-step graphs serve the remainder" % runner.group) if wl.graph_steps else
                             "the engine replays one captured CUDA graph per decoded token; the encoder is issued call by call",
                   "timed_steps": steps * reps, "repeats_of_the_K_steps_in_the_timed_region": reps,
                   "M": getattr(wl, "M", None), "K": getattr(wl, "K", None), "N": getattr(wl, "N", None)},
        "parity_checked": parity, "parity_attempts": parity_attempts, "kernel_ms": kernel_ms, "gpu_launches": launches * steps * reps, "clocks": clocks,
    }
    if name in ("c4", "c5") and (args.c4_layers or args.c4_tokens):
        line["config"]["reduced"] = (f"NOT the benchmark configuration: {args.c4_layers or 'all'} layers each, {wl.STEPS} tokens "
                                     "(a bounded run for profiler captures)")
    if name == "c5":
        line["config"].update({"batch_per_gpu": wl.batch, "tokens": wl.STEPS, "layers": f"{wl.ENC_LAYERS} blocks + {wl.DEC_LAYERS} layers",
                               "quantized_layers": wl.n_linear, "audio_seconds_per_step_per_gpu": wl.units_per_step(),
                               "encoder": "stand-in of FastConformer's shape (asrq_b200/conformer.py): NeMo's encoder body is not available"})
        line["phases"] = wl.phases()
    if name == "c4":
        line["config"].update({"batch_per_gpu": wl.batch, "tokens": wl.STEPS, "layers": f"{wl.LAYERS}+{wl.LAYERS}",
                               "linearq_layers": wl.n_linear, "audio_seconds_per_step_per_gpu": wl.units_per_step()})
        line["phases"] = wl.phases()
    if rank == 0:
        int8_tops = time_int8_peak(device) if name in ("c2", "c5") else None
        line["roofline"] = wl.roofline(kernel_ms, peaks, int8_tops)
        if e2e is not None:
            line["e2e"] = e2e
        if full and world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = run_cpu(type(wl), args.seed, budget_s=12.0, max_runs=20,
                                           case=getattr(wl, "case", None))
    _lib_ws = getattr(wl, "ws", None)
    if _lib_ws is not None:
        _lib.call("asrq_check_status", _lib_ws.data_ptr(), torch.cuda.current_stream().cuda_stream)
    else:
        import asrq_b200
        asrq_b200.check_status(device)
    return wl, line


def strong_scaling_c4(args, rank, world, device):
    """The 32 utterances of ONE batch divided among the ranks (dp.shard_range); time = max over ranks."""
    from asrq_b200 import dp
    lo, hi = dp.shard_range(WhisperLargeV3.B, rank, world)
    wl = WhisperLargeV3(device, args.seed, batch=hi - lo)
    for i in range(2):
        wl.step(i)
    torch.cuda.synchronize()
    dp.barrier()
    a = event()
    n = 3
    for i in range(n):
        wl.step(i)
    b = event()
    torch.cuda.synchronize()
    dp.barrier()
    ms = dp.max_over_ranks(a.elapsed_time(b)) / n
    return {"scaling": "strong", "global_batch": WhisperLargeV3.B, "per_rank_batch": hi - lo, "ms_per_step": ms,
            "value": WhisperLargeV3.B * 30.0 / (ms * 1e-3), "unit": "RTFx"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="c4")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the other workloads (the `also` rows)")
    ap.add_argument("--no-group", action="store_true", help="one step per CUDA graph instead of a graph of consecutive steps")
    ap.add_argument("--c4-layers", "--layers", dest="c4_layers", type=int, default=None,
                    help="whole-model workloads (c4, c5) at reduced depth (encoder and decoder layers each) and, with --tokens, "
                         "fewer tokens: for bounded profiler captures; the line's config says so and it is not the benchmark")
    ap.add_argument("--c4-tokens", "--tokens", dest="c4_tokens", type=int, default=None)
    args = ap.parse_args()
    if args.steps is None:
        args.steps = 5 if args.workload in ("c4", "c5") else 200
    if args.warmup is None:
        args.warmup = 3
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    from asrq_b200 import dp
    rank, local_rank, world = dp.env_world()
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the asrq_b200 path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dp.init()
    from asrq_b200 import _lib
    _lib.load()
    peaks = measured_peaks()

    wl, line = measure(args.workload, args, rank, local_rank, world, device, peaks, args.steps, args.warmup, True)
    del wl
    torch.cuda.empty_cache()
    if args.workload == "c4" and world > 1:
        s = strong_scaling_c4(args, rank, world, device)
        if rank == 0:
            line["strong_scaling"] = s
        torch.cuda.empty_cache()
    if world == 1 and not args.no_extra:
        also = []
        for other in ("c1", "c2", "c3", "large", "c5", "c4"):
            if other == args.workload:
                continue
            try:
                k = 3 if other in ("c4", "c5") else 200
                w2, l2 = measure(other, args, rank, local_rank, world, device, peaks, k, 3, other != "large")
                also.append(l2)
                del w2
                torch.cuda.empty_cache()
            except BaseException as e:  # a secondary row must not take the headline down
                also.append({"workload": other, "error": repr(e)})
        line["also"] = also
    dp.barrier()
    if rank == 0:
        emit(line)
    dp.finalize()


if __name__ == "__main__":
    # Standard output carries the one result line and nothing else: libraries that write to file
    # descriptor 1 (NCCL's version banner) are sent to standard error instead.
    sys.stdout.flush()
    _RESULT_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    main()
