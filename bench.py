#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c1|c3] [--impl ours|reference]

Prints ONE JSON line.  A "step" is one pass of the hot path over one batch of synthetic
input (seeded, the shapes and value distributions of the benchmark configs):

  c2 (default)  W4A4 LinearQQ: online Hadamard-4096 + per-token int4 activations, int4 g128
                weights, K=4096 N=1024 M=6000.  metric: int TOP/s of 2*M*N*K.
  c1            W4A16 LinearQ, RTN g128, K=1280 N=5120 M=1500 (+bias).  metric: TFLOP/s.
  c3            W4A16/W2A16 decode sweep, Qwen3-1.7B shapes, M in {1,2,4,8,16}, g64.
                metric: GB/s of algorithmic bytes.

``value`` is timed with inputs resident in HBM; ``e2e`` goes through the public module
(``LinearQ`` / ``LinearQQ`` ``.forward``) with pinned HOST input and output buffers, copies inside
the timed region.  With N > 1 (torchrun) every rank runs the same step on its own replica and
its own batch (weak scaling, no data-path collective); time is the max over ranks.

``--impl reference`` times the reference algorithm's CPU restatement (oracle/) on the host cores.
"""
from __future__ import annotations

import argparse
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


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

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


# ------------------------------------------------------------------------------------------
# workloads (device side)
# ------------------------------------------------------------------------------------------


class Workload:
    name = ""
    metric = ""
    unit = ""
    dtype = ""
    launches_per_step = 0

    def units_per_step(self):  # flops, int-ops or bytes per step per GPU
        raise NotImplementedError


class W4A4Config2(Workload):
    """BASELINE config 2."""
    name = "c2"
    metric = "linearq_w4a4_gemm_throughput"
    unit = "TOP/s"
    dtype = "fp8 e4m3 operands holding int4 codes, exact integer group sums in fp32 (tcgen05 kind::f8f6f4); fp16 in/out"
    M, K, N, G = 6000, 4096, 1024, 128
    launches_per_step = 2

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
        self.l2_note = f"rotating {nsets} input sets ({nsets * x.numel() * 2 >> 20} MiB > 126 MiB L2)"
        self.x_host = [t.cpu().pin_memory() for t in self.xs[:2]]
        self.y_host = torch.empty(self.M, self.N, dtype=torch.float16).pin_memory()

    def units_per_step(self):
        return 2.0 * self.M * self.N * self.K

    # algorithmic bytes of the two kernels
    def prologue_bytes(self):
        return self.M * self.K * 2 + self.M * self.K + self.M * 4  # x in, 8-bit operand out, scales out

    def gemm_bytes(self):
        return self.M * self.K + self.N * self.K + self.N * (self.K // self.G) * 2 + self.M * 4 + self.M * self.N * 2

    nsets = property(lambda self: len(self.xs))

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

    kernels = ["hadamard_quant", "w4a4_gemm"]

    def e2e_step(self, i):
        import asrq_b200
        xh = self.x_host[i % len(self.x_host)]
        asrq_b200.forward_host(self.layer, xh, self.y_host, chunks=E2E_CHUNKS)
        return xh.numel() * 2, self.y_host.numel() * 2

    def roofline(self, kernel_ms, peaks, int8_tops):
        ach = self.units_per_step() / (kernel_ms["w4a4_gemm"] * 1e-3) / 1e12
        out = {"kernel": "w4a4_gemm", "bound": "tensor", "achieved": ach, "unit": "TOP/s",
               "peak": int8_tops, "peak_source": "torch._int_mm 8192^3 timed in this run (8-bit tensor peak is not in MEASURED_PEAKS.json; "
                              "fp8 and int8 have the same nominal rate)",
               "frac": ach / int8_tops if int8_tops else None,
               "frac_of_2x_bf16_measured": ach / (2 * peaks["bf16_tflops"]),
               # dram__bytes_read.sum + dram__bytes_write.sum of one w4a4_tc_kernel launch, from the ncu capture
               # summarised in profiles/w4a4_prologue_and_gemm_c2.md (the 12 MB of outputs were still in L2)
               "traffic": 28899584, "traffic_algorithmic": self.gemm_bytes()}
        pro = self.prologue_bytes() / (kernel_ms["hadamard_quant"] * 1e-3) / 1e9
        out["prologue"] = {"kernel": "hadamard4096_quant_kernel", "bound": "hbm", "achieved": pro, "unit": "GB/s",
                           "peak": peaks["hbm_gbs"], "frac": pro / peaks["hbm_gbs"], "of": peaks["source"]}
        return out

    def cpu_sample(self):
        from oracle import linearq_oracle as O
        ms = 256
        x = self.case["x"][:ms]
        codes, sw, _ = O.prepare_w4a4_weight(self.case["w_fp"], self.G, True)

        def run():
            qa, sa, _ = O.hadamard_quant_int4(x, True)
            return O.w4a4_forward_fp32(qa, sa, codes, sw, self.case["bias"], self.G)
        return run, 2.0 * ms * self.N * self.K, f"first {ms} of {self.M} tokens, full K and N; prologue + grouped int GEMM"


class W4A16Config1(Workload):
    """BASELINE config 1."""
    name = "c1"
    metric = "linearq_w4a16_gemm_throughput"
    unit = "TFLOP/s"
    dtype = "f16 (fp32 accumulation)"
    M, K, N, G = 1500, 1280, 5120, 128
    launches_per_step = 1

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
        # one layer is 23 MB: rotate enough (x, W, y) sets to exceed L2 twice over
        per_set = self.algorithmic_bytes()
        nsets = (2 * L2_BYTES) // per_set + 1
        gen = torch.Generator().manual_seed(seed + 1)
        self.sets = []
        for r in range(nsets):
            perm = torch.randperm(self.N, generator=gen)
            self.sets.append(dict(
                x=c["x"][torch.randperm(self.M, generator=gen)].to(device).contiguous(),
                w=c["weight"][perm].to(device).contiguous(), s=c["scales"][perm].to(device).contiguous(),
                z=c["zeros"][perm].to(device).contiguous(), b=c["bias"][perm].to(device).contiguous(),
                y=torch.empty(self.M, self.N, dtype=torch.float16, device=device)))
        self.ws = torch.zeros(max(1 << 20, _lib.workspace_bytes(_lib.WS_LINEARQ, self.M, self.N, self.K)),
                              dtype=torch.uint8, device=device)
        self.l2_note = f"rotating {nsets} (x, W, y) sets ({nsets * per_set >> 20} MiB > 126 MiB L2)"
        self.x_host = [c["x"].pin_memory()]
        self.y_host = torch.empty(self.M, self.N, dtype=torch.float16).pin_memory()

    def units_per_step(self):
        return 2.0 * self.M * self.N * self.K

    def algorithmic_bytes(self):
        return (2 * self.M * self.K + self.N * self.K // 2 + 2 * self.N * (self.K // self.G) * 2 + 2 * self.N
                + 2 * self.M * self.N)

    nsets = property(lambda self: len(self.sets))

    def run_kernel(self, name, i):
        st = torch.cuda.current_stream().cuda_stream
        s = self.sets[i % len(self.sets)]
        self.lib.call("asrq_w4a16_gemm", s["x"].data_ptr(), s["w"].data_ptr(), s["s"].data_ptr(), s["z"].data_ptr(),
                      s["b"].data_ptr(), s["y"].data_ptr(), self.M, self.N, self.K, self.G, self.lib.F16,
                      self.ws.data_ptr(), self.ws.numel(), st)

    def step(self, i):
        self.run_kernel("gemm_a16_tc", i)

    kernels = ["gemm_a16_tc"]

    def e2e_step(self, i):
        import asrq_b200
        xh = self.x_host[0]
        asrq_b200.forward_host(self.layer, xh, self.y_host, chunks=E2E_CHUNKS)
        return xh.numel() * 2, self.y_host.numel() * 2

    def roofline(self, kernel_ms, peaks, int8_tops):
        ach = self.units_per_step() / (kernel_ms["gemm_a16_tc"] * 1e-3) / 1e12
        return {"kernel": "gemm_a16_tc2 (CTA pairs)", "bound": "tensor", "achieved": ach, "unit": "TFLOP/s",
                "peak": peaks["bf16_tflops"], "frac": ach / peaks["bf16_tflops"], "of": peaks["source"] + " (burst)",
                # dram bytes of one gemm_a16_tc2_kernel launch (the CTA-pair kernel) from the ncu capture summarised in
                # profiles/gemm_a16_tc_c1.md (x and W are L2 hits after the first touch, y was still in L2)
                "traffic": 7365376, "traffic_algorithmic": 22691840}

    def cpu_sample(self):
        from oracle import linearq_oracle as O
        c = self.case

        def run():
            return O.linearq_forward(c["x"].float(), c["weight"], c["scales"], c["zeros"], c["bias"].float(), 4, self.G)
        return run, self.units_per_step(), "the full layer (M=1500), fp32 activations: dequantize + torch.matmul"


class DecodeSweepConfig3(Workload):
    """BASELINE config 3: every (shape, bits, M) once per step, each on its own weight copy."""
    name = "c3"
    metric = "linearq_decode_gemv_bandwidth"
    unit = "GB/s"
    dtype = "f16 (fp32 accumulation)"
    SHAPES = [(2048, 6144), (6144, 2048), (2048, 4096)]
    MS = [1, 2, 4, 8, 16]
    G = 64

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
                    it = dict(m=m, k=k, n=n, bits=bits, x=base["x"][:m].to(device).contiguous(),
                              w=base["weight"][perm].to(device).contiguous(),
                              s=base["scales"][perm].to(device).contiguous(),
                              z=base["zeros"][perm].to(device).contiguous(),
                              y=torch.empty(m, n, dtype=torch.float16, device=device))
                    it["bytes"] = 2 * m * k + n * k * bits // 8 + 2 * n * (k // self.G) * 2 + 2 * m * n
                    total += it["bytes"]
                    self.items.append(it)
        self.case0 = O.make_c3(seed=seed, m=1, k=2048, n=6144, bits=4, group_size=self.G)
        self.total_bytes = total
        # the sweep touches ~143 MB of distinct weights per step; two copies make it > 2x L2
        self.copies = 2
        self.items2 = [dict(it, w=it["w"].clone(), s=it["s"].clone(), z=it["z"].clone()) for it in self.items]
        self.launches_per_step = len(self.items)
        self.ws = torch.zeros(_lib.workspace_bytes(_lib.WS_LINEARQ, 16, 6144, 6144), dtype=torch.uint8, device=device)
        self.l2_note = (f"{len(self.items)} launches per step replayed as one CUDA graph, each on its own weight copy "
                        f"({2 * total >> 20} MiB over two alternating sets > 126 MiB L2)")

    def units_per_step(self):
        return float(self.total_bytes)

    def _launch_all(self, items):
        st = torch.cuda.current_stream().cuda_stream
        for it in items:
            self.lib.call(f"asrq_w{it['bits']}a16_gemv", it["x"].data_ptr(), it["w"].data_ptr(), it["s"].data_ptr(),
                          it["z"].data_ptr(), None, it["y"].data_ptr(), it["m"], it["n"], it["k"], self.G,
                          self.lib.F16, self.ws.data_ptr(), self.ws.numel(), st)

    nsets = 2

    def run_kernel(self, name, i):
        self._launch_all(self.items if i % 2 == 0 else self.items2)

    def step(self, i):
        self.run_kernel("gemv_a16 (30 launches)", i)

    kernels = ["gemv_a16 (30 launches)"]

    def e2e_step(self, i):
        """The sweep through the C ABI with host activations: every launch's x comes from pinned host
        memory and its y goes back to pinned host memory."""
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

    def roofline(self, kernel_ms, peaks, int8_tops):
        ach = self.total_bytes / (kernel_ms["gemv_a16 (30 launches)"] * 1e-3) / 1e9
        return {"kernel": "gemv_a16", "bound": "hbm", "achieved": ach, "unit": "GB/s", "peak": peaks["hbm_gbs"],
                "frac": ach / peaks["hbm_gbs"], "of": peaks["source"],
                # ncu captured one launch of the sweep (W4 2048->6144, M=1): 7 101 440 B of DRAM reads for
                # 7 094 272 algorithmic bytes (profiles/gemv_a16_c3.md); the sweep's traffic is its algorithmic
                # bytes scaled by that ratio (every launch streams its weights exactly once)
                "traffic": self.total_bytes * 7101440.0 / 7094272.0}

    def cpu_sample(self):
        from oracle import linearq_oracle as O
        c = self.case0

        def run():
            return O.linearq_forward(c["x"].float(), c["weight"], c["scales"], c["zeros"], None, 4, self.G)
        b = 2 * 2048 + 6144 * 2048 // 2 + 2 * 6144 * 32 * 2 + 2 * 6144
        return run, float(b), "one launch of the sweep: W4 g64 K=2048 N=6144 M=1, dequantize + torch.matmul"


class DecodeLargeLayer(Workload):
    """Supplementary, not a BASELINE config: the decode kernel on one layer large enough that launch and
    ramp-up latency do not dominate (W4 g128, 8192 -> 28672, M=1; 112 MiB of packed weights per launch)."""
    name = "large"
    metric = "linearq_decode_gemv_bandwidth_large_layer"
    unit = "GB/s"
    dtype = "f16 (fp32 accumulation)"
    M, K, N, G = 1, 8192, 28672, 128
    launches_per_step = 1

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

    nsets = 3
    kernels = ["gemv_a16"]

    def units_per_step(self):
        return float(2 * self.M * self.K + self.N * self.K // 2 + 2 * self.N * (self.K // self.G) * 2 + 2 * self.M * self.N)

    def run_kernel(self, name, i):
        self.lib.call("asrq_w4a16_gemv", self.x.data_ptr(), self.ws_[i % 3].data_ptr(), self.s.data_ptr(),
                      self.z.data_ptr(), None, self.y.data_ptr(), self.M, self.N, self.K, self.G, self.lib.F16,
                      self.ws.data_ptr(), self.ws.numel(), torch.cuda.current_stream().cuda_stream)

    def step(self, i):
        self.run_kernel("gemv_a16", i)

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

    def cpu_sample(self):
        from oracle import linearq_oracle as O
        rows = 1024
        c = O.make_c3(seed=0, m=1, k=self.K, n=rows, bits=4, group_size=self.G)

        def run():
            return O.linearq_forward(c["x"].float(), c["weight"], c["scales"], c["zeros"], None, 4, self.G)
        b = 2 * self.K + rows * self.K // 2 + 2 * rows * (self.K // self.G) * 2 + 2 * rows
        return run, float(b), f"{rows} of {self.N} output features, full K, M=1: dequantize + torch.matmul"

    def roofline(self, kernel_ms, peaks, int8_tops):
        ach = self.units_per_step() / (kernel_ms["gemv_a16"] * 1e-3) / 1e9
        return {"kernel": "gemv_a16 (rounds variant)", "bound": "hbm", "achieved": ach, "unit": "GB/s",
                "peak": peaks["hbm_gbs"], "frac": ach / peaks["hbm_gbs"], "of": peaks["source"], "traffic": None}


E2E_CHUNKS = int(os.environ.get("ASRQ_BENCH_E2E_CHUNKS", "4"))  # token chunks of the host-to-host call (1: no overlap)

WORKLOADS = {"c1": W4A16Config1, "c2": W4A4Config2, "c3": DecodeSweepConfig3, "large": DecodeLargeLayer}


def library_gemm_same_shape(device, m, k, n, kind, reps=40):
    """Context for a tensor-bound roofline: the vendor library's plain dense GEMM on this very shape,
    timed by the protocol of the bench (one kernel per CUDA graph, graphs replayed back to back over
    rotating operands).  ``kind`` "f16": torch.matmul on fp16 operands (what the reference's
    dequantize-then-matmul path runs after its dequantisation); "int8": torch._int_mm.  Not a peak and
    not this library's code: a 20-50 us problem does not reach the 8192^3 rate in any implementation."""
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
        st = torch.cuda.Stream(device)
        graphs = []
        with torch.cuda.stream(st):
            for i in range(nset):
                fn(i)
                torch.cuda.synchronize(device)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=st):
                    fn(i)
                graphs.append(g)
            for g in graphs:
                g.replay()
            torch.cuda.synchronize(device)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st)
            for r in range(reps):
                graphs[r % nset].replay()
            e1.record(st)
            torch.cuda.synchronize(device)
        ms = e0.elapsed_time(e1) / reps
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
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            e1.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return 2 * 8192 ** 3 / (best * 1e-3) / 1e12
    except Exception:
        return None


def cpu_baseline(wl, kind="port", budget_s=15.0):
    run, units, sample = wl.cpu_sample()
    torch.set_num_threads(os.cpu_count() or 1)
    run()
    t0 = time.perf_counter()
    n = 0
    while True:
        run()
        n += 1
        if time.perf_counter() - t0 > budget_s or n >= 20:
            break
    dt = (time.perf_counter() - t0) / n
    scale = 1e12 if wl.unit in ("TOP/s", "TFLOP/s") else 1e9
    return {"value": units / dt / scale, "unit": wl.unit, "cores": torch.get_num_threads(), "kind": kind,
            "sample": sample, "ms_per_sample": dt * 1e3}


def run_reference(args, rank):
    """The reference algorithm's CPU implementation (oracle restatement) on the host cores."""
    if rank != 0:
        return
    sys.path.insert(0, ROOT)
    cls = WORKLOADS[args.workload]
    wl = cls.__new__(cls)
    from oracle import linearq_oracle as O
    if args.workload == "c2":
        wl.case = O.make_c2(seed=args.seed, m=512, k=cls.K, n=cls.N, group_size=cls.G)
    elif args.workload == "c1":
        wl.case = O.make_c1(seed=args.seed, m=cls.M, k=cls.K, n=cls.N, bits=4, group_size=cls.G)
    elif args.workload == "c3":
        wl.case0 = O.make_c3(seed=args.seed, m=1, k=2048, n=6144, bits=4, group_size=cls.G)
    run, units, sample = wl.cpu_sample()
    torch.set_num_threads(os.cpu_count() or 1)
    for _ in range(max(1, min(args.warmup, 3))):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    dt = (time.perf_counter() - t0) / args.steps
    scale = 1e12 if cls.unit in ("TOP/s", "TFLOP/s") else 1e9
    v = units / dt / scale
    line = {"impl": "reference", "metric": cls.metric, "value": v, "unit": cls.unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32 (CPU)", "data": "synthetic",
            "config": {"workload": args.workload, "note": "reference algorithm (dequantize + matmul / quantise + int GEMM) "
                       "restated in torch on the CPU; the reference's own Python cannot travel to the GPU box"},
            "cpu_baseline": {"value": v, "unit": cls.unit, "cores": torch.get_num_threads(), "kind": "port",
                             "sample": sample},
            "e2e": {"value": v, "unit": cls.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    emit(line)


_RESULT_OUT = sys.stdout


def emit(line):
    """Writes the result line to the process's original standard output."""
    _RESULT_OUT.write(json.dumps(line) + "\n")
    _RESULT_OUT.flush()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="c2")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary workloads")
    args = ap.parse_args()
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

    def capture(fn, n):
        """One CUDA graph per input set: a step issued call by call from Python is bound by the host (the
        ctypes call and the launch cost as much as these kernels run), so steps are replayed as graphs."""
        graphs = []
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(n):
                fn(i)
            torch.cuda.synchronize()
            for i in range(n):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    fn(i)
                graphs.append(g)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        return graphs

    def measure(name, steps, warmup, with_e2e):
        wl = WORKLOADS[name](device, args.seed + 1000 * rank)
        graphs = capture(wl.step, wl.nsets)
        for i in range(warmup):
            graphs[i % wl.nsets].replay()
        torch.cuda.synchronize()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        dp.barrier()
        torch.cuda.synchronize()
        t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_start.record()
        for i in range(steps):
            graphs[(warmup + i) % wl.nsets].replay()
        t_end.record()
        torch.cuda.synchronize()
        dp.barrier()
        clocks = sampler.stop() if rank == 0 else None
        total_ms = dp.max_over_ranks(t_start.elapsed_time(t_end))
        # each kernel alone, the same way (outside the timed region of the step)
        kernel_ms = {}
        if len(wl.kernels) == 1:
            kernel_ms[wl.kernels[0]] = t_start.elapsed_time(t_end) / steps
        else:
            for kname in wl.kernels:
                kg = capture(lambda i, kname=kname: wl.run_kernel(kname, i), wl.nsets)
                for i in range(3):
                    kg[i % wl.nsets].replay()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for i in range(steps):
                    kg[i % wl.nsets].replay()
                b.record()
                torch.cuda.synchronize()
                kernel_ms[kname] = a.elapsed_time(b) / steps
        e2e = None
        if with_e2e and wl.e2e_step(0) is not None:
            for i in range(3):
                wl.e2e_step(i)
            torch.cuda.synchronize()
            dp.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for i in range(steps):
                h2d, d2h = wl.e2e_step(i)
            b.record()
            torch.cuda.synchronize()
            dp.barrier()
            e2e_ms = dp.max_over_ranks(a.elapsed_time(b)) / steps
            scale = 1e12 if wl.unit in ("TOP/s", "TFLOP/s") else 1e9
            e2e = {"value": wl.units_per_step() * world / (e2e_ms * 1e-3) / scale, "unit": wl.unit,
                   "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                   "api": (f"asrq_b200.forward_host({type(wl.layer).__name__}, pinned host in, pinned host out, chunks={E2E_CHUNKS}): "
                           "copies in and out overlapped with the kernels chunk by chunk"
                           if hasattr(wl, "layer") else "the C-ABI decode calls with pinned host activations in and pinned host outputs back")}
        _lib.call("asrq_check_status", wl.ws.data_ptr(), torch.cuda.current_stream().cuda_stream)
        return wl, total_ms / steps, kernel_ms, clocks, e2e

    wl, ms_step, kernel_ms, clocks, e2e = measure(args.workload, args.steps, args.warmup, True)
    scale = 1e12 if wl.unit in ("TOP/s", "TFLOP/s") else 1e9
    value = wl.units_per_step() * world / (ms_step * 1e-3) / scale
    int8_tops = time_int8_peak(device) if (rank == 0 and args.workload == "c2") else None
    line = {
        "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": {"workload": f"{wl.name}: " + (wl.__doc__ or "").strip(), "per_gpu": "every rank runs the full step "
                   "on its own replica and batch; no data-path collective", "l2": wl.l2_note,
                   "launch": "each step is one CUDA-graph replay, captured once per input set (a step issued call by call from Python is host-bound)",
                   "M": getattr(wl, "M", None), "K": getattr(wl, "K", None), "N": getattr(wl, "N", None)},
        "kernel_ms": kernel_ms, "gpu_launches": wl.launches_per_step * args.steps, "clocks": clocks,
    }
    if rank == 0:
        line["roofline"] = wl.roofline(kernel_ms, peaks, int8_tops)
        if wl.name == "c1":
            line["roofline"]["library_gemm_same_shape"] = library_gemm_same_shape(device, wl.M, wl.K, wl.N, "f16")
        elif wl.name == "c2":
            line["roofline"]["library_gemm_same_shape"] = library_gemm_same_shape(device, wl.M, wl.K, wl.N, "int8")
            line["roofline"]["library_f16_gemm_same_shape"] = library_gemm_same_shape(device, wl.M, wl.K, wl.N, "f16")
        line["e2e"] = e2e
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(wl)
    del wl
    torch.cuda.empty_cache()
    if world == 1 and not args.no_extra:
        also = []
        for other in sorted(WORKLOADS):
            if other == args.workload:
                continue
            try:
                w2, ms2, k2, _, _ = measure(other, min(args.steps, 20), 3, False)
                sc2 = 1e12 if w2.unit in ("TOP/s", "TFLOP/s") else 1e9
                also.append({"workload": other, "metric": w2.metric, "value": w2.units_per_step() / (ms2 * 1e-3) / sc2,
                             "unit": w2.unit, "ms_per_step": ms2, "kernel_ms": k2,
                             "roofline": w2.roofline(k2, peaks, None)})
                if other == "c1":
                    also[-1]["roofline"]["library_gemm_same_shape"] = library_gemm_same_shape(device, w2.M, w2.K, w2.N, "f16")
                del w2
                torch.cuda.empty_cache()
            except Exception as e:  # a secondary row must not take the headline down
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
