#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--case NAME] [--tokens M]

Default case `flux_fp8` (the headline; N=1 and per rank at N>1): the four FP8 e4m3 FLUX.1-dev-shaped linears at
M = 4608 tokens (QKV 3072->9216, out-proj 3072->3072, MLP-up 3072->12288 + tanh-GELU, MLP-down 12288->3072 +
residual).  One step = for each linear: per-tensor e4m3 activation quantize (bf16 -> e4m3) + the tcgen05 FP8 GEMM
with its fused epilogue.  Other cases time the remaining configurations with the same harness:
    int8_sdxl    SDXL GEGLU-FF INT8 SmoothQuant linear, M=8192 K=640 N=5120 (dynamic per-token quantize + GEMM)
    w4a4         FLUX fused W4A4 linear, M=4608 K=3072 N=21504 (int4 group-64 quantize + GEMM)
    flux_block   one FLUX single-stream block through FluxSingleTransformerBlockOp (FP8 linears + library attention)
    flux_forward the FLUX.1-dev block stack (19 double + 38 single blocks, own weights each): ms per denoising step
    sdxl_ff      the whole SDXL GEGLU feed-forward block in INT8 (four launches)
    adaln_quant  fused AdaLN-modulation + int8 and e4m3 quantize of [4608, 3072] bf16
`--tokens` shrinks M (for profiler captures).  Synthetic seeded inputs, random weights.  Rank 0 prints ONE JSON line.

`value` is whole-job throughput with inputs resident in HBM; `e2e` is the same metric through the public API from
pinned HOST buffers (H2D of the step's activations and D2H of its result inside the timed region).
`--impl reference` times the CPU restatement of the reference's arithmetic (the oracle port, torch on all host
cores) on a bounded row sample of the same workload.
"""

import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {"bf16_sustained": float(p["bf16_tflops_sustained"]), "bf16_burst": float(p["bf16_tflops"]),
                "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    except Exception:
        return {"bf16_sustained": 1400.0, "bf16_burst": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self.stop_flag = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
        while not self.stop_flag.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    r = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    r = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.001)

    def result(self):
        self.stop_flag.set()
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_min_mhz": s[0], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def tensor_peak(peaks, mode, factor, what):
    """Measured tensor peak for the denominator of a roofline fraction.  mode "burst": the timed region is a short burst at
    flat clocks (a kernel timed alone) -> bf16_tflops; "sustained": a seconds-long region under the power cap ->
    bf16_tflops_sustained.  factor 2 for FP8 / INT8 (no FP8 peak is measured on this pool; dense FP8 / INT8 runs at twice
    the bf16 rate), 1 for 16-bit."""
    key = "bf16_burst" if mode == "burst" else "bf16_sustained"
    name = "bf16_tflops" if mode == "burst" else "bf16_tflops_sustained"
    return factor * peaks[key], "%s%s of MEASURED_PEAKS.json (%s, %s denominator)%s" % (
        "2 x " if factor == 2 else "", name, peaks["source"], mode, what)


def _gen(seed=0):
    return torch.Generator().manual_seed(seed)


# =================================================================================================== cases
class FluxFp8:
    """configs[1]: the four FP8 FLUX linears."""
    name = "flux_fp8"
    metric = "fp8_flux_linears_throughput"
    unit = "TFLOP/s"
    dtype = "f8e4m3 (fp32 accumulate in TMEM)"
    LINEARS = (("qkv", 3072, 9216, False, False), ("out_proj", 3072, 3072, False, False),
               ("mlp_up_gelu", 3072, 12288, True, False), ("mlp_down_residual", 12288, 3072, False, True))

    def __init__(self, tokens):
        self.tokens = tokens or 4608
        self.work_per_step = sum(2.0 * self.tokens * k * n for _, k, n, _, _ in self.LINEARS)  # FLOP
        self.scale = 1e12
        self.workload = ("configs[1]: FP8 e4m3 FLUX.1-dev linears, M=%d tokens, hidden 3072: QKV 3072->9216, out-proj "
                         "3072->3072, MLP-up 3072->12288 +GELU-tanh, MLP-down 12288->3072 +residual; per-tensor e4m3 "
                         "activation quantize before each (a standalone kernel for the first three, fused into the MLP-up "
                         "epilogue for the MLP-down input)" % self.tokens)
        self.launches_per_step = 2 * len(self.LINEARS) - 1
        self.timed_names = [l[0] for l in self.LINEARS]
        self.timed_work = [2.0 * self.tokens * k * n for _, k, n, _, _ in self.LINEARS]
        self.roof = {"bound": "tensor", "unit": "TFLOP/s", "kernel": "gemm_tcgen05_kernel<f8f6f4> (4 launches per step, one per linear)"}
        # dram__bytes_read + write per launch, mean of the four launches (profiles/gemm_tcgen05_fp8_flux_linears.md)
        self.traffic = 110.4e6 if self.tokens == 4608 else None

    def setup_gpu(self, dev):
        from lyradiff_b200 import ops
        self.ops = ops
        g = _gen()
        T = self.tokens
        self.lin = {}
        for name, k, n, gelu, residual in self.LINEARS:
            w = (torch.randn(n, k, generator=g) * 0.02).bfloat16().to(dev)
            s_w = torch.zeros(1, dtype=torch.float32, device=dev)
            ops.invoke_get_fp8_weight_scale(s_w, w)
            qw = torch.empty(n, k, dtype=torch.uint8, device=dev)
            ops.invoke_cuda_d2d_scale_cpy_convert(qw, w, s_w)
            del w
            self.lin[name] = {
                "x": torch.randn(T, k, generator=g).bfloat16().to(dev) if name != "mlp_down_residual" else None,
                "qx": torch.empty(T, k, dtype=torch.uint8, device=dev),
                "s_x": torch.tensor([6.0 / 448.0], dtype=torch.float32, device=dev),
                "qw": qw, "s_w": s_w,
                "bias": (torch.randn(n, generator=g) * 0.02).bfloat16().to(dev),
                "residual": torch.randn(T, n, generator=g).bfloat16().to(dev) if residual else None,
                "y": torch.empty(T, n, dtype=torch.bfloat16, device=dev),
            }
        self.h_in = torch.randn(T, 3072, generator=g).bfloat16().pin_memory()
        # end-to-end path: the step's activations (input of the first linear) arrive from the host, the result of the
        # last linear goes back; two device slots of each so that copies and compute of neighbouring steps overlap
        self.e2e_x = [self.lin["qkv"]["x"], torch.empty_like(self.lin["qkv"]["x"])]
        self.e2e_y = [self.lin["mlp_down_residual"]["y"], torch.empty_like(self.lin["mlp_down_residual"]["y"])]

    def step(self, events=None, io=None):
        ops = self.ops
        for i, (name, k, n, gelu, residual) in enumerate(self.LINEARS):
            L = self.lin[name]
            x = self.lin["mlp_up_gelu"]["y"] if name == "mlp_down_residual" else L["x"]
            y = L["y"]
            if io is not None and name == "qkv":
                x = io[0]
            if io is not None and name == "mlp_down_residual":
                y = io[1]
            if name != "mlp_down_residual":
                ops.invoke_cuda_d2d_scale_cpy_convert(L["qx"], x, L["s_x"])
            if events is not None:
                events[i][0].record()
            if name == "mlp_up_gelu":
                # the quantize of the down projection's input is fused into this GEMM's epilogue: GELU(...) goes out as e4m3
                D = self.lin["mlp_down_residual"]
                ops.gemm_fp8_quant_out(L["qw"], L["s_w"], L["qx"], L["s_x"], D["qx"], D["s_x"], torch.bfloat16, bias=L["bias"],
                                       is_gelu=True)
            else:
                ops.gemm_with_residual_and_bias_fp8(L["qw"], L["s_w"], L["qx"], L["s_x"], y, bias=L["bias"],
                                                    residual=L["residual"], is_gelu=gelu)
            if events is not None:
                events[i][1].record()

    def peak(self, peaks, mode):
        v, src = tensor_peak(peaks, mode, 2, ": dense FP8 at twice the bf16 rate; nominal dense FP8 is 4500")
        return v, src, 4500.0

    # ---- CPU restatement on a row sample
    def setup_cpu(self, rows):
        from oracle import quant as oq
        g = _gen()
        self.cpu = {}
        for name, k, n, gelu, residual in self.LINEARS:
            w = (torch.randn(n, k, generator=g) * 0.02).bfloat16()
            s_w = oq.fp8_amax_scale(w)
            self.cpu[name] = {"x": torch.randn(rows, k, generator=g).bfloat16(), "s_x": torch.tensor([6.0 / 448.0]), "s_w": s_w,
                              "w_t": oq.fp8_dequant(oq.fp8_quant(w, s_w)).t().contiguous(),
                              "bias": (torch.randn(n, generator=g) * 0.02).bfloat16(),
                              "residual": torch.randn(rows, n, generator=g).bfloat16() if residual else None}
        self.cpu_rows = rows

    def step_cpu(self):
        from oracle import gemm as og
        from oracle import quant as oq
        outs = {}
        for name, k, n, gelu, residual in self.LINEARS:
            L = self.cpu[name]
            x = outs["mlp_up_gelu"] if name == "mlp_down_residual" else L["x"]
            xf = oq.fp8_dequant(oq.fp8_quant(x, L["s_x"]))
            v = (xf @ L["w_t"]) * (float(L["s_x"]) * float(L["s_w"]))
            if residual:
                v = v + L["residual"].float()
            v = v + L["bias"].float()
            if gelu:
                v = og.gelu_tanh(v)
            outs[name] = v.to(torch.bfloat16)
        return outs

    cpu_note = "quantize + e4m3 GEMM as fp32 upcast matmul + epilogue, all four linears"


class Int8Sdxl:
    """configs[0]: SDXL GEGLU-FF INT8 SmoothQuant linear."""
    name = "int8_sdxl"
    metric = "int8_smoothquant_linear_throughput"
    unit = "TOP/s"
    dtype = "s8 (s32 accumulate in TMEM)"
    K, N = 640, 5120
    roof_scale = 1e9  # the roofline of this case is in GB/s while the metric is in TOP/s

    def __init__(self, tokens):
        self.tokens = tokens or 8192
        T = self.tokens
        self.work_per_step = 2.0 * T * self.K * self.N
        self.scale = 1e12
        self.workload = ("configs[0]: INT8 SmoothQuant W8A8 linear, SDXL GEGLU-FF shape M=%d K=640 N=5120: dynamic per-token "
                         "int8 quantize of fp16 X (with smoothing vector) + INT8 GEMM + dequant + bias -> fp16" % T)
        self.launches_per_step = 2
        self.timed_names = ["int8_gemm"]
        # the GEMM is bound by its fp16 output store: algorithmic bytes A + W + out + scales
        self.gemm_bytes = T * self.K + self.N * self.K + 2.0 * T * self.N + 4.0 * (T + self.N) + 2.0 * self.N
        self.timed_work = [self.gemm_bytes]
        self.roof = {"bound": "hbm", "unit": "GB/s", "kernel": "gemm_tcgen05_kernel<i8> (1 launch per step)"}
        self.traffic = 33.6e6 if T == 8192 else None  # profiles/gemm_tcgen05_int8_sdxl.md (most of the output is still in L2)

    @staticmethod
    def _inputs(rows, k, n):
        """Seeded inputs of configs[0]: X ~ N(0,1) with 5 % of the channels scaled x20, W ~ N(0,0.02), bias ~ N(0,0.02), and the
        SmoothQuant vector s_j = max|X_j|^0.5 / max|W_j|^0.5 (activations are multiplied by pre = 1/s)."""
        g = _gen()
        x = torch.randn(rows, k, generator=g)
        x[:, torch.randperm(k, generator=g)[:max(1, (k * 5) // 100)]] *= 20.0
        w = (torch.randn(n, k, generator=g) * 0.02).half()
        bias = (torch.randn(n, generator=g) * 0.02).half()
        x = x.half()
        smooth = x.float().abs().amax(dim=0).sqrt() / w.float().abs().amax(dim=0).sqrt()
        return x, w, bias, (1.0 / smooth).float()

    def setup_gpu(self, dev):
        from lyradiff_b200 import ops
        self.ops = ops
        x, w, bias, pre = self._inputs(self.tokens, self.K, self.N)
        self.x, self.pre, self.bias = x.to(dev), pre.to(dev), bias.to(dev)
        # the folded weight W / pre is quantized per output channel by the library's own load-time kernel
        self.qw = torch.empty(self.N, self.K, dtype=torch.int8, device=dev)
        self.s_w = torch.empty(self.N, dtype=torch.float32, device=dev)
        ops.invoke_get_int8_weight_scale(self.s_w, self.qw, w.to(dev), self.pre)
        self.qa = torch.empty(self.tokens, self.K, dtype=torch.int8, device=dev)
        self.sa = torch.empty(self.tokens, dtype=torch.float32, device=dev)
        self.y = torch.empty(self.tokens, self.N, dtype=torch.float16, device=dev)
        # a second output buffer alternates with the first so that consecutive steps do not rewrite lines still in L2
        self.y2 = torch.empty_like(self.y)
        self.h_in = x.pin_memory()
        self.e2e_x = [self.x, torch.empty_like(self.x)]
        self.e2e_y = [self.y, self.y2]
        self.flip = False

    def step(self, events=None, io=None):
        ops = self.ops
        self.flip = not self.flip
        x = self.x if io is None else io[0]
        y = (self.y if self.flip else self.y2) if io is None else io[1]
        ops.invoke_sq_input_quant(self.qa, x, self.pre, self.sa, dynamic=True)
        if events is not None:
            events[0][0].record()
        ops.run_gemm_int8(self.qa, self.qw, self.s_w, self.sa, y, bias=self.bias, per_token=True)
        if events is not None:
            events[0][1].record()

    def peak(self, peaks, mode):
        return peaks["hbm_gbs"], "hbm_gbs of MEASURED_PEAKS.json (%s); the fp16 output store bounds this shape" % peaks["source"], 7700.0

    def setup_cpu(self, rows):
        from oracle import quant as oq
        x, w, bias, pre = self._inputs(rows, self.K, self.N)
        qw, s_w = oq.int8_weight_quant_device(w, pre)
        self.cpu = {"x": x, "pre": pre, "bias": bias, "s_w": s_w, "qw_t": qw.t().contiguous()}
        self.cpu_rows = rows

    def step_cpu(self):
        from oracle import quant as oq
        c = self.cpu
        qa, sa = oq.sq_input_quant_dynamic(c["x"], c["pre"])
        acc = torch._int_mm(qa, c["qw_t"])
        y = (acc.float() * (c["s_w"][None, :] * sa[:, None])).half()
        return (y.float() + c["bias"].float()).half()

    cpu_note = "dynamic per-token int8 quantize + torch._int_mm + dequant + bias"


class SdxlFF:
    """The whole SDXL GEGLU feed-forward block in INT8 (configs[0] extended to the block it sits in): LayerNorm -> int8,
    640 -> 5120 GEMM, bias + GEGLU -> int8, 2560 -> 640 GEMM with bias and residual: four launches, no standalone
    elementwise pass (src/lyradiff/layers/basic_transformer/BasicTransformerInt8Block.cc:770-845)."""
    name = "sdxl_ff"
    metric = "int8_geglu_ff_block_throughput"
    unit = "TOP/s"
    dtype = "s8 (s32 accumulate in TMEM)"
    D, H = 640, 2560

    def __init__(self, tokens):
        self.tokens = tokens or 8192
        T = self.tokens
        self.work_per_step = 2.0 * T * (self.D * 2 * self.H + self.H * self.D)
        self.scale = 1e12
        self.workload = ("SDXL GEGLU feed-forward block in INT8 at M=%d: LayerNorm->int8, GEMM 640->5120, bias+GEGLU->int8, "
                         "GEMM 2560->640 + bias + residual -> fp16 (static input scales)" % T)
        self.launches_per_step = 4
        self.timed_names = ["gemm_up", "gemm_down"]
        self.timed_work = [2.0 * T * self.D * 2 * self.H, 2.0 * T * self.H * self.D]
        self.roof = {"bound": "tensor", "unit": "TOP/s", "kernel": "gemm_tcgen05_kernel<i8> (2 launches per step)"}
        self.traffic = None

    def setup_gpu(self, dev):
        from lyradiff_b200 import ops
        self.ops = ops
        g = _gen()
        T, D, H = self.tokens, self.D, self.H
        self.x = torch.randn(T, D, generator=g).half().to(dev)
        self.gamma = (1.0 + 0.1 * torch.randn(D, generator=g)).half().to(dev)
        self.beta = (0.1 * torch.randn(D, generator=g)).half().to(dev)
        self.pre1 = (0.5 + torch.rand(D, generator=g)).float().to(dev)
        self.pre2 = (0.5 + torch.rand(H, generator=g)).float().to(dev)
        self.s1 = torch.tensor([0.05], dtype=torch.float32, device=dev)
        self.s2 = torch.tensor([0.02], dtype=torch.float32, device=dev)
        self.w1 = torch.randint(-127, 128, (2 * H, D), generator=g, dtype=torch.int8).to(dev)
        self.w2 = torch.randint(-127, 128, (D, H), generator=g, dtype=torch.int8).to(dev)
        self.sw1 = (torch.rand(2 * H, generator=g) * 2e-4 + 1e-4).float().to(dev)
        self.sw2 = (torch.rand(D, generator=g) * 2e-4 + 1e-4).float().to(dev)
        self.b1 = (0.02 * torch.randn(2 * H, generator=g)).half().to(dev)
        self.b2 = (0.02 * torch.randn(D, generator=g)).half().to(dev)
        self.q1 = torch.empty(T, D, dtype=torch.int8, device=dev)
        self.h = torch.empty(T, 2 * H, dtype=torch.float16, device=dev)
        self.q2 = torch.empty(T, H, dtype=torch.int8, device=dev)
        self.y = torch.empty(T, D, dtype=torch.float16, device=dev)
        self.h_in = self.x.cpu().pin_memory()
        self.e2e_x = [self.x, torch.empty_like(self.x)]
        self.e2e_y = [self.y, torch.empty_like(self.y)]

    def step(self, events=None, io=None):
        ops = self.ops
        x = self.x if io is None else io[0]
        y = self.y if io is None else io[1]
        ops.invoke_layer_norm_int8o(self.q1, x, self.gamma, self.beta, self.pre1, self.s1)
        if events is not None:
            events[0][0].record()
        ops.run_gemm_int8(self.q1, self.w1, self.sw1, self.s1, self.h)
        if events is not None:
            events[0][1].record()
        ops.invoke_fused_add_bias_geglu_int8o(self.q2, self.h, self.b1, self.pre2, self.s2)
        if events is not None:
            events[1][0].record()
        ops.run_gemm_int8(self.q2, self.w2, self.sw2, self.s2, y, bias=self.b2, residual=x)
        if events is not None:
            events[1][1].record()

    def peak(self, peaks, mode):
        v, src = tensor_peak(peaks, mode, 2, " as the dense INT8 rate; at K = 640 the fp16 store of the first GEMM bounds the block")
        return v, src, 4500.0

    def setup_cpu(self, rows):
        g = _gen()
        D, H = self.D, self.H
        c = {"x": torch.randn(rows, D, generator=g).half()}
        c["gamma"] = (1.0 + 0.1 * torch.randn(D, generator=g)).half()
        c["beta"] = (0.1 * torch.randn(D, generator=g)).half()
        c["pre1"] = (0.5 + torch.rand(D, generator=g)).float()
        c["pre2"] = (0.5 + torch.rand(H, generator=g)).float()
        c["s1"], c["s2"] = torch.tensor([0.05]), torch.tensor([0.02])
        c["w1t"] = torch.randint(-127, 128, (2 * H, D), generator=g, dtype=torch.int8).t().contiguous()
        c["w2t"] = torch.randint(-127, 128, (D, H), generator=g, dtype=torch.int8).t().contiguous()
        c["sw1"] = (torch.rand(2 * H, generator=g) * 2e-4 + 1e-4).float()
        c["sw2"] = (torch.rand(D, generator=g) * 2e-4 + 1e-4).float()
        c["b1"] = (0.02 * torch.randn(2 * H, generator=g)).half()
        c["b2"] = (0.02 * torch.randn(D, generator=g)).half()
        self.cpu, self.cpu_rows = c, rows

    def step_cpu(self):
        from oracle import norms as on
        c = self.cpu
        q1, _ = on.layernorm_int8(c["x"], c["gamma"], c["beta"], c["pre1"], c["s1"])
        h = (torch._int_mm(q1, c["w1t"]).float() * (c["sw1"][None, :] * c["s1"])).half()
        q2 = on.geglu_int8(h, c["b1"], c["pre2"], c["s2"])
        y = (torch._int_mm(q2, c["w2t"]).float() * (c["sw2"][None, :] * c["s2"])).half()
        y = (y.float() + c["x"].float()).half()
        return (y.float() + c["b2"].float()).half()

    cpu_note = "LayerNorm->int8 + torch._int_mm + bias/GEGLU->int8 + torch._int_mm + residual + bias"


class FluxBlock:
    """One FLUX.1-dev single-stream block through torch.classes.lyradiff.FluxSingleTransformerBlockOp (the C++ class; the
    per-block unit of configs[4]): modulation, AdaLN + quantize, QKV, QK-norm + RoPE, attention, MLP, proj_out, gate +
    residual at 4608 tokens.  --python-mirror runs lyradiff_b200.flux_blocks instead (same launches, same bits)."""
    name = "flux_block"
    metric = "flux_single_block_throughput"
    unit = "TFLOP/s"
    dtype = "e4m3 linears (f32 accumulate in TMEM) + bf16 attention (f32 scores and accumulation in TMEM)"
    D, H, DH, MLP = 3072, 24, 128, 4

    def __init__(self, tokens):
        self.tokens = tokens or 4608
        T, D = self.tokens, self.D
        self.lin_flops = 2.0 * T * D * (3 * D + self.MLP * D + (self.MLP + 1) * D)
        self.attn_flops = 4.0 * T * T * D
        self.work_per_step = self.lin_flops + self.attn_flops
        self.scale = 1e12
        self.workload = ("one FLUX.1-dev single-stream block (the unit configs[4] repeats 38 times), FP8_W8A8, batch 1, %d tokens, "
                         "hidden 3072, 24 x 128 heads, random weights: %.3f TFLOP in FP8 linears + %.3f TFLOP in bf16 attention "
                         "(this library's tcgen05 kernel); the resident-input step is replayed as a CUDA graph" % (T, self.lin_flops / 1e12, self.attn_flops / 1e12))
        self.launches_per_step = 6   # AdaLN+quantize, QKV GEMM, QK-norm+RoPE, attention (e4m3 out), MLP GEMM, proj_out GEMM
        self.timed_names = ["block_forward"]
        self.timed_work = [self.work_per_step]
        self.roof = {"bound": "tensor", "unit": "TFLOP/s",
                     "kernel": "whole block: 3 gemm_tcgen05_kernel<f8f6f4> launches, attention_fwd_kernel and 2 element-wise kernels "
                               "of this library, plus one small library matmul (the 16-bit modulation linear)"}
        self.traffic = None

    def _state_dict(self, g, on_gpu=False):
        D, M = self.D, self.MLP
        p = "single_transformer_blocks.0."
        sd = {}
        for name, n, k, std in (("norm.linear", 3 * D, D, 0.02), ("attn.to_qkv", 3 * D, D, 0.02), ("proj_mlp", M * D, D, 0.02),
                                ("proj_out", D, (M + 1) * D, 0.02)):
            sd[p + name + ".weight"] = (torch.randn(n, k, generator=g) * std).bfloat16()
            sd[p + name + ".bias"] = (torch.randn(n, generator=g) * 0.02).bfloat16()
        sd[p + "attn.norm_q.weight"] = torch.ones(self.DH).bfloat16()
        sd[p + "attn.norm_k.weight"] = torch.ones(self.DH).bfloat16()
        for name in ("attn.to_qkv_input_scale", "proj_mlp_input_scale", "proj_out_input_scale"):
            sd[p + name] = torch.tensor([0.03])
        return p, sd

    def _inputs(self, g, rows):
        x = torch.randn(1, rows, self.D, generator=g).bfloat16()
        temb = torch.nn.functional.silu(torch.randn(1, self.D, generator=g)).bfloat16()
        ang = torch.rand(1, rows, self.DH // 2, generator=g) * 6.28
        rope = torch.stack([torch.cos(ang), -torch.sin(ang), torch.sin(ang), torch.cos(ang)], dim=-1).reshape(
            1, rows, self.DH // 2, 2, 2).bfloat16()
        return x, temb, rope

    use_mirror = False  # bench.py --python-mirror

    def _namespace(self):
        """The classes the step runs through: the C++ torch custom classes, or their Python mirrors."""
        if self.use_mirror:
            from lyradiff_b200 import flux_blocks, flux_model
            return flux_blocks, flux_model
        from lyradiff_b200 import torch_classes
        ns = torch_classes.load()
        return ns, ns

    def setup_gpu(self, dev):
        blocks_ns, _ = self._namespace()
        g = _gen()
        prefix, sd = self._state_dict(g, on_gpu=True)
        self.op = blocks_ns.FluxSingleTransformerBlockOp("bf16", self.D, self.H, self.DH, self.MLP, getattr(self, "quant_level", 1))
        self.op.initialize(blocks_ns.LyraDiffCommonContext())
        self.op.reload_model_from_state_dict(prefix, sd, "cpu")
        x, temb, rope = self._inputs(g, self.tokens)
        self.x, self.temb, self.rope = x.to(dev), temb.to(dev), rope.to(dev)
        self.y = torch.empty_like(self.x)
        self.h_in = x.pin_memory()
        self.e2e_x = [torch.empty_like(self.x), torch.empty_like(self.x)]   # the two device slots a step's input arrives in
        self.e2e_y = [self.y, torch.empty_like(self.y)]

    use_graph = True  # bench.py --no-graph turns the CUDA-graph replay off

    def _forward(self, x):
        return self.op.forward(x, self.rope, self.temb)

    def _capture(self):
        """One step on the resident input as a CUDA graph: the step is hundreds of short launches issued from Python,
        and replaying them as a graph takes the launch gaps out (the library's entry points allocate nothing and
        only enqueue, so they can be captured as they are)."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._forward(self.x)
        torch.cuda.current_stream().wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.graph_out = self._forward(self.x)

    def step(self, events=None, io=None):
        if events is not None:
            events[0][0].record()
        if self.use_graph:
            # The captured step reads self.x and leaves its result in self.graph_out.  End to end (io given) the step's
            # input slot is copied into self.x and the result out of self.graph_out on the step's own stream, so the graph
            # (hundreds of launches issued without host work in between) serves both timed regions.
            if getattr(self, "graph", None) is None:
                self._capture()
            if io is not None:
                self.x.copy_(io[0], non_blocking=True)
            self.graph.replay()
            if io is not None:
                io[1].copy_(self.graph_out, non_blocking=True)
        else:
            out = self._forward(self.x if io is None else io[0])
            if io is not None:
                io[1].copy_(out)
        if events is not None:
            events[0][1].record()

    def peak(self, peaks, mode):
        p16, _ = tensor_peak(peaks, mode, 1, "")
        blend = self.work_per_step / (self.lin_flops / (2.0 * p16) + self.attn_flops / p16)
        nominal = self.work_per_step / (self.lin_flops / 4500.0 + self.attn_flops / 2250.0)
        name = "bf16_tflops" if mode == "burst" else "bf16_tflops_sustained"
        return blend, ("FLOP-weighted blend of 2 x %s (FP8 linears) and %s (attention) of MEASURED_PEAKS.json (%s, %s denominator)"
                       % (name, name, peaks["source"], mode)), nominal

    def setup_cpu(self, rows):
        g = _gen()
        self.cpu_prefix, self.cpu_sd = self._state_dict(g)
        self.cpu_in = self._inputs(g, rows)
        self.cpu_rows = rows
        self.cpu_cache = {}
        self.step_cpu()  # quantizes the weights once, as loading the block does

    def cpu_work(self, rows):
        return 2.0 * rows * self.D * (3 * self.D + self.MLP * self.D + (self.MLP + 1) * self.D) + 4.0 * rows * rows * self.D

    def step_cpu(self):
        from oracle import blocks
        x, temb, rope = self.cpu_in
        return blocks.flux_single_block(x, rope, temb, self.cpu_sd, self.cpu_prefix, self.H, self.DH, self.MLP, 1, cache=self.cpu_cache)[0]

    cpu_note = "oracle block with weights quantized once: fp64 contractions of the e4m3 operands and exact attention over the sample's own rows"


class FluxBlockInt4(FluxBlock):
    """The same single-stream block at quant_level 7 (INT4_W4A4): every linear a W4A4 group-64 linear with its rank-32
    LoRA branch (int4 quantize + LoRA-down, grouped GEMM + LoRA-up + epilogue), proj_out as the reference's two linears."""
    name = "flux_block_int4"
    metric = "flux_single_block_int4_throughput"
    dtype = "int4 W4A4 linears (s32 per group of 64 in TMEM, f32 across groups) + bf16 library attention"

    def __init__(self, tokens):
        super().__init__(tokens)
        self.workload = self.workload.replace("FP8_W8A8", "INT4_W4A4 (rank-32 LoRA branches)").replace("in FP8 linears", "in W4A4 linears")
        self.launches_per_step = 16
        self.roof["kernel"] = ("whole block: 4 x (int4 quantize, LoRA-down, gemm_w4a4_kernel) + AdaLN, QK-norm/RoPE, attention and gate "
                               "kernels of this library, plus one small library matmul")

    def _state_dict(self, g, on_gpu=False):
        D, M = self.D, self.MLP
        p = "single_transformer_blocks.0."
        sd = {p + "norm.linear.weight": (torch.randn(3 * D, D, generator=g) * 0.02).bfloat16(),
              p + "norm.linear.bias": (torch.randn(3 * D, generator=g) * 0.02).bfloat16(),
              p + "attn.norm_q.weight": torch.ones(self.DH).bfloat16(), p + "attn.norm_k.weight": torch.ones(self.DH).bfloat16()}
        for name, n, k, bias in (("attn.to_qkv.", 3 * D, D, True), ("proj_mlp.", M * D, D, True), ("proj_out.linears.0.", D, D, True),
                                 ("proj_out.linears.1.linear.", D, M * D, False)):
            w = (torch.randn(n, k, generator=g) * 0.02).bfloat16()
            if on_gpu:   # the product packs its own weights (lyraq_weight_quant_int4_g64)
                from lyradiff_b200 import ops
                pw = torch.empty(n, k // 2, dtype=torch.uint8, device="cuda")
                sw = torch.empty(n, k // 64, dtype=torch.float32, device="cuda")
                ops.weight_quant_int4_g64(pw, sw, w.cuda())
                pw, sw = pw.cpu(), sw.cpu()
            else:        # CPU baseline: the oracle's restatement of the same rule
                from oracle import quant
                pw, sw, _ = quant.int4_weight_quant_g64(w)
            sd[p + name + "packed_weight"], sd[p + name + "weight_scale"] = pw, sw
            sd[p + name + "smooth"] = 0.5 + torch.rand(k, generator=g)
            sd[p + name + "lora_down"] = (torch.randn(32, k, generator=g) * 0.02).bfloat16()
            sd[p + name + "lora_up"] = (torch.randn(n, 32, generator=g) * 0.02).bfloat16()
            if bias:
                sd[p + name + "bias"] = (torch.randn(n, generator=g) * 0.02).bfloat16()
        return p, sd

    quant_level = 7

    def step_cpu(self):
        from oracle import blocks
        x, temb, rope = self.cpu_in
        return blocks.flux_single_block_int4(x, rope, temb, self.cpu_sd, self.cpu_prefix, self.H, self.DH, self.MLP, 7)[0]

    cpu_note = "oracle INT4 block: exact int32 group sums with fp32 rescale in group order, fp64 LoRA sums, exact attention over the sample's own rows"


class FluxForward(FluxBlock):
    """configs[4]: the whole FLUX.1-dev transformer through torch.classes.lyradiff.FluxTransformer2DModelOp -- embedders,
    19 double-stream + 38 single-stream blocks (each with its own random FP8 weights), norm_out and proj_out -- one image
    (4096 image + 512 text tokens) per GPU."""
    name = "flux_forward"
    metric = "flux_transformer_forward_throughput"
    N_DOUBLE, N_SINGLE, TXT, IN_CH, JOINT, POOLED = 19, 38, 512, 64, 4096, 768

    def __init__(self, tokens):
        FluxBlock.__init__(self, tokens)
        self.blocks = self.N_DOUBLE + self.N_SINGLE
        S, D = self.tokens - self.TXT, self.D
        outer = 2.0 * D * (S * self.IN_CH * 2 + self.TXT * self.JOINT)   # x_embedder, proj_out, context_embedder (16-bit, library)
        self.lin_flops *= self.blocks
        self.attn_flops *= self.blocks
        self.work_per_step = self.lin_flops + self.attn_flops + outer
        self.workload = ("configs[4]: FLUX.1-dev transformer forward, embedders + %d double-stream + %d single-stream blocks + "
                         "norm_out / proj_out, FP8_W8A8, random weights (each block its own), 1 image per GPU = %d image + %d text "
                         "tokens, hidden 3072, 24 x 128 heads; one step = one forward = one denoising step = %.1f TFLOP"
                         % (self.N_DOUBLE, self.N_SINGLE, S, self.TXT, self.work_per_step / 1e12))
        self.launches_per_step = self.N_DOUBLE * 15 + self.N_SINGLE * 6 + 1
        self.timed_names = ["transformer_forward"]
        self.timed_work = [self.work_per_step]
        self.roof["kernel"] = "whole model: 57 blocks, each 3 or 8 gemm_tcgen05_kernel<f8f6f4> launches + attention_fwd_kernel + " \
                              "element-wise kernels of this library, plus the small 16-bit modulation matmuls, embedders and output layer"

    def setup_gpu(self, dev):
        blocks_ns, model_ns = self._namespace()
        D, M, DH = self.D, self.MLP, self.DH
        g = torch.Generator(device=dev).manual_seed(0)
        sd = {}

        def lin(name, n, k, scale=0.03, quantized=True):
            sd[name + ".weight"] = (torch.randn(n, k, generator=g, device=dev, dtype=torch.float32) * 0.02).bfloat16()
            sd[name + ".bias"] = (torch.randn(n, generator=g, device=dev, dtype=torch.float32) * 0.02).bfloat16()
            if quantized:
                sd[name + "_input_scale"] = torch.tensor([scale])

        for i in range(self.N_DOUBLE):
            p = "transformer_blocks.%d." % i
            for norm in ("norm1", "norm1_context"):
                lin(p + norm + ".linear", 6 * D, D, quantized=False)
            for a, b in (("attn.to_qkv", "attn.to_out.0"), ("attn.to_added_qkv", "attn.to_add_out")):
                lin(p + a, 3 * D, D)
                lin(p + b, D, D)
            for ff in ("ff", "ff_context"):
                lin(p + ff + ".net.0.proj", 4 * D, D)
                lin(p + ff + ".net.2", D, 4 * D)
            for n in ("attn.norm_q.weight", "attn.norm_k.weight", "attn.norm_added_q.weight", "attn.norm_added_k.weight"):
                sd[p + n] = torch.ones(DH, device=dev).bfloat16()
        for i in range(self.N_SINGLE):
            p = "single_transformer_blocks.%d." % i
            lin(p + "norm.linear", 3 * D, D, quantized=False)
            lin(p + "attn.to_qkv", 3 * D, D)
            lin(p + "proj_mlp", M * D, D)
            lin(p + "proj_out", D, (M + 1) * D)
            sd[p + "attn.norm_q.weight"] = torch.ones(DH, device=dev).bfloat16()
            sd[p + "attn.norm_k.weight"] = torch.ones(DH, device=dev).bfloat16()
        lin("x_embedder", D, self.IN_CH, quantized=False)
        lin("context_embedder", D, self.JOINT, quantized=False)
        lin("proj_out", self.IN_CH, D, quantized=False)
        lin("norm_out.linear", 2 * D, D, quantized=False)
        for name, d_in in (("timestep_embedder", 256), ("guidance_embedder", 256), ("text_embedder", self.POOLED)):
            lin("time_text_embed.%s.linear_1" % name, D, d_in, quantized=False)
            lin("time_text_embed.%s.linear_2" % name, D, D, quantized=False)
        self.op = model_ns.FluxTransformer2DModelOp("bf16", self.IN_CH, self.N_DOUBLE, self.N_SINGLE, DH, self.H, self.POOLED,
                                                    self.JOINT, True, 1)
        self.op.initialize(blocks_ns.LyraDiffCommonContext())
        self.op.reload_transformer_model_from_state_dict(sd, "cuda")
        del sd
        cg = _gen()
        S = self.tokens - self.TXT
        from lyradiff_b200 import rope as rope_host
        side = int(round(S ** 0.5))
        if side * side == S:   # the table FLUX builds from its position ids: text rows (0,0,0), image rows (0, y, x)
            rope = rope_host.flux_rope_table(rope_host.flux_position_ids(self.TXT, side, side))[:, 0].bfloat16()
        else:
            _, _, rope = self._inputs(cg, self.tokens)
        img = torch.randn(1, S, self.IN_CH, generator=cg).bfloat16()
        self.txt = torch.randn(1, self.TXT, self.JOINT, generator=cg).bfloat16().to(dev)
        self.pooled = torch.randn(1, self.POOLED, generator=cg).bfloat16().to(dev)
        self.x, self.rope = img.to(dev), rope.to(dev)
        self.y = torch.empty(1, S, self.IN_CH, dtype=torch.bfloat16, device=dev)
        self.h_in = img.pin_memory()
        self.e2e_x = [torch.empty_like(self.x), torch.empty_like(self.x)]   # the two device slots a step's input arrives in
        self.e2e_y = [self.y, torch.empty_like(self.y)]

    def _forward(self, img):
        return self.op.transformer_forward(img, self.txt, self.rope, self.pooled, 500.0, 3500.0)

    def verify(self):
        """Before anything is timed: the full 19 + 38-block forward gives a finite result of sane amplitude, and the same
        bits twice (every sum inside has a fixed order).  The per-block parity against the oracle is what tests/ checks."""
        a = self._forward(self.x).float()
        b = self._forward(self.x).float()
        torch.cuda.synchronize()
        if not bool(torch.isfinite(a).all()):
            raise SystemExit("bench.py: the forward's output is not finite")
        if not torch.equal(a, b):
            raise SystemExit("bench.py: two forwards of the same input differ")
        amp = float(a.abs().mean())
        if not (1e-4 < amp < 1e4):
            raise SystemExit("bench.py: output amplitude %g out of range" % amp)
        return "output finite, mean |y| = %.4g, identical bits on a second forward" % amp

    def setup_cpu(self, rows):
        # the CPU baseline of this case is the single-stream block of the stack on a row sample (its work is counted per block)
        FluxBlock.setup_cpu(self, rows)

    def cpu_work(self, rows):
        return FluxBlock.cpu_work(self, rows)


class W4A4:
    """configs[2]: FLUX fused W4A4 linear."""
    name = "w4a4"
    metric = "w4a4_g64_linear_throughput"
    unit = "TOP/s"
    dtype = "s4 expanded to s8 (s32 per group in TMEM, fp32 across groups)"
    K, N = 3072, 21504

    def __init__(self, tokens):
        self.tokens = tokens or 4608
        self.work_per_step = 2.0 * self.tokens * self.K * self.N
        self.scale = 1e12
        self.workload = ("configs[2]: W4A4 group-64 linear M=%d K=3072 N=21504: int4 per-(token, group) quantize of bf16 X + "
                         "grouped GEMM with fp16 weight group scales -> bf16" % self.tokens)
        self.launches_per_step = 2
        self.timed_names = ["w4a4_gemm"]
        self.timed_work = [self.work_per_step]
        self.roof = {"bound": "tensor", "unit": "TOP/s", "kernel": "gemm_w4a4_kernel (1 launch per step)"}
        # profiles/gemm_w4a4_flux_fused.md: small-case capture scaled by the tiles processed
        self.traffic = 240.0e6 if self.tokens == 4608 else None

    def setup_gpu(self, dev):
        from lyradiff_b200 import ops
        self.ops = ops
        g = _gen()
        T, K, N = self.tokens, self.K, self.N
        self.x = torch.randn(T, K, generator=g).bfloat16().to(dev)
        w = (torch.randn(N, K, generator=g) * 0.02).bfloat16().to(dev)
        self.qw = torch.empty(N, K // 2, dtype=torch.uint8, device=dev)
        self.sw = torch.empty(N, K // 64, dtype=torch.float16, device=dev)
        ops.weight_quant_int4_g64(self.qw, self.sw, w)
        del w
        self.smooth = torch.ones(K, dtype=torch.float32, device=dev)
        self.q = torch.empty(T, K // 2, dtype=torch.uint8, device=dev)
        self.s = torch.empty(T, K // 64, dtype=torch.float32, device=dev)
        self.y = torch.empty(T, N, dtype=torch.bfloat16, device=dev)
        self.h_in = self.x.cpu().pin_memory()
        self.e2e_x = [self.x, torch.empty_like(self.x)]
        self.e2e_y = [self.y, torch.empty_like(self.y)]

    def step(self, events=None, io=None):
        ops = self.ops
        x = self.x if io is None else io[0]
        y = self.y if io is None else io[1]
        ops.invoke_fused_quantize_and_lora_down_simple(None, self.q, self.s, x, None, self.smooth)
        if events is not None:
            events[0][0].record()
        ops.invoke_fused_w4a4_gemm_and_lora_up(y, self.q, self.qw, None, None, self.s, self.sw)
        if events is not None:
            events[0][1].record()

    def peak(self, peaks, mode):
        v, src = tensor_peak(peaks, mode, 2, " as the dense INT8 rate; the kernel is bound by the per-group fp32 rescale on the CUDA "
                             "cores, not by the tensor pipe")
        return v, src, 4500.0

    def setup_cpu(self, rows):
        from oracle import quant as oq
        g = _gen()
        self.cpu = {"x": torch.randn(rows, self.K, generator=g).bfloat16()}
        w = (torch.randn(self.N, self.K, generator=g) * 0.02).bfloat16()
        _, sw, qw = oq.int4_weight_quant_g64(w)
        self.cpu["qw"], self.cpu["sw"] = qw, sw.half()
        self.cpu_rows = rows

    def step_cpu(self):
        from oracle import gemm as og
        from oracle import quant as oq
        _, sa, qa = oq.int4_quant_g64(self.cpu["x"], None)
        return og.w4a4_gemm(qa, self.cpu["qw"], sa, self.cpu["sw"], fma=False)

    cpu_note = "int4 group-64 quantize + per-group exact contraction + fp32 rescale"


class AdalnQuant:
    """configs[3]: fused AdaLN-modulation + quantize."""
    name = "adaln_quant"
    metric = "adaln_quant_bandwidth"
    unit = "GB/s"
    dtype = "bf16 in, fp32 statistics, int8 + f8e4m3 out"
    D = 3072

    def __init__(self, tokens):
        self.tokens = tokens or 4608
        T, D = self.tokens, self.D
        # read X, write int8 + per-token scales + e4m3 (scale/shift rows are negligible and L2-resident)
        self.work_per_step = 2.0 * T * D + T * D + 4.0 * T + T * D + 2 * 2.0 * D
        self.scale = 1e9
        self.workload = ("configs[3]: fused AdaLN-modulation + quantize, X bf16 [%d, 3072], LayerNorm eps 1e-6 no affine, "
                         "y = LN(x)(1+scale)+shift; emits int8 with per-token scales and e4m3 with a per-tensor scale in one "
                         "pass" % T)
        self.launches_per_step = 1
        self.timed_names = ["adaln_quant"]
        self.timed_work = [self.work_per_step]
        self.roof = {"bound": "hbm", "unit": "GB/s", "kernel": "adaln3072_e4m3_kernel<bf16, int8 + e4m3 out> (1 launch per step)"}
        self.traffic = 28.6e6 if T == 4608 else None  # profiles/adaln3072_4608x3072.md (outputs absorbed by L2)

    def setup_gpu(self, dev):
        from lyradiff_b200 import ops
        self.ops = ops
        g = _gen()
        T, D = self.tokens, self.D
        # several independent input/output sets (> 126 MB L2 in total) are rotated so that no step finds its data in L2
        self.nset = 4
        self.x = [torch.randn(1, T, D, generator=g).bfloat16().to(dev) for _ in range(self.nset)]
        self.sc = (torch.randn(1, D, generator=g) * 0.1).bfloat16().to(dev)
        self.sh = (torch.randn(1, D, generator=g) * 0.1).bfloat16().to(dev)
        self.q8 = [torch.empty(T, D, dtype=torch.int8, device=dev) for _ in range(self.nset)]
        self.s8 = torch.empty(T, dtype=torch.float32, device=dev)
        self.qf8 = [torch.empty(T, D, dtype=torch.uint8, device=dev) for _ in range(self.nset)]
        self.f8s = torch.tensor([8.0 / 448.0], dtype=torch.float32, device=dev)
        self.h_in = self.x[0].cpu().pin_memory()
        self.e2e_x = [self.x[0], self.x[1]]
        self.e2e_y = [self.q8[0], self.q8[1]]
        self.i = 0

    def step(self, events=None, io=None):
        i = self.i = (self.i + 1) % self.nset
        x = self.x[i] if io is None else io[0]
        q8 = self.q8[i] if io is None else io[1]
        if events is not None:
            events[0][0].record()
        self.ops.invoke_layer_norm_with_shift_and_scale(None, x, self.sc, self.sh, 1e-6, q8=q8, q8_scale=self.s8,
                                                        qf8=self.qf8[i], f8_scale=self.f8s)
        if events is not None:
            events[0][1].record()

    def peak(self, peaks, mode):
        return peaks["hbm_gbs"], "hbm_gbs of MEASURED_PEAKS.json (%s)" % peaks["source"], 7700.0

    def setup_cpu(self, rows):
        g = _gen()
        self.cpu = {"x": torch.randn(1, rows, self.D, generator=g).bfloat16(), "sc": (torch.randn(1, self.D, generator=g) * 0.1).bfloat16(),
                    "sh": (torch.randn(1, self.D, generator=g) * 0.1).bfloat16(), "f8": torch.tensor([8.0 / 448.0])}
        self.cpu_rows = rows

    def step_cpu(self):
        from oracle import norms
        c = self.cpu
        return norms.adaln_quant(c["x"], c["sc"], c["sh"], fp8_scale=c["f8"])

    cpu_note = "LayerNorm + modulation + int8 and e4m3 quantize"


class Attention:
    """The attention of one FLUX block (the 20 % of configs[4]'s FLOPs outside the linears): 4608 tokens, 24 heads x 128,
    bf16, packed QKV in, e4m3 out into the proj_out input window."""
    name = "attention"
    metric = "flux_attention_throughput"
    unit = "TFLOP/s"
    dtype = "bf16 (f32 scores and accumulation in TMEM, bf16 probabilities), e4m3 out"
    H, DH = 24, 128

    def __init__(self, tokens):
        self.tokens = tokens or 4608
        T = self.tokens
        self.work_per_step = 4.0 * T * T * self.H * self.DH
        self.scale = 1e12
        self.workload = ("attention of one FLUX.1-dev block: softmax(q k^T / sqrt(128)) v over %d tokens, 24 heads x 128, packed bf16 "
                         "QKV [%d, 9216] in, e4m3 [%d, 3072] out (per-tensor scale)" % (T, T, T))
        self.launches_per_step = 1
        self.timed_names = ["attention"]
        self.timed_work = [self.work_per_step]
        self.roof = {"bound": "tensor", "unit": "TFLOP/s", "kernel": "attention_fwd_kernel<bf16> (1 launch per step)"}
        self.traffic = 90.3e6 if self.tokens == 4608 else None   # profiles/attention_fwd_4608x24x128.md

    def setup_gpu(self, dev):
        from lyradiff_b200 import ops
        self.ops = ops
        g = _gen()
        T, W = self.tokens, self.H * self.DH
        # three input sets (85 MB each) rotate so that no step finds its q / k / v in L2 from the step before
        self.qkv = [torch.randn(T, 3 * W, generator=g).bfloat16().to(dev) for _ in range(3)]
        self.out = [torch.empty(T, W, dtype=torch.uint8, device=dev) for _ in range(2)]
        self.s = torch.tensor([0.02], dtype=torch.float32, device=dev)
        self.h_in = self.qkv[0].cpu().pin_memory()
        self.e2e_x = [self.qkv[0], self.qkv[1]]
        self.e2e_y = self.out
        self.i = 0

    def step(self, events=None, io=None):
        self.i = (self.i + 1) % 3
        qkv = self.qkv[self.i] if io is None else io[0]
        out = self.out[0] if io is None else io[1]
        if events is not None:
            events[0][0].record()
        self.ops.flash_attention(qkv, 1, self.tokens, self.H, self.DH, out=out, out_scale=self.s)
        if events is not None:
            events[0][1].record()

    def peak(self, peaks, mode):
        v, src = tensor_peak(peaks, mode, 1, "")
        return v, src, 2250.0

    def setup_cpu(self, rows):
        g = _gen()
        self.cpu = torch.randn(rows, 3, self.H, self.DH, generator=g).bfloat16()
        self.cpu_rows = rows

    def cpu_work(self, rows):
        return 4.0 * rows * rows * self.H * self.DH

    def step_cpu(self):
        from oracle import blocks
        x = self.cpu.permute(1, 2, 0, 3).unsqueeze(1)     # [3, 1, H, rows, Dh]
        return blocks.attention(x[0], x[1], x[2])

    cpu_note = "exact fp64 softmax attention over the sample's own rows"


CASES = {c.name: c for c in (FluxFp8, FluxBlock, FluxBlockInt4, FluxForward, Int8Sdxl, SdxlFF, W4A4, AdalnQuant, Attention)}


# =================================================================================================== CPU arm
CPU_ROWS = 256  # token rows of the bounded CPU sample, the same in the GPU arm's cpu_baseline and in --impl reference


def time_cpu(case, rows, steps, warmup):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    case.setup_cpu(rows)
    for _ in range(warmup):
        case.step_cpu()
    t0 = time.perf_counter()
    for _ in range(steps):
        case.step_cpu()
    dt = (time.perf_counter() - t0) / steps
    work = case.cpu_work(rows) if hasattr(case, "cpu_work") else case.work_per_step * rows / case.tokens
    return {"value": work / dt / case.scale, "unit": case.unit, "cores": cores, "kind": "port",
            "sample": "%d of %d token rows per step (%s), torch on %d threads, %d timed steps" % (
                rows, case.tokens, case.cpu_note, cores, steps),
            "ms_per_step_sample": dt * 1e3, "sample_work": work}


def run_reference(case, args, rank, world):
    """The reference arm: the CPU restatement of the reference's arithmetic for this path (the reference's own CUDA sources
    cannot be built or run on host cores), all host threads, K timed steps of a bounded row sample.  ms_per_step is the
    time of one sample step as measured; the figure scaled to the full row count sits in its own key."""
    if rank != 0:
        return
    rows = min(case.tokens, CPU_ROWS)
    base = time_cpu(case, rows, max(1, args.steps), max(1, min(args.warmup, 3)))
    line = {
        "impl": "reference", "metric": case.metric, "value": base["value"], "unit": case.unit, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step_sample"],
        "ms_per_step_scaled_to_all_rows": base["ms_per_step_sample"] * case.work_per_step / base["sample_work"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": case.dtype + " restated on CPU",
        "data": "synthetic",
        "config": {"workload": case.workload, "parallelism": "replicas x%d: one copy of the workload per GPU, no collective" % world,
                   "l2": "not applicable (host cores)"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": case.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


# =================================================================================================== GPU arm
def time_events(fn, steps):
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def measure_resident(case, steps, warmup, barrier, sampler=None):
    """Device-timed part of one case: a pass with an event pair around the dominant kernels (the roofline's per-launch
    durations) and, directly after it, `steps` steps with no event inside (the value).  Returns (ms per step, per-kernel ms)."""
    for _ in range(warmup):
        case.step()
    nt = len(case.timed_names)
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(nt)] for _ in range(steps)]
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    if sampler is not None:
        sampler.start()
    # An event between two kernels takes away the overlap of one kernel's set-up with its predecessor's tail that
    # dependent launch gives, so the per-kernel durations come from a pass of their own.
    for s in range(steps):
        case.step(ev[s])
    t_begin.record()
    for s in range(steps):
        case.step()
    t_end.record()
    barrier()
    timed_ms = [sum(ev[s][i][0].elapsed_time(ev[s][i][1]) for s in range(steps)) / steps for i in range(nt)]
    return t_begin.elapsed_time(t_end) / steps, timed_ms


def roofline_block(case, peaks, timed_ms, mode):
    rscale = getattr(case, "roof_scale", case.scale)
    achieved = sum(case.timed_work) / (sum(timed_ms) * 1e-3) / rscale
    peak, peak_source, nominal = case.peak(peaks, mode)
    roof = dict(case.roof)
    roof.update({"achieved": achieved, "peak": peak, "frac": achieved / peak, "traffic": getattr(case, "traffic", None),
                 "traffic_unit": "bytes of DRAM read + write per launch, from the ncu capture summarised under profiles/",
                 "peak_source": peak_source, "frac_of_nominal": achieved / nominal, "nominal": nominal,
                 "per_launch_ms": dict(zip(case.timed_names, timed_ms)),
                 "per_launch_achieved": dict(zip(case.timed_names, [w / (t * 1e-3) / rscale for w, t in zip(case.timed_work, timed_ms)]))})
    return roof


def sub_record(name, dev, peaks, steps):
    """One of the other configurations, timed alone with inputs resident (a burst at flat clocks): metric, ms, achieved,
    fraction of the measured peak, traffic."""
    case = CASES[name](0)
    case.setup_gpu(dev)
    ms_step, timed_ms = measure_resident(case, steps, 5, lambda: torch.cuda.synchronize())
    roof = roofline_block(case, peaks, timed_ms, "burst")
    rec = {"metric": case.metric, "value": case.work_per_step / (ms_step * 1e-3) / case.scale, "unit": case.unit,
           "ms_per_step": ms_step, "steps": steps, "workload": case.workload, "gpu_launches_per_step": case.launches_per_step,
           "roofline": {k: roof[k] for k in ("bound", "unit", "kernel", "achieved", "peak", "frac", "peak_source", "traffic",
                                             "per_launch_ms", "per_launch_achieved")}}
    del case
    torch.cuda.empty_cache()
    return rec


def library_baseline(dev, steps):
    """cuBLASLt FP8 (torch._scaled_mm) on the four FLUX linear shapes -- the reference's FP8 linear IS that library call
    (src/lyradiff/utils/cublasMMWrapper.cc:1251) -- and the library attention (torch SDPA) on the block's shape, timed in
    this run beside this library's kernels.  Measurement only: nothing in the product path calls them."""
    out = {"note": "library kernels timed beside this library's (cuBLASLt FP8 through torch._scaled_mm; cuDNN / flash attention "
                   "through torch SDPA); not on the product path", "steps": steps}
    T = 4608
    one = torch.ones((), dtype=torch.float32, device=dev)
    try:
        for name, k, n, _, _ in FluxFp8.LINEARS:
            a = torch.randn(T, k, device=dev).to(torch.float8_e4m3fn)
            b = torch.randn(n, k, device=dev).to(torch.float8_e4m3fn)
            fn = lambda: torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            for _ in range(5):
                fn()
            ms = time_events(fn, steps)
            out[name] = {"ms": ms, "tflops": 2.0 * T * k * n / (ms * 1e-3) / 1e12}
    except Exception as e:  # an unavailable library call must not cost the bench line
        out["fp8_error"] = repr(e)[:200]
    try:
        qkv = torch.randn(1, T, 3, 24, 128, device=dev).bfloat16()
        q, k_, v = (qkv.select(2, i).transpose(1, 2) for i in range(3))
        fn = lambda: torch.nn.functional.scaled_dot_product_attention(q, k_, v)
        for _ in range(5):
            fn()
        ms = time_events(fn, steps)
        out["attention"] = {"ms": ms, "tflops": 4.0 * T * T * 3072 / (ms * 1e-3) / 1e12}
    except Exception as e:
        out["attention_error"] = repr(e)[:200]
    return out


def run_ours(case, args, rank, world, local_rank):
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the GPU arm has no CPU fallback")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    from lyradiff_b200 import ops, replicas
    replicas.init("nccl", dev)  # only lines the ranks up for timing; no collective touches the data path

    def barrier():
        replicas.barrier(dev)

    def check_device():
        status, detail = ops.last_status()
        if status != 0:
            raise SystemExit("bench.py: device status %d (detail 0x%x)" % (status, detail))

    if args.no_dependent_launch:
        from lyradiff_b200 import _lib as _l
        _l.check(_l.lib().lyraq_debug_set_dependent_launch(0), "lyraq_debug_set_dependent_launch")
    if args.tile:
        from lyradiff_b200 import _lib
        _lib.check(_lib.lib().lyraq_debug_force_gemm_tile(args.tile), "lyraq_debug_force_gemm_tile")
    case.setup_gpu(dev)
    peaks = load_peaks()
    warmup = max(args.warmup, 3)
    checked = case.verify() if hasattr(case, "verify") else None
    check_device()

    # ---- timed region 1: kernels only, inputs resident
    sampler = ClockSampler(local_rank)
    ms_step, timed_ms = measure_resident(case, args.steps, warmup, barrier, sampler)
    clocks = sampler.result()
    ms_total = ms_step * args.steps
    check_device()

    # ---- timed region 2: end to end from pinned host buffers.  Every step copies its activations host -> device,
    # runs, and copies its result device -> host; the three stages of neighbouring steps overlap on three streams
    # (two device slots for the input and for the result), as a serving loop would run them.
    h_out = [torch.empty(case.e2e_y[0].shape, dtype=case.e2e_y[0].dtype).pin_memory() for _ in range(2)]
    s_in, s_run, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_run = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_steps(count):
        for i in range(count):
            b = i & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_run[b])          # the step that last read this input slot has finished
                case.e2e_x[b].copy_(case.h_in.view(case.e2e_x[b].shape), non_blocking=True)
                ev_in[b].record(s_in)
            with torch.cuda.stream(s_run):
                s_run.wait_event(ev_in[b])
                s_run.wait_event(ev_out[b])         # the result slot has been copied out
                case.step(io=(case.e2e_x[b], case.e2e_y[b]))
                ev_run[b].record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_run[b])
                h_out[b].copy_(case.e2e_y[b], non_blocking=True)
                ev_out[b].record(s_out)

    barrier()
    e2e_steps(4)
    barrier()
    e_begin, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_begin.record(s_in)
    e2e_steps(args.steps)
    s_out.wait_stream(s_run)
    s_out.wait_stream(s_in)
    e_end.record(s_out)
    barrier()
    ms_e2e = e_begin.elapsed_time(e_end)
    check_device()

    ms_total, ms_e2e = replicas.max_over_ranks([ms_total, ms_e2e], dev)

    if rank == 0:
        ms_step = ms_total / args.steps
        value = world * case.work_per_step / (ms_step * 1e-3) / case.scale
        e2e_value = world * case.work_per_step / (ms_e2e / args.steps * 1e-3) / case.scale
        # a region of half a second or more runs under the power cap: sustained peak; shorter ones are bursts at flat clocks
        mode = "sustained" if ms_total >= 500.0 else "burst"
        roof = roofline_block(case, peaks, timed_ms, mode)
        roof["timed_region_ms"] = ms_total
        line = {
            "metric": case.metric, "value": value, "unit": case.unit, "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": case.dtype,
            "data": "synthetic",
            "config": {"workload": case.workload, "parallelism": "replicas x%d: one copy of the workload per GPU, no collective" % world,
                       "l2": "no explicit flush: every step streams distinct tensors larger than the 126 MB L2 between reuses"},
            "e2e": {"value": e2e_value, "unit": case.unit, "h2d_bytes_per_step": case.h_in.numel() * case.h_in.element_size(),
                    "d2h_bytes_per_step": h_out[0].numel() * h_out[0].element_size(), "ms_per_step": ms_e2e / args.steps,
                    "overlap": "H2D, compute and D2H of neighbouring steps overlap on three streams (double-buffered slots)"},
            "gpu_launches": args.steps * case.launches_per_step,
            "clocks": clocks,
        }
        if checked is not None:
            line["config"]["checked_before_timing"] = checked
        if world == 1 and not args.no_subrecords and case.name == DEFAULT_CASE:
            # the other configurations and the library kernels, each timed alone after the headline (rank 0, N = 1 only)
            del case.op
            torch.cuda.empty_cache()
            subs = {}
            for name in ("flux_fp8", "int8_sdxl", "sdxl_ff", "w4a4", "adaln_quant", "attention"):
                subs[name] = sub_record(name, dev, peaks, 20)
                check_device()
            line["configs"] = subs
            line["library_baseline"] = library_baseline(dev, 20)
            # the dominant kernel of the forward is the FP8 GEMM (58 % of its device time): its roofline is the one of the
            # four FLUX linear shapes timed alone just above; the whole forward against the blended peak sits beside it
            line["forward_roofline"] = roof
            roof = dict(subs["flux_fp8"]["roofline"])
            roof["note"] = ("per-launch figures of gemm_tcgen05_kernel<f8f6f4> on the forward's four linear shapes, timed alone in "
                            "this run (configs.flux_fp8); the whole forward against the blended peak is in forward_roofline")
        line["roofline"] = roof
        line["cpu_baseline"] = time_cpu(case, min(case.tokens, CPU_ROWS), 3, 1)
        emit(line)
    replicas.shutdown()


DEFAULT_CASE = "flux_forward"


# The process's standard output carries exactly one thing, the JSON line: file descriptor 1 is pointed at standard error for
# the whole run (libraries such as NCCL print their banner to it), and the line goes to the descriptor saved here.
_RESULT_FD = None


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main():
    global _RESULT_FD
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--case", default=DEFAULT_CASE, choices=sorted(CASES))
    ap.add_argument("--tokens", type=int, default=0, help="override the number of token rows (0 = the configuration's own)")
    ap.add_argument("--tile", type=int, default=0, choices=[0, 2561, 1281, 2562],
                    help="force the dense-GEMM tile configuration (0 = automatic; see lyraq_debug_force_gemm_tile)")
    ap.add_argument("--no-graph", action="store_true",
                    help="flux_block / flux_forward: issue every launch from the host instead of replaying the step as a CUDA graph")
    ap.add_argument("--python-mirror", action="store_true",
                    help="flux_block / flux_forward: run the Python mirrors instead of the C++ torch classes (same launches)")
    ap.add_argument("--no-subrecords", action="store_true",
                    help="default case at N = 1: skip the sub-records of the other configurations and the library baseline")
    ap.add_argument("--no-dependent-launch", action="store_true",
                    help="launch the kernels as ordinary stream-ordered kernels (see lyraq_debug_set_dependent_launch)")
    args = ap.parse_args()
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    case = CASES[args.case](args.tokens)
    if args.no_graph:
        case.use_graph = False
    if args.python_mirror:
        case.use_mirror = True
    if args.impl == "reference":
        run_reference(case, args, rank, world)
    else:
        run_ours(case, args, rank, world, local_rank)


if __name__ == "__main__":
    main()
