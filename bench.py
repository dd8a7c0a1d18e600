#!/usr/bin/env python3
"""Benchmark of the QIPACK v6 packed-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--workload block|c4|c3|c5] [--m ROWS]

Workloads (BASELINE.json configs, zero-indexed as the survey reads them):
  block  configs[1], the default and the headline: the four linears of one Qwen-Image MMDiT block image
         stream under W4A4 (H256, g64) at M = 4096 tokens, hidden 3072 - fused q/k/v 3072->9216,
         attention out 3072->3072, MLP fc1 3072->12288, fc2 12288->3072 - each with its own activation
         rotation + quantisation (fp16 in) and fp16 outputs: 927.7 G operations per step.
  c4     configs[3]: the same block at M = 16384 (a 2048 x 2048 image), the shape the sharded scaling
         target is quoted on.
  c3     configs[2]: one denoising step of the 60-block stack under W4A16 g64: per block the four linears on
         the image stream (M = 4096) and on the text stream (M = 256, its own weights) plus the two M = 1
         modulation GEMVs 3072->18432.
  c5     configs[4]: the image-edit shape, rows 2 x (12288 + 512), 60 blocks, each linear W4A4 with
         probability 0.7 and W4A16 otherwise (seeded), through the dispatcher qi_linear.

N > 1 (launched by torch.distributed.run, one rank per GPU): every linear's packed weights are sharded by
output columns, rank r computes y[:, r*N/R:(r+1)*N/R] and the slices are all-gathered over NVLink; total
work is fixed (strong scaling). Every rank quantises all activation rows (--shard-quantiser: its share of
the rows, the codes and scales all-gathered: a quarter of the bytes of an fp16 output, but two more
collectives per linear in front of the GEMM).

Prints ONE JSON line. `value` is device-timed with inputs resident in HBM; `e2e` is the same metric through
the C ABI with host buffers (pinned) copied in and results copied out every step; `roofline` is the W4A4
GEMM kernel's achieved rate from CUDA events around its launches inside the timed region over the dense
8-bit tensor rate measured on this GPU in this run; `cpu_baseline` is the CPU oracle port timed on this
host on a bounded sample.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HIDDEN = 3072
# name, n, k, kind of activation
LINEARS = [("qkv", 9216, 3072, "outliers"), ("attn_out", 3072, 3072, "outliers"),
           ("fc1", 12288, 3072, "outliers"), ("fc2", 3072, 12288, "gelu")]
GEMV_N, GEMV_K = 18432, 3072  # the per-block modulation linear of config 3
METRIC = "packed W4A4/W4A16 GEMM TOPS at M=4096 block shapes, % of tensor/HBM roofline"
UNIT = "TOPS"
CPU_SAMPLE_ROWS = 256
CPU_PASSES = 5
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one w4a4_pair::gemm_kernel launch on the qkv
# shape at M = 4096, whose 2MNK is the average of the block's four launches: from the ncu capture that the
# kernel's profile summary records. Scaled by rows and ranks for other workloads; None for other kernels.
NCU_TRAFFIC_BYTES_QKV_M4096 = 82.7e6


def block_ops(m: int) -> float:
    return sum(2.0 * m * n * k for _, n, k, _ in LINEARS)


def workload_text(m: int) -> str:
    return (f"qwen-image MMDiT block image stream, W4A4 H256 g64, M={m} hidden=3072: qkv 3072->9216, "
            "out 3072->3072, fc1 3072->12288, fc2 12288->3072")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            data = json.load(handle)
        return {"hbm_gbs": data["hbm_gbs"], "bf16_burst": data["bf16_tflops"],
                "bf16_sustained": data["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


# ---- clocks ------------------------------------------------------------------------------------

class ClockSampler:
    """nvidia-smi sampled every 50 ms while the timed regions run."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.process, self.lines = index, None, []

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            time.sleep(0.15)  # the first sample takes a moment
        except OSError:
            self.process = None
        return self

    def _read(self):
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.process is not None:
            time.sleep(0.1)
            self.process.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        clocks, maxima, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                maxima.append(float(parts[2]))
            except ValueError:
                continue
            for name, value in zip(names, parts[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(clocks), "sm_max_mhz": max(maxima), "reasons": sorted(reasons),
                "samples": len(clocks)}


# ---- synthetic data (torch, on the device; not the hot path) ------------------------------------

def hadamard_matrix(torch, device):
    """The 256x256 matrix of the radix-4 butterfly (strides 1, 4, 16, 64): rotation = x @ H.T per chunk."""
    h4 = 0.5 * torch.tensor([[1, 1, 1, -1], [1, 1, -1, 1], [1, -1, 1, 1], [-1, 1, 1, 1]], dtype=torch.float64)
    h = torch.ones(1, 1, dtype=torch.float64)
    for _ in range(4):
        h = torch.kron(h4, h)  # the later pass (larger stride) is the outer factor
    return h.to(device=device, dtype=torch.float32)


def make_packed_w4a4(torch, generator, n, k, device):
    """W ~ N(0, 0.02) rounded to fp16, rotated by H256 per 256-chunk and quantised per 64-group to
    signed 4-bit codes with scale fp16(max|w'|/7) (int4_pack.cplus:322-363 without the clip search,
    which changes values, not timing). Returns codes [n, k/2] uint8, scales [n, k/64] fp16."""
    w = (torch.randn(n, k, generator=generator, device=device) * 0.02).half().float()
    h = hadamard_matrix(torch, device)
    rotated = (w.view(n, k // 256, 256) @ h.t()).view(n, k // 64, 64)
    peak = rotated.abs().amax(dim=-1)
    scale = torch.clamp(peak / 7.0, min=2.0 ** -24).half()
    codes = torch.clamp(torch.round(rotated / scale.float().unsqueeze(-1)), -7, 7).to(torch.int16).view(n, k) & 0xF
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).to(torch.uint8).contiguous()
    return packed, scale.contiguous()


def make_packed_w4a16(torch, generator, n, k, device):
    """Valid scheme-5 records with the value range of packed N(0, 0.02) weights: random codes, scales near
    0.1 / 15, minimums near -8 scales (the timing does not depend on the values)."""
    codes = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=device, generator=generator)
    scales = (torch.rand(n, k // 64, device=device, generator=generator) * 0.006 + 0.002).half()
    return codes, scales, (-8.0 * scales.float()).half()


def make_activations(torch, generator, m, k, kind, device):
    x = torch.randn(m, k, generator=generator, device=device)
    if kind == "outliers":
        channels = torch.randperm(k, generator=generator, device=device)[: max(1, k // 100)]
        x[:, channels] *= 20.0
    elif kind == "gelu":
        x = torch.nn.functional.gelu(x, approximate="tanh")
    elif kind == "silu":
        x = torch.nn.functional.silu(x)
    return x.half().contiguous()


def graph_timed(torch, stream, launch, count):
    """Average device time in ms of `count` launches replayed from one CUDA graph on `stream`: the small
    kernels run for a few microseconds, less than the host needs to issue one launch through ctypes."""
    with torch.cuda.stream(stream):
        for i in range(3):
            assert launch(i) == 0, "a launch was refused"
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(count):
                launch(i)
        graph.replay()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record(stream)
        graph.replay()
        end.record(stream)
        torch.cuda.synchronize()
    return begin.elapsed_time(end) / count


# ---- the path's other kernels, each against its own roofline ---------------------------------------

def other_kernels(qi, torch, device, stream, peaks, tensor_peaks, m):
    """W4A16 GEMM on the block's four shapes (tensor bound), the drop-in W4A4 GEMM on nibble-packed codes,
    the W4A16 M=1 GEMV and the activation quantiser (HBM bound). GEMV weights rotate through more copies
    than fit in L2; the other inputs are larger than L2 by themselves or compute bound."""
    handle = stream.cuda_stream
    generator = torch.Generator(device=device)
    generator.manual_seed(4321)
    out = {"peak_source": peaks["source"]}

    out["w4a16_gemm"] = []
    flops = seconds = 0.0
    for name, n, k, _ in LINEARS:
        codes, scales, minimums = make_packed_w4a16(torch, generator, n, k, device)
        x = torch.randn(m, k, device=device, generator=generator).half()
        y = torch.empty(m, n, dtype=torch.float16, device=device)
        ms = graph_timed(torch, stream, lambda i: qi.w4a16_gemm_ex(x, codes, scales, minimums, None, y, qi.DTYPE_F16, n, m, n, k, handle), 20)
        flops += 2.0 * m * n * k
        seconds += ms * 1e-3
        tflops = 2.0 * m * n * k / ms / 1e9
        out["w4a16_gemm"].append({"linear": name, "ms": ms, "tflops": tflops, "frac_of_fp16_mma_loop": tflops / tensor_peaks["f16"],
                                  "frac_of_bf16_burst": tflops / peaks["bf16_burst"]})
        del codes, scales, minimums, x, y
    achieved = flops / seconds / 1e12
    out["w4a16_gemm_roofline"] = {"bound": "tensor", "achieved": achieved, "peak": tensor_peaks["f16"], "unit": "TFLOP/s",
                                  "frac": achieved / tensor_peaks["f16"], "frac_of_bf16_burst": achieved / peaks["bf16_burst"],
                                  "frac_of_bf16_sustained": achieved / peaks["bf16_sustained"],
                                  "peak_source": tensor_peaks["how"]}

    # The entry points the reference binds, on its operand format (nibble-packed codes). By shape they widen both operands
    # into scratch memory of the stream's pool and run the byte-operand kernel on CTA pairs; the int8 kernel that widens
    # the nibbles in shared memory is timed beside it.
    packed, ops, seconds, int8_seconds = [], 0.0, 0.0, 0.0
    for name, n, k, _ in LINEARS:
        def signed_codes(rows):  # two codes in -7..7 per byte (-8 is not a code of the format)
            values = torch.randint(-7, 8, (rows, k), dtype=torch.int16, device=device, generator=generator) & 0xF
            return (values[:, 0::2] | (values[:, 1::2] << 4)).to(torch.uint8).contiguous()

        w_codes, a_codes = signed_codes(n), signed_codes(m)
        w_scales = (torch.rand(n, k // 64, device=device, generator=generator) * 5e-3 + 1e-3).half()
        a_scales = (torch.rand(m, k // 64, device=device, generator=generator) * 0.5 + 0.05).half()
        y = torch.empty(m, n, dtype=torch.float16, device=device)
        ms = graph_timed(torch, stream, lambda i: qi.w4a4_gemm_ex(a_codes, a_scales, w_codes, w_scales, None, y, qi.DTYPE_F16, n, m, n, k, handle), 10)
        int8_ms = graph_timed(torch, stream, lambda i: qi.w4a4_gemm_path_ex(a_codes, a_scales, w_codes, w_scales, None, y, qi.DTYPE_F16, n, m, n, k,
                                                                             qi.W4A4_PATH_INT8, handle), 10)
        ops += 2.0 * m * n * k
        seconds += ms * 1e-3
        int8_seconds += int8_ms * 1e-3
        packed.append({"linear": name, "ms": ms, "tops": 2.0 * m * n * k / ms / 1e9, "int8_kernel_ms": int8_ms})
        del w_codes, a_codes, w_scales, a_scales, y
    out["w4a4_packed"] = {"kernel": "qi_w4a4_gemm_ex (the drop-in ABI, nibble-packed operands): two widening kernels into (m + n) k bytes of "
                                    "pool scratch, then w4a4_pair::gemm_kernel; int8_kernel: w4a4::gemm_kernel on the nibbles",
                          "linears": packed, "tops": ops / seconds / 1e12, "frac_of_e4m3_mma_loop": ops / seconds / 1e12 / tensor_peaks["e4m3"],
                          "int8_kernel_tops": ops / int8_seconds / 1e12,
                          "int8_kernel_frac_of_int8_mma_loop": ops / int8_seconds / 1e12 / tensor_peaks["s8"]}

    n, k = GEMV_N, GEMV_K
    copies = [make_packed_w4a16(torch, generator, n, k, device) for _ in range(8)]  # 8 x 31.9 MB: none is in L2 at its turn
    x1 = make_activations(torch, generator, 1, k, "silu", device)
    y1 = torch.empty(1, n, dtype=torch.float16, device=device)
    ms = graph_timed(torch, stream, lambda i: qi.w4a16_gemv_ex(x1, *copies[i % 8], None, y1, qi.DTYPE_F16, n, 1, n, k, handle), 48)
    gemv_bytes = n * k // 2 + 2 * n * (k // 64) * 2 + 2 * k + 2 * n
    out["w4a16_gemv"] = {"n": n, "k": k, "us": ms * 1e3, "bytes": gemv_bytes,
                         "roofline": {"bound": "hbm", "achieved": gemv_bytes / ms / 1e6, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                      "frac": gemv_bytes / ms / 1e6 / peaks["hbm_gbs"]}}
    # the grouped form: sixteen matrices per launch (none of them in L2 at its turn: 510 MB per launch)
    group_copies = copies + [make_packed_w4a16(torch, generator, n, k, device) for _ in range(8)]
    group_outputs = [torch.empty(1, n, dtype=torch.float16, device=device) for _ in group_copies]
    table, keep = qi.gemv_items([(c, s_, m_, None, out_) for (c, s_, m_), out_ in zip(group_copies, group_outputs)])
    ms = graph_timed(torch, stream, lambda i: qi.w4a16_gemv_grouped_ex(x1, table, qi.DTYPE_F16, n, 1, n, k, handle), 6)
    per_matrix_ms = ms / len(group_copies)
    out["w4a16_gemv_grouped"] = {"n": n, "k": k, "matrices_per_launch": len(group_copies), "us_per_matrix": per_matrix_ms * 1e3,
                                 "bytes_per_matrix": gemv_bytes,
                                 "roofline": {"bound": "hbm", "achieved": gemv_bytes / per_matrix_ms / 1e6, "peak": peaks["hbm_gbs"],
                                              "unit": "GB/s", "frac": gemv_bytes / per_matrix_ms / 1e6 / peaks["hbm_gbs"]}}
    del copies, group_copies, group_outputs, table, keep

    out["quantiser"] = []
    for k in (3072, 12288):
        sets = 8 if k == 3072 else 3  # rotating inputs: 8 x 25 MB or 3 x 101 MB
        xs = [torch.randn(m, k, device=device, generator=generator).half() for _ in range(sets)]
        scales = torch.empty(m, k // 64, dtype=torch.float16, device=device)
        wide = torch.empty(m, k, dtype=torch.uint8, device=device)
        ms = graph_timed(torch, stream, lambda i: qi.w4a4_quantize_activations_wide_ex(xs[i % sets], qi.DTYPE_F16, None, scales, wide, m, k, handle), 4 * sets)
        traffic = m * k * 2 + m * k + m * (k // 64) * 2
        out["quantiser"].append({"k": k, "us": ms * 1e3, "bytes": traffic,
                                 "roofline": {"bound": "hbm", "achieved": traffic / ms / 1e6, "peak": peaks["hbm_gbs"],
                                              "unit": "GB/s", "frac": traffic / ms / 1e6 / peaks["hbm_gbs"]}})
        del xs, scales, wide
    assert qi.kernel_status() == 0, "a kernel gave up on a wait"
    return out


def reference_kernels_on_b200(torch, device, m):
    """The reference's own sm_75-era kernels (qwen_image_cuda/cuda/gemm.cu, compiled unmodified for sm_100a
    beside the oracle) timed on this GPU on the block's four shapes: a baseline figure, like the CPU leg.
    None where that build is absent."""
    path = os.path.join(ROOT, "oracle", "_ref", "libqi_ref_gemm.so")
    if not os.path.exists(path):
        return None
    ref = ctypes.CDLL(path)
    P, I = ctypes.c_void_p, ctypes.c_int
    ref.qi_w4a4_quantize_activations.argtypes = [P, P, P, I, I]
    ref.qi_w4a4_gemm.argtypes = [P, P, P, P, P, I, I, I]
    ref.qi_w4a16_gemm.argtypes = [P, P, P, P, P, I, I, I]
    generator = torch.Generator(device=device)
    generator.manual_seed(777)
    stream = torch.cuda.default_stream(device)  # the reference launches on the legacy default stream

    def timed(launch, count=5):
        for _ in range(2):
            assert launch() == 0
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record(stream)
        for _ in range(count):
            launch()
        end.record(stream)
        torch.cuda.synchronize()
        return begin.elapsed_time(end) / count

    def ptr(t):
        return ctypes.c_void_p(t.data_ptr())

    rows = []
    totals = {"w4a4": [0.0, 0.0], "w4a16": [0.0, 0.0]}
    for name, n, k, _ in LINEARS:
        x = torch.randn(m, k, device=device, generator=generator)
        a_codes = torch.empty(m, k // 2, dtype=torch.uint8, device=device)
        a_scales = torch.empty(m, k // 64, dtype=torch.float16, device=device)
        w_codes, w_scales = make_packed_w4a4(torch, generator, n, k, device)
        y = torch.empty(m, n, dtype=torch.float32, device=device)
        quant_ms = timed(lambda: ref.qi_w4a4_quantize_activations(ptr(x), ptr(a_codes), ptr(a_scales), m, k))
        w4a4_ms = timed(lambda: ref.qi_w4a4_gemm(ptr(a_codes), ptr(a_scales), ptr(w_codes), ptr(w_scales), ptr(y), m, n, k))
        codes, scales, minimums = make_packed_w4a16(torch, generator, n, k, device)
        x_half = x.half()
        w4a16_ms = timed(lambda: ref.qi_w4a16_gemm(ptr(x_half), ptr(codes), ptr(scales), ptr(minimums), ptr(y), m, n, k))
        ops = 2.0 * m * n * k
        rows.append({"linear": name, "quantise_us": quant_ms * 1e3, "w4a4_ms": w4a4_ms, "w4a4_tops": ops / w4a4_ms / 1e9,
                     "w4a16_ms": w4a16_ms, "w4a16_tflops": ops / w4a16_ms / 1e9})
        totals["w4a4"][0] += ops
        totals["w4a4"][1] += w4a4_ms + quant_ms
        totals["w4a16"][0] += ops
        totals["w4a16"][1] += w4a16_ms
        del x, a_codes, a_scales, w_codes, w_scales, y, codes, scales, minimums, x_half
    return {"kind": "reference", "what": "qwen_image_cuda/cuda/gemm.cu built for sm_100a, legacy default stream, fp32 in and out",
            "m": m, "linears": rows,
            "w4a4_block_tops_with_quantisers": totals["w4a4"][0] / totals["w4a4"][1] / 1e9,
            "w4a16_block_tflops": totals["w4a16"][0] / totals["w4a16"][1] / 1e9}


# ---- shared set-up ---------------------------------------------------------------------------------

class Job:
    """Device, ranks, the library and (N > 1) its sharding context."""

    def __init__(self, args):
        import torch
        import __graft_entry__ as entry

        self.torch = torch
        self.qi = entry.load_package()
        self.qi.lib()  # no fallback: the kernels are the product
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus and self.world == 1 and args.gpus > 1:
            raise SystemExit("launch N > 1 with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...")
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        self.dist, self.context = None, None
        if self.world > 1:
            import torch.distributed as dist
            self.dist = dist
            dist.init_process_group("nccl", device_id=self.device)
            holder = [self.qi.shard_unique_id() if self.rank == 0 else None]
            dist.broadcast_object_list(holder, src=0)
            self.context = self.qi.ShardContext(self.rank, self.world, holder[0])  # the library's own communicator (C ABI)
        self.stream = torch.cuda.Stream(device=self.device)
        self.handle = self.stream.cuda_stream

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, values):
        times = self.torch.tensor(values, dtype=self.torch.float64, device=self.device)
        if self.dist is not None:
            self.dist.all_reduce(times, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in times.tolist()]

    def close(self, peers=None):
        if self.dist is not None:
            self.torch.cuda.synchronize()
            self.dist.barrier()  # nobody unmaps a copy that another rank may still write
            if peers is not None:
                peers.close()
            self.context.destroy()
            self.dist.barrier()
            self.dist.destroy_process_group()


def tensor_peaks_now(qi):
    """Dense tcgen05.mma rates of this GPU, measured now: 0.2 s per kind, long enough for the power limit to act."""
    return {"f16": qi.probe_tensor_rate(0, 0.2), "e4m3": qi.probe_tensor_rate(1, 0.2), "s8": qi.probe_tensor_rate(2, 0.2),
            "how": "qi_probe_tensor_rate: every SM issuing dense tcgen05.mma 128x256xK from resident shared memory for 0.2 s, "
                   "measured in this run on this GPU"}


# ---- the W4A4 block (workloads block and c4) ----------------------------------------------------------

def run_block(args):
    job = Job(args)
    torch, qi, device, world, rank = job.torch, job.qi, job.device, job.world, job.rank
    dist, context, stream, stream_handle = job.dist, job.context, job.stream, job.handle
    m = args.m
    assert m % world == 0, "rows must divide by the number of ranks (the quantiser is sharded by rows)"
    generator = torch.Generator(device=device)
    generator.manual_seed(1234)  # same weights and activations on every rank
    shard_rows = world > 1 and args.shard_quantiser
    m_local = m // world if shard_rows else m
    row0 = rank * m_local if shard_rows else 0
    layers, full = [], []
    for name, n, k, kind in LINEARS:
        w_codes, w_scales = make_packed_w4a4(torch, generator, n, k, device)
        x = make_activations(torch, generator, m, k, kind, device)
        lo, n_local = qi.shard_plan(n, world, rank)
        w_local = w_codes[lo:lo + n_local].contiguous()
        w_wide = torch.empty(n_local, k, dtype=torch.uint8, device=device)
        assert qi.w4a4_widen_codes_ex(w_local, w_wide, n_local, k) == 0  # load-time step, like packing
        layer = {
            "name": name, "n": n, "k": k, "n_local": n_local, "lo": lo, "x": x,
            "w_codes": w_local, "w_wide": w_wide, "w_scales": w_scales[lo:lo + n_local].contiguous(),
            "a_codes": torch.empty(m, k // 2, dtype=torch.uint8, device=device),
            "a_wide": torch.empty(m, k, dtype=torch.uint8, device=device),
            "a_scales": torch.empty(m, k // 64, dtype=torch.float16, device=device),
            "y_local": torch.empty(m, n_local, dtype=torch.float16, device=device),
            "y_all": torch.empty(world, m, n_local, dtype=torch.float16, device=device) if world > 1 else None,
        }
        if shard_rows:  # this rank's rows of the quantiser's outputs, gathered into a_wide / a_codes / a_scales
            layer["a_wide_rows"] = torch.empty(m_local, k, dtype=torch.uint8, device=device)
            layer["a_codes_rows"] = torch.empty(m_local, k // 2, dtype=torch.uint8, device=device)
            layer["a_scales_rows"] = torch.empty(m_local, k // 64, dtype=torch.float16, device=device)
        if world > 1:
            full.append((w_codes, w_scales))  # kept until the gathered outputs have been checked
        del w_codes, w_scales
        layers.append(layer)
    wide_path = args.w4a4_path == "wide"
    gather_by_default = args.gather == "auto"
    if args.gather == "auto":
        # measured on the M = 4096 and M = 16384 blocks: on two GPUs the copy engines leave the GEMMs undisturbed
        # (1213 against 1018 TOP/s, 1426 against 1082); from four GPUs on they do not keep up and NCCL's all-gather wins
        args.gather = "copy" if world == 2 and wide_path else "nccl"
    fused = context is not None and args.gather == "fused" and wide_path
    # "copy": the GEMM writes its slice into this rank's whole output, then the copy engines carry it to the others
    # "slabs": the same with the whole output kept as slabs [ranks][rows][N/ranks], so that each copy is one contiguous block
    slabs = context is not None and args.gather == "slabs" and wide_path
    copied = slabs or (context is not None and args.gather == "copy" and wide_path)
    placed = fused or copied
    peers = None
    if placed:
        # Every rank holds every linear's whole output, all in ONE allocation that the other ranks map. Outputs
        # alternate between two sets step by step: a set is rewritten only after the barrier of the step in
        # between, which every rank reaches after its readers of that set were queued. Set 2: the end-to-end path.
        sizes = [(m * layer["n"] * 2 + 255) // 256 * 256 for layer in layers]
        pool = torch.empty(4 * sum(sizes), dtype=torch.uint8, device=device)

        def exchange(item):
            items = [None] * world
            dist.all_gather_object(items, item)
            return items

        try:
            peers = qi.PeerOutput(context, pool, exchange)
        except qi.PeerMappingError:
            if not gather_by_default:
                raise
            peers = None  # every rank gets here together: the ranks may not share memory on this box
            del pool
            args.gather, fused, slabs, copied, placed = "nccl", False, False, False, False
    if placed:
        offset = 0
        for layer, size in zip(layers, sizes):
            layer["whole"], layer["copies"], layer["mine"] = [], [], []
            for _ in range(4):
                flat = pool[offset:offset + m * layer["n"] * 2].view(torch.float16)
                if slabs:
                    layer["whole"].append(flat.view(world, m, layer["n_local"]))
                    layer["mine"].append(layer["whole"][-1][rank])
                    layer["copies"].append(peers.copies(offset + rank * m * layer["n_local"] * 2))
                else:
                    layer["whole"].append(flat.view(m, layer["n"]))
                    layer["mine"].append(layer["whole"][-1][:, layer["lo"]:layer["lo"] + layer["n_local"]])
                    layer["copies"].append(peers.copies(offset))
                offset += size
            layer["ldy"], layer["column"] = (layer["n_local"], 0) if slabs else (layer["n"], layer["lo"])
    torch.cuda.synchronize()

    launches = {"count": 0}
    gather_stream = torch.cuda.Stream(device=device) if context is not None else None

    def quantise(layer, x_in):
        k = layer["k"]
        if not shard_rows:
            if wide_path:
                return qi.w4a4_quantize_activations_wide_ex(x_in, qi.DTYPE_F16, None, layer["a_scales"], layer["a_wide"], m, k, stream_handle)
            return qi.w4a4_quantize_activations_ex(x_in, qi.DTYPE_F16, layer["a_codes"], layer["a_scales"], m, k, stream_handle)
        # this rank's rows, then every rank's codes and scales (moved as 2-byte words: [ranks][m_local][k] is [m][k])
        x_rows = x_in[row0:row0 + m_local]
        if wide_path:
            status = qi.w4a4_quantize_activations_wide_ex(x_rows, qi.DTYPE_F16, None, layer["a_scales_rows"], layer["a_wide_rows"], m_local, k, stream_handle)
            status = status or context.all_gather(layer["a_wide_rows"], layer["a_wide"], qi.DTYPE_F16, m_local, k // 2, stream_handle)
        else:
            status = qi.w4a4_quantize_activations_ex(x_rows, qi.DTYPE_F16, layer["a_codes_rows"], layer["a_scales_rows"], m_local, k, stream_handle)
            status = status or context.all_gather(layer["a_codes_rows"], layer["a_codes"], qi.DTYPE_F16, m_local, k // 4, stream_handle)
        return status or context.all_gather(layer["a_scales_rows"], layer["a_scales"], qi.DTYPE_F16, m_local, k // 64, stream_handle)

    def gemm(layer, y_out, output_set):
        k, n_local = layer["k"], layer["n_local"]
        if fused:
            return qi.w4a4_gemm_wide_scatter_ex(layer["a_wide"], layer["a_scales"], layer["w_wide"], layer["w_scales"], None,
                                                layer["copies"][output_set], (rank + 1) % world, qi.DTYPE_F16, layer["n"],
                                                layer["lo"], m, n_local, k, stream_handle)
        if copied:
            return qi.w4a4_gemm_wide_ex(layer["a_wide"], layer["a_scales"], layer["w_wide"], layer["w_scales"], None,
                                        layer["mine"][output_set], qi.DTYPE_F16, layer["ldy"], m, n_local, k, stream_handle)
        if wide_path:
            return qi.w4a4_gemm_wide_ex(layer["a_wide"], layer["a_scales"], layer["w_wide"], layer["w_scales"], None, y_out,
                                        qi.DTYPE_F16, n_local, m, n_local, k, stream_handle)
        path = qi.W4A4_PATH_INT8 if args.w4a4_path == "int8" else qi.W4A4_PATH_BY_SHAPE
        return qi.w4a4_gemm_path_ex(layer["a_codes"], layer["a_scales"], layer["w_codes"], layer["w_scales"], None, y_out,
                                    qi.DTYPE_F16, n_local, m, n_local, k, path, stream_handle)

    def step(index, record_gemm_events=None, slot=None):
        """One pass over the four linears. `slot` selects the end-to-end path's own input/output buffers."""
        output_set = index % 2 if slot is None else 2 + slot
        for layer in layers:
            x_in = layer["x"] if slot is None else layer["x_slots"][slot]
            y_out = layer["y_local"] if slot is None else layer["y_slots"][slot]
            status = quantise(layer, x_in)
            assert status == 0, f"quantise {layer['name']}: status {status}"
            if layer.get("gathered") is not None:
                stream.wait_event(layer["gathered"])  # the previous gather of this linear has read its slice
            if record_gemm_events is not None:
                start = torch.cuda.Event(enable_timing=True)
                start.record(stream)
            status = gemm(layer, y_out, output_set)
            assert status == 0, f"gemm {layer['name']}: cuda status {status}"
            if record_gemm_events is not None:
                stop = torch.cuda.Event(enable_timing=True)
                stop.record(stream)
                record_gemm_events.append((start, stop, layer))
            launches["count"] += 2
            if context is not None:
                # the gather of this linear runs on its own stream, under the next linear's kernels
                computed_event = torch.cuda.Event()
                computed_event.record(stream)
                gather_stream.wait_event(computed_event)
                if fused:  # the slices are already on their way: what is left is to know that every rank's have landed
                    status = context.barrier(gather_stream.cuda_stream)
                elif copied:
                    status = context.put_slice(layer["copies"][output_set], qi.DTYPE_F16, layer["ldy"], layer["column"], m,
                                               layer["n_local"], gather_stream.cuda_stream)
                    assert status == 0, f"put {layer['name']}: status {status}"
                    status = context.barrier(gather_stream.cuda_stream)
                else:
                    status = context.all_gather(y_out, layer["y_all"], qi.DTYPE_F16, m, layer["n_local"], gather_stream.cuda_stream)
                assert status == 0, f"all-gather {layer['name']}: status {status}"
                layer["gathered"] = torch.cuda.Event()
                layer["gathered"].record(gather_stream)
        if context is not None:
            stream.wait_stream(gather_stream)  # a step ends when its last slice has arrived everywhere

    for index in range(args.warmup):
        step(index)
    job.barrier()
    assert qi.kernel_status() == 0, "a kernel gave up on a wait during warm-up"

    verified = None
    if context is not None:
        # What every rank now holds as the whole output of each linear equals the same kernels run unsharded on this
        # rank's own GPU, bit for bit: sharded quantiser rows, gathered codes, column slices and their placement.
        last = (args.warmup - 1) % 2
        for layer, (w_codes, w_scales) in zip(layers, full):
            n, k = layer["n"], layer["k"]
            scales = torch.empty(m, k // 64, dtype=torch.float16, device=device)
            expected = torch.empty(m, n, dtype=torch.float16, device=device)
            if wide_path:
                a_wide = torch.empty(m, k, dtype=torch.uint8, device=device)
                w_wide = torch.empty(n, k, dtype=torch.uint8, device=device)
                assert qi.w4a4_quantize_activations_wide_ex(layer["x"], qi.DTYPE_F16, None, scales, a_wide, m, k, stream_handle) == 0
                assert qi.w4a4_widen_codes_ex(w_codes, w_wide, n, k, stream_handle) == 0
                assert qi.w4a4_gemm_wide_ex(a_wide, scales, w_wide, w_scales, None, expected, qi.DTYPE_F16, n, m, n, k, stream_handle) == 0
            else:
                a_codes = torch.empty(m, k // 2, dtype=torch.uint8, device=device)
                assert qi.w4a4_quantize_activations_ex(layer["x"], qi.DTYPE_F16, a_codes, scales, m, k, stream_handle) == 0
                assert qi.w4a4_gemm_ex(a_codes, scales, w_codes, w_scales, None, expected, qi.DTYPE_F16, n, m, n, k, stream_handle) == 0
            stream.synchronize()
            if placed:
                got = layer["whole"][last]
                got = got.permute(1, 0, 2).reshape(m, n) if slabs else got
            else:
                got = layer["y_all"].permute(1, 0, 2).reshape(m, n)
            assert torch.equal(got, expected), f"{layer['name']}: the gathered output differs from the unsharded one on rank {rank}"
            del expected, scales
        full.clear()
        job.barrier()
        verified = f"gathered outputs of all four linears bit-equal to the unsharded kernels on every one of {world} ranks"

    # ---- device-timed region: exactly `steps` steps
    launches["count"] = 0
    gemm_events = []
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(job.local_rank) as sampler:
        job.barrier()
        begin.record(stream)
        for index in range(args.steps):
            step(args.warmup + index, gemm_events)
        end.record(stream)
        job.barrier()
        elapsed_ms = begin.elapsed_time(end)
        timed_launches = launches["count"]
        assert qi.kernel_status() == 0, "a kernel gave up on a wait during the timed region"
        gemm_ms = sum(a.elapsed_time(b) for a, b, _ in gemm_events)
        gemm_ops = sum(2.0 * m * layer["n_local"] * layer["k"] for _, _, layer in gemm_events)

        # ---- end to end: host buffers in, host buffers out, every step
        # Three streams and two sets of device buffers: while step s computes, the inputs of step s + 1 come in and the
        # results of step s - 1 go out (PCIe is full duplex; the copies, not the kernels, set the pace).
        host_x = [layer["x"].cpu().pin_memory() for layer in layers]
        host_y = [torch.empty(m, layer["n_local"], dtype=torch.float16).pin_memory() for layer in layers]
        h2d = sum(t.numel() * t.element_size() for t in host_x)
        d2h = sum(t.numel() * t.element_size() for t in host_y)
        for layer in layers:
            layer["x_slots"] = [torch.empty_like(layer["x"]) for _ in range(2)]
            layer["y_slots"] = [torch.empty_like(layer["y_local"]) for _ in range(2)]
        in_stream, out_stream = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
        computed = [None, None]   # event: the kernels that read x_slots[i] / wrote y_slots[i] are done
        copied_out = [None, None]  # event: y_slots[i] has reached the host

        def e2e_step(index):
            slot = index % 2
            if computed[slot] is not None:
                in_stream.wait_event(computed[slot])       # the step that read this input slot is done
            with torch.cuda.stream(in_stream):
                for layer, hx in zip(layers, host_x):
                    layer["x_slots"][slot].copy_(hx, non_blocking=True)
            arrived = torch.cuda.Event()
            arrived.record(in_stream)
            stream.wait_event(arrived)
            if copied_out[slot] is not None:
                stream.wait_event(copied_out[slot])         # the results last written to this output slot are on the host
            step(index, slot=slot)
            computed[slot] = torch.cuda.Event()
            computed[slot].record(stream)
            out_stream.wait_event(computed[slot])
            with torch.cuda.stream(out_stream):
                for layer, hy in zip(layers, host_y):
                    if placed:  # this rank's slice of its whole output
                        hy.copy_(layer["mine"][2 + slot], non_blocking=True)
                    else:
                        hy.copy_(layer["y_slots"][slot], non_blocking=True)
            copied_out[slot] = torch.cuda.Event()
            copied_out[slot].record(out_stream)

        e2e_steps = max(4, min(args.steps, 20))
        for index in range(4):
            e2e_step(index)
        job.barrier()
        e2e_begin, e2e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2e_begin.record(in_stream)  # the streams are idle here: the first thing to run is the first copy on in_stream
        for index in range(e2e_steps):
            e2e_step(index)
        out_stream.wait_stream(stream)
        out_stream.wait_stream(in_stream)
        e2e_end.record(out_stream)   # after the last result has reached the host
        job.barrier()
        e2e_ms = e2e_begin.elapsed_time(e2e_end)

    elapsed_ms, e2e_ms, gemm_ms = job.max_over_ranks([elapsed_ms, e2e_ms, gemm_ms])

    result = None
    if rank == 0:
        peaks = measured_peaks()
        tensor_peaks = tensor_peaks_now(qi)
        ops_per_step = block_ops(m)
        value = ops_per_step * args.steps / (elapsed_ms * 1e-3) / 1e12
        e2e_value = ops_per_step * e2e_steps / (e2e_ms * 1e-3) / 1e12
        # one GPU's GEMM launches: operations of its column slices over the time of its launches
        achieved = gemm_ops / (gemm_ms * 1e-3) / 1e12
        eight_bit_peak = tensor_peaks["s8" if args.w4a4_path == "int8" else "e4m3"]
        working_set = sum(l["w_wide"].numel() + l["x"].numel() * 2 + l["a_wide"].numel() + l["y_local"].numel() * 2
                          for l in layers)
        if world == 1:
            parallelism = "single GPU"
        else:
            how = ("slices stored to every GPU by the GEMM epilogue + barrier" if fused else
                   f"slices put on every GPU by the copy engines ({'slabs' if slabs else 'row-major'}) + barrier" if copied else
                   "NCCL all-gather of the output slices")
            parallelism = (f"N-sharded x{world}, {how}; activation quantiser "
                           + ("sharded by rows, codes and scales all-gathered" if shard_rows else "replicated"))
        result = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": ("int4 codes, exact int8 tensor-core group dots, fp32 fold" if args.w4a4_path == "int8" else
                      "int4 codes (one E4M3 byte each), exact fp32 tensor-core group dots, fp32 fold"),
            "data": "synthetic: W ~ N(0,0.02) rotated (H256) and quantised to int4 g64 on the device, "
                    "X fp16 ~ N(0,1) with 1% outlier channels x20 (fc2 input: GELU-tanh of N(0,1)); seed 1234",
            "config": {"workload": workload_text(m), "name": args.workload, "m": m, "ops_per_step": ops_per_step,
                       "w4a4_path": args.w4a4_path, "parallelism": parallelism, "outputs": "fp16",
                       "l2": f"per-step working set {working_set / 1e6:.0f} MB per GPU exceeds the 126 MB L2"},
            "gpu_launches": timed_launches,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
            "roofline": {"kernel": "w4a4::gemm_kernel" if args.w4a4_path == "int8" else "w4a4_pair::gemm_kernel", "bound": "tensor",
                         "achieved": achieved, "peak": eight_bit_peak, "unit": "TOP/s", "frac": achieved / eight_bit_peak,
                         "frac_of_2x_bf16_burst": achieved / (2.0 * peaks["bf16_burst"]),
                         "frac_of_2x_bf16_sustained": achieved / (2.0 * peaks["bf16_sustained"]),
                         "traffic": (NCU_TRAFFIC_BYTES_QKV_M4096 * (m / 4096.0) / world) if wide_path else None,
                         "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of the qkv launch at "
                                           "M=4096 (its 2MNK is the average of the four launches), scaled by rows and ranks",
                         "peak_source": tensor_peaks["how"] + f"; bf16 figures of MEASURED_PEAKS.json ({peaks['source']})",
                         "tensor_peaks_measured_now": {key: tensor_peaks[key] for key in ("f16", "e4m3", "s8")},
                         "launches_timed": len(gemm_events), "avg_launch_ms": gemm_ms / max(1, len(gemm_events))},
            "clocks": sampler.summary(),
        }
        if verified is not None:
            result["verified"] = verified
        if world == 1 and not args.no_other_kernels:
            result["other_kernels"] = other_kernels(qi, torch, device, stream, peaks, tensor_peaks, m)
            if not args.no_cpu_baseline:
                result["other_kernels"]["reference_kernels_on_b200"] = reference_kernels_on_b200(torch, device, m)
    job.close(peers)
    return result


# ---- the W4A4 block with paired splits (N > 1, --parallel pairs) ------------------------------------------

def run_block_pairs(args):
    """The block with the splits paired the way the block's data flow allows, so that no wide tensor is gathered:
    qkv and fc1 are split by output columns and their slices stay on their GPU (attention works on whole heads, the
    activation function on elements); out and fc2 are split by INPUT columns - the slice a GPU computed in the linear
    before is the slice it needs - and their float32 partial results are summed over the GPUs (all-reduce) and stored
    as fp16. Where an input split would cut a 256-input Hadamard block (out at 8 GPUs: 384 inputs per GPU) the
    linear falls back to output columns with an all-gather. The sums run on a second stream under the next kernels."""
    job = Job(args)
    torch, qi, device, world, rank = job.torch, job.qi, job.device, job.world, job.rank
    context, stream, handle = job.context, job.stream, job.handle
    assert context is not None, "--parallel pairs is a multi-GPU mode"
    m = args.m
    scatter = args.sum == "reduce-scatter"
    assert m % world == 0, "rows must divide by the number of ranks"
    generator = torch.Generator(device=device)
    generator.manual_seed(1234)
    layers, full = [], []
    for name, n, k, kind in LINEARS:
        w_codes, w_scales = make_packed_w4a4(torch, generator, n, k, device)
        x = make_activations(torch, generator, m, k, kind, device)
        split = "columns" if name in ("qkv", "fc1") else "inputs"
        if split == "inputs":
            try:
                k_lo, k_local = qi.shard_plan_inputs(k, qi.SCHEME_W4A4_H256, world, rank)
            except ValueError:
                split = "columns+gather"
        if split == "inputs":
            n_local, lo = n, 0
            w_local = w_codes[:, k_lo // 2:(k_lo + k_local) // 2].contiguous()
            scales_local = w_scales[:, k_lo // 64:(k_lo + k_local) // 64].contiguous()
            x_local = x[:, k_lo:k_lo + k_local].contiguous()
        else:
            k_lo, k_local = 0, k
            lo, n_local = qi.shard_plan(n, world, rank)
            w_local = w_codes[lo:lo + n_local].contiguous()
            scales_local = w_scales[lo:lo + n_local].contiguous()
            x_local = x
        w_wide = torch.empty(n_local, k_local, dtype=torch.uint8, device=device)
        assert qi.w4a4_widen_codes_ex(w_local, w_wide, n_local, k_local) == 0
        layers.append({
            "name": name, "n": n, "k": k, "split": split, "n_local": n_local, "lo": lo, "k_lo": k_lo, "k_local": k_local,
            "x": x_local, "w_wide": w_wide, "w_scales": scales_local,
            "a_wide": torch.empty(m, k_local, dtype=torch.uint8, device=device),
            "a_scales": torch.empty(m, k_local // 64, dtype=torch.float16, device=device),
            "y_local": torch.empty(m, n_local, dtype=torch.float16, device=device) if split != "inputs" else None,
            "y_sum": torch.empty(m, n, dtype=torch.float32, device=device) if split == "inputs" else None,
            "y_half": torch.empty(m // world if scatter else m, n, dtype=torch.float16, device=device) if split == "inputs" else None,
            "y_share": torch.empty(m // world, n, dtype=torch.float32, device=device) if split == "inputs" and scatter else None,
            "y_all": torch.empty(world, m, n_local, dtype=torch.float16, device=device) if split == "columns+gather" else None,
        })
        full.append((w_codes, w_scales, x))
    torch.cuda.synchronize()
    launches = {"count": 0}
    side = torch.cuda.Stream(device=device)

    def step(index, events=None, slot=None):
        for layer in layers:
            k_local, n_local = layer["k_local"], layer["n_local"]
            x_in = layer["x"] if slot is None else layer["x_slots"][slot]
            assert qi.w4a4_quantize_activations_wide_ex(x_in, qi.DTYPE_F16, None, layer["a_scales"], layer["a_wide"], m, k_local, handle) == 0
            if layer.get("summed") is not None:
                stream.wait_event(layer["summed"])  # the previous sum or gather has read this linear's output buffer
            if events is not None:
                start = torch.cuda.Event(enable_timing=True)
                start.record(stream)
            if layer["split"] == "inputs":
                status = qi.w4a4_gemm_wide_ex(layer["a_wide"], layer["a_scales"], layer["w_wide"], layer["w_scales"], None,
                                              layer["y_sum"], qi.DTYPE_F32, n_local, m, n_local, k_local, handle)
            else:
                y_out = layer["y_local"] if slot is None else layer["y_slots"][slot]
                status = qi.w4a4_gemm_wide_ex(layer["a_wide"], layer["a_scales"], layer["w_wide"], layer["w_scales"], None,
                                              y_out, qi.DTYPE_F16, n_local, m, n_local, k_local, handle)
            assert status == 0, f"gemm {layer['name']}: cuda status {status}"
            if events is not None:
                stop = torch.cuda.Event(enable_timing=True)
                stop.record(stream)
                events.append((start, stop, layer))
            launches["count"] += 2
            if layer["split"] == "columns":
                continue
            computed = torch.cuda.Event()
            computed.record(stream)
            side.wait_event(computed)
            if layer["split"] == "inputs":
                y_half = layer["y_half"] if slot is None else layer["y_slots"][slot]
                if scatter:
                    status = context.reduce_scatter(layer["y_sum"], layer["y_share"], (m // world) * layer["n"], side.cuda_stream)
                    status = status or qi.f32_to_f16_ex(layer["y_share"], y_half, (m // world) * layer["n"], side.cuda_stream)
                else:
                    status = context.all_reduce(layer["y_sum"], m * layer["n"], side.cuda_stream)
                    status = status or qi.f32_to_f16_ex(layer["y_sum"], y_half, m * layer["n"], side.cuda_stream)
                launches["count"] += 1
            else:
                status = context.all_gather(y_out, layer["y_all"], qi.DTYPE_F16, m, n_local, side.cuda_stream)
            assert status == 0, f"sum or gather {layer['name']}: status {status}"
            layer["summed"] = torch.cuda.Event()
            layer["summed"].record(side)
        stream.wait_stream(side)  # a step ends when its last sum has arrived everywhere

    for index in range(args.warmup):
        step(index)
    job.barrier()
    assert qi.kernel_status() == 0, "a kernel gave up on a wait during warm-up"

    # What each rank holds equals the unsharded kernels on its own GPU: column slices bit for bit, the summed linears
    # to the rounding of `world` float32 partial sums and one fp16 store.
    worst = 0.0
    for layer, (w_codes, w_scales, x) in zip(layers, full):
        n, k = layer["n"], layer["k"]
        scales = torch.empty(m, k // 64, dtype=torch.float16, device=device)
        expected = torch.empty(m, n, dtype=torch.float16, device=device)
        a_wide = torch.empty(m, k, dtype=torch.uint8, device=device)
        w_wide = torch.empty(n, k, dtype=torch.uint8, device=device)
        assert qi.w4a4_quantize_activations_wide_ex(x, qi.DTYPE_F16, None, scales, a_wide, m, k, handle) == 0
        assert qi.w4a4_widen_codes_ex(w_codes, w_wide, n, k, handle) == 0
        assert qi.w4a4_gemm_wide_ex(a_wide, scales, w_wide, w_scales, None, expected, qi.DTYPE_F16, n, m, n, k, handle) == 0
        stream.synchronize()
        if layer["split"] == "inputs":
            share = m // world
            got = layer["y_half"].float()
            want = (expected[rank * share:(rank + 1) * share] if scatter else expected).float()
            error = float(((got - want).abs() / (want.abs() + 1e-3 * want.abs().max())).max())
            worst = max(worst, error)
            assert error <= 2e-3, f"{layer['name']}: the summed output is {error:.2e} away from the unsharded one on rank {rank}"
        elif layer["split"] == "columns":
            assert torch.equal(layer["y_local"], expected[:, layer["lo"]:layer["lo"] + layer["n_local"]]), \
                f"{layer['name']}: the column slice differs from the unsharded output on rank {rank}"
        else:
            assert torch.equal(layer["y_all"].permute(1, 0, 2).reshape(m, n), expected), \
                f"{layer['name']}: the gathered output differs from the unsharded one on rank {rank}"
        del expected, scales, a_wide, w_wide
    full.clear()
    torch.cuda.empty_cache()
    job.barrier()
    verified = (f"on every one of {world} ranks: column slices bit-equal to the unsharded kernels, summed linears within "
                f"{worst:.1e} relative of them (float32 partial sums in NCCL's order, one fp16 store)")

    launches["count"] = 0
    gemm_events = []
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(job.local_rank) as sampler:
        job.barrier()
        begin.record(stream)
        for index in range(args.steps):
            step(args.warmup + index, gemm_events)
        end.record(stream)
        job.barrier()
        elapsed_ms = begin.elapsed_time(end)
        timed_launches = launches["count"]
        assert qi.kernel_status() == 0, "a kernel gave up on a wait during the timed region"
        gemm_ms = sum(a.elapsed_time(b) for a, b, _ in gemm_events)
        gemm_ops = sum(2.0 * m * layer["n_local"] * layer["k_local"] for _, _, layer in gemm_events)

        # end to end: every rank brings in the inputs it needs (its input slice for the summed linears) and takes out
        # what it produced (its column slice, or its share of the rows of a summed output), every step
        host_x = [layer["x"].cpu().pin_memory() for layer in layers]
        rows = m // world
        host_y = [torch.empty((rows, layer["n"]) if layer["split"] == "inputs" else (m, layer["n_local"]), dtype=torch.float16).pin_memory()
                  for layer in layers]
        h2d = sum(t.numel() * t.element_size() for t in host_x)
        d2h = sum(t.numel() * t.element_size() for t in host_y)
        for layer in layers:
            layer["x_slots"] = [torch.empty_like(layer["x"]) for _ in range(2)]
            layer["y_slots"] = [torch.empty_like(layer["y_half"] if layer["split"] == "inputs" else layer["y_local"]) for _ in range(2)]
        in_stream, out_stream = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
        computed, copied_out = [None, None], [None, None]

        def e2e_step(index):
            slot = index % 2
            if computed[slot] is not None:
                in_stream.wait_event(computed[slot])
            with torch.cuda.stream(in_stream):
                for layer, hx in zip(layers, host_x):
                    layer["x_slots"][slot].copy_(hx, non_blocking=True)
            arrived = torch.cuda.Event()
            arrived.record(in_stream)
            stream.wait_event(arrived)
            if copied_out[slot] is not None:
                stream.wait_event(copied_out[slot])
            step(index, slot=slot)
            computed[slot] = torch.cuda.Event()
            computed[slot].record(stream)
            out_stream.wait_event(computed[slot])
            with torch.cuda.stream(out_stream):
                for layer, hy in zip(layers, host_y):
                    source = layer["y_slots"][slot]
                    hy.copy_(source[rank * rows:(rank + 1) * rows] if layer["split"] == "inputs" and not scatter else source, non_blocking=True)
            copied_out[slot] = torch.cuda.Event()
            copied_out[slot].record(out_stream)

        e2e_steps = max(4, min(args.steps, 20))
        for index in range(4):
            e2e_step(index)
        job.barrier()
        e2e_begin, e2e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2e_begin.record(in_stream)
        for index in range(e2e_steps):
            e2e_step(index)
        out_stream.wait_stream(stream)
        out_stream.wait_stream(in_stream)
        e2e_end.record(out_stream)
        job.barrier()
        e2e_ms = e2e_begin.elapsed_time(e2e_end)

    elapsed_ms, e2e_ms, gemm_ms = job.max_over_ranks([elapsed_ms, e2e_ms, gemm_ms])
    result = None
    if rank == 0:
        peaks = measured_peaks()
        tensor_peaks = tensor_peaks_now(qi)
        ops_per_step = block_ops(m)
        achieved = gemm_ops / (gemm_ms * 1e-3) / 1e12
        splits = ", ".join(f"{layer['name']}: {layer['split']}" for layer in layers)
        result = {
            "metric": METRIC, "value": ops_per_step * args.steps / (elapsed_ms * 1e-3) / 1e12, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": "int4 codes (one E4M3 byte each), exact fp32 tensor-core group dots, fp32 fold",
            "data": "synthetic: W ~ N(0,0.02) rotated (H256) and quantised to int4 g64 on the device, "
                    "X fp16 ~ N(0,1) with 1% outlier channels x20 (fc2 input: GELU-tanh of N(0,1)); seed 1234",
            "config": {"workload": workload_text(m), "name": args.workload, "m": m, "ops_per_step": ops_per_step,
                       "w4a4_path": "wide", "outputs": "fp16",
                       "parallelism": f"paired splits x{world} ({splits}); float32 partial results summed by NCCL "
                                      + ("reduce-scatter (each rank keeps its share of the rows)" if scatter else "all-reduce")
                                      + " on a second stream, then stored as fp16; activation quantiser on each rank's own inputs",
                       "l2": "per-step working set exceeds the 126 MB L2"},
            "gpu_launches": timed_launches,
            "e2e": {"value": ops_per_step * e2e_steps / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
            "roofline": {"kernel": "w4a4_pair::gemm_kernel", "bound": "tensor", "achieved": achieved, "peak": tensor_peaks["e4m3"],
                         "unit": "TOP/s", "frac": achieved / tensor_peaks["e4m3"],
                         "frac_of_2x_bf16_burst": achieved / (2.0 * peaks["bf16_burst"]),
                         "frac_of_2x_bf16_sustained": achieved / (2.0 * peaks["bf16_sustained"]),
                         "traffic": NCU_TRAFFIC_BYTES_QKV_M4096 * (m / 4096.0) / world,
                         "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of the qkv launch at "
                                           "M=4096 (its 2MNK is the average of the four launches), scaled by rows and ranks",
                         "peak_source": tensor_peaks["how"] + f"; bf16 figures of MEASURED_PEAKS.json ({peaks['source']})",
                         "tensor_peaks_measured_now": {key: tensor_peaks[key] for key in ("f16", "e4m3", "s8")},
                         "launches_timed": len(gemm_events), "avg_launch_ms": gemm_ms / max(1, len(gemm_events))},
            "clocks": sampler.summary(), "verified": verified,
        }
    job.close()
    return result


# ---- the 60-block stacks (workloads c3 and c5) ------------------------------------------------------

def run_stack(args):
    """One denoising step's packed linears through the dispatcher (qi_linear / qi_shard_linear), block after block.
    c3: every linear scheme 5, two streams with their own weights, two modulation GEMVs per block.
    c5: rows 2 x (12288 + 512) in one stream, scheme 6 with probability 0.7 per linear (seeded), else scheme 5."""
    job = Job(args)
    torch, qi, device, world, rank = job.torch, job.qi, job.device, job.world, job.rank
    context, stream, handle = job.context, job.stream, job.handle
    generator = torch.Generator(device=device)
    generator.manual_seed(4242)
    host_random = __import__("random").Random(4242)  # the per-linear policy, the same on every rank
    blocks = args.blocks
    if args.workload == "c3":
        streams = [("image", 4096), ("text", 256)]
        gemvs_per_block = 2
    else:
        streams = [("edit", 2 * (12288 + 512))]
        gemvs_per_block = 0
    k_max = max(k for _, _, k, _ in LINEARS)
    policy_counts = {"w4a4": 0, "w4a16": 0}

    def make_record(n, k, keep_whole):
        """This rank's shard of a fresh random record, and (keep_whole, N > 1) the whole record for the check below."""
        scheme6 = args.workload == "c5" and host_random.random() < 0.7
        lo, n_local = qi.shard_plan(n, world, rank)
        whole = None
        if scheme6:
            policy_counts["w4a4"] += 1
            all_codes, all_scales = make_packed_w4a4(torch, generator, n, k, device)
            codes, scales = all_codes[lo:lo + n_local].contiguous(), all_scales[lo:lo + n_local].contiguous()
            wide = torch.empty(n_local, k, dtype=torch.uint8, device=device)
            assert qi.w4a4_widen_codes_ex(codes, wide, n_local, k) == 0
            if keep_whole:
                all_wide = torch.empty(n, k, dtype=torch.uint8, device=device)
                assert qi.w4a4_widen_codes_ex(all_codes, all_wide, n, k) == 0
                whole = qi.PackedLinear(qi.SCHEME_W4A4_H256, n, k, all_codes, all_scales, weights_wide=all_wide)
            return qi.PackedLinear(qi.SCHEME_W4A4_H256, n_local, k, codes, scales, weights_wide=wide), whole
        policy_counts["w4a16"] += 1
        codes, scales, minimums = make_packed_w4a16(torch, generator, n, k, device)
        if keep_whole:
            whole = qi.PackedLinear(qi.SCHEME_W4A16, n, k, codes, scales, minimums)
        return qi.PackedLinear(qi.SCHEME_W4A16, n_local, k, codes[lo:lo + n_local].contiguous(),
                               scales[lo:lo + n_local].contiguous(), minimums[lo:lo + n_local].contiguous()), whole

    plan = []  # (record, stream index, linear index)
    whole_records = []  # the last block's records unsharded, with their place: what the gathered outputs are checked against
    gemv_records = []
    for block in range(blocks):
        for stream_index in range(len(streams)):
            for linear_index, (_, n, k, _) in enumerate(LINEARS):
                record, whole = make_record(n, k, world > 1 and block == blocks - 1)
                plan.append((record, stream_index, linear_index))
                if whole is not None:
                    whole_records.append((whole, stream_index, linear_index))
        for _ in range(gemvs_per_block):
            gemv_records.append(make_packed_w4a16(torch, generator, GEMV_N, GEMV_K, device))
    inputs, outputs, works, slabs = [], [], [], []
    for _, rows in streams:
        inputs.append([make_activations(torch, generator, rows, k, kind, device) for _, _, k, kind in LINEARS])
        outputs.append([torch.empty(rows, qi.shard_plan(n, world, rank)[1], dtype=torch.float16, device=device) for _, n, _, _ in LINEARS])
        slabs.append([torch.empty(world, rows, qi.shard_plan(n, world, rank)[1], dtype=torch.float16, device=device)
                      if world > 1 else None for _, n, _, _ in LINEARS])
        works.append(qi.LinearWork(torch.empty(rows * k_max // 2, dtype=torch.uint8, device=device),
                                   torch.empty(rows * k_max // 64, dtype=torch.float16, device=device),
                                   torch.empty(rows * k_max, dtype=torch.float16, device=device),
                                   wide=torch.empty(rows * k_max, dtype=torch.uint8, device=device)))
    gemv_x = make_activations(torch, generator, 1, GEMV_K, "silu", device)
    # every block's modulation linears read the same conditioning vector: one grouped launch per 64 matrices at the
    # start of the step instead of one launch per matrix inside its block
    gemv_table = gemv_keep = None
    if gemv_records:
        gemv_table, gemv_keep = qi.gemv_items([(codes, scales, minimums, None, torch.empty(1, GEMV_N, dtype=torch.float16, device=device))
                                               for codes, scales, minimums in gemv_records])
    launches = {"count": 0}

    def step():
        if gemv_table is not None:  # replicated on every rank: 32 MB of weights each
            assert qi.w4a16_gemv_grouped_ex(gemv_x, gemv_table, qi.DTYPE_F16, GEMV_N, 1, GEMV_N, GEMV_K, handle) == 0
            launches["count"] += (len(gemv_table) + 63) // 64
        for position, (record, stream_index, linear_index) in enumerate(plan):
            rows = streams[stream_index][1]
            x, y = inputs[stream_index][linear_index], outputs[stream_index][linear_index]
            if context is None:
                status = qi.linear(record, works[stream_index], x, y, rows, input_dtype=qi.DTYPE_F16,
                                   output_dtype=qi.DTYPE_F16, stream=handle)
            else:
                status = context.linear(record, works[stream_index], x, y, slabs[stream_index][linear_index], rows,
                                        input_dtype=qi.DTYPE_F16, output_dtype=qi.DTYPE_F16, stream=handle)
            assert status == 0, f"linear {position}: status {status}"
            launches["count"] += 2 if record.scheme == qi.SCHEME_W4A4_H256 else 1

    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            step()
    job.barrier()
    assert qi.kernel_status() == 0, "a kernel gave up on a wait during warm-up"
    verified = None
    if context is not None:
        # The slabs hold what the last block left: gathered, they equal the same dispatcher on the whole record on this
        # rank's own GPU, bit for bit (the buffers are reused block after block, so the last block is what can be checked).
        for whole, stream_index, linear_index in whole_records:
            rows = streams[stream_index][1]
            expected = torch.empty(rows, whole.n, dtype=torch.float16, device=device)
            assert qi.linear(whole, works[stream_index], inputs[stream_index][linear_index], expected, rows,
                             input_dtype=qi.DTYPE_F16, output_dtype=qi.DTYPE_F16, stream=handle) == 0
            stream.synchronize()
            got = slabs[stream_index][linear_index].permute(1, 0, 2).reshape(rows, whole.n)
            assert torch.equal(got, expected), f"stream {stream_index} linear {linear_index}: the gathered output differs on rank {rank}"
            del expected
        whole_records.clear()
        torch.cuda.empty_cache()
        job.barrier()
        verified = (f"gathered outputs of the last block's {len(streams) * len(LINEARS)} linears bit-equal to the unsharded "
                    f"dispatcher on every one of {world} ranks")
    launches["count"] = 0
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(job.local_rank) as sampler:
        job.barrier()
        begin.record(stream)
        for _ in range(args.steps):
            step()
        end.record(stream)
        job.barrier()
        elapsed_ms = begin.elapsed_time(end)
        timed_launches = launches["count"]
        assert qi.kernel_status() == 0, "a kernel gave up on a wait during the timed region"
        # end to end: the step's first inputs come from pinned host memory and its last outputs go back, every step
        host_in = [inputs[i][0].cpu().pin_memory() for i in range(len(streams))]
        host_out = [torch.empty_like(outputs[i][3], device="cpu").pin_memory() for i in range(len(streams))]
        e2e_steps = max(2, min(args.steps, 5))
        e2e_begin, e2e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        job.barrier()
        with torch.cuda.stream(stream):
            e2e_begin.record(stream)
            for _ in range(e2e_steps):
                for i in range(len(streams)):
                    inputs[i][0].copy_(host_in[i], non_blocking=True)
                step()
                for i in range(len(streams)):
                    host_out[i].copy_(outputs[i][3], non_blocking=True)
            e2e_end.record(stream)
        job.barrier()
        e2e_ms = e2e_begin.elapsed_time(e2e_end)
    elapsed_ms, e2e_ms = job.max_over_ranks([elapsed_ms, e2e_ms])
    result = None
    if rank == 0:
        peaks = measured_peaks()
        tensor_peaks = tensor_peaks_now(qi)
        ops = blocks * sum(block_ops(rows) for _, rows in streams)
        gemv_bytes = GEMV_N * GEMV_K // 2 + 2 * GEMV_N * (GEMV_K // 64) * 2
        value = ops * args.steps / (elapsed_ms * 1e-3) / 1e12
        share6 = policy_counts["w4a4"] / max(1, policy_counts["w4a4"] + policy_counts["w4a16"])
        # a mixed stack is measured against the mix of the two tensor peaks its operations see
        peak = 1.0 / (share6 / tensor_peaks["e4m3"] + (1.0 - share6) / tensor_peaks["f16"])
        result = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp16 x int4 (W4A16) and int4 x int4 (W4A4) packed linears, fp32 accumulate",
            "data": "synthetic: random valid QIPACK v6 records, X fp16 ~ N(0,1) with 1% outlier channels x20 (fc2: GELU-tanh); seed 4242",
            "config": {"workload": ("60-block W4A16 g64 linear stack of one denoising step: image M=4096 + text M=256, two M=1 "
                                    "modulation GEMVs 3072->18432 per block (all of a step's in one grouped launch per 64)" if args.workload == "c3" else
                                    "image-edit stack: rows 2 x (12288 + 512), 60 blocks x 4 linears, each W4A4 with probability 0.7 else W4A16 (seeded)"),
                       "name": args.workload, "blocks": blocks, "ops_per_step": ops,
                       "gemv_bytes_per_step": gemv_bytes * gemvs_per_block * blocks,
                       "policy": dict(policy_counts), "parallelism": "single GPU" if world == 1 else f"N-sharded x{world} + NCCL all-gather (qi_shard_linear)",
                       "outputs": "fp16", "l2": "weights of one step exceed the 126 MB L2 many times over"},
            "gpu_launches": timed_launches,
            "e2e": {"value": ops * e2e_steps / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
                    "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in host_in),
                    "d2h_bytes_per_step": sum(t.numel() * t.element_size() for t in host_out), "steps": e2e_steps,
                    "ms_per_step": e2e_ms / e2e_steps},
            "roofline": {"kernel": "the stack's GEMM kernels together (whole step)", "bound": "tensor", "achieved": value / world, "peak": peak,
                         "unit": "TOP/s", "frac": value / world / peak, "traffic": None,
                         "peak_source": tensor_peaks["how"] + "; harmonic mix of the fp16 and FP8 rates by the share of W4A4 linears",
                         "tensor_peaks_measured_now": {key: tensor_peaks[key] for key in ("f16", "e4m3", "s8")}},
            "clocks": sampler.summary(),
        }
        if verified is not None:
            result["verified"] = verified
    job.close()
    return result


# ---- the CPU arm: the oracle port on this host's cores ----------------------------------------------

def cpu_port(rows: int, passes: int, warmup: int):
    """Times the CPU restatement of the block's four linears (oracle/qipack_oracle.c, threaded over every host
    core this process may use, whatever OMP_NUM_THREADS says) on the first `rows` activation rows.
    Returns (TOPS from the median pass, cores, median seconds per pass, passes)."""
    import numpy as np
    from oracle import qipack_oracle as qo

    rng = np.random.default_rng(1234)
    cores = qo.available_cores()
    work = []
    for _, n, k, _ in LINEARS:
        values = rng.integers(-7, 8, size=(n, k), dtype=np.int8).astype(np.int16) & 0xF
        codes = (values[:, 0::2] | (values[:, 1::2] << 4)).astype(np.uint8)
        scales = rng.uniform(1e-3, 6e-3, size=(n, k // 64)).astype(np.float16).view(np.uint16)
        x = rng.standard_normal((rows, k), dtype=np.float32).astype(np.float16)
        work.append((x, codes, scales))
    times = []
    for index in range(warmup + passes):
        start = time.perf_counter()
        for x, codes, scales in work:
            qo.w4a4_linear_fast(x, codes, scales, threads=cores)
        if index >= warmup:
            times.append(time.perf_counter() - start)
    seconds = statistics.median(times)
    return block_ops(rows) / seconds / 1e12, cores, seconds, len(times)


def cpu_sample_text(m, seconds, passes):
    return (f"first {CPU_SAMPLE_ROWS} of {m} rows of each of the block's four linears, activation quantisation included; "
            f"median of {passes} passes of {seconds:.2f} s after one warm-up pass")


def run_reference(args):
    """The reference's path on the host cores. The reference engine has no CPU implementation of
    these linears and its NumPy evaluator cannot travel, so this is the C port of the same
    arithmetic (kind "port"); each step is the block's four linears on a bounded row sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    passes = max(CPU_PASSES, min(args.steps, 30))  # a pass takes a few tenths of a second
    tops, cores, seconds, passes = cpu_port(CPU_SAMPLE_ROWS, passes, 1)
    sample = cpu_sample_text(args.m, seconds, passes)
    return {
        "impl": "reference", "metric": METRIC, "value": tops, "unit": UNIT, "n_gpus": args.gpus, "steps": passes,
        "warmup": 1, "ms_per_step": seconds * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int4 codes, int32 dots, fp32 fold", "data": "synthetic",
        "config": {"workload": workload_text(args.m), "name": args.workload, "m": CPU_SAMPLE_ROWS, "sample": sample},
        "cpu_baseline": {"value": tops, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--workload", default="block", choices=["block", "c4", "c3", "c5"],
                        help="block: configs[1] (headline); c4: the block at M=16384; c3: the W4A16 stack; c5: the mixed image-edit stack")
    parser.add_argument("--m", type=int, default=None, help="rows of the block workloads (default 4096; c4: 16384)")
    parser.add_argument("--blocks", type=int, default=60, help="blocks of the stack workloads")
    parser.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU and reference-kernel legs (profiling runs)")
    parser.add_argument("--no-other-kernels", action="store_true",
                        help="skip the W4A16 GEMM / GEMV / quantiser figures (profiling runs)")
    parser.add_argument("--w4a4-path", default="wide", choices=["packed", "int8", "wide"],
                        help="packed: the drop-in entry points on nibble-packed codes, kernel by shape (both operands widened into "
                             "pool scratch for the CTA-pair kernel); int8: the same entry points held to the int8 kernel that widens "
                             "the nibbles in shared memory; wide: byte-wide E4M3 codes on CTA pairs (weights widened once at load)")
    parser.add_argument("--gather", default="auto", choices=["auto", "fused", "copy", "slabs", "nccl"],
                        help="N > 1: how the column slices reach every GPU. auto: copy on two GPUs, nccl on more. nccl: an all-gather after each GEMM; fused: the "
                             "GEMM's epilogue stores its slice into every GPU's output over NVLink, a barrier follows; copy: the copy "
                             "engines carry the slice to every GPU, a barrier follows; slabs: the same with outputs [ranks][rows][N/ranks]")
    parser.add_argument("--parallel", default="columns", choices=["columns", "pairs"],
                        help="N > 1, block workloads: columns: every linear split by output columns and its slices gathered (the "
                             "default); pairs: qkv and fc1 by output columns without a gather, out and fc2 by input columns with an "
                             "all-reduce of the float32 partial results")
    parser.add_argument("--sum", default="all-reduce", choices=["all-reduce", "reduce-scatter"],
                        help="--parallel pairs: what becomes of the partial results of out and fc2. all-reduce: every GPU ends with the "
                             "whole output (the operator's contract). reduce-scatter: GPU r ends with rows [r M / N, (r + 1) M / N) only - "
                             "half the bytes - for a pipeline whose next kernels (layer norm, quantiser) work on rows")
    parser.add_argument("--shard-quantiser", action="store_true",
                        help="N > 1: every rank quantises its share of the rows and the codes and scales are all-gathered, "
                             "instead of every rank quantising all rows (measured slower on 2 GPUs: two more NCCL launches "
                             "per linear in front of the GEMM cost more than the quantiser they save)")
    args = parser.parse_args()
    if args.m is None:
        args.m = 16384 if args.workload == "c4" else 4096
    stack = args.workload in ("c3", "c5")
    if args.steps is None:
        args.steps = 3 if stack else (200 if args.m <= 4096 else 50)
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else max(args.warmup, 1)

    if args.impl == "reference":
        result = run_reference(args)
        if result is not None:
            print(json.dumps(result), flush=True)
        return
    pairs = args.parallel == "pairs" and not stack and int(os.environ.get("WORLD_SIZE", "1")) > 1
    result = run_stack(args) if stack else run_block_pairs(args) if pairs else run_block(args)
    if result is None:
        return
    if not args.no_cpu_baseline and result["n_gpus"] == 1:
        tops, cores, seconds, passes = cpu_port(CPU_SAMPLE_ROWS, CPU_PASSES, 1)
        result["cpu_baseline"] = {"value": tops, "unit": UNIT, "cores": cores, "kind": "port",
                                  "sample": cpu_sample_text(args.m, seconds, passes)}
    print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
