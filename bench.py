#!/usr/bin/env python3
"""Benchmark of the QIPACK v6 packed-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One step = one pass over the four linears of one Qwen-Image MMDiT block image stream at
1024x1024 under W4A4 (H256, g64): M = 4096 image tokens, hidden 3072 —
fused q/k/v 3072->9216, attention out 3072->3072, MLP fc1 3072->12288, fc2 12288->3072 —
each with its own activation rotation + quantisation (fp16 in) and fp16 outputs.
2*M*N*K summed over the four linears = 927.7 G operations per step.

N > 1 (launched by torch.distributed.run, one rank per GPU): every linear's packed weights are
sharded by output columns, rank r computes y[:, r*N/R:(r+1)*N/R] and the slices are
all-gathered over NVLink; total work is fixed (strong scaling).

Prints ONE JSON line. `value` is device-timed with inputs resident in HBM; `e2e` is the same
metric through the C ABI with host buffers (pinned) copied in and results copied out every step
(copies of neighbouring steps overlap the kernels on separate streams);
`roofline` is the W4A4 GEMM kernel's achieved rate from CUDA events around its launches inside
the timed region; `cpu_baseline` is the CPU oracle port timed on this host on a bounded sample.
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

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M_TOKENS = 4096
HIDDEN = 3072
# name, n, k, kind of activation
LINEARS = [("qkv", 9216, 3072, "outliers"), ("attn_out", 3072, 3072, "outliers"),
           ("fc1", 12288, 3072, "outliers"), ("fc2", 3072, 12288, "gelu")]
OPS_PER_STEP = sum(2.0 * M_TOKENS * n * k for _, n, k, _ in LINEARS)
METRIC = "packed W4A4/W4A16 GEMM TOPS at M=4096 block shapes, % of tensor/HBM roofline"
UNIT = "TOPS"
WORKLOAD = "qwen-image MMDiT block image stream, W4A4 H256 g64, M=4096 hidden=3072: qkv 3072->9216, out 3072->3072, fc1 3072->12288, fc2 12288->3072"
CPU_SAMPLE_ROWS = 256
# DRAM bytes of one w4a4_pair::gemm_kernel launch of average size (42.3 MB read + 36.5 MB written), from ncu
NCU_TRAFFIC_BYTES_PER_AVERAGE_LAUNCH = 78.8e6


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
    """nvidia-smi sampled every 200 ms while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.process, self.lines = index, None, []

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None
        return self

    def _read(self):
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.process is not None:
            time.sleep(0.25)
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


def make_activations(torch, generator, m, k, kind, device):
    x = torch.randn(m, k, generator=generator, device=device)
    if kind == "outliers":
        channels = torch.randperm(k, generator=generator, device=device)[: max(1, k // 100)]
        x[:, channels] *= 20.0
    elif kind == "gelu":
        x = torch.nn.functional.gelu(x, approximate="tanh")
    return x.half().contiguous()


# ---- the path's other kernels, each against its own roofline ---------------------------------------

def other_kernels(qi, torch, device, stream, peaks, m):
    """W4A16 GEMM on the block's four shapes (tensor bound), the W4A16 M=1 GEMV and the activation
    quantiser (HBM bound), timed with CUDA events around a CUDA graph on `stream`. GEMV weights rotate through more
    copies than fit in L2; the other inputs are larger than L2 by themselves or compute bound."""
    handle = stream.cuda_stream
    generator = torch.Generator(device=device)
    generator.manual_seed(4321)

    def timed(launch, count):
        """Average device time of `count` launches replayed from one CUDA graph: the kernels here run for
        a few microseconds, less than the host needs to issue one launch through ctypes."""
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

    def affine_pack(n, k):
        codes = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=device, generator=generator)
        scales = (torch.rand(n, k // 64, device=device, generator=generator) * 0.006 + 0.002).half()
        return codes, scales, (-8.0 * scales.float()).half()

    out = {"w4a16_gemm": [], "peak_source": peaks["source"]}
    flops = seconds = 0.0
    for name, n, k, _ in LINEARS:
        codes, scales, minimums = affine_pack(n, k)
        x = torch.randn(m, k, device=device, generator=generator).half()
        y = torch.empty(m, n, dtype=torch.float16, device=device)
        ms = timed(lambda i: qi.w4a16_gemm_ex(x, codes, scales, minimums, None, y, qi.DTYPE_F16, n, m, n, k, handle), 20)
        flops += 2.0 * m * n * k
        seconds += ms * 1e-3
        out["w4a16_gemm"].append({"linear": name, "ms": ms, "tflops": 2.0 * m * n * k / ms / 1e9})
        del codes, scales, minimums, x, y
    achieved = flops / seconds / 1e12
    out["w4a16_gemm_roofline"] = {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_sustained"], "unit": "TFLOP/s",
                                  "frac": achieved / peaks["bf16_sustained"]}

    n, k = 9216, 3072  # q/k/v of one token: the decode-shaped call
    copies = [affine_pack(n, k) for _ in range(12)]  # 12 x 15.4 MB: no copy is still in L2 when its turn comes again
    x1 = torch.randn(1, k, device=device, generator=generator).half()
    y1 = torch.empty(1, n, dtype=torch.float16, device=device)
    ms = timed(lambda i: qi.w4a16_gemv_ex(x1, *copies[i % 12], None, y1, qi.DTYPE_F16, n, 1, n, k, handle), 48)
    gemv_bytes = n * k // 2 + 2 * n * (k // 64) * 2 + 2 * k + 2 * n
    out["w4a16_gemv"] = {"n": n, "k": k, "us": ms * 1e3, "bytes": gemv_bytes,
                         "roofline": {"bound": "hbm", "achieved": gemv_bytes / ms / 1e6, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                      "frac": gemv_bytes / ms / 1e6 / peaks["hbm_gbs"]}}
    del copies

    out["quantiser"] = []
    for k in (3072, 12288):
        sets = 8 if k == 3072 else 3  # rotating inputs: 8 x 25 MB or 3 x 101 MB
        xs = [torch.randn(m, k, device=device, generator=generator).half() for _ in range(sets)]
        scales = torch.empty(m, k // 64, dtype=torch.float16, device=device)
        wide = torch.empty(m, k, dtype=torch.uint8, device=device)
        ms = timed(lambda i: qi.w4a4_quantize_activations_wide_ex(xs[i % sets], qi.DTYPE_F16, None, scales, wide, m, k, handle), 4 * sets)
        traffic = m * k * 2 + m * k + m * (k // 64) * 2
        out["quantiser"].append({"k": k, "us": ms * 1e3, "bytes": traffic,
                                 "roofline": {"bound": "hbm", "achieved": traffic / ms / 1e6, "peak": peaks["hbm_gbs"],
                                              "unit": "GB/s", "frac": traffic / ms / 1e6 / peaks["hbm_gbs"]}})
        del xs, scales, wide
    assert qi.kernel_status() == 0, "a kernel gave up on a wait"
    return out


# ---- the b200 arm ---------------------------------------------------------------------------------

def run_b200(args):
    import torch
    import __graft_entry__ as entry

    qi = entry.load_package()
    qi.lib()  # no fallback: the kernels are the product
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch N > 1 with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    context = None
    if world > 1:
        import torch.distributed as dist_module
        dist = dist_module
        dist.init_process_group("nccl", device_id=device)
        holder = [qi.shard_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(holder, src=0)
        context = qi.ShardContext(rank, world, holder[0])  # the library's own communicator (C ABI)

    generator = torch.Generator(device=device)
    generator.manual_seed(1234)  # same weights and activations on every rank
    stream = torch.cuda.Stream(device=device)
    stream_handle = stream.cuda_stream
    m = M_TOKENS
    layers = []
    for name, n, k, kind in LINEARS:
        w_codes, w_scales = make_packed_w4a4(torch, generator, n, k, device)
        x = make_activations(torch, generator, m, k, kind, device)
        lo, n_local = qi.shard_plan(n, world, rank)
        w_local = w_codes[lo:lo + n_local].contiguous()
        w_wide = torch.empty(n_local, k, dtype=torch.uint8, device=device)
        assert qi.w4a4_widen_codes_ex(w_local, w_wide, n_local, k) == 0  # load-time step, like packing
        layer = {
            "name": name, "n": n, "k": k, "n_local": n_local, "x": x,
            "w_codes": w_local, "w_wide": w_wide, "w_scales": w_scales[lo:lo + n_local].contiguous(),
            "a_codes": torch.empty(m, k // 2, dtype=torch.uint8, device=device),
            "a_wide": torch.empty(m, k, dtype=torch.uint8, device=device),
            "a_scales": torch.empty(m, k // 64, dtype=torch.float16, device=device),
            "y_local": torch.empty(m, n_local, dtype=torch.float16, device=device),
            "y_all": torch.empty(world, m, n_local, dtype=torch.float16, device=device) if world > 1 else None,
        }
        del w_codes, w_scales
        layers.append(layer)
    # Without the all-gather: every rank holds every linear's whole output, all of them in ONE allocation that the
    # other ranks map, and the GEMM's epilogue stores its slice into every rank's copy (buffer 0: the device-timed
    # loop; 1 and 2: the end-to-end path's two slots).
    if args.gather == "auto":
        args.gather = "copy" if world == 2 and args.w4a4_path == "wide" else "nccl"
    fused = context is not None and args.gather == "fused" and args.w4a4_path == "wide"
    # "copy": the GEMM writes its slice into this rank's whole output, then the copy engines carry it to the others
    # "slabs": the same with the whole output kept as slabs [ranks][rows][N/ranks], so that each copy is one contiguous block
    slabs = context is not None and args.gather == "slabs" and args.w4a4_path == "wide"
    copied = slabs or (context is not None and args.gather == "copy" and args.w4a4_path == "wide")
    placed = fused or copied
    peers = None
    if placed:
        sizes = [(m * layer["n"] * 2 + 255) // 256 * 256 for layer in layers]
        pool = torch.empty(3 * sum(sizes), dtype=torch.uint8, device=device)

        def exchange(item):
            items = [None] * world
            dist.all_gather_object(items, item)
            return items

        peers = qi.PeerOutput(context, pool, exchange)
        offset = 0
        for layer, size in zip(layers, sizes):
            layer["lo"] = qi.shard_plan(layer["n"], world, rank)[0]
            layer["whole"], layer["copies"], layer["mine"] = [], [], []
            for _ in range(3):
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
            # rows of the matrix the slice lives in, and the slice's first column there
            layer["ldy"], layer["column"] = (layer["n_local"], 0) if slabs else (layer["n"], layer["lo"])
    torch.cuda.synchronize()

    launches = {"count": 0}
    gather_stream = torch.cuda.Stream(device=device) if context is not None else None

    def step(record_gemm_events=None, slot=None):
        """One pass over the four linears. `slot` selects the end-to-end path's own input/output buffers."""
        for layer in layers:
            k, n_local = layer["k"], layer["n_local"]
            x_in = layer["x"] if slot is None else layer["x_slots"][slot]
            y_out = layer["y_local"] if slot is None else layer["y_slots"][slot]
            if args.w4a4_path == "wide":
                status = qi.w4a4_quantize_activations_wide_ex(x_in, qi.DTYPE_F16, None, layer["a_scales"],
                                                              layer["a_wide"], m, k, stream_handle)
            else:
                status = qi.w4a4_quantize_activations_ex(x_in, qi.DTYPE_F16, layer["a_codes"], layer["a_scales"],
                                                         m, k, stream_handle)
            assert status == 0, f"quantise {layer['name']}: cuda status {status}"
            if layer.get("gathered") is not None:
                stream.wait_event(layer["gathered"])  # the previous gather of this linear has read its slice
            if record_gemm_events is not None:
                start = torch.cuda.Event(enable_timing=True)
                start.record(stream)
            if fused:
                status = qi.w4a4_gemm_wide_scatter_ex(layer["a_wide"], layer["a_scales"], layer["w_wide"], layer["w_scales"],
                                                      None, layer["copies"][0 if slot is None else slot + 1],
                                                      (rank + 1) % world, qi.DTYPE_F16, layer["n"], layer["lo"], m,
                                                      n_local, k, stream_handle)
            elif copied:
                status = qi.w4a4_gemm_wide_ex(layer["a_wide"], layer["a_scales"], layer["w_wide"], layer["w_scales"],
                                              None, layer["mine"][0 if slot is None else slot + 1], qi.DTYPE_F16,
                                              layer["ldy"], m, n_local, k, stream_handle)
            elif args.w4a4_path == "wide":
                status = qi.w4a4_gemm_wide_ex(layer["a_wide"], layer["a_scales"], layer["w_wide"], layer["w_scales"],
                                              None, y_out, qi.DTYPE_F16, n_local, m, n_local, k, stream_handle)
            else:
                status = qi.w4a4_gemm_ex(layer["a_codes"], layer["a_scales"], layer["w_codes"], layer["w_scales"], None,
                                         y_out, qi.DTYPE_F16, n_local, m, n_local, k, stream_handle)
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
                    status = context.put_slice(layer["copies"][0 if slot is None else slot + 1], qi.DTYPE_F16, layer["ldy"],
                                               layer["column"], m, n_local, gather_stream.cuda_stream)
                    assert status == 0, f"put {layer['name']}: status {status}"
                    status = context.barrier(gather_stream.cuda_stream)
                else:
                    status = context.all_gather(y_out, layer["y_all"], qi.DTYPE_F16, m, n_local, gather_stream.cuda_stream)
                assert status == 0, f"all-gather {layer['name']}: status {status}"
                layer["gathered"] = torch.cuda.Event()
                layer["gathered"].record(gather_stream)
        if context is not None:
            stream.wait_stream(gather_stream)  # a step ends when its last slice has arrived everywhere

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    assert qi.kernel_status() == 0, "a kernel gave up on a wait during warm-up"
    if placed:
        # every rank's whole outputs, as its peers wrote them, equal what the all-gather of the slices gives
        for layer in layers:
            status = qi.w4a4_gemm_wide_ex(layer["a_wide"], layer["a_scales"], layer["w_wide"], layer["w_scales"], None,
                                          layer["y_local"], qi.DTYPE_F16, layer["n_local"], m, layer["n_local"],
                                          layer["k"], stream_handle)
            assert status == 0
            assert context.all_gather(layer["y_local"], layer["y_all"], qi.DTYPE_F16, m, layer["n_local"], stream_handle) == 0
            stream.synchronize()
            gathered = layer["y_all"] if slabs else layer["y_all"].permute(1, 0, 2).reshape(m, layer["n"])
            assert torch.equal(gathered, layer["whole"][0]), f"{layer['name']}: the peers' stores differ from the all-gather"
        barrier()

    # ---- device-timed region: exactly `steps` steps
    launches["count"] = 0
    gemm_events = []
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as sampler:
        barrier()
        begin.record(stream)
        for _ in range(args.steps):
            step(gemm_events)
        end.record(stream)
        barrier()
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
        step(slot=slot)
        computed[slot] = torch.cuda.Event()
        computed[slot].record(stream)
        out_stream.wait_event(computed[slot])
        with torch.cuda.stream(out_stream):
            for layer, hy in zip(layers, host_y):
                if placed:  # this rank's slice of its whole output
                    hy.copy_(layer["mine"][slot + 1], non_blocking=True)
                else:
                    hy.copy_(layer["y_slots"][slot], non_blocking=True)
        copied_out[slot] = torch.cuda.Event()
        copied_out[slot].record(out_stream)

    e2e_steps = max(4, min(args.steps, 20))
    for index in range(4):
        e2e_step(index)
    barrier()
    e2e_begin, e2e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_begin.record(in_stream)  # the streams are idle here: the first thing to run is the first copy on in_stream
    for index in range(e2e_steps):
        e2e_step(index)
    out_stream.wait_stream(stream)
    out_stream.wait_stream(in_stream)
    e2e_end.record(out_stream)   # after the last result has reached the host
    barrier()
    e2e_ms = e2e_begin.elapsed_time(e2e_end)

    times = torch.tensor([elapsed_ms, e2e_ms, gemm_ms], dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, gemm_ms = (float(v) for v in times.tolist())

    result = None
    if rank == 0:
        peaks = measured_peaks()
        value = OPS_PER_STEP * args.steps / (elapsed_ms * 1e-3) / 1e12
        e2e_value = OPS_PER_STEP * e2e_steps / (e2e_ms * 1e-3) / 1e12
        # one GPU's GEMM launches: operations of its column slices over the time of its launches
        achieved = gemm_ops / (gemm_ms * 1e-3) / 1e12
        int8_peak = 2.0 * peaks["bf16_sustained"]
        working_set = sum(l["w_wide"].numel() + l["x"].numel() * 2 + l["a_wide"].numel() + l["y_local"].numel() * 2
                          for l in layers)
        result = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": ("int4 codes, exact int8 tensor-core group dots, fp32 fold" if args.w4a4_path == "packed" else
                      "int4 codes (one E4M3 byte each), exact fp32 tensor-core group dots, fp32 fold"),
            "data": "synthetic: W ~ N(0,0.02) rotated (H256) and quantised to int4 g64 on the device, "
                    "X fp16 ~ N(0,1) with 1% outlier channels x20 (fc2 input: GELU-tanh of N(0,1)); seed 1234",
            "config": {"workload": WORKLOAD, "m": m, "ops_per_step": OPS_PER_STEP, "w4a4_path": args.w4a4_path,
                       "parallelism": "single GPU" if world == 1 else (f"N-sharded x{world}, slices stored to every GPU by the GEMM epilogue + barrier" if fused else
                                                                              f"N-sharded x{world}, slices put on every GPU by the copy engines ({'slabs' if slabs else 'row-major'}) + barrier" if copied
                                                                              else f"N-sharded x{world} + NCCL all-gather"),
                       "outputs": "fp16", "l2": f"per-step working set {working_set / 1e6:.0f} MB per GPU exceeds the 126 MB L2"},
            "gpu_launches": timed_launches,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
            "roofline": {"kernel": "w4a4::gemm_kernel" if args.w4a4_path == "packed" else "w4a4_pair::gemm_kernel", "bound": "tensor", "achieved": achieved, "peak": int8_peak,
                         "unit": "TOP/s", "frac": achieved / int8_peak,
                         "traffic": (NCU_TRAFFIC_BYTES_PER_AVERAGE_LAUNCH / world) if args.w4a4_path == "wide" else None,
                         "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of the qkv launch "
                                           "(its 2MNK is the average of the four launches), profiles/w4a4_pair_gemm_block_m4096.md",
                         "peak_source": f"2 x the sustained bf16 figure of MEASURED_PEAKS.json ({peaks['source']}); "
                                        "no 8-bit figure is measured; fp8 and int8 run at twice the bf16 rate",
                         "launches_timed": len(gemm_events), "avg_launch_ms": gemm_ms / max(1, len(gemm_events))},
            "clocks": sampler.summary(),
        }
        if world == 1 and not args.no_other_kernels:
            result["other_kernels"] = other_kernels(qi, torch, device, stream, peaks, m)
    if dist is not None:
        torch.cuda.synchronize()
        dist.barrier()  # nobody unmaps a copy that another rank may still write
        if peers is not None:
            peers.close()
        context.destroy()
        dist.barrier()
        dist.destroy_process_group()
    return result


# ---- the CPU arm: the oracle port on this host's cores ----------------------------------------------

def cpu_port(rows: int, repeats: int, warmup: int, min_seconds: float = 0.0):
    """Times the CPU restatement of the same four linears (oracle/qipack_oracle.c, threaded over all
    host cores) on the first `rows` activation rows, `repeats` passes or more until `min_seconds` have
    gone by. Returns (TOPS, cores, seconds per pass)."""
    import numpy as np
    from oracle import qipack_oracle as qo

    rng = np.random.default_rng(1234)
    cores = qo.max_threads()
    work = []
    for _, n, k, _ in LINEARS:
        values = rng.integers(-7, 8, size=(n, k), dtype=np.int8).astype(np.int16) & 0xF
        codes = (values[:, 0::2] | (values[:, 1::2] << 4)).astype(np.uint8)
        scales = rng.uniform(1e-3, 6e-3, size=(n, k // 64)).astype(np.float16).view(np.uint16)
        x = rng.standard_normal((rows, k), dtype=np.float32).astype(np.float16)
        work.append((x, codes, scales))
    for _ in range(warmup):
        for x, codes, scales in work[:1]:
            qo.w4a4_linear_fast(x, codes, scales, threads=cores)
    start = time.perf_counter()
    passes = 0
    while passes < repeats or time.perf_counter() - start < min_seconds:
        for x, codes, scales in work:
            qo.w4a4_linear_fast(x, codes, scales, threads=cores)
        passes += 1
    seconds = (time.perf_counter() - start) / passes
    ops = sum(2.0 * rows * n * k for _, n, k, _ in LINEARS)
    return ops / seconds / 1e12, cores, seconds


def run_reference(args):
    """The reference's path on the host cores. The reference engine has no CPU implementation of
    these linears and its NumPy evaluator cannot travel, so this is the C port of the same
    arithmetic (kind "port"); each step is the block's four linears on a bounded row sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    steps = max(1, min(args.steps, 60))  # a pass takes a few tenths of a second: the run stays well under a minute
    tops, cores, seconds = cpu_port(CPU_SAMPLE_ROWS, steps, min(args.warmup, 1))
    sample = f"first {CPU_SAMPLE_ROWS} of {M_TOKENS} rows of each of the four linears, activation quantisation included"
    return {
        "impl": "reference", "metric": METRIC, "value": tops, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": min(args.warmup, 1), "ms_per_step": seconds * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int4 codes, int32 dots, fp32 fold", "data": "synthetic",
        "config": {"workload": WORKLOAD, "m": CPU_SAMPLE_ROWS, "sample": sample},
        "cpu_baseline": {"value": tops, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU leg (profiling runs)")
    parser.add_argument("--no-other-kernels", action="store_true",
                        help="skip the W4A16 GEMM / GEMV / quantiser figures (profiling runs)")
    parser.add_argument("--w4a4-path", default="wide", choices=["packed", "wide"],
                        help="packed: the drop-in kernels on nibble-packed codes (int8 tensor-core dots); "
                             "wide: byte-wide E4M3 codes on CTA pairs (weights widened once at load)")
    parser.add_argument("--gather", default="auto", choices=["auto", "fused", "copy", "slabs", "nccl"],
                        help="auto: what measured fastest on B200 boxes (copy on 2 GPUs, nccl on 4 and 8). "
                             "N > 1: how the column slices reach every GPU. fused: the GEMM's epilogue stores its slice "
                             "into every GPU's output over NVLink, a barrier follows; copy: the copy engines carry the "
                             "slice to every GPU, a barrier follows; slabs: the same with outputs [ranks][rows][N/ranks] (contiguous copies); nccl: an all-gather after each GEMM")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    if args.impl == "reference":
        result = run_reference(args)
        if result is not None:
            print(json.dumps(result), flush=True)
        return
    result = run_b200(args)
    if result is None:
        return
    if not args.no_cpu_baseline and result["n_gpus"] == 1:
        tops, cores, seconds = cpu_port(CPU_SAMPLE_ROWS, 1, 1, min_seconds=12.0)
        result["cpu_baseline"] = {
            "value": tops, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"first {CPU_SAMPLE_ROWS} of {M_TOKENS} rows of each of the four linears "
                      f"({seconds:.2f} s per pass, passes repeated for 12 s of CPU work), activation quantisation included"}
    print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
