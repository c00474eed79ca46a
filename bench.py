"""Benchmark of the quantized-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--detail]

Headline workload (`config.workload`): the Q3 decode GEMV set of one dense Qwen-27B-shaped decoder layer - q 5120x5120,
k and v 1024x5120, o 5120x5120, gate and up 17408x5120, down 5120x17408 (N x K) - at M = 1 and M = 3 activation rows:
14 quantized GEMVs per step, called one by one through the C ABI on one stream with programmatic dependent launch, the
weights rotated over several resident copies of the layer so that no step finds its weights in L2. The metric is the
algorithmic bytes of the step (weight planes + activations + outputs, each byte once) per second. `extra` carries the
same measurement for the NVFP4 and trellis layouts and the NVFP4 prefill GEMM.

With --gpus N (launched under torch.distributed.run) every weight matrix is split along N over the ranks, each rank
runs its slices into one packed output buffer, and the slices of a step are joined with one NCCL all-gather.

`--impl reference` times the CPU restatement of the reference's dequant + matmul (oracle/oracle.c) on the host cores.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LOCAL_RANK = int(os.environ.get("LOCAL_RANK", "0"))
WORLD = int(os.environ.get("WORLD_SIZE", "1"))
RANK = int(os.environ.get("RANK", "0"))

import numpy as np  # noqa: E402

LAYER = [("q", 5120, 5120), ("k", 1024, 5120), ("v", 1024, 5120), ("o", 5120, 5120), ("gate", 17408, 5120),
         ("up", 17408, 5120), ("down", 5120, 17408)]   # (name, N, K)
HEADLINE_ROWS = (1, 3)
WEIGHT_SEED = 0xE0
ACTIVATION_SEED = 0xA0
SIGMA = 0.02


def read_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def seeded_weights(index: int, n: int, k: int) -> np.ndarray:
    rng = np.random.default_rng(WEIGHT_SEED + index)
    return rng.standard_normal((n, k), dtype=np.float32) * np.float32(SIGMA)


def seeded_rows(rows: int, k: int) -> np.ndarray:
    from oracle import oracle_np as O
    return O.bf16_bits(np.random.default_rng(ACTIVATION_SEED + rows).standard_normal((rows, k)).astype(np.float32))


def algorithmic_bytes(fmt: str, n: int, k: int, rows: int, w: int = 48) -> int:
    from euhedral_b200 import layouts
    weights = {"q3": layouts.q3_algorithmic_bytes(n, k), "nvfp4": layouts.nvfp4_algorithmic_bytes(n, k),
               "trellis": layouts.trellis_algorithmic_bytes(n, k, w, 1)}[fmt]
    return weights + 2 * rows * k + 2 * rows * n


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of this rank's GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.stop, self.thread = index, [], threading.Event(), None

    def _run(self):
        while not self.stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([part.strip() for part in out.split(",")])
            except Exception:
                pass
            self.stop.wait(0.1)

    def __enter__(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()
        return self

    def __exit__(self, *exc):
        self.stop.set()
        self.thread.join(timeout=6)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [name for i, name in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": int(self.samples[0][1]) if self.samples[0][1].isdigit() else None,
                "reasons": reasons, "samples": len(self.samples)}


# ---------------------------------------------------------------------------------------------------------------------
# reference arm: the CPU restatement on the host cores
# ---------------------------------------------------------------------------------------------------------------------

def cpu_layer_pass(blobs, rows_list, threads):
    from oracle import oracle_c as OC
    total = 0
    start = time.perf_counter()
    for (name, n, k), blob in zip(LAYER, blobs):
        for rows in rows_list:
            OC.q3_linear(seeded_rows(rows, k), blob, n, k, threads=threads)
            total += algorithmic_bytes("q3", n, k, rows)
    return total, time.perf_counter() - start


def cpu_blobs():
    from oracle import oracle_c as OC
    return [OC.q3_quantize(seeded_weights(i, n, k)) for i, (name, n, k) in enumerate(LAYER)]


def run_reference(args):
    if RANK != 0:
        return
    from oracle import oracle_c as OC
    threads = OC.default_threads()
    blobs = cpu_blobs()
    for _ in range(min(args.warmup, 1)):
        cpu_layer_pass(blobs, HEADLINE_ROWS, threads)
    total_bytes, total_time = 0, 0.0
    for _ in range(args.steps):
        b, t = cpu_layer_pass(blobs, HEADLINE_ROWS, threads)
        total_bytes += b
        total_time += t
    value = total_bytes / total_time / 1e9
    line = {
        "impl": "reference", "metric": "quantized GEMV algorithmic GB/s (Q3 decode layer set, M=1 and M=3)", "value": value,
        "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_time / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "Q3 decode GEMV set, one Qwen-27B-shaped layer, M in {1,3}", "layer": [list(s) for s in LAYER]},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": "the whole step: 7 matrices x M in {1,3}, plain-C dequant + FP32 dot, row-parallel threads"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------------------------

class Resident:
    """One format's layer set on this rank: `copies` resident copies of every (sharded) weight tensor, the activation
    rows, output buffers and the launch closure of every GEMV of a step."""

    def __init__(self, torch, gpu, fmt: str, rows_list, copies: int, world: int, rank: int, sms: int, w: int = 48, only=None):
        from euhedral_b200 import sharding, synthetic
        from euhedral_b200.formats import (GroupedLinearFormat, LinearLaunch, Nvfp4Format, TensorHandle, TrellisFormat,
                                           TrellisSettings)
        self.torch, self.gpu, self.fmt, self.rows_list, self.copies = torch, gpu, fmt, rows_list, copies
        self.calls = []          # (launch per copy, n_local, n, k, rows)
        self.keep = []
        self.bytes_per_step = 0
        self.h2d = self.d2h = 0
        self.outputs = []
        self.inputs = {}
        self.host_inputs = {}
        # The step's distinct activation tensors live in one packed buffer on each side, so that the end-to-end step
        # uploads them from pinned memory with ONE copy.
        shapes = [(rows, k) for rows in rows_list for k in sorted({k for _, _, k in LAYER})]
        total_in = sum(rows * k for rows, k in shapes)
        self.host_packed_in = torch.empty(total_in, dtype=torch.int16).pin_memory()
        self.packed_in = torch.empty(total_in, dtype=torch.int16, device="cuda")
        cursor = 0
        for rows, k in shapes:
            self.host_packed_in[cursor:cursor + rows * k].copy_(synthetic.bf16_rows(rows, k, ACTIVATION_SEED + rows).view(torch.int16).reshape(-1))
            self.host_inputs[(rows, k)] = self.host_packed_in[cursor:cursor + rows * k]
            self.inputs[(rows, k)] = self.packed_in[cursor:cursor + rows * k]
            cursor += rows * k
        self.packed_in.copy_(self.host_packed_in)
        self.h2d_bytes = 2 * total_in
        settings = TrellisSettings.for_device(sms) if TRELLIS_TARGET_PER_SM is None else TrellisSettings(target_ctas=TRELLIS_TARGET_PER_SM * sms)
        # Every output slice of a step lives in one packed buffer, so that a multi-GPU step joins them with ONE all-gather.
        unit = 128 if fmt == "trellis" else 16
        total = sum(rows * sharding.shard_range(n, world, rank, unit)[1] for name, n, k in LAYER if only in (None, name) for rows in rows_list)
        self.packed = torch.empty(total, dtype=torch.int16, device="cuda")
        self.gathered = torch.empty(total * world, dtype=torch.int16, device="cuda") if world > 1 else self.packed
        self.host_result = torch.empty(total * world, dtype=torch.int16).pin_memory()
        cursor = 0
        for index, (name, n, k) in enumerate(LAYER):
            if only is not None and name != only:
                continue
            first, local = sharding.shard_range(n, world, rank, 128 if fmt == "trellis" else 16)
            if fmt in ("q3", "nvfp4"):
                # N(0, 0.02^2) weights rounded on the device exactly as the converter rounds them; a shard is cut from
                # the whole tensor (NVFP4's tensor scale is the whole tensor's).
                build, cut = (synthetic.q3_tensor, sharding.q3_rows) if fmt == "q3" else (synthetic.nvfp4_tensor, sharding.nvfp4_rows)
                whole = build(synthetic.gaussian(n, k, WEIGHT_SEED + index, SIGMA, device="cuda"))
                blob = whole if world == 1 else torch.from_numpy(cut(whole.cpu().numpy(), n, k, first, local)).cuda()
                del whole
                operator = GroupedLinearFormat() if fmt == "q3" else Nvfp4Format()
            else:
                # Random trellis words with the reference test-suite's scale distributions (its encoder is not part of
                # this build); the K split is planned from the unsharded shape so shards keep the whole object's order.
                payload, suh, svh, ends = synthetic.trellis_object(local, k, w, WEIGHT_SEED + index, 1, device="cuda")
                splits = TrellisFormat.splits(k, n, settings.target_ctas)
                operator = TrellisFormat(TrellisSettings(target_ctas=splits * (local // 128)))
                assert TrellisFormat.splits(k, local, splits * (local // 128)) == splits
            for rows in rows_list:
                launches = []
                out = self.packed[cursor:cursor + rows * local].view(rows, local)
                cursor += rows * local
                for copy in range(copies):
                    if fmt == "trellis":
                        tensors = [a.clone() for a in (payload, suh, svh, ends)]
                        shapes = [payload.shape, (1, k), (local,), (1,)]
                        handles = [TensorHandle(f"{name}{i}", tuple(s), t.data_ptr(), t.numel() * t.element_size()) for i, (t, s) in enumerate(zip(tensors, shapes))]
                        need = operator.scratch_bytes(gpu, rows, k, local, 1)
                        scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
                        self.keep += tensors + [scratch]
                        launch = LinearLaunch(self.inputs[(rows, k)].data_ptr(), out.data_ptr(), handles, rows, k, local,
                                              scratch=scratch.data_ptr(), scratch_bytes=need, row_exact=True)
                    else:
                        tensor = blob.clone()
                        self.keep.append(tensor)
                        handle = TensorHandle(name, (local, k), tensor.data_ptr(), tensor.numel())
                        launch = LinearLaunch(self.inputs[(rows, k)].data_ptr(), out.data_ptr(), [handle], rows, k, local, row_exact=True)
                    launches.append((operator, launch))
                self.calls.append((launches, out, local, n, k, rows))
                self.bytes_per_step += algorithmic_bytes(fmt, local, k, rows, w)
                self.d2h += 2 * rows * local * world
        self.launches_per_step = len(self.calls) * (3 if fmt == "trellis" else 1)

    def step(self, iteration: int, world: int):
        from euhedral_b200 import sharding
        for launches, out, local, n, k, rows in self.calls:
            operator, launch = launches[iteration % self.copies]
            operator.linear(self.gpu, launch)
        if world > 1:
            sharding.gather_packed(self.packed, self.gathered)

    def step_e2e(self, iteration: int, world: int):
        """The same step fed from pinned host memory: the step's activation tensors are uploaded from pinned memory (one
        copy of the packed buffer), and the step's whole result (every rank's slices) is read back to pinned memory at
        the end."""
        from euhedral_b200 import sharding
        self.gpu.copy_upload_to_device(self.packed_in.data_ptr(), self.host_packed_in.data_ptr(), self.h2d_bytes)
        for launches, out, local, n, k, rows in self.calls:
            operator, launch = launches[iteration % self.copies]
            operator.linear(self.gpu, launch)
        if world > 1:
            sharding.gather_packed(self.packed, self.gathered)
        self.gpu.copy_device_to_readback(self.host_result.data_ptr(), self.gathered.data_ptr(), self.gathered.numel() * 2)


def timed(torch, dist, world, steps, warmup, body):
    """max over ranks of the device time of `steps` calls of body(i), after `warmup` untimed calls."""
    for i in range(warmup):
        body(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(torch.cuda.current_stream())
    for i in range(steps):
        body(warmup + i)
    stop.record(torch.cuda.current_stream())
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    seconds = start.elapsed_time(stop) / 1e3
    if world > 1:
        t = torch.tensor([seconds], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        seconds = float(t.item())
    return seconds


def measure_format(torch, dist, gpu, fmt, rows_list, copies, world, rank, sms, steps, warmup, stream, e2e=False, only=None, graph=False):
    """graph=True: the step of every weight copy is captured once into a CUDA graph (plain stream capture of the same
    C-ABI calls) and the timed region replays the graphs - what the launches cost on the device, without the Python
    launch planning of the trellis operator (three table launches per linear, tens of microseconds of host time)."""
    resident = Resident(torch, gpu, fmt, rows_list, copies, world, rank, sms, only=only)
    with torch.cuda.stream(stream), gpu.submit(stream.cuda_stream, pdl=True):
        body = lambda i: resident.step(i, world)
        if graph:
            for i in range(copies):
                body(i)   # plans, tensor maps and occupancy look-ups are made before the capture
            torch.cuda.synchronize()
            graphs = []
            for copy in range(copies):
                captured = torch.cuda.CUDAGraph()
                with torch.cuda.graph(captured, stream=stream):
                    resident.step(copy, world)
                graphs.append(captured)
            body = lambda i: graphs[i % copies].replay()
        seconds = timed(torch, dist, world, steps, warmup, body)
        total_bytes = resident.bytes_per_step
        if world > 1:
            t = torch.tensor([float(total_bytes)], device="cuda", dtype=torch.float64)
            dist.all_reduce(t)
            total_bytes = float(t.item())
        result = {"gbs": total_bytes * steps / seconds / 1e9, "ms_per_step": seconds / steps * 1e3, "bytes_per_step": total_bytes,
                  "launches_per_step": resident.launches_per_step}
        if e2e:
            seconds = timed(torch, dist, world, steps, warmup, lambda i: resident.step_e2e(i, world))
            result["e2e_gbs"] = total_bytes * steps / seconds / 1e9
            result["h2d"], result["d2h"] = resident.h2d_bytes, resident.d2h
    assert gpu.take_device_error() == 0, "a kernel's bounded wait gave up"
    del resident
    torch.cuda.empty_cache()
    return result


def measure_prefill(torch, gpu, stream, steps, warmup, rows=4096, detail=False):
    """NVFP4 prefill GEMM over the seven layer shapes at `rows` tokens: TFLOP/s of 2 M N K (one logical product)."""
    from euhedral_b200 import layouts, synthetic
    if not gpu.nvfp4_native_available():
        return None
    tensors, flops = [], 0
    for index, (name, n, k) in enumerate(LAYER):
        blob = synthetic.nvfp4_tensor(synthetic.gaussian(n, k, WEIGHT_SEED + index, SIGMA, device="cuda"))
        x = synthetic.bf16_rows(rows, k, ACTIVATION_SEED, device="cuda")
        y = torch.empty((rows, n), dtype=torch.int16, device="cuda")
        tensors.append((blob, x, y, n, k))
        flops += 2 * rows * n * k
    need = max(layouts.activation_bytes(rows, k) for _, _, k in LAYER)
    gpu.native_scratch(need)

    def body(_):
        for blob, x, y, n, k in tensors:
            if not gpu.linear_nvfp4_native_bf16(x.data_ptr(), blob.data_ptr(), y.data_ptr(), rows, k, n, blob.numel()):
                raise RuntimeError("native route declined")

    with torch.cuda.stream(stream), gpu.submit(stream.cuda_stream, pdl=True):
        try:
            seconds = timed(torch, None, 1, steps, warmup, body)
        except RuntimeError:
            return None
    result = {"rows": rows, "tflops": flops * steps / seconds / 1e12, "issued_tflops": 2 * flops * steps / seconds / 1e12,
              "ms_per_step": seconds / steps * 1e3}
    if detail:
        per_shape = {}
        with torch.cuda.stream(stream), gpu.submit(stream.cuda_stream, pdl=True):
            for (name, n, k), item in zip(LAYER, tensors):
                blob, x, y, _, _ = item

                def one(_, item=item):
                    blob, x, y, n, k = item
                    gpu.linear_nvfp4_native_bf16(x.data_ptr(), blob.data_ptr(), y.data_ptr(), rows, k, n, blob.numel())
                t = timed(torch, None, 1, steps, warmup, one)
                per_shape[name] = round(2 * rows * n * k * steps / t / 1e12, 1)
        result["per_shape_tflops"] = per_shape
    return result


# dram__bytes_read.sum + dram__bytes_write.sum of one captured gate launch over its algorithmic bytes (profiles/q3_gemv_gate_m3.md).
Q3_TRAFFIC_RATIO = 36.27 / 36.34


TRELLIS_TARGET_PER_SM = None   # --trellis-target-per-sm: K-split target blocks per SM (kernels.trellis.target-blocks); None = the operator's default


def run_ours(args):
    global TRELLIS_TARGET_PER_SM
    TRELLIS_TARGET_PER_SM = args.trellis_target_per_sm
    os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "8")
    import torch
    dist = None
    world = WORLD
    torch.cuda.set_device(LOCAL_RANK)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", LOCAL_RANK))
    from euhedral_b200.gpu import CudaGpuMemory
    gpu = CudaGpuMemory()   # raises when the CUDA library is missing: no fallback
    sms = gpu.multiprocessor_count()
    stream = torch.cuda.Stream()
    peak, peak_kind = read_peaks()
    copies = 3
    if args.prefill_only:
        r = measure_prefill(torch, gpu, stream, args.steps, args.warmup, rows=args.prefill_only, detail=True)
        if RANK == 0:
            print(json.dumps({"prefill_rows": args.prefill_only, **(r or {"unavailable": True})}))
        return
    if args.only:
        # One matrix alone (profiling and per-shape numbers): FORMAT:NAME:ROWS, e.g. q3:gate:3
        fmt, name, rows = args.only.split(":")
        r = measure_format(torch, dist, gpu, fmt, (int(rows),), 4, world, RANK, sms, args.steps, args.warmup, stream, only=name,
                           graph=args.graph)
        if RANK == 0:
            print(json.dumps({"only": args.only, "gbs": r["gbs"], "frac_of_hbm_peak": r["gbs"] / (peak * world), "us_per_launch_set": r["ms_per_step"] * 1e3,
                              "bytes": r["bytes_per_step"]}))
        return
    with ClockSampler(LOCAL_RANK) as clocks:
        head = measure_format(torch, dist, gpu, "q3", HEADLINE_ROWS, copies, world, RANK, sms, args.steps, args.warmup, stream, e2e=True)
    extra = {}
    if True:
        for fmt, rows_list in (("nvfp4", (1, 5)), ("trellis", (1, 5))):
            try:
                replay = fmt == "trellis" and world == 1
                r = measure_format(torch, dist, gpu, fmt, rows_list, copies, world, RANK, sms, max(3, args.steps // 2), 3, stream, graph=replay)
                extra[fmt] = {"rows": list(rows_list), "gbs": round(r["gbs"], 1), "frac_of_hbm_peak": round(r["gbs"] / (peak * world), 4),
                              "ms_per_step": round(r["ms_per_step"], 4), "launch": "CUDA graph replay" if replay else "eager calls"}
            except Exception as error:   # reported, never hidden
                extra[fmt] = {"error": repr(error)}
        if world == 1:
            try:
                extra["nvfp4_prefill"] = measure_prefill(torch, gpu, stream, 3, 3)
            except Exception as error:
                extra["nvfp4_prefill"] = {"error": repr(error)}
    cpu = None
    if RANK == 0 and world == 1:
        from oracle import oracle_c as OC
        threads = OC.default_threads()
        b, t = cpu_layer_pass(cpu_blobs(), HEADLINE_ROWS, threads)
        cpu = {"value": b / t / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
               "sample": "one whole step (7 matrices x M in {1,3}) on the plain-C restatement, row-parallel threads"}
    if RANK == 0:
        line = {
            "metric": "quantized GEMV algorithmic GB/s (Q3 decode layer set, M=1 and M=3)", "value": head["gbs"], "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "bf16 x int3 -> f32", "data": "synthetic",
            "config": {"workload": "Q3 decode GEMV set, one Qwen-27B-shaped layer, M in {1,3}", "layer": [list(s) for s in LAYER],
                       "weights": "N(0, 0.02^2) seeded, rounded as the converter rounds Q3G64_F16S", "activations": "N(0,1) as BF16",
                       "l2": f"weights rotate over {copies} resident copies of the layer ({copies * head['bytes_per_step'] / 2 / 1e6:.0f} MB > 126 MB L2)",
                       "parallelism": f"n-sharded x{world}, one NCCL all-gather of the step's packed output slices" if world > 1 else "single GPU",
                       "launch": "one C-ABI call per GEMV, one stream, programmatic dependent launch"},
            "roofline": {"bound": "hbm", "achieved": head["gbs"], "peak": peak * world, "unit": "GB/s", "frac": head["gbs"] / (peak * world),
                         "traffic": head["bytes_per_step"] * Q3_TRAFFIC_RATIO, "traffic_unit": "bytes per step",
                         "traffic_note": "ncu dram bytes of the gate launch (36.27 MB read, 36.34 MB algorithmic) scaled to the step's bytes",
                         "peak_kind": f"of {peak_kind}", "kernel": "gemv::kernel<q3::Format, ...> (every launch of the timed region)"},
            "e2e": {"value": head.get("e2e_gbs"), "unit": "GB/s", "h2d_bytes_per_step": head.get("h2d"), "d2h_bytes_per_step": head.get("d2h")},
            "gpu_launches": head["launches_per_step"] * args.steps,
            "clocks": clocks.summary(),
            "extra": extra,
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=30)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--detail", action="store_true")
    parser.add_argument("--prefill-only", type=int, default=0, help="time the NVFP4 prefill GEMM over the layer shapes at this many rows")
    parser.add_argument("--trellis-target-per-sm", type=int, default=None, help="K-split target blocks per SM of the trellis operator")
    parser.add_argument("--graph", action="store_true", help="with --only: replay the calls from a captured CUDA graph")
    parser.add_argument("--only", default=None, help="FORMAT:NAME:ROWS - time one matrix alone, e.g. q3:gate:3")
    args = parser.parse_args()
    if args.impl == "reference":
        args.steps = min(args.steps, 10)
        run_reference(args)
    else:
        args.warmup = max(args.warmup, 3)
        run_ours(args)


if __name__ == "__main__":
    main()
