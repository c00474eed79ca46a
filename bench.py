"""Benchmark of the quantized-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--headline-only]

One GPU (`config.workload`): the Q3 decode GEMV set of one dense Qwen-27B-shaped decoder layer - q 5120x5120, k and v
1024x5120, o 5120x5120, gate and up 17408x5120, down 5120x17408 (N x K) - at M = 1 and M = 3 activation rows. A step is
every GEMV of the set once: per row count one grouped C-ABI call over the six tensors that share K = 5120 and one call
for down, on one stream with programmatic dependent launch, the weights rotated over several resident copies of the
layer so that no step finds its weights in L2. The metric is the algorithmic bytes of the step (weight planes +
activations + outputs, each byte once) per second. `extra` carries the same set through the reference's one-call-per-
tensor entry points, the NVFP4 and trellis layouts, a per-shape table at M = 1..5, the NVFP4 prefill GEMM at 4096, 32768
and 131072 tokens, and the 64-layer NVFP4 sweep (one decode step at M = 5 plus one 32768-token prefill).

With --gpus N (launched under torch.distributed.run) the line's value is the decode step of that 64-layer sweep: every
weight matrix is split along N over the ranks, each rank runs its slices of a layer into one packed buffer, and the
slices of every four layers are joined with one NCCL all-gather that overlaps the next layers' GEMVs; the step is
replayed from a CUDA graph. The total work is fixed
(strong scaling); `extra.sweep64` reports the prefill part and the exchange times.

`--impl reference` times the CPU restatement of the reference's dequant + matmul (oracle/oracle.c) on the host cores.
"""

from __future__ import annotations

import argparse
import ctypes as C
import json
import math
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
L2_BYTES = 126e6
TRELLIS_WIDTH = 48
SWEEP_LAYERS = 64
SWEEP_GATHER = 4            # layers whose output slices travel in one all-gather
SWEEP_DISTINCT = 8          # distinct seeded layers of the sweep; layer i holds its own copy of the bytes of layer i % 8
FP4_NOMINAL_TFLOPS = 9000.0


def read_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm": float(data["hbm_gbs"]), "bf16": float(data.get("bf16_tflops", 0.0)),
                "bf16_sustained": float(data.get("bf16_tflops_sustained", 0.0)), "kind": "measured"}
    return {"hbm": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "kind": "fallback"}


def seeded_weights(index: int, n: int, k: int) -> np.ndarray:
    rng = np.random.default_rng(WEIGHT_SEED + index)
    return rng.standard_normal((n, k), dtype=np.float32) * np.float32(SIGMA)


def seeded_rows(rows: int, k: int) -> np.ndarray:
    from oracle import oracle_np as O
    return O.bf16_bits(np.random.default_rng(ACTIVATION_SEED + rows).standard_normal((rows, k)).astype(np.float32))


def algorithmic_bytes(fmt: str, n: int, k: int, rows: int, w: int = TRELLIS_WIDTH) -> int:
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
# the CPU restatement on the host cores: reference arm and cpu_baseline
# ---------------------------------------------------------------------------------------------------------------------

def cpu_layer_pass(blobs, rows_list, threads, only=None):
    from oracle import oracle_c as OC
    total = 0
    start = time.perf_counter()
    for (name, n, k), blob in zip(LAYER, blobs):
        if only is not None and name not in only:
            continue
        for rows in rows_list:
            OC.q3_linear(seeded_rows(rows, k), blob, n, k, threads=threads)
            total += algorithmic_bytes("q3", n, k, rows)
    return total, time.perf_counter() - start


def cpu_blobs():
    from oracle import oracle_c as OC
    return [OC.q3_quantize(seeded_weights(i, n, k)) for i, (name, n, k) in enumerate(LAYER)]


def cpu_baseline(blobs):
    """The plain-C restatement on every host thread (warmed), on one thread (a bounded sample), and the NumPy
    restatement of the converter's own dequantize + matmul the way a user of the reference's Python tools would run it."""
    from oracle import oracle_c as OC
    from oracle import oracle_np as O
    threads = OC.default_threads()
    cpu_layer_pass(blobs, HEADLINE_ROWS, threads)                      # warm
    b, t = cpu_layer_pass(blobs, HEADLINE_ROWS, threads)
    b1, t1 = cpu_layer_pass(blobs, HEADLINE_ROWS, 1, only=("q",))      # one thread: the q matrix at M = 1 and 3
    n, k = 1024, 5120
    blob = OC.nvfp4_quantize(seeded_weights(1, n, k))
    x = O.bf16_to_f32(seeded_rows(1, k))
    start = time.perf_counter()
    dense = O.nvfp4_dense(blob.tobytes(), n, k)
    middle = time.perf_counter()
    for _ in range(10):
        x @ dense.T
    stop = time.perf_counter()
    numpy_bytes = algorithmic_bytes("nvfp4", n, k, 1)
    return {"value": b / t / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": "one whole warmed step (7 matrices x M in {1,3}) on the plain-C restatement, row-parallel threads",
            "single_thread": {"value": b1 / t1 / 1e9, "unit": "GB/s", "sample": "q 5120x5120 at M = 1 and 3, one thread"},
            "numpy_as_shipped": {"value": numpy_bytes / ((middle - start) + (stop - middle) / 10) / 1e9, "unit": "GB/s",
                                 "dequantize_s": middle - start, "matmul_s": (stop - middle) / 10,
                                 "sample": "NumPy dequantize of an NVFP4 1024x5120 tensor + x @ W.T at M = 1 (the converter's own path)"}}


def run_reference(args):
    """The CPU restatement of the path on all host threads, on the metric and config of the repo's own arm at this N:
    one GPU: the Q3 layer set at M = 1 and 3 (a whole step per step); more: the NVFP4 decode sweep at M = 5, each step a
    bounded sample of it (one of the 64 layers: the seven matrices once)."""
    if RANK != 0:
        return
    from oracle import oracle_c as OC
    threads = OC.default_threads()
    sweep = args.gpus > 1
    if sweep:
        blobs = [OC.nvfp4_quantize(seeded_weights(i, n, k)) for i, (name, n, k) in enumerate(LAYER)]

        def one_pass():
            total, start = 0, time.perf_counter()
            for (name, n, k), blob in zip(LAYER, blobs):
                OC.nvfp4_linear(seeded_rows(5, k), blob, n, k, threads=threads)
                total += algorithmic_bytes("nvfp4", n, k, 5)
            return total, time.perf_counter() - start
    else:
        blobs = cpu_blobs()

        def one_pass():
            return cpu_layer_pass(blobs, HEADLINE_ROWS, threads)
    for _ in range(max(1, min(args.warmup, 3))):
        one_pass()
    total_bytes, total_time = 0, 0.0
    for _ in range(args.steps):
        b, t = one_pass()
        total_bytes += b
        total_time += t
    value = total_bytes / total_time / 1e9
    if sweep:
        metric = "quantized GEMV algorithmic GB/s (NVFP4 64-layer decode sweep, M=5, N-sharded)"
        config = {"workload": "64-layer Qwen-27B-shaped NVFP4 sweep: one decode step at M = 5", "layer": [list(s) for s in LAYER]}
        sample = "one of the 64 layers per step (the rate does not depend on the layer): 7 NVFP4 matrices at M = 5, plain-C dequant + FP32 dot, row-parallel threads"
    else:
        metric = "quantized GEMV algorithmic GB/s (Q3 decode layer set, M=1 and M=3)"
        config = {"workload": "Q3 decode GEMV set, one Qwen-27B-shaped layer, M in {1,3}", "layer": [list(s) for s in LAYER]}
        sample = "the whole step: 7 matrices x M in {1,3}, plain-C dequant + FP32 dot, row-parallel threads"
    line = {
        "impl": "reference", "metric": metric, "value": value,
        "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_time / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------------------------

class Bench:
    def __init__(self, torch, dist, world, rank):
        from euhedral_b200.gpu import CudaGpuMemory
        self.torch, self.dist, self.world, self.rank = torch, dist, world, rank
        self.gpu = CudaGpuMemory()   # raises when the CUDA library is missing: no fallback
        self.lib = self.gpu.lib
        self.sms = self.gpu.multiprocessor_count()
        self.stream = torch.cuda.Stream()
        self.peaks = read_peaks()
        self._converter, self._trellis = None, {}
        self.convert_seconds, self.convert_tiles, self.convert_error = 0.0, 0, 0.0

    def check(self, status):
        if status != 0:
            raise RuntimeError(f"C ABI call failed with status {status}")

    def timed(self, steps, warmup, body):
        """max over ranks of the device time of `steps` calls of body(i), after `warmup` untimed calls."""
        torch = self.torch
        for i in range(warmup):
            body(i)
        torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(torch.cuda.current_stream())
        for i in range(steps):
            body(warmup + i)
        stop.record(torch.cuda.current_stream())
        torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        seconds = start.elapsed_time(stop) / 1e3
        if self.world > 1:
            t = torch.tensor([seconds], device="cuda", dtype=torch.float64)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            seconds = float(t.item())
        return seconds

    def submit(self):
        return self.gpu.submit(self.stream.cuda_stream, pdl=True)

    # ---- tensors ------------------------------------------------------------------------------------------------------
    def weight(self, fmt, index, n, k, first=0, local=None):
        """Device tensors of one weight in `fmt`: rows [first, first + local) of the whole seeded tensor."""
        from euhedral_b200 import sharding, synthetic
        torch = self.torch
        local = n if local is None else local
        if fmt == "trellis":
            return self.trellis_fused([(index, local, k)])
        build, cut = (synthetic.q3_tensor, sharding.q3_rows) if fmt == "q3" else (synthetic.nvfp4_tensor, sharding.nvfp4_rows)
        whole = build(synthetic.gaussian(n, k, WEIGHT_SEED + index, SIGMA, device="cuda"))
        if local == n:
            return (whole,)
        # a shard is cut from the whole tensor (NVFP4's tensor scale is the whole tensor's)
        return (torch.from_numpy(cut(whole.cpu().numpy(), n, k, first, local)).cuda(),)

    def trellis_member(self, index, n, k):
        """The seeded N(0, 0.02^2) weight `index` converted to a trellis object by this build's converter (uncalibrated
        path, 3 bits per weight); converted once per process."""
        from euhedral_b200 import synthetic, trellis_convert
        key = (index, n, k)
        if key not in self._trellis:
            if self._converter is None:
                self._converter = trellis_convert.TrellisConverter("cuda")
            begin = time.perf_counter()
            dense = synthetic.gaussian(n, k, WEIGHT_SEED + index, SIGMA, device="cuda")
            self._trellis[key] = self._converter.quantize(dense, TRELLIS_WIDTH / 16, seed=WEIGHT_SEED + index)
            self.torch.cuda.synchronize()
            self.convert_seconds += time.perf_counter() - begin
            self.convert_tiles += (n // 16) * (k // 16)
            self.convert_error = max(self.convert_error, self._trellis[key].proxy)
        return self._trellis[key]

    def trellis_fused(self, members):
        """(payload, suh [s, k], svh, ends) of the members (index, n, k) side by side along n."""
        from euhedral_b200 import trellis_convert
        return trellis_convert.TrellisConverter.fuse([self.trellis_member(*member) for member in members])

    def rows(self, rows, k):
        from euhedral_b200 import synthetic
        return synthetic.bf16_rows(rows, k, ACTIVATION_SEED + rows, device="cuda")


class LayerSet:
    """One format's layer set on one GPU: `copies` resident copies of every weight tensor, packed activation and output
    buffers on the host (pinned) and the device, and the C-ABI calls of a step in two shapes: one call per tensor (the
    reference's entry points) or one grouped call per row count over the tensors that share K."""

    def __init__(self, bench: Bench, fmt: str, rows_list, copies: int):
        torch = bench.torch
        self.bench, self.fmt, self.rows_list, self.copies = bench, fmt, rows_list, copies
        self.keep = []
        ks = sorted({k for _, _, k in LAYER})
        total_in = sum(rows * k for rows in rows_list for k in ks)
        self.host_in = torch.empty(total_in, dtype=torch.int16).pin_memory()
        self.device_in = torch.empty(total_in, dtype=torch.int16, device="cuda")
        self.inputs, cursor = {}, 0
        for rows in rows_list:
            for k in ks:
                self.host_in[cursor:cursor + rows * k].copy_(bench.rows(rows, k).view(-1).cpu())
                self.inputs[(rows, k)] = self.device_in[cursor:cursor + rows * k]
                cursor += rows * k
        self.device_in.copy_(self.host_in)
        self.h2d = 2 * total_in
        total_out = sum(rows * n for rows in rows_list for _, n, _ in LAYER)
        self.device_out = torch.empty(total_out, dtype=torch.int16, device="cuda")
        self.host_out = torch.empty(total_out, dtype=torch.int16).pin_memory()
        self.d2h = 2 * total_out
        self.outputs, cursor = {}, 0
        for rows in rows_list:
            for name, n, _ in LAYER:
                self.outputs[(rows, name)] = self.device_out[cursor:cursor + rows * n]
                cursor += rows * n
        self.weights = {}      # name -> list over copies of tuples of tensors
        for index, (name, n, k) in enumerate(LAYER):
            first = bench.weight(fmt, index, n, k)
            self.weights[name] = [first] + [tuple(t.clone() for t in first) for _ in range(copies - 1)]
        self.bytes_per_step = sum(algorithmic_bytes(fmt, n, k, rows) for rows in rows_list for _, n, k in LAYER)
        self.scratch = None
        if fmt == "trellis":
            # ... and the layer as the reference's converter stores it: fused objects with one input scale vector per member
            # (query_key_value: three segments; gate_up: two), tools/euhedral_artifacts/trellis.py:128-146.
            self.fused = [("query_key_value", 7168, 5120, 3), ("o", 5120, 5120, 1), ("gate_up", 34816, 5120, 2), ("down", 5120, 17408, 1)]
            members = {"query_key_value": (0, 1, 2), "o": (3,), "gate_up": (4, 5), "down": (6,)}
            self.fused_weights = {}
            for name, _, _, _ in self.fused:
                first = bench.trellis_fused([(i, LAYER[i][1], LAYER[i][2]) for i in members[name]])
                self.fused_weights[name] = [first] + [tuple(t.clone() for t in first) for _ in range(copies - 1)]
            self.fused_out = torch.empty(max(rows_list) * 34816, dtype=torch.int16, device="cuda")
            shapes = [(n, k, 1) for _, n, k in LAYER] + [(n, k, s) for _, n, k, s in self.fused]
            need = max(bench.lib.euhedral_b200_linear_trellis_scratch_bytes(rows, k, n, s, 0) for rows in rows_list for n, k, s in shapes)
            self.scratch = [torch.empty(need, dtype=torch.uint8, device="cuda") for _ in LAYER]
            self.scratch_bytes = need
        self._build_calls()

    def _build_calls(self):
        lib, fmt = self.bench.lib, self.fmt
        self.single, self.grouped = [[] for _ in range(self.copies)], [[] for _ in range(self.copies)]
        for copy in range(self.copies):
            for rows in self.rows_list:
                for position, (name, n, k) in enumerate(LAYER):
                    tensors = self.weights[name][copy]
                    x, y = self.inputs[(rows, k)].data_ptr(), self.outputs[(rows, name)].data_ptr()
                    if fmt == "trellis":
                        payload, suh, svh, ends = tensors
                        args = (x, payload.data_ptr(), suh.data_ptr(), svh.data_ptr(), ends.data_ptr(), y, self.scratch[position].data_ptr(),
                                self.scratch_bytes, rows, k, n, TRELLIS_WIDTH, 1, 0)
                        self.single[copy].append((lib.euhedral_b200_linear_trellis_bf16, args))
                    else:
                        entry = lib.euhedral_cuda_linear_q3_bf16 if fmt == "q3" else lib.euhedral_cuda_linear_nvfp4_bf16
                        self.single[copy].append((entry, (x, tensors[0].data_ptr(), y, rows, k, n, tensors[0].numel())))
                if fmt == "trellis":
                    for position, (name, n, k, segments) in enumerate(self.fused):
                        payload, suh, svh, ends = self.fused_weights[name][copy]
                        self.grouped[copy].append((lib.euhedral_b200_linear_trellis_bf16,
                                                   (self.inputs[(rows, k)].data_ptr(), payload.data_ptr(), suh.data_ptr(), svh.data_ptr(), ends.data_ptr(),
                                                    self.fused_out.data_ptr(), self.scratch[position].data_ptr(), self.scratch_bytes, rows, k, n,
                                                    TRELLIS_WIDTH, segments, 0)))
                    continue
                entry = lib.euhedral_b200_linear_group_q3_bf16 if fmt == "q3" else lib.euhedral_b200_linear_group_nvfp4_bf16
                for k in sorted({k for _, _, k in LAYER}):
                    members = [(name, n) for name, n, kk in LAYER if kk == k]
                    count = len(members)
                    blobs = [self.weights[name][copy][0] for name, _ in members]
                    args = (count, (C.c_void_p * count)(*[self.inputs[(rows, k)].data_ptr()] * count),
                            (C.c_void_p * count)(*[b.data_ptr() for b in blobs]),
                            (C.c_void_p * count)(*[self.outputs[(rows, name)].data_ptr() for name, _ in members]), rows, k,
                            (C.c_uint32 * count)(*[n for _, n in members]), (C.c_uint64 * count)(*[b.numel() for b in blobs]))
                    self.grouped[copy].append((entry, args))

    def step(self, iteration: int, grouped: bool):
        calls = (self.grouped if grouped else self.single)[iteration % self.copies]
        for entry, args in calls:
            status = entry(*args)
            if status != 0:
                raise RuntimeError(f"C ABI call failed with status {status}")

    def step_e2e(self, iteration: int, grouped: bool):
        """The same step fed from pinned host memory: the step's activation tensors are uploaded (one copy of the packed
        buffer) and the step's whole result is read back to pinned memory, all on the step's stream."""
        gpu = self.bench.gpu
        gpu.copy_upload_to_device(self.device_in.data_ptr(), self.host_in.data_ptr(), self.h2d)
        self.step(iteration, grouped)
        gpu.copy_device_to_readback(self.host_out.data_ptr(), self.device_out.data_ptr(), self.d2h)

    def launches(self, grouped: bool):
        return len((self.grouped if grouped else self.single)[0])   # every call is one launch


def measure_layer_set(bench: Bench, fmt, rows_list, copies, steps, warmup, e2e=False):
    torch = bench.torch
    layer = LayerSet(bench, fmt, rows_list, copies)
    result = {"rows": list(rows_list), "bytes_per_step": layer.bytes_per_step}
    with torch.cuda.stream(bench.stream), bench.submit():
        for label, grouped in (("fused_objects" if fmt == "trellis" else "grouped", True), ("single", False)):
            seconds = bench.timed(steps, warmup, lambda i: layer.step(i, grouped))
            gbs = layer.bytes_per_step * steps / seconds / 1e9
            result[label] = {"gbs": gbs, "frac_of_hbm_peak": gbs / bench.peaks["hbm"], "us_per_step": seconds / steps * 1e6,
                             "calls_per_step": len((layer.grouped if grouped else layer.single)[0]), "launches_per_step": layer.launches(grouped)}
        if e2e:
            seconds = bench.timed(steps, warmup, lambda i: layer.step_e2e(i, True))
            result["e2e_gbs"] = layer.bytes_per_step * steps / seconds / 1e9
            result["h2d"], result["d2h"] = layer.h2d, layer.d2h
    assert bench.gpu.take_device_error() == 0, "a kernel's bounded wait gave up"
    if fmt == "trellis":
        result["weights"] = {"source": "N(0, 0.02^2) seeded, converted by this build's trellis converter (uncalibrated path, 3 bits per weight)",
                             "tiles": bench.convert_tiles, "convert_seconds": bench.convert_seconds,
                             "tiles_per_s": bench.convert_tiles / max(bench.convert_seconds, 1e-9),
                             "worst_rounding_mse_rotated": bench.convert_error}
    del layer
    torch.cuda.empty_cache()
    return result


def measure_per_shape(bench: Bench, steps_floor=40):
    """Every distinct layer shape alone, M = 1..5, each format: one C-ABI call per launch, programmatic dependent launch,
    the tensor rotated over enough copies to exceed the L2 two and a half times."""
    torch, lib = bench.torch, bench.lib
    distinct = {"q": ("q", "o"), "k": ("k", "v"), "gate": ("gate", "up"), "down": ("down",),
                "query_key_value": ("query_key_value",), "gate_up": ("gate_up",)}
    # ... and the fused objects the reference's converter emits and its host calls as one tensor
    shapes = list(LAYER) + [("query_key_value", 7168, 5120), ("gate_up", 34816, 5120)]
    table = {}
    for fmt in ("nvfp4", "q3", "trellis"):
        for index, (name, n, k) in enumerate(shapes):
            if name not in distinct:
                continue
            members = {"query_key_value": (0, 1, 2), "gate_up": (4, 5)}.get(name)
            if fmt == "trellis" and members:      # the converter's fused objects: the members side by side
                first = bench.trellis_fused([(i, LAYER[i][1], LAYER[i][2]) for i in members])
            else:
                first = bench.weight(fmt, index, n, k)
            size = sum(t.numel() * t.element_size() for t in first)
            copies = int(min(128, max(3, math.ceil(2.5 * L2_BYTES / size) + 1)))
            tensors = [first] + [tuple(t.clone() for t in first) for _ in range(copies - 1)]
            scratch = None
            if fmt == "trellis":
                segments = first[3].numel()
                need = lib.euhedral_b200_linear_trellis_scratch_bytes(5, k, n, segments, 0)
                scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
            for rows in (1, 2, 3, 4, 5):
                x = bench.rows(rows, k)
                y = torch.empty(rows * n, dtype=torch.int16, device="cuda")

                def body(i):
                    t = tensors[i % copies]
                    if fmt == "trellis":
                        bench.check(lib.euhedral_b200_linear_trellis_bf16(x.data_ptr(), t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr(), t[3].data_ptr(),
                                                                           y.data_ptr(), scratch.data_ptr(), need, rows, k, n, TRELLIS_WIDTH, segments, 0))
                    elif fmt == "q3":
                        bench.check(lib.euhedral_cuda_linear_q3_bf16(x.data_ptr(), t[0].data_ptr(), y.data_ptr(), rows, k, n, t[0].numel()))
                    else:
                        bench.check(lib.euhedral_cuda_linear_nvfp4_bf16(x.data_ptr(), t[0].data_ptr(), y.data_ptr(), rows, k, n, t[0].numel()))

                launches = max(steps_floor, 2 * copies)
                with torch.cuda.stream(bench.stream), bench.submit():
                    seconds = bench.timed(launches, copies, body)
                us = seconds / launches * 1e6
                gbs = algorithmic_bytes(fmt, n, k, rows) / us / 1e3
                for alias in distinct[name]:
                    table[f"{fmt}:{alias}:{rows}"] = [round(us, 2), round(gbs, 1), round(gbs / bench.peaks["hbm"], 4)]
            del tensors, first
            torch.cuda.empty_cache()
    return {"columns": ["us per launch", "GB/s", "fraction of HBM peak"], "note": "key = format:shape:M; trellis at 48 words per tile",
            "rows": table}


def measure_prefill(bench: Bench, rows, steps, warmup):
    """NVFP4 prefill GEMM over the seven layer shapes at `rows` tokens through the reference's native entry point
    (quantize + scale repack + GEMM per call): TFLOP/s of 2 M N K (one logical product; the kernel issues one MMA per
    activation term, twice that)."""
    from euhedral_b200 import layouts, synthetic
    torch, gpu, lib = bench.torch, bench.gpu, bench.lib
    if not gpu.nvfp4_native_available():
        return None
    tensors, flops, xs = [], 0, {}
    for index, (name, n, k) in enumerate(LAYER):
        blob = bench.weight("nvfp4", index, n, k)[0]
        if k not in xs:
            xs[k] = torch.randn((rows, k), device="cuda", dtype=torch.bfloat16, generator=torch.Generator(device="cuda").manual_seed(ACTIVATION_SEED)).view(torch.int16)
        tensors.append((blob, xs[k], n, k))
        flops += 2 * rows * n * k
    y = torch.empty((rows, max(n for _, n, _ in LAYER)), dtype=torch.int16, device="cuda")
    need = max(lib.euhedral_cuda_nvfp4_native_scratch_bytes(rows, k, n) for _, n, k in LAYER)
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")

    def body(_):
        for blob, x, n, k in tensors:
            bench.check(lib.euhedral_cuda_linear_nvfp4_native_bf16(x.data_ptr(), blob.data_ptr(), y.data_ptr(), scratch.data_ptr(), rows, k, n, blob.numel(), need))

    def quantize_only(_):
        for blob, x, n, k in tensors:
            bench.check(lib.euhedral_b200_nvfp4_native_quantize(x.data_ptr(), scratch.data_ptr(), rows, k, need))

    # The same layer as the reference's host calls it: the fused objects its converter emits (query_key_value as one tensor
    # of 7168 rows, gate_up as one of 34816 rows through the paired SwiGLU region), four calls instead of seven.
    x5, x17 = xs[5120], xs[17408]
    fused = [(lib.euhedral_cuda_linear_nvfp4_native_bf16, bench.weight("nvfp4", 16, 7168, 5120)[0], x5, 7168, 5120),
             (lib.euhedral_cuda_linear_nvfp4_native_bf16, tensors[3][0], x5, 5120, 5120),
             (lib.euhedral_cuda_nvfp4_native_gate_up_swiglu_bf16, bench.weight("nvfp4", 17, 34816, 5120)[0], x5, 34816, 5120),
             (lib.euhedral_cuda_linear_nvfp4_native_bf16, tensors[6][0], x17, 5120, 17408)]
    fused_need = max(lib.euhedral_cuda_nvfp4_native_scratch_bytes(rows, k, n) for _, _, _, n, k in fused)
    fused_scratch = torch.empty(fused_need, dtype=torch.uint8, device="cuda")

    def fused_body(_):
        for entry, blob, x, n, k in fused:
            bench.check(entry(x.data_ptr(), blob.data_ptr(), y.data_ptr(), fused_scratch.data_ptr(), rows, k, n, blob.numel(), fused_need))

    with torch.cuda.stream(bench.stream), bench.submit():
        seconds = bench.timed(steps, warmup, body)
        quantize_seconds = bench.timed(steps, 1, quantize_only)
        fused_seconds = bench.timed(steps, 1, fused_body)
    issued = 2 * flops * steps / seconds / 1e12
    result = {"rows": rows, "tflops": flops * steps / seconds / 1e12, "issued_tflops": issued, "ms_per_layer": seconds / steps * 1e3,
              "quantize_ms_per_layer": quantize_seconds / steps * 1e3, "quantize_share": quantize_seconds / seconds,
              "fused_objects": {"calls": "query_key_value 7168x5120, o, gate_up 34816x5120 with SwiGLU in the epilogue, down",
                                "ms_per_layer": fused_seconds / steps * 1e3, "issued_tflops": 2 * flops * steps / fused_seconds / 1e12,
                                "frac_of_nominal_fp4": 2 * flops * steps / fused_seconds / 1e12 / FP4_NOMINAL_TFLOPS},
              "roofline": {"bound": "tensor", "achieved": issued, "algorithmic": flops * steps / seconds / 1e12, "peak": FP4_NOMINAL_TFLOPS,
                           "unit": "TFLOP/s", "frac": issued / FP4_NOMINAL_TFLOPS,
                           "peak_kind": "nominal dense FP4 (MEASURED_PEAKS.json has no FP4 figure)",
                           "algorithmic_over_measured_bf16_burst": flops * steps / seconds / 1e12 / bench.peaks["bf16"] if bench.peaks["bf16"] else None,
                           "note": "achieved = issued FLOP (two activation terms); algorithmic = 2 M N K"}}
    assert gpu.take_device_error() == 0
    del tensors, xs, y, scratch, fused, fused_scratch
    torch.cuda.empty_cache()
    return result


def measure_trellis_prefill(bench: Bench, rows, steps, warmup):
    """Trellis prefill of the layer's four fused objects at `rows` tokens through the one-call entry (rotate, decode to BF16,
    tcgen05 BF16 linear per segment with the rotate-back in its epilogue): TFLOP/s of 2 M N K against the measured BF16
    peak; and the BF16 linear alone on the decoded weight of the largest object."""
    torch, gpu, lib = bench.torch, bench.gpu, bench.lib
    objects = [("query_key_value", (0, 1, 2), 7168, 5120), ("o", (3,), 5120, 5120), ("gate_up", (4, 5), 34816, 5120), ("down", (6,), 5120, 17408)]
    xs, calls, flops = {}, [], 0
    need = max(lib.euhedral_b200_prefill_trellis_scratch_bytes(rows, k, n, len(members)) for _, members, n, k in objects)
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    y = torch.empty((rows, 34816), dtype=torch.int16, device="cuda")
    keep = []
    for name, members, n, k in objects:
        payload, suh, svh, ends = bench.trellis_fused([(i, LAYER[i][1], LAYER[i][2]) for i in members])
        if k not in xs:
            xs[k] = torch.randn((rows, k), device="cuda", dtype=torch.bfloat16, generator=torch.Generator(device="cuda").manual_seed(ACTIVATION_SEED)).view(torch.int16)
        host_ends = (C.c_int32 * len(members))(*ends.tolist())
        keep.append((payload, suh, svh, ends, host_ends))
        calls.append((xs[k].data_ptr(), payload.data_ptr(), suh.data_ptr(), svh.data_ptr(), ends.data_ptr(), C.cast(host_ends, C.c_void_p), y.data_ptr(),
                      scratch.data_ptr(), need, rows, k, n, TRELLIS_WIDTH, len(members)))
        flops += 2 * rows * n * k

    def body(_):
        for args in calls:
            bench.check(lib.euhedral_b200_prefill_trellis_bf16(*args))

    # the BF16 linear alone, on the weight the gate_up call just decoded into the scratch (4096 x 34816 x 5120)
    decoded = scratch.data_ptr() + ((2 * rows * 5120 * 2 + 255) // 256) * 256

    def linear_alone(_):
        bench.check(lib.euhedral_b200_linear_bf16(xs[5120].data_ptr(), decoded, y.data_ptr(), rows, 5120, 34816))

    with torch.cuda.stream(bench.stream), bench.submit():
        seconds = bench.timed(steps, warmup, body)
        bench.check(lib.euhedral_b200_prefill_trellis_bf16(*calls[2]))
        linear_seconds = bench.timed(steps, 1, linear_alone)
    assert gpu.take_device_error() == 0
    tflops, alone = flops * steps / seconds / 1e12, 2 * rows * 34816 * 5120 * steps / linear_seconds / 1e12
    peak = bench.peaks["bf16"]
    result = {"rows": rows, "calls": "query_key_value 7168x5120 (3 segments), o, gate_up 34816x5120 (2 segments), down; 3 bits per weight",
              "ms_per_layer": seconds / steps * 1e3, "tflops": tflops,
              "bf16_linear_alone": {"shape": f"{rows} x 34816 x 5120", "ms": linear_seconds / steps * 1e3, "tflops": alone,
                                    "frac_of_measured_bf16": alone / peak if peak else None,
                                    "frac_of_sustained_bf16": alone / bench.peaks["bf16_sustained"] if bench.peaks["bf16_sustained"] else None},
              "roofline": {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s", "frac": tflops / peak if peak else None,
                           "peak_kind": f"of {bench.peaks['kind']} (cuBLAS BF16 burst)",
                           "frac_of_sustained": tflops / bench.peaks["bf16_sustained"] if bench.peaks["bf16_sustained"] else None,
                           "note": "2 M N K over the whole call: the rotate and the decode of the payload to BF16 run before the GEMM and count as time, not as FLOP; "
                                   "back-to-back millisecond launches run under the power cap, where cuBLAS sustains bf16_tflops_sustained"}}
    del keep, calls, scratch, y, xs
    torch.cuda.empty_cache()
    return result


def measure_q3_prefill(bench: Bench, rows, steps, warmup):
    """Q3 prefill of the layer at `rows` tokens through the reference's Q3 MX entry points (two exact BF16 terms per weight
    written to the scratch, one tcgen05 BF16 GEMM over both): TFLOP/s of 2 M N K; the GEMM issues twice that."""
    torch, gpu, lib = bench.torch, bench.gpu, bench.lib
    tensors, flops, xs = [], 0, {}
    for index, (name, n, k) in enumerate(LAYER):
        blob = bench.weight("q3", index, n, k)[0]
        if k not in xs:
            xs[k] = torch.randn((rows, k), device="cuda", dtype=torch.bfloat16, generator=torch.Generator(device="cuda").manual_seed(ACTIVATION_SEED)).view(torch.int16)
        tensors.append((blob, xs[k], n, k))
        flops += 2 * rows * n * k
    need = max(lib.euhedral_cuda_q3_mx_scratch_bytes(rows, k, n) for _, n, k in LAYER)
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    y = torch.empty((rows, max(n for _, n, _ in LAYER)), dtype=torch.int16, device="cuda")

    def body(_):
        for blob, x, n, k in tensors:
            bench.check(lib.euhedral_cuda_linear_q3_mx_bf16(x.data_ptr(), blob.data_ptr(), y.data_ptr(), scratch.data_ptr(), rows, k, n, blob.numel(), need))

    with torch.cuda.stream(bench.stream), bench.submit():
        seconds = bench.timed(steps, warmup, body)
    assert gpu.take_device_error() == 0
    tflops, peak = flops * steps / seconds / 1e12, bench.peaks["bf16"]
    result = {"rows": rows, "ms_per_layer": seconds / steps * 1e3, "tflops": tflops, "issued_tflops": 2 * tflops,
              "roofline": {"bound": "tensor", "achieved": 2 * tflops, "algorithmic": tflops, "peak": peak, "unit": "TFLOP/s",
                           "frac": 2 * tflops / peak if peak else None, "peak_kind": f"of {bench.peaks['kind']} (cuBLAS BF16 burst)",
                           "frac_of_sustained": 2 * tflops / bench.peaks["bf16_sustained"] if bench.peaks["bf16_sustained"] else None,
                           "note": "achieved = issued FLOP (two BF16 terms per weight); algorithmic = 2 M N K; the expansion of the codes runs before the GEMM and counts as time"}}
    del tensors, xs, y, scratch
    torch.cuda.empty_cache()
    return result


class Sweep:
    """The 64-layer NVFP4 sweep, N-sharded: every rank holds rows [g N / G, (g + 1) N / G) of every matrix of every layer."""

    def __init__(self, bench: Bench, prefill_rows=32768, decode_rows=5):
        from euhedral_b200 import sharding
        torch, world, rank = bench.torch, bench.world, bench.rank
        self.bench, self.decode_rows, self.prefill_rows = bench, decode_rows, prefill_rows
        self.shards = [sharding.shard_range(n, world, rank, 16) for _, n, _ in LAYER]
        distinct = []
        for layer in range(SWEEP_DISTINCT):
            distinct.append([bench.weight("nvfp4", 7 * layer + i, n, k, *self.shards[i])[0] for i, (_, n, k) in enumerate(LAYER)])
        self.layers = [distinct[i] if i < SWEEP_DISTINCT else [t.clone() for t in distinct[i % SWEEP_DISTINCT]] for i in range(SWEEP_LAYERS)]
        self.x = {k: bench.rows(decode_rows, k) for k in sorted({k for _, _, k in LAYER})}
        # The output slices of SWEEP_GATHER consecutive layers share one packed buffer and travel in one all-gather.
        self.layer_outputs = decode_rows * sum(local for _, local in self.shards)
        self.slot_count = 4
        self.packed = [torch.empty(SWEEP_GATHER * self.layer_outputs, dtype=torch.int16, device="cuda") for _ in range(self.slot_count)]
        self.gathered = [torch.empty(world * SWEEP_GATHER * self.layer_outputs, dtype=torch.int16, device="cuda") for _ in range(self.slot_count)] if world > 1 else self.packed
        self.comm = torch.cuda.Stream()
        self.events = [torch.cuda.Event() for _ in range(self.slot_count)]
        self.done = [torch.cuda.Event() for _ in range(self.slot_count)]
        self.decode_bytes = SWEEP_LAYERS * sum(algorithmic_bytes("nvfp4", local, k, decode_rows) for (_, _, k), (_, local) in zip(LAYER, self.shards))
        self.prefill_flops = SWEEP_LAYERS * sum(2 * prefill_rows * local * k for (_, _, k), (_, local) in zip(LAYER, self.shards))
        self._calls = {}

    def decode_calls(self, layer):
        """The two grouped C-ABI calls of a layer (K = 5120: six tensors; K = 17408: down), writing into the layer's place
        in its gather group's packed buffer."""
        if layer not in self._calls:
            lib, rows = self.bench.lib, self.decode_rows
            slot, place = (layer // SWEEP_GATHER) % self.slot_count, layer % SWEEP_GATHER
            calls, cursor = [], place * self.layer_outputs
            outputs = []
            for (_, _, k), (_, local) in zip(LAYER, self.shards):
                outputs.append(self.packed[slot][cursor:cursor + rows * local].data_ptr())
                cursor += rows * local
            for k in sorted({k for _, _, k in LAYER}):
                members = [i for i, (_, _, kk) in enumerate(LAYER) if kk == k]
                count = len(members)
                blobs = [self.layers[layer][i] for i in members]
                calls.append((count, (C.c_void_p * count)(*[self.x[k].data_ptr()] * count), (C.c_void_p * count)(*[b.data_ptr() for b in blobs]),
                              (C.c_void_p * count)(*[outputs[i] for i in members]), rows, k, (C.c_uint32 * count)(*[self.shards[i][1] for i in members]),
                              (C.c_uint64 * count)(*[b.numel() for b in blobs])))
            self._calls[layer] = calls
        return self._calls[layer]

    def decode_step(self, _):
        """One decode step over the 64 layers: two grouped calls per layer; the packed output slices of every
        SWEEP_GATHER layers are joined by one all-gather on a second stream while the next layers' GEMVs run."""
        from euhedral_b200 import sharding
        torch, bench = self.bench.torch, self.bench
        main = torch.cuda.current_stream()
        for layer in range(SWEEP_LAYERS):
            slot = (layer // SWEEP_GATHER) % self.slot_count
            if bench.world > 1 and layer % SWEEP_GATHER == 0 and layer >= SWEEP_GATHER * self.slot_count:
                main.wait_event(self.done[slot])    # the gather that last read this slot's packed buffer has finished
            for args in self.decode_calls(layer):
                bench.check(bench.lib.euhedral_b200_linear_group_nvfp4_bf16(*args))
            if bench.world > 1 and layer % SWEEP_GATHER == SWEEP_GATHER - 1:
                self.events[slot].record(main)
                with torch.cuda.stream(self.comm):
                    self.comm.wait_event(self.events[slot])
                    sharding.gather_packed(self.packed[slot], self.gathered[slot])
                    self.done[slot].record(self.comm)
        if bench.world > 1:
            for slot in range(self.slot_count):
                main.wait_event(self.done[slot])

    def captured_step(self):
        """The same step recorded once into a CUDA graph (plain stream capture of the same C-ABI calls and collectives) and
        replayed: what the reference's host does with decode steps (docs/kernels/CUDA_GRAPHS.md), and the only way the
        host keeps up with 128 launches of a few microseconds each."""
        torch, bench = self.bench.torch, self.bench
        for _ in range(2):
            self.decode_step(0)   # plans, tensor maps and the collective's buffers are made before the capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=bench.stream):
            self.decode_step(0)
        return graph

    def exchange_only(self, _):
        """The step's all-gathers alone, back to back on the step's stream."""
        from euhedral_b200 import sharding
        for group in range(SWEEP_LAYERS // SWEEP_GATHER):
            slot = group % self.slot_count
            sharding.gather_packed(self.packed[slot], self.gathered[slot])

    def check_against_one_gpu(self):
        """Layer 0's gathered decode output equals, bit for bit, what one GPU computes from the whole tensors."""
        from euhedral_b200 import sharding, synthetic
        torch, bench, rows = self.bench.torch, self.bench, self.decode_rows
        with torch.cuda.stream(bench.stream), bench.submit():
            for args in self.decode_calls(0):
                bench.check(bench.lib.euhedral_b200_linear_group_nvfp4_bf16(*args))
            if bench.world > 1:
                sharding.gather_packed(self.packed[0], self.gathered[0])
        torch.cuda.synchronize()
        if bench.rank != 0:
            return True
        pieces = self.gathered[0].view(bench.world, -1)
        cursor, same = 0, True
        for i, (name, n, k) in enumerate(LAYER):
            local = self.shards[i][1]
            got = torch.cat([pieces[g, cursor:cursor + rows * local].view(rows, local) for g in range(bench.world)], dim=1)
            cursor += rows * local
            whole = synthetic.nvfp4_tensor(synthetic.gaussian(n, k, WEIGHT_SEED + i, SIGMA, device="cuda"))
            y = torch.empty((rows, n), dtype=torch.int16, device="cuda")
            torch.cuda.synchronize()
            bench.check(bench.lib.euhedral_cuda_linear_nvfp4_bf16(self.x[k].data_ptr(), whole.data_ptr(), y.data_ptr(), rows, k, n, whole.numel()))
            torch.cuda.synchronize()
            same = same and bool(torch.equal(got, y))
            del whole
        return same

    def prefill(self, steps, warmup):
        """One 32768-token prefill over the 64 layers: per matrix the native call on this rank's slice, then an all-gather
        of the [M, N / G] output slices on a second stream, overlapped with the next matrix."""
        from euhedral_b200 import sharding
        torch, bench, rows = self.bench.torch, self.bench, self.prefill_rows
        lib = bench.lib
        if not bench.gpu.nvfp4_native_available():
            return None
        xs = {k: torch.randn((rows, k), device="cuda", dtype=torch.bfloat16, generator=torch.Generator(device="cuda").manual_seed(ACTIVATION_SEED)).view(torch.int16)
              for k in sorted({k for _, _, k in LAYER})}
        widest = max(local for _, local in self.shards)
        ys = [torch.empty(rows * widest, dtype=torch.int16, device="cuda") for _ in range(2)]
        gathered = [torch.empty(bench.world * rows * widest, dtype=torch.int16, device="cuda") for _ in range(2)] if bench.world > 1 else None
        need = max(lib.euhedral_cuda_nvfp4_native_scratch_bytes(rows, k, local) for (_, _, k), (_, local) in zip(LAYER, self.shards))
        scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
        ready = [torch.cuda.Event() for _ in range(2)]
        free = [torch.cuda.Event() for _ in range(2)]

        def body(_, exchange=True):
            main = torch.cuda.current_stream()
            turn = 0
            for layer in range(SWEEP_LAYERS):
                for i, (_, _, k) in enumerate(LAYER):
                    local = self.shards[i][1]
                    blob = self.layers[layer][i]
                    slot = turn % 2
                    turn += 1
                    if bench.world > 1 and exchange:
                        main.wait_event(free[slot])
                    bench.check(lib.euhedral_cuda_linear_nvfp4_native_bf16(xs[k].data_ptr(), blob.data_ptr(), ys[slot].data_ptr(), scratch.data_ptr(), rows, k,
                                                                            local, blob.numel(), need))
                    if bench.world > 1 and exchange:
                        ready[slot].record(main)
                        with torch.cuda.stream(self.comm):
                            self.comm.wait_event(ready[slot])
                            count = rows * local
                            sharding.gather_packed(ys[slot][:count], gathered[slot][:bench.world * count])
                            free[slot].record(self.comm)
            if bench.world > 1 and exchange:
                for slot in range(2):
                    main.wait_event(free[slot])

        with torch.cuda.stream(bench.stream), bench.submit():
            seconds = bench.timed(steps, warmup, body)
            compute_seconds = bench.timed(steps, 0, lambda i: body(i, exchange=False)) if bench.world > 1 else seconds
        flops = self.prefill_flops
        if bench.world > 1:
            t = torch.tensor([float(flops)], device="cuda", dtype=torch.float64)
            bench.dist.all_reduce(t)
            flops = float(t.item())
        gathered_bytes = SWEEP_LAYERS * sum(2 * rows * n for _, n, _ in LAYER) if bench.world > 1 else 0
        return {"rows": rows, "tflops": flops * steps / seconds / 1e12, "issued_tflops": 2 * flops * steps / seconds / 1e12, "ms_per_step": seconds / steps * 1e3,
                "ms_per_step_without_exchange": compute_seconds / steps * 1e3, "all_gather_bytes_per_step": gathered_bytes,
                "frac_of_nominal_fp4": 2 * flops * steps / seconds / 1e12 / (FP4_NOMINAL_TFLOPS * bench.world)}


def measure_sweep(bench: Bench, steps, warmup, prefill=True):
    torch = bench.torch
    sweep = Sweep(bench)
    same = sweep.check_against_one_gpu()
    with torch.cuda.stream(bench.stream), bench.submit():
        eager_seconds = bench.timed(max(2, steps // 3), 2, sweep.decode_step)
        graph = sweep.captured_step()
        seconds = bench.timed(steps, warmup, lambda _: graph.replay())
        exchange = bench.timed(steps, 1, sweep.exchange_only) if bench.world > 1 else 0.0
        # End to end: the step's activations come from pinned host memory and the outputs of the step's last gather group
        # (every rank's slices of its last four layers) go back to pinned host memory, on the step's stream.
        host_x = {k: x.cpu().pin_memory() for k, x in sweep.x.items()}
        last = sweep.gathered[(SWEEP_LAYERS // SWEEP_GATHER - 1) % sweep.slot_count]
        host_out = torch.empty(last.shape, dtype=last.dtype).pin_memory()

        def end_to_end(_):
            for k, x in sweep.x.items():
                x.copy_(host_x[k], non_blocking=True)
            graph.replay()
            host_out.copy_(last, non_blocking=True)

        e2e_seconds = bench.timed(steps, warmup, end_to_end)
    total = float(sweep.decode_bytes)
    if bench.world > 1:
        t = torch.tensor([total], device="cuda", dtype=torch.float64)
        bench.dist.all_reduce(t)
        total = float(t.item())
    gbs = total * steps / seconds / 1e9
    result = {"layers": SWEEP_LAYERS, "decode_rows": sweep.decode_rows, "decode_gbs": gbs, "decode_frac_of_hbm_peak": gbs / (bench.peaks["hbm"] * bench.world),
              "decode_ms_per_step": seconds / steps * 1e3, "decode_bytes_per_step": total, "decode_calls_per_step": 2 * SWEEP_LAYERS,
              "decode_launch": "the step replayed from a CUDA graph captured over the same C-ABI calls and collectives",
              "decode_ms_per_step_eager_calls": eager_seconds / max(2, steps // 3) * 1e3,
              "all_gather_ms_per_step_alone": exchange / steps * 1e3 if bench.world > 1 else 0.0,
              "all_gathers_per_step": SWEEP_LAYERS // SWEEP_GATHER if bench.world > 1 else 0,
              "e2e_gbs": total * steps / e2e_seconds / 1e9, "e2e_h2d_bytes_per_step": sum(x.numel() * 2 for x in host_x.values()),
              "e2e_d2h_bytes_per_step": host_out.numel() * 2,
              "gathered_equals_one_gpu_bitwise": same,
              "weights": f"{SWEEP_DISTINCT} distinct seeded layers, every one of the {SWEEP_LAYERS} layers in memory of its own"}
    if prefill:
        try:
            result["prefill"] = sweep.prefill(max(1, min(steps, 2)), 1)
        except Exception as error:   # reported, never hidden
            result["prefill"] = {"error": repr(error)}
    assert bench.gpu.take_device_error() == 0
    del sweep
    torch.cuda.empty_cache()
    return result


def run_ours(args):
    os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "8")
    import torch
    dist = None
    world = WORLD
    torch.cuda.set_device(LOCAL_RANK)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", LOCAL_RANK))
    bench = Bench(torch, dist, world, RANK)
    peak = bench.peaks["hbm"]
    copies = 3
    extra = {}
    line = {"n_gpus": world, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "data": "synthetic", "unit": "GB/s"}
    if world == 1:
        with ClockSampler(LOCAL_RANK) as clocks:
            head = measure_layer_set(bench, "q3", HEADLINE_ROWS, copies, args.steps, args.warmup, e2e=True)
        grouped = head["grouped"]
        line.update({
            "metric": "quantized GEMV algorithmic GB/s (Q3 decode layer set, M=1 and M=3)", "value": grouped["gbs"],
            "ms_per_step": grouped["us_per_step"] / 1e3, "dtype": "bf16 x int3 -> f32",
            "config": {"workload": "Q3 decode GEMV set, one Qwen-27B-shaped layer, M in {1,3}", "layer": [list(s) for s in LAYER],
                       "weights": "N(0, 0.02^2) seeded, rounded as the converter rounds Q3G64_F16S", "activations": "N(0,1) as BF16",
                       "l2": f"weights rotate over {copies} resident copies of the layer ({copies * head['bytes_per_step'] / 2 / 1e6:.0f} MB > 126 MB L2)",
                       "parallelism": "single GPU",
                       "launch": "per row count one grouped C-ABI call over the six K = 5120 tensors and one call for down: 4 calls per step, "
                                 "one stream, programmatic dependent launch"},
            "roofline": {"bound": "hbm", "achieved": grouped["gbs"], "peak": peak, "unit": "GB/s", "frac": grouped["gbs"] / peak,
                         "traffic": None, "traffic_note": "per-launch DRAM bytes of the dominant kernel are in the ncu summary under profiles/ "
                                                           "(dram__bytes_read.sum equals the algorithmic bytes of the launch within 0.1 %)",
                         "peak_kind": f"of {bench.peaks['kind']}", "kernel": "gemv::kernel<q3::Format, 5, true> (every launch of the timed region)"},
            "e2e": {"value": head.get("e2e_gbs"), "unit": "GB/s", "h2d_bytes_per_step": head.get("h2d"), "d2h_bytes_per_step": head.get("d2h"),
                    "note": "per step: the activations uploaded from pinned host memory, the four C-ABI calls, every result read back to pinned "
                            "memory, all on one stream (the same step recorded by stream capture and replayed measured the same)"},
            "gpu_launches": grouped["launches_per_step"] * args.steps,
        })
        extra["q3_one_call_per_tensor"] = head["single"]
        wanted = set() if args.headline_only else {name.strip() for name in args.extras.split(",") if name.strip()}
        if wanted:
            for fmt, rows_list in (("nvfp4", (1, 5)), ("trellis", (1, 5))):
                if fmt not in wanted:
                    continue
                try:
                    extra[fmt] = measure_layer_set(bench, fmt, rows_list, copies, max(3, args.steps // 2), 3)
                except Exception as error:   # reported, never hidden
                    extra[fmt] = {"error": repr(error)}
            if "per_shape" in wanted:
                try:
                    extra["per_shape"] = measure_per_shape(bench)
                    key = "nvfp4:gate:1"
                    extra["config1_nvfp4_gate_m1"] = dict(zip(("us", "gbs", "frac_of_hbm_peak"), extra["per_shape"]["rows"][key]))
                except Exception as error:
                    extra["per_shape"] = {"error": repr(error)}
            if "prefill" in wanted:
                try:
                    extra["q3_prefill"] = measure_q3_prefill(bench, 4096, 4, 2)
                except Exception as error:
                    extra["q3_prefill"] = {"error": repr(error)}
            if "trellis" in wanted and "prefill" in wanted:
                try:
                    extra["trellis_prefill"] = measure_trellis_prefill(bench, 4096, 4, 2)
                except Exception as error:
                    extra["trellis_prefill"] = {"error": repr(error)}
            if "prefill" in wanted:
                extra["nvfp4_prefill"] = {}
                for rows in (4096, 32768, 131072):
                    try:
                        extra["nvfp4_prefill"][str(rows)] = measure_prefill(bench, rows, 3, 3 if rows < 100000 else 1)
                    except Exception as error:
                        extra["nvfp4_prefill"][str(rows)] = {"error": repr(error)}
            if "sweep64" in wanted:
                try:
                    extra["sweep64"] = measure_sweep(bench, 3, 2)
                except Exception as error:
                    extra["sweep64"] = {"error": repr(error)}
        if RANK == 0:
            line["cpu_baseline"] = cpu_baseline(cpu_blobs())
    else:
        with ClockSampler(LOCAL_RANK) as clocks:
            sweep = measure_sweep(bench, args.steps, args.warmup, prefill=not args.headline_only)
        line.update({
            "metric": "quantized GEMV algorithmic GB/s (NVFP4 64-layer decode sweep, M=5, N-sharded)", "value": sweep["decode_gbs"],
            "ms_per_step": sweep["decode_ms_per_step"], "dtype": "bf16 x e2m1 x e4m3 -> f32",
            "config": {"workload": "64-layer Qwen-27B-shaped NVFP4 sweep: one decode step at M = 5 (value) plus one 32768-token prefill (extra)",
                       "layer": [list(s) for s in LAYER], "weights": "N(0, 0.02^2) seeded, rounded as the converter rounds NVFP4",
                       "activations": "N(0,1) as BF16",
                       "l2": f"{sweep['decode_bytes_per_step'] / world / 1e6:.0f} MB of weights per rank and step, each byte read once",
                       "parallelism": f"every matrix N-sharded x{world}; one NCCL all-gather of the packed output slices of every {SWEEP_GATHER} layers, "
                                      "overlapped with the next layers' GEMVs on a second stream",
                       "launch": "two grouped C-ABI calls per layer with programmatic dependent launch, the whole step replayed from a CUDA graph"},
            "roofline": {"bound": "hbm", "achieved": sweep["decode_gbs"], "peak": peak * world, "unit": "GB/s", "frac": sweep["decode_gbs"] / (peak * world),
                         "traffic": None, "peak_kind": f"of {bench.peaks['kind']}", "kernel": "gemv::kernel<nvfp4::Format, 3, true>"},
            "e2e": {"value": sweep["e2e_gbs"], "unit": "GB/s", "h2d_bytes_per_step": sweep["e2e_h2d_bytes_per_step"],
                    "d2h_bytes_per_step": sweep["e2e_d2h_bytes_per_step"],
                    "note": "per rank and step: the activations uploaded from pinned host memory, the graph replayed, the gathered outputs "
                            "of the last four layers read back to pinned host memory"},
            "gpu_launches": sweep["decode_calls_per_step"] * args.steps,
        })
        extra["sweep64"] = sweep
    if RANK == 0:
        line["clocks"] = clocks.summary()
        line["extra"] = extra
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
    parser.add_argument("--headline-only", action="store_true", help="skip the measurements reported under `extra`")
    parser.add_argument("--extras", default="nvfp4,trellis,per_shape,prefill,sweep64",
                        help="comma-separated measurements to report under `extra` on one GPU (default: all of nvfp4, trellis, per_shape, prefill, sweep64)")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        args.warmup = max(args.warmup, 3)
        run_ours(args)


if __name__ == "__main__":
    main()
