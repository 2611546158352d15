"""Benchmark of the decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl reference]

Workload (N = 1): the Qwen3-8B Q4_K_M-shaped dense decode chain — 36 layers of
q/k/v/o, fused gate/up + SwiGLU and down projections plus the 4096 x 151936
output head, random Q4_K / Q6_K blocks, bf16 activations — one token step per
"step".  `value` is tokens/s with everything resident in HBM (one recorded
command replayed per step); `e2e` is the same step driven through the C ABI with
the step's input copied from pinned host memory and the logits read back to the
host inside the timed region.  `roofline` is measured on the dominant kernel
(fused Q4_K gate/up GEMV) with CUDA events in this process, rotating over every
layer's weights so reads come from HBM, not L2.  `cpu_baseline` times the CPU
oracle (the restated reference arithmetic) on one layer of the same weights on
the host cores.

With N > 1 (launched by torch.distributed.run, one process per GPU) output rows
are sharded tensor-parallel and activations are re-assembled with an NCCL
all-gather after every projection: strong scaling of the same token step.

`--impl reference` times only the CPU oracle with all host threads (the
reference has no CPU implementation of this path; the oracle is its restated
shader arithmetic).
"""
from __future__ import annotations

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

METRIC = "decode tok/s, Qwen3-8B Q4_K_M shape (Q4_K/Q6_K GEMV chain)"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class _NvmlPoller:
    """SM clock and clock-event reasons read through NVML every 10 ms on a thread (read-only queries): the
    timed region of a short run is over before nvidia-smi's 100 ms loop has sampled it twice."""
    BITS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, device: int):
        self.sm, self.reasons, self.max_mhz, self.thread = [], set(), None, None
        try:
            import threading
            import pynvml
            pynvml.nvmlInit()
            self.nv, self.h = pynvml, pynvml.nvmlDeviceGetHandleByIndex(device)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.stop_flag = threading.Event()
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()
        except Exception:
            self.thread = None

    def _run(self):
        nv = self.nv
        read = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self.stop_flag.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                mask = int(read(self.h))
                for bit, name in self.BITS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                break
            self.stop_flag.wait(0.01)

    def stop(self):
        if self.thread:
            self.stop_flag.set()
            self.thread.join(timeout=2)
        return self.sm, self.reasons, self.max_mhz


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 100 ms while timing, and the same through NVML
    every 10 ms."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device, self.proc, self.path = device, None, None

    def start(self):
        self.nvml = _NvmlPoller(self.device)
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.device)], stdout=self.out,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        nv_sm, nv_reasons, nv_max = self.nvml.stop() if getattr(self, "nvml", None) else ([], set(), None)
        if not self.proc:
            if nv_sm:
                return {"sm_mhz": statistics.median(nv_sm), "sm_max_mhz": nv_max, "samples": len(nv_sm),
                        "reasons": sorted(nv_reasons), "source": "nvml every 10 ms"}
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                p = [c.strip() for c in line.split(",")]
                if len(p) < 9:
                    continue
                try:
                    sm.append(float(p[1]))
                    smax.append(float(p[2]))
                except ValueError:
                    continue
                for name, val in zip(names, p[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        os.unlink(self.path)
        if nv_sm:       # the denser record; nvidia-smi's samples and reasons are merged in
            return {"sm_mhz": statistics.median(nv_sm + sm), "sm_max_mhz": max(smax + [nv_max]) if nv_max else (max(smax) if smax else None),
                    "samples": len(nv_sm) + len(sm), "reasons": sorted(reasons | nv_reasons),
                    "source": "nvml every 10 ms + nvidia-smi every 100 ms"}
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def workload_config(shape, batch: int, layers: int, world: int, step_bytes: int, activations: str = "bf16") -> dict:
    """The workload description both arms print (identical for the same command line)."""
    return {"workload": "%s dense decode GEMV chain (configs[%d]), batch %d" % (shape.name, 2 if shape.gelu else 1, batch),
            "layers": layers, "hidden": shape.hidden, "ffn": shape.ffn, "vocab": shape.vocab,
            "weights": "random Q4_0 blocks" if shape.gelu else "random Q4_K/Q6_K blocks",
            "activations": "%s between projections, fp32 accumulate" % activations,
            "parallelism": "tp%d rows" % world if world > 1 else "single GPU",
            "l2": "inputs larger than L2: %.2f GB of weights streamed per step" % (step_bytes / 1e9 / world)}


def cpu_chain_step(oc, h0, threads: int) -> float:
    """Seconds for the oracle's chain to run one whole token step (every projection of every layer and the
    head: scalar dequantise + fp32 dot, rows over `threads`)."""
    t0 = time.perf_counter()
    oc.step(h0, f64=False, threads=threads)
    return time.perf_counter() - t0


def run_reference(args):
    """The CPU arm: the oracle's own chain on the host cores, one WHOLE token step per step (all 36 layers'
    distinct weights and the head, 4.92 GB), measured, not scaled."""
    from ingot_b200.chain import QWEN3_8B
    from oracle import chain_check as CK
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    shape = QWEN3_8B
    threads = os.cpu_count() or 1
    oc = CK.OracleChain(shape, layers=args.layers, seed=0, bf16=True)
    h0 = np.random.default_rng(1).normal(0, 1, shape.hidden).astype(np.float32)
    for _ in range(max(min(args.warmup, 1), 1)):          # one untimed step pages the weights in; more would only repeat it
        cpu_chain_step(oc, h0, threads)
    times = [cpu_chain_step(oc, h0, threads) for _ in range(args.steps)]
    sec = sum(times) / len(times)
    value = args.batch / sec
    sample = "measured: %d whole token steps (%d layers + head, %.2f GB of distinct weights each) on %d threads" % (
        args.steps, oc.n_layers, oc.bytes / 1e9, threads)
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(shape, args.batch, oc.n_layers, max(args.gpus, 1), oc.bytes),
            "note": "CPU oracle: restated reference shader arithmetic; the reference itself has no CPU path",
            "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--layers", type=int, default=None, help="debug: fewer layers (invalid as a benchmark)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extra", action="store_true",
                    help="skip the prefill GEMM and MoE tables that the default single-GPU line carries under \"gemm\" and \"moe\"")
    ap.add_argument("--profile-kernel", default=None,
                    help="run only this GEMV (gate_up_q4k, down_q6k, q_q4k, k_q4k, v_q6k, head_q6k) over --layers "
                         "layers, a small case for ncu; prints its timing and exits")
    ap.add_argument("--reps", type=int, default=2, help="sweeps over the layers in --profile-kernel mode")
    ap.add_argument("--activations", default="bf16", choices=["bf16", "f32"],
                    help="activation type between the projections (bf16 is the benchmark configuration)")
    ap.add_argument("--pdl", type=int, default=1, help="0: launch without programmatic dependent launch (comparison)")
    ap.add_argument("--graph", type=int, default=1, help="0: issue every step's launches instead of replaying a recorded command")
    ap.add_argument("--fused-norm", type=int, default=1, help="0: add_rms as separate launches (comparison)")
    ap.add_argument("--chain", type=int, default=0,
                    help="1: the one-token step of a single GPU runs as one persistent kernel (ingot_chain_*); 0: one launch per projection, replayed as a CUDA graph")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: peer = the projections store their row shards as tagged words into every rank's window "
                         "(ingot_group_*); nccl = one NCCL all-gather after each projection (comparison)")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of layer 0 and the logits after the timed region")
    ap.add_argument("--group-scope", type=int, default=1,
                    help="0: the projections of an independent scope on their own streams instead of one grid (comparison)")
    ap.add_argument("--no-mma", type=int, default=0, help="1: streaming GEMVs on the fp32 CUDA-core kernel (comparison)")
    ap.add_argument("--tcgen05-gemv", type=int, default=0, help="1: Q4_K one-token GEMVs on the tcgen05 int8 kernel")
    ap.add_argument("--workload", default="chain", choices=["chain", "gemma", "moe", "gemm"],
                    help="chain: the Qwen3-8B dense decode step (the headline line); gemma: the Gemma-3-4B Q4_0 decode "
                         "step; moe: the Qwen3-30B-A3B expert-routed FFN chain; gemm: the prefill dequant-GEMM table")
    ap.add_argument("--tokens", type=int, nargs="*", default=None,
                    help="token counts of --workload gemm (default 512 2048 8192) and moe (default 1 8 32)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from ingot_b200 import BF16, F32, Gpu, _abi
    from ingot_b200.chain import GEMMA3_4B, QWEN3_8B, DecodeChain, weight_bytes_per_token
    from ingot_b200.gpu import Buffer

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    stream = torch.cuda.Stream(device=local)
    torch.cuda.set_stream(stream)
    gpu = Gpu(local)
    gpu.set_stream(stream.cuda_stream)
    gpu.set_option(_abi.OPT_TCGEN05_GEMV, args.tcgen05_gemv)
    gpu.set_option(_abi.OPT_NO_MMA, args.no_mma)
    gpu.set_option(_abi.OPT_PDL, args.pdl)
    gpu.set_option(_abi.OPT_GROUP_SCOPE, args.group_scope)

    shape = GEMMA3_4B if args.workload == "gemma" else QWEN3_8B
    metric = METRIC if args.workload == "chain" else "decode tok/s, Gemma-3-4B Q4_0 shape (Q4_0 GEMV chain)"
    x_kind = BF16 if args.activations == "bf16" else F32
    if args.workload == "gemm":
        args.tokens = args.tokens or [512, 2048, 8192]
        out = run_gemm(torch, gpu, stream, args, rank, world, local)
        if rank == 0:
            print(json.dumps(out), flush=True)
        if world > 1:
            torch.cuda.synchronize()
            dist.barrier()
            sys.stdout.flush()
            os._exit(0)
        gpu.close()
        return
    if args.workload == "moe":
        args.tokens = args.tokens or [1, 8, 32]
        return run_moe(torch, gpu, stream, args, rank, world, local)
    if args.profile_kernel:
        chain = DecodeChain(gpu, shape, batch=args.batch, x_kind=x_kind, seed=0, layers=args.layers or 4, packed=not args.no_mma)
        peaks, peak_src = measured_peaks()
        roof, per = kernel_rooflines(torch, gpu, chain, stream, peaks, peak_src, only=args.profile_kernel,
                                     reps=args.reps, digits=bool(args.tcgen05_gemv))
        print(json.dumps({"profile_kernel": args.profile_kernel, "layers": chain.n_layers, **per[args.profile_kernel]}))
        gpu.close()
        return

    def all_gather(part: Buffer, full: Buffer, batch: int, rows_local: int):
        n = batch * rows_local
        src = _tensor_view(torch, part.ptr, n, local)
        dst = _tensor_view(torch, full.ptr, n * world, local)
        dist.all_gather_into_tensor(dst, src)

    group = None
    if world > 1 and args.exchange == "peer" and args.fused_norm and args.batch == 1:
        n_layers = shape.layers if args.layers is None else args.layers
        window = 4 * args.batch * (shape.q + 2 * shape.hidden + shape.ffn + shape.vocab) + 8 * 256
        group = connect_group(torch, dist, gpu, rank, world, local, window, DecodeChain.exchange_slots(n_layers))
    chain = DecodeChain(gpu, shape, batch=args.batch, x_kind=x_kind, seed=0, rank=rank, world=world, group=group,
                        all_gather=all_gather if world > 1 else None, layers=args.layers, packed=not args.no_mma, fused_norm=bool(args.fused_norm),
                        keep_host=1 if (rank == 0 and world == 1 and not (args.no_cpu and args.no_parity)) else 0)
    h0 = np.random.default_rng(1).normal(0, 1, (args.batch, shape.hidden)).astype(np.float32)
    gpu._check(gpu._lib.ingot_buffer_upload(gpu._h, chain.h_in.ptr, h0.ctypes.data, h0.nbytes))
    gpu.complete()

    use_graph = True
    tgraph = None
    fused = None
    if world == 1 and args.chain and chain.fused_norm:
        chain.step()                      # once through the one-by-one path (also sizes every buffer)
        gpu.complete()
        fused = chain.record_chain()
        graph = None
    elif world == 1:
        graph = chain.record() if args.graph else None
    elif group is not None:
        # no collective inside the step: the library records it itself.  One eager step first, all ranks in step.
        chain.step()
        gpu.complete()
        dist.barrier()
        graph = chain.record() if args.graph else None
    else:
        # the step contains NCCL all-gathers: let torch record it (its NCCL bindings join the
        # capture), after eager steps have created the communicator
        graph = None
        for _ in range(2):
            chain.step()
        torch.cuda.synchronize()
        dist.barrier()
        tgraph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(tgraph, stream=stream, capture_error_mode="thread_local"):
            chain.step()

    def one_step():
        if fused is not None:
            fused.submit()
        elif graph is not None:
            graph.submit()
        elif tgraph is not None:
            tgraph.replay()
        else:
            chain.step()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # clocks are sampled from the warm-up to the end of the end-to-end loop: the timed regions are
    # tens of milliseconds, shorter than one sampling period
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        one_step()
    gpu.complete()
    launches_per_step = chain.launches_per_step
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        one_step()
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    gpu.complete()
    ms_per_step = ms / args.steps
    value = args.batch * 1000.0 / ms_per_step

    # ---- end to end through the C ABI: pinned host input in, logits out, every step ----
    host_in, host_out = _pinned(gpu, h0.nbytes), _pinned(gpu, 4 * args.batch * shape.vocab)
    C_memmove(host_in, h0)
    for _ in range(2):
        _e2e_step(gpu, chain, one_step, host_in, h0.nbytes, host_out)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        _e2e_step(gpu, chain, one_step, host_in, h0.nbytes, host_out)
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=f"cuda:{local}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    # ---- roofline of the dominant kernel, measured here with CUDA events ----
    peaks, peak_src = measured_peaks()
    roof, per_kernel = None, None
    if world == 1:
        roof, per_kernel = kernel_rooflines(torch, gpu, chain, stream, peaks, peak_src)
    clocks = sampler.stop() if rank == 0 else None

    cpu, parity = None, None
    if rank == 0 and world == 1 and not args.no_parity and chain.host and chain.fused_norm and args.batch == 1:
        # outside the timed region: the head (on the inputs the last step left) and every projection of layer 0, each
        # against the oracle's f64 dot on the inputs the operator read (oracle/chain_check.py)
        from oracle import chain_check as CK
        ops = chain.fused_ops()
        picked = [ops[-1]] + [op for op in ops if op.layer == 0]
        records = CK.check_fused_ops(gpu, chain, picked, chain.host)
        parity = {"parity_checked": True, "operators": len(records),
                  "worst_error_over_bound": max(r["max_err_over_tol"] for r in records)}
    if rank == 0 and world == 1 and not args.no_cpu and chain.host:
        # the oracle on the host cores: the same weights' layer 0 and the head, measured (a bounded sample of the step:
        # 633 MB of its 4.92 GB); tok/s = 1 / (36 x the layer's time + the head's time)
        from oracle import oracle as O
        threads = os.cpu_count() or 1
        def cpu_time(keys):
            t0 = time.perf_counter()
            for key in keys:
                raw, cols, rows, kind = chain.host[key]
                O.matvec_f32(raw, cols, rows, kind, np.ones(cols, np.float32), threads=threads)
            return time.perf_counter() - t0
        layer_keys = [(0, r) for r in ("q", "k", "v", "o", "gate", "up", "down")]
        cpu_time(layer_keys)
        t_layer = min(cpu_time(layer_keys) for _ in range(2))
        t_head = cpu_time([(chain.n_layers, "head")])
        cpu = {"value": args.batch / (chain.n_layers * t_layer + t_head), "unit": "tok/s", "cores": threads, "kind": "port",
               "sample": "measured on layer 0 (%.1f ms) and the head (%.1f ms) of the same weights; the step is %d such layers and the head"
                         % (t_layer * 1e3, t_head * 1e3, chain.n_layers)}

    extra = {}
    if rank == 0 and world == 1 and args.workload == "chain" and args.batch == 1 and args.layers is None and not args.no_extra \
            and not args.profile_kernel:
        # the other two measured configurations, each with a clock record of its own (they are not part of `value`):
        # the prefill dequant-GEMM table (configs[4]) and the expert-routed FFN chain (configs[3])
        other = argparse.Namespace(**vars(args))
        other.steps, other.warmup, other.layers = 10, 3, None
        s2 = ClockSampler(local)
        s2.start()
        other.tokens = [512, 2048, 8192]
        g = run_gemm(torch, gpu, stream, other)
        extra["gemm"] = {"workload": g["workload"], "unit": "TFLOP/s", "bound": "tensor", "peak": g["peak"], "peak_source": g["peak_source"],
                         "steps": other.steps, "warmup": other.warmup, "shapes": g["shapes"], "clocks": s2.stop()}
        s3 = ClockSampler(local)
        s3.start()
        other.tokens = [1, 8, 32]
        rows = run_moe(torch, gpu, stream, other, rank, world, local, table_only=True)
        extra["moe"] = {"workload": "qwen3-30b-a3b expert-routed FFN chain (configs[3]), 48 layers, one GPU", "unit": "tok/s",
                        "steps": other.steps, "warmup": other.warmup, "by_tokens": rows, "clocks": s3.stop()}
    if rank == 0:
        total_bytes = weight_bytes_per_token(shape) if args.layers is None else chain.bytes_streamed
        line = {
            "metric": metric, "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(shape, args.batch, chain.n_layers, world, total_bytes, args.activations),
            "launch_mode": ("one persistent kernel per step (chain of %(projections)d projections, %(waits)d grid-wide waits, %(stages)d stages of %(stage_bytes)d bytes per SM)" % fused.info())
                                 if fused is not None else "one recorded command (CUDA graph) per step" + (
                                 " incl. NCCL all-gathers" if world > 1 and group is None else
                                 "; row shards exchanged by the projections themselves (tagged 8-byte words stored into every rank's window, polled by the next projection)" if world > 1 else ""),
            "hbm_gbs_effective": total_bytes / world / (ms_per_step * 1e-3) / 1e9,
            "hbm_frac_of_peak_chain": total_bytes / world / (ms_per_step * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "e2e": {"value": args.batch * 1000.0 / e2e_ms, "unit": "tok/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(h0.nbytes), "d2h_bytes_per_step": int(4 * args.batch * shape.vocab)},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks, "roofline": roof, "kernels": per_kernel, "cpu_baseline": cpu,
        }
        if parity:
            line.update(parity)
        line.update(extra)
        print(json.dumps(line), flush=True)
    if world > 1:
        # leave without tearing the communicator down: the recorded step holds NCCL work, and
        # destroying the process group under it can block; every rank is past its last collective
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)
    gpu.close()


# ---- helpers ------------------------------------------------------------------------

def connect_group(torch, dist, gpu, rank, world, local, window_bytes, slots):
    """One rank's end of an ingot_group_* group; the 64-byte IPC handles travel over the process group, nothing else does."""
    from ingot_b200.gpu import Group
    group = Group(gpu, rank, world, window_bytes, slots)
    mine = torch.frombuffer(bytearray(group.handle), dtype=torch.uint8).to(f"cuda:{local}")
    everyone = torch.empty(64 * world, dtype=torch.uint8, device=f"cuda:{local}")
    dist.all_gather_into_tensor(everyone, mine)
    group.connect(bytes(everyone.cpu().numpy()))
    dist.barrier()
    return group


def run_moe(torch, gpu, stream, args, rank, world, local, table_only=False):
    """Qwen3-30B-A3B-shaped expert-routed FFN chain: 48 layers of route_topk -> routed gate/up + SiLU ->
    routed down -> moe_sum, Q4_K experts, synthetic N(0,1) router logits, for each token count.
    With N > 1 ranks the 128 experts are split expert-parallel (rank r owns experts [r*128/N, ...)) and the SAME
    total step runs on more GPUs (strong scaling).  --exchange peer (default): the tokens are split over the ranks
    too, every rank routes its own and the rows travel to the experts' owners and back (token all-to-all,
    ingot_ep_*; a count that does not divide leaves the last ranks with fewer tokens).  --exchange nccl: every rank
    sees all tokens, runs its experts' pairs, and one NCCL all-reduce per layer completes the output (comparison)."""
    from ingot_b200.moe import QWEN3_30B_A3B, MoeChain, expert_bytes
    from ingot_b200.gpu import Buffer
    dist = None
    if world > 1:
        import torch.distributed as dist

    def all_reduce(buf: Buffer, n: int):
        dist.all_reduce(_tensor_view(torch, buf.ptr, n, local))

    s = QWEN3_30B_A3B
    peaks, peak_src = measured_peaks()
    results = []
    a2a = world > 1 and args.exchange == "peer"

    def own(tokens: int) -> tuple[int, int]:
        """This rank's span of the step's tokens (token all-to-all), else all of them."""
        if not a2a:
            return 0, tokens
        per = -(-tokens // world)
        return min(rank * per, tokens), min((rank + 1) * per, tokens)

    most = max(-(-t // world) if a2a else t for t in args.tokens)
    group = None
    if a2a:
        from ingot_b200.gpu import EpExchange
        n_layers = args.layers or s.layers
        group = connect_group(torch, dist, gpu, rank, world, local, EpExchange.window_bytes(world, most * s.top, s.hidden),
                              MoeChain.exchange_slots(n_layers))
    chain = MoeChain(gpu, s, tokens=most, seed=0, rank=rank, world=world, all_reduce=all_reduce if world > 1 else None,
                     layers=args.layers, local_weights_only=True, group=group)
    for tokens in args.tokens:
        t0, t1 = own(tokens)
        chain.tokens = t1 - t0              # the buffers are sized for the largest count
        if a2a:
            chain.set_capacity(-(-tokens // world) * s.top)       # places per region: the most pairs a rank has in this step
        rng = np.random.default_rng(100 + tokens)
        logits = rng.normal(0, 1, (tokens, s.experts)).astype(np.float32)[t0:t1].copy()
        x = rng.normal(0, 1, (tokens, s.hidden)).astype(np.float32)[t0:t1].copy()
        if t1 > t0:
            gpu._check(gpu._lib.ingot_buffer_upload(gpu._h, chain.logits.ptr, logits.ctypes.data, logits.nbytes))
            gpu._check(gpu._lib.ingot_buffer_upload(gpu._h, chain.x.ptr, x.ctypes.data, x.nbytes))
        gpu.complete()
        graph, tgraph = None, None
        if a2a:
            torch.cuda.synchronize()
            dist.barrier()                  # every rank's inputs are in place before anybody's rows arrive
            chain.step()
            gpu.complete()
            dist.barrier()
            graph = chain.record()
        elif world == 1:
            chain.step()
            gpu.complete()
            graph = chain.record()
        else:
            for _ in range(2):
                chain.step()
            torch.cuda.synchronize()
            dist.barrier()
            tgraph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(tgraph, stream=stream, capture_error_mode="thread_local"):
                chain.step()

        def one_step():
            if graph is not None:
                graph.submit()
            else:
                tgraph.replay()

        for _ in range(args.warmup):
            one_step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            one_step()
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        if world > 1:
            t = torch.tensor([ms], device=f"cuda:{local}")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        ids = gpu.read_bytes(chain.ids).view(np.uint32)[:(t1 - t0) * s.top]
        if a2a:                             # the step's experts: the union over the ranks' own tokens
            seen = torch.zeros(s.experts, dtype=torch.int32, device=f"cuda:{local}")
            if len(ids):
                seen[torch.from_numpy(np.unique(ids).astype(np.int64)).to(seen.device)] = 1
            dist.all_reduce(seen, op=dist.ReduceOp.MAX)
            unique = int(seen.sum().item())
        else:
            unique = int(len(np.unique(ids)))
        algo = chain.n_layers * unique * expert_bytes(s)        # every layer routes the same synthetic logits
        results.append({"tokens": tokens, "ms_per_step": ms, "tok_per_s": tokens * 1000.0 / ms, "unique_experts": unique,
                        "expert_bytes_per_step": algo, "gbs": algo / (ms * 1e-3) / 1e9,
                        "frac_of_hbm_peak": algo / (ms * 1e-3) / 1e9 / (peaks["hbm_gbs"] * world),
                        "launches_per_step": chain.launches_per_step})
        del graph, tgraph
    if table_only:                      # the caller's own line carries the table (single GPU)
        del chain
        return results
    if rank == 0:
        head = results[0]
        print(json.dumps({"metric": "decode tok/s, Qwen3-30B-A3B shape (expert-routed Q4_K GEMV chain)", "value": head["tok_per_s"],
                          "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                          "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                          "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                          "config": {"workload": "qwen3-30b-a3b expert-routed FFN chain (configs[3]), tokens %s" % args.tokens,
                                     "layers": args.layers or s.layers, "experts": s.experts, "top": s.top,
                                     "parallelism": ("ep%d, token all-to-all inside the library (peer stores, tagged words)" % world if a2a else
                                                     "ep%d, tokens replicated, one NCCL all-reduce per layer" % world) if world > 1 else "single GPU",
                                     "peak_source": peak_src},
                          "by_tokens": results}), flush=True)
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)
    gpu.close()


def run_gemm(torch, gpu, stream, args, rank=0, world=1, local=0):
    """The batched prefill dequant-GEMM: Q4_K 4096 -> 12288 and Q6_K 12288 -> 4096 against bf16
    activations of `--tokens` rows, timed alone with CUDA events; TFLOP/s against the measured
    dense bf16 peak (burst figure: each shape is timed in isolation).  With N > 1 ranks the weight rows are
    split (rank r multiplies rows [r R / N, (r + 1) R / N): block quantisation runs along K, so the GGUF
    layout is kept), the activations are replicated, and an NCCL all-gather assembles Y on every rank as
    [rank][token][rows / N]; both the multiplication alone and multiplication + all-gather are timed (max over
    ranks), the same total work on more GPUs (strong scaling)."""
    from ingot_b200 import BF16, synth
    from ingot_b200.chain import shard_rows
    dist = None
    if world > 1:
        import torch.distributed as dist
    peaks, peak_src = measured_peaks()
    rows_out = []
    launches = 0

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        sec = e0.elapsed_time(e1) * 1e-3 / args.steps
        if world > 1:
            t = torch.tensor([sec], device=f"cuda:{local}")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec = float(t.item())
        return sec

    for kind, name, cols, rows in ((synth.Q4_K, "q4_k", 4096, 12288), (synth.Q6_K, "q6_k", 12288, 4096)):
        r0, r1 = shard_rows(rows, rank, world)
        mine = r1 - r0
        raw = synth.random_matrix(kind, cols, mine, seed=5 + 1000 * rank)
        w = gpu.bytes(raw)
        stride = synth.stride_of(kind, cols)
        for m in args.tokens:
            x = np.random.default_rng(m).normal(0, 1, (m, cols)).astype(np.float32)
            xb = gpu.bf16(x)
            y = gpu.zeros(m * mine)
            whole = gpu.zeros(m * mine * world) if world > 1 else None

            def multiply():
                gpu.gemm(None, w, cols, mine, stride, kind, 0, xb, m, BF16, out=y)

            def multiply_and_gather():
                multiply()
                dist.all_gather_into_tensor(_tensor_view(torch, whole.ptr, m * mine * world, local), _tensor_view(torch, y.ptr, m * mine, local))

            sec = timed(multiply)
            launches += 2 * args.steps
            flops = 2.0 * m * cols * rows
            row = {"kind": name, "cols": cols, "rows": rows, "tokens": m, "us": sec * 1e6,
                   "tflops": flops / sec / 1e12, "frac": flops / sec / 1e12 / (peaks["bf16_tflops"] * world),
                   "tok_per_s": m / sec}
            if world > 1:
                sec_g = timed(multiply_and_gather)
                row.update({"us_with_all_gather": sec_g * 1e6, "tok_per_s_with_all_gather": m / sec_g,
                            "all_gather_bytes_per_rank": 4 * m * mine * (world - 1)})
            rows_out.append(row)
            for b in (xb, y, whole):
                if b is not None:
                    b.release()
        w.release()
    head = max((r for r in rows_out if r["kind"] == "q4_k"), key=lambda r: r["tokens"])
    return {"metric": "prefill tok/s, Q4_K 4096 -> 12288 dequant-GEMM at %d tokens" % head["tokens"],
            "value": head["tok_per_s"], "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": head["us"] * 1e-3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 x dequantised bf16 weights, f32 accumulation", "data": "synthetic",
            "config": {"workload": "prefill dequant-GEMM (configs[4])",
                       "parallelism": "weight rows split over %d ranks, activations replicated" % world if world > 1 else "single GPU",
                       "peak_source": peak_src},
            "workload": "prefill dequant-GEMM (configs[4])", "unit_roofline": "TFLOP/s", "peak": peaks["bf16_tflops"],
            "peak_source": peak_src, "bound": "tensor", "gpu_launches": launches, "shapes": rows_out}


def _tensor_view(torch, ptr: int, n_f32: int, device: int):
    """A float32 torch tensor over `n_f32` elements of device memory owned by the library
    (used only to hand activation buffers to NCCL)."""
    class _Holder:
        pass
    h = _Holder()
    h.__cuda_array_interface__ = {"shape": (n_f32,), "typestr": "<f4", "data": (ptr, False), "version": 3,
                                  "strides": None}
    return torch.as_tensor(h, device=f"cuda:{device}")


def _pinned(gpu, nbytes: int) -> int:
    import ctypes as C
    p = C.c_void_p()
    gpu._check(gpu._lib.ingot_host_alloc(gpu._h, nbytes, C.byref(p)))
    return p.value


def C_memmove(dst_ptr: int, arr: np.ndarray) -> None:
    import ctypes as C
    C.memmove(dst_ptr, arr.ctypes.data, arr.nbytes)


def _e2e_step(gpu, chain, one_step, host_in: int, in_bytes: int, host_out: int) -> None:
    gpu._check(gpu._lib.ingot_buffer_upload(gpu._h, chain.h_in.ptr, host_in, in_bytes))
    one_step()
    gpu._check(gpu._lib.ingot_buffer_read(gpu._h, host_out, chain.logits.ptr, chain.logits.nbytes))


def ncu_traffic(kernel: str):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of `kernel` from the committed ncu
    summary (profiles/ncu_traffic.json), or None when it has not been captured."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    try:
        with open(path) as f:
            return json.load(f).get(kernel)
    except (OSError, ValueError):
        return None


def kernel_rooflines(torch, gpu, chain, stream, peaks, peak_src, only=None, reps=None, digits=False):
    """Times each distinct GEMV of the step alone (CUDA events on the launching stream),
    rotating over all layers' weights so every launch streams from HBM."""
    from ingot_b200 import synth
    s, b = chain.shape, chain.batch
    xb = 2
    lib, h = gpu._lib, gpu._h

    def timed(fn, reps):
        """Seconds per launch: one sweep over all layers recorded as a command and replayed, so
        host launch cost is out of the picture and consecutive launches chain as in a token step."""
        for i in range(len(chain.weights)):
            fn(i)
        gpu.complete()
        gpu.record()
        for i in range(len(chain.weights)):
            fn(i)
        graph = gpu.end_record()
        graph.submit()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            graph.submit()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e-3 / (reps * len(chain.weights))

    if chain.packed:        # the packed rows the timed launches read (the fused step does not write them)
        chain._norm(chain.h_in, None, None, chain.xn, s.hidden)
        chain._norm(chain.q, None, None, chain.a, s.q)
        chain._norm(chain.act, None, None, chain.actn, s.ffn)
        gpu.complete()
    xd = None
    if digits:      # the tcgen05 int8 GEMV reads activations as digit rows (Q4_K weights)
        from ingot_b200 import X_DIGITS
        xd = gpu.pack_digits(chain.xn, 1, s.hidden, chain.x_kind)

    def x_of(x, kind):
        if xd is not None and kind == synth.Q4_K and x is chain.xn:
            return xd.ptr, X_DIGITS
        return chain._x(x)

    # with the norms fused, a projection reads the fp32 vector its norm would read
    fp32_of = {id(chain.xn): chain.h_in, id(chain.a): chain.q, id(chain.actn): chain.act}
    rb = int(chain.x_kind != 0)

    def proj(role, x, y):
        def fn(i):
            w = chain.weights[i][role]
            t = w.t
            if chain.fused_norm and xd is None:
                gpu._check(lib.ingot_matmul_normed(h, w.buffer.ptr, t.dims[0], t.dims[1], t.stride, t.kind, 0, fp32_of[id(x)].ptr,
                                                   None, None, None, 1e-6, 0, rb, y.ptr))
                return
            xp, xk = x_of(x, t.kind)
            gpu._check(lib.ingot_matmul(h, w.buffer.ptr, t.dims[0], t.dims[1], t.stride, t.kind, 0, xp, xk, b, y.ptr))
        return fn

    def gate_up(i):
        g, u = chain.weights[i]["gate"], chain.weights[i]["up"]
        t = g.t
        if chain.fused_norm and xd is None:
            gpu._check(lib.ingot_gate_up_normed(h, g.buffer.ptr, u.buffer.ptr, t.dims[0], t.dims[1], t.stride, t.kind,
                                                chain.h_in.ptr, None, None, None, 1e-6, 0, rb, int(s.gelu), chain.act.ptr))
            return
        xp, xk = x_of(chain.xn, t.kind)
        gpu._check(lib.ingot_gate_up(h, g.buffer.ptr, u.buffer.ptr, t.dims[0], t.dims[1], t.stride, t.kind, xp, xk, b, int(s.gelu),
                                     chain.act.ptr))

    out = {}
    reps = reps or max(1, 144 // max(len(chain.weights), 1))
    kn = {synth.Q4_K: "q4k", synth.Q6_K: "q6k", synth.Q4_0: "q4_0", synth.Q8_0: "q8_0"}
    k = s.kinds
    cases = [("gate_up_" + kn[k["gate"]], gate_up, 2 * s.ffn * synth.stride_of(k["gate"], s.hidden), s.hidden, s.ffn),
             ("down_" + kn[k["down"]], proj("down", chain.actn, chain.d), s.hidden * synth.stride_of(k["down"], s.ffn), s.ffn, s.hidden),
             ("q_" + kn[k["q"]], proj("q", chain.xn, chain.q), s.q * synth.stride_of(k["q"], s.hidden), s.hidden, s.q),
             ("k_" + kn[k["k"]], proj("k", chain.xn, chain.k), s.kv * synth.stride_of(k["k"], s.hidden), s.hidden, s.kv),
             ("v_" + kn[k["v"]], proj("v", chain.xn, chain.v), s.kv * synth.stride_of(k["v"], s.hidden), s.hidden, s.kv)]
    if chain.independent_qkv:       # the three projections of one layer inside the independent scope (one grid)
        fq, fk, fv = proj("q", chain.xn, chain.q), proj("k", chain.xn, chain.k), proj("v", chain.xn, chain.v)
        def qkv(i):
            with gpu.independent():
                fk(i); fv(i); fq(i)
        cases.append(("qkv_scope", qkv, sum(c[2] for c in cases[2:5]), s.hidden, s.q + 2 * s.kv))
    head_name = "head_" + kn[k["head"]]
    for name, fn, wbytes, cols, rows in cases:
        if only and name != only:
            continue
        sec = timed(fn, reps)
        algo = wbytes + b * cols * xb + b * rows * 4
        out[name] = {"us": sec * 1e6, "bytes": algo, "gbs": algo / sec / 1e9, "frac": algo / sec / 1e9 / peaks["hbm_gbs"]}
    if only and only != head_name:
        return None, out
    # the head: one matrix of 510 MB, far larger than L2 on its own
    t = chain.head.t
    def head(i):
        if chain.fused_norm and xd is None:
            gpu._check(lib.ingot_matmul_normed(h, chain.head.buffer.ptr, t.dims[0], t.dims[1], t.stride, t.kind, 0, chain.h_in.ptr,
                                               None, None, None, 1e-6, 0, rb, chain.logits.ptr))
            return
        xp, xk = chain._x(chain.xn)
        gpu._check(lib.ingot_matmul(h, chain.head.buffer.ptr, t.dims[0], t.dims[1], t.stride, t.kind, 0, xp, xk, b,
                                    chain.logits.ptr))
    for _ in range(2):
        head(0)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(8):
        head(0)
    e1.record(stream)
    torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) * 1e-3 / 8
    algo = t.dims[1] * t.stride + b * t.dims[0] * xb + b * t.dims[1] * 4
    out[head_name] = {"us": sec * 1e6, "bytes": algo, "gbs": algo / sec / 1e9, "frac": algo / sec / 1e9 / peaks["hbm_gbs"]}
    if only:
        return None, out
    gname = "gate_up_" + kn[k["gate"]]
    g = out[gname]
    roof = {"bound": "hbm", "kernel": "gemv_mma_kernel<%s, 1 token, gate+up fused> %d -> 2 x %d" % (kn[k["gate"]], s.hidden, s.ffn),
            "achieved": g["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": g["frac"], "peak_source": peak_src,
            "bytes_per_launch": g["bytes"], "us_per_launch": g["us"], "traffic": ncu_traffic(gname)}
    return roof, out


if __name__ == "__main__":
    main()
