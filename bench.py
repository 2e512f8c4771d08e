#!/usr/bin/env python
"""Benchmark of the fused Ulysses projection hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (BASELINE.json configs[1]): Llama-3-8B-shaped BF16 forward, context parallel degree
CP = N with 16K tokens per rank (weak scaling; CP8 = global sequence 128K), hidden 4096,
32 Q / 8 KV heads, head_dim 128.  One step = QKVProj GEMM -> sequence-to-head all-to-all
(weight [6144, 4096]) followed by head-to-sequence all-to-all -> OProj GEMM (weight
[4096, 4096]), each one fused kernel launched through the C ABI.  At N = 1 the all-to-all is
the local repack, i.e. the "pure GEMM + route" point of the scaling curve.

Prints ONE JSON line.  `value` is the whole-job throughput in PFLOPS (algorithmic
2*M*N*K FLOPs of both GEMMs, all ranks, over the max-over-ranks device time); `per_gpu` is the
reference's own way of quoting it (PFLOPS/GPU).  Further keys of the line:

  e2e        the same step from pinned HOST buffers, host<->device copies inside the timed
             region (uploads, kernels and downloads on three streams ordered by events; with
             peers the routed buffers are double-buffered so that no step needs a host barrier)
  validated  after the timed regions the outputs are poisoned, one more step runs, and a row
             sample of both operators is compared with the CPU oracle (GEMM within the reference's
             tolerance, routed / gathered elements bit-exact incl. what peers wrote here); the
             routed tensors are also compared at full size, bit for bit, with an NCCL all-to-all of
             the same local outputs.  A failure makes the run exit non-zero.
  separate_baseline  torch.matmul (cuBLASLt) + pack + NCCL all_to_all_single as separate kernels
  pure_gemm_148sm / cublas   retention denominators (this library's pure GEMM, cuBLASLt)
  sustained  >= 2 s of back-to-back steps against the sustained measured peak
  nvlink     algorithmic bytes each routed kernel moves over NVLink / its device time
  others     the other benchmark configurations (BF16 backward, C3, C4, C5) from bench_suite.py

`--impl reference` times the CPU restatement of the path (the reference has no CPU
implementation of the fused operators, only host oracle pieces) on all host cores, on a bounded
row sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "fused GEMM+A2A PFLOPS/GPU (max over ranks) at CP2/4/8; % of full-SM GEMM"
TOKENS_PER_RANK = 16384
HIDDEN, Q_HEADS, KV_HEADS, HEAD_DIM = 4096, 32, 8, 128
QKV_N = (Q_HEADS + 2 * KV_HEADS) * HEAD_DIM  # 6144
OPROJ_K = Q_HEADS * HEAD_DIM                  # 4096
FLOPS_PER_RANK = 2.0 * TOKENS_PER_RANK * HIDDEN * (QKV_N + OPROJ_K)
QKV_FLOPS = 2.0 * TOKENS_PER_RANK * HIDDEN * QKV_N

# DRAM bytes (read + write) of one launch of the fused QKV kernel at this workload on one GPU
# (direct route, CTA pairs): dram__bytes_read.sum + dram__bytes_write.sum of a stored ncu capture,
# not re-measured by this program.
QKV_DRAM_TRAFFIC_BYTES_STORED_CAPTURE = 876_308_736

_RESULT_FD = None


def emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def measured_peaks():
    """(burst TFLOP/s, sustained TFLOP/s, where the numbers come from)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            data = json.load(f)
        return (float(data["bf16_tflops"]), float(data.get("bf16_tflops_sustained", data["bf16_tflops"])),
                "measured (MEASURED_PEAKS.json)")
    return 1590.0, 1400.0, "fallback (earlier pool measurement)"


def all_host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


# --------------------------------------------------------------------------------------------
# CPU arm: the oracle port timed on the host cores
# --------------------------------------------------------------------------------------------

def cpu_step_factory(rows: int, threads: int):
    """Returns (step_fn, flops_per_step, description, threads) for a `rows`-row sample of the workload."""
    import numpy as np
    from oracle import oracle as O
    L = O.lib()
    L.fo_set_num_threads(threads)  # torchrun exports OMP_NUM_THREADS=1; the sample may use every core
    rng = np.random.default_rng(20260906)
    bf16 = lambda a: O.f32_to_bf16(a.astype(np.float32))
    x = bf16(rng.standard_normal((rows, HIDDEN)))
    w_qkv = bf16(rng.standard_normal((QKV_N, HIDDEN)) * 0.02)
    w_o = bf16(rng.standard_normal((HIDDEN, OPROJ_K)) * 0.02)
    attn = bf16(rng.standard_normal((rows, OPROJ_K)))
    local = np.zeros((rows, QKV_N), dtype=np.uint16)
    planar = np.zeros(rows * QKV_N, dtype=np.uint16)
    staging = np.zeros((rows, OPROJ_K), dtype=np.uint16)
    out = np.zeros((rows, HIDDEN), dtype=np.uint16)
    planar_table = O.ptr_array([planar])
    attn_table = O.ptr_array([attn])
    keep_alive = (planar, attn)  # the pointer tables hold raw addresses only

    def step():
        assert keep_alive is not None
        assert L.fo_gemm_bf16(0, O.ptr(x), HIDDEN, O.ptr(w_qkv), HIDDEN, O.ptr(local), QKV_N, rows, QKV_N,
                              HIDDEN, 1.0, 0.0) == 0
        L.fo_qkv_forward_route(1, 0, 1, rows, Q_HEADS, KV_HEADS, HEAD_DIM, O.ptr(local), QKV_N, planar_table)
        L.fo_oproj_forward_gather(1, 0, 1, rows, OPROJ_K, 0, 0, attn_table, O.ptr(staging))
        assert L.fo_gemm_bf16(0, O.ptr(staging), OPROJ_K, O.ptr(w_o), OPROJ_K, O.ptr(out), HIDDEN, rows,
                              HIDDEN, OPROJ_K, 1.0, 0.0) == 0

    flops = 2.0 * rows * HIDDEN * (QKV_N + OPROJ_K)
    sample = (f"{rows} of {TOKENS_PER_RANK} rows of one rank (both GEMMs full N and K, scalar route and "
              f"gather of those rows); throughput is per sampled FLOP, not extrapolated")
    return step, flops, sample, L.fo_num_threads()


def run_reference_arm(args):
    """The CPU implementation of the path on ALL host cores (one process: under torchrun rank 0
    computes, the other ranks leave at once), each step a 512-row sample of one rank's workload."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    try:
        os.sched_setaffinity(0, range(os.cpu_count() or 1))
    except (AttributeError, OSError):
        pass
    step, flops, sample, cores = cpu_step_factory(rows=512, threads=all_host_cores())
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    elapsed = time.perf_counter() - t0
    value = flops * args.steps / elapsed / 1e15
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "PFLOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(args.gpus),
        "note": ("whole-host CPU throughput (all cores, one process); it does not grow with --gpus, so against it "
                 "the GPU arm's `value` is N GPUs vs one host and `per_gpu` is one GPU vs one host"),
        "cpu_baseline": {"value": value, "unit": "PFLOPS", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "PFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def workload_config(n_gpus):
    return {
        "workload": "Llama-3-8B-shaped BF16 forward: QKVProj->A2A (W [6144,4096]) + A2A->OProj (W [4096,4096])",
        "context_parallel": n_gpus, "tokens_per_rank": TOKENS_PER_RANK,
        "global_seq": TOKENS_PER_RANK * n_gpus, "hidden": HIDDEN, "q_heads": Q_HEADS, "kv_heads": KV_HEADS,
        "head_dim": HEAD_DIM, "l2": "inputs larger than L2 (per step 0.5 GB of operands and outputs vs 126 MB L2)",
    }


# --------------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------------

class ClockSampler:
    """Reads (never sets) SM clock and clock-event reasons of one GPU through NVML every few
    milliseconds while a timed region runs (a 50 ms region gets several samples; polling much
    faster than that delays this process's own kernel launches);
    falls back to an `nvidia-smi -lms` child when the NVML python module is missing."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    REASON_BITS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                   "sw_power_cap": 0x4}

    def __init__(self, uuid: str | None, period_s: float = 0.01):
        self.period_s = period_s
        self.samples, self.proc, self.thread, self.nvml, self.handle = [], None, None, None, None
        self.stop_flag = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.handle = (pynvml.nvmlDeviceGetHandleByUUID(uuid.encode() if hasattr(uuid, "encode") else uuid)
                           if uuid else pynvml.nvmlDeviceGetHandleByIndex(0))
            self.smax = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:  # noqa: BLE001 - any NVML problem selects the fallback
            self.nvml = None
        cmd = ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"]
        if uuid:
            cmd += ["-i", uuid]
        try:
            self.proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _poll(self):
        nv = self.nvml
        while not self.stop_flag.is_set():
            try:
                sm = float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                self.samples.append((time.perf_counter(), (sm, self.smax, mask)))
            except Exception:  # noqa: BLE001
                pass
            time.sleep(self.period_s)

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def window(self, t0, t1):
        """Summary of the samples taken between two perf_counter stamps (the sampler keeps running)."""
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        sm, smax, reasons = [], [], set()
        if self.nvml is not None:
            rows = [s for (t, s) in list(self.samples) if t0 <= t <= t1] or [s for (_, s) in self.samples[-3:]]
            for clock, top, mask in rows:
                sm.append(clock)
                smax.append(top)
                reasons.update(name for name in names if mask & self.REASON_BITS[name])
            source = "nvml"
        elif self.proc is not None:
            time.sleep(0.12)
            rows = [s for (t, s) in list(self.samples) if t0 - 0.05 <= t <= t1 + 0.05] or [s for (_, s) in self.samples]
            for row in rows:
                cells = [c.strip() for c in row.split(",")]
                try:
                    sm.append(float(cells[0]))
                    smax.append(float(cells[1]))
                except (ValueError, IndexError):
                    continue
                reasons.update(name for name, cell in zip(names, cells[3:7]) if cell == "Active")
            source = "nvidia-smi"
        else:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source available"]}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": source}

    def close(self):
        self.stop_flag.set()
        if self.thread is not None and self.nvml is not None:
            self.thread.join(timeout=1.0)
        if self.proc is not None:
            self.proc.terminate()


def bind_to_gpu_numa_node(torch, device_index: int):
    """Runs this process (and so first-touches its pinned host buffers) on the CPUs of the NUMA node
    the GPU hangs off.  Reads sysfs only.  Returns the node, or None when it cannot be told."""
    try:
        props = torch.cuda.get_device_properties(device_index)
        bdf = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            text = f.read().strip()
        cpus = set()
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= set(os.sched_getaffinity(0))
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return node
    except Exception:  # noqa: BLE001 - containers may hide sysfs; the run goes on unbound
        return None


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------

def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    from fuse_b200 import _native as N
    from fuse_b200 import api, synthetic
    from fuse_b200.world import World

    world_size = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world_size != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world_size}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    original_affinity = os.sched_getaffinity(0) if hasattr(os, "sched_getaffinity") else None
    numa_node = bind_to_gpu_numa_node(torch, local_rank)
    if world_size > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    N.lib()  # fail loudly here if the CUDA library is missing

    m, cp = TOKENS_PER_RANK, world_size
    rows_global = m * cp
    q_local, kv_local, shard = Q_HEADS // cp * HEAD_DIM, KV_HEADS // cp * HEAD_DIM, OPROJ_K // cp
    u32, bf16 = torch.int32, torch.bfloat16
    world = World(rank, world_size, local_rank)
    # Two sets of the routed buffers: the device-timed loop uses set 0; the end-to-end loop alternates.
    spec = {"qkv_done": cp * N.READY_FLAG_STRIDE * 4}
    for s in (0, 1):
        spec[f"qkv_planar{s}"] = rows_global * (QKV_N // cp) * 2   # this rank's Q | K | V after the all-to-all
        spec[f"attn_out{s}"] = rows_global * shard * 2             # this rank's head shard of attention output
        spec[f"attn_ready{s}"] = N.READY_FLAG_STRIDE * 4
    sym = world.allocate(spec)
    x = torch.empty(m, HIDDEN, dtype=bf16, device=dev)
    w_qkv = torch.empty(QKV_N, HIDDEN, dtype=bf16, device=dev)
    w_o = torch.empty(HIDDEN, OPROJ_K, dtype=bf16, device=dev)
    local_qkv = torch.empty(m, QKV_N, dtype=bf16, device=dev)
    staging = torch.empty(m, OPROJ_K, dtype=bf16, device=dev)
    out = torch.empty(m, HIDDEN, dtype=bf16, device=dev)
    planar = [sym[f"qkv_planar{s}"].view(bf16) for s in (0, 1)]
    attn = [sym[f"attn_out{s}"].view(bf16) for s in (0, 1)]
    seed = synthetic.rank_seed(rank)
    assert api.generate_bf16(x.data_ptr(), x.numel(), seed + 1000, 1.0, normal=True) == 0
    assert api.generate_bf16(attn[0].data_ptr(), attn[0].numel(), seed + 2000, 1.0, normal=True) == 0
    attn[1].copy_(attn[0])
    assert api.generate_bf16(w_qkv.data_ptr(), w_qkv.numel(), synthetic.BASE_SEED + 11, 0.02, normal=True) == 0
    assert api.generate_bf16(w_o.data_ptr(), w_o.numel(), synthetic.BASE_SEED + 17, 0.02, normal=True) == 0

    qkv_problem = N.GemmProblem(m, QKV_N, HIDDEN, raster=N.RASTER_ALONG_M, max_swizzle_size=args.swizzle)
    qkv_route = N.UlyssesRoute(world_size=cp, rank=rank, batch=1, global_seq=rows_global, seq_local=m,
                               q_heads=Q_HEADS, kv_heads=KV_HEADS, head_dim=HEAD_DIM, kind=N.ROUTE_QKV_GQA_PACK)
    qkv_ready = torch.zeros(api.qkv_ready_elements(qkv_problem), dtype=u32, device=dev)
    qkv = N.GemmA2AParams(lhs=x.data_ptr(), rhs_nt=w_qkv.data_ptr(), local_output=local_qkv.data_ptr(),
                          ready=qkv_ready.data_ptr(), gemm=qkv_problem, route=qkv_route,
                          num_comm_ctas=args.qkv_comm, epoch=0)
    o_problem = N.GemmProblem(m, HIDDEN, OPROJ_K, raster=N.RASTER_ALONG_N, max_swizzle_size=args.swizzle)
    o_route = N.UlyssesRoute(world_size=cp, rank=rank, batch=1, global_seq=rows_global, seq_local=m,
                             q_heads=Q_HEADS, head_dim=HEAD_DIM, kind=N.ROUTE_HEAD_TO_SEQUENCE,
                             direction=N.ROUTE_INVERSE)
    o_ready = torch.zeros(api.a2a_lhs_gemm_ready_elements(o_problem, o_route), dtype=u32, device=dev)
    oproj = N.A2AGemmParams(input_staging=staging.data_ptr(), rhs_nt=w_o.data_ptr(), output=out.data_ptr(),
                            ready=o_ready.data_ptr(), gemm=o_problem, route=o_route,
                            num_comm_ctas=args.oproj_comm, epoch=0)
    for peer in range(cp):
        qkv.peer_route_done_epoch[peer] = sym["qkv_done"].peer_ptrs[peer]

    stream = torch.cuda.current_stream()
    epoch = [0]

    def barrier():
        torch.cuda.synchronize()
        if world_size > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(values):
        t = torch.tensor(values, dtype=torch.float64, device=dev)
        if world_size > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t.cpu()]

    qkv_options = N.Options()
    qkv_options.flags = N.QKV_ROUTE_DIRECT if args.qkv_route == "direct" else N.QKV_ROUTE_COMM_CTAS

    def launch_qkv(buffers: int = 0):
        qkv.epoch = epoch[0]
        for peer in range(cp):
            qkv.peer_output[peer] = sym[f"qkv_planar{buffers}"].peer_ptrs[peer]
        rc = api.launch_gemm_a2a_cutlass(qkv, stream.cuda_stream, qkv_options)
        if rc:
            raise RuntimeError(f"launch_gemm_a2a_cutlass -> cudaError {rc}")

    def launch_oproj(buffers: int = 0, upstream: bool = False, options=None):
        oproj.epoch = epoch[0]
        oproj.input_epoch = epoch[0] if upstream else 0
        for peer in range(cp):
            oproj.peer_input[peer] = sym[f"attn_out{buffers}"].peer_ptrs[peer]
            oproj.peer_input_ready[peer] = sym[f"attn_ready{buffers}"].peer_ptrs[peer] if upstream else None
        rc = api.launch_a2a_gemm_cutlass(oproj, stream.cuda_stream, options)
        if rc:
            raise RuntimeError(f"launch_a2a_gemm_cutlass -> cudaError {rc}")

    def step():
        epoch[0] += 1
        launch_qkv()
        launch_oproj()

    def check_status(where):
        status = api.read_status(clear=True)
        if status[0]:
            raise RuntimeError(f"device wait gave up during {where}: {status[:8]}")

    # ---- device-resident throughput ----------------------------------------------------------
    # The clock sampler starts before the warm-up: opening NVML takes milliseconds, and a rank that
    # entered the timed region late would make every other rank wait in its first launch.
    sampler = (ClockSampler("GPU-" + str(torch.cuda.get_device_properties(local_rank).uuid), args.clock_period_ms * 1e-3)
               if rank == 0 else None)
    events = [torch.cuda.Event(enable_timing=True) for _ in range(2 * args.steps + 1)]
    barrier()
    for _ in range(args.warmup):
        step()
    check_status("warm-up")
    barrier()
    launches_before = api.launch_count()
    t0 = time.perf_counter()
    events[0].record(stream)
    for i in range(args.steps):
        epoch[0] += 1
        launch_qkv()
        events[2 * i + 1].record(stream)
        launch_oproj()
        events[2 * i + 2].record(stream)
    barrier()
    t1 = time.perf_counter()
    gpu_launches = api.launch_count() - launches_before
    clocks = sampler.window(t0, t1) if sampler else None
    check_status("timed region")
    total_ms = events[0].elapsed_time(events[-1])
    qkv_ms = sum(events[2 * i].elapsed_time(events[2 * i + 1]) for i in range(args.steps)) / args.steps
    oproj_ms = sum(events[2 * i + 1].elapsed_time(events[2 * i + 2]) for i in range(args.steps)) / args.steps
    total_ms, qkv_ms, oproj_ms = max_over_ranks([total_ms, qkv_ms, oproj_ms])
    ms_per_step = total_ms / args.steps

    def time_loop(fn, count):
        """Device time per call of `count` back-to-back calls (max over ranks)."""
        for _ in range(3):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(count):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return max_over_ranks([e0.elapsed_time(e1) / count])[0]

    # ---- pure GEMMs on all SMs (retention denominators): this library's, and cuBLASLt's --------
    pure, cublas = {}, {}
    if not args.skip_pure:
        pure["qkv"] = time_loop(lambda: api.launch_batched_cutlass_reference(qkv, stream.cuda_stream, 0), args.steps)
        pure["oproj"] = time_loop(lambda: api.launch_a2a_gemm_cutlass_reference(oproj, stream.cuda_stream, 0), args.steps)
        y_ref = torch.empty(m, QKV_N, dtype=bf16, device=dev)
        o_ref = torch.empty(m, HIDDEN, dtype=bf16, device=dev)
        cublas["qkv"] = time_loop(lambda: torch.matmul(x, w_qkv.t(), out=y_ref), args.steps)
        cublas["oproj"] = time_loop(lambda: torch.matmul(staging, w_o.t(), out=o_ref), args.steps)
        del y_ref, o_ref
        barrier()

    # ---- sustained: >= 2 s of back-to-back steps under the power cap ----------------------------
    sustained = None
    if args.sustained_s > 0:
        count = max(args.steps, int(args.sustained_s * 1e3 / ms_per_step) + 1)
        barrier()
        ts0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(count):
            step()
        e1.record(stream)
        barrier()
        ts1 = time.perf_counter()
        check_status("sustained region")
        sustained_ms = max_over_ranks([e0.elapsed_time(e1) / count])[0]
        sustained = {"steps": count, "seconds": sustained_ms * count * 1e-3, "ms_per_step": sustained_ms,
                     "per_gpu": FLOPS_PER_RANK / (sustained_ms * 1e-3) / 1e15,
                     "clocks": sampler.window(ts0, ts1) if sampler else None}

    # ---- the same work as separate kernels: cuBLASLt GEMM + pack + NCCL all_to_all_single ------
    segments = ((0, Q_HEADS * HEAD_DIM, q_local), (Q_HEADS * HEAD_DIM, KV_HEADS * HEAD_DIM, kv_local),
                ((Q_HEADS + KV_HEADS) * HEAD_DIM, KV_HEADS * HEAD_DIM, kv_local))

    def nccl_route_qkv(y, planar_out):
        """Sequence -> head all-to-all of a [M, 6144] projection into a planar Q | K | V buffer."""
        base = 0
        for first, width, local_width in segments:
            send = y[:, first:first + width].view(m, cp, local_width).transpose(0, 1).contiguous()  # [dest, M, w]
            recv = planar_out[base:base + rows_global * local_width].view(cp, m * local_width)
            if cp > 1:
                dist.all_to_all_single(recv, send.view(cp, m * local_width))
            else:
                recv.copy_(send.view(cp, m * local_width))
            base += rows_global * local_width

    def nccl_gather_attn(attn_in, staging_out):
        """Head -> sequence all-to-all of the head-sharded attention output into [M, K]."""
        send = attn_in.view(cp, m * shard)                     # rows of destination d are contiguous
        recv = torch.empty_like(send)
        if cp > 1:
            dist.all_to_all_single(recv, send)
        else:
            recv.copy_(send)
        staging_out.view(m, cp, shard).copy_(recv.view(cp, m, shard).transpose(0, 1))

    separate = None
    if not args.skip_separate:
        y_sep = torch.empty(m, QKV_N, dtype=bf16, device=dev)
        planar_sep = torch.empty_like(planar[0])
        staging_sep = torch.empty_like(staging)
        out_sep = torch.empty_like(out)

        def sep_qkv():
            torch.matmul(x, w_qkv.t(), out=y_sep)
            nccl_route_qkv(y_sep, planar_sep)

        def sep_oproj():
            nccl_gather_attn(attn[0], staging_sep)
            torch.matmul(staging_sep, w_o.t(), out=out_sep)

        sep_qkv_ms = time_loop(sep_qkv, args.steps)
        sep_oproj_ms = time_loop(sep_oproj, args.steps)
        separate = {"what": "torch.matmul (cuBLASLt) + pack copy + NCCL all_to_all_single (QKV: three, one per "
                            "planar segment); NCCL all_to_all_single + unpack copy + torch.matmul (OProj)",
                    "qkv_ms": sep_qkv_ms, "oproj_ms": sep_oproj_ms, "ms_per_step": sep_qkv_ms + sep_oproj_ms,
                    "per_gpu": FLOPS_PER_RANK / ((sep_qkv_ms + sep_oproj_ms) * 1e-3) / 1e15,
                    "fused_speedup": (sep_qkv_ms + sep_oproj_ms) / ms_per_step}
        del y_sep, out_sep, staging_sep
        barrier()

    # ---- end to end from pinned host buffers --------------------------------------------------
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    x_host = torch.empty(x.shape, dtype=bf16).pin_memory()
    attn_host = torch.empty(attn[0].shape, dtype=bf16).pin_memory()
    x_host.copy_(x)
    attn_host.copy_(attn[0])
    planar_host = torch.empty(planar[0].shape, dtype=bf16).pin_memory()
    out_host = torch.empty(out.shape, dtype=bf16).pin_memory()
    # one pinned flag line per step: the host runs ahead of the copies that read them
    flag_host = torch.zeros(e2e_steps + 2, N.READY_FLAG_STRIDE, dtype=u32).pin_memory()
    attn_flag = [sym[f"attn_ready{s}"].view(u32) for s in (0, 1)]
    h2d = x_host.numel() * 2 + attn_host.numel() * 2 + N.READY_FLAG_STRIDE * 4
    d2h = planar_host.numel() * 2 + out_host.numel() * 2

    # Three streams: uploads, the two fused kernels, downloads.  PCIe is full duplex, so a step's
    # downloads run beside the next uploads; events order every buffer's reuse (a kernel never
    # overwrites an output that is still being read back, an upload never overwrites an input that
    # a kernel still reads).  With peers, the buffers other ranks touch -- the planar Q|K|V they
    # push into and the attention shard they pull from -- alternate between two sets, and two local
    # rules make a host barrier unnecessary:
    #   * projection i+1 is launched only when the read-back of step i's planar tensor is done.  A
    #     peer's projection i+2 (which writes set i%2 again) cannot start before its projection i+1
    #     has finished, i.e. before every rank's projection i+1 has STARTED (the kernels end with a
    #     cross-rank completion handshake) -- so it starts after this rank's read-back of step i;
    #   * the upload of attention i+2 (set i%2 again) waits for this rank's projection i+1 to finish;
    #     by the same handshake every peer has then started projection i+1 and so finished pulling
    #     attention i (stream order on the peer).
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    new_event = lambda: torch.cuda.Event()
    state = {"planar_read": None, "out_read": None, "qkv_done": None, "oproj_done": None, "step": 0}

    def e2e_step():
        epoch[0] += 1
        b = state["step"] % 2 if world_size > 1 else 0
        with torch.cuda.stream(s_in):
            if state["qkv_done"] is not None:
                s_in.wait_event(state["qkv_done"])     # the previous projection has read x (and see above)
            x.copy_(x_host, non_blocking=True)
            x_ready = new_event()
            x_ready.record(s_in)
            if world_size == 1 and state["oproj_done"] is not None:
                s_in.wait_event(state["oproj_done"])   # the previous output projection has read attn
            attn[b].copy_(attn_host, non_blocking=True)
            line = flag_host[state["step"] % flag_host.shape[0]]
            state["step"] += 1
            line.fill_(epoch[0])
            attn_flag[b].copy_(line, non_blocking=True)  # upstream epoch: published after the payload
            attn_ready = new_event()
            attn_ready.record(s_in)
        stream.wait_event(x_ready)
        if state["planar_read"] is not None:
            stream.wait_event(state["planar_read"])    # the previous Q|K|V has been read back
        launch_qkv(b)
        state["qkv_done"] = new_event()
        state["qkv_done"].record(stream)
        stream.wait_event(attn_ready)
        if state["out_read"] is not None:
            stream.wait_event(state["out_read"])
        launch_oproj(b, upstream=True)
        state["oproj_done"] = new_event()
        state["oproj_done"].record(stream)
        with torch.cuda.stream(s_out):
            s_out.wait_event(state["qkv_done"])
            planar_host.copy_(planar[b], non_blocking=True)
            state["planar_read"] = new_event()
            state["planar_read"].record(s_out)
            s_out.wait_event(state["oproj_done"])
            out_host.copy_(out, non_blocking=True)
            state["out_read"] = new_event()
            state["out_read"].record(s_out)

    def e2e_join():
        torch.cuda.synchronize()
        if world_size > 1:
            dist.barrier()

    barrier()
    e2e_step()
    e2e_step()
    e2e_join()
    ta = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_join()  # every upload, kernel and download of the timed steps has finished
    tb = time.perf_counter()
    check_status("end-to-end region")
    e2e_ms = max_over_ranks([(tb - ta) * 1e3 / e2e_steps])[0]
    checksum = float(out_host[:64].float().abs().sum()) + float(planar_host[:64].float().abs().sum())
    del x_host, attn_host, planar_host, out_host

    # ---- full-size validation against the CPU oracle (outside every timed region) --------------
    validated = None
    if not args.skip_validate:
        from tests import fullsize as F
        F.use_host_threads(world_size)
        barrier()
        F.poison(local_qkv, planar[0], staging, out)
        barrier()
        step()
        torch.cuda.synchronize()  # no host barrier: this rank's kernels end only when the peers' pushes are in
        check_status("validation step")
        rows = F.sample_rows(m, count=args.validate_rows)
        qkv_check = F.check_qkv_forward(cp, rank, m, Q_HEADS, KV_HEADS, HEAD_DIM, x, w_qkv, local_qkv, planar[0], rows)
        oproj_check = F.check_oproj_forward(cp, rank, m, OPROJ_K, attn[0], staging, w_o, out, rows)
        validated = F.merge(qkv_check, oproj_check)
        validated["sample"] = (f"{len(rows)} rows per rank and operator (first and last 32 rows of the rank, seeded "
                               f"spread between), every column; routed elements of those rows from EVERY source rank")
        if separate is not None:
            # full size, on the device: the routed tensors against an NCCL all-to-all of the same values
            nccl_route_qkv(local_qkv, planar_sep)
            staging_ref = torch.empty_like(staging)
            nccl_gather_attn(attn[0], staging_ref)
            full = [bool(torch.equal(planar_sep.view(torch.int16), planar[0].view(torch.int16))),
                    bool(torch.equal(staging_ref.view(torch.int16), staging.view(torch.int16)))]
            flags = max_over_ranks([0.0 if full[0] else 1.0, 0.0 if full[1] else 1.0])
            validated["full_size_vs_nccl_all_to_all"] = {"qkv_routed_bitexact": flags[0] == 0.0,
                                                         "oproj_gathered_bitexact": flags[1] == 0.0,
                                                         "elements": int(planar[0].numel() + staging.numel()) * cp}
            validated["ok"] = bool(validated["ok"] and flags[0] == 0.0 and flags[1] == 0.0)
            del staging_ref
        barrier()
    if separate is not None:
        del planar_sep

    # ---- NVLink: algorithmic bytes of each routed kernel over its device time -------------------
    nvlink = None
    if world_size > 1:
        out_bytes = 2.0 * m * QKV_N * (cp - 1) / cp
        in_bytes = 2.0 * m * OPROJ_K * (cp - 1) / cp
        nvlink = {"qkv_gemm_a2a": {"bytes_out": out_bytes, "gbps": out_bytes / (qkv_ms * 1e-3) / 1e9,
                                   "frac_of_900": out_bytes / (qkv_ms * 1e-3) / 900e9},
                  "a2a_oproj_gemm": {"bytes_in": in_bytes, "gbps": in_bytes / (oproj_ms * 1e-3) / 1e9,
                                     "frac_of_900": in_bytes / (oproj_ms * 1e-3) / 900e9},
                  "note": "algorithmic bytes / CUDA-event time of the whole fused kernel (tensor-bound, so this is the "
                          "rate the transfer needs, not what the links can do)"}
        if not args.skip_copy_only:
            # the pull alone: communication CTAs only, compute CTAs leave at once
            os.environ["FUSE_B200_EMBEDDED_PULL"] = "0"
            copy_options = N.Options()
            copy_options.flags = N.COMM_ONLY
            saved = oproj.num_comm_ctas
            oproj.num_comm_ctas = args.copy_only_ctas

            def pull_only():
                epoch[0] += 1
                launch_oproj(0, options=copy_options)

            try:
                copy_ms = time_loop(pull_only, 10)
                status = api.read_status(clear=True)
                if status[0] == 0:
                    nvlink["copy_only"] = {"what": f"lhs pull alone: {args.copy_only_ctas} communication CTAs, no GEMM",
                                           "bytes_in": in_bytes, "ms": copy_ms, "gbps": in_bytes / (copy_ms * 1e-3) / 1e9,
                                           "frac_of_900": in_bytes / (copy_ms * 1e-3) / 900e9}
                else:
                    nvlink["copy_only"] = {"error": f"device wait gave up: {status[:8]}"}
            finally:
                oproj.num_comm_ctas = saved
                os.environ.pop("FUSE_B200_EMBEDDED_PULL", None)
            barrier()

    # ---- the other benchmark configurations ----------------------------------------------------
    others = None
    if not args.skip_others:
        import bench_suite
        del x, local_qkv, staging, out
        torch.cuda.empty_cache()
        ctx = bench_suite.Context(rank, world_size, local_rank, world, samples=args.other_samples, warmup=3,
                                  validate=not args.skip_validate, validate_rows=args.validate_rows)
        others = bench_suite.run(ctx, only=set(args.others.split(",")) if args.others != "all" else None)

    if sampler:
        sampler.close()
    if rank == 0:
        burst, sustained_peak, peak_source = measured_peaks()
        achieved = QKV_FLOPS / (qkv_ms * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": FLOPS_PER_RANK * world_size / (ms_per_step * 1e-3) / 1e15,
            "unit": "PFLOPS", "n_gpus": world_size, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": workload_config(world_size),
            "per_gpu": FLOPS_PER_RANK / (ms_per_step * 1e-3) / 1e15,
            "value_is": "whole-job PFLOPS over all ranks; per_gpu is the metric's PFLOPS/GPU",
            "kernels": {
                "qkv_gemm_a2a": {"ms": qkv_ms, "pflops_per_gpu": QKV_FLOPS / (qkv_ms * 1e-3) / 1e15,
                                 "route": args.qkv_route,
                                 "comm_ctas": ((args.qkv_comm or "auto") if args.qkv_route == "comm"
                                               else "none: every CTA computes, the epilogue pushes")},
                "a2a_oproj_gemm": {"ms": oproj_ms,
                                   "pflops_per_gpu": (FLOPS_PER_RANK - QKV_FLOPS) / (oproj_ms * 1e-3) / 1e15,
                                   "comm_ctas": args.oproj_comm or "auto",
                                   # Auto: the host planner decides (on B200: one warp of every compute CTA
                                   # pulls, no SM given up); an explicit budget means communication CTAs
                                   "pull": ("planner's choice" if args.oproj_comm == 0 and "FUSE_B200_EMBEDDED_PULL" not in os.environ
                                            else ("communication CTAs" if os.environ.get("FUSE_B200_EMBEDDED_PULL", "0") == "0"
                                                  else "embedded copy warps"))},
            },
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": burst, "unit": "TFLOP/s",
                         "frac": achieved / burst,
                         "traffic": (QKV_DRAM_TRAFFIC_BYTES_STORED_CAPTURE
                                     if args.qkv_route == "direct" and world_size == 1 else None),
                         "traffic_source": "stored ncu capture of this kernel and workload (one GPU), not re-measured here",
                         "kernel": ("pair_gemm_kernel<QkvDirect> (QKVProj GEMM -> A2A, CTA pairs)" if args.qkv_route == "direct"
                                    else "fused_gemm_kernel<256,4,QkvPush> (QKVProj GEMM -> A2A)"),
                         "peak_source": peak_source + ", burst figure: the kernel is timed in a short loop"},
            "e2e": {"value": FLOPS_PER_RANK * world_size / (e2e_ms * 1e-3) / 1e15, "unit": "PFLOPS",
                    "per_gpu": FLOPS_PER_RANK / (e2e_ms * 1e-3) / 1e15,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                    "h2d_gbps_per_rank": h2d / (e2e_ms * 1e-3) / 1e9, "d2h_gbps_per_rank": d2h / (e2e_ms * 1e-3) / 1e9,
                    "steps": e2e_steps, "checksum": checksum, "host_numa_node": numa_node,
                    "host_barrier_per_step": False},
            "gpu_launches": int(gpu_launches), "clocks": clocks,
        }
        if pure:
            line["pure_gemm_148sm"] = {
                "qkv_ms": pure["qkv"], "oproj_ms": pure["oproj"],
                "qkv_retention": pure["qkv"] / qkv_ms, "oproj_retention": pure["oproj"] / oproj_ms,
            }
            line["cublas"] = {"what": "torch.matmul (cuBLASLt) on the same operands, GEMM only",
                              "qkv_ms": cublas["qkv"], "oproj_ms": cublas["oproj"],
                              "qkv_retention": cublas["qkv"] / qkv_ms, "oproj_retention": cublas["oproj"] / oproj_ms}
        if sustained is not None:
            sustained["frac_of_sustained_peak"] = sustained["per_gpu"] * 1e3 / sustained_peak
            sustained["peak"] = sustained_peak
            line["sustained"] = sustained
        if separate is not None:
            line["separate_baseline"] = separate
        if validated is not None:
            line["validated"] = validated
        if nvlink is not None:
            line["nvlink"] = nvlink
        if others is not None:
            line["others"] = others
        if world_size == 1 and not args.skip_cpu:
            if original_affinity is not None:
                os.sched_setaffinity(0, original_affinity)
            cpu_step, flops, sample, cores = cpu_step_factory(rows=args.cpu_rows, threads=all_host_cores())
            cpu_step()
            tc = time.perf_counter()
            reps = 0
            while reps < 2 or time.perf_counter() - tc < 10.0:
                cpu_step()
                reps += 1
            cpu_s = (time.perf_counter() - tc) / reps
            line["cpu_baseline"] = {"value": flops / cpu_s / 1e15, "unit": "PFLOPS", "cores": cores,
                                    "kind": "port", "sample": sample}
        emit(line)
    barrier()
    world.close()
    if world_size > 1:
        dist.destroy_process_group()
    failed = [name for name, block in (("validated", validated),) if block is not None and not block["ok"]]
    if others is not None:
        failed += [f"others.{row['name']}" for row in others if row.get("validated") is not None and not row["validated"]["ok"]]
    if failed:
        sys.stderr.write(f"VALIDATION FAILED: {failed}\n")
        raise SystemExit(3)


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="fuse_b200", choices=["fuse_b200", "reference"])
    parser.add_argument("--qkv-comm", type=int, default=0, help="communication CTAs of the QKV operator (0: Auto)")
    parser.add_argument("--oproj-comm", type=int, default=0, help="communication CTAs of the OProj operator (0: Auto)")
    parser.add_argument("--swizzle", type=int, default=8)
    parser.add_argument("--qkv-route", default="direct", choices=["comm", "direct"],
                        help="QKV routing from communication CTAs or from the GEMM epilogue")
    parser.add_argument("--e2e-steps", type=int, default=10)
    parser.add_argument("--cpu-rows", type=int, default=1024)
    parser.add_argument("--clock-period-ms", type=float, default=10.0)
    parser.add_argument("--sustained-s", type=float, default=2.0)
    parser.add_argument("--validate-rows", type=int, default=256)
    parser.add_argument("--others", default="all", help="comma list of bwd,c3,c4,c5 (default all)")
    parser.add_argument("--other-samples", type=int, default=5)
    parser.add_argument("--copy-only-ctas", type=int, default=32)
    parser.add_argument("--skip-cpu", action="store_true")
    parser.add_argument("--skip-pure", action="store_true")
    parser.add_argument("--skip-separate", action="store_true")
    parser.add_argument("--skip-validate", action="store_true")
    parser.add_argument("--skip-others", action="store_true")
    parser.add_argument("--skip-copy-only", action="store_true")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup
    # Standard output carries the one JSON line and nothing else: whatever libraries print there
    # (NCCL's version banner, for one) goes to standard error instead.
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
