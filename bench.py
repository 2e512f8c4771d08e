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
reference's own way of quoting it (PFLOPS/GPU).  `e2e` runs the same step from pinned HOST
buffers with the host<->device copies inside the timed region: every step uploads its inputs and
downloads both results; uploads, kernels and downloads run on three streams ordered by events, so
a step's downloads overlap the next uploads (one GPU) -- the copies are still all inside the
timed region, which ends when the last download has finished.  `--impl reference` times the
CPU restatement of the path (the reference has no CPU implementation of the fused operators,
only host oracle pieces) on the host cores, on a bounded row sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes as C
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

# DRAM bytes (read + write) of one launch of the dominant kernel (the fused QKV kernel at this
# workload, context-parallel size 1, direct route, CTA pairs), dram__bytes_read.sum +
# dram__bytes_write.sum of the ncu capture summarised in profiles/pair_gemm_kernel_forward_c2_ncu.md.
QKV_DRAM_TRAFFIC_BYTES = 876_308_736


_RESULT_FD = None


def emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            data = json.load(f)
        return float(data["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    return 1590.0, "fallback (earlier pool measurement, burst)"


# --------------------------------------------------------------------------------------------
# CPU arm: the oracle port timed on the host cores
# --------------------------------------------------------------------------------------------

def cpu_step_factory(rows: int, world: int = 1):
    """Returns (step_fn, flops_per_step, description) for a `rows`-row sample of the workload."""
    import numpy as np
    from oracle import oracle as O
    L = O.lib()
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
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    step, flops, sample, cores = cpu_step_factory(rows=512)
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
    milliseconds while the timed region runs (a 50 ms region gets several samples; polling much
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

    def stop(self, t0, t1):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        sm, smax, reasons = [], [], set()
        if self.nvml is not None:
            self.stop_flag.set()
            self.thread.join(timeout=1.0)
            rows = [s for (t, s) in self.samples if t0 <= t <= t1] or [s for (_, s) in self.samples[-3:]]
            for clock, top, mask in rows:
                sm.append(clock)
                smax.append(top)
                reasons.update(name for name in names if mask & self.REASON_BITS[name])
            source = "nvml"
        elif self.proc is not None:
            time.sleep(0.12)
            self.proc.terminate()
            rows = [s for (t, s) in self.samples if t0 - 0.05 <= t <= t1 + 0.05] or [s for (_, s) in self.samples]
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
    if world_size > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    N.lib()  # fail loudly here if the CUDA library is missing

    m, cp = TOKENS_PER_RANK, world_size
    rows_global = m * cp
    u32, bf16 = torch.int32, torch.bfloat16
    world = World(rank, world_size, local_rank)
    sym = world.allocate({
        "qkv_planar": rows_global * (QKV_N // cp) * 2,      # this rank's Q | K | V after the all-to-all
        "qkv_done": cp * N.READY_FLAG_STRIDE * 4,
        "attn_out": rows_global * (OPROJ_K // cp) * 2,       # this rank's head shard of attention output
        "attn_ready": N.READY_FLAG_STRIDE * 4,
    })
    x = torch.empty(m, HIDDEN, dtype=bf16, device=dev)
    w_qkv = torch.empty(QKV_N, HIDDEN, dtype=bf16, device=dev)
    w_o = torch.empty(HIDDEN, OPROJ_K, dtype=bf16, device=dev)
    local_qkv = torch.empty(m, QKV_N, dtype=bf16, device=dev)
    staging = torch.empty(m, OPROJ_K, dtype=bf16, device=dev)
    out = torch.empty(m, HIDDEN, dtype=bf16, device=dev)
    attn = sym["attn_out"].view(bf16)
    seed = synthetic.rank_seed(rank)
    assert api.generate_bf16(x.data_ptr(), x.numel(), seed + 1000, 1.0, normal=True) == 0
    assert api.generate_bf16(attn.data_ptr(), attn.numel(), seed + 2000, 1.0, normal=True) == 0
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
        qkv.peer_output[peer] = sym["qkv_planar"].peer_ptrs[peer]
        qkv.peer_route_done_epoch[peer] = sym["qkv_done"].peer_ptrs[peer]
        oproj.peer_input[peer] = sym["attn_out"].peer_ptrs[peer]

    stream = torch.cuda.current_stream()
    epoch = [0]

    def barrier():
        torch.cuda.synchronize()
        if world_size > 1:
            dist.barrier()
        torch.cuda.synchronize()

    qkv_options = N.Options()
    qkv_options.flags = N.QKV_ROUTE_DIRECT if args.qkv_route == "direct" else N.QKV_ROUTE_COMM_CTAS

    def launch_qkv():
        qkv.epoch = epoch[0]
        rc = api.launch_gemm_a2a_cutlass(qkv, stream.cuda_stream, qkv_options)
        if rc:
            raise RuntimeError(f"launch_gemm_a2a_cutlass -> cudaError {rc}")

    def launch_oproj(upstream: bool = False):
        oproj.epoch = epoch[0]
        oproj.input_epoch = epoch[0] if upstream else 0
        for peer in range(cp):
            oproj.peer_input_ready[peer] = sym["attn_ready"].peer_ptrs[peer] if upstream else None
        rc = api.launch_a2a_gemm_cutlass(oproj, stream.cuda_stream)
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
    clocks = sampler.stop(t0, t1) if sampler else None
    check_status("timed region")
    total_ms = events[0].elapsed_time(events[-1])
    qkv_ms = sum(events[2 * i].elapsed_time(events[2 * i + 1]) for i in range(args.steps)) / args.steps
    oproj_ms = sum(events[2 * i + 1].elapsed_time(events[2 * i + 2]) for i in range(args.steps)) / args.steps
    times = torch.tensor([total_ms, qkv_ms, oproj_ms], dtype=torch.float64, device=dev)
    if world_size > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, qkv_ms, oproj_ms = (float(v) for v in times.cpu())
    ms_per_step = total_ms / args.steps

    # ---- pure GEMM on all SMs (the retention denominator) -------------------------------------
    pure = {}
    if not args.skip_pure:
        for name, fn, params in (("qkv", api.launch_batched_cutlass_reference, qkv),
                                 ("oproj", api.launch_a2a_gemm_cutlass_reference, oproj)):
            for _ in range(3):
                fn(params, stream.cuda_stream, 0)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(args.steps):
                fn(params, stream.cuda_stream, 0)
            e1.record(stream)
            torch.cuda.synchronize()
            pure[name] = e0.elapsed_time(e1) / args.steps
        barrier()

    # ---- end to end from pinned host buffers --------------------------------------------------
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    x_host = torch.empty(x.shape, dtype=bf16).pin_memory()
    attn_host = torch.empty(attn.shape, dtype=bf16).pin_memory()
    x_host.copy_(x)
    attn_host.copy_(attn)
    planar = sym["qkv_planar"].view(bf16)
    planar_host = torch.empty(planar.shape, dtype=bf16).pin_memory()
    out_host = torch.empty(out.shape, dtype=bf16).pin_memory()
    # one pinned flag line per step: the host runs ahead of the copies that read them
    flag_host = torch.zeros(e2e_steps + 1, N.READY_FLAG_STRIDE, dtype=u32).pin_memory()
    attn_flag = sym["attn_ready"].view(u32)
    h2d = x_host.numel() * 2 + attn_host.numel() * 2 + N.READY_FLAG_STRIDE * 4
    d2h = planar_host.numel() * 2 + out_host.numel() * 2

    # Three streams: uploads, the two fused kernels, downloads.  PCIe is full duplex, so a step's
    # downloads run beside the next uploads; events order every buffer's reuse (a kernel never
    # overwrites an output that is still being read back, an upload never overwrites an input that
    # a kernel still reads).  With peers (N > 1) every step ends with a host barrier, because a
    # peer may still be pulling this rank's attention output; on one GPU the steps overlap.
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    new_event = lambda: torch.cuda.Event()
    state = {"planar_read": None, "out_read": None, "qkv_done": None, "oproj_done": None, "step": 0}

    def e2e_step():
        epoch[0] += 1
        with torch.cuda.stream(s_in):
            if state["qkv_done"] is not None:
                s_in.wait_event(state["qkv_done"])     # the previous projection has read x
            x.copy_(x_host, non_blocking=True)
            x_ready = new_event()
            x_ready.record(s_in)
            if state["oproj_done"] is not None:
                s_in.wait_event(state["oproj_done"])   # the previous output projection has read attn
            attn.copy_(attn_host, non_blocking=True)
            line = flag_host[state["step"] % flag_host.shape[0]]
            state["step"] += 1
            line.fill_(epoch[0])
            attn_flag.copy_(line, non_blocking=True)  # upstream epoch: published after the payload
            attn_ready = new_event()
            attn_ready.record(s_in)
        stream.wait_event(x_ready)
        if state["planar_read"] is not None:
            stream.wait_event(state["planar_read"])    # the previous Q|K|V has been read back
        launch_qkv()
        state["qkv_done"] = new_event()
        state["qkv_done"].record(stream)
        stream.wait_event(attn_ready)
        if state["out_read"] is not None:
            stream.wait_event(state["out_read"])
        launch_oproj(upstream=True)
        state["oproj_done"] = new_event()
        state["oproj_done"].record(stream)
        with torch.cuda.stream(s_out):
            s_out.wait_event(state["qkv_done"])
            planar_host.copy_(planar, non_blocking=True)
            state["planar_read"] = new_event()
            state["planar_read"].record(s_out)
            s_out.wait_event(state["oproj_done"])
            out_host.copy_(out, non_blocking=True)
            state["out_read"] = new_event()
            state["out_read"].record(s_out)
        if world_size > 1:
            barrier()

    def e2e_join():
        torch.cuda.synchronize()
        if world_size > 1:
            dist.barrier()

    e2e_step()
    e2e_join()
    ta = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_join()  # every upload, kernel and download of the timed steps has finished
    tb = time.perf_counter()
    check_status("end-to-end region")
    e2e_ms = torch.tensor([(tb - ta) * 1e3 / e2e_steps], dtype=torch.float64, device=dev)
    if world_size > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_ms = float(e2e_ms.cpu())
    checksum = float(out_host[:64].float().abs().sum()) + float(planar_host[:64].float().abs().sum())

    if rank == 0:
        peak, peak_source = measured_peaks()
        achieved = QKV_FLOPS / (qkv_ms * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": FLOPS_PER_RANK * world_size / (ms_per_step * 1e-3) / 1e15,
            "unit": "PFLOPS", "n_gpus": world_size, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": workload_config(world_size),
            "per_gpu": FLOPS_PER_RANK / (ms_per_step * 1e-3) / 1e15,
            "kernels": {
                "qkv_gemm_a2a": {"ms": qkv_ms, "pflops_per_gpu": QKV_FLOPS / (qkv_ms * 1e-3) / 1e15,
                                 "route": args.qkv_route,
                                 "comm_ctas": args.qkv_comm if args.qkv_route == "comm" else 0},
                "a2a_oproj_gemm": {"ms": oproj_ms,
                                   "pflops_per_gpu": (FLOPS_PER_RANK - QKV_FLOPS) / (oproj_ms * 1e-3) / 1e15,
                                   "comm_ctas": args.oproj_comm,
                                   # the library's default: one warp of every compute CTA pulls (no SM
                                   # given up); FUSE_B200_EMBEDDED_PULL=0 selects communication CTAs
                                   "pull": ("embedded copy warps" if os.environ.get("FUSE_B200_EMBEDDED_PULL", "1") != "0"
                                            else "communication CTAs")},
            },
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak,
                         "traffic": QKV_DRAM_TRAFFIC_BYTES if args.qkv_route == "direct" and world_size == 1 else None,
                         "kernel": ("pair_gemm_kernel<QkvDirect> (QKVProj GEMM -> A2A, CTA pairs)" if args.qkv_route == "direct"
                                    else "fused_gemm_kernel<256,4,QkvPush> (QKVProj GEMM -> A2A)"),
                         "peak_source": peak_source},
            "e2e": {"value": FLOPS_PER_RANK * world_size / (e2e_ms * 1e-3) / 1e15, "unit": "PFLOPS",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                    "steps": e2e_steps, "checksum": checksum},
            "gpu_launches": int(gpu_launches), "clocks": clocks,
        }
        if pure:
            line["pure_gemm_148sm"] = {
                "qkv_ms": pure["qkv"], "oproj_ms": pure["oproj"],
                "qkv_retention": pure["qkv"] / qkv_ms, "oproj_retention": pure["oproj"] / oproj_ms,
            }
        if world_size == 1 and not args.skip_cpu:
            cpu_step, flops, sample, cores = cpu_step_factory(rows=args.cpu_rows)
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


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="fuse_b200", choices=["fuse_b200", "reference"])
    parser.add_argument("--qkv-comm", type=int, default=16)
    parser.add_argument("--oproj-comm", type=int, default=20)
    parser.add_argument("--swizzle", type=int, default=8)
    parser.add_argument("--qkv-route", default="direct", choices=["comm", "direct"],
                        help="QKV routing from communication CTAs or from the GEMM epilogue")
    parser.add_argument("--e2e-steps", type=int, default=10)
    parser.add_argument("--cpu-rows", type=int, default=1024)
    parser.add_argument("--clock-period-ms", type=float, default=10.0)
    parser.add_argument("--skip-cpu", action="store_true")
    parser.add_argument("--skip-pure", action="store_true")
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
