#!/usr/bin/env python
"""Throughput, retention and validation of every fused operator at the benchmark geometries other
than the forward pair bench.py itself reports -- one rank per GPU.

    python bench_suite.py [--only bwd,c3,c4,c5] [--scale S]           # one GPU (routes are local)
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 bench_suite.py

bench.py imports `run()` and folds the rows into its JSON line (`others`).  Each row: device time
(CUDA events, max over ranks, median of `samples` launches after warm-up), PFLOPS per GPU on the
algorithmic FLOPs, the same GEMM alone on all SMs with this library's kernel ("pure") and with
cuBLASLt where it offers the operation, retention = pure / fused, NVLink bytes the operator moves per
launch over its time, and `validated`: outputs poisoned, one more launch, a row sample against the
CPU oracle (tests/fullsize.py).  Geometries (tokens per rank fixed, weak scaling in the ranks):
  bwd BF16 backward of the Llama-3-8B layer   M 16384, QKV [6144, 4096], OProj [4096, 4096]
  c3  Llama-3-70B MXFP8 A2A->OProj            M 32768, N = K = 8192
  c4  Qwen3-32B MXFP8 QKV full backward       M 65536, H 5120, QKV 10240
  c5  MoE dispatch + FC1 BF16                 8192 tokens per rank, H 7168, 32 experts per rank, top-8, N 4096
Inputs are generated on the device from seeds; --scale shrinks the rows of c3/c4/c5 for a quick run."""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from fuse_b200 import _native as N  # noqa: E402
from fuse_b200 import api, synthetic  # noqa: E402
from fuse_b200.world import World  # noqa: E402

BF16, U8, I32 = torch.bfloat16, torch.uint8, torch.int32


class Context:
    def __init__(self, rank, world_size, local_rank, world: World, samples=5, warmup=3, validate=True,
                 validate_rows=256, scale=1.0, comm=0):
        self.rank, self.world_size, self.local_rank, self.world = rank, world_size, local_rank, world
        self.samples, self.warmup, self.validate, self.validate_rows = samples, warmup, validate, validate_rows
        self.scale, self.comm = scale, comm
        self.dev = torch.device("cuda", local_rank)
        self.stream = torch.cuda.current_stream().cuda_stream
        self.seed = synthetic.rank_seed(rank)

    def barrier(self):
        torch.cuda.synchronize()
        if self.world_size > 1:
            dist.barrier()

    def gen(self, shape, seed, scale):
        t = torch.empty(shape, dtype=BF16, device=self.dev)
        assert api.generate_bf16(t.data_ptr(), t.numel(), seed, scale, normal=True) == 0
        return t

    def fill(self, tensor, seed, scale):
        assert api.generate_bf16(tensor.data_ptr(), tensor.numel(), seed, scale, normal=True) == 0

    def scratch(self, nbytes):
        buf = torch.empty(nbytes + 256, dtype=U8, device=self.dev)
        return buf, (buf.data_ptr() + 255) // 256 * 256

    def sample(self, fn):
        """One launch between barriers; device milliseconds, max over ranks."""
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = fn()
        if isinstance(rc, int) and rc != 0:
            raise RuntimeError(f"launch failed with cudaError {rc}")
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device=self.dev)
        if self.world_size > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def median_ms(self, fn):
        for _ in range(self.warmup):
            self.sample(fn)
        return statistics.median(self.sample(fn) for _ in range(self.samples))

    def check_status(self, label):
        status = api.read_status()
        assert status[0] == 0, f"{label}: device wait gave up {status[:8]}"

    def row(self, name, fused, flops, pure=None, cublas=None, nvlink_bytes=None, nvlink_dir="in", extra=None):
        """fused / pure / cublas: callables that launch once (fused gets the next epoch itself)."""
        ms = self.median_ms(fused)
        self.check_status(name)
        rec = {"name": name, "ms": ms, "pflops_per_gpu": flops / ms / 1e12, "flops_per_launch": flops}
        if pure is not None:
            pure_ms = self.median_ms(pure)
            rec["pure"] = {"ms": pure_ms, "pflops": flops / pure_ms / 1e12,
                           "what": "this library's GEMM of the same M, N, K alone on all 148 SMs"}
            rec["retention"] = pure_ms / ms
        if cublas is not None:
            try:
                cublas_ms = self.median_ms(cublas)
                rec["cublas"] = {"ms": cublas_ms, "pflops": flops / cublas_ms / 1e12, "retention": cublas_ms / ms}
            except Exception as error:  # noqa: BLE001 - cuBLASLt may not offer the operation
                rec["cublas"] = {"unavailable": str(error).splitlines()[0][:200]}
        if nvlink_bytes is not None and self.world_size > 1:
            rec["nvlink"] = {f"bytes_{nvlink_dir}": nvlink_bytes, "gbps": nvlink_bytes / (ms * 1e-3) / 1e9,
                             "frac_of_900": nvlink_bytes / (ms * 1e-3) / 900e9}
        if extra:
            rec.update(extra)
        return rec


def _pure_bf16(ctx, m, n, k):
    """Callable launching this library's pure NT GEMM of the given size on fresh operands."""
    a, b, d = ctx.gen((m, k), 71, 1.0), ctx.gen((n, k), 72, 0.02), torch.empty((m, n), dtype=BF16, device=ctx.dev)
    p = N.GemmA2AParams(lhs=a.data_ptr(), rhs_nt=b.data_ptr(), local_output=d.data_ptr(),
                        gemm=N.GemmProblem(m, n, k, raster=N.RASTER_ALONG_M, max_swizzle_size=8), num_comm_ctas=1, epoch=1)
    keep = (a, b, d)
    return (lambda: api.launch_batched_cutlass_reference(p, ctx.stream, 0)), keep


def _pure_mxfp8(ctx, m, n, k):
    """Callable launching this library's pure block-scaled GEMM [m, n, k] on prepared operands."""
    act = ctx.gen((m, k), 73, 1.0)
    qd = torch.empty((m, k), dtype=U8, device=ctx.dev)
    qs = torch.empty(api.mxfp8_scale_bytes(m, k), dtype=U8, device=ctx.dev)
    assert api.quantize_mxfp8(act.data_ptr(), k, m, k, qd.data_ptr(), qs.data_ptr(), ctx.stream) == 0
    torch.cuda.synchronize()
    del act
    w = ctx.gen((n, k), 74, 0.02)
    out = torch.empty((m, n), dtype=BF16, device=ctx.dev)
    prob = N.GemmProblem(m, n, k, max_swizzle_size=8)
    rc, ws = api.gemm_a2a_mxfp8_workspace_size(prob)
    assert rc == 0
    buf, base = ctx.scratch(ws)
    pq = N.GemmA2AParams(rhs_nt=w.data_ptr(), local_output=out.data_ptr(), gemm=prob, num_comm_ctas=0, epoch=1)  # all SMs
    pure = N.Mxfp8GemmA2AParams(projection=pq, workspace=base, workspace_bytes=ws,
                                activation=N.Mxfp8Activation(data=qd.data_ptr(), scales=qs.data_ptr(),
                                                             data_bytes=qd.numel(), scale_bytes=qs.numel()))
    assert api.prepare_gemm_a2a_mxfp8(pure, ctx.stream) == 0
    torch.cuda.synchronize()
    keep = (qd, qs, out, buf, pure, w)
    e8m0 = getattr(torch, "float8_e8m0fnu", None)

    def cublas():
        if e8m0 is None:
            raise RuntimeError("this torch has no float8_e8m0fnu scale type")
        w_off = base - buf.data_ptr()
        wq = buf[w_off:w_off + n * k].view(n, k)
        ws_off = w_off + (n * k + 255) // 256 * 256
        wsf = buf[ws_off:ws_off + api.mxfp8_scale_bytes(n, k)]
        return torch._scaled_mm(qd.view(torch.float8_e4m3fn), wq.view(torch.float8_e4m3fn).t(), scale_a=qs.view(e8m0),
                                scale_b=wsf.view(e8m0), out_dtype=BF16)

    return (lambda: api.launch_gemm_a2a_mxfp8_compute_reference(pure, ctx.stream)), cublas, keep


def _merge(ctx, *checks):
    from tests import fullsize as F
    return F.merge(*checks)


# ---------------------------------------------------------------------------------------------------
# BF16 backward of the Llama-3-8B layer
# ---------------------------------------------------------------------------------------------------

def run_bwd(ctx: Context):
    cp, rank, dev, stream = ctx.world_size, ctx.rank, ctx.dev, ctx.stream
    m, hid, q, kv, d = 16384, 4096, 32, 8, 128
    n, k_o = (q + 2 * kv) * d, q * d
    rows = m * cp
    rows_out = []
    x, wq, wo = ctx.gen((m, hid), ctx.seed + 1000, 1.0), ctx.gen((n, hid), 11, 0.02), ctx.gen((hid, k_o), 17, 0.02)
    bp = N.QkvBackwardDataParams(local_tokens=m, hidden=hid, batch=1, q_heads=q, kv_heads=kv, head_dim=d,
                                 world_size=cp, rank=rank, num_comm_ctas=ctx.comm, epoch=0)
    bp.gemm_tuning.max_swizzle_size = 1  # the reference's default tuning (backward_common.h:33-37)
    sym = ctx.world.allocate({"b_staging": m * n * 2, "b_done": cp * 128, "b_done2": cp * 128,
                              "b_gattn": rows * (k_o // cp) * 2, "b_ready": api.qkv_backward_ready_elements(bp) * 4})
    planes = [ctx.gen((rows, h // cp * d), ctx.seed + 100 * i + 101, 0.01) for i, h in enumerate((q, kv, kv))]
    dx = torch.empty((m, hid), dtype=BF16, device=dev)
    staging = sym["b_staging"].view(BF16).view(m, n)
    bp.grad_q, bp.grad_k, bp.grad_v = (t.data_ptr() for t in planes)
    bp.weight, bp.grad_input = wq.data_ptr(), dx.data_ptr()
    for r in range(cp):
        bp.peer_dqkv_staging[r] = sym["b_staging"].peer_ptrs[r]
        bp.peer_ready[r] = sym["b_ready"].peer_ptrs[r]
        bp.peer_done_epoch[r] = sym["b_done"].peer_ptrs[r]
    epoch = [0]

    def qkv_b():
        epoch[0] += 1
        bp.epoch = epoch[0]
        return api.launch_qkv_backward_data(bp, stream)

    dw = torch.empty((n, hid), dtype=BF16, device=dev)
    wparams = N.QkvBackwardWeightParams(dqkv_staging=staging.data_ptr(), saved_input=x.data_ptr(),
                                        grad_weight=dw.data_ptr(), local_tokens=m, hidden=hid, q_heads=q,
                                        kv_heads=kv, head_dim=d)
    qkv_flops = 2.0 * m * n * hid
    pure_d, keep_d = _pure_bf16(ctx, m, hid, n)       # dX[M, H] = dQKV[M, QKV] W : M x H x QKV
    rows_out.append(ctx.row("bwd BF16 QKV backward data (reverse A2A -> dX)", qkv_b, qkv_flops, pure=pure_d,
                            cublas=lambda: torch.matmul(staging, wq, out=dx),
                            nvlink_bytes=2.0 * m * n * (cp - 1) / cp, nvlink_dir="out"))
    del keep_d, pure_d
    pure_w, keep_w = _pure_bf16(ctx, n, hid, m)       # dW[QKV, H] = dQKV^T X : QKV x H x M
    rows_out.append(ctx.row("bwd BF16 QKV backward weight (local dW)", lambda: api.launch_qkv_backward_weight(wparams, stream),
                            qkv_flops, pure=pure_w, cublas=lambda: torch.matmul(staging.t(), x, out=dw)))
    del keep_w, pure_w
    if ctx.validate:
        from tests import fullsize as F
        ctx.barrier()
        F.poison(staging, dx, dw)
        ctx.barrier()
        qkv_b()
        torch.cuda.synchronize()
        assert api.launch_qkv_backward_weight(wparams, stream) == 0
        torch.cuda.synchronize()
        ctx.check_status("bwd validation")
        picked = F.sample_rows(m, count=ctx.validate_rows)
        data = F.check_qkv_backward_data(cp, rank, m, q, kv, d, planes, wq, staging, dx, picked)
        weight = F.check_weight_gradient(staging, x, dw, F.sample_rows(n, count=64, edge=8))
        rows_out[-2]["validated"] = _merge(ctx, data)
        rows_out[-1]["validated"] = _merge(ctx, weight)
        ctx.barrier()

    dy = ctx.gen((m, hid), ctx.seed + 301, 0.01)
    da = torch.empty((m, k_o), dtype=BF16, device=dev)
    saved = ctx.gen((m, k_o), ctx.seed + 302, 1.0)
    routed = sym["b_gattn"].view(BF16)
    op = N.OprojBackwardDataParams(grad_output=dy.data_ptr(), weight=wo.data_ptr(), local_grad_attention=da.data_ptr(),
                                   local_tokens=m, hidden=hid, batch=1, q_heads=q, head_dim=d, world_size=cp,
                                   rank=rank, num_comm_ctas=ctx.comm, epoch=0)
    op.gemm_tuning.max_swizzle_size = 1  # the reference's default tuning; 8 measured 5 % slower here
    for r in range(cp):
        op.peer_grad_attention[r] = sym["b_gattn"].peer_ptrs[r]
        op.peer_done_epoch[r] = sym["b_done2"].peer_ptrs[r]

    def oproj_b():
        epoch[0] += 1
        op.epoch = epoch[0]
        return api.launch_oproj_backward_data(op, stream)

    dwo = torch.empty((hid, k_o), dtype=BF16, device=dev)
    ow = N.OprojBackwardWeightParams(grad_output=dy.data_ptr(), saved_attention=saved.data_ptr(),
                                     grad_weight=dwo.data_ptr(), local_tokens=m, hidden=hid, q_heads=q, head_dim=d)
    o_flops = 2.0 * m * k_o * hid
    pure_o, keep_o = _pure_bf16(ctx, m, k_o, hid)
    rows_out.append(ctx.row("bwd BF16 OProj backward data (dA -> A2A)", oproj_b, o_flops, pure=pure_o,
                            cublas=lambda: torch.matmul(dy, wo, out=da),
                            nvlink_bytes=2.0 * m * k_o * (cp - 1) / cp, nvlink_dir="out"))
    del keep_o, pure_o
    pure_ow, keep_ow = _pure_bf16(ctx, hid, k_o, m)
    rows_out.append(ctx.row("bwd BF16 OProj backward weight (local dWo)", lambda: api.launch_oproj_backward_weight(ow, stream),
                            o_flops, pure=pure_ow, cublas=lambda: torch.matmul(dy.t(), saved, out=dwo)))
    del keep_ow, pure_ow
    if ctx.validate:
        from tests import fullsize as F
        ctx.barrier()
        F.poison(da, routed, dwo)
        ctx.barrier()
        oproj_b()
        torch.cuda.synchronize()
        assert api.launch_oproj_backward_weight(ow, stream) == 0
        torch.cuda.synchronize()
        ctx.check_status("bwd oproj validation")
        picked = F.sample_rows(m, count=ctx.validate_rows)
        data = F.check_oproj_backward_data(cp, rank, m, k_o, dy, wo, da, routed, picked)
        weight = F.check_weight_gradient(dy, saved, dwo, F.sample_rows(hid, count=64, edge=8))
        rows_out[-2]["validated"] = _merge(ctx, data)
        rows_out[-1]["validated"] = _merge(ctx, weight)
        ctx.barrier()
    return rows_out


# ---------------------------------------------------------------------------------------------------
# C3: Llama-3-70B MXFP8 A2A -> OProj
# ---------------------------------------------------------------------------------------------------

def run_c3(ctx: Context):
    cp, rank, dev, stream = ctx.world_size, ctx.rank, ctx.dev, ctx.stream
    m = max(256, int(32768 * ctx.scale) // 256 * 256)
    nk, heads, d = 8192, 64, 128
    rows, shard = m * cp, nk // cp
    sb = api.mxfp8_scale_bytes(rows, shard)
    sym = ctx.world.allocate({"c3_data": rows * shard, "c3_scales": sb})
    src = ctx.gen((rows, shard), ctx.seed + 2000, 1.0)
    assert api.quantize_mxfp8(src.data_ptr(), shard, rows, shard, sym["c3_data"].local.data_ptr(),
                              sym["c3_scales"].local.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    del src
    w = ctx.gen((nk, nk), 17, 0.02)
    out = torch.empty((m, nk), dtype=BF16, device=dev)
    prob = N.GemmProblem(m, nk, nk, raster=N.RASTER_ALONG_N, max_swizzle_size=8)
    rc, ws = api.a2a_gemm_mxfp8_workspace_size(prob)
    assert rc == 0
    buf, base = ctx.scratch(ws)
    route = N.UlyssesRoute(world_size=cp, rank=rank, batch=1, global_seq=rows, seq_local=m, q_heads=heads, head_dim=d,
                           kind=N.ROUTE_HEAD_TO_SEQUENCE, direction=N.ROUTE_INVERSE)
    proj = N.A2AGemmParams(rhs_nt=w.data_ptr(), output=out.data_ptr(), gemm=prob, route=route,
                           num_comm_ctas=ctx.comm, epoch=0)
    mp = N.Mxfp8A2AGemmParams(projection=proj, workspace=base, workspace_bytes=ws)
    for r in range(cp):
        mp.activation[r] = N.Mxfp8Activation(data=sym["c3_data"].peer_ptrs[r], scales=sym["c3_scales"].peer_ptrs[r],
                                             data_bytes=rows * shard, scale_bytes=sb)
    epoch = [0]

    def mx_oproj():
        epoch[0] += 1
        mp.projection.epoch = epoch[0]
        return api.launch_a2a_gemm_mxfp8_cutlass(mp, stream)

    pure, cublas, keep = _pure_mxfp8(ctx, m, nk, nk)
    flops = 2.0 * m * nk * nk
    rec = ctx.row(f"c3 MXFP8 A2A->OProj (M {m}, N = K = 8192)", mx_oproj, flops, pure=pure, cublas=cublas,
                  nvlink_bytes=m * nk * (1 + 1 / 32) * (cp - 1) / cp, nvlink_dir="in")
    del keep, pure, cublas
    if ctx.validate:
        from tests import fullsize as F
        ctx.barrier()
        F.poison(out)
        buf.fill_(0xA5)
        ctx.barrier()
        mx_oproj()
        torch.cuda.synchronize()
        ctx.check_status("c3 validation")
        view = api.a2a_gemm_mxfp8_staging_view(mp)
        off, soff, w0 = view.data - buf.data_ptr(), view.scales - buf.data_ptr(), base - buf.data_ptr()
        staged = buf[off:off + m * nk].view(m, nk)
        staged_scales = buf[soff:soff + view.scale_bytes]
        wq = buf[w0:w0 + nk * nk].view(nk, nk)
        wsf = buf[w0 + nk * nk:w0 + nk * nk + api.mxfp8_scale_bytes(nk, nk)]  # nk * nk is a multiple of 256
        picked = F.sample_rows(m, count=ctx.validate_rows)
        check = F.check_oproj_forward_mxfp8(cp, rank, m, nk, sym["c3_data"].local.view(rows, shard), sym["c3_scales"].local,
                                            staged, staged_scales, w, wq, wsf, out, picked)
        rec["validated"] = _merge(ctx, check)
        ctx.barrier()
    return [rec]


# ---------------------------------------------------------------------------------------------------
# MXFP8 QKV forward at the Llama-3-8B shape (the a6 operator; not a BASELINE config, measured for completeness)
# ---------------------------------------------------------------------------------------------------

def run_a6(ctx: Context):
    cp, rank, dev, stream = ctx.world_size, ctx.rank, ctx.dev, ctx.stream
    m, hid, q, kv, d = 16384, 4096, 32, 8, 128
    n, rows = (q + 2 * kv) * d, m * cp
    sym = ctx.world.allocate({"a6_planar": rows * (n // cp) * 2, "a6_done": cp * 128})
    x = ctx.gen((m, hid), ctx.seed + 1000, 1.0)
    xq = torch.empty((m, hid), dtype=U8, device=dev)
    xs = torch.zeros(api.mxfp8_scale_bytes(m, hid), dtype=U8, device=dev)
    assert api.quantize_mxfp8(x.data_ptr(), hid, m, hid, xq.data_ptr(), xs.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    del x
    w = ctx.gen((n, hid), 11, 0.02)
    local = torch.empty((m, n), dtype=BF16, device=dev)
    prob = N.GemmProblem(m, n, hid, raster=N.RASTER_ALONG_M, max_swizzle_size=8)
    rc, ws = api.gemm_a2a_mxfp8_workspace_size(prob)
    assert rc == 0
    buf, base = ctx.scratch(ws)
    route = N.UlyssesRoute(world_size=cp, rank=rank, batch=1, global_seq=rows, seq_local=m, q_heads=q, kv_heads=kv,
                           head_dim=d, kind=N.ROUTE_QKV_GQA_PACK)
    ready = torch.zeros(api.qkv_ready_elements(prob), dtype=torch.int32, device=dev)
    proj = N.GemmA2AParams(rhs_nt=w.data_ptr(), local_output=local.data_ptr(), ready=ready.data_ptr(), gemm=prob,
                           route=route, num_comm_ctas=ctx.comm, epoch=0)
    for r in range(cp):
        proj.peer_output[r] = sym["a6_planar"].peer_ptrs[r]
        proj.peer_route_done_epoch[r] = sym["a6_done"].peer_ptrs[r]
    mp = N.Mxfp8GemmA2AParams(projection=proj, workspace=base, workspace_bytes=ws,
                              activation=N.Mxfp8Activation(data=xq.data_ptr(), scales=xs.data_ptr(),
                                                           data_bytes=xq.numel(), scale_bytes=xs.numel()))
    opts = N.Options()
    opts.flags = 0 if ctx.comm else N.QKV_ROUTE_DIRECT
    epoch = [0]

    def mx_qkv():
        epoch[0] += 1
        mp.projection.epoch = epoch[0]
        return api.launch_gemm_a2a_mxfp8_cutlass(mp, stream, opts)

    pure, cublas, keep = _pure_mxfp8(ctx, m, n, hid)
    rec = ctx.row(f"a6 MXFP8 QKVProj->A2A (M {m}, N {n}, K {hid}, W quantised in-kernel)", mx_qkv, 2.0 * m * n * hid,
                  pure=pure, cublas=cublas, nvlink_bytes=2.0 * m * n * (cp - 1) / cp, nvlink_dir="out")
    del keep, pure, cublas
    if ctx.validate:
        from tests import fullsize as F
        ctx.barrier()
        F.poison(local, sym["a6_planar"].view(BF16))
        buf.fill_(0xA5)
        ctx.barrier()
        assert mx_qkv() == 0
        torch.cuda.synchronize()
        ctx.check_status("a6 validation")
        ctx.barrier()
        w0 = base - buf.data_ptr()
        wq = buf[w0:w0 + n * hid].view(n, hid)
        sf0 = w0 + (n * hid + 255) // 256 * 256
        wsf = buf[sf0:sf0 + api.mxfp8_scale_bytes(n, hid)]
        picked = F.sample_rows(m, count=ctx.validate_rows)
        check = F.check_qkv_forward_mxfp8(cp, rank, m, q, kv, d, xq, xs, w, wq, wsf, local, sym["a6_planar"].view(BF16),
                                          picked)
        rec["validated"] = _merge(ctx, check)
        ctx.barrier()
    return [rec]


# ---------------------------------------------------------------------------------------------------
# MXFP8 output-projection backward at the Llama-3-70B shape (the other half of a10; not a BASELINE config)
# ---------------------------------------------------------------------------------------------------

def run_a10(ctx: Context):
    cp, rank, dev, stream = ctx.world_size, ctx.rank, ctx.dev, ctx.stream
    m = max(256, int(32768 * ctx.scale) // 256 * 256)
    hid, q, d = 8192, 64, 128
    a, rows = q * d, m * cp
    sym = ctx.world.allocate({"a10_routed": rows * (a // cp) * 2, "a10_done": cp * 128})
    dy = ctx.gen((m, hid), ctx.seed + 301, 0.01)
    dyq = torch.empty((m, hid), dtype=U8, device=dev)
    dys = torch.zeros(api.mxfp8_scale_bytes(m, hid), dtype=U8, device=dev)
    assert api.quantize_mxfp8(dy.data_ptr(), hid, m, hid, dyq.data_ptr(), dys.data_ptr(), stream) == 0
    wo = ctx.gen((hid, a), 17, 0.02)
    saved = ctx.gen((m, a), ctx.seed + 302, 1.0)
    da = torch.empty((m, a), dtype=BF16, device=dev)
    dwo = torch.empty((hid, a), dtype=BF16, device=dev)
    routed = sym["a10_routed"].view(BF16)
    proj = N.OprojBackwardDataParams(weight=wo.data_ptr(), local_grad_attention=da.data_ptr(), local_tokens=m, hidden=hid,
                                     batch=1, q_heads=q, head_dim=d, world_size=cp, rank=rank,
                                     num_comm_ctas=ctx.comm or 16, epoch=0)
    proj.gemm_tuning.max_swizzle_size = 1
    for r in range(cp):
        proj.peer_grad_attention[r] = sym["a10_routed"].peer_ptrs[r]
        proj.peer_done_epoch[r] = sym["a10_done"].peer_ptrs[r]
    rc, ws = api.oproj_backward_mxfp8_data_workspace_size(proj)
    assert rc == 0
    buf, base = ctx.scratch(ws)
    mp = N.Mxfp8OprojBackwardDataParams(projection=proj, grad_output=N.Mxfp8Activation(
        data=dyq.data_ptr(), scales=dys.data_ptr(), data_bytes=dyq.numel(), scale_bytes=dys.numel()),
        workspace=base, workspace_bytes=ws)
    wproj = N.OprojBackwardWeightParams(grad_output=dy.data_ptr(), saved_attention=saved.data_ptr(),
                                        grad_weight=dwo.data_ptr(), local_tokens=m, hidden=hid, q_heads=q, head_dim=d)
    rc, ws2 = api.oproj_backward_mxfp8_weight_workspace_size(wproj)
    assert rc == 0
    buf2, base2 = ctx.scratch(ws2)
    wp = N.Mxfp8OprojBackwardWeightParams(projection=wproj, workspace=base2, workspace_bytes=ws2)
    epoch = [0]

    def data():
        epoch[0] += 1
        mp.projection.epoch = epoch[0]
        return api.launch_oproj_backward_mxfp8_data(mp, stream)

    def weight():
        return api.launch_oproj_backward_mxfp8_weight(wp, stream)

    flops = 2.0 * m * hid * a
    pure, cublas, keep = _pure_mxfp8(ctx, m, a, hid)
    data_row = ctx.row(f"a10 MXFP8 OProj backward data (M {m}: dA -> A2A, incl. Wo^T quantisation)", data, flops, pure=pure,
                       cublas=cublas, nvlink_bytes=2.0 * m * a * (cp - 1) / cp, nvlink_dir="out")
    del keep, pure, cublas
    pure, cublas, keep = _pure_mxfp8(ctx, hid, a, m)
    weight_row = ctx.row("a10 MXFP8 OProj backward weight (two transposed quantisations + dWo)", weight, flops, pure=pure,
                         cublas=cublas)
    del keep, pure, cublas
    if ctx.validate:
        from tests import fullsize as F
        ctx.barrier()
        F.poison(da, dwo, routed)
        ctx.barrier()
        assert data() == 0 and weight() == 0
        torch.cuda.synchronize()
        ctx.check_status("a10 validation")
        ctx.barrier()
        picked = F.sample_rows(m, count=ctx.validate_rows)
        check_d = F.check_oproj_backward_data_mxfp8(cp, rank, m, a, dyq, dys, wo, da, routed.view(rows, a // cp), picked)
        check_w = F.check_weight_gradient_mxfp8(dy, saved, dwo, F.sample_rows(hid, count=64, edge=8),
                                                F.sample_rows(a, count=512, edge=16))
        data_row["validated"] = _merge(ctx, check_d)
        weight_row["validated"] = _merge(ctx, check_w)
        ctx.barrier()
    return [data_row, weight_row]


# ---------------------------------------------------------------------------------------------------
# C4: Qwen3-32B MXFP8 QKV full backward
# ---------------------------------------------------------------------------------------------------

def run_c4(ctx: Context):
    cp, rank, dev, stream = ctx.world_size, ctx.rank, ctx.dev, ctx.stream
    m = max(256, int(65536 * ctx.scale) // 256 * 256)
    hid, q, kv, d = 5120, 64, 8, 128
    width, rows = (q + 2 * kv) * d, m * cp
    names, heads = ("q", "k", "v"), (q, kv, kv)
    spec = {}
    for nm, h in zip(names, heads):
        pw = h // cp * d
        spec[f"c4_{nm}8"] = rows * pw
        spec[f"c4_{nm}s"] = api.mxfp8_scale_bytes(rows, pw)
        spec[f"c4_{nm}m"] = rows * pw * 2
    spec["c4_done"] = cp * 128
    sym = ctx.world.allocate(spec)
    for i, (nm, h) in enumerate(zip(names, heads)):
        pw = h // cp * d
        master = sym[f"c4_{nm}m"].local
        assert api.generate_bf16(master.data_ptr(), rows * pw, ctx.seed + 100 * i + 101, 0.01, True) == 0
        assert api.quantize_mxfp8(master.data_ptr(), pw, rows, pw, sym[f"c4_{nm}8"].local.data_ptr(),
                                  sym[f"c4_{nm}s"].local.data_ptr(), stream) == 0
    w = ctx.gen((width, hid), 11, 0.02)
    x = ctx.gen((m, hid), ctx.seed + 1000, 1.0)
    staging = torch.empty((m, width), dtype=BF16, device=dev)
    dx = torch.empty((m, hid), dtype=BF16, device=dev)
    dw = torch.empty((width, hid), dtype=BF16, device=dev)
    proj = N.QkvBackwardDataParams(weight=w.data_ptr(), grad_input=dx.data_ptr(), local_tokens=m, hidden=hid, batch=1,
                                   q_heads=q, kv_heads=kv, head_dim=d, world_size=cp, rank=rank,
                                   num_comm_ctas=ctx.comm, epoch=0)
    proj.gemm_tuning.max_swizzle_size = 8
    ready = torch.zeros(api.qkv_backward_ready_elements(proj), dtype=I32, device=dev)
    proj.peer_dqkv_staging[rank] = staging.data_ptr()
    proj.peer_ready[rank] = ready.data_ptr()
    for r in range(cp):
        proj.peer_done_epoch[r] = sym["c4_done"].peer_ptrs[r]
    rc, ws = api.qkv_backward_mxfp8_data_workspace_size(proj)
    wproj = N.QkvBackwardWeightParams(dqkv_staging=staging.data_ptr(), saved_input=x.data_ptr(), grad_weight=dw.data_ptr(),
                                      local_tokens=m, hidden=hid, q_heads=q, kv_heads=kv, head_dim=d)
    rc2, ws2 = api.qkv_backward_mxfp8_weight_workspace_size(wproj)
    assert rc == 0 and rc2 == 0
    buf, base = ctx.scratch(ws)         # the data phase's quantised W^T and packed lhs stay for the validation
    buf2, base2 = ctx.scratch(ws2)
    mp = N.Mxfp8QkvBackwardDataParams(projection=proj, workspace=base, workspace_bytes=ws)
    for r in range(cp):
        acts = [N.Mxfp8Activation(data=sym[f"c4_{nm}8"].peer_ptrs[r], scales=sym[f"c4_{nm}s"].peer_ptrs[r],
                                  data_bytes=spec[f"c4_{nm}8"], scale_bytes=spec[f"c4_{nm}s"]) for nm in names]
        mp.peer_input[r] = N.Mxfp8QkvBackwardInput(grad_q=acts[0], grad_k=acts[1], grad_v=acts[2],
                                                   master_q=sym["c4_qm"].peer_ptrs[r], master_k=sym["c4_km"].peer_ptrs[r],
                                                   master_v=sym["c4_vm"].peer_ptrs[r])
    wp = N.Mxfp8QkvBackwardWeightParams(projection=wproj, workspace=base2, workspace_bytes=ws2)
    full = N.Mxfp8QkvBackwardParams(data=mp, weight=wp, weight_mode=0)
    epoch = [0]

    def data_phase():
        epoch[0] += 1
        mp.projection.epoch = epoch[0]
        return api.launch_qkv_backward_mxfp8_data(mp, stream)

    def full_backward():
        epoch[0] += 1
        full.data.projection.epoch = epoch[0]
        return api.launch_qkv_backward_mxfp8(full, stream)

    # the two HBM-bound quantiser kernels of the weight phase, alone (measured first, before the long GEMM
    # sequences heat the part): 2 B read + 1.03 B written per element
    probe = ctx.gen((m, width), 7, 0.01)
    qa = torch.empty((width, m), dtype=U8, device=dev)
    qas = torch.empty(api.mxfp8_scale_bytes(width, m), dtype=U8, device=dev)
    t_ms = ctx.median_ms(lambda: api.quantize_mxfp8_transposed(probe.data_ptr(), width, m, width, qa.data_ptr(),
                                                               qas.data_ptr(), stream))
    r_ms = ctx.median_ms(lambda: api.quantize_mxfp8(probe.data_ptr(), width, m, width, qa.data_ptr(), qas.data_ptr(), stream))
    quant_bytes = m * width * (2 + 1 + 1 / 32)
    quantisers = {"name": "c4 K32 quantisers alone (staging [M, 10240])", "bound": "hbm", "bytes_per_launch": quant_bytes,
                  "transposed": {"ms": t_ms, "gbps": quant_bytes / (t_ms * 1e-3) / 1e9},
                  "row_wise": {"ms": r_ms, "gbps": quant_bytes / (r_ms * 1e-3) / 1e9}}
    del qa, qas, probe
    torch.cuda.empty_cache()
    flops = 2.0 * m * hid * width
    pull_bytes = m * width * (3.0 + 1.0 / 32) * (cp - 1) / cp  # E4M3 + scales + BF16 masters
    pure_d, cublas_d, keep_d = _pure_mxfp8(ctx, m, hid, width)
    data_row = ctx.row(f"c4 MXFP8 QKV backward data (M {m}: pull -> dX, incl. W^T quantisation)", data_phase, flops,
                       pure=pure_d, cublas=cublas_d, nvlink_bytes=pull_bytes, nvlink_dir="in")
    del keep_d, pure_d, cublas_d
    torch.cuda.empty_cache()
    pure_w, cublas_w, keep_w = _pure_mxfp8(ctx, width, hid, m)
    weight_row = ctx.row("c4 MXFP8 QKV backward weight (two transposed quantisations + dW)",
                         lambda: api.launch_qkv_backward_mxfp8_weight(wp, stream), flops, pure=pure_w, cublas=cublas_w)
    del keep_w, pure_w, cublas_w
    torch.cuda.empty_cache()
    # the denominator of the full backward: both pure GEMMs launched back to back in ONE timed sample, so
    # that it runs under the same power cap as the 9 ms fused sequence (summing two short bursts would not)
    pure_d, cublas_d, keep_d = _pure_mxfp8(ctx, m, hid, width)
    pure_w, cublas_w, keep_w = _pure_mxfp8(ctx, width, hid, m)

    def both_pure():
        rc = pure_d()
        return rc if rc else pure_w()

    def both_cublas():
        cublas_d()
        return cublas_w()

    full_row = ctx.row("c4 MXFP8 QKV full backward (data + weight)", full_backward, 2 * flops, pure=both_pure,
                       cublas=both_cublas, nvlink_bytes=pull_bytes, nvlink_dir="in")
    full_row["pure"]["what"] = "this library's two pure block-scaled GEMMs (dX and dW shapes) back to back in one sample"
    del keep_d, pure_d, cublas_d, keep_w, pure_w, cublas_w
    torch.cuda.empty_cache()
    if ctx.validate:
        from tests import fullsize as F
        ctx.barrier()
        F.poison(staging, dx, dw)
        buf.fill_(0xA5)
        ctx.barrier()
        full_backward()
        torch.cuda.synchronize()
        ctx.check_status("c4 validation")
        a256 = lambda v: (v + 255) // 256 * 256
        w0 = base - buf.data_ptr()
        wq = buf[w0:w0 + hid * width].view(hid, width)
        s0 = w0 + a256(hid * width)
        wsf = buf[s0:s0 + api.mxfp8_scale_bytes(hid, width)]
        l0 = s0 + a256(api.mxfp8_scale_bytes(hid, width))
        packed = buf[l0:l0 + m * width].view(m, width)
        ls0 = l0 + a256(m * width)
        packed_scales = buf[ls0:ls0 + api.mxfp8_scale_bytes(m, width)]
        picked = F.sample_rows(m, count=ctx.validate_rows)
        masters = [sym[f"c4_{nm}m"].view(BF16).view(rows, h // cp * d) for nm, h in zip(names, heads)]
        planes_q = [sym[f"c4_{nm}8"].local.view(rows, h // cp * d) for nm, h in zip(names, heads)]
        planes_s = [sym[f"c4_{nm}s"].local for nm in names]
        data = F.check_qkv_backward_data_mxfp8(cp, rank, m, q, kv, masters, planes_q, planes_s, w, staging, packed,
                                               packed_scales, wq, wsf, dx, picked)
        weight = F.check_weight_gradient_mxfp8(staging, x, dw, F.sample_rows(width, count=64, edge=8),
                                               F.sample_rows(hid, count=512, edge=16))
        data_row["validated"] = _merge(ctx, data)
        weight_row["validated"] = _merge(ctx, weight)
        full_row["validated"] = _merge(ctx, data, weight)
        ctx.barrier()
    return [data_row, weight_row, full_row, quantisers]


# ---------------------------------------------------------------------------------------------------
# C5: MoE dispatch -> expert FC1
# ---------------------------------------------------------------------------------------------------

def run_c5(ctx: Context):
    from oracle import oracle as O  # routing tables of the synthetic workload come from the oracle's builders
    cp, rank, dev, stream = ctx.world_size, ctx.rank, ctx.dev, ctx.stream
    tokens, hid, e_local, topk, n = max(256, int(8192 * ctx.scale)), 7168, 32, 8, 4096
    experts = e_local * cp
    sym = ctx.world.allocate({"c5_tokens": tokens * hid * 2, "c5_started": cp * 128, "c5_done": cp * 128})
    ctx.fill(sym["c5_tokens"].view(BF16), ctx.seed + 5, 1.0)
    # seeded skewed routes: scores ~ N(0,1) + Zipf(1.1) bias per expert; every rank builds all ranks' tables
    rng = np.random.default_rng(synthetic.GROUPED_SEED)
    bias = np.log(1.0 / (rng.permutation(experts) + 1.0) ** 1.1)
    chosen = []
    for r in range(cp):
        scores = (np.random.default_rng(synthetic.GROUPED_SEED + 17 * r).standard_normal((tokens, experts)) + bias).astype(np.float32)
        picked = np.empty((tokens, topk), dtype=np.int32)
        O.lib().fo_moe_topk(O.ptr(np.ascontiguousarray(scores)), tokens, experts, topk, O.ptr(picked))
        chosen.append(picked)
    offs = np.empty(e_local + 1, dtype=np.int32)
    total = O.lib().fo_moe_build_rows(cp, rank, e_local, tokens, topk, O.ptr_array(chosen), O.ptr(offs), None)
    src = np.empty((max(total, 1), 3), dtype=np.int32)
    O.lib().fo_moe_build_rows(cp, rank, e_local, tokens, topk, O.ptr_array(chosen), O.ptr(offs), O.ptr(src))
    counts = np.diff(offs)
    cap = int(-(-max(int(counts.max()), 1) // 256) * 256)
    w = ctx.gen((e_local, n, hid), 1000 + rank, 0.02)
    lhs = torch.empty((e_local, cap, hid), dtype=BF16, device=dev)
    eo = torch.empty((e_local, cap, n), dtype=BF16, device=dev)
    ptrs = lambda t: torch.tensor([t[i].data_ptr() for i in range(e_local)], dtype=torch.int64, device=dev)
    lp, wp, op_ = ptrs(lhs), ptrs(w), ptrs(eo)
    offs_d, src_d = torch.from_numpy(offs.astype(np.int64)).to(dev), torch.from_numpy(src).to(dev)
    gp = N.Bf16GroupedGemmParams(lhs=lp.data_ptr(), weight_nt=wp.data_ptr(), output=op_.data_ptr(),
                                 row_offsets=offs_d.data_ptr(), source=src_d.data_ptr(), experts=e_local, n=n, k=hid,
                                 expert_row_capacity=cap, rank=rank, world_size=cp, topk=topk)
    per_rank = np.zeros(cp, np.int64)
    for r in range(cp):
        per_rank += np.bincount((chosen[r] // e_local).ravel(), minlength=cp)
    busiest, mean_rows = int(per_rank.max()), float(per_rank.mean())
    gp.policy = N.GroupedGemmPolicy(num_comm_ctas=ctx.comm, num_compute_ctas=148, tile_n=256, mma_sm_count=2)  # 0: Auto
    for r in range(cp):
        gp.peer_input[r] = sym["c5_tokens"].peer_ptrs[r]
        gp.peer_started[r] = sym["c5_started"].peer_ptrs[r]
        gp.peer_done[r] = sym["c5_done"].peer_ptrs[r]
    rc, plan = api.create_bf16_a2a_grouped_gemm(gp)
    assert rc == 0, rc
    pure_rows = -(-busiest // 256) * 256
    pure, keep = _pure_bf16(ctx, pure_rows, n, hid)
    rec = ctx.row(f"c5 MoE dispatch+FC1 (EP{cp}, {busiest} routed rows on the busiest rank, mean {mean_rows:.0f})",
                  lambda: api.launch_bf16_grouped_gemm(plan, stream), 2.0 * busiest * n * hid, pure=pure,
                  nvlink_bytes=2.0 * busiest * hid * (cp - 1) / cp, nvlink_dir="in",
                  extra={"busiest_rank_rows": busiest, "mean_rank_rows": mean_rows,
                         "policy": {"num_comm_ctas": ctx.comm or "auto", "mma_sm_count": 2, "tile_n": 256}})
    rec["pure"]["what"] = (f"dense-equivalent: one [{pure_rows}, {n}, {hid}] GEMM of this library on all 148 SMs "
                           "(the busiest rank's rows against one expert-sized weight)")
    rec["pflops_per_gpu_mean_rank"] = 2.0 * mean_rows * n * hid / rec["ms"] / 1e12
    rec["pflops_per_gpu_is"] = "the busiest rank's rows over the max-over-ranks time; mean_rank uses the mean rows"
    del keep, pure
    if ctx.validate:
        from tests import fullsize as F
        ctx.barrier()
        F.poison(lhs, eo)
        ctx.barrier()
        assert api.launch_bf16_grouped_gemm(plan, stream) == 0
        torch.cuda.synchronize()
        ctx.check_status("c5 validation")
        check = F.check_moe_dispatch_fc1(cp, sym["c5_tokens"].view(BF16).view(tokens, hid), lhs, eo, w, offs, src)
        rec["validated"] = _merge(ctx, check)
        rec["validated"]["sample"] = "every dispatched row bit-exact on the device; FC1 of ~10 rows per expert vs the oracle"
        ctx.barrier()
    ctx.barrier()
    api.destroy_bf16_grouped_gemm(plan)
    del lhs, eo, w
    torch.cuda.empty_cache()

    # ---- the way back: expert FC2 (intermediate 2048 -> hidden 7168) whose epilogue scatters every branch
    # row to the rank that owns the token (same routes; no weighting or top-k reduction in the operator)
    inter = 2048
    csym = ctx.world.allocate({"c5_received": tokens * topk * hid * 2, "c5_started2": cp * 128, "c5_done2": cp * 128})
    received = csym["c5_received"].view(BF16).view(tokens * topk, hid)
    act = ctx.gen((e_local, cap, inter), ctx.seed + 9, 1.0)
    w2 = ctx.gen((e_local, hid, inter), 2000 + rank, 0.02)
    out2 = torch.empty((e_local, cap, hid), dtype=BF16, device=dev)
    ap_, w2p, o2p = ptrs(act), ptrs(w2), ptrs(out2)
    cpar = N.Bf16GroupedGemmParams(lhs=ap_.data_ptr(), weight_nt=w2p.data_ptr(), output=o2p.data_ptr(),
                                   row_offsets=offs_d.data_ptr(), source=src_d.data_ptr(), experts=e_local, n=hid, k=inter,
                                   expert_row_capacity=cap, rank=rank, world_size=cp, topk=topk)
    cpar.policy = N.GroupedGemmPolicy(num_comm_ctas=2, num_compute_ctas=146, tile_n=256, mma_sm_count=2)
    for r in range(cp):
        cpar.peer_output[r] = csym["c5_received"].peer_ptrs[r]
        cpar.peer_started[r] = csym["c5_started2"].peer_ptrs[r]
        cpar.peer_done[r] = csym["c5_done2"].peer_ptrs[r]
    rc, cplan = api.create_bf16_grouped_gemm_a2a(cpar)
    assert rc == 0, rc
    pure2, keep2 = _pure_bf16(ctx, pure_rows, hid, inter)
    crec = ctx.row(f"c5 MoE FC2+combine (EP{cp}, K 2048 -> N 7168, {busiest} rows on the busiest rank)",
                   lambda: api.launch_bf16_grouped_gemm(cplan, stream), 2.0 * busiest * hid * inter, pure=pure2,
                   nvlink_bytes=2.0 * busiest * hid * (cp - 1) / cp, nvlink_dir="out",
                   extra={"busiest_rank_rows": busiest, "mean_rank_rows": mean_rows,
                          "policy": {"mma_sm_count": 2, "tile_n": 256, "note": "every CTA computes; the epilogue scatters"}})
    crec["pflops_per_gpu_mean_rank"] = 2.0 * mean_rows * hid * inter / crec["ms"] / 1e12
    del keep2, pure2
    if ctx.validate:
        from tests import fullsize as F
        ctx.barrier()
        F.poison(out2, received)
        ctx.barrier()
        assert api.launch_bf16_grouped_gemm(cplan, stream) == 0
        torch.cuda.synchronize()  # no host barrier: the kernel ends when every owner has written into this rank
        ctx.check_status("c5 combine validation")
        check = F.check_moe_fc2_combine(cp, rank, act, w2, out2, received, offs, src[:total], chosen, e_local, topk)
        crec["validated"] = _merge(ctx, check)
        crec["validated"]["sample"] = ("1024 branch rows per rank bit-exact against the owner's slab row; FC2 of ~10 rows per "
                                       "expert vs the oracle; no branch row left unwritten")
        ctx.barrier()
    ctx.barrier()
    api.destroy_bf16_grouped_gemm(cplan)
    return [rec, crec]


RUNNERS = {"bwd": run_bwd, "a6": run_a6, "c3": run_c3, "a10": run_a10, "c4": run_c4, "c5": run_c5}


def run(ctx: Context, only=None):
    """Runs the requested configurations; returns the rows (the same list on every rank)."""
    if ctx.validate:
        from tests import fullsize as F
        F.use_host_threads(ctx.world_size)
    rows = []
    for name, runner in RUNNERS.items():
        if only and name not in only:
            continue
        rows += runner(ctx)
        torch.cuda.empty_cache()
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--samples", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--scale", type=float, default=1.0, help="scale rows per rank of c3/c4/c5")
    ap.add_argument("--only", default="", help="comma list of bwd,a6,c3,a10,c4,c5")
    ap.add_argument("--comm", type=int, default=0, help="communication CTAs of every operator (0: Auto, the host planner)")
    ap.add_argument("--skip-validate", action="store_true")
    ap.add_argument("--json", action="store_true", help="print the rows as one JSON line as well")
    args = ap.parse_args()
    world_size = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world_size > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    N.lib()
    world = World(rank, world_size, local_rank)
    ctx = Context(rank, world_size, local_rank, world, samples=args.samples, warmup=args.warmup,
                  validate=not args.skip_validate, scale=args.scale, comm=args.comm)
    rows = run(ctx, only=set(x for x in args.only.split(",") if x) or None)
    if rank == 0:
        for r in rows:
            if "pflops_per_gpu" not in r:
                print(f"{r['name']:78s} transposed {r['transposed']['gbps']:7.0f} GB/s  row-wise {r['row_wise']['gbps']:7.0f} GB/s")
                continue
            line = f"{r['name']:78s} {r['ms']:8.3f} ms {r['pflops_per_gpu']:6.3f} PFLOPS/GPU"
            if "pure" in r:
                line += f" | pure {r['pure']['ms']:8.3f} ms {r['pure']['pflops']:6.3f} P retention {r['retention'] * 100:5.1f}%"
            if "cublas" in r and "ms" in r["cublas"]:
                line += f" | cuBLASLt {r['cublas']['pflops']:6.3f} P"
            if "validated" in r:
                line += f" | validated {r['validated']['ok']}"
            print(line, flush=True)
        if args.json:
            print(json.dumps(rows))
    ctx.barrier()
    world.close()
    if world_size > 1:
        dist.destroy_process_group()
    bad = [r["name"] for r in rows if r.get("validated") is not None and not r["validated"]["ok"]]
    if bad:
        sys.stderr.write(f"VALIDATION FAILED: {bad}\n")
        raise SystemExit(3)


if __name__ == "__main__":
    main()
