"""Throughput of every fused operator at the benchmark geometries, one rank per GPU.

    python -m fuse_b200.perf_suite                      # one GPU (routes are local)
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m fuse_b200.perf_suite

Prints one line per operator: device time (CUDA events, max over ranks, median of `--samples`
launches after warm-up), PFLOPS per GPU on the algorithmic FLOPs, and the same GEMM alone on all
SMs ("pure") with the retention fused/pure.  Geometries (tokens per rank, weak scaling in the
number of ranks):
  c2  Llama-3-8B BF16 forward      M 16384, QKV [6144, 4096], OProj [4096, 4096]
  c3  Llama-3-70B MXFP8 OProj      M 65536 / ranks * ... (32768 rows per rank), N = K = 8192
  c4  Qwen3-32B MXFP8 QKV backward M `--c4-rows` (65536 at full size), H 5120, QKV 10240
  c5  MoE dispatch + FC1 BF16      8192 tokens per rank, H 7168, 32 experts per rank, top-8, N 4096
Inputs are generated on the device from seeds; the heavy configurations can be scaled down with
--scale for a quick run."""
from __future__ import annotations

import argparse
import os
import statistics

import numpy as np
import torch
import torch.distributed as dist

from . import _native as N
from . import api, synthetic
from .world import World


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--samples", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--scale", type=float, default=1.0, help="scale rows per rank of c3/c4/c5")
    ap.add_argument("--only", default="", help="comma list of c2,c3,c4,c5,bwd")
    ap.add_argument("--comm", type=int, default=16)
    ap.add_argument("--bwd-along-m", type=int, default=0, help="tile raster of the data-gradient GEMMs")
    ap.add_argument("--bwd-swizzle", type=int, default=8)
    args = ap.parse_args()
    world_size = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world_size > 1:
        dist.init_process_group("nccl", device_id=dev)
    N.lib()
    only = set(x for x in args.only.split(",") if x)
    stream = torch.cuda.current_stream().cuda_stream
    bf16, u8, i32 = torch.bfloat16, torch.uint8, torch.int32
    cp = world_size

    def barrier():
        torch.cuda.synchronize()
        if world_size > 1:
            dist.barrier()

    def gen(shape, seed, scale, dtype=bf16):
        t = torch.empty(shape, dtype=dtype, device=dev)
        assert api.generate_bf16(t.data_ptr(), t.numel(), seed, scale, normal=True) == 0
        return t

    def timed(fn, label, flops, pure_fn=None):
        """fn(epoch) launches one operator; returns after printing the line."""
        epoch = [0]

        def sample(f):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            epoch[0] += 1
            rc = f(epoch[0])
            assert rc == 0, f"{label}: cudaError {rc}"
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1)], device=dev)
            if world_size > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t)

        for _ in range(args.warmup):
            sample(fn)
        ms = statistics.median(sample(fn) for _ in range(args.samples))
        status = api.read_status()
        assert status[0] == 0, f"{label}: device wait gave up {status[:8]}"
        line = f"{label:34s} {ms:8.3f} ms {flops / ms / 1e12:7.3f} PFLOPS/GPU"
        if pure_fn is not None:
            for _ in range(args.warmup):
                sample(pure_fn)
            pure = statistics.median(sample(pure_fn) for _ in range(args.samples))
            line += f" | pure {pure:8.3f} ms {flops / pure / 1e12:7.3f} P | retention {pure / ms * 100:5.1f}%"
        if rank == 0:
            print(line, flush=True)
        return ms

    world = World(rank, world_size, local_rank)
    seed = synthetic.rank_seed(rank)
    direct = N.Options()
    direct.flags = N.QKV_ROUTE_DIRECT

    def ptr_table(sym, name):
        return sym[name].peer_ptrs

    # ------------------------------------------------------------------------------------- c2
    if not only or "c2" in only:
        m, hid, q, kv, d = 16384, 4096, 32, 8, 128
        n, k_o = (q + 2 * kv) * d, q * d
        rows = m * cp
        sym = world.allocate({"c2_planar": rows * (n // cp) * 2, "c2_done": cp * 128, "c2_attn": rows * (k_o // cp) * 2})
        x, wq, wo = gen((m, hid), seed + 1000, 1.0), gen((n, hid), 11, 0.02), gen((hid, k_o), 17, 0.02)
        assert api.generate_bf16(sym["c2_attn"].local.data_ptr(), rows * (k_o // cp), seed + 2000, 1.0, True) == 0
        local, staging, out = (torch.empty(s, dtype=bf16, device=dev) for s in ((m, n), (m, k_o), (m, hid)))
        prob = N.GemmProblem(m, n, hid, raster=N.RASTER_ALONG_M, max_swizzle_size=8)
        route = N.UlyssesRoute(world_size=cp, rank=rank, batch=1, global_seq=rows, seq_local=m, q_heads=q, kv_heads=kv,
                               head_dim=d, kind=N.ROUTE_QKV_GQA_PACK)
        ready = torch.zeros(api.qkv_ready_elements(prob), dtype=i32, device=dev)
        p = N.GemmA2AParams(lhs=x.data_ptr(), rhs_nt=wq.data_ptr(), local_output=local.data_ptr(), ready=ready.data_ptr(),
                            gemm=prob, route=route, num_comm_ctas=args.comm, epoch=0)
        for r in range(cp):
            p.peer_output[r] = ptr_table(sym, "c2_planar")[r]
            p.peer_route_done_epoch[r] = ptr_table(sym, "c2_done")[r]

        def qkv(e):
            p.epoch = e
            return api.launch_gemm_a2a_cutlass(p, stream, direct)

        timed(qkv, "c2 BF16 QKVProj->A2A", 2.0 * m * n * hid, lambda e: api.launch_batched_cutlass_reference(p, stream, 0))
        oprob = N.GemmProblem(m, hid, k_o, raster=N.RASTER_ALONG_N, max_swizzle_size=8)
        oroute = N.UlyssesRoute(world_size=cp, rank=rank, batch=1, global_seq=rows, seq_local=m, q_heads=q, head_dim=d,
                                kind=N.ROUTE_HEAD_TO_SEQUENCE, direction=N.ROUTE_INVERSE)
        oready = torch.zeros(api.a2a_lhs_gemm_ready_elements(oprob, oroute), dtype=i32, device=dev)
        po = N.A2AGemmParams(input_staging=staging.data_ptr(), rhs_nt=wo.data_ptr(), output=out.data_ptr(),
                             ready=oready.data_ptr(), gemm=oprob, route=oroute, num_comm_ctas=args.comm, epoch=0)
        for r in range(cp):
            po.peer_input[r] = ptr_table(sym, "c2_attn")[r]

        def oproj(e):
            po.epoch = e
            return api.launch_a2a_gemm_cutlass(po, stream)

        timed(oproj, "c2 BF16 A2A->OProj", 2.0 * m * hid * k_o, lambda e: api.launch_a2a_gemm_cutlass_reference(po, stream, 0))

        if not only or "bwd" in only:
            # BF16 backward of the same layer (B and W phases timed separately, as the reference does)
            bsym = world.allocate({"b_staging": m * n * 2, "b_done": cp * 128, "b_done2": cp * 128,
                                   "b_gattn": rows * (k_o // cp) * 2})
            bp = N.QkvBackwardDataParams(local_tokens=m, hidden=hid, batch=1, q_heads=q, kv_heads=kv, head_dim=d,
                                         world_size=cp, rank=rank, num_comm_ctas=args.comm, epoch=0)
            bp.gemm_tuning.max_swizzle_size = args.bwd_swizzle
            bp.gemm_tuning.along_m = args.bwd_along_m
            bready = world.allocate({"b_ready": api.qkv_backward_ready_elements(bp) * 4})
            planes = [gen((rows, h // cp * d), seed + 100 * i + 101, 0.01) for i, h in enumerate((q, kv, kv))]
            dx = torch.empty((m, hid), dtype=bf16, device=dev)
            bp.grad_q, bp.grad_k, bp.grad_v = (t.data_ptr() for t in planes)
            bp.weight, bp.grad_input = wq.data_ptr(), dx.data_ptr()
            for r in range(cp):
                bp.peer_dqkv_staging[r] = bsym["b_staging"].peer_ptrs[r]
                bp.peer_ready[r] = bready["b_ready"].peer_ptrs[r]
                bp.peer_done_epoch[r] = bsym["b_done"].peer_ptrs[r]

            def qkv_b(e):
                bp.epoch = e
                return api.launch_qkv_backward_data(bp, stream)

            dw = torch.empty((n, hid), dtype=bf16, device=dev)
            wparams = N.QkvBackwardWeightParams(dqkv_staging=bsym["b_staging"].local.data_ptr(), saved_input=x.data_ptr(),
                                                grad_weight=dw.data_ptr(), local_tokens=m, hidden=hid, q_heads=q,
                                                kv_heads=kv, head_dim=d)
            timed(qkv_b, "c2 BF16 QKV backward data", 2.0 * m * n * hid)
            timed(lambda e: api.launch_qkv_backward_weight(wparams, stream), "c2 BF16 QKV backward weight", 2.0 * m * n * hid)
            dy = gen((m, hid), seed + 301, 0.01)
            da = torch.empty((m, k_o), dtype=bf16, device=dev)
            op = N.OprojBackwardDataParams(grad_output=dy.data_ptr(), weight=wo.data_ptr(), local_grad_attention=da.data_ptr(),
                                           local_tokens=m, hidden=hid, batch=1, q_heads=q, head_dim=d, world_size=cp,
                                           rank=rank, num_comm_ctas=args.comm, epoch=0)
            op.gemm_tuning.max_swizzle_size = args.bwd_swizzle
            op.gemm_tuning.along_m = args.bwd_along_m
            for r in range(cp):
                op.peer_grad_attention[r] = bsym["b_gattn"].peer_ptrs[r]
                op.peer_done_epoch[r] = bsym["b_done2"].peer_ptrs[r]

            def oproj_b(e):
                op.epoch = e
                return api.launch_oproj_backward_data(op, stream)

            dwo = torch.empty((hid, k_o), dtype=bf16, device=dev)
            ow = N.OprojBackwardWeightParams(grad_output=dy.data_ptr(), saved_attention=staging.data_ptr(),
                                             grad_weight=dwo.data_ptr(), local_tokens=m, hidden=hid, q_heads=q, head_dim=d)
            timed(oproj_b, "c2 BF16 OProj backward data", 2.0 * m * k_o * hid)
            timed(lambda e: api.launch_oproj_backward_weight(ow, stream), "c2 BF16 OProj backward weight", 2.0 * m * k_o * hid)
        del x, wq, wo, local, staging, out
        torch.cuda.empty_cache()

    # ------------------------------------------------------------------------------------- c3
    if not only or "c3" in only:
        m = max(128, int(32768 * args.scale) // 128 * 128)
        nk, heads, d = 8192, 64, 128
        rows, shard = m * cp, nk // cp
        sb = api.mxfp8_scale_bytes(rows, shard)
        sym = world.allocate({"c3_data": rows * shard, "c3_scales": sb})
        src = gen((rows, shard), seed + 2000, 1.0)
        assert api.quantize_mxfp8(src.data_ptr(), shard, rows, shard, sym["c3_data"].local.data_ptr(),
                                  sym["c3_scales"].local.data_ptr(), stream) == 0
        del src
        w = gen((nk, nk), 17, 0.02)
        out = torch.empty((m, nk), dtype=bf16, device=dev)
        prob = N.GemmProblem(m, nk, nk, raster=N.RASTER_ALONG_N, max_swizzle_size=8)
        rc, ws = api.a2a_gemm_mxfp8_workspace_size(prob)
        scratch = torch.empty(ws + 256, dtype=u8, device=dev)
        base = (scratch.data_ptr() + 255) // 256 * 256
        route = N.UlyssesRoute(world_size=cp, rank=rank, batch=1, global_seq=rows, seq_local=m, q_heads=heads, head_dim=d,
                               kind=N.ROUTE_HEAD_TO_SEQUENCE, direction=N.ROUTE_INVERSE)
        proj = N.A2AGemmParams(rhs_nt=w.data_ptr(), output=out.data_ptr(), gemm=prob, route=route,
                               num_comm_ctas=args.comm, epoch=0)
        mp = N.Mxfp8A2AGemmParams(projection=proj, workspace=base, workspace_bytes=ws)
        for r in range(cp):
            mp.activation[r] = N.Mxfp8Activation(data=sym["c3_data"].peer_ptrs[r], scales=sym["c3_scales"].peer_ptrs[r],
                                                 data_bytes=rows * shard, scale_bytes=sb)

        def mx_oproj(e):
            mp.projection.epoch = e
            return api.launch_a2a_gemm_mxfp8_cutlass(mp, stream)

        # pure block-scaled GEMM of the same shape on all SMs (prepared operands)
        act = gen((m, nk), seed + 5, 1.0)
        qd = torch.empty((m, nk), dtype=u8, device=dev)
        qs = torch.empty(api.mxfp8_scale_bytes(m, nk), dtype=u8, device=dev)
        assert api.quantize_mxfp8(act.data_ptr(), nk, m, nk, qd.data_ptr(), qs.data_ptr(), stream) == 0
        del act
        rc, ws2 = api.gemm_a2a_mxfp8_workspace_size(prob)
        scratch2 = torch.empty(ws2 + 256, dtype=u8, device=dev)
        base2 = (scratch2.data_ptr() + 255) // 256 * 256
        pq = N.GemmA2AParams(rhs_nt=w.data_ptr(), local_output=out.data_ptr(), gemm=N.GemmProblem(m, nk, nk, max_swizzle_size=8),
                             num_comm_ctas=1, epoch=1)
        pure = N.Mxfp8GemmA2AParams(projection=pq, workspace=base2, workspace_bytes=ws2,
                                    activation=N.Mxfp8Activation(data=qd.data_ptr(), scales=qs.data_ptr(),
                                                                 data_bytes=qd.numel(), scale_bytes=qs.numel()))
        assert api.prepare_gemm_a2a_mxfp8(pure, stream) == 0
        timed(mx_oproj, f"c3 MXFP8 A2A->OProj (M {m})", 2.0 * m * nk * nk,
              lambda e: api.launch_gemm_a2a_mxfp8_compute_reference(pure, stream))
        del w, out, scratch, scratch2, qd, qs
        torch.cuda.empty_cache()

    # ------------------------------------------------------------------------------------- c5
    if not only or "c5" in only:
        tokens, hid, e_local, topk, n = max(256, int(8192 * args.scale)), 7168, 32, 8, 4096
        experts = e_local * cp
        sym = world.allocate({"c5_tokens": tokens * hid * 2, "c5_started": cp * 128, "c5_done": cp * 128})
        assert api.generate_bf16(sym["c5_tokens"].local.data_ptr(), tokens * hid, seed + 5, 1.0, True) == 0
        # seeded skewed routes: scores ~ N(0,1) + Zipf(1.1) bias; every rank builds all ranks' tables
        rng = np.random.default_rng(synthetic.GROUPED_SEED)
        bias = np.log(1.0 / (rng.permutation(experts) + 1.0) ** 1.1)
        chosen = []
        for r in range(cp):
            scores = np.random.default_rng(synthetic.GROUPED_SEED + 17 * r).standard_normal((tokens, experts)) + bias
            chosen.append(np.argsort(-scores, axis=1, kind="stable")[:, :topk].astype(np.int32))
        counts, srcs = [], []
        for e in range(e_local):
            ge = rank * e_local + e
            parts = []
            for r in range(cp):
                tok, slot = np.nonzero(chosen[r] == ge)
                parts.append(np.stack([np.full_like(tok, r), tok, slot], 1))
            rows_e = np.concatenate(parts) if parts else np.zeros((0, 3), np.int64)
            counts.append(len(rows_e))
            srcs.append(rows_e)
        offs = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
        src = np.concatenate(srcs).astype(np.int32)
        cap = int(-(-max(counts) // 256) * 256)
        w = gen((e_local, n, hid), 1000 + rank, 0.02)
        lhs = torch.empty((e_local, cap, hid), dtype=bf16, device=dev)
        eo = torch.empty((e_local, cap, n), dtype=bf16, device=dev)
        ptrs = lambda t: torch.tensor([t[i].data_ptr() for i in range(e_local)], dtype=torch.int64, device=dev)
        lp, wp, op_ = ptrs(lhs), ptrs(w), ptrs(eo)
        offs_d, src_d = torch.from_numpy(offs).to(dev), torch.from_numpy(src).to(dev)
        gp = N.Bf16GroupedGemmParams(lhs=lp.data_ptr(), weight_nt=wp.data_ptr(), output=op_.data_ptr(),
                                     row_offsets=offs_d.data_ptr(), source=src_d.data_ptr(), experts=e_local, n=n, k=hid,
                                     expert_row_capacity=cap, rank=rank, world_size=cp, topk=topk)
        # the timed figure is the max over ranks, i.e. the busiest rank's: count its rows
        per_rank = np.zeros(cp, np.int64)
        for r in range(cp):
            per_rank += np.bincount((chosen[r] // e_local).ravel(), minlength=cp)
        total_rows = int(per_rank.max())
        flops = 2.0 * total_rows * n * hid
        for comm, compute, mma in ((args.comm, 148 - args.comm, 1), (args.comm, 148 - args.comm, 2), (20, 128, 2)):
            gp.policy = N.GroupedGemmPolicy(num_comm_ctas=comm, num_compute_ctas=compute, tile_n=256, mma_sm_count=mma)
            for r in range(cp):
                gp.peer_input[r] = sym["c5_tokens"].peer_ptrs[r]
                gp.peer_started[r] = sym["c5_started"].peer_ptrs[r]
                gp.peer_done[r] = sym["c5_done"].peer_ptrs[r]
            rc, plan = api.create_bf16_a2a_grouped_gemm(gp)
            assert rc == 0, rc
            timed(lambda e: api.launch_bf16_grouped_gemm(plan, stream),
                  f"c5 MoE dispatch+FC1 ({total_rows} rows on the busiest rank, comm {comm}, mma_sm {mma})", flops)
            barrier()
            api.destroy_bf16_grouped_gemm(plan)
        # pure grouped GEMM denominator: the same rows as one dense GEMM per expert is not
        # available as a single kernel here; report the dense-equivalent pure GEMM instead
        del w, lhs, eo
        torch.cuda.empty_cache()

    # ------------------------------------------------------------------------------------- c4
    if not only or "c4" in only:
        m = max(128, int(65536 * args.scale) // 128 * 128)
        hid, q, kv, d = 5120, 64, 8, 128
        width, rows = (q + 2 * kv) * d, m * cp
        names = ("q", "k", "v")
        spec = {}
        for nm, h in zip(names, (q, kv, kv)):
            pw = h // cp * d
            spec[f"c4_{nm}8"] = rows * pw
            spec[f"c4_{nm}s"] = api.mxfp8_scale_bytes(rows, pw)
            spec[f"c4_{nm}m"] = rows * pw * 2
        spec["c4_done"] = cp * 128
        sym = world.allocate(spec)
        for i, (nm, h) in enumerate(zip(names, (q, kv, kv))):
            pw = h // cp * d
            master = sym[f"c4_{nm}m"].local
            assert api.generate_bf16(master.data_ptr(), rows * pw, seed + 100 * i + 101, 0.01, True) == 0
            assert api.quantize_mxfp8(master.data_ptr(), pw, rows, pw, sym[f"c4_{nm}8"].local.data_ptr(),
                                      sym[f"c4_{nm}s"].local.data_ptr(), stream) == 0
        w = gen((width, hid), 11, 0.02)
        x = gen((m, hid), seed + 1000, 1.0)
        staging = torch.empty((m, width), dtype=bf16, device=dev)
        dx = torch.empty((m, hid), dtype=bf16, device=dev)
        dw = torch.empty((width, hid), dtype=bf16, device=dev)
        proj = N.QkvBackwardDataParams(weight=w.data_ptr(), grad_input=dx.data_ptr(), local_tokens=m, hidden=hid, batch=1,
                                       q_heads=q, kv_heads=kv, head_dim=d, world_size=cp, rank=rank,
                                       num_comm_ctas=args.comm, epoch=0)
        proj.gemm_tuning.max_swizzle_size = 8
        ready = torch.zeros(api.qkv_backward_ready_elements(proj), dtype=i32, device=dev)
        proj.peer_dqkv_staging[rank] = staging.data_ptr()
        proj.peer_ready[rank] = ready.data_ptr()
        for r in range(cp):
            proj.peer_done_epoch[r] = sym["c4_done"].peer_ptrs[r]
        rc, ws = api.qkv_backward_mxfp8_data_workspace_size(proj)
        wproj = N.QkvBackwardWeightParams(dqkv_staging=staging.data_ptr(), saved_input=x.data_ptr(), grad_weight=dw.data_ptr(),
                                          local_tokens=m, hidden=hid, q_heads=q, kv_heads=kv, head_dim=d)
        rc, ws2 = api.qkv_backward_mxfp8_weight_workspace_size(wproj)
        scratch = torch.empty(max(ws, ws2) + 256, dtype=u8, device=dev)
        base = (scratch.data_ptr() + 255) // 256 * 256
        mp = N.Mxfp8QkvBackwardDataParams(projection=proj, workspace=base, workspace_bytes=ws)
        for r in range(cp):
            acts = [N.Mxfp8Activation(data=sym[f"c4_{nm}8"].peer_ptrs[r], scales=sym[f"c4_{nm}s"].peer_ptrs[r],
                                      data_bytes=spec[f"c4_{nm}8"], scale_bytes=spec[f"c4_{nm}s"]) for nm in names]
            mp.peer_input[r] = N.Mxfp8QkvBackwardInput(grad_q=acts[0], grad_k=acts[1], grad_v=acts[2],
                                                       master_q=sym["c4_qm"].peer_ptrs[r], master_k=sym["c4_km"].peer_ptrs[r],
                                                       master_v=sym["c4_vm"].peer_ptrs[r])
        wp = N.Mxfp8QkvBackwardWeightParams(projection=wproj, workspace=base, workspace_bytes=ws2)
        full = N.Mxfp8QkvBackwardParams(data=mp, weight=wp, weight_mode=0)

        def data_phase(e):
            mp.projection.epoch = e
            return api.launch_qkv_backward_mxfp8_data(mp, stream)

        def full_backward(e):
            full.data.projection.epoch = e
            return api.launch_qkv_backward_mxfp8(full, stream)

        timed(data_phase, f"c4 MXFP8 QKV backward data (M {m})", 2.0 * m * hid * width)
        timed(lambda e: api.launch_qkv_backward_mxfp8_weight(wp, stream), "c4 MXFP8 QKV backward weight", 2.0 * m * hid * width)
        timed(full_backward, "c4 MXFP8 QKV full backward", 4.0 * m * hid * width)

    barrier()
    world.close()
    if world_size > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
