"""One rank of a real multi-GPU parity run (launched by tests/test_gpu_multirank.py through
torch.distributed.run, one process per GPU).  Every rank runs the QKV operator and the output
projection operator against its peers' symmetric buffers and checks its own results against
the CPU oracle, which simulates all ranks from the same seeds."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from fuse_b200 import _native as N  # noqa: E402
from fuse_b200 import api, synthetic  # noqa: E402
from fuse_b200.world import World  # noqa: E402
from oracle import oracle as O  # noqa: E402


def bits(t):
    return t.detach().view(torch.int16).cpu().numpy().view(np.uint16)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    route_mode = sys.argv[1] if len(sys.argv) > 1 else "direct"
    batch, s, q, kv, d, k = 1, 512, 8 * world // 2, 8, 128, 512
    if kv % world:
        kv = world
    m, n = batch * s, (q + 2 * kv) * d
    rows = batch * s * world
    ko = q * d
    w = World(rank, world, local_rank)
    sym = w.allocate({"planar": rows * (n // world) * 2, "done": world * N.READY_FLAG_STRIDE * 4,
                      "attn": rows * (ko // world) * 2})
    lhs = [synthetic.normal_bf16((m, k), synthetic.rank_seed(r) + 1000, 1.0) for r in range(world)]
    wq = synthetic.normal_bf16((n, k), synthetic.BASE_SEED + 11, 0.02)
    attn_all = [synthetic.normal_bf16((rows, ko // world), synthetic.rank_seed(r) + 2000, 1.0) for r in range(world)]
    wo = synthetic.normal_bf16((512, ko), synthetic.BASE_SEED + 17, 0.02)  # 256-wide tiles: CTA pairs
    to_dev = lambda a: torch.from_numpy(a.view(np.int16)).to(dev).view(torch.bfloat16)
    x, wq_d, wo_d = to_dev(lhs[rank]), to_dev(wq), to_dev(wo)
    sym["attn"].view(torch.bfloat16).copy_(to_dev(attn_all[rank]).reshape(-1))
    sym["planar"].view(torch.int16).fill_(-1)
    local = torch.full((m, n), -1, dtype=torch.int16, device=dev).view(torch.bfloat16)
    staging = torch.full((m, ko), -1, dtype=torch.int16, device=dev).view(torch.bfloat16)
    out = torch.full((m, 512), -1, dtype=torch.int16, device=dev).view(torch.bfloat16)
    torch.cuda.synchronize()
    dist.barrier()

    problem = N.GemmProblem(m, n, k, max_swizzle_size=4)
    route = N.UlyssesRoute(world_size=world, rank=rank, batch=batch, global_seq=s * world, seq_local=s,
                           q_heads=q, kv_heads=kv, head_dim=d, kind=N.ROUTE_QKV_GQA_PACK)
    ready = torch.zeros(api.qkv_ready_elements(problem), dtype=torch.int32, device=dev)
    p = N.GemmA2AParams(lhs=x.data_ptr(), rhs_nt=wq_d.data_ptr(), local_output=local.data_ptr(),
                        ready=ready.data_ptr(), gemm=problem, route=route, num_comm_ctas=8, epoch=1)
    for r in range(world):
        p.peer_output[r] = sym["planar"].peer_ptrs[r]
        p.peer_route_done_epoch[r] = sym["done"].peer_ptrs[r]
    opts = N.Options()
    opts.wait_budget_ns = 2_000_000_000
    opts.flags = N.QKV_ROUTE_DIRECT if route_mode == "direct" else N.QKV_ROUTE_COMM_CTAS
    for epoch in (1, 2):  # second launch re-uses flags with the next epoch
        p.epoch = epoch
        assert api.launch_gemm_a2a_cutlass(p, 0, opts) == 0
    torch.cuda.synchronize()
    status = api.read_status()
    assert status[0] == 0, status[:8]
    # When this rank's kernel has finished, every peer's pushes into it are complete
    # (cross-rank completion handshake): no host barrier before reading.
    want_local, want_peers = O.qkv_forward(world, batch, s, q, kv, d, lhs, wq)
    ok, worst, bad = O.within_tolerance(bits(local), want_local[rank])
    assert ok, ("local", worst, bad)
    ok, worst, bad = O.within_tolerance(bits(sym["planar"].view(torch.bfloat16)), want_peers[rank])
    assert ok, ("planar", worst, bad)

    # ---- the same operator with the all-to-all of V deferred (UlyssesRoute.defer_v_a2a): Q | K per row in
    # ONE tensor per destination, V only in the local output, completion_epoch published locally
    dist.barrier()  # every rank has read its planar buffer before the next launch writes into it
    sym["planar"].view(torch.int16).fill_(-1)
    torch.cuda.synchronize()
    dist.barrier()
    completion = torch.zeros(N.READY_FLAG_STRIDE, dtype=torch.int32, device=dev)
    p.route.defer_v_a2a = 1
    p.completion_epoch = completion.data_ptr()
    p.epoch = 3
    assert api.launch_gemm_a2a_cutlass(p, 0, opts) == 0
    torch.cuda.synchronize()
    status = api.read_status()
    assert status[0] == 0, status[:8]
    assert int(completion[0]) == 3
    want_local, want_peers = O.qkv_forward(world, batch, s, q, kv, d, lhs, wq, defer_v=True)
    ok, worst, bad = O.within_tolerance(bits(local), want_local[rank])
    assert ok, ("local with V deferred", worst, bad)
    got = bits(sym["planar"].view(torch.bfloat16))
    routed = want_peers[rank] != 0xFFFF   # (a routed BF16 value is never the all-ones NaN pattern)
    assert (got[~routed] == 0xFFFF).all(), "an element outside Q | K was written with V deferred"
    ok, worst, bad = O.within_tolerance(got[routed], want_peers[rank][routed])
    assert ok, ("Q | K with V deferred", worst, bad)
    p.route.defer_v_a2a = 0
    p.completion_epoch = None

    dist.barrier()
    o_problem = N.GemmProblem(m, 512, ko, max_swizzle_size=8)
    o_route = N.UlyssesRoute(world_size=world, rank=rank, batch=batch, global_seq=s * world, seq_local=s,
                             kind=N.ROUTE_HEAD_TO_SEQUENCE, direction=N.ROUTE_INVERSE)
    o_ready = torch.zeros(api.a2a_lhs_gemm_ready_elements(o_problem, o_route), dtype=torch.int32, device=dev)
    po = N.A2AGemmParams(input_staging=staging.data_ptr(), rhs_nt=wo_d.data_ptr(), output=out.data_ptr(),
                         ready=o_ready.data_ptr(), gemm=o_problem, route=o_route, num_comm_ctas=8, epoch=1)
    for r in range(world):
        po.peer_input[r] = sym["attn"].peer_ptrs[r]
    assert api.launch_a2a_gemm_cutlass(po, 0, opts) == 0
    torch.cuda.synchronize()
    status = api.read_status()
    assert status[0] == 0, status[:8]
    want_staging, want_out = O.oproj_forward(world, rank, batch, s, attn_all, wo)
    assert np.array_equal(bits(staging), want_staging), "gathered lhs differs"
    ok, worst, bad = O.within_tolerance(bits(out), want_out)
    assert ok, ("oproj", worst, bad)
    dist.barrier()  # peers' inputs stay immutable until every rank is done

    # ---- the forward pair again at a size where every rank runs several waves of 256 x 256 tiles
    # (10 x 24 QKV tiles on 74 CTA pairs, K wrap of the pull), checked by row samples: GEMM rows against
    # the oracle, routed / gathered elements traced through the oracle's maps, bit-exact ------------
    from tests import fullsize as F
    F.use_host_threads(world)
    bs, bq, bkv, bk = 2560, 32, 8, 1024
    bn, bko = (bq + 2 * bkv) * d, bq * d
    brows = bs * world
    bsym = w.allocate({"big_planar": brows * (bn // world) * 2, "big_done": world * N.READY_FLAG_STRIDE * 4,
                       "big_attn": brows * (bko // world) * 2})
    gen = lambda shape, seed, scale: to_dev(synthetic.normal_bf16(shape, seed, scale))
    bx, bwq, bwo = gen((bs, bk), synthetic.rank_seed(rank) + 31, 1.0), gen((bn, bk), 41, 0.02), gen((1024, bko), 43, 0.02)
    bsym["big_attn"].view(torch.bfloat16).copy_(gen((brows, bko // world), synthetic.rank_seed(rank) + 37, 1.0).reshape(-1))
    blocal = torch.full((bs, bn), -1, dtype=torch.int16, device=dev).view(torch.bfloat16)
    bstaging = torch.full((bs, bko), -1, dtype=torch.int16, device=dev).view(torch.bfloat16)
    bout = torch.full((bs, 1024), -1, dtype=torch.int16, device=dev).view(torch.bfloat16)
    bsym["big_planar"].view(torch.int16).fill_(-1)
    bproblem = N.GemmProblem(bs, bn, bk, raster=N.RASTER_ALONG_M, max_swizzle_size=8)
    broute = N.UlyssesRoute(world_size=world, rank=rank, batch=1, global_seq=brows, seq_local=bs, q_heads=bq, kv_heads=bkv,
                            head_dim=d, kind=N.ROUTE_QKV_GQA_PACK)
    bready = torch.zeros(api.qkv_ready_elements(bproblem), dtype=torch.int32, device=dev)
    bp_ = N.GemmA2AParams(lhs=bx.data_ptr(), rhs_nt=bwq.data_ptr(), local_output=blocal.data_ptr(), ready=bready.data_ptr(),
                          gemm=bproblem, route=broute, num_comm_ctas=0 if route_mode == "direct" else 8, epoch=1)
    for r in range(world):
        bp_.peer_output[r] = bsym["big_planar"].peer_ptrs[r]
        bp_.peer_route_done_epoch[r] = bsym["big_done"].peer_ptrs[r]
    torch.cuda.synchronize()
    dist.barrier()
    assert api.launch_gemm_a2a_cutlass(bp_, 0, opts) == 0
    boprob = N.GemmProblem(bs, 1024, bko, raster=N.RASTER_ALONG_N, max_swizzle_size=8)
    boroute = N.UlyssesRoute(world_size=world, rank=rank, batch=1, global_seq=brows, seq_local=bs,
                             kind=N.ROUTE_HEAD_TO_SEQUENCE, direction=N.ROUTE_INVERSE)
    boready = torch.zeros(api.a2a_lhs_gemm_ready_elements(boprob, boroute), dtype=torch.int32, device=dev)
    bpo = N.A2AGemmParams(input_staging=bstaging.data_ptr(), rhs_nt=bwo.data_ptr(), output=bout.data_ptr(),
                          ready=boready.data_ptr(), gemm=boprob, route=boroute, num_comm_ctas=0, epoch=1)  # Auto
    for r in range(world):
        bpo.peer_input[r] = bsym["big_attn"].peer_ptrs[r]
    assert api.launch_a2a_gemm_cutlass(bpo, 0, opts) == 0
    torch.cuda.synchronize()
    status = api.read_status()
    assert status[0] == 0, status[:8]
    picked = F.sample_rows(bs, count=96)
    qc = F.check_qkv_forward(world, rank, bs, bq, bkv, d, bx, bwq, blocal, bsym["big_planar"].view(torch.bfloat16), picked)
    oc = F.check_oproj_forward(world, rank, bs, bko, bsym["big_attn"].view(torch.bfloat16), bstaging, bwo, bout, picked)
    verdict = F.merge(qc, oc)
    assert verdict["ok"], verdict
    dist.barrier()

    # ---- QKV backward: sender push into the peers' staging, flags released on the destination ----
    hidden = 512
    planes_all = [tuple(synthetic.normal_bf16((rows, heads // world * d), synthetic.rank_seed(r) + 100 * seg + 101, 0.01)
                        for seg, heads in enumerate((q, kv, kv))) for r in range(world)]
    wb = synthetic.normal_bf16((n, hidden), synthetic.BASE_SEED + 23, 0.02)
    bp = N.QkvBackwardDataParams(local_tokens=m, hidden=hidden, batch=batch, q_heads=q, kv_heads=kv, head_dim=d,
                                 world_size=world, rank=rank, num_comm_ctas=8, epoch=1, alpha=1.0)
    bsym = w.allocate({"bwd_staging": m * n * 2, "bwd_ready": api.qkv_backward_ready_elements(bp) * 4,
                       "bwd_done": world * N.READY_FLAG_STRIDE * 4})
    mine = [to_dev(pl) for pl in planes_all[rank]]
    wb_d = to_dev(wb)
    dx = torch.full((m, hidden), -1, dtype=torch.int16, device=dev).view(torch.bfloat16)
    bp.grad_q, bp.grad_k, bp.grad_v = (t.data_ptr() for t in mine)
    bp.weight, bp.grad_input = wb_d.data_ptr(), dx.data_ptr()
    for r in range(world):
        bp.peer_dqkv_staging[r] = bsym["bwd_staging"].peer_ptrs[r]
        bp.peer_ready[r] = bsym["bwd_ready"].peer_ptrs[r]
        bp.peer_done_epoch[r] = bsym["bwd_done"].peer_ptrs[r]
    torch.cuda.synchronize()
    dist.barrier()
    assert api.launch_qkv_backward_data(bp, 0, opts) == 0
    torch.cuda.synchronize()
    status = api.read_status()
    assert status[0] == 0, status[:8]
    want_staging, want_dx, _ = O.qkv_backward(world, rank, batch, s, q, kv, d, planes_all, wb,
                                              synthetic.normal_bf16((m, hidden), 1, 1.0))
    assert np.array_equal(bits(bsym["bwd_staging"].view(torch.bfloat16)).reshape(m, n), want_staging), "bwd staging"
    ok, worst, bad = O.within_tolerance(bits(dx), want_dx, 0.02, 0.02)
    assert ok, ("dX", worst, bad)
    dist.barrier()

    # ---- MoE dispatch: entry/exit handshakes with every peer, row gather across ranks ------------
    experts_local, tokens, topk, mk, mn = 4, 96, 2, 512, 256
    rng = np.random.default_rng(11)
    chosen = [rng.integers(0, experts_local * world, (tokens, topk)).astype(np.int32) for _ in range(world)]
    for c in chosen:
        c[:, 1] = (c[:, 0] + 1 + c[:, 1] % (experts_local * world - 1)) % (experts_local * world)  # distinct experts
    offs = np.empty(experts_local + 1, dtype=np.int32)
    total = O.lib().fo_moe_build_rows(world, rank, experts_local, tokens, topk, O.ptr_array(chosen), O.ptr(offs), None)
    src = np.empty((max(total, 1), 3), dtype=np.int32)
    O.lib().fo_moe_build_rows(world, rank, experts_local, tokens, topk, O.ptr_array(chosen), O.ptr(offs), O.ptr(src))
    toks_all = [synthetic.normal_bf16((tokens, mk), synthetic.GROUPED_SEED + 31 * r, 1.0) for r in range(world)]
    ew = synthetic.normal_bf16((experts_local, mn, mk), synthetic.GROUPED_SEED + 1000 + rank, 0.02)
    cap = 256
    msym = w.allocate({"moe_tokens": tokens * mk * 2, "moe_started": world * N.READY_FLAG_STRIDE * 4,
                       "moe_done": world * N.READY_FLAG_STRIDE * 4})
    msym["moe_tokens"].view(torch.bfloat16).copy_(to_dev(toks_all[rank]).reshape(-1))
    ew_d = to_dev(ew)
    lhs = torch.full((experts_local, cap, mk), 0x7f7f, dtype=torch.int16, device=dev).view(torch.bfloat16)
    eo = torch.full((experts_local, cap, mn), 0x7f7f, dtype=torch.int16, device=dev).view(torch.bfloat16)
    ptrs = lambda t: torch.tensor([t[i].data_ptr() for i in range(experts_local)], dtype=torch.int64, device=dev)
    lp, wp, op = ptrs(lhs), ptrs(ew_d), ptrs(eo)
    offs_d = torch.from_numpy(offs.astype(np.int64)).to(dev)
    src_d = torch.from_numpy(src).to(dev)
    gp = N.Bf16GroupedGemmParams(lhs=lp.data_ptr(), weight_nt=wp.data_ptr(), output=op.data_ptr(),
                                 row_offsets=offs_d.data_ptr(), source=src_d.data_ptr(), experts=experts_local,
                                 n=mn, k=mk, expert_row_capacity=cap, rank=rank, world_size=world, topk=topk)
    for r in range(world):
        gp.peer_input[r] = msym["moe_tokens"].peer_ptrs[r]
        gp.peer_started[r] = msym["moe_started"].peer_ptrs[r]
        gp.peer_done[r] = msym["moe_done"].peer_ptrs[r]
    want_lhs = np.full((experts_local, cap, mk), 0x7f7f, dtype=np.uint16)
    want_eo = np.full((experts_local, cap, mn), 0x7f7f, dtype=np.uint16)
    assert O.lib().fo_moe_dispatch_fc1(experts_local, O.ptr(offs), O.ptr(src), O.ptr_array(toks_all), O.ptr(ew), mn, mk,
                                       cap, O.ptr(want_lhs), O.ptr(want_eo)) == 0
    # one-CTA tiles, CTA pairs with communication CTAs, CTA pairs with the embedded pull (Auto)
    for mma_sm_count, dispatch_ctas in ((1, 6), (2, 6), (2, 0)):
        gp.policy = N.GroupedGemmPolicy(num_comm_ctas=dispatch_ctas, num_compute_ctas=128, tile_n=256,
                                        mma_sm_count=mma_sm_count)
        lhs.view(torch.int16).fill_(0x7f7f)
        eo.view(torch.int16).fill_(0x7f7f)
        rc, plan = api.create_bf16_a2a_grouped_gemm(gp)
        assert rc == 0, rc
        torch.cuda.synchronize()
        dist.barrier()
        for _ in range(2):
            assert api.launch_bf16_grouped_gemm(plan, 0, opts) == 0
        torch.cuda.synchronize()
        status = api.read_status()
        assert status[0] == 0, status[:8]
        assert np.array_equal(bits(lhs), want_lhs), "dispatched rows"
        for e in range(experts_local):
            cnt = int(offs[e + 1] - offs[e])
            ok, worst, bad = O.within_tolerance(bits(eo)[e, :cnt], want_eo[e, :cnt], 0.002, 0.008)
            assert ok, ("moe", mma_sm_count, e, worst, bad)
        assert api.destroy_bf16_grouped_gemm(plan) == 0
        dist.barrier()

    # ---- MoE combine: expert FC2 whose epilogue scatters branch rows into the owners' buffers ------
    routes_all = []
    for r in range(world):
        o = np.empty(experts_local + 1, dtype=np.int32)
        tot = O.lib().fo_moe_build_rows(world, r, experts_local, tokens, topk, O.ptr_array(chosen), O.ptr(o), None)
        sr = np.empty((max(tot, 1), 3), dtype=np.int32)
        O.lib().fo_moe_build_rows(world, r, experts_local, tokens, topk, O.ptr_array(chosen), O.ptr(o), O.ptr(sr))
        routes_all.append((o, sr[:tot]))
    ck, cn = 256, 512
    act_all = [synthetic.normal_bf16((experts_local, cap, ck), synthetic.GROUPED_SEED + 77 + r, 1.0) for r in range(world)]
    w2_all = [synthetic.normal_bf16((experts_local, cn, ck), synthetic.GROUPED_SEED + 2000 + r, 0.02) for r in range(world)]
    want_recv = [np.full((tokens * topk, cn), 0x7f7f, dtype=np.uint16) for _ in range(world)]
    want_slab = None
    for r in range(world):  # every rank simulates all ranks: the owners' rows land in its own expectation
        slab = np.full((experts_local, cap, cn), 0x7f7f, dtype=np.uint16)
        assert O.lib().fo_moe_fc2_combine(experts_local, O.ptr(routes_all[r][0]), O.ptr(np.ascontiguousarray(routes_all[r][1])),
                                          O.ptr(act_all[r]), O.ptr(w2_all[r]), cn, ck, cap, topk, O.ptr(slab),
                                          O.ptr_array(want_recv)) == 0
        if r == rank:
            want_slab = slab
    csym = w.allocate({"comb_recv": tokens * topk * cn * 2, "comb_started": world * N.READY_FLAG_STRIDE * 4,
                       "comb_done": world * N.READY_FLAG_STRIDE * 4})
    act_d, w2_d = to_dev(act_all[rank]), to_dev(w2_all[rank])
    slab_d = torch.full((experts_local, cap, cn), 0x7f7f, dtype=torch.int16, device=dev).view(torch.bfloat16)
    ap, w2p, sp = ptrs(act_d), ptrs(w2_d), ptrs(slab_d)
    cp_ = N.Bf16GroupedGemmParams(lhs=ap.data_ptr(), weight_nt=w2p.data_ptr(), output=sp.data_ptr(),
                                  row_offsets=offs_d.data_ptr(), source=src_d.data_ptr(), experts=experts_local,
                                  n=cn, k=ck, expert_row_capacity=cap, rank=rank, world_size=world, topk=topk)
    for r in range(world):
        cp_.peer_output[r] = csym["comb_recv"].peer_ptrs[r]
        cp_.peer_started[r] = csym["comb_started"].peer_ptrs[r]
        cp_.peer_done[r] = csym["comb_done"].peer_ptrs[r]
    for mma_sm_count in (1, 2):
        cp_.policy = N.GroupedGemmPolicy(num_comm_ctas=2, num_compute_ctas=128, tile_n=256, mma_sm_count=mma_sm_count)
        csym["comb_recv"].view(torch.int16).fill_(0x7f7f)
        slab_d.view(torch.int16).fill_(0x7f7f)
        rc, cplan = api.create_bf16_grouped_gemm_a2a(cp_)
        assert rc == 0, rc
        torch.cuda.synchronize()
        dist.barrier()
        assert api.launch_bf16_grouped_gemm(cplan, 0, opts) == 0
        torch.cuda.synchronize()  # the kernel ends only when every owner has written into this rank
        status = api.read_status()
        assert status[0] == 0, status[:8]
        got_slab = bits(slab_d)
        for e in range(experts_local):
            cnt = int(offs[e + 1] - offs[e])
            ok, worst, bad = O.within_tolerance(got_slab[e, :cnt], want_slab[e, :cnt], 0.002, 0.008)
            assert ok, ("combine slab", mma_sm_count, e, worst, bad)
            assert (got_slab[e, cnt:] == 0x7f7f).all()
        ok, worst, bad = O.within_tolerance(bits(csym["comb_recv"].view(torch.bfloat16)).reshape(tokens * topk, cn),
                                            want_recv[rank], 0.002, 0.008)
        assert ok, ("combine received", mma_sm_count, worst, bad)
        assert api.destroy_bf16_grouped_gemm(cplan) == 0
        dist.barrier()

    # ---- MXFP8 output projection: bytes and scale bytes pulled from every peer ------------------
    to_dev_u8 = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    shard = ko // world
    mx_n = 512
    quant = [O.mxfp8_quantize(a) for a in attn_all]
    wmx = synthetic.normal_bf16((mx_n, ko), synthetic.BASE_SEED + 17, 0.02)
    want_wq, want_wsf = O.mxfp8_quantize(wmx)
    xsym = w.allocate({"mx_data": rows * shard, "mx_scales": len(quant[0][1])})
    xsym["mx_data"].local.copy_(to_dev_u8(quant[rank][0]).reshape(-1))
    xsym["mx_scales"].local.copy_(to_dev_u8(quant[rank][1]))
    wmx_d = to_dev(wmx)
    mx_problem = N.GemmProblem(m, mx_n, ko, max_swizzle_size=8)
    rc, ws_bytes = api.a2a_gemm_mxfp8_workspace_size(mx_problem)
    assert rc == 0
    scratch = torch.full((ws_bytes + 256,), 0x5A, dtype=torch.uint8, device=dev)
    base = (scratch.data_ptr() + 255) // 256 * 256
    mx_out = torch.full((m, mx_n), -1, dtype=torch.int16, device=dev).view(torch.bfloat16)
    mproj = N.A2AGemmParams(rhs_nt=wmx_d.data_ptr(), output=mx_out.data_ptr(), gemm=mx_problem, route=o_route,
                            num_comm_ctas=8, epoch=1)
    mxp = N.Mxfp8A2AGemmParams(projection=mproj, workspace=base, workspace_bytes=ws_bytes)
    for r in range(world):
        mxp.activation[r] = N.Mxfp8Activation(data=xsym["mx_data"].peer_ptrs[r], scales=xsym["mx_scales"].peer_ptrs[r],
                                              data_bytes=rows * shard, scale_bytes=len(quant[0][1]))
    torch.cuda.synchronize()
    dist.barrier()
    assert api.launch_a2a_gemm_mxfp8_cutlass(mxp, 0, opts) == 0
    torch.cuda.synchronize()
    status = api.read_status()
    assert status[0] == 0, status[:8]
    want_data = np.empty((m, ko), dtype=np.uint8)
    want_scales = np.zeros(O.lib().fo_mxfp8_scale_bytes(m, ko), dtype=np.uint8)
    for row in range(m):
        src_row = O.lib().fo_global_row(world, rank, s, 0, row)
        for j in range(world):
            want_data[row, j * shard:(j + 1) * shard] = quant[j][0][src_row]
            for kk in range(0, shard, 32):
                want_scales[O.lib().fo_mxfp8_scale_offset(row, j * shard + kk, ko)] = \
                    quant[j][1][O.lib().fo_mxfp8_scale_offset(src_row, kk, shard)]
    view = api.a2a_gemm_mxfp8_staging_view(mxp)
    off = view.data - scratch.data_ptr()
    assert np.array_equal(scratch[off:off + m * ko].cpu().numpy().reshape(m, ko), want_data), "mxfp8 gathered bytes"
    soff = view.scales - scratch.data_ptr()
    assert np.array_equal(scratch[soff:soff + view.scale_bytes].cpu().numpy(), want_scales), "mxfp8 gathered scales"
    ok, worst, bad = O.within_tolerance(bits(mx_out), O.gemm_mxfp8(want_data, want_scales, want_wq, want_wsf))
    assert ok, ("mxfp8 oproj", worst, bad)
    dist.barrier()

    # ---- MXFP8 QKV backward data: quantised gradients, scale atoms and BF16 masters pulled -------
    planes_q = [tuple(O.mxfp8_quantize(pl) for pl in planes_all[r]) for r in range(world)]
    names = ("q", "k", "v")
    spec = {}
    for seg, name in enumerate(names):
        spec[f"g{name}_data"] = planes_q[0][seg][0].size
        spec[f"g{name}_scales"] = planes_q[0][seg][1].size
        spec[f"g{name}_master"] = planes_all[0][seg].size * 2
    spec["mxb_done"] = world * N.READY_FLAG_STRIDE * 4
    gsym = w.allocate(spec)
    for seg, name in enumerate(names):
        gsym[f"g{name}_data"].local.copy_(to_dev_u8(planes_q[rank][seg][0]).reshape(-1))
        gsym[f"g{name}_scales"].local.copy_(to_dev_u8(planes_q[rank][seg][1]))
        gsym[f"g{name}_master"].view(torch.bfloat16).copy_(to_dev(planes_all[rank][seg]).reshape(-1))
    mx_staging = torch.full((m, n), -1, dtype=torch.int16, device=dev).view(torch.bfloat16)
    mx_dx = torch.full((m, hidden), -1, dtype=torch.int16, device=dev).view(torch.bfloat16)
    bproj = N.QkvBackwardDataParams(weight=wb_d.data_ptr(), grad_input=mx_dx.data_ptr(), local_tokens=m, hidden=hidden,
                                    batch=batch, q_heads=q, kv_heads=kv, head_dim=d, world_size=world, rank=rank,
                                    num_comm_ctas=8, epoch=1, alpha=1.0)
    bproj.gemm_tuning.max_swizzle_size = 4
    mx_ready = torch.zeros(api.qkv_backward_ready_elements(bproj), dtype=torch.int32, device=dev)
    bproj.peer_dqkv_staging[rank] = mx_staging.data_ptr()
    bproj.peer_ready[rank] = mx_ready.data_ptr()
    for r in range(world):
        bproj.peer_done_epoch[r] = gsym["mxb_done"].peer_ptrs[r]
    rc, ws_bytes = api.qkv_backward_mxfp8_data_workspace_size(bproj)
    assert rc == 0
    scratch2 = torch.full((ws_bytes + 256,), 0x5A, dtype=torch.uint8, device=dev)
    mbp = N.Mxfp8QkvBackwardDataParams(projection=bproj, workspace=(scratch2.data_ptr() + 255) // 256 * 256,
                                       workspace_bytes=ws_bytes)
    act = lambda r, name, seg: N.Mxfp8Activation(
        data=gsym[f"g{name}_data"].peer_ptrs[r], scales=gsym[f"g{name}_scales"].peer_ptrs[r],
        data_bytes=planes_q[0][seg][0].size, scale_bytes=planes_q[0][seg][1].size)
    for r in range(world):
        mbp.peer_input[r] = N.Mxfp8QkvBackwardInput(
            grad_q=act(r, "q", 0), grad_k=act(r, "k", 1), grad_v=act(r, "v", 2),
            master_q=gsym["gq_master"].peer_ptrs[r], master_k=gsym["gk_master"].peer_ptrs[r],
            master_v=gsym["gv_master"].peer_ptrs[r])
    torch.cuda.synchronize()
    dist.barrier()
    assert api.launch_qkv_backward_mxfp8_data(mbp, 0, opts) == 0
    torch.cuda.synchronize()
    status = api.read_status()
    assert status[0] == 0, status[:8]
    assert np.array_equal(bits(mx_staging), want_staging), "mxfp8 backward: routed BF16 masters"
    import ctypes as C
    packed = np.empty((m, n), dtype=np.uint8)
    packed_s = np.zeros(O.lib().fo_mxfp8_scale_bytes(m, n), dtype=np.uint8)
    owner, seg_out, off_out = C.c_int32(), C.c_int32(), C.c_int64()
    for row in range(m):
        for head in range(q + 2 * kv):
            O.lib().fo_qkv_backward_source(world, rank, s, q, kv, d, 0, row, head * d, C.byref(owner), C.byref(seg_out),
                                           C.byref(off_out))
            data, scales = planes_q[owner.value][seg_out.value]
            pw = data.shape[1]
            src_row, src_col = off_out.value // pw, off_out.value % pw
            packed[row, head * d:(head + 1) * d] = data[src_row, src_col:src_col + d]
            for kk in range(0, d, 32):
                packed_s[O.lib().fo_mxfp8_scale_offset(row, head * d + kk, n)] = \
                    scales[O.lib().fo_mxfp8_scale_offset(src_row, src_col + kk, pw)]
    wt_q, wt_s = O.mxfp8_quantize_transposed(wb)
    ok, worst, bad = O.within_tolerance(bits(mx_dx), O.gemm_mxfp8(packed, packed_s, wt_q, wt_s))
    assert ok, ("mxfp8 dX", worst, bad)
    dist.barrier()

    # ---- BF16 output-projection backward: dA = dY Wo, pushed sequence -> head to every peer ------
    ob_hidden = 256
    dys = [synthetic.normal_bf16((m, ob_hidden), synthetic.rank_seed(r) + 301, 0.01) for r in range(world)]
    wob = synthetic.normal_bf16((ob_hidden, ko), synthetic.BASE_SEED + 17, 0.02)
    osym = w.allocate({"ob_routed": rows * (ko // world) * 2, "ob_done": world * N.READY_FLAG_STRIDE * 4})
    osym["ob_routed"].view(torch.int16).fill_(-1)
    dy_d, wob_d = to_dev(dys[rank]), to_dev(wob)
    da = torch.full((m, ko), -1, dtype=torch.int16, device=dev).view(torch.bfloat16)
    obp = N.OprojBackwardDataParams(grad_output=dy_d.data_ptr(), weight=wob_d.data_ptr(),
                                    local_grad_attention=da.data_ptr(), local_tokens=m, hidden=ob_hidden, batch=batch,
                                    q_heads=q, head_dim=d, world_size=world, rank=rank, num_comm_ctas=8, epoch=1,
                                    alpha=1.0)
    obp.gemm_tuning.max_swizzle_size = 4
    ob_ready = torch.zeros(api.oproj_backward_ready_elements(obp), dtype=torch.int32, device=dev)
    obp.ready = ob_ready.data_ptr()
    for r in range(world):
        obp.peer_grad_attention[r] = osym["ob_routed"].peer_ptrs[r]
        obp.peer_done_epoch[r] = osym["ob_done"].peer_ptrs[r]
    torch.cuda.synchronize()
    dist.barrier()
    assert api.launch_oproj_backward_data(obp, 0, opts) == 0
    torch.cuda.synchronize()
    status = api.read_status()
    assert status[0] == 0, status[:8]
    want_da, want_routed, _ = O.oproj_backward(world, batch, s, q, d, dys, wob,
                                               [np.zeros((m, ko), dtype=np.uint16)] * world)
    ok, worst, bad = O.within_tolerance(bits(da), want_da[rank], 0.02, 0.02)
    assert ok, ("dA", worst, bad)
    ok, worst, bad = O.within_tolerance(bits(osym["ob_routed"].view(torch.bfloat16)), want_routed[rank].reshape(-1),
                                        0.02, 0.02)
    assert ok, ("routed dA", worst, bad)
    dist.barrier()
    w.close()
    dist.destroy_process_group()
    print(f"MULTIRANK PASS rank {rank}/{world} route={route_mode}", flush=True)


if __name__ == "__main__":
    main()
