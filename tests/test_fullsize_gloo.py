"""The benchmark's full-size checker (tests/fullsize.py) run as two gloo ranks on CPU: fed with
the oracle's own simulation of both ranks it must pass; with one routed element or one GEMM
element changed it must say so.  This is the host-side logic of the multi-rank validation
(sampled source rows travel between ranks; receiver-view maps trace every sampled element)."""
import os
import socket
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent('''
    import os, sys
    sys.path.insert(0, __ROOT__)
    import numpy as np, torch, torch.distributed as dist
    from fuse_b200 import synthetic
    from oracle import oracle as O
    from tests import fullsize as F
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    F.use_host_threads(world)
    s, q, kv, d, k = 192, 4, 2, 64, 128
    n = (q + 2 * kv) * d
    as_t = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)
    lhs = [synthetic.normal_bf16((s, k), 100 + r, 1.0) for r in range(world)]
    w = synthetic.normal_bf16((n, k), 7, 0.02)
    local, planar = O.qkv_forward(world, 1, s, q, kv, d, lhs, w)
    rows = F.sample_rows(s, count=48, edge=8)
    check = F.check_qkv_forward(world, rank, s, q, kv, d, as_t(lhs[rank]), as_t(w), as_t(local[rank]),
                                as_t(planar[rank]), rows)
    assert check["gemm"]["ok"] and check["route_bitexact"] and check["unwritten_routed"] == 0, check
    # one routed element of a sampled row changed on rank 1 only
    broken = planar[rank].copy()
    if rank == 1:
        broken[int(rows[3]) * (q // world * d) + 5] ^= 1
    check2 = F.check_qkv_forward(world, rank, s, q, kv, d, as_t(lhs[rank]), as_t(w), as_t(local[rank]),
                                 as_t(broken), rows)
    assert check2["route_bitexact"] == (rank != 1), check2
    assert F.merge(check)["ok"] and not F.merge(check2)["ok"]

    ko = q * d
    attn = [synthetic.normal_bf16((s * world, ko // world), 200 + r, 1.0) for r in range(world)]
    wo = synthetic.normal_bf16((96, ko), 9, 0.02)
    for causal in (False, True):
        staging, out = O.oproj_forward(world, rank, 1, s, attn, wo, causal=causal)
        check = F.check_oproj_forward(world, rank, s, ko, as_t(attn[rank]), as_t(staging), as_t(wo), as_t(out), rows,
                                      causal=causal)
        assert check["gemm"]["ok"] and check["route_bitexact"], check
        bad_out = out.copy()
        bad_out[int(rows[0]), 1] = 0x4000  # 2.0: far outside the tolerance
        check = F.check_oproj_forward(world, rank, s, ko, as_t(attn[rank]), as_t(staging), as_t(wo), as_t(bad_out),
                                      rows, causal=causal)
        assert not check["gemm"]["ok"] and check["gemm"]["bad"] == 1, check

    # ---- BF16 backward ----------------------------------------------------------------------
    hid = 96
    rows_g = s * world
    planes = [tuple(synthetic.normal_bf16((rows_g, h // world * d), 300 + 10 * r + seg, 0.01)
                    for seg, h in enumerate((q, kv, kv))) for r in range(world)]
    wb = synthetic.normal_bf16((n, hid), 11, 0.02)
    xs = synthetic.normal_bf16((s, hid), 400 + rank, 1.0)
    for causal in (False, True):
        staging, dx, dw = O.qkv_backward(world, rank, 1, s, q, kv, d, planes, wb, xs, causal=causal)
        check = F.check_qkv_backward_data(world, rank, s, q, kv, d, [as_t(p) for p in planes[rank]], as_t(wb),
                                          as_t(staging), as_t(dx), rows, causal=causal)
        assert check["gemm"]["ok"] and check["route_bitexact"], check
        bad = staging.copy()
        bad[int(rows[5]), 7] ^= 2
        check = F.check_qkv_backward_data(world, rank, s, q, kv, d, [as_t(p) for p in planes[rank]], as_t(wb),
                                          as_t(bad), as_t(dx), rows, causal=causal)
        assert not check["route_bitexact"] and check["route_mismatches"] == 1, check
        picked = np.array([0, 5, n - 1])
        check = F.check_weight_gradient(as_t(staging), as_t(xs), as_t(dw), picked)
        assert check["gemm"]["ok"], check
        dys = [synthetic.normal_bf16((s, hid), 500 + r, 0.01) for r in range(world)]
        wob = synthetic.normal_bf16((hid, ko), 13, 0.02)
        da, routed, _ = O.oproj_backward(world, 1, s, q, d, dys, wob, [np.zeros((s, ko), np.uint16)] * world,
                                         causal=causal)
        check = F.check_oproj_backward_data(world, rank, s, ko, as_t(dys[rank]), as_t(wob), as_t(da[rank]),
                                            as_t(routed[rank]), rows, causal=causal)
        assert check["gemm"]["ok"] and check["route_bitexact"], check

    # ---- MXFP8 output projection: gathered bytes and re-homed scale bytes -------------------------
    sm = 256                      # whole scale atoms per 128-row group
    kx = 256 * world
    shard = kx // world
    u8_t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    attn_mx = [synthetic.normal_bf16((sm * world, shard), 600 + r, 1.0) for r in range(world)]
    quant = [O.mxfp8_quantize(a) for a in attn_mx]
    wmx = synthetic.normal_bf16((64, kx), 17, 0.02)
    wq, ws = O.mxfp8_quantize(wmx)
    staged = np.empty((sm, kx), np.uint8)
    staged_s = np.zeros(O.lib().fo_mxfp8_scale_bytes(sm, kx), np.uint8)
    for row in range(sm):
        src_row = O.lib().fo_global_row(world, rank, sm, 0, row)
        for j in range(world):
            staged[row, j * shard:(j + 1) * shard] = quant[j][0][src_row]
            for kk in range(0, shard, 32):
                staged_s[O.lib().fo_mxfp8_scale_offset(row, j * shard + kk, kx)] = \
                    quant[j][1][O.lib().fo_mxfp8_scale_offset(src_row, kk, shard)]
    out_mx = O.gemm_mxfp8(staged, staged_s, wq, ws)
    rows_mx = F.sample_rows(sm, count=40, edge=8)
    check = F.check_oproj_forward_mxfp8(world, rank, sm, kx, u8_t(quant[rank][0]), u8_t(quant[rank][1]), u8_t(staged),
                                        u8_t(staged_s), as_t(wmx), u8_t(wq), u8_t(ws), as_t(out_mx), rows_mx)
    assert check["gemm"]["ok"] and check["route_bitexact"], check
    bad_s = staged_s.copy()
    bad_s[O.lib().fo_mxfp8_scale_offset(int(rows_mx[2]), 64, kx)] ^= 1
    check = F.check_oproj_forward_mxfp8(world, rank, sm, kx, u8_t(quant[rank][0]), u8_t(quant[rank][1]), u8_t(staged),
                                        u8_t(bad_s), as_t(wmx), u8_t(wq), u8_t(ws), as_t(out_mx), rows_mx)
    assert not check["route_bitexact"], check

    # ---- MXFP8 QKV forward ----------------------------------------------------------------------
    qf, kvf, df, kf = 2 * world, world, 128, 256
    nf = (qf + 2 * kvf) * df
    acts = [O.mxfp8_quantize(synthetic.normal_bf16((sm, kf), 800 + r, 1.0)) for r in range(world)]
    wf = synthetic.normal_bf16((nf, kf), 29, 0.02)
    wfq, wfs = O.mxfp8_quantize(wf)
    locals_f = [O.gemm_mxfp8(a[0], a[1], wfq, wfs) for a in acts]
    planar_f = [np.full(sm * world * nf // world, 0xFFFF, dtype=np.uint16) for _ in range(world)]
    table_f = O.ptr_array(planar_f)
    for r in range(world):
        O.lib().fo_qkv_forward_route(world, r, 1, sm, qf, kvf, df, O.ptr(locals_f[r]), nf, table_f)
    check = F.check_qkv_forward_mxfp8(world, rank, sm, qf, kvf, df, u8_t(acts[rank][0]), u8_t(acts[rank][1]), as_t(wf),
                                      u8_t(wfq), u8_t(wfs), as_t(locals_f[rank]), as_t(planar_f[rank]), rows_mx)
    assert check["gemm"]["ok"] and check["route_bitexact"] and check["unwritten_routed"] == 0, check
    bad_w = wfq.copy()
    bad_w[3, 5] ^= 1                       # one byte of the in-kernel weight quantisation
    check = F.check_qkv_forward_mxfp8(world, rank, sm, qf, kvf, df, u8_t(acts[rank][0]), u8_t(acts[rank][1]), as_t(wf),
                                      u8_t(bad_w), u8_t(wfs), as_t(locals_f[rank]), as_t(planar_f[rank]), rows_mx)
    assert not check["route_bitexact"], check

    # ---- MXFP8 output-projection backward data ----------------------------------------------------
    hb, qb = 128, 2 * world
    ab = qb * 128
    dys_b = [synthetic.normal_bf16((sm, hb), 900 + r, 0.01) for r in range(world)]
    dyq_b = [O.mxfp8_quantize(x) for x in dys_b]
    wob = synthetic.normal_bf16((hb, ab), 31, 0.02)
    wobq, wobs = O.mxfp8_quantize_transposed(wob)
    da_b = [O.gemm_mxfp8(dq[0], dq[1], wobq, wobs) for dq in dyq_b]
    shard_b = ab // world
    routed_b = np.empty((sm * world, shard_b), np.uint16)          # this rank's head shard of every rank's dA
    for src in range(world):
        routed_b[src * sm:(src + 1) * sm] = da_b[src][:, rank * shard_b:(rank + 1) * shard_b]
    check = F.check_oproj_backward_data_mxfp8(world, rank, sm, ab, u8_t(dyq_b[rank][0]), u8_t(dyq_b[rank][1]), as_t(wob),
                                              as_t(da_b[rank]), as_t(routed_b), rows_mx)
    assert check["gemm"]["ok"] and check["route_bitexact"], check
    bad_r = routed_b.copy()
    bad_r[int(rows_mx[1]), 3] ^= 1
    check = F.check_oproj_backward_data_mxfp8(world, rank, sm, ab, u8_t(dyq_b[rank][0]), u8_t(dyq_b[rank][1]), as_t(wob),
                                              as_t(da_b[rank]), as_t(bad_r), rows_mx)
    assert not check["route_bitexact"], check

    # ---- MXFP8 QKV backward data --------------------------------------------------------------
    import ctypes as C
    qm, kvm, dm, hm = 2 * world, world, 128, 64
    width_m = (qm + 2 * kvm) * dm
    planes_m = [tuple(synthetic.normal_bf16((sm * world, h // world * dm), 700 + 10 * r + seg, 0.01)
                      for seg, h in enumerate((qm, kvm, kvm))) for r in range(world)]
    planes_mq = [tuple(O.mxfp8_quantize(pl) for pl in planes_m[r]) for r in range(world)]
    wbm = synthetic.normal_bf16((width_m, hm), 23, 0.02)
    staging_m, _, _ = O.qkv_backward(world, rank, 1, sm, qm, kvm, dm, planes_m, wbm, synthetic.normal_bf16((sm, hm), 1, 1.0))
    packed = np.empty((sm, width_m), np.uint8)
    packed_s = np.zeros(O.lib().fo_mxfp8_scale_bytes(sm, width_m), np.uint8)
    owner, seg_out, off_out = C.c_int32(), C.c_int32(), C.c_int64()
    for row in range(sm):
        for head in range(qm + 2 * kvm):
            O.lib().fo_qkv_backward_source(world, rank, sm, qm, kvm, dm, 0, row, head * dm, C.byref(owner),
                                           C.byref(seg_out), C.byref(off_out))
            data, scales = planes_mq[owner.value][seg_out.value]
            pw = data.shape[1]
            src_row, src_col = off_out.value // pw, off_out.value % pw
            packed[row, head * dm:(head + 1) * dm] = data[src_row, src_col:src_col + dm]
            for kk in range(0, dm, 32):
                packed_s[O.lib().fo_mxfp8_scale_offset(row, head * dm + kk, width_m)] = \
                    scales[O.lib().fo_mxfp8_scale_offset(src_row, src_col + kk, pw)]
    wt_q, wt_s = O.mxfp8_quantize_transposed(wbm)
    dx_m = O.gemm_mxfp8(packed, packed_s, wt_q, wt_s)
    check = F.check_qkv_backward_data_mxfp8(
        world, rank, sm, qm, kvm, [as_t(p) for p in planes_m[rank]], [u8_t(qd) for qd, _ in planes_mq[rank]],
        [u8_t(qs) for _, qs in planes_mq[rank]], as_t(wbm), as_t(staging_m), u8_t(packed), u8_t(packed_s), u8_t(wt_q),
        u8_t(wt_s), as_t(dx_m), rows_mx)
    assert check["gemm"]["ok"] and check["route_bitexact"], check
    xs_m = synthetic.normal_bf16((sm, hm), 800 + rank, 1.0)
    aq, asc = O.mxfp8_quantize_transposed(staging_m)
    bq, bsc = O.mxfp8_quantize_transposed(xs_m)
    dw_m = O.gemm_mxfp8(aq, asc, bq, bsc)
    check = F.check_weight_gradient_mxfp8(as_t(staging_m), as_t(xs_m), as_t(dw_m), np.array([0, 3, width_m - 1]),
                                          np.array([1, 2, hm - 1]))
    assert check["gemm"]["ok"], check

    # ---- MoE dispatch + FC1 ---------------------------------------------------------------------
    e_local, t, topk, mk, mn, cap = 3, 40, 2, 64, 32, 64
    rng = np.random.default_rng(5)
    scores = [rng.standard_normal((t, e_local * world)).astype(np.float32) for _ in range(world)]
    chosen = []
    for sc in scores:
        c = np.empty((t, topk), np.int32)
        O.lib().fo_moe_topk(O.ptr(sc), t, e_local * world, topk, O.ptr(c))
        chosen.append(c)
    offs = np.empty(e_local + 1, np.int32)
    total = O.lib().fo_moe_build_rows(world, rank, e_local, t, topk, O.ptr_array(chosen), O.ptr(offs), None)
    src = np.empty((max(total, 1), 3), np.int32)
    O.lib().fo_moe_build_rows(world, rank, e_local, t, topk, O.ptr_array(chosen), O.ptr(offs), O.ptr(src))
    toks = [synthetic.normal_bf16((t, mk), 900 + r, 1.0) for r in range(world)]
    ew = synthetic.normal_bf16((e_local, mn, mk), 950 + rank, 0.02)
    lhs_m = np.full((e_local, cap, mk), 0xFFFF, np.uint16)
    eo_m = np.full((e_local, cap, mn), 0xFFFF, np.uint16)
    assert O.lib().fo_moe_dispatch_fc1(e_local, O.ptr(offs), O.ptr(src), O.ptr_array(toks), O.ptr(ew), mn, mk, cap,
                                       O.ptr(lhs_m), O.ptr(eo_m)) == 0
    check = F.check_moe_dispatch_fc1(world, as_t(toks[rank]), as_t(lhs_m), as_t(eo_m), as_t(ew), offs, src, per_expert=4)
    assert check["gemm"]["ok"] and check["route_bitexact"] and check["unwritten_local"] == 0, check
    lhs_m[0, 0, 3] ^= 1
    check = F.check_moe_dispatch_fc1(world, as_t(toks[rank]), as_t(lhs_m), as_t(eo_m), as_t(ew), offs, src, per_expert=4)
    assert (not check["route_bitexact"]) == (offs[1] > offs[0]), check

    # ---- MoE FC2 + combine: every rank simulates all ranks, then checks its own -----------------
    routes = []
    for r in range(world):
        o = np.empty(e_local + 1, np.int32)
        tot = O.lib().fo_moe_build_rows(world, r, e_local, t, topk, O.ptr_array(chosen), O.ptr(o), None)
        sr = np.empty((max(tot, 1), 3), np.int32)
        O.lib().fo_moe_build_rows(world, r, e_local, t, topk, O.ptr_array(chosen), O.ptr(o), O.ptr(sr))
        routes.append((o, sr[:tot]))
    lhs_c = [synthetic.normal_bf16((e_local, cap, mk), 1000 + r, 1.0) for r in range(world)]
    w_c = [synthetic.normal_bf16((e_local, mn, mk), 1100 + r, 0.02) for r in range(world)]
    recv_c = [np.full((t * topk, mn), 0xFFFF, np.uint16) for _ in range(world)]
    outs_c = []
    for r in range(world):
        out_r = np.full((e_local, cap, mn), 0xFFFF, np.uint16)
        assert O.lib().fo_moe_fc2_combine(e_local, O.ptr(routes[r][0]), O.ptr(np.ascontiguousarray(routes[r][1])), O.ptr(lhs_c[r]),
                                          O.ptr(w_c[r]), mn, mk, cap, topk, O.ptr(out_r), O.ptr_array(recv_c)) == 0
        outs_c.append(out_r)
    check = F.check_moe_fc2_combine(world, rank, as_t(lhs_c[rank]), as_t(w_c[rank]), as_t(outs_c[rank]), as_t(recv_c[rank]),
                                    routes[rank][0], routes[rank][1], chosen, e_local, topk, sample=64, per_expert=4)
    assert check["gemm"]["ok"] and check["route_bitexact"] and check["unwritten_routed"] == 0, check
    broken = recv_c[rank].copy()
    broken[0, 0] ^= 1          # branch (token 0, slot 0) is always in the sample
    check = F.check_moe_fc2_combine(world, rank, as_t(lhs_c[rank]), as_t(w_c[rank]), as_t(outs_c[rank]), as_t(broken),
                                    routes[rank][0], routes[rank][1], chosen, e_local, topk, sample=64, per_expert=4)
    assert not check["route_bitexact"], check

    dist.barrier()
    dist.destroy_process_group()
    print("FULLSIZE PASS", rank)
''').replace("__ROOT__", repr(ROOT))


def test_fullsize_checker_with_two_gloo_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    result = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert result.returncode == 0, result.stdout[-3000:] + result.stderr[-3000:]
    assert result.stdout.count("FULLSIZE PASS") == 2
