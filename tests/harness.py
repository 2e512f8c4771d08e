"""GPU-side helpers for the parity tests: move BF16 bit patterns to the device, drive the
operators through the C ABI (fuse_b200.api), bring results back as numpy bit patterns.

Several ranks are emulated on ONE GPU by launching each rank's kernel in turn on one stream
with all `peer_*` pointers aimed at buffers of the same device; the cross-rank completion wait
is skipped (FUSE_B200_SKIP_PEER_WAIT) because later launches play the peers."""
from __future__ import annotations

import numpy as np
import torch

from fuse_b200 import _native as N
from fuse_b200 import api

DEV = "cuda:0"
POISON = 0xFFFF  # BF16 NaN pattern: outputs are poisoned before every run


def to_device(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(DEV).view(torch.bfloat16)


def to_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().view(torch.int16).cpu().numpy().view(np.uint16)


def poisoned(*shape) -> torch.Tensor:
    return torch.full(shape, -1, dtype=torch.int16, device=DEV).view(torch.bfloat16)


def options(wait_ms: float = 500.0, flags: int = 0, block_n: int = 0) -> N.Options:
    o = N.Options()
    o.wait_budget_ns = int(wait_ms * 1e6)
    o.flags = flags
    o.block_n = block_n
    return o


def check_status():
    torch.cuda.synchronize()
    status = api.read_status(clear=True)
    assert status[0] == 0, f"device wait gave up: {status[:8]}"


def qkv_forward(world, batch, seq_local, q_heads, kv_heads, head_dim, lhs_bits, w_bits, comm=4,
                alpha=1.0, raster=N.RASTER_HEURISTIC, swizzle=4, block_n=0, epochs=1, route="comm",
                vector_epilogue=False, defer_v=False, interleaved=False):
    """Runs every rank of the QKV operator (route: "comm" CTAs or "direct" epilogue push).  Returns (local_outputs, peer_outputs) as bits.
    defer_v: UlyssesRoute.defer_v_a2a (V stays local, Q | K share one tensor per destination) with a
    completion_epoch word per rank, which must hold the last epoch afterwards."""
    m = batch * seq_local
    n = (q_heads + 2 * kv_heads) * head_dim
    k = w_bits.shape[1]
    rows = batch * seq_local * world
    w = to_device(w_bits)
    xs = [to_device(x) for x in lhs_bits]
    problem = N.GemmProblem(m, n, k, raster=raster, max_swizzle_size=swizzle)
    local = [poisoned(m, n) for _ in range(world)]
    peer = [poisoned(rows * n // world) for _ in range(world)]
    done = [torch.zeros(world * N.READY_FLAG_STRIDE, dtype=torch.int32, device=DEV) for _ in range(world)]
    ready = [torch.zeros(api.qkv_ready_elements(problem), dtype=torch.int32, device=DEV) for _ in range(world)]
    completion = [torch.zeros(N.READY_FLAG_STRIDE, dtype=torch.int32, device=DEV) for _ in range(world)]
    route_flag = N.QKV_ROUTE_DIRECT if route == "direct" else N.QKV_ROUTE_COMM_CTAS
    opts = options(flags=(N.SKIP_PEER_WAIT if world > 1 else 0) | route_flag |
                   (N.VECTOR_EPILOGUE if vector_epilogue else 0), block_n=block_n)
    for epoch in range(1, epochs + 1):
        for r in range(world):
            route = N.UlyssesRoute(world_size=world, rank=r, batch=batch, global_seq=seq_local * world,
                                   seq_local=seq_local, q_heads=q_heads, kv_heads=kv_heads,
                                   head_dim=head_dim, kind=N.ROUTE_QKV_GQA_PACK, defer_v_a2a=int(defer_v),
                                   qkv_peer_interleaved=int(interleaved))
            p = N.GemmA2AParams(lhs=xs[r].data_ptr(), rhs_nt=w.data_ptr(), local_output=local[r].data_ptr(),
                                ready=ready[r].data_ptr(), gemm=problem, route=route, num_comm_ctas=comm,
                                epoch=epoch, alpha=alpha,
                                completion_epoch=completion[r].data_ptr() if defer_v else None)
            for peer_rank in range(world):
                p.peer_output[peer_rank] = peer[peer_rank].data_ptr()
                p.peer_route_done_epoch[peer_rank] = done[peer_rank].data_ptr()
            rc = api.launch_gemm_a2a_cutlass(p, 0, opts)
            assert rc == 0, f"launch_gemm_a2a_cutlass -> cudaError {rc}"
    check_status()
    for d in done:  # every source told every destination
        assert (d[::N.READY_FLAG_STRIDE][:world] == epochs).all()
    for c in completion:  # the local completion word: the last epoch with the deferred V, untouched otherwise
        assert int(c[0]) == (epochs if defer_v else 0)
    return [to_bits(t) for t in local], [to_bits(t) for t in peer]


def oproj_forward(world, rank, batch, seq_local, peer_bits, w_bits, comm=4, causal=False, cyclic=False,
                  alpha=1.0, raster=N.RASTER_HEURISTIC, swizzle=8, block_n=0, pull="bulk",
                  vector_epilogue=False):
    """Runs one rank of the output-projection operator (pull: "bulk" copy pipeline or "vector"
    loads/stores).  Returns (staging, output) bits."""
    n, k = w_bits.shape
    m = batch * seq_local
    w = to_device(w_bits)
    peers = [to_device(x) for x in peer_bits]
    staging, out = poisoned(m, k), poisoned(m, n)
    problem = N.GemmProblem(m, n, k, raster=raster, max_swizzle_size=swizzle)
    route = N.UlyssesRoute(world_size=world, rank=rank, batch=batch, global_seq=seq_local * world,
                           seq_local=seq_local, kind=N.ROUTE_HEAD_TO_SEQUENCE, direction=N.ROUTE_INVERSE,
                           causal_load_balanced=int(causal), cyclic_peer_order=int(cyclic))
    ready = torch.zeros(api.a2a_lhs_gemm_ready_elements(problem, route), dtype=torch.int32, device=DEV)
    p = N.A2AGemmParams(input_staging=staging.data_ptr(), rhs_nt=w.data_ptr(), output=out.data_ptr(),
                        ready=ready.data_ptr(), gemm=problem, route=route, num_comm_ctas=comm, epoch=1,
                        alpha=alpha)
    for q in range(world):
        p.peer_input[q] = peers[q].data_ptr()
    flags = (N.VECTOR_PULL if pull == "vector" else 0) | (N.VECTOR_EPILOGUE if vector_epilogue else 0)
    rc = api.launch_a2a_gemm_cutlass(p, 0, options(block_n=block_n, flags=flags))
    assert rc == 0, f"launch_a2a_gemm_cutlass -> cudaError {rc}"
    check_status()
    return to_bits(staging), to_bits(out)


def qkv_backward(world, batch, seq_local, q_heads, kv_heads, head_dim, planes_bits, w_bits, x_bits, comm=4,
                 causal=False, alpha=1.0, beta=0.0, dw_init_bits=None, block_n=0, tuning=(1, False), vector=False,
                 starved_first=False):
    """Runs every rank of the QKV backward (data + weight).  planes_bits[r] = (dQ, dK, dV) of rank r.
    Several ranks on one GPU: every rank's communication CTAs push first (COMM_ONLY), then every
    rank's GEMM runs (COMPUTE_ONLY).  Returns per rank (staging, dX, dW) bits.
    starved_first: before that, rank 0's GEMM is launched alone at epoch 1 with a 30 ms wait
    budget -- nobody has pushed, so its head gates run out -- and the launch must report the
    time-out WITHOUT telling any peer that its transfers are complete; the real run then uses
    epoch 2."""
    m = batch * seq_local
    width = (q_heads + 2 * kv_heads) * head_dim
    hidden = w_bits.shape[1]
    w = to_device(w_bits)
    planes = [[to_device(pl) for pl in planes_bits[r]] for r in range(world)]
    xs = [to_device(x) for x in x_bits]
    staging = [poisoned(m, width) for _ in range(world)]
    dx = [poisoned(m, hidden) for _ in range(world)]
    dw = [to_device(dw_init_bits[r]) if dw_init_bits is not None else poisoned(width, hidden) for r in range(world)]
    done = [torch.zeros(world * N.READY_FLAG_STRIDE, dtype=torch.int32, device=DEV) for _ in range(world)]
    params = []
    for r in range(world):
        p = N.QkvBackwardDataParams(grad_q=planes[r][0].data_ptr(), grad_k=planes[r][1].data_ptr(),
                                    grad_v=planes[r][2].data_ptr(), weight=w.data_ptr(),
                                    grad_input=dx[r].data_ptr(), local_tokens=m, hidden=hidden, batch=batch,
                                    q_heads=q_heads, kv_heads=kv_heads, head_dim=head_dim, world_size=world,
                                    rank=r, num_comm_ctas=comm, epoch=1, causal_load_balanced=int(causal),
                                    alpha=alpha)
        p.gemm_tuning.max_swizzle_size = tuning[0]
        p.gemm_tuning.along_m = int(tuning[1])
        params.append(p)
    ready = [torch.zeros(api.qkv_backward_ready_elements(params[0]), dtype=torch.int32, device=DEV)
             for _ in range(world)]
    for p in params:
        for peer in range(world):
            p.peer_dqkv_staging[peer] = staging[peer].data_ptr()
            p.peer_ready[peer] = ready[peer].data_ptr()
            p.peer_done_epoch[peer] = done[peer].data_ptr()
    if starved_first:
        assert world > 1
        opts = options(wait_ms=30.0, flags=N.COMPUTE_ONLY | N.SKIP_PEER_WAIT, block_n=block_n)
        rc = api.launch_qkv_backward_data(params[0], 0, opts)
        assert rc == 0, f"launch_qkv_backward_data -> cudaError {rc}"
        torch.cuda.synchronize()
        status = api.read_status(clear=True)
        assert status[0] != 0 and status[1] in (1, 2, 3), f"the starved launch did not report: {status[:8]}"
        for d in done:  # a failed launch publishes no completion epoch
            assert int(d.abs().sum()) == 0, "a launch that timed out told its peers that it was complete"
        for p in params:
            p.epoch = 2
    phases = [0] if world == 1 else [N.COMM_ONLY, N.COMPUTE_ONLY]
    for phase in phases:
        for p in params:
            opts = options(flags=phase | (N.SKIP_PEER_WAIT if world > 1 else 0) | (N.VECTOR_PULL if vector else 0),
                           block_n=block_n)
            rc = api.launch_qkv_backward_data(p, 0, opts)
            assert rc == 0, f"launch_qkv_backward_data -> cudaError {rc}"
    check_status()
    for r in range(world):
        wp = N.QkvBackwardWeightParams(dqkv_staging=staging[r].data_ptr(), saved_input=xs[r].data_ptr(),
                                       grad_weight=dw[r].data_ptr(), local_tokens=m, hidden=hidden,
                                       q_heads=q_heads, kv_heads=kv_heads, head_dim=head_dim, alpha=alpha,
                                       beta=beta)
        rc = api.launch_qkv_backward_weight(wp, 0)
        assert rc == 0, f"launch_qkv_backward_weight -> cudaError {rc}"
    check_status()
    return [(to_bits(staging[r]), to_bits(dx[r]), to_bits(dw[r])) for r in range(world)]


def oproj_backward(world, batch, seq_local, q_heads, head_dim, dy_bits, wo_bits, attn_bits, comm=4,
                   causal=False, alpha=1.0, route="direct", vector_epilogue=False, block_n=0):
    """Runs every rank of the output-projection backward.  Returns (dA list, routed list, dWo list)."""
    m = batch * seq_local
    hidden, a = wo_bits.shape
    rows = batch * seq_local * world
    wo = to_device(wo_bits)
    dys = [to_device(x) for x in dy_bits]
    attn = [to_device(x) for x in attn_bits]
    da = [poisoned(m, a) for _ in range(world)]
    routed = [poisoned(rows * (a // world)) for _ in range(world)]
    dwo = [poisoned(hidden, a) for _ in range(world)]
    done = [torch.zeros(world * N.READY_FLAG_STRIDE, dtype=torch.int32, device=DEV) for _ in range(world)]
    for r in range(world):
        p = N.OprojBackwardDataParams(grad_output=dys[r].data_ptr(), weight=wo.data_ptr(),
                                      local_grad_attention=da[r].data_ptr(), local_tokens=m, hidden=hidden,
                                      batch=batch, q_heads=q_heads, head_dim=head_dim, world_size=world, rank=r,
                                      num_comm_ctas=comm, epoch=1, causal_load_balanced=int(causal), alpha=alpha)
        p.gemm_tuning.max_swizzle_size = 4
        ready = torch.zeros(api.oproj_backward_ready_elements(p), dtype=torch.int32, device=DEV)
        p.ready = ready.data_ptr()
        for peer in range(world):
            p.peer_grad_attention[peer] = routed[peer].data_ptr()
            p.peer_done_epoch[peer] = done[peer].data_ptr()
        flags = (N.SKIP_PEER_WAIT if world > 1 else 0) | (N.VECTOR_EPILOGUE if vector_epilogue else 0) | \
            (N.QKV_ROUTE_COMM_CTAS if route == "comm" else N.QKV_ROUTE_DIRECT)
        rc = api.launch_oproj_backward_data(p, 0, options(flags=flags, block_n=block_n))
        assert rc == 0, f"launch_oproj_backward_data -> cudaError {rc}"
        wp = N.OprojBackwardWeightParams(grad_output=dys[r].data_ptr(), saved_attention=attn[r].data_ptr(),
                                         grad_weight=dwo[r].data_ptr(), local_tokens=m, hidden=hidden,
                                         q_heads=q_heads, head_dim=head_dim, alpha=alpha)
        rc = api.launch_oproj_backward_weight(wp, 0)
        assert rc == 0, f"launch_oproj_backward_weight -> cudaError {rc}"
        torch.cuda.synchronize()
    check_status()
    return [to_bits(t) for t in da], [to_bits(t) for t in routed], [to_bits(t) for t in dwo]


def to_device_u8(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def quantize_mxfp8(source_bits: np.ndarray, transposed: bool = False):
    """Runs the CUDA quantiser on a [rows, cols] BF16 array.  Returns (data, scales) numpy uint8."""
    rows, cols = source_bits.shape
    src = to_device(source_bits)
    out_rows, out_k = (cols, rows) if transposed else (rows, cols)
    data = torch.full((out_rows, out_k), 0xAB, dtype=torch.uint8, device=DEV)
    # zero-filled: K-block slots of a partly used scale atom are never written by the quantiser
    scales = torch.zeros(api.mxfp8_scale_bytes(out_rows, out_k), dtype=torch.uint8, device=DEV)
    fn = api.quantize_mxfp8_transposed if transposed else api.quantize_mxfp8
    rc = fn(src.data_ptr(), cols, rows, cols, data.data_ptr(), scales.data_ptr(), 0)
    assert rc == 0, f"quantize -> cudaError {rc}"
    torch.cuda.synchronize()
    return data.cpu().numpy(), scales.cpu().numpy()


def qkv_forward_mxfp8(world, batch, seq_local, q_heads, kv_heads, head_dim, act_data, act_scales, w_bits, comm=4,
                      alpha=1.0, route="direct", mode="full", swizzle=4, block_n=0):
    """Runs every rank of the MXFP8 QKV operator.  act_data[r] uint8 [M, K], act_scales[r] native
    scale bytes; w_bits BF16 master weight [N, K].  mode: "full" (weight quantised in-kernel),
    "prepared" (prepare + prequantised launch) or "compute" (GEMM only, no routing).
    Returns (local_outputs, peer_outputs, quantised_weight (data, scales))."""
    m = batch * seq_local
    n, k = w_bits.shape
    rows = batch * seq_local * world
    w = to_device(w_bits)
    problem = N.GemmProblem(m, n, k, max_swizzle_size=swizzle)
    rc, ws_bytes = api.gemm_a2a_mxfp8_workspace_size(problem)
    assert rc == 0
    local = [poisoned(m, n) for _ in range(world)]
    peer = [poisoned(rows * n // world) for _ in range(world)]
    done = [torch.zeros(world * N.READY_FLAG_STRIDE, dtype=torch.int32, device=DEV) for _ in range(world)]
    ready = [torch.zeros(api.qkv_ready_elements(problem), dtype=torch.int32, device=DEV) for _ in range(world)]
    workspaces = []
    flags = (N.SKIP_PEER_WAIT if world > 1 else 0) | (N.QKV_ROUTE_DIRECT if route == "direct" else N.QKV_ROUTE_COMM_CTAS)
    for r in range(world):
        data, scales = to_device_u8(act_data[r]), to_device_u8(act_scales[r])
        workspace = torch.full((ws_bytes + 256,), 0x5A, dtype=torch.uint8, device=DEV)
        base = (workspace.data_ptr() + 255) // 256 * 256
        workspaces.append((workspace, base))
        route_rec = N.UlyssesRoute(world_size=world, rank=r, batch=batch, global_seq=seq_local * world,
                                   seq_local=seq_local, q_heads=q_heads, kv_heads=kv_heads, head_dim=head_dim,
                                   kind=N.ROUTE_QKV_GQA_PACK)
        proj = N.GemmA2AParams(rhs_nt=w.data_ptr(), local_output=local[r].data_ptr(), ready=ready[r].data_ptr(),
                               gemm=problem, route=route_rec, num_comm_ctas=comm, epoch=1, alpha=alpha)
        for q in range(world):
            proj.peer_output[q] = peer[q].data_ptr()
            proj.peer_route_done_epoch[q] = done[q].data_ptr()
        mp = N.Mxfp8GemmA2AParams(projection=proj, workspace=base, workspace_bytes=ws_bytes,
                                  activation=N.Mxfp8Activation(data=data.data_ptr(), scales=scales.data_ptr(),
                                                               data_bytes=data.numel(), scale_bytes=scales.numel()))
        opts = options(flags=flags, block_n=block_n)
        if mode == "full":
            rc = api.launch_gemm_a2a_mxfp8_cutlass(mp, 0, opts)
        else:
            rc = api.prepare_gemm_a2a_mxfp8(mp, 0)
            assert rc == 0, f"prepare -> cudaError {rc}"
            rc = (api.launch_gemm_a2a_mxfp8_prequantized(mp, 0, opts) if mode == "prepared"
                  else api.launch_gemm_a2a_mxfp8_compute_reference(mp, 0))
        assert rc == 0, f"mxfp8 launch -> cudaError {rc}"
        torch.cuda.synchronize()
    check_status()
    workspace, base = workspaces[0]
    offset = base - workspace.data_ptr()
    wq = workspace[offset:offset + n * k].cpu().numpy().reshape(n, k)
    sf_off = offset + (n * k + 255) // 256 * 256
    wsf = workspace[sf_off:sf_off + api.mxfp8_scale_bytes(n, k)].cpu().numpy()
    return [to_bits(t) for t in local], [to_bits(t) for t in peer], (wq, wsf)


def oproj_forward_mxfp8(world, rank, batch, seq_local, peer_data, peer_scales, w_bits, comm=4, causal=False,
                        cyclic=False, alpha=1.0, block_n=0, window=(0, 0), expect_rc=0):
    """One rank of the MXFP8 output-projection operator.  peer_data[p] uint8 [B*S_global, K/world],
    peer_scales[p] its native scale bytes.  Returns (staged bytes [M,K], staged scales, output bits)."""
    n, k = w_bits.shape
    m = batch * seq_local
    w = to_device(w_bits)
    problem = N.GemmProblem(m, n, k, max_swizzle_size=8)
    rc, ws_bytes = api.a2a_gemm_mxfp8_workspace_size(problem)
    assert rc == 0
    workspace = torch.full((ws_bytes + 256,), 0x5A, dtype=torch.uint8, device=DEV)  # garbage scratch
    base = (workspace.data_ptr() + 255) // 256 * 256
    out = poisoned(m, n)
    datas = [to_device_u8(x) for x in peer_data]
    scales = [to_device_u8(x) for x in peer_scales]
    route = N.UlyssesRoute(world_size=world, rank=rank, batch=batch, global_seq=seq_local * world,
                           seq_local=seq_local, kind=N.ROUTE_HEAD_TO_SEQUENCE, direction=N.ROUTE_INVERSE,
                           causal_load_balanced=int(causal), cyclic_peer_order=int(cyclic))
    proj = N.A2AGemmParams(rhs_nt=w.data_ptr(), output=out.data_ptr(), gemm=problem, route=route,
                           num_comm_ctas=comm, epoch=1, alpha=alpha)
    mp = N.Mxfp8A2AGemmParams(projection=proj, workspace=base, workspace_bytes=ws_bytes,
                              m_window_tiles=window[0], n_group_tiles=window[1])
    for q in range(world):
        mp.activation[q] = N.Mxfp8Activation(data=datas[q].data_ptr(), scales=scales[q].data_ptr(),
                                             data_bytes=datas[q].numel(), scale_bytes=scales[q].numel())
    rc = api.launch_a2a_gemm_mxfp8_cutlass(mp, 0, options(block_n=block_n))
    if expect_rc != 0:
        assert rc == expect_rc, f"launch_a2a_gemm_mxfp8_cutlass -> cudaError {rc}, expected {expect_rc}"
        return None
    assert rc == 0, f"launch_a2a_gemm_mxfp8_cutlass -> cudaError {rc}"
    check_status()
    view = api.a2a_gemm_mxfp8_staging_view(mp)
    off = view.data - workspace.data_ptr()
    staged = workspace[off:off + m * k].cpu().numpy().reshape(m, k)
    soff = view.scales - workspace.data_ptr()
    staged_scales = workspace[soff:soff + view.scale_bytes].cpu().numpy()
    return staged, staged_scales, to_bits(out)


def moe_dispatch_fc1(world, rank, experts_local, tokens_bits, weights_bits, row_offsets, sources, capacity,
                     comm=4, compute=128, tile_n=256, launches=1, second_route=None, mma_sm_count=1,
                     starved_first=False, graph=False):
    """One rank of the MoE dispatch -> FC1 grouped GEMM.  tokens_bits[r] [T, K] per rank;
    weights_bits [experts_local, N, K]; row_offsets int64 [E+1]; sources int32 [rows, 3].
    Returns (lhs [E, capacity, K] bits, output [E, capacity, N] bits); unused capacity holds 0x7f7f.
    With `second_route` = (row_offsets, sources) the same plan is launched again with new device
    routes (no re-creation), and that launch's results are returned.
    starved_first (world > 1): the plan is first launched with a 30 ms wait budget while no peer has
    entered the invocation -- the pull's wait for the peers' started epoch runs out, the launch must
    return with a status record -- and is then launched normally.
    graph: after one eager launch the launch is captured into a CUDA graph once, and every launch
    counted by `launches` and the one with `second_route` is a replay of that graph (the row counts
    and routes are read on the device, so a replay follows new routes)."""
    e, n, k = weights_bits.shape
    toks = [to_device(t) for t in tokens_bits]
    w = to_device(weights_bits)
    poison = lambda *shape: torch.full(shape, 0x7f7f, dtype=torch.int16, device=DEV).view(torch.bfloat16)
    lhs, out = poison(e, capacity, k), poison(e, capacity, n)
    ptrs = lambda t: torch.tensor([t[i].data_ptr() for i in range(e)], dtype=torch.int64, device=DEV)
    lhs_ptrs, w_ptrs, out_ptrs = ptrs(lhs), ptrs(w), ptrs(out)
    max_rows = max(int(row_offsets[-1]), int(second_route[0][-1]) if second_route else 0, 1)
    offs = torch.from_numpy(np.ascontiguousarray(row_offsets, dtype=np.int64)).to(DEV)
    src = torch.zeros((max_rows, 3), dtype=torch.int32, device=DEV)
    src[:len(sources)] = torch.from_numpy(np.ascontiguousarray(sources, dtype=np.int32)).to(DEV)
    started = [torch.zeros(world * N.READY_FLAG_STRIDE, dtype=torch.int32, device=DEV) for _ in range(world)]
    done = [torch.zeros(world * N.READY_FLAG_STRIDE, dtype=torch.int32, device=DEV) for _ in range(world)]
    p = N.Bf16GroupedGemmParams(lhs=lhs_ptrs.data_ptr(), weight_nt=w_ptrs.data_ptr(), output=out_ptrs.data_ptr(),
                                row_offsets=offs.data_ptr(), source=src.data_ptr(), experts=e, n=n, k=k,
                                expert_row_capacity=capacity, rank=rank, world_size=world, topk=1)
    p.policy = N.GroupedGemmPolicy(num_comm_ctas=comm, num_compute_ctas=compute, tile_n=tile_n,
                                   mma_sm_count=mma_sm_count)
    for r in range(world):
        p.peer_input[r] = toks[r].data_ptr()
        p.peer_started[r] = started[r].data_ptr()
        p.peer_done[r] = done[r].data_ptr()
    rc, plan = api.create_bf16_a2a_grouped_gemm(p)
    assert rc == 0, f"create_bf16_a2a_grouped_gemm -> cudaError {rc}"
    opts = options(flags=N.SKIP_PEER_WAIT if world > 1 else 0)
    launch = lambda: api.launch_bf16_grouped_gemm(plan, 0, opts)
    if graph:
        assert launch() == 0
        torch.cuda.synchronize()
        captured = torch.cuda.CUDAGraph()
        with torch.cuda.graph(captured):
            rc = api.launch_bf16_grouped_gemm(plan, torch.cuda.current_stream().cuda_stream, opts)
            assert rc == 0, f"launch_bf16_grouped_gemm under stream capture -> cudaError {rc}"
        lhs.view(torch.int16).fill_(0x7f7f)
        out.view(torch.int16).fill_(0x7f7f)

        def launch():
            captured.replay()
            return 0
    if starved_first:
        assert world > 1
        rc = api.launch_bf16_grouped_gemm(plan, 0, options(wait_ms=30.0))
        assert rc == 0, f"launch_bf16_grouped_gemm -> cudaError {rc}"
        torch.cuda.synchronize()
        status = api.read_status(clear=True)
        assert status[0] != 0 and status[1] in (1, 2, 3), f"the starved launch did not report: {status[:8]}"
        lhs.view(torch.int16).fill_(0x7f7f)
        out.view(torch.int16).fill_(0x7f7f)
        launches += 1  # the started epoch below counts every launch
        for _ in range(launches - 1):
            rc = launch()
            assert rc == 0, f"launch_bf16_grouped_gemm -> cudaError {rc}"
        check_status()
    else:
        for _ in range(launches):
            rc = launch()
            assert rc == 0, f"launch_bf16_grouped_gemm -> cudaError {rc}"
        check_status()
    if second_route is not None:
        lhs.view(torch.int16).fill_(0x7f7f)
        out.view(torch.int16).fill_(0x7f7f)
        offs.copy_(torch.from_numpy(np.ascontiguousarray(second_route[0], dtype=np.int64)))
        src[:len(second_route[1])] = torch.from_numpy(np.ascontiguousarray(second_route[1], dtype=np.int32)).to(DEV)
        rc = launch()
        assert rc == 0
        check_status()
    result = to_bits(lhs), to_bits(out)
    assert int(started[0][rank * N.READY_FLAG_STRIDE]) == launches + (1 if second_route else 0) + (1 if graph else 0)
    assert api.destroy_bf16_grouped_gemm(plan) == 0
    return result


def moe_fc2_combine(world, experts_local, lhs_bits, weights_bits, row_offsets, sources, capacity, tokens, topk,
                    tile_n=256, mma_sm_count=1, launches=1, starved_first=False):
    """Every rank of the expert FC2 -> combine operator, emulated one after the other on one GPU.
    lhs_bits[r] [E, capacity, K], weights_bits[r] [E, N, K], row_offsets[r] int64 [E+1], sources[r]
    int32 [rows, 3] per rank r.  Returns (outputs [r] -> [E, capacity, N] bits, received [r] ->
    [tokens * topk, N] bits); rows nobody routes and unused capacity keep the poison 0x7f7f."""
    e, n, k = weights_bits[0].shape
    poison = lambda *shape: torch.full(shape, 0x7f7f, dtype=torch.int16, device=DEV).view(torch.bfloat16)
    received = [poison(tokens * topk, n) for _ in range(world)]
    started = [torch.zeros(world * N.READY_FLAG_STRIDE, dtype=torch.int32, device=DEV) for _ in range(world)]
    done = [torch.zeros(world * N.READY_FLAG_STRIDE, dtype=torch.int32, device=DEV) for _ in range(world)]
    outputs = []
    ptrs = lambda t: torch.tensor([t[i].data_ptr() for i in range(e)], dtype=torch.int64, device=DEV)
    for r in range(world):
        lhs, w, out = to_device(lhs_bits[r]), to_device(weights_bits[r]), poison(e, capacity, n)
        lhs_ptrs, w_ptrs, out_ptrs = ptrs(lhs), ptrs(w), ptrs(out)
        offs = torch.from_numpy(np.ascontiguousarray(row_offsets[r], dtype=np.int64)).to(DEV)
        src = torch.zeros((max(len(sources[r]), 1), 3), dtype=torch.int32, device=DEV)
        src[:len(sources[r])] = torch.from_numpy(np.ascontiguousarray(sources[r], dtype=np.int32)).to(DEV)
        p = N.Bf16GroupedGemmParams(lhs=lhs_ptrs.data_ptr(), weight_nt=w_ptrs.data_ptr(), output=out_ptrs.data_ptr(),
                                    row_offsets=offs.data_ptr(), source=src.data_ptr(), experts=e, n=n, k=k,
                                    expert_row_capacity=capacity, rank=r, world_size=world, topk=topk)
        p.policy = N.GroupedGemmPolicy(num_comm_ctas=4, num_compute_ctas=128, tile_n=tile_n, mma_sm_count=mma_sm_count)
        for q in range(world):
            p.peer_output[q] = received[q].data_ptr()
            p.peer_started[q] = started[q].data_ptr()
            p.peer_done[q] = done[q].data_ptr()
        rc, plan = api.create_bf16_grouped_gemm_a2a(p)
        assert rc == 0, f"create_bf16_grouped_gemm_a2a -> cudaError {rc}"
        opts = options(flags=N.SKIP_PEER_WAIT if world > 1 else 0)
        if starved_first and r == 0:
            # no destination has entered the invocation: the wait before the first remote write runs
            # out, and the failed launch must not tell anyone that its rows are in place
            assert world > 1
            rc = api.launch_bf16_grouped_gemm(plan, 0, options(wait_ms=30.0))
            assert rc == 0, f"launch_bf16_grouped_gemm -> cudaError {rc}"
            torch.cuda.synchronize()
            status = api.read_status(clear=True)
            assert status[0] != 0 and status[1] in (1, 2, 3), f"the starved launch did not report: {status[:8]}"
            for d_ in done:
                assert int(d_.abs().sum()) == 0, "a combine launch that timed out published its done epoch"
            for t in received:
                assert int((t.view(torch.int16) != 0x7f7f).sum()) == 0, "a starved combine launch wrote remote rows"
            out.view(torch.int16).fill_(0x7f7f)
            started[0].zero_()  # the starved launch's own started epoch: the checks below count clean launches
            api.destroy_bf16_grouped_gemm(plan)
            rc, plan = api.create_bf16_grouped_gemm_a2a(p)
            assert rc == 0
        for _ in range(launches):
            rc = api.launch_bf16_grouped_gemm(plan, 0, opts)
            assert rc == 0, f"launch_bf16_grouped_gemm -> cudaError {rc}"
        check_status()
        outputs.append(to_bits(out))
        assert api.destroy_bf16_grouped_gemm(plan) == 0
    for r in range(world):  # every source told every destination (and itself) that its rows are in place
        assert (done[r][::N.READY_FLAG_STRIDE][:world] == launches).all()
    return outputs, [to_bits(t) for t in received]


def _aligned_scratch(nbytes):
    buf = torch.full((nbytes + 256,), 0x5A, dtype=torch.uint8, device=DEV)
    return buf, (buf.data_ptr() + 255) // 256 * 256


def _activation(data_t, scales_t):
    return N.Mxfp8Activation(data=data_t.data_ptr(), scales=scales_t.data_ptr(), data_bytes=data_t.numel(),
                             scale_bytes=scales_t.numel())


def qkv_backward_mxfp8(world, rank, batch, seq_local, q_heads, kv_heads, planes_bits, planes_q, w_bits, x_bits,
                       comm=4, causal=False, alpha=1.0, beta=0.0, dw_init_bits=None, vector=False):
    """One rank of the MXFP8 QKV backward (data + weight).  planes_bits[r] = BF16 (dQ, dK, dV) masters of
    rank r, planes_q[r] = their ((data, scales), ...) quantisations.  Returns (staging, dX, dW) bits."""
    d = 128
    m = batch * seq_local
    width = (q_heads + 2 * kv_heads) * d
    hidden = w_bits.shape[1]
    w, x = to_device(w_bits), to_device(x_bits)
    masters = [[to_device(pl) for pl in planes_bits[r]] for r in range(world)]
    quant = [[(to_device_u8(q[0]), to_device_u8(q[1])) for q in planes_q[r]] for r in range(world)]
    staging, dx = poisoned(m, width), poisoned(m, hidden)
    dw = to_device(dw_init_bits) if dw_init_bits is not None else poisoned(width, hidden)
    done = [torch.zeros(world * N.READY_FLAG_STRIDE, dtype=torch.int32, device=DEV) for _ in range(world)]
    proj = N.QkvBackwardDataParams(weight=w.data_ptr(), grad_input=dx.data_ptr(), local_tokens=m, hidden=hidden,
                                   batch=batch, q_heads=q_heads, kv_heads=kv_heads, head_dim=d, world_size=world,
                                   rank=rank, num_comm_ctas=comm, epoch=1, causal_load_balanced=int(causal), alpha=alpha)
    proj.gemm_tuning.max_swizzle_size = 4
    ready = torch.zeros(api.qkv_backward_ready_elements(proj), dtype=torch.int32, device=DEV)
    proj.peer_dqkv_staging[rank] = staging.data_ptr()
    proj.peer_ready[rank] = ready.data_ptr()
    for peer in range(world):
        proj.peer_done_epoch[peer] = done[peer].data_ptr()
    rc, ws_bytes = api.qkv_backward_mxfp8_data_workspace_size(proj)
    assert rc == 0
    scratch, base = _aligned_scratch(ws_bytes)
    mp = N.Mxfp8QkvBackwardDataParams(projection=proj, workspace=base, workspace_bytes=ws_bytes)
    for peer in range(world):
        mp.peer_input[peer] = N.Mxfp8QkvBackwardInput(
            grad_q=_activation(*quant[peer][0]), grad_k=_activation(*quant[peer][1]), grad_v=_activation(*quant[peer][2]),
            master_q=masters[peer][0].data_ptr(), master_k=masters[peer][1].data_ptr(), master_v=masters[peer][2].data_ptr())
    rc = api.launch_qkv_backward_mxfp8_data(mp, 0, options(flags=(N.SKIP_PEER_WAIT if world > 1 else 0) |
                                                            (N.VECTOR_PULL if vector else 0)))
    assert rc == 0, f"launch_qkv_backward_mxfp8_data -> cudaError {rc}"
    check_status()
    wproj = N.QkvBackwardWeightParams(dqkv_staging=staging.data_ptr(), saved_input=x.data_ptr(),
                                      grad_weight=dw.data_ptr(), local_tokens=m, hidden=hidden, q_heads=q_heads,
                                      kv_heads=kv_heads, head_dim=d, alpha=alpha, beta=beta)
    rc, ws2 = api.qkv_backward_mxfp8_weight_workspace_size(wproj)
    assert rc == 0
    scratch2, base2 = _aligned_scratch(ws2)
    wp = N.Mxfp8QkvBackwardWeightParams(projection=wproj, workspace=base2, workspace_bytes=ws2)
    rc = api.launch_qkv_backward_mxfp8_weight(wp, 0)
    assert rc == 0, f"launch_qkv_backward_mxfp8_weight -> cudaError {rc}"
    check_status()
    del scratch, scratch2
    return to_bits(staging), to_bits(dx), to_bits(dw)


def oproj_backward_mxfp8(world, batch, seq_local, q_heads, dy_bits, dy_q, wo_bits, attn_bits, causal=False,
                         alpha=1.0):
    """Every rank of the MXFP8 output-projection backward.  Returns (dA list, routed list, dWo list)."""
    d = 128
    m, a = batch * seq_local, q_heads * d
    hidden = wo_bits.shape[0]
    rows = batch * seq_local * world
    wo = to_device(wo_bits)
    da = [poisoned(m, a) for _ in range(world)]
    routed = [poisoned(rows * (a // world)) for _ in range(world)]
    dwo = [poisoned(hidden, a) for _ in range(world)]
    done = [torch.zeros(world * N.READY_FLAG_STRIDE, dtype=torch.int32, device=DEV) for _ in range(world)]
    for r in range(world):
        dy, attn = to_device(dy_bits[r]), to_device(attn_bits[r])
        dq = (to_device_u8(dy_q[r][0]), to_device_u8(dy_q[r][1]))
        proj = N.OprojBackwardDataParams(weight=wo.data_ptr(), local_grad_attention=da[r].data_ptr(), local_tokens=m,
                                         hidden=hidden, batch=batch, q_heads=q_heads, head_dim=d, world_size=world,
                                         rank=r, num_comm_ctas=4, epoch=1, causal_load_balanced=int(causal), alpha=alpha)
        proj.gemm_tuning.max_swizzle_size = 4
        for peer in range(world):
            proj.peer_grad_attention[peer] = routed[peer].data_ptr()
            proj.peer_done_epoch[peer] = done[peer].data_ptr()
        rc, ws = api.oproj_backward_mxfp8_data_workspace_size(proj)
        assert rc == 0
        scratch, base = _aligned_scratch(ws)
        mp = N.Mxfp8OprojBackwardDataParams(projection=proj, grad_output=_activation(*dq), workspace=base,
                                            workspace_bytes=ws)
        rc = api.launch_oproj_backward_mxfp8_data(mp, 0, options(flags=N.SKIP_PEER_WAIT if world > 1 else 0))
        assert rc == 0, f"launch_oproj_backward_mxfp8_data -> cudaError {rc}"
        wproj = N.OprojBackwardWeightParams(grad_output=dy.data_ptr(), saved_attention=attn.data_ptr(),
                                            grad_weight=dwo[r].data_ptr(), local_tokens=m, hidden=hidden,
                                            q_heads=q_heads, head_dim=d, alpha=alpha)
        rc, ws2 = api.oproj_backward_mxfp8_weight_workspace_size(wproj)
        assert rc == 0
        scratch2, base2 = _aligned_scratch(ws2)
        wp = N.Mxfp8OprojBackwardWeightParams(projection=wproj, workspace=base2, workspace_bytes=ws2)
        rc = api.launch_oproj_backward_mxfp8_weight(wp, 0)
        assert rc == 0, f"launch_oproj_backward_mxfp8_weight -> cudaError {rc}"
        torch.cuda.synchronize()
        del scratch, scratch2
    check_status()
    return [to_bits(t) for t in da], [to_bits(t) for t in routed], [to_bits(t) for t in dwo]
