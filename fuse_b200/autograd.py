"""torch.autograd wrappers of the fused Ulysses projections (one object per rank).

    proj = UlyssesProjections(world, batch=1, seq_local=S, hidden=H, q_heads=32, kv_heads=8, head_dim=128)
    q, k, v = proj.qkv(x, w_qkv)          # x [B*S, H] (this rank's sequence shard) -> this rank's heads,
                                          # every position: [B*S_global, local_heads*d] each
    a = attention(q, k, v)                # caller's attention, [B*S_global, q_local*d]
    y = proj.oproj(a, w_o)                # head->sequence all-to-all + output projection, [B*S, H]
    y.backward(dy)                        # fused backward: dA routed back, dX, dW_qkv, dW_o

The reference checks its fused backward boundaries against `torch.nn.functional.linear` and native
autograd (benchmarks/sm90/backward/backward_torch_autograd.py: conformance of
launch_qkv_backward / launch_oproj_backward through a raw-pointer bridge); this module is that
bridge turned into `torch.autograd.Function`s over the C ABI, and tests/test_gpu_autograd.py is
the same conformance check.

Buffers that other ranks write into or read from live in symmetric memory (`World`): the planar
Q/K/V destination, the attention output the peers pull, the packed gradient staging and the routed
attention gradient.  What a caller keeps (Q, K, V, dA, saved operands) is copied out into torch
tensors, so the symmetric buffers are free again as soon as the copy has run; a peer can only write
the next invocation into them after this rank has taken part in the invocation in between (every
operator ends with, or is gated by, an epoch handshake between the ranks).  All ranks must call the
operators in the same order.  Weight gradients are local (no cross-rank reduction: the caller owns
it, include/fuse/operators/ulysses/oproj_backward.h:202 of the reference); with
`reduce_weight_grads=True` this caller-side step is done here: a hook on each weight leaf starts the
all-reduce of its `.grad` over the group, on NCCL's own stream, as soon as autograd has stored it,
so the reduction of dW_o travels under the attention and QKV backward kernels;
`finish_weight_grads()` makes the current stream wait for the reductions still in flight (call it
before the optimizer reads the gradients).  The hook reduces what `.grad` holds, so with gradient
accumulation switch `reduce_weight_grads` on for the last micro-batch only."""
from __future__ import annotations

import torch

from . import _native as N
from . import api
from .world import World

BF16 = torch.bfloat16


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} -> cudaError {rc}")


class UlyssesProjections:
    def __init__(self, world: World, *, batch: int, seq_local: int, hidden: int, q_heads: int, kv_heads: int,
                 head_dim: int, max_swizzle_size: int = 8, tag: str = "ulysses", reduce_weight_grads: bool = False):
        cp = world.world_size
        if q_heads % cp or kv_heads % cp:
            raise ValueError("heads must divide over the ranks")
        self.world, self.cp, self.rank = world, cp, world.rank
        self.batch, self.seq_local, self.hidden = batch, seq_local, hidden
        self.q_heads, self.kv_heads, self.head_dim = q_heads, kv_heads, head_dim
        self.swizzle = max_swizzle_size
        self.m = batch * seq_local
        self.rows_global = batch * seq_local * cp
        self.q_local, self.kv_local = q_heads // cp * head_dim, kv_heads // cp * head_dim
        self.width = (q_heads + 2 * kv_heads) * head_dim
        self.attn_width = q_heads * head_dim
        self.device = torch.device("cuda", world.device)
        planar = self.rows_global * (self.q_local + 2 * self.kv_local) * 2
        attn = self.rows_global * self.q_local * 2
        line = cp * N.READY_FLAG_STRIDE * 4
        t = tag
        self._names = dict(planar=f"{t}_planar", qkv_done=f"{t}_qkv_done", attn0=f"{t}_attn0", attn1=f"{t}_attn1",
                           attn_ready=f"{t}_attn_ready", dqkv=f"{t}_dqkv", dqkv_ready=f"{t}_dqkv_ready",
                           dqkv_done=f"{t}_dqkv_done", dattn=f"{t}_dattn", dattn_done=f"{t}_dattn_done")
        probe = N.QkvBackwardDataParams(local_tokens=self.m, hidden=hidden, batch=batch, q_heads=q_heads,
                                        kv_heads=kv_heads, head_dim=head_dim, world_size=cp, rank=self.rank)
        self._dqkv_ready_words = api.qkv_backward_ready_elements(probe)
        sym = world.allocate({
            self._names["planar"]: planar, self._names["qkv_done"]: line,
            self._names["attn0"]: attn, self._names["attn1"]: attn, self._names["attn_ready"]: 256,
            self._names["dqkv"]: self.m * self.width * 2, self._names["dqkv_ready"]: self._dqkv_ready_words * 4,
            self._names["dqkv_done"]: line, self._names["dattn"]: attn, self._names["dattn_done"]: line})
        self.sym = {key: sym[name] for key, name in self._names.items()}
        for key in ("qkv_done", "attn_ready", "dqkv_ready", "dqkv_done", "dattn_done"):
            self.sym[key].local.zero_()
        torch.cuda.synchronize(self.device)
        self.local_qkv = torch.empty((self.m, self.width), dtype=BF16, device=self.device)
        self._qkv_problem = N.GemmProblem(self.m, self.width, hidden, raster=N.RASTER_ALONG_M,
                                          max_swizzle_size=max_swizzle_size)
        self._o_problem = N.GemmProblem(self.m, hidden, self.attn_width, raster=N.RASTER_ALONG_N,
                                        max_swizzle_size=max_swizzle_size)
        self._o_route = N.UlyssesRoute(world_size=cp, rank=self.rank, batch=batch, global_seq=seq_local * cp,
                                       seq_local=seq_local, q_heads=q_heads, head_dim=head_dim,
                                       kind=N.ROUTE_HEAD_TO_SEQUENCE, direction=N.ROUTE_INVERSE)
        self._qkv_ready = torch.zeros(api.qkv_ready_elements(self._qkv_problem), dtype=torch.int32, device=self.device)
        self._o_ready = torch.zeros(api.a2a_lhs_gemm_ready_elements(self._o_problem, self._o_route),
                                    dtype=torch.int32, device=self.device)
        probe_o = N.OprojBackwardDataParams(local_tokens=self.m, hidden=hidden, batch=batch, q_heads=q_heads,
                                            head_dim=head_dim, world_size=cp, rank=self.rank)
        self._dattn_ready = torch.zeros(api.oproj_backward_ready_elements(probe_o), dtype=torch.int32,
                                        device=self.device)
        self._epochs = dict(qkv=0, oproj=0, qkv_bwd=0, oproj_bwd=0)
        self._attn_slot = 0
        self.reduce_weight_grads = reduce_weight_grads and cp > 1
        self._pending = []

    # ------------------------------------------------------------------ cross-rank weight gradients
    def _hook(self, weight: torch.Tensor) -> None:
        """Once per weight leaf: start the all-reduce of its gradient when autograd has stored it."""
        if not (weight.is_leaf and weight.requires_grad) or getattr(weight, "_fuse_b200_hooked", False):
            return
        import torch.distributed as dist

        def start(param):
            if self.reduce_weight_grads and param.grad is not None:
                self._pending.append(dist.all_reduce(param.grad, group=self.world.group, async_op=True))

        weight.register_post_accumulate_grad_hook(start)
        weight._fuse_b200_hooked = True

    def finish_weight_grads(self) -> None:
        """The current stream waits for every weight-gradient reduction still in flight."""
        for work in self._pending:
            work.wait()
        self._pending.clear()

    # ------------------------------------------------------------------ plumbing
    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def _next(self, op: str) -> int:
        self._epochs[op] += 1
        return self._epochs[op]

    def attention_buffer(self) -> torch.Tensor:
        """The symmetric buffer the next `oproj` call reads, as [B*S_global, q_local*d]: an attention
        kernel that writes here saves `oproj` its copy."""
        return self.sym[f"attn{self._attn_slot}"].view(BF16).view(self.rows_global, self.q_local)

    # ------------------------------------------------------------------ raw launches (no autograd)
    def _qkv_forward(self, x: torch.Tensor, w: torch.Tensor):
        route = N.UlyssesRoute(world_size=self.cp, rank=self.rank, batch=self.batch,
                               global_seq=self.seq_local * self.cp, seq_local=self.seq_local, q_heads=self.q_heads,
                               kv_heads=self.kv_heads, head_dim=self.head_dim, kind=N.ROUTE_QKV_GQA_PACK)
        p = N.GemmA2AParams(lhs=x.data_ptr(), rhs_nt=w.data_ptr(), local_output=self.local_qkv.data_ptr(),
                            ready=self._qkv_ready.data_ptr(), gemm=self._qkv_problem, route=route, num_comm_ctas=0,
                            epoch=self._next("qkv"))
        for peer in range(self.cp):
            p.peer_output[peer] = self.sym["planar"].peer_ptrs[peer]
            p.peer_route_done_epoch[peer] = self.sym["qkv_done"].peer_ptrs[peer]
        _check(api.launch_gemm_a2a_cutlass(p, self._stream(), N.Options()), "launch_gemm_a2a_cutlass")
        planar = self.sym["planar"].view(BF16)
        q_elems, kv_elems = self.rows_global * self.q_local, self.rows_global * self.kv_local
        q = planar[:q_elems].view(self.rows_global, self.q_local).clone()
        k = planar[q_elems:q_elems + kv_elems].view(self.rows_global, self.kv_local).clone()
        v = planar[q_elems + kv_elems:q_elems + 2 * kv_elems].view(self.rows_global, self.kv_local).clone()
        return q, k, v

    def _oproj_forward(self, attn: torch.Tensor, w: torch.Tensor):
        slot = self._attn_slot
        buf = self.sym[f"attn{slot}"]
        mine = buf.view(BF16).view(self.rows_global, self.q_local)
        if attn.data_ptr() != mine.data_ptr():
            mine.copy_(attn)
        self._attn_slot ^= 1
        epoch = self._next("oproj")
        # upstream epoch word: published on the stream behind the attention output, awaited by the pulling ranks
        ready_word = self.sym["attn_ready"].local.view(torch.int32)
        ready_word[slot * 32:slot * 32 + 1].fill_(epoch)
        staging = torch.empty((self.m, self.attn_width), dtype=BF16, device=self.device)
        out = torch.empty((self.m, self.hidden), dtype=BF16, device=self.device)
        p = N.A2AGemmParams(input_staging=staging.data_ptr(), rhs_nt=w.data_ptr(), output=out.data_ptr(),
                            ready=self._o_ready.data_ptr(), gemm=self._o_problem, route=self._o_route,
                            num_comm_ctas=0, epoch=epoch, input_epoch=epoch)
        for peer in range(self.cp):
            p.peer_input[peer] = self.sym[f"attn{slot}"].peer_ptrs[peer]
            p.peer_input_ready[peer] = self.sym["attn_ready"].peer_ptrs[peer] + slot * 128
        _check(api.launch_a2a_gemm_cutlass(p, self._stream()), "launch_a2a_gemm_cutlass")
        return out, staging

    def _qkv_backward(self, dq, dk, dv, x, w):
        dx = torch.empty((self.m, self.hidden), dtype=BF16, device=self.device)
        dw = torch.empty((self.width, self.hidden), dtype=BF16, device=self.device)
        p = N.QkvBackwardDataParams(grad_q=dq.data_ptr(), grad_k=dk.data_ptr(), grad_v=dv.data_ptr(),
                                    weight=w.data_ptr(), grad_input=dx.data_ptr(), local_tokens=self.m,
                                    hidden=self.hidden, batch=self.batch, q_heads=self.q_heads,
                                    kv_heads=self.kv_heads, head_dim=self.head_dim, world_size=self.cp,
                                    rank=self.rank, num_comm_ctas=0, epoch=self._next("qkv_bwd"))
        p.gemm_tuning.max_swizzle_size = 1  # the reference's default backward tuning, the fastest measured here
        for peer in range(self.cp):
            p.peer_dqkv_staging[peer] = self.sym["dqkv"].peer_ptrs[peer]
            p.peer_ready[peer] = self.sym["dqkv_ready"].peer_ptrs[peer]
            p.peer_done_epoch[peer] = self.sym["dqkv_done"].peer_ptrs[peer]
        _check(api.launch_qkv_backward_data(p, self._stream()), "launch_qkv_backward_data")
        wp = N.QkvBackwardWeightParams(dqkv_staging=self.sym["dqkv"].local.data_ptr(), saved_input=x.data_ptr(),
                                       grad_weight=dw.data_ptr(), local_tokens=self.m, hidden=self.hidden,
                                       q_heads=self.q_heads, kv_heads=self.kv_heads, head_dim=self.head_dim)
        _check(api.launch_qkv_backward_weight(wp, self._stream()), "launch_qkv_backward_weight")
        return dx, dw

    def _oproj_backward(self, dy, w, staging):
        da = torch.empty((self.m, self.attn_width), dtype=BF16, device=self.device)
        dw = torch.empty((self.hidden, self.attn_width), dtype=BF16, device=self.device)
        p = N.OprojBackwardDataParams(grad_output=dy.data_ptr(), weight=w.data_ptr(),
                                      local_grad_attention=da.data_ptr(), ready=self._dattn_ready.data_ptr(),
                                      local_tokens=self.m, hidden=self.hidden, batch=self.batch,
                                      q_heads=self.q_heads, head_dim=self.head_dim, world_size=self.cp,
                                      rank=self.rank, num_comm_ctas=0, epoch=self._next("oproj_bwd"))
        p.gemm_tuning.max_swizzle_size = 1  # the reference's default backward tuning, the fastest measured here
        for peer in range(self.cp):
            p.peer_grad_attention[peer] = self.sym["dattn"].peer_ptrs[peer]
            p.peer_done_epoch[peer] = self.sym["dattn_done"].peer_ptrs[peer]
        _check(api.launch_oproj_backward_data(p, self._stream()), "launch_oproj_backward_data")
        wp = N.OprojBackwardWeightParams(grad_output=dy.data_ptr(), saved_attention=staging.data_ptr(),
                                         grad_weight=dw.data_ptr(), local_tokens=self.m, hidden=self.hidden,
                                         q_heads=self.q_heads, head_dim=self.head_dim)
        _check(api.launch_oproj_backward_weight(wp, self._stream()), "launch_oproj_backward_weight")
        d_attn = self.sym["dattn"].view(BF16).view(self.rows_global, self.q_local).clone()
        return d_attn, dw

    # ------------------------------------------------------------------ autograd entry points
    def qkv(self, x: torch.Tensor, w_qkv: torch.Tensor):
        """x [B*S_local, hidden], w_qkv [(q+2kv)*d, hidden] -> (Q, K, V) of this rank's heads."""
        self._expect(x, (self.m, self.hidden), "x")
        self._expect(w_qkv, (self.width, self.hidden), "w_qkv")
        if self.cp > 1:
            self._hook(w_qkv)
        return _QkvProjection.apply(self, x, w_qkv)

    def oproj(self, attn: torch.Tensor, w_o: torch.Tensor):
        """attn [B*S_global, q_local*d] (this rank's heads), w_o [hidden, q_heads*d] -> y [B*S_local, hidden]."""
        self._expect(attn, (self.rows_global, self.q_local), "attn")
        self._expect(w_o, (self.hidden, self.attn_width), "w_o")
        if self.cp > 1:
            self._hook(w_o)
        return _OutputProjection.apply(self, attn, w_o)

    def _expect(self, t: torch.Tensor, shape, name: str) -> None:
        if t.dtype != BF16 or tuple(t.shape) != tuple(shape) or not t.is_contiguous() or t.device != self.device:
            raise ValueError(f"{name}: expected contiguous bfloat16 {tuple(shape)} on {self.device}, got "
                             f"{t.dtype} {tuple(t.shape)} on {t.device}")


class _QkvProjection(torch.autograd.Function):
    @staticmethod
    def forward(ctx, proj: UlyssesProjections, x, w):
        ctx.proj = proj
        ctx.save_for_backward(x, w)
        return proj._qkv_forward(x, w)

    @staticmethod
    def backward(ctx, dq, dk, dv):
        x, w = ctx.saved_tensors
        proj = ctx.proj
        grads = []
        for g, width in ((dq, proj.q_local), (dk, proj.kv_local), (dv, proj.kv_local)):
            if g is None:
                g = torch.zeros((proj.rows_global, width), dtype=BF16, device=proj.device)
            grads.append(g.contiguous())
        dx, dw = proj._qkv_backward(grads[0], grads[1], grads[2], x, w)
        return None, dx, dw


class _OutputProjection(torch.autograd.Function):
    @staticmethod
    def forward(ctx, proj: UlyssesProjections, attn, w):
        out, staging = proj._oproj_forward(attn, w)
        ctx.proj = proj
        ctx.save_for_backward(w, staging)  # the gathered lhs is the weight gradient's operand
        return out

    @staticmethod
    def backward(ctx, dy):
        w, staging = ctx.saved_tensors
        d_attn, dw = ctx.proj._oproj_backward(dy.contiguous(), w, staging)
        return None, d_attn, dw
