"""Expert parallelism with the exchanges fused into the block's own movement kernels.

Same partition and same math as `expert_parallel.py` (routed experts split contiguously over the
ranks of one node, router and shared experts replicated; the reference, src/model/moe.py:345-418,
is single-GPU), but no all-to-all and no second permute on the receiving side:

  home   router + dispatch of its own tokens (the block's kernels) -> per-expert counts
         -- all-gather of the counts [E] --                              (304 bytes per rank)
  home   plan: where each of its pairs lives in its owner's slot-ordered buffer
         PUSH: the token permute writes every row straight into that buffer over NVLink
         -- phase boundary --
  owner  grouped GEMMs of the block on its buffer (up/gate + GLU, down + router weight)
         -- phase boundary --
  home   PULL: the token-major combine reads each pair's row from its owner's output buffer;
         the shared experts' rows (computed at home from x in place) join the same fp32 sum

and the mirror image in the backward (push dOut rows, owner runs dHidden / dX / both weight
gradients, home pulls dX rows and d topk_w). Nothing is read on the host: buffers are sized for
the worst case and the live lengths stay on the device, as in the single-GPU block.

One rank's work is split into phase methods of `EPRank`, so the same code serves
  * `LoopbackGroup`: G virtual ranks in one process on one device (peer pointers are then local
    pointers) -- how the path is tested where fewer GPUs than ranks are available, and
  * `SymmetricGroup`: one process per GPU; the exchange buffers are one symmetric-memory arena per
    rank, the phase boundaries a tiny NCCL all-reduce on the compute stream.
"""
from typing import List, Optional, Sequence

import torch

from . import kernels as K
from . import moe_kernel as MK
from .expert_parallel import expert_partition

_BUFFERS = (            # (name, kind): "rows" = [cap, d_model] bf16, "i32" / "b16" = [cap] vectors
    ("xs", "rows"), ("douts", "rows"), ("y", "rows"), ("ydx", "rows"),
    ("sid", "i32"), ("pw", "b16"), ("dtw", "b16"),
)


def arena_layout(cap: int, d_model: int):
    """Byte offset of every exchange buffer inside a rank's arena, and the arena size."""
    off, out = 0, {}
    for name, kind in _BUFFERS:
        nbytes = cap * (d_model * 2 if kind == "rows" else 4 if kind == "i32" else 2)
        out[name] = off
        off += (nbytes + 255) // 256 * 256
    return out, off


class EPRank:
    """One rank of the expert-parallel block: its plan, its exchange buffers, its phases."""

    def __init__(self, rank: int, world: int, n_experts: int, top_k: int, n_shared: int,
                 d_model: int, tokens_per_rank: int, arena: torch.Tensor):
        self.rank, self.world = rank, world
        self.E, self.k, self.S, self.D, self.T = n_experts, top_k, n_shared, d_model, tokens_per_rank
        bounds = expert_partition(n_experts, world)
        self.lo, self.hi = bounds[rank]
        self.next_lo = bounds[(rank + 1) % world][0]
        self.n_local = self.hi - self.lo
        self.cap = self.capacity(world, tokens_per_rank, top_k, n_experts)
        dev = arena.device
        self.bounds_dev = torch.tensor([b[0] for b in bounds] + [n_experts], dtype=torch.int32,
                                       device=dev)
        layout, size = arena_layout(self.cap, d_model)
        assert arena.dtype == torch.uint8 and arena.numel() >= size
        self.arena, self.layout = arena, layout

        def view(name, dtype, shape):
            n = shape[0] * (shape[1] if len(shape) > 1 else 1)
            return arena[layout[name]:].view(dtype)[:n].view(shape)

        self.xs = view("xs", torch.bfloat16, (self.cap, d_model))
        self.douts = view("douts", torch.bfloat16, (self.cap, d_model))
        self.y = view("y", torch.bfloat16, (self.cap, d_model))
        self.ydx = view("ydx", torch.bfloat16, (self.cap, d_model))
        self.sid = view("sid", torch.int32, (self.cap,))
        self.pw = view("pw", torch.bfloat16, (self.cap,))
        self.dtw = view("dtw", torch.bfloat16, (self.cap,))
        self.peer_base: List[int] = []        # arena base pointer of every rank, set by the group
        # the shared experts only need this rank's own tokens: they run on a second stream, under
        # the pushes, the phase boundaries and the owner's GEMMs
        self.side = torch.cuda.Stream(device=dev)

    @staticmethod
    def capacity(world: int, tokens_per_rank: int, top_k: int, n_experts: int) -> int:
        """Rows of an owner's buffers: every pair of every rank could pick its experts."""
        n_local = max(hi - lo for lo, hi in expert_partition(n_experts, world))
        return K.l_cap(world * tokens_per_rank * top_k, n_local)

    def _peers(self, name: str) -> List[int]:
        return [base + self.layout[name] for base in self.peer_base]

    # ------------------------------------------------------------------ forward
    def f1_route(self, x, router_w, logit_bias, normalize: bool, full_softmax: bool):
        """Router + dispatch of this rank's tokens over all E (+ S) experts. Returns the counts
        [E] int32 that the ranks all-gather."""
        self.x = x.contiguous()
        self.wp = MK.pad_router_weight(router_w, x.dtype)
        self.logits = K.down_gemm(self.x, self.wp, None, None, 1, None, None, 0)[0]
        (self.w_all, self.idx_all, self.colsum, self.sids, self.eids, self.offs, self.counts_all,
         self.npp, self.inv) = K.router_dispatch(self.logits, logit_bias, self.E, self.k, self.S,
                                                 normalize, full_softmax)
        self.logit_bias, self.normalize, self.full_softmax = logit_bias, normalize, full_softmax
        return self.counts_all[: self.E]

    def f2_push(self, cnt_all):
        """Plan from the all-gathered counts [G, E], then push this rank's token rows (with their
        row index and router weight) into the owners' buffers."""
        (self.owner_of, self.send_row0, self.own_offs, self.own_counts, self.own_npp,
         self.own_eids) = K.ep_plan(cnt_all.contiguous(), self.bounds_dev, self.rank,
                                    self.n_local, self.cap // K.ALIGN_M)
        self.pair_rank, self.pair_row = K.ep_pair_map(self.idx_all, self.inv, self.offs,
                                                      self.owner_of, self.send_row0, self.E,
                                                      self.world)
        K.ep_pad_fix(self.own_offs, self.own_counts, self.n_local, self.xs, self.sid, self.cap)
        self.routed_live = self.offs[self.E: self.E + 1]     # start of the first shared run
        # every rank starts its walk at its pairs for the next rank's experts, so that at any one
        # time the ranks write to different owners
        self.first_slot = self.offs[self.next_lo: self.next_lo + 1]
        K.ep_push_rows(self.x, self.k + self.S, self.sids, self.routed_live, self.pair_rank,
                       self.pair_row, self._peers("xs"), self._peers("sid"), self._peers("pw"),
                       self.w_all, first_slot=self.first_slot)

    def f3_experts(self, w_in, w_out, w_sh_in, w_sh_out, activation: str, keep: bool):
        """Owner: the grouped GEMMs over the rows that were pushed here. Home: the shared experts
        on x in place (fixed-group schedule), on the side stream -- call `f3_shared` first if they
        should also run under the push and the phase boundary."""
        act = MK._act_id(activation)
        self.act = act
        if getattr(self, "_shared_for", None) is not self.x:
            self.f3_shared(w_sh_in, w_sh_out, activation, keep)
        hid, a1 = K.up_gemm(self.xs, w_in, self.own_eids, self.own_npp, 0, act, keep)
        K.down_gemm(hid, w_out, self.own_eids, self.own_npp, 0, self.sid, self.pw, self.cap,
                    out=self.y)
        self.a1 = a1
        self.w_in, self.w_out = w_in, w_out

    def f3_shared(self, w_sh_in, w_sh_out, activation: str, keep: bool):
        """The shared experts' forward on the side stream (needs only f1's x)."""
        self.w_sh_in, self.w_sh_out = w_sh_in, w_sh_out
        self.y_sh, self.a1_sh = None, None
        self._shared_for = self.x
        if not self.S:
            return
        act = MK._act_id(activation)
        main = torch.cuda.current_stream(self.x.device)
        self.side.wait_stream(main)
        with torch.cuda.stream(self.side):
            hid_s, self.a1_sh = K.up_gemm(self.x, w_sh_in, None, None, self.S, act, keep)
            self.y_sh = K.down_gemm(hid_s, w_sh_out, None, None, self.S, None, None, 0)
        self.y_sh.record_stream(main)

    def f4_pull(self, aux_coef: float = 0.0, residual: Optional[torch.Tensor] = None):
        """Home: combine, reading every pair's row where it was computed. Returns (out, aux)."""
        torch.cuda.current_stream(self.x.device).wait_stream(self.side)
        tables = self._peers("y") + ([self.y_sh.data_ptr()] if self.S else [])
        out = K.ep_pull_combine(tables, self.pair_rank, self.pair_row, self.T, self.k + self.S,
                                self.D, self.x, residual)
        aux = None
        if self.full_softmax:
            aux = K.balance_loss(self.colsum, self.counts_all, self.E, self.T, aux_coef)
        self.aux_coef = aux_coef
        return out, aux

    # ----------------------------------------------------------------- backward
    def b1_push(self, grad_out):
        self.grad_out = grad_out.to(self.x.dtype).contiguous()
        K.ep_pad_fix(self.own_offs, self.own_counts, self.n_local, self.douts)
        K.ep_push_rows(self.grad_out, self.k + self.S, self.sids, self.routed_live, self.pair_rank,
                       self.pair_row, self._peers("douts"), first_slot=self.first_slot)
        self.ydx_sh = None
        if self.S:      # the shared experts' backward, on the side stream from here on
            main = torch.cuda.current_stream(self.x.device)
            self.side.wait_stream(main)
            with torch.cuda.stream(self.side):
                da1_s, hidw_s, _ = K.dhidden_glu_bwd(self.grad_out, self.w_sh_out, None, None,
                                                     self.S, None, None, 0, self.a1_sh, self.act,
                                                     False)
                self.ydx_sh = K.dx_gemm(da1_s, self.w_sh_in, None, None, self.S)
                self.dw_sh_in = K.wgrad(self.x, da1_s, None, self.S, b_grouped=True)
                self.dw_sh_out = K.wgrad(hidw_s, self.grad_out, None, self.S, a_grouped=True)
            for t in (self.ydx_sh, self.dw_sh_in, self.dw_sh_out):
                t.record_stream(main)

    def b2_experts(self):
        """Owner: dHidden + GLU backward, dX, both weight gradients of its experts (they stay
        here); home: the same for the shared experts."""
        da1, hidw, _ = K.dhidden_glu_bwd(self.douts, self.w_out, self.own_eids, self.own_npp, 0,
                                         self.sid, self.pw, self.cap, self.a1, self.act, True,
                                         dtw_out=self.dtw)
        K.dx_gemm(da1, self.w_in, self.own_eids, self.own_npp, 0, out=self.ydx)
        self.dw_in = K.wgrad(self.xs, da1, self.own_offs, self.n_local)
        self.dw_out = K.wgrad(hidw, self.douts, self.own_offs, self.n_local)

    def b3_pull(self, grad_aux: Optional[torch.Tensor] = None):
        """Home: d topk_w and dX rows from the owners, the router's backward, the combine.
        Returns (dx, d_router_w [D, E])."""
        ks = self.k + self.S
        torch.cuda.current_stream(self.x.device).wait_stream(self.side)
        dtw = K.ep_pull_vec(self._peers("dtw"), self.pair_rank, self.pair_row, self.T, ks, self.k,
                            self.x)
        d_aux = None if grad_aux is None else grad_aux.to(torch.float32).reshape(1)
        dl = K.router_fused_bwd(self.logits, self.logit_bias, self.idx_all, dtw, self.E, self.k,
                                self.S, self.normalize, self.full_softmax, d_aux, self.counts_all,
                                self.aux_coef, self.logits.shape[1])
        d_router = K.copy_cols(K.wgrad(self.x, dl, None, 1)[0], self.E)
        dx_router = K.dx_gemm(dl, self.wp, None, None, 1)[0]
        tables = self._peers("ydx") + ([self.ydx_sh.data_ptr()] if self.S else [])
        dx = K.ep_pull_combine(tables, self.pair_rank, self.pair_row, self.T, ks, self.D, self.x,
                               dx_router)
        return dx, d_router


# ------------------------------------------------------------------------------------ groups
class LoopbackGroup:
    """G virtual ranks in one process on one device: every "peer" buffer is a local one and the
    phases of all ranks simply run one after the other on the current stream."""

    def __init__(self, world: int, n_experts: int, top_k: int, n_shared: int, d_model: int,
                 tokens_per_rank: int, device):
        cap = EPRank.capacity(world, tokens_per_rank, top_k, n_experts)
        _, size = arena_layout(cap, d_model)
        self.ranks = [EPRank(r, world, n_experts, top_k, n_shared, d_model, tokens_per_rank,
                             torch.empty(size, dtype=torch.uint8, device=device))
                      for r in range(world)]
        bases = [r.arena.data_ptr() for r in self.ranks]
        for r in self.ranks:
            r.peer_base = bases

    def forward(self, xs: Sequence[torch.Tensor], router, w_in, w_out, w_sh_in, w_sh_out,
                activation: str, keep: bool = True):
        """xs[r] = rank r's tokens; w_in / w_out the FULL routed stacks (each rank uses its
        slice). Returns the per-rank outputs."""
        full = bool(router.wants_probs()) if hasattr(router, "wants_probs") else False
        bias = router.logit_bias
        bias = None if bias is None else bias.to(torch.float32).contiguous()
        counts = [r.f1_route(x, router.W.detach(), bias, bool(router.normalize_weights), full)
                  for r, x in zip(self.ranks, xs)]
        cnt_all = torch.stack(counts)
        for r in self.ranks:
            r.f2_push(cnt_all)
        for r in self.ranks:
            r.f3_experts(w_in[r.lo:r.hi].contiguous(), w_out[r.lo:r.hi].contiguous(), w_sh_in,
                         w_sh_out, activation, keep)
        return [r.f4_pull(float(router.aux_loss_coef)) for r in self.ranks]

    def backward(self, grad_outs: Sequence[torch.Tensor]):
        """Returns per rank (dx, d_router_w, dW_in_local, dW_out_local, dW_sh_in, dW_sh_out)."""
        for r, g in zip(self.ranks, grad_outs):
            r.b1_push(g)
        for r in self.ranks:
            r.b2_experts()
        res = []
        for r in self.ranks:
            dx, d_router = r.b3_pull()
            res.append((dx, d_router, r.dw_in, r.dw_out, getattr(r, "dw_sh_in", None),
                        getattr(r, "dw_sh_out", None)))
        return res


class SymmetricGroup:
    """One process per GPU. The exchange buffers of a rank are one symmetric-memory arena, so
    every rank holds a peer pointer to every other rank's buffers; the phase boundaries are a
    one-element all-reduce on the compute stream (stream-ordered: a rank's kernels of the next
    phase start after every rank's kernels of the previous one have finished)."""

    def __init__(self, n_experts: int, top_k: int, n_shared: int, d_model: int,
                 tokens_per_rank: int, device, group=None):
        import os
        import torch.distributed as dist
        # only plain peer loads / stores are used here: no multicast mapping of the arena is needed
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        self.dist, self.group = dist, group
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        cap = EPRank.capacity(world, tokens_per_rank, top_k, n_experts)
        _, size = arena_layout(cap, d_model)
        arena = symm_mem.empty(size, dtype=torch.uint8, device=device)
        handle = symm_mem.rendezvous(arena, group if group is not None else dist.group.WORLD)
        self.handle = handle                     # keeps the peer mappings alive
        self.me = EPRank(rank, world, n_experts, top_k, n_shared, d_model, tokens_per_rank, arena)
        self.me.peer_base = [int(p) for p in handle.buffer_ptrs]
        self.flag = torch.zeros(1, device=device)
        self.n_experts, self.world = n_experts, world
        self.timing = False          # set True to collect per-phase CUDA events (see phase_times)
        self._marks = []

    def mark(self, name: str) -> None:
        """Start of a phase on the compute stream (only when `timing` is on)."""
        if self.timing:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._marks.append((name, ev))

    def phase_times(self):
        """Mean milliseconds per phase over the steps marked so far ({name: ms}), then forgets
        them. A phase lasts from its mark to the next one; "end" closes the last phase of a step.
        Synchronises."""
        torch.cuda.synchronize()
        total, count = {}, {}
        for (name, ev), (nxt, ev2) in zip(self._marks, self._marks[1:]):
            if name == "end":
                continue
            total[name] = total.get(name, 0.0) + ev.elapsed_time(ev2)
            count[name] = count.get(name, 0) + 1
        self._marks = []
        return {n: total[n] / count[n] for n in total}

    def boundary(self) -> None:
        self.dist.all_reduce(self.flag, group=self.group)

    def gather_counts(self, counts: torch.Tensor) -> torch.Tensor:
        out = torch.empty((self.world, self.n_experts), dtype=torch.int32, device=counts.device)
        self.dist.all_gather_into_tensor(out, counts.contiguous(), group=self.group)
        return out


class _EPPushBlock(torch.autograd.Function):
    """The expert-parallel block of one rank as a single autograd node."""

    @staticmethod
    def forward(ctx, x, router_w, w_in_local, w_out_local, w_sh_in, w_sh_out, grp, logit_bias,
                normalize, full_softmax, aux_coef, activation):
        me = grp.me
        keep = any(t is not None and t.requires_grad
                   for t in (x, router_w, w_in_local, w_out_local, w_sh_in, w_sh_out))
        cast = lambda t: None if t is None else t.detach().to(x.dtype).contiguous()
        grp.mark("route")
        counts = me.f1_route(x.detach(), router_w.detach(), logit_bias, normalize, full_softmax)
        cnt_all = grp.gather_counts(counts)
        me.f3_shared(cast(w_sh_in), cast(w_sh_out), activation, keep)
        grp.mark("push x")
        me.f2_push(cnt_all)
        grp.mark("wait 1")
        grp.boundary()
        grp.mark("owner fwd")
        me.f3_experts(cast(w_in_local), cast(w_out_local), cast(w_sh_in), cast(w_sh_out),
                      activation, keep)
        grp.mark("wait 2")
        grp.boundary()
        grp.mark("pull y")
        out, aux = me.f4_pull(aux_coef)
        grp.mark("end")
        ctx.grp = grp
        ctx.has_shared = w_sh_in is not None
        ctx.router_dtype = router_w.dtype
        if aux is None:
            aux = torch.zeros((), dtype=torch.float32, device=x.device)
        ctx.mark_non_differentiable(cnt_all)
        return out, aux, cnt_all

    @staticmethod
    def backward(ctx, grad_out, grad_aux, _unused):
        grp, me = ctx.grp, ctx.grp.me
        if grad_out is None:
            grad_out = torch.zeros_like(me.x)
        grp.mark("push dOut")
        me.b1_push(grad_out)
        grp.mark("wait 3")
        grp.boundary()
        grp.mark("owner bwd")
        me.b2_experts()
        grp.mark("wait 4")
        grp.boundary()
        grp.mark("pull dX + router bwd")
        dx, d_router = me.b3_pull(grad_aux if me.full_softmax else None)
        grp.mark("end")
        dsi = me.dw_sh_in if ctx.has_shared else None
        dso = me.dw_sh_out if ctx.has_shared else None
        return (dx, d_router.to(ctx.router_dtype), me.dw_in, me.dw_out, dsi, dso, None, None, None,
                None, None, None)


def ep_push_block_forward(x, router, w_in_local, w_out_local, w_sh_in, w_sh_out, activation: str,
                          grp: SymmetricGroup):
    """The expert-parallel block on this rank over peer memory: (out [T, D], aux_loss fp32,
    counts of every rank's tokens per expert [G, E] int32). Same arguments as
    expert_parallel.ep_block_forward plus the group object that owns the exchange buffers (one per
    layer: the forward's buffers are read again by the backward)."""
    bias = router.logit_bias
    bias = None if bias is None else bias.to(torch.float32).contiguous()
    full = bool(router.wants_probs()) if hasattr(router, "wants_probs") else False
    return _EPPushBlock.apply(x, router.W, w_in_local, w_out_local, w_sh_in, w_sh_out, grp, bias,
                              bool(router.normalize_weights), full, float(router.aux_loss_coef),
                              activation)
